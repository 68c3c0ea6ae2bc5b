"""Feed-forward parts: the dense SwiGLU MLP and the sparse expert block.

Reference: dense MLP as three cuBLAS products and an elementwise kernel
(src/layers/mlp.cpp:225-303, src/kernels/swiglu_kernel.cu:16-26); expert block
in src/layers/moe.cpp:185-296 (router product into FP16, one-thread-per-token
top-k, indices copied to the host, every used expert run on all tokens and
masked, shared expert added last).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..ops import functional as F
from .base import FeedForward, Runtime, StepContext, TensorDecl, WeightedRowSum, linear, linear_swiglu
from .tuning import TUNING


class SwiGLUMLP(FeedForward):
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T``.  params: ``hidden_size``, ``intermediate_size``.

    Tensors: ``<prefix>{gate,up}_proj.weight [I, H]``, ``<prefix>down_proj.weight [H, I]``.
    """

    graph_safe = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.H = int(self.params["hidden_size"])
        self.I = int(self.params["intermediate_size"])

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        return [TensorDecl(p + "gate_proj.weight", (self.I, self.H)),
                TensorDecl(p + "up_proj.weight", (self.I, self.H)),
                TensorDecl(p + "down_proj.weight", (self.H, self.I))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        self.w_gate_up = torch.cat([m(tensors[p + "gate_proj.weight"], dev),
                                    m(tensors[p + "up_proj.weight"], dev)], dim=0)
        self.w_down = m(tensors[p + "down_proj.weight"], dev)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return linear(linear_swiglu(x, self.w_gate_up, self.rt.act), self.w_down, torch.float32)


class SparseMoE(FeedForward):
    """Softmax router, top-k routed SwiGLU experts, optional sigmoid-gated shared expert.

    params: ``hidden_size``, ``num_experts``, ``top_k``, ``expert_intermediate_size``,
    ``shared_intermediate_size`` (0 = no shared expert), ``norm_topk_prob``.

    Tensors: ``<prefix>gate.weight [E, H]``;
    ``<prefix>experts.{e}.{gate,up}_proj.weight [mI, H]``, ``.down_proj.weight [H, mI]``;
    ``<prefix>shared_expert.{gate,up,down}_proj.weight``, ``<prefix>shared_expert_gate.weight [1, H]``.
    """

    graph_safe = True
    # which kernel a step of a given size takes, and where the shared expert is forked, are measured
    # thresholds: parts/tuning.py

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.E = int(p["num_experts"])
        self.K = int(p["top_k"])
        self.mI = int(p["expert_intermediate_size"])
        self.sI = int(p.get("shared_intermediate_size", 0))
        self.norm_topk = bool(p.get("norm_topk_prob", False))
        if not 1 <= self.K <= min(self.E, 32):
            raise ValueError(f"moe: top_k {self.K} must lie in [1, min(32, num_experts={self.E})]")
        self.last_routing = None
        self.keep_routing = False
        self._side_stream = None
        self._side_stream_big = None

    # recorded routing survives capture: the graph is keyed by the switch, and a replay refreshes the
    # recorded tensors in place
    def capture_key(self):
        return bool(self.keep_routing)

    def side_outputs(self):
        return self.last_routing if self.keep_routing else None

    def adopt_side_outputs(self, outputs) -> None:
        self.last_routing = outputs

    def tensor_decls(self) -> List[TensorDecl]:
        p = self.prefix
        out = [TensorDecl(p + "gate.weight", (self.E, self.H))]
        for e in range(self.E):
            q = f"{p}experts.{e}."
            out += [TensorDecl(q + "gate_proj.weight", (self.mI, self.H)),
                    TensorDecl(q + "up_proj.weight", (self.mI, self.H)),
                    TensorDecl(q + "down_proj.weight", (self.H, self.mI))]
        if self.sI > 0:
            q = p + "shared_expert."
            out += [TensorDecl(q + "gate_proj.weight", (self.sI, self.H)),
                    TensorDecl(q + "up_proj.weight", (self.sI, self.H)),
                    TensorDecl(q + "down_proj.weight", (self.H, self.sI)),
                    TensorDecl(p + "shared_expert_gate.weight", (1, self.H))]
        return out

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        m, dev, p = rt.precision.matrix, rt.device, self.prefix
        # router and shared gate feed float32 dot products only
        self.w_router = rt.precision.small(tensors[p + "gate.weight"], dev)
        self.w_gate_up = torch.empty(self.E, 2 * self.mI, self.H, dtype=rt.act, device=dev)
        self.w_down = torch.empty(self.E, self.H, self.mI, dtype=rt.act, device=dev)
        for e in range(self.E):
            q = f"{p}experts.{e}."
            self.w_gate_up[e, :self.mI].copy_(tensors[q + "gate_proj.weight"])
            self.w_gate_up[e, self.mI:].copy_(tensors[q + "up_proj.weight"])
            self.w_down[e].copy_(tensors[q + "down_proj.weight"])
        self.w_shared_gate = None
        if self.sI > 0:
            q = p + "shared_expert."
            self.w_shared_gate_up = torch.cat([m(tensors[q + "gate_proj.weight"], dev),
                                               m(tensors[q + "up_proj.weight"], dev)], dim=0)
            self.w_shared_down = m(tensors[q + "down_proj.weight"], dev)
            g = rt.precision.small(tensors[p + "shared_expert_gate.weight"], dev).reshape(-1)
            self.w_shared_gate = g.to(self.w_router.dtype).contiguous()
        # the one-launch routing of decode-sized steps counts its blocks in these words
        self._route_small_max = F.route_small_max_tokens()
        self._route_ticket = torch.zeros(1 + self._route_small_max, dtype=torch.int32, device=dev)
        self._pairs_max = min(self._route_small_max, F.skinny_pairs_max_tokens())
        self._tc = (rt.act == torch.bfloat16 and F.grouped_gemm_tc_supported(self.H)
                    and F.grouped_gemm_tc_supported(self.mI) and self.H % 8 == 0)
        self._skinny = (rt.act == torch.bfloat16 and F.grouped_gemm_skinny_supported(self.H)
                        and F.grouped_gemm_skinny_supported(self.mI))

    def _shared_expert(self, x: torch.Tensor) -> torch.Tensor:
        return linear(linear_swiglu(x, self.w_shared_gate_up, self.rt.act), self.w_shared_down, torch.float32)

    def _fork_shared_expert(self, x: torch.Tensor):
        """Start the shared expert on a second stream, beside the routed experts.  The routing of the smallest steps is a chain of short
        dependent loads that a concurrent weight stream slows down, so there the fork comes after
        it; larger steps, whose shared expert is a library product that would crowd the expert
        kernels off the device, fork first."""
        main = torch.cuda.current_stream()
        # Large steps run the shared expert as library products whose blocks fill an SM: on a stream of
        # higher priority they take their SMs ahead of the routing's small kernels, which slip into what
        # is left, whatever order the two streams' first kernels reach the device in.
        big = x.shape[0] > TUNING.shared_expert_priority_stream_min_tokens
        if big:
            if self._side_stream_big is None:
                self._side_stream_big = torch.cuda.Stream(device=x.device, priority=-1)
            side = self._side_stream_big
        else:
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=x.device)
            side = self._side_stream
        side.wait_stream(main)
        with torch.cuda.stream(side):
            shared = self._shared_expert(x)
        shared.record_stream(main)
        return side, shared

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return self.forward_deferred(x, ctx).materialize()

    def forward_deferred(self, x: torch.Tensor, ctx: StepContext) -> WeightedRowSum:
        """Everything but the weighted sum of the experts' rows (and of the shared expert's): the
        norm that follows forms it inside its own kernel."""
        return self._run(x, ctx, None)

    def forward_from_residual(self, hidden: torch.Tensor, delta, norm, ctx: StepContext):
        """The smallest steps run the residual addition, an RMSNorm and the routing in one launch
        (the routing's blocks read the row anyway); the others take the norm's own kernel."""
        T = hidden.shape[0]
        rms = norm.rms_parameters()
        if ctx.prefetch is not None and self.sI > 0:
            # the routing that comes first hardly touches memory: the shared expert's weights arrive beside it
            ctx.prefetch((self.w_shared_gate_up, self.w_shared_down))
        if (rms is not None and T <= TUNING.shared_expert_fork_after_routing_max_tokens and self._by_pair(T)
                and F.norm_route_small_takes(self.H, self.E, self.w_shared_gate is not None, self.w_router.dtype)
                and (delta is None or isinstance(delta, torch.Tensor))):
            x, idx, w, gate, probs = F.moe_norm_route_small(
                hidden, delta, rms[0], rms[1], self.rt.act, self.w_router, self.w_shared_gate, self.K,
                self.norm_topk, want_probs=self.keep_routing)
            return self._run(x, ctx, (idx, w, gate, probs))
        return super().forward_from_residual(hidden, delta, norm, ctx)

    def _few_rows_per_expert(self, T: int) -> bool:
        """Whether a step of T tokens takes the decode-sized expert products (every used expert's weights
        read once into mma.sync fragments) rather than the tcgen05 product: the smallest steps always
        (their form splits the inner dimension over a block's warps and streams at the memory's speed),
        larger ones up to the tuned number of rows per expert; without the tcgen05 product (inner sizes it
        does not take) up to 8 rows per expert, beyond which re-reading weights per 16 rows costs more than
        the plain kernel."""
        if not self._skinny:
            return False
        if T <= F.skinny_pairs_split_inner_max_tokens() and T <= self._pairs_max:
            return True
        rows = TUNING.expert_skinny_rows_per_expert if self._tc else 8
        return T * self.K <= rows * self.E

    def _by_pair(self, T: int) -> bool:
        """... and without a permutation (result rows indexed by (token, slot) pair)."""
        return T <= self._pairs_max and self._few_rows_per_expert(T)

    def _run(self, x: torch.Tensor, ctx: StepContext, routed) -> WeightedRowSum:
        T = x.shape[0]
        shared = side = inv_perm = None
        overlap = self.sI > 0 and TUNING.shared_expert_overlap
        n = T * self.K
        if self._by_pair(T):
            # decode-sized step: routing in one launch, no permutation; every used expert's weights
            # are read once and result rows are indexed by (token, slot) pair
            fork_first = T > TUNING.shared_expert_fork_after_routing_max_tokens
            if overlap and fork_first:
                side, shared = self._fork_shared_expert(x)
            if routed is not None:
                idx, w, gate, probs = routed
            else:
                idx, w, gate, probs, _, _, _ = F.moe_route_small(
                    x, self.w_router, self.w_shared_gate, self.K, self.norm_topk, self._route_ticket,
                    want_probs=self.keep_routing, permute=False)
            if overlap and not fork_first:
                side, shared = self._fork_shared_expert(x)
            act = F.grouped_gemm_skinny_pairs(x, idx, self.w_gate_up, True)
            y = F.grouped_gemm_skinny_pairs(act, idx, self.w_down, False)
            if ctx.prefetch is not None:
                # while the experts' rows are summed and normalised, the next layer's first weights arrive
                ctx.prefetch(ctx.prefetch_upcoming)
        else:
            fork_first = T > TUNING.shared_expert_fork_after_permutation_max_tokens
            if overlap and fork_first:
                side, shared = self._fork_shared_expert(x)
            # (the float32 path routes every step with the same kernel: same bits however the work is cut)
            if T <= min(self._route_small_max, TUNING.route_with_permutation_one_launch_max_tokens) \
                    and self.rt.act == torch.bfloat16:
                idx, w, gate, probs, offsets, sorted_token, inv_perm = F.moe_route_small(
                    x, self.w_router, self.w_shared_gate, self.K, self.norm_topk, self._route_ticket,
                    want_probs=self.keep_routing)
            else:
                idx, w, gate, probs = F.moe_router(x, self.w_router, self.w_shared_gate, self.K, self.norm_topk,
                                                   want_probs=self.keep_routing)
                offsets, sorted_token, inv_perm = F.moe_permute(idx, self.E)
            if overlap and not fork_first:
                side, shared = self._fork_shared_expert(x)
            if self._few_rows_per_expert(T):
                # a few rows per expert: bound by reading each used expert once
                act = F.grouped_gemm_skinny(x, sorted_token, self.w_gate_up, offsets, n, True)
                y = F.grouped_gemm_skinny(act, None, self.w_down, offsets, n, False)
            elif self._tc:
                # many rows per expert: tensor-core tiles over the rows gathered into expert order
                xs = F.gather_rows(x, sorted_token)
                act = F.grouped_gemm_tc(xs, self.w_gate_up, offsets, True)
                y = F.grouped_gemm_tc(act, self.w_down, offsets, False)
            else:
                act = F.grouped_gemm_plain(x, sorted_token, self.w_gate_up, offsets, n, True, self.rt.act)
                y = F.grouped_gemm_plain(act, None, self.w_down, offsets, n, False, torch.float32)
        if self.keep_routing:
            self.last_routing = (idx, w, probs)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        elif self.sI > 0:
            shared = self._shared_expert(x)
        return WeightedRowSum(y, inv_perm, w, shared, gate if shared is not None else None)


register_part("feed_forward", "swiglu_mlp", SwiGLUMLP)
register_part("feed_forward", "sparse_moe", SparseMoE)
