"""Grouped-query attention over the paged cache.

Reference: src/layers/attention.cpp:666-878 (three cuBLAS products, three bias
kernels, two rotary kernels, two scatter kernels, the paged attention kernel,
one more product, with block tables rebuilt and uploaded in every layer).
Here: one library product for q, k and v together, one kernel for bias +
rotation + cache write, one attention kernel chosen by the shape of the batch,
one library product for the output.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import part_class, register_part
from ..config.spec import PartSpec
from ..ops import functional as F
from .base import CacheBinding, KVNeed, Mixer, Runtime, StepContext, TensorDecl, linear
from .tuning import TUNING


class GQAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``bias``
    (q/k/v projections carry a bias), ``window`` (0 = all keys), ``position``
    (a ``PartSpec`` of category ``position``), ``shares_cache`` (this layer has no
    k/v projections and reads the cache another schedule entry wrote).

    Tensors: ``<prefix>{q,k,v}_proj.weight [out, hidden]``, ``.bias [out]`` if
    ``bias``, ``<prefix>o_proj.weight [hidden, num_heads*head_dim]``.
    """

    graph_safe = True

    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        p = self.params
        self.H = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.bias = bool(p.get("bias", False))
        self.window = int(p.get("window", 0))
        self.shares_cache = bool(p.get("shares_cache", False))
        pos: PartSpec = p.get("position") or PartSpec("none")
        self.position = part_class("position", pos.kind)(pos.params, prefix)
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads are not a multiple of {self.nkv} key/value heads")
        if self.d % 2 or not 2 <= self.d <= 256:
            raise ValueError(f"attention: head_dim {self.d} must be even and at most 256")

    # -- weights ----------------------------------------------------------- #
    def _proj_names(self) -> List[str]:
        return ["q_proj"] if self.shares_cache else ["q_proj", "k_proj", "v_proj"]

    def tensor_decls(self) -> List[TensorDecl]:
        out = []
        for n in self._proj_names():
            rows = (self.nh if n == "q_proj" else self.nkv) * self.d
            out.append(TensorDecl(f"{self.prefix}{n}.weight", (rows, self.H), "matrix"))
            if self.bias:
                out.append(TensorDecl(f"{self.prefix}{n}.bias", (rows,), "bias"))
        out.append(TensorDecl(f"{self.prefix}o_proj.weight", (self.H, self.nh * self.d), "matrix"))
        return out

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        prec, dev = rt.precision, rt.device
        names = self._proj_names()
        self.w_qkv = torch.cat([prec.matrix(tensors[f"{self.prefix}{n}.weight"], dev) for n in names], dim=0)
        self.b_qkv = None
        if self.bias:
            bs = [prec.small(tensors[f"{self.prefix}{n}.bias"], dev) for n in names]
            if len({b.dtype for b in bs}) > 1:
                bs = [b.float() for b in bs]
            self.b_qkv = torch.cat(bs, dim=0).contiguous()
        self.w_o = prec.matrix(tensors[f"{self.prefix}o_proj.weight"], dev)
        self.inv_freq = self.position.table(dev)
        self.rot_dim = self.position.rot_dim if self.inv_freq is not None else self.d
        self._tensor_core_prefill = rt.act == torch.bfloat16 and F.prefill_attention_supported(self.d)
        # decode-sized steps: projection, bias, rotation and cache write in one kernel
        self._fused_qkv_rows = 0
        if (rt.act == torch.bfloat16 and not self.shares_cache
                and F.qkv_skinny_supported(self.H, self.d, self.rot_dim if self.inv_freq is not None else 0)):
            self._fused_qkv_rows = F.qkv_skinny_max_rows()
            self._b_qkv_f32 = None if self.b_qkv is None else self.b_qkv.float()

    def prefetch_first(self, ctx: StepContext, cache: Optional[CacheBinding]) -> None:
        """The q/k/v weights.  (Asking for the cache pages of the batch as well was measured and not kept:
        the split-KV kernel is bound by the latency of its one wave, not by where its lines come from.)"""
        F.l2_prefetch(self.w_qkv)

    # -- cache ------------------------------------------------------------- #
    def cache_need(self):
        return KVNeed(self.nkv, self.d, self.window)

    def scratch_need(self, max_requests: int, max_context: int) -> Dict[str, int]:
        if not F.decode_attention_supported(self.d):
            return {}
        splits = -(-max_context // min(F.DECODE_SPLIT_SIZES))
        return {"attn_part_o": max_requests * self.nh * splits * self.d,
                "attn_part_ml": max_requests * self.nh * splits * 2}

    # -- forward ----------------------------------------------------------- #
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        view = ctx.kv_groups[cache.group]
        kc = view.k[cache.layer_slot]
        vc = view.v[cache.layer_slot]
        if ctx.num_tokens <= self._fused_qkv_rows:
            q = F.qkv_skinny(x, self.w_qkv, self._b_qkv_f32, ctx.positions, self.inv_freq, view.slot_mapping,
                             kc, vc, self.nh, self.nkv, self.d, view.page_size)
            if ctx.prefetch is not None:
                ctx.prefetch((self.w_o,))       # arrives while the attention over the cache runs
        else:
            qkv = linear(x, self.w_qkv, torch.float32)
            nkv_in = 0 if self.shares_cache else self.nkv
            q = F.qkv_post(qkv, self.b_qkv, ctx.positions, self.inv_freq, self.rot_dim,
                           view.slot_mapping if nkv_in else None, kc if nkv_in else None, vc if nkv_in else None,
                           self.nh, nkv_in, self.d, view.page_size, self.rt.act)
        # The float32 path takes one attention kernel for every step (key tiles at absolute positions: a
        # query's sums run in the same order however its step was cut or batched); the bfloat16 path picks
        # the fastest kernel for the step's shape.
        if self.rt.act == torch.float32:
            a = F.attention(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len, self.window)
        elif ctx.all_decode and "attn_part_o" in ctx.scratch and F.decode_attention_supported(self.d):
            # one or two requests alone cannot fill the device with splits of 512 keys
            split = TUNING.decode_split(ctx.num_requests, F.decode_split_size())
            splits = -(-ctx.max_kv_len // split)
            a = F.decode_attention(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len,
                                   ctx.scratch["attn_part_o"], ctx.scratch["attn_part_ml"], splits, self.window,
                                   split=split)
        elif self._tensor_core_prefill:
            prefill = (F.prefill_attention_tc if F.prefill_attention_tc_supported(self.d, view.page_size)
                       else F.prefill_attention)
            n = ctx.num_leading_decodes
            if (TUNING.mixed_step_decode_kernel_min_requests <= n < ctx.num_requests
                    and "attn_part_o" in ctx.scratch and F.decode_attention_supported(self.d)):
                # A prompt portion beside decoding requests: the requests that bring one token stand first.
                # Their attention is a stream over their whole caches, which the split-KV kernel reads at
                # the memory's speed; a prefill kernel would spend a 128-query tile on each of them.  Both
                # kernels index the step's rows through q_start, so each takes its requests and all rows.
                a = torch.empty_like(q)
                split = F.decode_split_size()
                F.decode_attention(q[:n], kc, vc, view.block_table[:n], ctx.q_start[:n + 1], ctx.kv_len[:n],
                                   ctx.scratch["attn_part_o"], ctx.scratch["attn_part_ml"],
                                   -(-ctx.leading_decodes_max_kv_len // split), self.window, out=a[:n], split=split)
                prefill(q, kc, vc, view.block_table[n:], ctx.q_start[n:], ctx.kv_len[n:], ctx.max_q_len, self.window,
                        out=a)
            else:
                a = prefill(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len, self.window)
        else:
            a = F.attention(q, kc, vc, view.block_table, ctx.q_start, ctx.kv_len, ctx.max_q_len, self.window)
        return linear(a.view(ctx.num_tokens, self.nh * self.d), self.w_o, torch.float32)


register_part("mixer", "gqa_attention", GQAttention)
