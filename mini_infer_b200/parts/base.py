"""Interfaces of the parts a model is put together from.

A part is built from a :class:`~mini_infer_b200.config.spec.PartSpec` (its kind
and constants) and a checkpoint prefix; it declares the tensors it needs,
takes them at load time, and runs on the tensors the step hands it.  No part
imports a model or asks which model it is in.

Categories and what each must provide:

``norm``          ``apply(hidden, delta, rows) -> normed``: add ``delta`` into the
                  float32 residual stream ``hidden`` (if given) and return the
                  normalised rows in the activation dtype.
``position``      ``table(device)`` and ``rot_dim``: the rotation frequencies the
                  attention kernels apply to queries and keys (or none).
``mixer``         ``cache_need()`` (what it keeps per token or per request),
                  ``forward(x, ctx, cache) -> y`` with ``x [T, H]`` activations and
                  ``y [T, H]`` float32.
``feed_forward``  ``forward(x, ctx) -> y``, same shapes.
``block``         ``forward(layer, hidden, pending, ctx, cache) -> pending``: the
                  arrangement of norms, mixer and feed-forward around the residual.
``embedding``     ``forward(token_ids) -> hidden`` float32.
``lm_head``       ``forward(x) -> logits`` float32.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- #
# tensors a part expects in the checkpoint
# --------------------------------------------------------------------------- #

@dataclass(frozen=True)
class TensorDecl:
    """One checkpoint tensor: full name, shape, and its role.

    ``role`` decides the random initialisation (``matrix``, ``bias``: N(0, 0.02);
    ``norm``: 1 + N(0, 0.02)) and the storage rule: in the bfloat16 path a
    ``matrix`` feeds tensor-core products and is held in bfloat16, while ``norm``
    and ``bias`` tensors, which are only ever read into 32-bit arithmetic, keep
    32 bits if the file stores them so.
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"


# --------------------------------------------------------------------------- #
# precision path
# --------------------------------------------------------------------------- #

@dataclass(frozen=True)
class Precision:
    """One of the two paths through the whole model.

    ``float32``: weights, activations, cache and every product in true 32-bit
    (TF32 and reduced-precision reductions are switched off).
    ``bfloat16``: matrices, activations between products and the cache in
    bfloat16; the residual stream, norms, softmax, router, rotation angles and
    every accumulation in float32.
    """

    name: str

    @property
    def act(self) -> torch.dtype:
        return torch.float32 if self.name == "float32" else torch.bfloat16

    def matrix(self, t: torch.Tensor, device) -> torch.Tensor:
        return t.to(device=device, dtype=self.act).contiguous()

    def small(self, t: torch.Tensor, device) -> torch.Tensor:
        """Norm weights and biases: widened in the 32-bit path; otherwise kept as stored
        (float16 is widened to float32: it has no kernel type of its own)."""
        if self.name == "float32" or t.dtype == torch.float16:
            return t.to(device=device, dtype=torch.float32).contiguous()
        return t.to(device=device).contiguous()


def precision_from_name(name: str) -> Precision:
    alias = {"fp32": "float32", "float32": "float32", "f32": "float32",
             "bf16": "bfloat16", "bfloat16": "bfloat16"}
    if name not in alias:
        raise ValueError(f"unknown dtype '{name}': choose bfloat16 or float32")
    return Precision(alias[name])


@dataclass
class Runtime:
    """What a part needs to know about where it runs."""

    precision: Precision
    device: torch.device

    @property
    def act(self) -> torch.dtype:
        return self.precision.act


def configure_matmul_exactness() -> None:
    """No TF32, no reduced-precision split-k reductions: library products accumulate in float32.  These are
    process-wide PyTorch switches: whatever else multiplies matrices in this process afterwards runs under
    them as well."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    torch.set_float32_matmul_precision("highest")


# --------------------------------------------------------------------------- #
# what a part keeps between steps: see cache/needs.py
# --------------------------------------------------------------------------- #

from ..cache.needs import KVNeed, PagedCacheNeed, StateNeed  # noqa: E402  (re-exported for part authors)


# --------------------------------------------------------------------------- #
# what a step hands to the parts
# --------------------------------------------------------------------------- #

@dataclass
class KVGroupView:
    """Device metadata of one cache group for the current step, and the group's tensors: for every
    tensor its need names, ``[layers_in_group, pages, *shape of one page]`` (for keys and values:
    ``k`` and ``v`` of ``[layers, pages, nkv, page_size, d]``)."""

    block_table: torch.Tensor      # [B, max_pages] int32, -1 = no page
    slot_mapping: torch.Tensor     # [T] int32: page * page_size + offset of each new token
    page_size: int
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)

    @property
    def k(self) -> torch.Tensor:
        return self.tensors["k"]

    @property
    def v(self) -> torch.Tensor:
        return self.tensors["v"]


@dataclass
class CacheBinding:
    """Where one schedule entry's mixer finds its cache."""

    kind: str                       # "kv" | "state" | "none"
    group: int = -1                 # index of the KV group, or of the state tensor
    layer_slot: int = -1            # layer index inside the KV group
    writes: bool = True             # False: reads the cache another entry writes


@dataclass
class StepContext:
    """Everything about the current batch that parts may read.  All device tensors are int32."""

    num_tokens: int
    num_requests: int
    max_q_len: int                  # longest portion in the batch
    max_kv_len: int                 # longest context in the batch (after this step)
    all_decode: bool                # every request brings exactly one token
    token_ids: torch.Tensor         # [T]
    positions: torch.Tensor         # [T] absolute position of each token in its request
    q_start: torch.Tensor           # [B+1] first token of each request in the batch
    kv_len: torch.Tensor            # [B] context length of each request after this step
    req_of_token: torch.Tensor      # [T]
    state_slot: torch.Tensor        # [B] state slot of each request
    fresh: torch.Tensor             # [B] 1 if the request's first token is in this step
    kv_groups: List[KVGroupView] = field(default_factory=list)
    states: List[torch.Tensor] = field(default_factory=list)   # [slots, *shape] per state user
    scratch: Dict[str, torch.Tensor] = field(default_factory=dict)
    # Hints for decode-sized steps (None when switched off).  ``prefetch(what)``: once the kernels queued so
    # far have finished, ask L2 on a second stream, beside whatever is queued next, for ``what``: a sequence
    # of weight tensors, or a function that issues the requests itself.  ``prefetch_upcoming``: a function
    # that asks for what the layer after this one reads first (set by the model before each layer), so
    # that a layer's last part can call ``ctx.prefetch(ctx.prefetch_upcoming)`` while its own tail runs.
    prefetch: Optional[Any] = None
    prefetch_upcoming: Optional[Any] = None
    # launch this step's decode-sized kernels as programmatic dependents of the kernels before them
    dependent_launch: bool = False
    # how many requests at the front of the step bring exactly one token (the scheduler puts decoding
    # requests first), and the longest context among them: a mixer may serve them with its decode kernel
    # and the prompt portions behind them with its prefill kernel
    num_leading_decodes: int = 0
    leading_decodes_max_kv_len: int = 0
    # the last rows of the step (one token each) belong to no request: they fill a captured batch up to its
    # size, are written nowhere and their logits are dropped
    rows_of_no_request: int = 0
    # host copies, for parts written in plain PyTorch (tests' toy parts)
    host_q_start: Sequence[int] = ()
    host_kv_len: Sequence[int] = ()
    host_state_slot: Sequence[int] = ()


# --------------------------------------------------------------------------- #
# part base classes
# --------------------------------------------------------------------------- #

class Part:
    category = ""

    def __init__(self, params: Mapping[str, Any], prefix: str):
        self.params = dict(params)
        self.prefix = prefix

    def tensor_decls(self) -> List[TensorDecl]:
        return []

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        """Take the declared tensors (CPU or device, stored dtype) and keep what forward needs."""
        self.rt = rt

    def prefetch_first(self, ctx: "StepContext", cache: Optional["CacheBinding"]) -> None:
        """Ask L2 (``ops.functional.l2_prefetch*``, on the current stream) for what this part reads first
        in a decode-sized step: called on a second stream while the part before it runs its last,
        latency-bound kernels.  Default: nothing."""

    # -- a forward pass captured as a CUDA graph -------------------------------------------- #
    def capture_key(self):
        """A hashable value for every setting of this part that changes which kernels its forward
        launches (a recording switch, say): a captured pass is replayed only under the same key."""
        return None

    def side_outputs(self):
        """What forward leaves on the part beside its return value (recorded routing, say), or None.
        Tensors made while a pass was captured are refreshed in place by every replay; the runner
        keeps them with the graph and hands them back through :meth:`adopt_side_outputs` after a
        replay, so that a reader finds them where an eager pass would have left them."""
        return None

    def adopt_side_outputs(self, outputs) -> None:
        pass


class Deferred:
    """A part's output that has not been written out yet.  A consumer that can fold the computation
    into its own kernel says so with ``accepts_deferred`` and is handed the object; every other consumer
    gets the tensor (:func:`resolve`)."""

    def materialize(self) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class WeightedRowSum(Deferred):
    """``out[t] = sum_k weights[t, k] * rows[index[t, k]] + scale[t] * extra[t]`` (float32; without
    ``index`` the rows are taken in order, ``rows[t * K + k]``; ``extra`` and ``scale`` come together
    or not at all)."""

    rows: torch.Tensor
    index: Optional[torch.Tensor]
    weights: torch.Tensor
    extra: Optional[torch.Tensor]
    scale: Optional[torch.Tensor]

    def materialize(self) -> torch.Tensor:
        from ..ops import functional as F
        return F.moe_combine(self.rows, self.index, self.weights, self.extra, self.scale)


def resolve(pending):
    return pending.materialize() if isinstance(pending, Deferred) else pending


class Norm(Part):
    category = "norm"
    accepts_deferred = False    # True: ``apply`` takes a Deferred as ``delta``

    def apply(self, hidden: torch.Tensor, delta: Optional[torch.Tensor],
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def rms_parameters(self) -> Optional[Tuple[torch.Tensor, float]]:
        """``(weight, eps)`` if this norm is ``x * rsqrt(mean(x^2) + eps) * weight`` and nothing else, so
        that the part that follows may run it inside a kernel of its own; None otherwise."""
        return None


def apply_norm(norm: "Norm", hidden: torch.Tensor, pending, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``norm.apply`` with a pending output that may be deferred."""
    if isinstance(pending, Deferred) and not norm.accepts_deferred:
        pending = pending.materialize()
    return norm.apply(hidden, pending, rows)


class PositionEncoding(Part):
    category = "position"
    rot_dim = 0

    def table(self, device) -> Optional[torch.Tensor]:
        return None


class Mixer(Part):
    category = "mixer"

    def cache_need(self):
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheBinding) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def forward_deferred(self, x: torch.Tensor, ctx: StepContext):
        """As ``forward``, but the result may be a :class:`Deferred` whose last step the consumer runs."""
        return self.forward(x, ctx)

    def forward_from_residual(self, hidden: torch.Tensor, delta, norm: "Norm", ctx: StepContext):
        """``forward_deferred(norm(hidden + delta))`` with ``hidden`` updated; a feed-forward may
        override it to run the norm inside its first kernel."""
        return self.forward_deferred(apply_norm(norm, hidden, delta), ctx)


class Embedding(Part):
    category = "embedding"

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class LMHead(Part):
    category = "lm_head"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of a layer's parts around the residual stream.

    ``roles`` maps every role the arrangement wires to its registry category; a layer description must
    provide exactly these (it is checked when the layer is built).  ``forward`` gets the built layer
    (parts by role: ``layer.mixer`` or ``layer.parts["mixer"]``), the float32 residual stream, the output
    of the part before that has not been added yet (``pending``), and ``caches``: for every role that
    keeps a cache, where it finds it."""

    category = "block"
    accepts_deferred = False    # True: ``forward`` takes a Deferred as ``pending`` and may return one
    roles: Mapping[str, str] = {}

    def forward(self, layer: "BuiltLayer", hidden: torch.Tensor, pending: Optional[torch.Tensor],
                ctx: StepContext, caches: Mapping[str, CacheBinding]) -> torch.Tensor:
        raise NotImplementedError

    def prefetch_layer(self, layer: "BuiltLayer", ctx: StepContext, caches: Mapping[str, CacheBinding]) -> None:
        """``prefetch_first`` of whichever part of ``layer`` this arrangement runs first."""


class BuiltLayer:
    """The instantiated parts of one ``LayerSpec``: ``block`` and ``parts`` by role (a role can be read
    as an attribute: ``layer.mixer``)."""

    def __init__(self, name: str, block: Block, parts: Dict[str, Part]):
        self.name = name
        self.block = block
        self.parts = dict(parts)

    def __getattr__(self, role: str) -> Part:
        parts = self.__dict__.get("parts")
        if parts is not None and role in parts:
            return parts[role]
        raise AttributeError(f"layer '{self.__dict__.get('name')}' has no part in the role '{role}'")

    def all_parts(self) -> List[Part]:
        return list(self.parts.values()) + [self.block]


from .tuning import TUNING  # noqa: E402


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
    """``silu(x @ w_gate.T) * (x @ w_up.T)`` in the activation dtype; ``w_gate_up`` holds the gate
    rows then the up rows (src/layers/mlp.cpp:255-279 runs two products and an elementwise kernel)."""
    from ..ops import functional as F
    if x.is_cuda and x.shape[0] <= TUNING.dense_skinny_max_tokens and F.dense_skinny_takes(x, w_gate_up):
        return F.dense_skinny(x, w_gate_up, swiglu_pair=True)
    return F.swiglu(linear(x, w_gate_up, act_dtype))


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``x @ w.T``; ``w`` is ``[out, in]`` as stored in checkpoints.

    bfloat16 path: the library product the reference also uses for every dense projection (cuBLAS,
    src/layers/attention.cpp:45-55, src/layers/mlp.cpp:120-130), accumulating in float32, or the engine's
    own decode kernel for the smallest steps.  float32 path (both operands float32): the engine's own
    CUDA-core kernel, which adds in one fixed order whatever the number of rows, so that this path gives
    the same bits however the work is cut and batched."""
    from ..ops import functional as F
    if x.is_cuda and x.dtype == torch.float32 and w.dtype == torch.float32 and out_dtype == torch.float32:
        return F.dense_f32(x, w)
    if out_dtype == torch.float32 and x.is_cuda and x.shape[0] <= TUNING.dense_skinny_max_tokens:
        if F.dense_skinny_takes(x, w):
            return F.dense_skinny(x, w)
    if x.dtype == out_dtype:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)
