"""Plain, slow Qwen2-MoE: the oracle every engine test compares with.

Whole sequences, no cache, no batching, one function per part, float32 (or
float64 with ``dtype=torch.float64``) on whatever device the weights are on.
It shares no code with ``mini_infer_b200``: it reads ``config.json`` as a
dictionary and the checkpoint as a ``{name: tensor}`` dictionary.

The reference's own model code (src/model/transformer_model.cpp, src/layers/*,
src/kernels/*.cu) is CUDA + cuBLAS, FP16 only, accepts head sizes 64 and 128
only (src/kernels/paged_attn_kernel.cu:313-315) and cannot be built or run on
a CPU, so this file rests on the reference's formulas, cited per function, and
not on outputs of the reference.  Where the reference has a quirk that a
checkpoint's ``config.json`` contradicts (it never reads ``norm_topk_prob``,
``decoder_sparse_step``, ``mlp_only_layers``, ``use_sliding_window``), the
config wins, and the function says so.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- #
# parts
# --------------------------------------------------------------------------- #

def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """``y_j = x_j * rsqrt(mean_j(x_j^2) + eps) * w_j``.

    src/kernels/rmsnorm_kernel.cu:43-64 (sum of squares, ``rsqrtf(sum/D + eps)``,
    then ``x * rrms * w``; the add-one variant is off for this family).
    """
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def rope_inv_freq(head_dim: int, theta: float, dtype=torch.float32) -> Tensor:
    """``inv_freq[i] = 1 / theta^(2i/d)`` for ``i < d/2`` (src/layers/rope.cpp:20-29)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / head_dim)
    return inv.to(dtype)


def apply_rope(x: Tensor, positions: Tensor, theta: float) -> Tensor:
    """Half-split rotation of ``x [S, heads, d]`` by absolute ``positions [S]``.

    ``y_i = x_i cos - x_{i+d/2} sin``; ``y_{i+d/2} = x_{i+d/2} cos + x_i sin`` with
    angle ``pos * inv_freq[i]`` (src/kernels/rope_kernel.cu:46-53, angles
    src/kernels/rope_kernel.cu:65-77).  The reference rounds cos/sin to FP16
    tables; that rounding is not reproduced.
    """
    d = x.shape[-1]
    half = d // 2
    inv = rope_inv_freq(d, theta, torch.float32).to(x.device)
    ang = positions.to(torch.float32)[:, None] * inv[None, :]          # float32 product, as the kernel
    ang = ang.to(x.dtype)
    c = torch.cos(ang)[:, None, :]
    s = torch.sin(ang)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def attention_scores_softmax_pv(q: Tensor, k: Tensor, v: Tensor, window: int = 0) -> Tensor:
    """Causal grouped-query attention of one whole sequence.

    ``q [S, nh, d]``, ``k, v [S, nkv, d]``; head ``h`` reads kv head ``h // (nh/nkv)``
    (src/kernels/paged_attn_kernel.cu:130); score ``q.k / sqrt(d)``
    (src/layers/attention.cpp:849); key ``j`` is visible from query ``p`` iff
    ``j <= p`` (src/kernels/paged_attn_kernel.cu:228-231) and, with a window
    ``W > 0``, ``j >= p - W + 1`` (src/kernels/paged_attn_kernel.cu:232-236);
    softmax and the weighted sum of values as in :250-287.
    """
    S, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    scale = 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    pos = torch.arange(S, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[None, :] >= (pos[:, None] - window + 1)
    for h in range(nh):
        kh = k[:, h // g, :]
        vh = v[:, h // g, :]
        s = (q[:, h, :] @ kh.T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out


def attention(x: Tensor, w: Dict[str, Tensor], prefix: str, nh: int, nkv: int, d: int,
              theta: float, window: int) -> Tensor:
    """Projections with bias, rotation of q and k, attention, output projection.

    ``q = x Wq^T + bq`` etc. with row-major ``[out, in]`` weights
    (src/layers/attention.cpp:714-740), rotation of q and k only (:771-780),
    ``o = attn Wo^T`` without bias (:872-876).
    """
    S = x.shape[0]
    q = x @ w[prefix + "q_proj.weight"].T
    k = x @ w[prefix + "k_proj.weight"].T
    v = x @ w[prefix + "v_proj.weight"].T
    if prefix + "q_proj.bias" in w:
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    pos = torch.arange(S, device=x.device)
    q = apply_rope(q.view(S, nh, d), pos, theta)
    k = apply_rope(k.view(S, nkv, d), pos, theta)
    v = v.view(S, nkv, d)
    a = attention_scores_softmax_pv(q, k, v, window)
    return a.reshape(S, nh * d) @ w[prefix + "o_proj.weight"].T


def swiglu_mlp(x: Tensor, gate_w: Tensor, up_w: Tensor, down_w: Tensor) -> Tensor:
    """``(silu(x Wg^T) * (x Wu^T)) Wd^T`` with ``silu(g) = g / (1 + exp(-g))``.

    src/layers/mlp.cpp:255-300, src/kernels/swiglu_kernel.cu:16-26.
    """
    g = x @ gate_w.T
    u = x @ up_w.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ down_w.T


def route(x: Tensor, router_w: Tensor, top_k: int, norm_topk_prob: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """Router probabilities, chosen experts and their weights.

    Logits ``z = x Wg^T`` (src/layers/moe.cpp:215-220); ``K`` rounds of arg-max
    with strict ``>`` scanning experts upwards, so the lowest index wins a tie
    (src/kernels/moe_kernel.cu:28-47).  The reference then takes a softmax over
    the ``K`` chosen logits (:49-62), which equals softmax over all experts
    followed by renormalising the chosen ones: it always behaves as
    ``norm_topk_prob = true``.  Here the key is honoured: ``false`` keeps the
    plain softmax-over-all probabilities of the chosen experts.

    Returns ``(probs [S, E], idx [S, K], weights [S, K])``.
    """
    z = x @ router_w.T
    probs = torch.softmax(z, dim=-1)
    S, E = probs.shape
    idx = torch.empty(S, top_k, dtype=torch.long, device=x.device)
    work = probs.clone()
    for k in range(top_k):
        # torch.max over a dimension returns the first maximal index on CPU; make it explicit
        m = work.max(dim=-1, keepdim=True).values
        first = (work == m).to(torch.int64).argmax(dim=-1)
        idx[:, k] = first
        work.scatter_(1, first[:, None], float("-inf"))
    wts = probs.gather(1, idx)
    if norm_topk_prob:
        wts = wts / wts.sum(dim=-1, keepdim=True)
    return probs, idx, wts


def moe_block(x: Tensor, w: Dict[str, Tensor], prefix: str, num_experts: int, top_k: int,
              norm_topk_prob: bool, has_shared: bool,
              forced_idx: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """Routed experts in slot order, then the gated shared expert.

    ``out[t] = sum_k w[t,k] Expert_{idx[t,k]}(x[t])`` (src/layers/moe.cpp:229-270;
    the reference runs each used expert on all tokens and masks, the sum is the
    same), then ``out += sigmoid(x . w_sg) * Expert_shared(x)``
    (src/layers/moe.cpp:272-293, src/kernels/moe_kernel.cu:126-146).

    ``forced_idx`` replaces the arg-max choice (weights are still read from the
    probabilities): used to judge an engine whose near-tie went the other way.
    Returns ``(out, idx, probs)``.
    """
    probs, idx, wts = route(x, w[prefix + "gate.weight"], top_k, norm_topk_prob)
    if forced_idx is not None:
        idx = forced_idx.to(idx.device).long()
        wts = probs.gather(1, idx)
        if norm_topk_prob:
            wts = wts / wts.sum(dim=-1, keepdim=True)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(top_k):
            e = int(idx[t, k])
            p = f"{prefix}experts.{e}."
            y = swiglu_mlp(x[t:t + 1], w[p + "gate_proj.weight"], w[p + "up_proj.weight"],
                           w[p + "down_proj.weight"])
            out[t] += wts[t, k] * y[0]
    if has_shared:
        p = prefix + "shared_expert."
        sh = swiglu_mlp(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
        gamma = x @ w[prefix + "shared_expert_gate.weight"].T           # [S, 1]
        out = out + (1.0 / (1.0 + torch.exp(-gamma))) * sh
    return out, idx, probs


def moe_block_by_expert(x: Tensor, w: Dict[str, Tensor], prefix: str, num_experts: int, top_k: int,
                        norm_topk_prob: bool, has_shared: bool,
                        forced_idx: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """The same block as :func:`moe_block` with the loops turned inside out: for every expert, all
    the tokens routed to it at once.  Sums per token run over slots in the order of the experts'
    indices instead of the order of the slots, so results agree up to rounding; it exists because
    the token-by-token form is too slow at real layer sizes."""
    probs, idx, wts = route(x, w[prefix + "gate.weight"], top_k, norm_topk_prob)
    if forced_idx is not None:
        idx = forced_idx.to(idx.device).long()
        wts = probs.gather(1, idx)
        if norm_topk_prob:
            wts = wts / wts.sum(dim=-1, keepdim=True)
    out = torch.zeros_like(x)
    for e in range(num_experts):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        p = f"{prefix}experts.{e}."
        y = swiglu_mlp(x[tok], w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
        out.index_add_(0, tok, wts[tok, slot][:, None] * y)
    if has_shared:
        p = prefix + "shared_expert."
        sh = swiglu_mlp(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])
        gamma = x @ w[prefix + "shared_expert_gate.weight"].T
        out = out + (1.0 / (1.0 + torch.exp(-gamma))) * sh
    return out, idx, probs


# --------------------------------------------------------------------------- #
# the model
# --------------------------------------------------------------------------- #

def _cfg(cfg: dict, key: str, default):
    v = cfg.get(key, default)
    return default if v is None else v


def layer_is_sparse(cfg: dict, i: int) -> bool:
    """Sparse iff the model has experts, ``i`` is not in ``mlp_only_layers`` and
    ``(i + 1) % decoder_sparse_step == 0``.  The reference decides per model, not
    per layer (src/model/transformer_model.cpp:141-156)."""
    return (_cfg(cfg, "num_experts", 0) > 0 and i not in _cfg(cfg, "mlp_only_layers", [])
            and (i + 1) % _cfg(cfg, "decoder_sparse_step", 1) == 0)


def layer_window(cfg: dict, i: int) -> int:
    if _cfg(cfg, "use_sliding_window", False) and i >= _cfg(cfg, "max_window_layers", 0):
        return int(_cfg(cfg, "sliding_window", 0))
    return 0


def forward(cfg: dict, weights: Dict[str, Tensor], token_ids: Sequence[int], dtype=torch.float32,
            forced_routing: Optional[Dict[int, Tensor]] = None,
            record: Optional[dict] = None, by_expert: bool = False) -> Tensor:
    """Logits ``[S, V]`` of one whole sequence.

    Block: ``a = x + Attn(RMSNorm_in(x))``; ``y = a + FFN(RMSNorm_post(a))``
    (src/model/transformer_model.h:25-28, src/model/transformer_model.cpp:578-641);
    embedding without scaling (:561-565); final norm and ``lm_head``, which is
    the embedding matrix when ``tie_word_embeddings`` (:644-673, :355-361).

    ``record`` (a dict) receives per-layer routing (``idx``, ``probs``) and the
    hidden state after each layer.
    """
    w = weights if all(v.dtype == dtype for v in weights.values()) else {k: v.to(dtype) for k, v in weights.items()}
    dev = next(iter(w.values())).device
    ids = torch.as_tensor(list(token_ids), dtype=torch.long, device=dev)
    H = cfg["hidden_size"]
    nh = cfg["num_attention_heads"]
    nkv = _cfg(cfg, "num_key_value_heads", nh)
    d = _cfg(cfg, "head_dim", 0) or H // nh
    eps = float(_cfg(cfg, "rms_norm_eps", 1e-6))
    theta = float(_cfg(cfg, "rope_theta", 10000.0))
    h = w["model.embed_tokens.weight"][ids]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = rms_norm(h, w[p + "input_layernorm.weight"], eps)
        h = h + attention(x, w, p + "self_attn.", nh, nkv, d, theta, layer_window(cfg, i))
        x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        if layer_is_sparse(cfg, i):
            forced = forced_routing.get(i) if forced_routing else None
            if by_expert:
                y, idx, probs = moe_block_by_expert(
                    x, w, p + "mlp.", cfg["num_experts"], cfg["num_experts_per_tok"],
                    bool(_cfg(cfg, "norm_topk_prob", False)),
                    _cfg(cfg, "shared_expert_intermediate_size", 0) > 0, forced)
            else:
                y, idx, probs = moe_block(
                    x, w, p + "mlp.", cfg["num_experts"], cfg["num_experts_per_tok"],
                    bool(_cfg(cfg, "norm_topk_prob", False)),
                    _cfg(cfg, "shared_expert_intermediate_size", 0) > 0, forced)
            if record is not None:
                record.setdefault("routing", {})[i] = (idx, probs)
        else:
            y = swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                           w[p + "mlp.down_proj.weight"])
        h = h + y
        if record is not None:
            record.setdefault("hidden", {})[i] = h
    x = rms_norm(h, w["model.norm.weight"], eps)
    lm = w["model.embed_tokens.weight"] if _cfg(cfg, "tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ lm.T


# --------------------------------------------------------------------------- #
# sampling (the engine's own rules; the reference's top-p kernel falls back to
# greedy above 30000 vocabulary entries, src/kernels/sampling_kernel.cu:216-220,
# and picks uniformly inside the nucleus, :186-199 - neither is reproduced)
# --------------------------------------------------------------------------- #

_PHILOX_M0 = 0xD2511F53
_PHILOX_M1 = 0xCD9E8D57
_PHILOX_W0 = 0x9E3779B9
_PHILOX_W1 = 0xBB67AE85
_MASK = 0xFFFFFFFF


def philox4x32(counter: Tuple[int, int, int, int], key: Tuple[int, int], rounds: int = 10):
    """Philox-4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(rounds):
        p0 = _PHILOX_M0 * c0
        p1 = _PHILOX_M1 * c2
        hi0, lo0 = (p0 >> 32) & _MASK, p0 & _MASK
        hi1, lo1 = (p1 >> 32) & _MASK, p1 & _MASK
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & _MASK, lo1, (hi0 ^ c3 ^ k1) & _MASK, lo0
        k0 = (k0 + _PHILOX_W0) & _MASK
        k1 = (k1 + _PHILOX_W1) & _MASK
    return c0, c1, c2, c3


def uniform_for(seed: int, stream: int, index: int) -> float:
    """The uniform in [0, 1) that decides token number ``index`` of sampling
    stream ``stream`` under ``seed``: 24 high bits of the first Philox word."""
    r = philox4x32((index & _MASK, (index >> 32) & _MASK, stream & _MASK, (stream >> 32) & _MASK),
                   (seed & _MASK, (seed >> 32) & _MASK))
    return (r[0] >> 8) * (1.0 / 16777216.0)


def greedy(logits: Tensor) -> int:
    """Arg-max; the lowest index wins among equal logits."""
    m = logits.max()
    return int((logits == m).nonzero()[0, 0])


def nucleus_cdf(logits: Tensor, temperature: float, top_p: float) -> Tuple[Tensor, Tensor]:
    """``p = softmax(logits / T)``; with ``top_p < 1`` the nucleus is every token whose probability is at
    least ``tau``, the largest probability value for which the tokens at or above it hold a mass of at
    least ``top_p``.  Returns the cumulative nucleus mass in index order (float64, not normalised) and
    the nucleus as a mask."""
    p = torch.softmax(logits.to(torch.float32) / temperature, dim=-1)
    keep = torch.ones_like(p, dtype=torch.bool)
    if top_p < 1.0:
        vals = torch.sort(p, descending=True).values
        cum = torch.cumsum(vals.to(torch.float64), dim=0)
        n = int((cum < top_p).sum()) + 1
        tau = vals[min(n, vals.numel()) - 1]
        keep = p >= tau
    pk = torch.where(keep, p, torch.zeros_like(p)).to(torch.float64)
    return torch.cumsum(pk, dim=0), keep


def sample(logits: Tensor, temperature: float, top_p: float, u: float) -> int:
    """The token is the first, in index order, whose cumulative nucleus mass (:func:`nucleus_cdf`)
    exceeds ``u * (nucleus mass)``; arg-max at temperature 0."""
    if temperature <= 0.0:
        return greedy(logits)
    cdf, keep = nucleus_cdf(logits, temperature, top_p)
    target = u * float(cdf[-1])
    hit = (cdf > target).nonzero()
    if hit.numel() == 0:
        return int(keep.nonzero()[-1, 0])
    return int(hit[0, 0])


def generate(cfg: dict, weights: Dict[str, Tensor], prompt: Sequence[int], max_new_tokens: int,
             temperature: float = 0.0, top_p: float = 1.0, seed: int = 42, stream: int = 0,
             stop_ids: Sequence[int] = (), dtype=torch.float32) -> List[int]:
    """Token by token, recomputing the whole sequence each time."""
    ids = list(prompt)
    out: List[int] = []
    for n in range(max_new_tokens):
        logits = forward(cfg, weights, ids, dtype)[-1]
        tok = sample(logits, temperature, top_p, uniform_for(seed, stream, n))
        out.append(tok)
        ids.append(tok)
        if tok in stop_ids:
            break
    return out
