"""Python faces of the CUDA kernels: check the tensors, pass the pointers.

Every function runs on the current CUDA stream of the tensors' device and
returns its output tensor.  Shapes a kernel cannot take are refused with an
error; nothing falls back to PyTorch.
"""

from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch

from .library import KernelError, check, library

F32 = torch.float32
BF16 = torch.bfloat16
I32 = torch.int32

_CODES = {torch.float32: 0, torch.bfloat16: 1}


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise TypeError(f"{what}: dtype {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _chk(t: Optional[torch.Tensor], what: str, dtype=None, shape=None) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise RuntimeError(f"{what}: tensor is on {t.device}; the kernels run on CUDA only and have no fallback")
    if not t.is_contiguous():
        raise ValueError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{what}: expected {dtype}, got {t.dtype}")
    if shape is not None:
        actual = t.shape
        bad = len(shape) != len(actual)
        if not bad:
            for s, a in zip(shape, actual):
                if s is not None and s != a:
                    bad = True
                    break
        if bad:
            raise ValueError(f"{what}: expected shape {list(shape)}, got {list(actual)}")


# --------------------------------------------------------------------------- #
# Debug mode: with MINI_INFER_DEBUG_BOUNDS=1 in the environment every index that a kernel will follow
# (token ids, row lists, cache slots, block tables, lengths, expert choices and offsets, permutations) is
# checked on the host before the launch, and a bad one raises a KernelError that names the tensor, the
# first bad place and its value, instead of becoming an access outside a buffer.  It synchronises the
# device at every op, so it is for chasing a fault, not for serving.  (The reference checks none of these;
# its kernels return silently on a size they do not take, src/kernels/paged_attn_kernel.cu:313-315.)
# --------------------------------------------------------------------------- #
import os as _os

DEBUG_BOUNDS = _os.environ.get("MINI_INFER_DEBUG_BOUNDS", "0") not in ("", "0")
debug_checks_run = 0


def _bad(what: str, msg: str):
    from .library import KernelError
    raise KernelError(f"{what}: {msg} (found by MINI_INFER_DEBUG_BOUNDS before the launch)")


def _dbg_range(t: Optional[torch.Tensor], lo: int, hi: int, what: str) -> None:
    """Every element of ``t`` lies in ``[lo, hi)``."""
    global debug_checks_run
    if t is None or t.numel() == 0:
        return
    debug_checks_run += 1
    flat = t.reshape(-1)
    bad = ((flat < lo) | (flat >= hi)).nonzero()
    if bad.numel():
        i = int(bad[0, 0])
        _bad(what, f"element {i} is {int(flat[i])}, outside [{lo}, {hi})")


def _dbg_offsets(offsets: torch.Tensor, n_rows: int, what: str) -> None:
    """Expert offsets rise from 0 to the number of rows."""
    global debug_checks_run
    debug_checks_run += 1
    o = offsets.cpu().tolist()
    if o[0] != 0 or o[-1] != n_rows or any(b < a for a, b in zip(o, o[1:])):
        _bad(what, f"offsets {o[:8]}... do not rise from 0 to {n_rows}")


def _dbg_batch(what: str, q_start: torch.Tensor, kv_len: torch.Tensor, block_table: torch.Tensor, T: int,
               num_pages: int, page_size: int, window: int, max_q_len: Optional[int] = None) -> None:
    """The layout of a ragged batch over a paged cache: ``q_start`` rises within 0 .. T (a call may cover
    only the first or the last requests of a step's rows), every request's length covers its new tokens and
    fits its table, and every page that a query of this step reads (all of them, or those its window reaches)
    is a real page."""
    global debug_checks_run
    debug_checks_run += 1
    qs, kv, bt = q_start.cpu().tolist(), kv_len.cpu().tolist(), block_table.cpu()
    B, max_pages = bt.shape
    if qs[0] < 0 or qs[-1] > T or any(b <= a for a, b in zip(qs, qs[1:])):
        _bad(what, f"q_start {qs} does not rise within 0 .. {T}")
    for b in range(B):
        n_q, n = qs[b + 1] - qs[b], kv[b]
        if max_q_len is not None and n_q > max_q_len:
            _bad(what, f"request {b} brings {n_q} tokens, max_q_len says {max_q_len}")
        if n < n_q or n > max_pages * page_size:
            _bad(what, f"request {b}: kv_len {n} with {n_q} new tokens and a table of {max_pages} pages of {page_size}")
        first = 0 if window <= 0 else max(0, n - n_q - window + 1)
        row = bt[b]
        for i in range(first // page_size, -(-n // page_size)):
            p = int(row[i])
            if not 0 <= p < num_pages:
                _bad(what, f"request {b} reads page entry {i} = {p}, the cache has {num_pages} pages")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device, as the integer the launchers take."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


# --------------------------------------------------------------------------- #

def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` as float32 ``[T, H]``."""
    _chk(ids, "embed_gather ids", I32)
    _chk(table, "embed_gather table")
    T = ids.numel()
    V, H = table.shape
    if out is None:
        out = torch.empty(T, H, dtype=F32, device=table.device)
    _chk(out, "embed_gather out", F32, (T, H))
    if DEBUG_BOUNDS:
        _dbg_range(ids, 0, V, "embed_gather ids")
    check(library().mi_embed_gather(_ptr(ids), _ptr(table), _code(table, "embed_gather table"), _ptr(out),
                                    T, H, V, _stream()), "embed_gather")
    return out


def add_rmsnorm(hidden: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``hidden += delta`` (if given; written back unless ``rows``), then RMSNorm.

    ``rows`` (int32) selects and orders the rows to normalise; ``hidden`` is then
    left untouched.
    """
    _chk(hidden, "add_rmsnorm hidden", F32)
    T, H = hidden.shape
    _chk(delta, "add_rmsnorm delta", F32, (T, H))
    _chk(weight, "add_rmsnorm weight", None, (H,))
    _chk(rows, "add_rmsnorm rows", I32)
    n = T if rows is None else rows.numel()
    if out is None:
        out = torch.empty(n, H, dtype=out_dtype, device=hidden.device)
    _chk(out, "add_rmsnorm out", out_dtype, (n, H))
    if DEBUG_BOUNDS:
        _dbg_range(rows, 0, T, "add_rmsnorm rows")
    check(library().mi_add_rmsnorm(_ptr(hidden), _ptr(delta), _ptr(rows), _ptr(weight),
                                   _code(weight, "add_rmsnorm weight"), _ptr(out), _code(out, "add_rmsnorm out"),
                                   n, H, float(eps), _stream()), "add_rmsnorm")
    return out


def qkv_post(qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
             inv_freq: Optional[torch.Tensor], rot_dim: int, slot_mapping: Optional[torch.Tensor],
             k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], nh: int, nkv: int, d: int,
             page_size: int, out_dtype: torch.dtype, q_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Bias, rotary position encoding of q and k, cache write of k and v.

    ``qkv`` is float32 ``[T, (nh + 2*nkv) * d]`` (``nkv = 0``: queries only, nothing
    is written).  ``k_cache``/``v_cache`` are one layer's ``[pages, nkv, page_size, d]``.
    Returns ``q [T, nh, d]`` in ``out_dtype``.
    """
    _chk(qkv, "qkv_post qkv", F32)
    T = qkv.shape[0]
    width = (nh + 2 * nkv) * d
    _chk(qkv, "qkv_post qkv", F32, (T, width))
    _chk(bias, "qkv_post bias", None, (width,))
    _chk(positions, "qkv_post positions", I32, (T,))
    _chk(inv_freq, "qkv_post inv_freq", F32)
    if inv_freq is not None and inv_freq.numel() != rot_dim // 2:
        raise ValueError(f"qkv_post: {inv_freq.numel()} frequencies for {rot_dim} rotary dims")
    if nkv > 0:
        _chk(slot_mapping, "qkv_post slot_mapping", I32, (T,))
        _chk(k_cache, "qkv_post k_cache", out_dtype, (None, nkv, page_size, d))
        _chk(v_cache, "qkv_post v_cache", out_dtype, (None, nkv, page_size, d))
        if slot_mapping is None or k_cache is None or v_cache is None:
            raise ValueError("qkv_post: key/value heads need a cache and a slot mapping")
    if q_out is None:
        q_out = torch.empty(T, nh, d, dtype=out_dtype, device=qkv.device)
    _chk(q_out, "qkv_post q_out", out_dtype, (T, nh, d))
    wcode = _code(bias, "qkv_post bias") if bias is not None else 0
    if DEBUG_BOUNDS and nkv > 0:
        _dbg_range(slot_mapping, -1, k_cache.shape[0] * page_size, "qkv_post slot_mapping")     # -1: not cached
    check(library().mi_qkv_post(_ptr(qkv), _ptr(bias), wcode, _ptr(positions), _ptr(inv_freq),
                                _ptr(slot_mapping), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                _code(q_out, "qkv_post q_out"), T, nh, nkv, d, rot_dim, page_size, _stream()),
          "qkv_post")
    return q_out


def swiglu(gu: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gu[:, :I]) * gu[:, I:]`` for ``gu [T, 2I]``."""
    _chk(gu, "swiglu input")
    T, two_i = gu.shape
    if two_i % 2:
        raise ValueError("swiglu: the input width must be even (gate | up)")
    inter = two_i // 2
    if out is None:
        out = torch.empty(T, inter, dtype=gu.dtype, device=gu.device)
    _chk(out, "swiglu out", gu.dtype, (T, inter))
    check(library().mi_swiglu(_ptr(gu), _ptr(out), _code(gu, "swiglu input"), T, inter, _stream()), "swiglu")
    return out


def moe_combine(y: torch.Tensor, inv_perm: Optional[torch.Tensor], weights: torch.Tensor,
                shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_k weights[t,k] * y[inv_perm[t,k]] + gate[t] * shared[t]`` (float32);
    without ``inv_perm`` the rows of ``y`` are indexed by pair, ``y[t*K + k]``."""
    T, K = weights.shape
    _chk(y, "moe_combine y", F32, (T * K, None))
    H = y.shape[1]
    _chk(inv_perm, "moe_combine inv_perm", I32)
    _chk(weights, "moe_combine weights", F32)
    _chk(shared, "moe_combine shared", F32, (T, H))
    _chk(gate, "moe_combine gate", F32, (T,))
    if (shared is None) != (gate is None):
        raise ValueError("moe_combine: shared output and gate come together")
    if out is None:
        out = torch.empty(T, H, dtype=F32, device=y.device)
    _chk(out, "moe_combine out", F32, (T, H))
    if DEBUG_BOUNDS:
        _dbg_range(inv_perm, 0, T * K, "moe_combine inv_perm")
    check(library().mi_moe_combine(_ptr(y), _ptr(inv_perm), _ptr(weights), _ptr(shared), _ptr(gate), _ptr(out),
                                   T, H, K, _stream()), "moe_combine")
    return out


def combine_add_rmsnorm(hidden: torch.Tensor, y: torch.Tensor, inv_perm: Optional[torch.Tensor],
                        weights: torch.Tensor, shared: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                        norm_weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                        rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`moe_combine` and the :func:`add_rmsnorm` that takes its result as ``delta``, in one kernel:
    the combined rows are added to ``hidden`` (written back unless ``rows``) and normalised without
    ever being stored.  Bit for bit the result of the two separate calls."""
    _chk(hidden, "combine_add_rmsnorm hidden", F32)
    T, H = hidden.shape
    if weights.shape[0] != T:
        raise ValueError("combine_add_rmsnorm: one row of expert weights per row of hidden")
    K = weights.shape[1]
    _chk(y, "combine_add_rmsnorm y", F32, (T * K, H))
    _chk(inv_perm, "combine_add_rmsnorm inv_perm", I32)
    _chk(weights, "combine_add_rmsnorm weights", F32)
    _chk(shared, "combine_add_rmsnorm shared", F32, (T, H))
    _chk(gate, "combine_add_rmsnorm gate", F32, (T,))
    if (shared is None) != (gate is None):
        raise ValueError("combine_add_rmsnorm: shared output and gate come together")
    _chk(norm_weight, "combine_add_rmsnorm weight", None, (H,))
    _chk(rows, "combine_add_rmsnorm rows", I32)
    n = T if rows is None else rows.numel()
    out = torch.empty(n, H, dtype=out_dtype, device=hidden.device)
    if DEBUG_BOUNDS:
        _dbg_range(inv_perm, 0, T * K, "combine_add_rmsnorm inv_perm")
        _dbg_range(rows, 0, T, "combine_add_rmsnorm rows")
    check(library().mi_combine_add_rmsnorm(_ptr(hidden), _ptr(y), _ptr(inv_perm), _ptr(weights), _ptr(shared),
                                           _ptr(gate), K, _ptr(rows), _ptr(norm_weight),
                                           _code(norm_weight, "combine_add_rmsnorm weight"), _ptr(out),
                                           _code(out, "combine_add_rmsnorm out"), n, H, float(eps), _stream()),
          "combine_add_rmsnorm")
    return out


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
              q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int, window: int = 0,
              scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of a ragged batch over the paged cache (tiled kernel, any head size <= 256)."""
    _chk(q, "attention q")
    T, nh, d = q.shape
    _chk(k_cache, "attention k_cache", q.dtype)
    _, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "attention v_cache", q.dtype, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"attention: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "attention block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "attention q_start", I32, (B + 1,))
    _chk(kv_len, "attention kv_len", I32, (B,))
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "attention out", q.dtype, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if DEBUG_BOUNDS:
        _dbg_batch("attention", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window), int(max_q_len))
    check(library().mi_attn_tiled(_ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q, "attention q"),
                                  _ptr(block_table), _ptr(q_start), _ptr(kv_len), _ptr(out), B, int(max_q_len),
                                  nh, nkv, d, page_size, max_pages, int(window), float(scale), _stream()),
          "attention")
    return out


def prefill_attention_supported(d: int) -> bool:
    return bool(library().mi_attn_prefill_supported(int(d)))


def prefill_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                      q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int, window: int = 0,
                      scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contract as :func:`attention`, on tensor cores: bfloat16, head sizes 64 and 128."""
    _chk(q, "prefill_attention q", BF16)
    T, nh, d = q.shape
    _chk(k_cache, "prefill_attention k_cache", BF16)
    _, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "prefill_attention v_cache", BF16, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"prefill_attention: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "prefill_attention block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "prefill_attention q_start", I32, (B + 1,))
    _chk(kv_len, "prefill_attention kv_len", I32, (B,))
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "prefill_attention out", BF16, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if DEBUG_BOUNDS:
        _dbg_batch("prefill_attention", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window),
                   int(max_q_len))
    check(library().mi_attn_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(q_start),
                                    _ptr(kv_len), _ptr(out), B, int(max_q_len), nh, nkv, d, page_size, max_pages,
                                    int(window), float(scale), _stream()), "prefill_attention")
    return out


def prefill_attention_tc_supported(d: int, page_size: int) -> bool:
    return bool(library().mi_attn_prefill_tc_supported(int(d), int(page_size)))


def prefill_attention_tc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                         q_start: torch.Tensor, kv_len: torch.Tensor, max_q_len: int, window: int = 0,
                         scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same contract as :func:`attention`, on the tcgen05 tensor cores (TMA-fed, accumulators in
    tensor memory): bfloat16, head sizes 64 and 128, pages of 8 to 128 tokens.  Call
    :func:`check_tc_status` after the step: a wait inside the kernel that ran out is reported there."""
    global _tc_pending
    _chk(q, "prefill_attention_tc q", BF16)
    T, nh, d = q.shape
    _chk(k_cache, "prefill_attention_tc k_cache", BF16)
    num_pages, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "prefill_attention_tc v_cache", BF16, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"prefill_attention_tc: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "prefill_attention_tc block_table", I32)
    B, max_pages = block_table.shape
    _chk(q_start, "prefill_attention_tc q_start", I32, (B + 1,))
    _chk(kv_len, "prefill_attention_tc kv_len", I32, (B,))
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "prefill_attention_tc out", BF16, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    dev = q.device
    if dev not in _tc_status:
        _tc_status[dev] = torch.zeros(1, dtype=I32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_batch("prefill_attention_tc", q_start, kv_len, block_table, T, num_pages, page_size, int(window),
                   int(max_q_len))
    check(library().mi_attn_prefill_tc(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(q_start),
                                       _ptr(kv_len), _ptr(out), _ptr(_tc_status[dev]), T, B, int(max_q_len), nh, nkv,
                                       d, page_size, num_pages, max_pages, int(window), float(scale), _stream()),
          "prefill_attention_tc")
    _tc_pending = True
    return out


def decode_attention_supported(d: int) -> bool:
    return bool(library().mi_attn_decode_supported(int(d)))


def decode_split_size() -> int:
    """Keys per split of the decode attention by default."""
    return int(library().mi_attn_decode_split_size())


DECODE_SPLIT_SIZES = (128, 256, 512)      # the split sizes the decode attention is built for


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                     q_start: torch.Tensor, kv_len: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                     max_splits: int, window: int = 0, scale: Optional[float] = None,
                     out: Optional[torch.Tensor] = None, split: Optional[int] = None) -> torch.Tensor:
    """Split-KV attention when every request brings exactly one token.

    ``part_o`` (``>= B*nh*max_splits*d`` floats) and ``part_ml`` (``>= B*nh*max_splits*2``)
    are scratch; ``max_splits >= ceil(longest kv_len / split)`` with ``split`` keys per split
    (one of ``DECODE_SPLIT_SIZES``, default ``decode_split_size()``): smaller splits spread one or
    two requests over more blocks.
    """
    _chk(q, "decode_attention q")
    T, nh, d = q.shape
    _chk(k_cache, "decode_attention k_cache", q.dtype)
    _, nkv, page_size, d2 = k_cache.shape
    _chk(v_cache, "decode_attention v_cache", q.dtype, tuple(k_cache.shape))
    if d2 != d:
        raise ValueError(f"decode_attention: head_dim of q ({d}) and of the cache ({d2}) differ")
    _chk(block_table, "decode_attention block_table", I32)
    B, max_pages = block_table.shape
    if T != B:
        raise ValueError(f"decode_attention: {T} tokens for {B} requests; each request brings exactly one")
    _chk(q_start, "decode_attention q_start", I32, (B + 1,))
    _chk(kv_len, "decode_attention kv_len", I32, (B,))
    _chk(part_o, "decode_attention part_o", F32)
    _chk(part_ml, "decode_attention part_ml", F32)
    if part_o.numel() < B * nh * max_splits * d or part_ml.numel() < B * nh * max_splits * 2:
        raise ValueError("decode_attention: scratch too small for this batch and split count")
    if out is None:
        out = torch.empty_like(q)
    _chk(out, "decode_attention out", q.dtype, (T, nh, d))
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    if split is None:
        split = decode_split_size()
    if DEBUG_BOUNDS:
        _dbg_batch("decode_attention", q_start, kv_len, block_table, T, k_cache.shape[0], page_size, int(window), 1)
        longest = int(kv_len.max())
        if max_splits * int(split) < longest - int(split) // 4:
            _bad("decode_attention", f"{max_splits} splits of {split} keys cannot hold the longest request ({longest})")
    check(library().mi_attn_decode_split(_ptr(q), _ptr(k_cache), _ptr(v_cache), _code(q, "decode_attention q"),
                                         _ptr(block_table), _ptr(q_start), _ptr(kv_len), _ptr(out), _ptr(part_o),
                                         _ptr(part_ml), B, nh, nkv, d, page_size, max_pages, int(max_splits),
                                         int(split), int(window), float(scale), _stream()), "decode_attention")
    return out


def moe_router(x: torch.Tensor, router_w: torch.Tensor, shared_gate_w: Optional[torch.Tensor], top_k: int,
               norm_topk: bool, want_probs: bool = False
               ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Router of one layer.  Returns ``(idx [T,K] int32, w [T,K] f32, gate [T] f32 | None, probs | None)``."""
    _chk(x, "moe_router x")
    T, H = x.shape
    _chk(router_w, "moe_router weight", None, (None, H))
    E = router_w.shape[0]
    if shared_gate_w is not None:
        _chk(shared_gate_w, "moe_router shared gate", router_w.dtype)
        if shared_gate_w.numel() != H:
            raise ValueError("moe_router: the shared-expert gate must have hidden_size entries")
    dev = x.device
    idx = torch.empty(T, top_k, dtype=I32, device=dev)
    w = torch.empty(T, top_k, dtype=F32, device=dev)
    gate = torch.empty(T, dtype=F32, device=dev) if shared_gate_w is not None else None
    probs = torch.empty(T, E, dtype=F32, device=dev) if want_probs else None
    z = torch.empty(T, E + 1, dtype=F32, device=dev)
    check(library().mi_moe_router(_ptr(x), _code(x, "moe_router x"), _ptr(router_w), _ptr(shared_gate_w),
                                  _code(router_w, "moe_router weight"), _ptr(z), _ptr(idx), _ptr(w), _ptr(gate),
                                  _ptr(probs), T, H, E, int(top_k), int(bool(norm_topk)), _stream()),
          "moe_router")
    return idx, w, gate, probs


def moe_permute(topk_idx: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable sort of the (token, slot) pairs by expert.

    Returns ``(offsets [E+1], sorted_token [T*K], inv_perm [T*K])``, all int32.
    """
    _chk(topk_idx, "moe_permute idx", I32)
    T, K = topk_idx.shape
    dev = topk_idx.device
    offsets = torch.empty(num_experts + 1, dtype=I32, device=dev)
    sorted_token = torch.empty(T * K, dtype=I32, device=dev)
    inv_perm = torch.empty(T * K, dtype=I32, device=dev)
    counts = torch.empty(num_experts, dtype=I32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_range(topk_idx, 0, int(num_experts), "moe_permute expert indices")
    check(library().mi_moe_permute(_ptr(topk_idx), _ptr(offsets), _ptr(sorted_token), _ptr(inv_perm), _ptr(counts), T,
                                   int(num_experts), K, _stream()), "moe_permute")
    return offsets, sorted_token, inv_perm


def route_small_max_tokens() -> int:
    return int(library().mi_moe_route_small_max_tokens())


def moe_route_small(x: torch.Tensor, router_w: torch.Tensor, shared_gate_w: Optional[torch.Tensor], top_k: int,
                    norm_topk: bool, ticket: torch.Tensor, want_probs: bool = False, permute: bool = True):
    """:func:`moe_router` and (with ``permute``) :func:`moe_permute` of a step of a few tokens in
    one launch.

    ``ticket`` holds ``1 + T`` (or more) int32 counters that are zero before the first call and
    belong to the caller (the kernel leaves them zero); calls that share them must not overlap.  Returns
    ``(idx, w, gate, probs, offsets, sorted_token, inv_perm)``, the last three None without
    ``permute``.
    """
    _chk(x, "moe_route_small x")
    T, H = x.shape
    _chk(router_w, "moe_route_small weight", None, (None, H))
    E = router_w.shape[0]
    if shared_gate_w is not None:
        _chk(shared_gate_w, "moe_route_small shared gate", router_w.dtype)
        if shared_gate_w.numel() != H:
            raise ValueError("moe_route_small: the shared-expert gate must have hidden_size entries")
    _chk(ticket, "moe_route_small ticket", I32)
    if ticket.numel() < 1 + T:
        raise ValueError(f"moe_route_small: {ticket.numel()} ticket counters for {T} tokens (1 + T wanted)")
    dev = x.device
    idx = torch.empty(T, top_k, dtype=I32, device=dev)
    w = torch.empty(T, top_k, dtype=F32, device=dev)
    gate = torch.empty(T, dtype=F32, device=dev) if shared_gate_w is not None else None
    probs = torch.empty(T, E, dtype=F32, device=dev) if want_probs else None
    z = torch.empty(T, E + 1, dtype=F32, device=dev)
    offsets = sorted_token = inv_perm = None
    if permute:
        offsets = torch.empty(E + 1, dtype=I32, device=dev)
        sorted_token = torch.empty(T * top_k, dtype=I32, device=dev)
        inv_perm = torch.empty(T * top_k, dtype=I32, device=dev)
    check(library().mi_moe_route_small(
        _ptr(x), _code(x, "moe_route_small x"), _ptr(router_w), _ptr(shared_gate_w),
        _code(router_w, "moe_route_small weight"), _ptr(z), _ptr(ticket), _ptr(idx), _ptr(w), _ptr(gate), _ptr(probs),
        _ptr(offsets), _ptr(sorted_token), _ptr(inv_perm), T, H, E, int(top_k), int(bool(norm_topk)), _stream()),
        "moe_route_small")
    return idx, w, gate, probs, offsets, sorted_token, inv_perm


def norm_route_small_takes(hidden_size: int, num_experts: int = 1, gated: bool = False,
                           weight_dtype: torch.dtype = torch.bfloat16) -> bool:
    """Whether :func:`moe_norm_route_small` takes a router of these sizes (its blocks keep their share of the
    router's rows in shared memory)."""
    return bool(library().mi_moe_norm_route_small_takes(int(hidden_size), int(num_experts), int(bool(gated)),
                                                        2 if weight_dtype == torch.bfloat16 else 4))


def moe_norm_route_small(hidden: torch.Tensor, delta: Optional[torch.Tensor], norm_weight: torch.Tensor, eps: float,
                         out_dtype: torch.dtype, router_w: torch.Tensor, shared_gate_w: Optional[torch.Tensor],
                         top_k: int, norm_topk: bool, want_probs: bool = False):
    """:func:`add_rmsnorm` and the routing of a step of a few tokens in one launch (a cluster of blocks per token):
    ``hidden += delta``, the normalised rows ``x`` (of ``out_dtype``) and the routing computed from
    them.  Returns ``(x, idx, w, gate, probs)``."""
    _chk(hidden, "moe_norm_route_small hidden", F32)
    T, H = hidden.shape
    _chk(delta, "moe_norm_route_small delta", F32, (T, H))
    _chk(norm_weight, "moe_norm_route_small norm weight", None, (H,))
    _chk(router_w, "moe_norm_route_small weight", None, (None, H))
    E = router_w.shape[0]
    if shared_gate_w is not None:
        _chk(shared_gate_w, "moe_norm_route_small shared gate", router_w.dtype)
        if shared_gate_w.numel() != H:
            raise ValueError("moe_norm_route_small: the shared-expert gate must have hidden_size entries")
    dev = hidden.device
    x = torch.empty(T, H, dtype=out_dtype, device=dev)
    idx = torch.empty(T, top_k, dtype=I32, device=dev)
    w = torch.empty(T, top_k, dtype=F32, device=dev)
    gate = torch.empty(T, dtype=F32, device=dev) if shared_gate_w is not None else None
    probs = torch.empty(T, E, dtype=F32, device=dev) if want_probs else None
    check(library().mi_moe_norm_route_small(
        _ptr(hidden), _ptr(delta), _ptr(norm_weight), _code(norm_weight, "moe_norm_route_small norm weight"),
        float(eps), _ptr(x), _code(x, "moe_norm_route_small x"), _ptr(router_w), _ptr(shared_gate_w),
        _code(router_w, "moe_norm_route_small weight"), _ptr(idx), _ptr(w), _ptr(gate),
        _ptr(probs), T, H, E, int(top_k), int(bool(norm_topk)), _stream()), "moe_norm_route_small")
    return x, idx, w, gate, probs


def grouped_gemm_plain(a: torch.Tensor, gather: Optional[torch.Tensor], w: torch.Tensor, offsets: torch.Tensor,
                       n_rows: int, swiglu_pair: bool, out_dtype: torch.dtype) -> torch.Tensor:
    """Per-expert product of sorted rows (float arithmetic).

    ``w`` is ``[E, Nout, K]`` or, with ``swiglu_pair``, ``[E, 2*Nout, K]`` (gate rows,
    then up rows) and the result is ``silu(gate) * up``.  Row ``r`` of the result
    uses ``a[gather[r]]`` (or ``a[r]``) and the expert whose offset range holds ``r``.
    """
    _chk(a, "grouped_gemm a")
    Kd = a.shape[1]
    _chk(w, "grouped_gemm w", None, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    _chk(gather, "grouped_gemm gather", I32)
    _chk(offsets, "grouped_gemm offsets", I32, (E + 1,))
    out = torch.empty(n_rows, nout, dtype=out_dtype, device=a.device)
    if DEBUG_BOUNDS:
        _dbg_offsets(offsets, int(n_rows), "grouped_gemm_plain")
        _dbg_range(gather, 0, a.shape[0], "grouped_gemm_plain gather")
        if gather is None and a.shape[0] < n_rows:
            _bad("grouped_gemm_plain", f"{n_rows} rows wanted, the input has {a.shape[0]}")
    check(library().mi_grouped_gemm_plain(_ptr(a), _code(a, "grouped_gemm a"), _ptr(gather), _ptr(w),
                                          _code(w, "grouped_gemm w"), _ptr(offsets), _ptr(out),
                                          _code(out, "grouped_gemm out"), int(n_rows), E, nout, Kd,
                                          1 if swiglu_pair else 0, _stream()), "grouped_gemm_plain")
    return out


def l2_prefetch(t: torch.Tensor, max_bytes: Optional[int] = None) -> None:
    """Ask L2 for the first ``max_bytes`` bytes (all, if None) of a contiguous tensor; a hint, on the
    current stream, that returns at once."""
    _chk(t, "l2_prefetch tensor")
    n = t.numel() * t.element_size()
    if max_bytes is not None:
        n = min(n, int(max_bytes))
    check(library().mi_l2_prefetch(_ptr(t), n, _stream()), "l2_prefetch")


class dependent_launch:
    """``with dependent_launch(True):`` the kernels of decode-sized steps that are written for it (they wait
    for the kernels before them at their first line) are launched so that the device may place their blocks
    while the kernel before them in the stream is still running; a pass captured under it replays so."""

    def __init__(self, on: bool):
        self.on = bool(on)

    def __enter__(self):
        self.before = library().mi_set_dependent_launch(int(self.on))
        return self

    def __exit__(self, *exc):
        library().mi_set_dependent_launch(self.before)
        return False


def dense_f32(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` in true float32 (``x [T, K]``, ``w [N, K]``): every output element is one chain of
    fused multiply-adds over ``k`` in ascending order, so a row's result does not depend on how many rows
    there are.  The dense product of the float32 path."""
    _chk(x, "dense_f32 x", F32)
    T, K = x.shape
    _chk(w, "dense_f32 w", F32, (None, K))
    N = w.shape[0]
    out = torch.empty(T, N, dtype=F32, device=x.device)
    check(library().mi_dense_f32(_ptr(x), _ptr(w), _ptr(out), T, N, K, _stream()), "dense_f32")
    return out


def grouped_gemm_skinny_supported(kd: int) -> bool:
    return bool(library().mi_grouped_gemm_skinny_supported(int(kd)))


def grouped_gemm_skinny(a: torch.Tensor, gather: Optional[torch.Tensor], w: torch.Tensor, offsets: torch.Tensor,
                        n_rows: int, swiglu_pair: bool) -> torch.Tensor:
    """The grouped product for a few rows per expert (decode), bfloat16 on tensor cores.

    Same contract as :func:`grouped_gemm_plain`; the result is bfloat16 with ``swiglu_pair``
    (the activation that feeds the down projection) and float32 without.
    """
    _chk(a, "grouped_gemm_skinny a", BF16)
    Kd = a.shape[1]
    _chk(w, "grouped_gemm_skinny w", BF16, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    _chk(gather, "grouped_gemm_skinny gather", I32)
    _chk(offsets, "grouped_gemm_skinny offsets", I32, (E + 1,))
    out = torch.empty(n_rows, nout, dtype=BF16 if swiglu_pair else F32, device=a.device)
    if DEBUG_BOUNDS:
        _dbg_offsets(offsets, int(n_rows), "grouped_gemm_skinny")
        _dbg_range(gather, 0, a.shape[0], "grouped_gemm_skinny gather")
        if gather is None and a.shape[0] < n_rows:
            _bad("grouped_gemm_skinny", f"{n_rows} rows wanted, the input has {a.shape[0]}")
    check(library().mi_grouped_gemm_skinny(_ptr(a), _ptr(gather), _ptr(w), _ptr(offsets), _ptr(out), E, nout, Kd,
                                           1 if swiglu_pair else 0, _stream()), "grouped_gemm_skinny")
    return out


def dense_skinny_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether :func:`dense_skinny` takes this product: bfloat16, a few rows, inner size a multiple of 32."""
    return (x.dtype == BF16 and w.dtype == BF16 and x.dim() == 2 and x.is_contiguous() and w.is_contiguous()
            and 1 <= x.shape[0] <= library().mi_dense_skinny_max_rows() and x.shape[1] % 32 == 0)


def dense_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 swiglu_pair: bool = False) -> torch.Tensor:
    """``x @ w.T (+ bias)`` for a step of a few tokens (decode), every weight read once.

    ``x`` [T, K] and ``w`` [N, K] bfloat16, ``bias`` float32 [N] or None.  Returns float32
    [T, N]; with ``swiglu_pair`` the rows of ``w`` are N/2 gate rows then N/2 up rows and the
    result is ``silu(gate) * up`` as bfloat16 [T, N/2].
    """
    _chk(x, "dense_skinny x", BF16)
    T, Kd = x.shape
    _chk(w, "dense_skinny w", BF16, (None, Kd))
    wrows = w.shape[0]
    if swiglu_pair and wrows % 2:
        raise KernelError(f"dense_skinny: {wrows} weight rows cannot hold gate and up halves")
    nout = wrows // 2 if swiglu_pair else wrows
    if bias is not None:
        _chk(bias, "dense_skinny bias", F32, (wrows,))
    out = torch.empty(T, nout, dtype=BF16 if swiglu_pair else F32, device=x.device)
    check(library().mi_dense_skinny(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), T, nout, Kd,
                                    1 if swiglu_pair else 0, _stream()), "dense_skinny")
    return out


def qkv_skinny_supported(kd: int, d: int, rot_dim: int) -> bool:
    """Whether :func:`qkv_skinny` takes this geometry (``rot_dim`` 0: no rotation)."""
    return bool(library().mi_qkv_skinny_supported(int(kd), int(d), int(rot_dim)))


def qkv_skinny_max_rows() -> int:
    return int(library().mi_dense_skinny_max_rows())


def qkv_skinny(x: torch.Tensor, w_qkv: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor,
               inv_freq: Optional[torch.Tensor], slot_mapping: torch.Tensor, k_cache: torch.Tensor,
               v_cache: torch.Tensor, nh: int, nkv: int, d: int, page_size: int) -> torch.Tensor:
    """The q/k/v projection of a step of a few tokens with bias, rotary encoding and cache write
    in the same kernel (what a library product followed by :func:`qkv_post` does).

    ``x`` [T, K] and ``w_qkv`` [(nh + 2*nkv) * d, K] bfloat16, ``bias`` float32 or None.  Returns
    ``q [T, nh, d]`` bfloat16; k and v of row ``t`` go to ``slot_mapping[t]`` of the caches.
    """
    _chk(x, "qkv_skinny x", BF16)
    T, Kd = x.shape
    width = (nh + 2 * nkv) * d
    _chk(w_qkv, "qkv_skinny weight", BF16, (width, Kd))
    _chk(bias, "qkv_skinny bias", F32, (width,))
    _chk(positions, "qkv_skinny positions", I32, (T,))
    _chk(inv_freq, "qkv_skinny inv_freq", F32, (d // 2,))
    _chk(slot_mapping, "qkv_skinny slot_mapping", I32, (T,))
    _chk(k_cache, "qkv_skinny k_cache", BF16, (None, nkv, page_size, d))
    _chk(v_cache, "qkv_skinny v_cache", BF16, tuple(k_cache.shape))
    q = torch.empty(T, nh, d, dtype=BF16, device=x.device)
    if DEBUG_BOUNDS:
        _dbg_range(slot_mapping, -1, k_cache.shape[0] * page_size, "qkv_skinny slot_mapping")   # -1: not cached
    check(library().mi_qkv_skinny(_ptr(x), _ptr(w_qkv), _ptr(bias), _ptr(positions), _ptr(inv_freq),
                                  _ptr(slot_mapping), _ptr(q), _ptr(k_cache), _ptr(v_cache), T, Kd, nh, nkv, d,
                                  page_size, _stream()), "qkv_skinny")
    return q


def skinny_pairs_max_tokens() -> int:
    return int(library().mi_grouped_gemm_skinny_pairs_max_tokens())


def skinny_pairs_split_inner_max_tokens() -> int:
    """Steps of up to this many tokens take the form of :func:`grouped_gemm_skinny_pairs` whose blocks own
    16 features and split the inner dimension over their warps."""
    return int(library().mi_grouped_gemm_skinny_pairs_split_inner_max_tokens())


def grouped_gemm_skinny_pairs(a: torch.Tensor, topk_idx: torch.Tensor, w: torch.Tensor,
                              swiglu_pair: bool) -> torch.Tensor:
    """The decode-sized grouped product without a permutation: row ``t*K + k`` of the result
    belongs to the pair (token t, slot k) and is computed under expert ``topk_idx[t, k]``.

    With ``swiglu_pair`` ``a`` is ``[T, Kd]`` (a token's row serves its K pairs) and the result is
    the bfloat16 activation ``[T*K, Nout]``; without, ``a`` is ``[T*K, Kd]`` indexed by pair and
    the result float32.
    """
    _chk(topk_idx, "grouped_gemm_skinny_pairs idx", I32)
    T, K = topk_idx.shape
    _chk(a, "grouped_gemm_skinny_pairs a", BF16, (T if swiglu_pair else T * K, None))
    Kd = a.shape[1]
    _chk(w, "grouped_gemm_skinny_pairs w", BF16, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    out = torch.empty(T * K, nout, dtype=BF16 if swiglu_pair else F32, device=a.device)
    if DEBUG_BOUNDS:
        _dbg_range(topk_idx, 0, E, "grouped_gemm_skinny_pairs expert indices")
    check(library().mi_grouped_gemm_skinny_pairs(_ptr(a), _ptr(topk_idx), _ptr(w), _ptr(out), T, K, E, nout, Kd,
                                                 1 if swiglu_pair else 0, _stream()), "grouped_gemm_skinny_pairs")
    return out


def grouped_gemm_tc_supported(kd: int) -> bool:
    """The tcgen05 grouped product takes any number of output features; its inner size must be a multiple
    of 64 (one 128-byte swizzle row of bfloat16)."""
    return bool(library().mi_grouped_gemm_tc_supported(int(kd)))


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """``x[rows]`` for a bfloat16 matrix (the sorted copy the tensor-core grouped product reads)."""
    _chk(x, "gather_rows x", BF16)
    _chk(rows, "gather_rows rows", I32)
    out = torch.empty(rows.numel(), x.shape[1], dtype=BF16, device=x.device)
    if DEBUG_BOUNDS:
        _dbg_range(rows, 0, x.shape[0], "gather_rows rows")
    check(library().mi_gather_rows_bf16(_ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1], _stream()),
          "gather_rows")
    return out


_tc_status = {}
_tc_pending = False


TC_FORMS = (0, 1, 2, 3)


def grouped_gemm_tc(a_sorted: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, swiglu_pair: bool,
                    form: Optional[int] = None) -> torch.Tensor:
    """The grouped product for many rows per expert (prefill): tcgen05 tensor cores fed by TMA.

    ``a_sorted [N, K]`` holds the rows already in expert order.  Result as for
    :func:`grouped_gemm_skinny`.  Call :func:`check_tc_status` after the step: a wait inside the
    kernel that ran out is reported there rather than hanging the device.  ``form`` picks one of the
    kernel's forms (``TC_FORMS``: one block per tile with row tiles of 128 or 256, persistent with
    row tiles of 160 or 256); the library chooses by the rows per expert when it is None.
    """
    global _tc_pending
    _chk(a_sorted, "grouped_gemm_tc a", BF16)
    n_rows, Kd = a_sorted.shape
    _chk(w, "grouped_gemm_tc w", BF16, (None, None, Kd))
    E, wrows, _ = w.shape
    nout = wrows // 2 if swiglu_pair else wrows
    _chk(offsets, "grouped_gemm_tc offsets", I32, (E + 1,))
    dev = a_sorted.device
    if dev not in _tc_status:
        _tc_status[dev] = torch.zeros(1, dtype=I32, device=dev)
    out = torch.empty(n_rows, nout, dtype=BF16 if swiglu_pair else F32, device=dev)
    if DEBUG_BOUNDS:
        _dbg_offsets(offsets, int(n_rows), "grouped_gemm_tc")
    check(library().mi_grouped_gemm_tc_form(_ptr(a_sorted), _ptr(w), _ptr(offsets), _ptr(out), _ptr(_tc_status[dev]),
                                            n_rows, E, nout, Kd, 1 if swiglu_pair else 0,
                                            -1 if form is None else int(form), _stream()), "grouped_gemm_tc")
    _tc_pending = True
    return out


def grouped_gemm_tc_inject_wait_fault(skip_k_block: int, wait_limit: int) -> None:
    """For the test of the bounded waits: the next :func:`grouped_gemm_tc` with ``form`` 0 or 1 leaves out
    the loads of one k block and waits at most ``wait_limit`` rounds, so a wait runs out, the kernel
    returns by itself, and :func:`check_tc_status` raises.  The launch after it is a normal one."""
    lib = library()
    lib.mi_grouped_gemm_tc_test_fault.argtypes = [ctypes.c_int, ctypes.c_uint]
    lib.mi_grouped_gemm_tc_test_fault.restype = None
    lib.mi_grouped_gemm_tc_test_fault(int(skip_k_block), int(wait_limit))


def check_tc_status() -> None:
    """Raise if a bounded wait inside a tensor-core kernel gave up since the last check (synchronises
    only when such a kernel was launched)."""
    global _tc_pending
    if not _tc_pending:
        return
    _tc_pending = False
    for dev, st in _tc_status.items():
        code = int(st.item())
        if code:
            st.zero_()
            from .library import KernelError
            raise KernelError(f"tcgen05 kernel on {dev}: a wait ran out (code {code}; grouped product: "
                              f"1 = producer waiting for a free stage, 2 = MMA waiting for data, "
                              f"3 = epilogue waiting for the accumulators; prefill attention: 11-19); "
                              f"results of that step are invalid")


def random_fill(out: torch.Tensor, key: Tuple[int, int], scale: float, offset: float) -> torch.Tensor:
    """Fill ``out`` (float32, bfloat16 or float16, contiguous) with the counter-based values of
    ``weights.random_init``: element ``i`` depends on ``(key, i)`` only."""
    _chk(out, "random_fill out")
    codes = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
    if out.dtype not in codes:
        raise TypeError(f"random_fill: dtype {out.dtype} is not float32, bfloat16 or float16")
    with torch.cuda.device(out.device):
        check(library().mi_random_fill(_ptr(out), codes[out.dtype], out.numel(), int(key[0]) & 0xFFFFFFFF,
                                       int(key[1]) & 0xFFFFFFFF, float(scale), float(offset), _stream()),
              "random_fill")
    return out


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                top_p: Optional[torch.Tensor] = None, u: Optional[torch.Tensor] = None,
                probs_scratch: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 ``logits [R, V]``; rows with temperature <= 0 are greedy."""
    _chk(logits, "sample_rows logits", F32)
    R, V = logits.shape
    _chk(temperature, "sample_rows temperature", F32, (R,))
    _chk(top_p, "sample_rows top_p", F32, (R,))
    _chk(u, "sample_rows u", F32, (R,))
    if temperature is not None and probs_scratch is None:
        probs_scratch = torch.empty(R, V, dtype=F32, device=logits.device)
    _chk(probs_scratch, "sample_rows scratch", F32, (R, V))
    if out is None:
        out = torch.empty(R, dtype=I32, device=logits.device)
    _chk(out, "sample_rows out", I32, (R,))
    check(library().mi_sample_rows(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(u), _ptr(probs_scratch),
                                   _ptr(out), R, V, _stream()), "sample_rows")
    return out
