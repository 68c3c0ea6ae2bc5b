"""Load the CUDA library and declare its C entry points.

There is exactly one way to run an op: through this library, on a CUDA device.
If it cannot be built or loaded the import of an op fails with the reason; no
op has a CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from typing import Optional

_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[str] = None

P = c_void_p
I = c_int
F = c_float
L = c_int64

_SIGNATURES = {
    "mi_embed_gather": [P, P, I, P, I, I, I, P],
    "mi_add_rmsnorm": [P, P, P, P, I, P, I, I, I, F, P],
    "mi_qkv_post": [P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P],
    "mi_swiglu": [P, P, I, L, I, P],
    "mi_moe_combine": [P, P, P, P, P, P, I, I, I, P],
    "mi_combine_add_rmsnorm": [P, P, P, P, P, P, I, P, P, I, P, I, I, I, F, P],
    "mi_attn_tiled": [P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_decode": [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_decode_split": [P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P],
    "mi_moe_router": [P, I, P, P, I, P, P, P, P, P, I, I, I, I, I, P],
    "mi_moe_permute": [P, P, P, P, P, I, I, I, P],
    "mi_grouped_gemm_plain": [P, I, P, P, I, P, P, I, I, I, I, I, I, P],
    "mi_sample_rows": [P, P, P, P, P, P, I, I, P],
    "mi_grouped_gemm_skinny": [P, P, P, P, P, I, I, I, I, P],
    "mi_moe_route_small": [P, I, P, P, I, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P],
    "mi_moe_norm_route_small": [P, P, P, I, F, P, I, P, P, I, P, P, P, P, I, I, I, I, I, P],
    "mi_grouped_gemm_skinny_pairs": [P, P, P, P, I, I, I, I, I, I, P],
    "mi_qkv_skinny": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "mi_dense_skinny": [P, P, P, P, I, I, I, I, P],
    "mi_gather_rows_bf16": [P, P, P, I, I, P],
    "mi_attn_prefill": [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "mi_attn_prefill_tc": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P],
    "mi_grouped_gemm_tc": [P, P, P, P, P, I, I, I, I, I, P],
    "mi_grouped_gemm_tc_form": [P, P, P, P, P, I, I, I, I, I, I, P],
    "mi_random_fill": [P, I, L, ctypes.c_uint, ctypes.c_uint, F, F, P],
    "mi_dense_f32": [P, P, P, I, I, I, P],
    "mi_l2_prefetch": [P, ctypes.c_ulonglong, P],
}


def library() -> ctypes.CDLL:
    """The loaded library; built at the first call of a fresh checkout."""
    global _lib, _lib_path
    if _lib is not None:
        return _lib
    from ..csrc.build import build
    path = build()
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise RuntimeError(f"mini_infer_b200: cannot load {path}: {e}") from e
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.mi_last_error.restype = c_char_p
    lib.mi_last_error.argtypes = []
    lib.mi_launch_count.restype = ctypes.c_longlong
    lib.mi_launch_count.argtypes = []
    lib.mi_attn_decode_supported.argtypes = [I]
    lib.mi_attn_decode_supported.restype = c_int
    lib.mi_attn_prefill_supported.argtypes = [I]
    lib.mi_attn_prefill_supported.restype = c_int
    lib.mi_grouped_gemm_tc_supported.argtypes = [I]
    lib.mi_grouped_gemm_tc_supported.restype = c_int
    lib.mi_grouped_gemm_skinny_supported.argtypes = [I]
    lib.mi_grouped_gemm_skinny_supported.restype = c_int
    lib.mi_moe_route_small_max_tokens.argtypes = []
    lib.mi_moe_route_small_max_tokens.restype = c_int
    lib.mi_moe_norm_route_small_max_width.argtypes = []
    lib.mi_moe_norm_route_small_max_width.restype = c_int
    lib.mi_set_dependent_launch.argtypes = [c_int]
    lib.mi_set_dependent_launch.restype = c_int
    lib.mi_moe_norm_route_small_takes.argtypes = [c_int, c_int, c_int, c_int]
    lib.mi_moe_norm_route_small_takes.restype = c_int
    lib.mi_grouped_gemm_skinny_pairs_split_inner_max_tokens.argtypes = []
    lib.mi_grouped_gemm_skinny_pairs_split_inner_max_tokens.restype = c_int
    lib.mi_grouped_gemm_skinny_pairs_max_tokens.argtypes = []
    lib.mi_grouped_gemm_skinny_pairs_max_tokens.restype = c_int
    lib.mi_attn_prefill_tc_supported.argtypes = [I, I]
    lib.mi_attn_prefill_tc_supported.restype = c_int
    lib.mi_qkv_skinny_supported.argtypes = [I, I, I]
    lib.mi_qkv_skinny_supported.restype = c_int
    lib.mi_dense_skinny_max_rows.argtypes = []
    lib.mi_dense_skinny_max_rows.restype = c_int
    lib.mi_attn_decode_split_size.argtypes = []
    lib.mi_attn_decode_split_size.restype = c_int
    _lib = lib
    _lib_path = path
    return lib


def launch_count() -> int:
    """Kernels of this library queued so far in this process."""
    return int(library().mi_launch_count())


def library_path() -> Optional[str]:
    return _lib_path


class KernelError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        msg = library().mi_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what} refused or failed (code {code}): {msg}")
