"""Seeded random weights: as a tensor source, or written out as a model folder.

Every matrix, bias and embedding is close to N(0, 0.02); norm weights are 1 + that.
Element ``i`` of the tensor called ``name`` under ``seed`` is a pure function of
``(seed, name, i)``: Philox-4x32-10 keyed by a hash of seed and name, counter ``i``,
whose eight 16-bit halves are summed (an exact integer, close to normal), centred,
scaled by one float32 multiplication and shifted by one float32 addition.  The host
function below (numpy) and the device kernel (``csrc/random_init.cu``) do the same
integer and float32 steps, so a tensor made on a CUDA device, on the host, or read back
from a written folder has the same bits, in any order and one tensor at a time.  The
reference has no random-weight mode; its tests fill buffers with a counter generator on
the host (tests/test_helpers.h:44-57).
"""

from __future__ import annotations

import hashlib
import math
import os
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from ..parts.base import TensorDecl
from .safetensors_io import write_safetensors

INIT_STD = 0.02
_HALVES_MEAN = 262140                       # 8 * 65535 / 2
_HALVES_STD = math.sqrt(8 * (65536.0 ** 2 - 1.0) / 12.0)
_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def tensor_key(seed: int, name: str) -> Tuple[int, int]:
    """The two 32-bit Philox key words of a tensor: the first eight bytes of SHA-256("seed:name")."""
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:4], "little"), int.from_bytes(h[4:8], "little")


def fill_scale(std: float) -> np.float32:
    return np.float32(std / _HALVES_STD)


def random_values_host(n: int, key: Tuple[int, int], std: float, offset: float, first: int = 0) -> np.ndarray:
    """Elements ``first .. first + n`` of a tensor as float32 (the host form of ``random_fill_kernel``)."""
    mask = np.uint64(0xFFFFFFFF)
    out = np.empty(n, dtype=np.float32)
    scale, off = fill_scale(std), np.float32(offset)
    step = 1 << 20
    for lo in range(0, n, step):
        i = np.arange(first + lo, first + min(n, lo + step), dtype=np.uint64)
        c0, c1 = i & mask, i >> np.uint64(32)
        c2 = np.zeros_like(i)
        c3 = np.zeros_like(i)
        k0, k1 = np.uint64(key[0]), np.uint64(key[1])
        for _ in range(10):
            p0, p1 = np.uint64(_M0) * c0, np.uint64(_M1) * c2
            c0, c1, c2, c3 = (p1 >> np.uint64(32)) ^ c1 ^ k0, p1 & mask, (p0 >> np.uint64(32)) ^ c3 ^ k1, p0 & mask
            k0, k1 = (k0 + np.uint64(_W0)) & mask, (k1 + np.uint64(_W1)) & mask
        s = np.zeros(i.shape, dtype=np.int64)
        for c in (c0, c1, c2, c3):
            s += (c & np.uint64(0xFFFF)).astype(np.int64) + (c >> np.uint64(16)).astype(np.int64)
        v = (s - _HALVES_MEAN).astype(np.float32) * scale      # one rounding
        out[lo:lo + i.shape[0]] = v + off                       # and another: never a fused multiply-add
    return out


def random_tensor(shape: Tuple[int, ...], key: Tuple[int, int], std: float, offset: float, dtype: torch.dtype,
                  device: torch.device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    if device.type == "cuda":
        from ..ops.functional import random_fill
        return random_fill(torch.empty(tuple(shape), dtype=dtype, device=device), key, float(fill_scale(std)),
                           float(offset))
    return torch.from_numpy(random_values_host(n, key, std, offset)).reshape(tuple(shape)).to(dtype)


class RandomSource:
    """A tensor source (same interface as ``FolderSource``) that makes tensors up."""

    def __init__(self, decls: Iterable[TensorDecl], seed: int, dtype: torch.dtype = torch.bfloat16,
                 device: str = "cpu", std: float = INIT_STD):
        self._decls: Dict[str, TensorDecl] = {d.name: d for d in decls}
        self.seed = int(seed)
        self._dtype = dtype
        self.device = torch.device(device)
        self.std = std

    def names(self) -> List[str]:
        return list(self._decls)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._decls[name].shape)

    def dtype(self, name: str) -> torch.dtype:
        return self._dtype

    def describe(self) -> str:
        return f"random(seed={self.seed})"

    def read(self, name: str) -> torch.Tensor:
        d = self._decls[name]
        return random_tensor(tuple(d.shape), tensor_key(self.seed, name), self.std,
                             1.0 if d.role == "norm" else 0.0, self._dtype, self.device)


def write_model_folder(folder: str, config_json: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = INIT_STD, device: str = "cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` with seeded random weights for the
    architecture that ``config_json`` names.  ``device`` is where the numbers are made (the file is
    the same either way; a CUDA device is much faster for large models).  Returns the folder."""
    import json
    from ..engine.model import declared_tensors
    from ..config.registry import build_model_spec

    spec = build_model_spec(config_json)
    decls = declared_tensors(spec)
    src = RandomSource(decls, seed, dtype, device, std)
    os.makedirs(folder, exist_ok=True)
    cj = dict(config_json)
    cj.setdefault("torch_dtype", {torch.bfloat16: "bfloat16", torch.float32: "float32",
                                  torch.float16: "float16"}[dtype])
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cj, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(d.name, tuple(d.shape), dtype) for d in decls], src.read)
    return folder
