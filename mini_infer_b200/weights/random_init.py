"""Seeded random weights: as a tensor source, or written out as a model folder.

Every matrix, bias and embedding is N(0, 0.02); norm weights are 1 + N(0, 0.02).
Each tensor has a generator of its own, keyed by the seed and the tensor's
name, so tensors can be produced in any order, one at a time, on the host or on
a CUDA device (the two do not give the same numbers: a folder written by the
host generator is the portable form).  The reference has no random-weight mode;
its tests fill buffers with a xorshift generator (tests/test_helpers.h:44-57).
"""

from __future__ import annotations

import hashlib
import os
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..parts.base import TensorDecl
from .safetensors_io import write_safetensors

INIT_STD = 0.02


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


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
        g = torch.Generator(device=self.device)
        g.manual_seed(_tensor_seed(self.seed, name))
        t = torch.randn(tuple(d.shape), generator=g, dtype=torch.float32, device=self.device) * self.std
        if d.role == "norm":
            t += 1.0
        return t.to(self._dtype)


def write_model_folder(folder: str, config_json: dict, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = INIT_STD) -> str:
    """Write ``config.json`` and ``model.safetensors`` with seeded random weights for the
    architecture that ``config_json`` names.  Returns the folder."""
    import json
    from ..engine.model import declared_tensors
    from ..config.registry import build_model_spec

    spec = build_model_spec(config_json)
    decls = declared_tensors(spec)
    src = RandomSource(decls, seed, dtype, "cpu", std)
    os.makedirs(folder, exist_ok=True)
    cj = dict(config_json)
    cj.setdefault("torch_dtype", {torch.bfloat16: "bfloat16", torch.float32: "float32",
                                  torch.float16: "float16"}[dtype])
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cj, f, indent=2)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      [(d.name, tuple(d.shape), dtype) for d in decls], src.read)
    return folder
