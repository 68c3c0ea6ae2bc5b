"""Bringing a checkpoint and a model description together.

The parts of a built model declare the tensors they expect
(:class:`~mini_infer_b200.parts.base.TensorDecl`); this module compares that
manifest with what a source holds *before* anything is read and raises one
error that lists every missing tensor, every unexpected one and every wrong
shape.  The reference checks tensor by tensor while loading and stops at the
first problem ("missing weight <name>", src/model/weight_mapper.cpp:42-49; "bad
shape", :51-67) and silently skips absent optional tensors
(src/model/transformer_model.cpp:274-289).

Sources: a model folder (:class:`FolderSource`) or seeded random tensors
(:class:`~mini_infer_b200.weights.random_init.RandomSource`).
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from ..parts.base import TensorDecl
from .safetensors_io import CheckpointFolder


class WeightError(ValueError):
    """Checkpoint and model do not fit; the message lists every problem."""

    def __init__(self, message: str, missing: Sequence[str] = (), unexpected: Sequence[str] = (),
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = (),
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


class FolderSource:
    """Tensors of ``config.json``'s folder, read lazily from safetensors."""

    def __init__(self, folder: str):
        self.folder = folder
        self.ckpt = CheckpointFolder(folder)

    def names(self) -> List[str]:
        return self.ckpt.names()

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.ckpt.info(name).shape

    def dtype(self, name: str) -> torch.dtype:
        return self.ckpt.info(name).dtype

    def read(self, name: str) -> torch.Tensor:
        return self.ckpt.read(name)

    def describe(self) -> str:
        return self.folder


_FLOAT_DTYPES = (torch.float32, torch.float16, torch.bfloat16)


def check_manifest(decls: Iterable[TensorDecl], source, allow_unexpected: Sequence[str] = ()) -> None:
    """Raise :class:`WeightError` unless ``source`` holds exactly the declared tensors."""
    decls = list(decls)
    have = set(source.names())
    want = {d.name for d in decls}
    missing = sorted(want - have)
    unexpected = sorted(n for n in have - want if n not in allow_unexpected)
    wrong_shape, wrong_dtype = [], []
    for d in decls:
        if d.name in have:
            got = tuple(source.shape(d.name))
            if got != tuple(d.shape):
                wrong_shape.append((d.name, got, tuple(d.shape)))
            dt = source.dtype(d.name)
            if dt not in _FLOAT_DTYPES:
                wrong_dtype.append((d.name, str(dt)))
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = [f"checkpoint {source.describe()} does not fit the model:"]

    def block(title, items, fmt):
        if items:
            lines.append(f"  {title} ({len(items)}):")
            for it in items[:40]:
                lines.append("    " + fmt(it))
            if len(items) > 40:
                lines.append(f"    ... and {len(items) - 40} more")

    block("missing tensors", missing, lambda n: n)
    block("unexpected tensors", unexpected, lambda n: n)
    block("wrong shapes", wrong_shape, lambda t: f"{t[0]}: found {list(t[1])}, expected {list(t[2])}")
    block("wrong dtypes", wrong_dtype, lambda t: f"{t[0]}: found {t[1]}, expected a floating type")
    raise WeightError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)


class LazyTensors(Mapping):
    """``tensors[name]`` reads the tensor when a part asks for it, so a large
    checkpoint is never held twice."""

    def __init__(self, source, names: Iterable[str]):
        self._source = source
        self._names = list(names)

    def __getitem__(self, name: str) -> torch.Tensor:
        return self._source.read(name)

    def __iter__(self):
        return iter(self._names)

    def __len__(self) -> int:
        return len(self._names)

    def __contains__(self, name) -> bool:
        return name in self._names
