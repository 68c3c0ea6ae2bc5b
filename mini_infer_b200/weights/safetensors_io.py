"""Reading and writing the safetensors container, without a helper library.

Format (as the reference reads it, src/model/safetensors_loader.cpp:44-116):
eight bytes of little-endian header length ``n``, ``n`` bytes of JSON mapping
each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header; ``__metadata__`` is skipped), then
the data.  Sharded checkpoints carry ``model.safetensors.index.json`` whose
``weight_map`` sends each name to its shard
(src/model/safetensors_loader.cpp:137-187).

Unlike the reference, which maps every unknown dtype string to FP32
(src/model/safetensors_loader.cpp:21-29), an unknown dtype is an error here.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import torch

_DTYPES = {
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I32": torch.int32,
    "I64": torch.int64,
}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}
_ITEMSIZE = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2, torch.int32: 4, torch.int64: 8}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int
    shard: str


class SafetensorsFile:
    """One memory-mapped ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"safetensors: cannot open {path}") from e
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"safetensors: {path} is too short to hold a header")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"safetensors: {path} header length {hlen} exceeds the file")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"safetensors: {path} has an unreadable header: {e}") from e
        self._data_start = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self.tensors: Dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = meta.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"safetensors: tensor '{name}' in {path} has unsupported dtype {dt!r}")
            dtype = _DTYPES[dt]
            shape = tuple(int(x) for x in meta["shape"])
            begin, end = (int(x) for x in meta["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            if end - begin != numel * _ITEMSIZE[dtype] or begin < 0 or self._data_start + end > size:
                # src/model/safetensors_loader.cpp:108-113
                raise SafetensorsError(
                    f"safetensors: tensor '{name}' in {path}: byte range [{begin}, {end}) does not match "
                    f"shape {list(shape)} of {dt}")
            self.tensors[name] = TensorInfo(name, dtype, shape, begin, end, path)

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that aliases the mapping (read-only memory: clone or move it)."""
        info = self.tensors[name]
        n = info.end - info.begin
        if n == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        buf = memoryview(self._mm)[self._data_start + info.begin: self._data_start + info.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the buffer is not writable
            t = torch.frombuffer(buf, dtype=info.dtype)
        return t.reshape(info.shape)

    def close(self) -> None:
        try:
            self._mm.close()
        except (BufferError, ValueError):
            pass  # tensors that alias the mapping are still alive
        self._f.close()


class CheckpointFolder:
    """All tensors of a model folder: one file or an index over shards."""

    def __init__(self, folder: str):
        self.folder = folder
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        if os.path.exists(index):
            with open(index) as f:
                wm = json.load(f).get("weight_map")
            if not isinstance(wm, dict):
                raise SafetensorsError(f"safetensors: {index} has no weight_map")
            for name, shard in wm.items():
                self._where[name] = os.path.join(folder, shard)
        elif os.path.exists(single):
            sf = SafetensorsFile(single)
            self._files[single] = sf
            for name in sf.tensors:
                self._where[name] = single
        else:
            raise SafetensorsError(
                f"safetensors: {folder} holds neither model.safetensors nor model.safetensors.index.json")

    def _file(self, path: str) -> SafetensorsFile:
        if path not in self._files:
            self._files[path] = SafetensorsFile(path)
        return self._files[path]

    def names(self) -> List[str]:
        return list(self._where)

    def info(self, name: str) -> TensorInfo:
        sf = self._file(self._where[name])
        if name not in sf.tensors:
            raise SafetensorsError(f"safetensors: index sends '{name}' to {sf.path}, which does not hold it")
        return sf.tensors[name]

    def read(self, name: str) -> torch.Tensor:
        return self._file(self._where[name]).read(name)

    def close(self) -> None:
        for sf in self._files.values():
            sf.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      producer) -> None:
    """Stream a checkpoint to ``path``.

    ``tensors`` lists (name, shape, dtype) in file order; ``producer(name)``
    returns the tensor when its turn comes, so a large model never has to be
    held whole.
    """
    entries = list(tensors)
    header: Dict[str, dict] = {}
    off = 0
    for name, shape, dtype in entries:
        if dtype not in _DTYPE_NAMES:
            raise SafetensorsError(f"safetensors: cannot write dtype {dtype} of '{name}'")
        numel = 1
        for s in shape:
            numel *= int(s)
        n = numel * _ITEMSIZE[dtype]
        header[name] = {"dtype": _DTYPE_NAMES[dtype], "shape": [int(s) for s in shape],
                        "data_offsets": [off, off + n]}
        off += n
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for name, shape, dtype in entries:
            t = producer(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise SafetensorsError(
                    f"safetensors: producer gave {list(t.shape)} {t.dtype} for '{name}', "
                    f"declared {list(shape)} {dtype}")
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write((t if t.dim() else t.reshape(1)).view(torch.uint8).numpy())
    os.replace(tmp, path)
