"""From a model folder (or a configuration and a seed) to a loaded :class:`Model`."""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from ..config.model_config import read_config_json
from ..config.registry import build_model_spec
from ..parts.base import Runtime, configure_matmul_exactness, precision_from_name
from ..weights.loader import FolderSource
from ..weights.random_init import RandomSource
from .model import Model


def _runtime(dtype: str, device) -> Runtime:
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError(f"mini_infer_b200 runs on a CUDA device only (asked for '{device}'); "
                           f"there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("mini_infer_b200: no CUDA device is available; there is no CPU path")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.set_device(dev)
    configure_matmul_exactness()
    from ..ops.library import library
    library()  # build or load the kernels now: fail here, loudly, rather than in the first step
    return Runtime(precision_from_name(dtype), dev)


def load_model(folder: str, dtype: str = "bfloat16", device="cuda:0") -> Tuple[Model, Runtime, Dict[str, Any]]:
    """Read ``config.json``, pick the architecture from the registry, load ``model.safetensors``.

    Side effect on the whole process: PyTorch's matrix-product switches are set so that library products
    accumulate in true float32 (no TF32, no reduced-precision reductions for bfloat16 or float16 inputs;
    :func:`configure_matmul_exactness`).  Both precision paths need them, and everything else that runs
    PyTorch products in the same process afterwards inherits them."""
    cj = read_config_json(folder)
    spec = build_model_spec(cj)
    rt = _runtime(dtype, device)
    model = Model(spec)
    model.load(FolderSource(folder), rt)
    return model, rt, cj


def random_model(config_json: Dict[str, Any], seed: int, dtype: str = "bfloat16", device="cuda:0",
                 spec=None) -> Tuple[Model, Runtime]:
    """A model with seeded random weights generated on the device (no folder is written)."""
    spec = spec or build_model_spec(config_json)
    rt = _runtime(dtype, device)
    model = Model(spec)
    src = RandomSource(model.tensor_decls(), seed, rt.act, str(rt.device))
    model.load(src, rt)
    return model, rt
