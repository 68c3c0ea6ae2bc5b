"""Position encodings that act on queries and keys inside the attention part.

``rope``: half-split rotary encoding; ``inv_freq[i] = theta^(-2i/rot_dim)``
(src/layers/rope.cpp:20-29); the rotation itself, with angles computed in
float32 from the absolute position, runs in the kernel that also adds the
projection bias and writes the cache (reference: cos/sin tables rounded to
FP16, src/kernels/rope_kernel.cu:65-77, and a separate rotation kernel, :27-54).

``none``: queries and keys are used as projected.

A further rotary variant (other frequencies, partial rotation) is a new class
that returns another table and ``rot_dim``; the kernel takes both as arguments.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..config.registry import register_part
from .base import PositionEncoding


class RotaryEncoding(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rot_dim`` (default ``head_dim``)."""

    graph_safe = True

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        d = int(self.params["head_dim"])
        self.rot_dim = int(self.params.get("rot_dim", d))
        if self.rot_dim % 2 or not 0 < self.rot_dim <= d:
            raise ValueError(f"rope: rot_dim {self.rot_dim} must be even and within head_dim {d}")
        self.theta = float(self.params["theta"])
        self._table = {}

    def table(self, device) -> Optional[torch.Tensor]:
        key = str(device)
        if key not in self._table:
            i = torch.arange(self.rot_dim // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rot_dim)
            self._table[key] = inv.to(torch.float32).to(device)
        return self._table[key]


class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    rot_dim = 0

    def table(self, device) -> Optional[torch.Tensor]:
        return None


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
