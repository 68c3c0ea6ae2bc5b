"""RMSNorm, fused with the residual addition that precedes it.

Reference: ``y = x * rsqrt(mean(x^2) + eps) * w`` in src/kernels/rmsnorm_kernel.cu:43-64,
the residual addition as a separate kernel (src/kernels/model_utils_kernel.cu:31-42).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..ops import functional as F
from .base import Deferred, Norm, Runtime, TensorDecl, WeightedRowSum


class RMSNorm(Norm):
    """params: ``size``, ``eps``.  Tensor: ``<prefix>weight [size]``."""

    graph_safe = True
    accepts_deferred = True

    def tensor_decls(self) -> List[TensorDecl]:
        return [TensorDecl(self.prefix + "weight", (self.params["size"],), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.eps = float(self.params["eps"])
        self.weight = rt.precision.small(tensors[self.prefix + "weight"], rt.device)

    def rms_parameters(self):
        return self.weight, self.eps

    def apply(self, hidden: torch.Tensor, delta: Optional[torch.Tensor],
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(delta, WeightedRowSum):
            # the sum is formed row by row inside the norm's kernel and never written out
            return F.combine_add_rmsnorm(hidden, delta.rows, delta.index, delta.weights, delta.extra, delta.scale,
                                         self.weight, self.eps, self.rt.act, rows)
        if isinstance(delta, Deferred):
            delta = delta.materialize()
        return F.add_rmsnorm(hidden, delta, self.weight, self.eps, self.rt.act, rows)


register_part("norm", "rmsnorm", RMSNorm)
