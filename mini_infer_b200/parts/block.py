"""Block arrangement, embedding and output head.

``prenorm_residual``: ``a = x + Mixer(Norm1(x))``; ``y = a + FFN(Norm2(a))``
(src/model/transformer_model.h:25-28, src/model/transformer_model.cpp:578-641).
The residual stream ``hidden`` is float32 in both precision paths.  A part's
output is not added at once: it travels as ``pending`` to the next norm, whose
kernel adds it while it reads the row anyway.  A feed-forward may even leave its last
step (the weighted sum of its experts' rows) to that kernel: ``pending`` is then a
``Deferred``.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..ops import functional as F
from .base import (Block, BuiltLayer, CacheBinding, Embedding, LMHead, Runtime, StepContext, TensorDecl,
                   apply_norm, linear)


class PreNormResidual(Block):
    graph_safe = True
    accepts_deferred = True
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, layer: BuiltLayer, hidden: torch.Tensor, pending, ctx: StepContext, caches):
        x = apply_norm(layer.mixer_norm, hidden, pending)
        y = layer.mixer.forward(x, ctx, caches.get("mixer"))
        return layer.feed_forward.forward_from_residual(hidden, y, layer.feed_forward_norm, ctx)

    def prefetch_layer(self, layer: BuiltLayer, ctx: StepContext, caches) -> None:
        layer.mixer.prefetch_first(ctx, caches.get("mixer"))


class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``hidden_size``.  Tensor: ``<prefix>weight [V, H]``; no scaling
    (src/model/transformer_model.cpp:561-565)."""

    graph_safe = True

    def tensor_decls(self) -> List[TensorDecl]:
        return [TensorDecl(self.prefix + "weight", (self.params["vocab_size"], self.params["hidden_size"]))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = rt.precision.matrix(tensors[self.prefix + "weight"], rt.device)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return F.embed_gather(token_ids, self.weight)


class LinearHead(LMHead):
    """params: ``vocab_size``, ``hidden_size``, ``tied_to`` (name of the embedding tensor, or
    None).  Tensor: ``<prefix>weight [V, H]`` unless tied (src/model/transformer_model.cpp:355-361;
    the reference deep-copies the tied matrix, here it is the same storage)."""

    graph_safe = True

    def tensor_decls(self) -> List[TensorDecl]:
        if self.params.get("tied_to"):
            return []
        return [TensorDecl(self.prefix + "weight", (self.params["vocab_size"], self.params["hidden_size"]))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.weight = None
        if not self.params.get("tied_to"):
            self.weight = rt.precision.matrix(tensors[self.prefix + "weight"], rt.device)

    def tie(self, embedding_weight: torch.Tensor) -> None:
        self.weight = embedding_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, torch.float32)


register_part("block", "prenorm_residual", PreNormResidual)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear", LinearHead)
