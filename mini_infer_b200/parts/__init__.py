"""Built-in parts.  Importing this package registers them by kind."""

from . import base  # noqa: F401
from . import norm, position, attention, feed_forward, block  # noqa: F401
from .base import (Block, BuiltLayer, CacheBinding, Deferred, Embedding, FeedForward, KVGroupView, KVNeed, LMHead, Mixer, Norm,
                   PagedCacheNeed, Part, PositionEncoding, Precision, Runtime, StateNeed, StepContext, TensorDecl, WeightedRowSum,
                   apply_norm, linear, precision_from_name, resolve)

__all__ = ["Block", "BuiltLayer", "CacheBinding", "Deferred", "Embedding", "FeedForward", "KVGroupView", "KVNeed", "PagedCacheNeed", "LMHead", "Mixer",
           "Norm", "Part", "PositionEncoding", "Precision", "Runtime", "StateNeed", "StepContext", "TensorDecl",
           "WeightedRowSum", "apply_norm", "linear", "precision_from_name", "resolve"]
