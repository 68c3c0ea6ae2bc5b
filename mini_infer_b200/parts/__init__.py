"""Built-in parts.  Importing this package registers them by kind."""

from . import base  # noqa: F401
from . import norm, position, attention, feed_forward, block  # noqa: F401
from .base import (Block, BuiltLayer, CacheBinding, Embedding, FeedForward, KVNeed, LMHead, Mixer, Norm, Part,
                   PositionEncoding, Precision, Runtime, StateNeed, StepContext, TensorDecl, linear,
                   precision_from_name)

__all__ = ["Block", "BuiltLayer", "CacheBinding", "Embedding", "FeedForward", "KVNeed", "LMHead", "Mixer", "Norm",
           "Part", "PositionEncoding", "Precision", "Runtime", "StateNeed", "StepContext", "TensorDecl", "linear",
           "precision_from_name"]
