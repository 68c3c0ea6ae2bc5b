"""``mini_infer_sdk``: the reference's import name for the Python entry point (offline mode only)."""

from mini_infer_b200.sdk import (BatchInfer, BatchResult, BatchStats, ChatMessage, ChatSession, GenerationResult,
                                 InferenceConfig, MiniInfer, SamplingConfig, SamplingMode)

__version__ = "0.2.0"
__all__ = ["MiniInfer", "GenerationResult", "InferenceConfig", "SamplingConfig", "SamplingMode", "ChatSession",
           "ChatMessage", "BatchInfer", "BatchResult", "BatchStats"]
