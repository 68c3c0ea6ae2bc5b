"""Architectures this engine builds.  Importing the package registers them by name."""

from . import qwen2_moe  # noqa: F401
