"""Checkpoints: the safetensors container, the manifest check, random weights."""

from .loader import FolderSource, LazyTensors, WeightError, check_manifest
from .random_init import RandomSource, write_model_folder
from .safetensors_io import CheckpointFolder, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["FolderSource", "LazyTensors", "WeightError", "check_manifest", "RandomSource", "write_model_folder",
           "CheckpointFolder", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
