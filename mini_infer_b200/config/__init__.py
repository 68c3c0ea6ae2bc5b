"""Typed configuration, model description and the registries."""

from .model_config import ConfigError, Qwen2MoeConfig, architecture_name, read_config_json
from .registry import (UnknownArchitecture, UnknownPart, build_model_spec, known_architectures, known_parts,
                       part_class, register_architecture, register_part)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule

__all__ = ["ConfigError", "Qwen2MoeConfig", "architecture_name", "read_config_json", "UnknownArchitecture",
           "UnknownPart", "build_model_spec", "known_architectures", "known_parts", "part_class",
           "register_architecture", "register_part", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry",
           "default_schedule"]
