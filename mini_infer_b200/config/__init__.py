"""Typed configuration, model description and the registries."""

from .model_config import ConfigError, Qwen2MoeConfig, architecture_name, read_config_json
from .registry import (UnknownArchitecture, UnknownPart, build_model_spec, known_architectures, known_parts,
                       part_class, register_architecture, register_part)
from .spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule, prenorm_layer

__all__ = ["ConfigError", "Qwen2MoeConfig", "architecture_name", "read_config_json", "UnknownArchitecture",
           "UnknownPart", "build_model_spec", "known_architectures", "known_parts", "part_class",
           "register_architecture", "register_part", "LayerPart", "LayerSpec", "prenorm_layer", "ModelSpec", "PartSpec", "ScheduleEntry",
           "default_schedule"]
