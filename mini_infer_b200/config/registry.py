"""Registries: architecture name -> model builder, (category, kind) -> part class.

The reference keeps a static switch from a ``ModelArch`` enum to a traits
struct (src/model/arch_registry.h:31-62) and buckets every unknown
``model_type`` with Qwen/LLaMA (src/model/model_config.cpp:44-51).  Here the
key is the string in ``config.json``'s ``architectures[0]``, an unknown name is
an error that lists the known ones, and a second table maps part kinds to
their classes so that a layer description can be resolved without the model
knowing which parts exist.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Tuple

from .spec import ModelSpec

# name -> (builder(config_json_dict) -> ModelSpec, description)
_ARCHITECTURES: Dict[str, Tuple[Callable[[Dict[str, Any]], ModelSpec], str]] = {}

# category -> kind -> class
PART_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "lm_head")
_PARTS: Dict[str, Dict[str, type]] = {c: {} for c in PART_CATEGORIES}


class UnknownArchitecture(KeyError):
    pass


class UnknownPart(KeyError):
    pass


def register_architecture(name: str, builder: Callable[[Dict[str, Any]], ModelSpec],
                          description: str = "") -> None:
    """Make ``name`` (as written in ``architectures[0]``) buildable."""
    _ARCHITECTURES[name] = (builder, description)


def known_architectures() -> List[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def build_model_spec(config_json: Dict[str, Any]) -> ModelSpec:
    """Turn the dictionary of ``config.json`` into a validated :class:`ModelSpec`."""
    from .model_config import architecture_name
    _ensure_builtin()
    name = architecture_name(config_json)
    if name not in _ARCHITECTURES:
        raise UnknownArchitecture(
            f"unknown architecture '{name}'; this engine builds: {', '.join(sorted(_ARCHITECTURES))}")
    spec = _ARCHITECTURES[name][0](config_json)
    spec.validate()
    return spec


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in _PARTS:
        raise UnknownPart(f"unknown part category '{category}'; categories: {', '.join(PART_CATEGORIES)}")
    _PARTS[category][kind] = cls


def part_class(category: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[category][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(category, {}))) or "(none)"
        raise UnknownPart(f"no {category} part of kind '{kind}' is registered; known: {known}") from None


def known_parts(category: str) -> List[str]:
    _ensure_builtin()
    return sorted(_PARTS[category])


_builtin_loaded = False


def _ensure_builtin() -> None:
    """Import the modules whose import registers the built-in parts and models."""
    global _builtin_loaded
    if _builtin_loaded:
        return
    _builtin_loaded = True
    import importlib
    importlib.import_module("mini_infer_b200.parts")
    importlib.import_module("mini_infer_b200.models")
