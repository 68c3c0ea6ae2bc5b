"""Data that describes a model as an arrangement of parts.

A model is not a class hierarchy here but a :class:`ModelSpec`: a tuple of
:class:`LayerSpec` (each naming its block arrangement and, by *role*, the parts
the arrangement wires together: for the usual pre-norm block a mixer, a
feed-forward and two norms; another arrangement names other roles) plus a
*schedule*, the order in which layers run.  The schedule is data as well: it
may name a layer twice (the weights are shared, each run has a cache of its
own) and an entry may read the cache that an earlier entry wrote instead of
writing one.

The reference hard-wires one arrangement into ``TransformerModel``
(src/model/transformer_model.cpp:118-185 builds it, :545-675 runs it) and its
``ArchTraits`` (src/model/arch_registry.h:20-62) are never consulted by the
forward pass; here the description is what the engine executes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part chosen by ``kind`` from the part registry, with its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerPart:
    """One part of a layer: its registry category, its kind and constants, and its checkpoint
    sub-prefix below the layer's name."""

    category: str
    spec: PartSpec
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One set of weights: a block kind and the parts it arranges, by role.

    ``name`` is the checkpoint prefix of the layer (``model.layers.3``).  Which roles there are is the
    block kind's business (``Block.roles``): the pre-norm residual block wants ``mixer``, ``feed_forward``,
    ``mixer_norm`` and ``feed_forward_norm``; a block with four norms, or without a feed-forward, is
    another block class with other roles, and nothing else changes.  A role's ``PartSpec`` can be read as
    an attribute (``layer.mixer``).
    """

    name: str
    block: PartSpec
    parts: Mapping[str, LayerPart]

    def __getattr__(self, role: str) -> PartSpec:
        if role in ("name", "block", "parts") or role.startswith("__"):
            raise AttributeError(role)
        try:
            return self.parts[role].spec
        except KeyError:
            raise AttributeError(f"layer '{self.name}' has no part in the role '{role}' "
                                 f"(roles: {', '.join(self.parts)})") from None

    def with_part(self, role: str, spec: PartSpec, category: Optional[str] = None,
                  prefix: Optional[str] = None) -> "LayerSpec":
        """A copy with the part of ``role`` replaced (or added: then ``category`` is needed)."""
        old = self.parts.get(role)
        if old is None and category is None:
            raise ValueError(f"layer '{self.name}': a new role '{role}' needs its category")
        part = LayerPart(category or old.category, spec, prefix if prefix is not None else (old.prefix if old else ""))
        return LayerSpec(self.name, self.block, {**self.parts, role: part})

    def renamed(self, name: str) -> "LayerSpec":
        return LayerSpec(name, self.block, dict(self.parts))


def prenorm_layer(name: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                  feed_forward_norm: PartSpec, block: PartSpec = PartSpec("prenorm_residual"),
                  mixer_prefix: str = "self_attn.", feed_forward_prefix: str = "mlp.",
                  mixer_norm_prefix: str = "input_layernorm.",
                  feed_forward_norm_prefix: str = "post_attention_layernorm.") -> LayerSpec:
    """The usual layer: norm, mixer, norm, feed-forward around a residual stream, with the checkpoint
    names of the LLaMA/Qwen family."""
    return LayerSpec(name, block, {
        "mixer_norm": LayerPart("norm", mixer_norm, mixer_norm_prefix),
        "mixer": LayerPart("mixer", mixer, mixer_prefix),
        "feed_forward_norm": LayerPart("norm", feed_forward_norm, feed_forward_norm_prefix),
        "feed_forward": LayerPart("feed_forward", feed_forward, feed_forward_prefix),
    })


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_from`` names an earlier schedule position
    whose caches this run reads, role by role (it then writes none of its own)."""

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_context: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    lm_head: PartSpec
    embedding_prefix: str = "model.embed_tokens."
    final_norm_prefix: str = "model.norm."
    lm_head_prefix: str = "lm_head."

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("ModelSpec: a model needs at least one layer")
        if not self.schedule:
            raise ValueError("ModelSpec: the schedule is empty")
        for pos, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"ModelSpec: schedule[{pos}] names layer {e.layer}, "
                                 f"the model has {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < pos:
                    raise ValueError(f"ModelSpec: schedule[{pos}].cache_from={e.cache_from} "
                                     f"must name an earlier schedule position")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ValueError(f"ModelSpec: schedule[{pos}].cache_from={e.cache_from} "
                                     f"names an entry that owns no cache itself")


def default_schedule(num_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i) for i in range(num_layers))
