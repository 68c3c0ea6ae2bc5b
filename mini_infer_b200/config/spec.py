"""Data that describes a model as an arrangement of parts.

A model is not a class hierarchy here but a :class:`ModelSpec`: a tuple of
:class:`LayerSpec` (each naming, by *kind* and parameters, its mixer, its
feed-forward, its two norms and the block arrangement that wires them) plus a
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
class LayerSpec:
    """One set of weights: a mixer, a feed-forward, their norms, a block kind.

    ``name`` is the checkpoint prefix of the layer (``model.layers.3``).
    """

    name: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: PartSpec = PartSpec("prenorm_residual")
    # checkpoint sub-prefixes of the parts below ``name``
    mixer_prefix: str = "self_attn."
    feed_forward_prefix: str = "mlp."
    mixer_norm_prefix: str = "input_layernorm."
    feed_forward_norm_prefix: str = "post_attention_layernorm."


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_from`` names an earlier schedule position
    whose cache this run reads (it then writes none of its own)."""

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
