"""A model as built parts, put together from a :class:`ModelSpec`.

``build_model`` resolves every part kind through the registry, so a layer whose
mixer or feed-forward kind was registered elsewhere (a test's toy part, a new
architecture) is built by the same code.  ``Model.forward`` is the whole
forward pass of one step: embedding, the schedule of layers, final norm on the
wanted rows, output head.  Reference: src/model/transformer_model.cpp:545-675,
which norms and projects every row; here only the rows whose logits are wanted.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import KVGroupSpec, plan_groups
from ..config.registry import part_class
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..parts.base import (BuiltLayer, CacheBinding, KVNeed, Part, Runtime, StateNeed, StepContext, TensorDecl,
                          apply_norm, resolve)


def _make(category: str, spec: PartSpec, prefix: str) -> Part:
    return part_class(category, spec.kind)(spec.params, prefix)


def build_layer(ls: LayerSpec) -> BuiltLayer:
    base = ls.name + "." if ls.name else ""
    return BuiltLayer(
        name=ls.name,
        mixer=_make("mixer", ls.mixer, base + ls.mixer_prefix),
        feed_forward=_make("feed_forward", ls.feed_forward, base + ls.feed_forward_prefix),
        mixer_norm=_make("norm", ls.mixer_norm, base + ls.mixer_norm_prefix),
        feed_forward_norm=_make("norm", ls.feed_forward_norm, base + ls.feed_forward_norm_prefix),
        block=_make("block", ls.block, base),
    )


class Model:
    """Parts of a whole model, before (``__init__``) and after (``load``) the weights arrive."""

    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = _make("embedding", spec.embedding, spec.embedding_prefix)
        self.layers: List[BuiltLayer] = [build_layer(ls) for ls in spec.layers]
        self.final_norm = _make("norm", spec.final_norm, spec.final_norm_prefix)
        self.lm_head = _make("lm_head", spec.lm_head, spec.lm_head_prefix)
        # debugging: ``layer_observer(schedule position, residual stream after that entry [T, H] float32)``
        # is called after every schedule entry of an eager forward pass (the reference's counterpart is
        # debug_print_tensor, src/model/transformer_model.cpp:24-61)
        self.layer_observer = None
        self._plan_caches()

    # -- what the model keeps between steps --------------------------------- #
    def _plan_caches(self) -> None:
        kv_needs: List[Tuple[int, KVNeed]] = []
        self.state_needs: List[Tuple[int, StateNeed]] = []
        needs = []
        for pos, e in enumerate(self.spec.schedule):
            need = self.layers[e.layer].mixer.cache_need()
            needs.append(need)
            if e.cache_from is not None:
                src = needs[e.cache_from]
                if not isinstance(need, KVNeed) or not isinstance(src, KVNeed) or \
                        (need.num_kv_heads, need.head_dim) != (src.num_kv_heads, src.head_dim):
                    raise ValueError(f"schedule[{pos}] reads the cache of schedule[{e.cache_from}], "
                                     f"whose geometry differs")
                continue
            if isinstance(need, KVNeed):
                kv_needs.append((pos, need))
            elif isinstance(need, StateNeed):
                self.state_needs.append((pos, need))
            elif need is not None:
                raise TypeError(f"schedule[{pos}]: cache_need() returned {type(need).__name__}")
        self.kv_groups, where = plan_groups(kv_needs)
        self.bindings: List[CacheBinding] = []
        state_index = {pos: i for i, (pos, _) in enumerate(self.state_needs)}
        for pos, e in enumerate(self.spec.schedule):
            if e.cache_from is not None:
                g, li = where[e.cache_from]
                self.bindings.append(CacheBinding("kv", g, li, writes=False))
            elif pos in where:
                g, li = where[pos]
                self.bindings.append(CacheBinding("kv", g, li, writes=True))
            elif pos in state_index:
                self.bindings.append(CacheBinding("state", state_index[pos], -1, True))
            else:
                self.bindings.append(CacheBinding("none"))

    # -- weights ------------------------------------------------------------ #
    def all_parts(self) -> List[Part]:
        parts: List[Part] = [self.embedding]
        for layer in self.layers:
            parts.extend(layer.parts())
        parts += [self.final_norm, self.lm_head]
        return parts

    def tensor_decls(self) -> List[TensorDecl]:
        out: List[TensorDecl] = []
        seen = set()
        for p in self.all_parts():
            for d in p.tensor_decls():
                if d.name in seen:
                    raise ValueError(f"two parts declare the tensor '{d.name}'")
                seen.add(d.name)
                out.append(d)
        return out

    def load(self, source, rt: Runtime, strict: bool = True) -> None:
        from ..weights.loader import LazyTensors, check_manifest
        decls = self.tensor_decls()
        allow = []
        tied = self.spec.lm_head.get("tied_to")
        if tied:
            # checkpoints of tied models often still carry the head; it is ignored, not an error
            allow.append(self.spec.lm_head_prefix + "weight")
        if strict:
            check_manifest(decls, source, allow_unexpected=allow)
        tensors = LazyTensors(source, [d.name for d in decls])
        for p in self.all_parts():
            p.load(tensors, rt)
        if tied:
            self.lm_head.tie(self.embedding.weight)
        self.rt = rt

    def scratch_need(self, max_requests: int, max_context: int) -> Dict[str, int]:
        need: Dict[str, int] = {}
        for layer in self.layers:
            fn = getattr(layer.mixer, "scratch_need", None)
            if fn:
                for k, v in fn(max_requests, max_context).items():
                    need[k] = max(need.get(k, 0), v)
        return need

    # -- one forward pass ---------------------------------------------------- #
    def forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run all tokens of ``ctx``; return float32 logits ``[R, V]`` for ``logit_rows`` (int32
        token indices), or None when no logits are wanted (the cache is still written)."""
        hidden = self.embedding.forward(ctx.token_ids)
        pending = None
        for pos, e in enumerate(self.spec.schedule):
            layer = self.layers[e.layer]
            if not layer.block.accepts_deferred:
                pending = resolve(pending)
            pending = layer.block.forward(layer, hidden, pending, ctx, self.bindings[pos])
            if self.layer_observer is not None:
                # the addition of a part's output is left to the next norm's kernel; form it here
                self.layer_observer(pos, hidden if pending is None else hidden + resolve(pending))
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        x = apply_norm(self.final_norm, hidden, pending, rows=logit_rows)
        return self.lm_head.forward(x)


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    return Model(spec).tensor_decls()
