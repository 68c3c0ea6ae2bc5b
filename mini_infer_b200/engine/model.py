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

from ..cache.manager import plan_groups
from ..ops import functional as F
from ..config.registry import part_class
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..parts.base import (BuiltLayer, CacheBinding, PagedCacheNeed, Part, Runtime, StateNeed, StepContext,
                          TensorDecl, apply_norm, resolve)


def _make(category: str, spec: PartSpec, prefix: str) -> Part:
    return part_class(category, spec.kind)(spec.params, prefix)


def build_layer(ls: LayerSpec) -> BuiltLayer:
    """Instantiate the block and every part the layer names; the block kind says which roles it wires,
    and a description that lacks one, or brings one the block does not know, is refused."""
    base = ls.name + "." if ls.name else ""
    block = _make("block", ls.block, base)
    wanted = dict(getattr(block, "roles", {}) or {})
    if wanted:
        missing = [r for r in wanted if r not in ls.parts]
        extra = [r for r in ls.parts if r not in wanted]
        wrong = [r for r in wanted if r in ls.parts and ls.parts[r].category != wanted[r]]
        if missing or extra or wrong:
            raise ValueError(f"layer '{ls.name}': block '{ls.block.kind}' arranges the roles {sorted(wanted)}; "
                             f"missing {missing}, unknown {extra}, of another category {wrong}")
    parts = {role: _make(lp.category, lp.spec, base + lp.prefix) for role, lp in ls.parts.items()}
    return BuiltLayer(ls.name, block, parts)


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
        """Every part of a layer may keep something between steps (``cache_need()``): entries per token in
        pages, or a fixed-size state per request.  An owner is a (schedule position, role) pair; owners
        with the same paged need share a group (a pool and block tables of its own).  ``bindings[pos]``
        maps the roles of schedule entry ``pos`` that keep a cache to where they find it."""
        paged: List[Tuple[Tuple[int, str], PagedCacheNeed]] = []
        self.state_needs: List[Tuple[Tuple[int, str], StateNeed]] = []
        needs: List[Dict[str, object]] = []
        for pos, e in enumerate(self.spec.schedule):
            mine: Dict[str, object] = {}
            for role, part in self.layers[e.layer].parts.items():
                fn = getattr(part, "cache_need", None)
                need = fn() if fn else None
                if need is None:
                    continue
                if not isinstance(need, (PagedCacheNeed, StateNeed)):
                    raise TypeError(f"schedule[{pos}] {role}: cache_need() returned {type(need).__name__}")
                mine[role] = need
            needs.append(mine)
            for role, need in mine.items():
                if e.cache_from is not None and isinstance(need, PagedCacheNeed):
                    src = needs[e.cache_from].get(role)
                    if not isinstance(src, PagedCacheNeed) or src.geometry() != need.geometry():
                        raise ValueError(f"schedule[{pos}] reads the cache of schedule[{e.cache_from}], "
                                         f"whose geometry differs")
                    continue
                if isinstance(need, PagedCacheNeed):
                    paged.append(((pos, role), need))
                else:
                    self.state_needs.append(((pos, role), need))
        self.kv_groups, where = plan_groups(paged)
        state_index = {owner: i for i, (owner, _) in enumerate(self.state_needs)}
        self.bindings: List[Dict[str, CacheBinding]] = []
        for pos, e in enumerate(self.spec.schedule):
            found: Dict[str, CacheBinding] = {}
            for role, need in needs[pos].items():
                if isinstance(need, StateNeed):
                    found[role] = CacheBinding("state", state_index[(pos, role)], -1, True)
                elif e.cache_from is not None:
                    g, li = where[(e.cache_from, role)]
                    found[role] = CacheBinding("kv", g, li, writes=False)
                else:
                    g, li = where[(pos, role)]
                    found[role] = CacheBinding("kv", g, li, writes=True)
            self.bindings.append(found)

    # -- weights ------------------------------------------------------------ #
    def all_parts(self) -> List[Part]:
        parts: List[Part] = [self.embedding]
        for layer in self.layers:
            parts.extend(layer.all_parts())
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
        for part in self.all_parts():
            fn = getattr(part, "scratch_need", None)
            if fn:
                for k, v in fn(max_requests, max_context).items():
                    need[k] = max(need.get(k, 0), v)
        return need

    # -- one forward pass ---------------------------------------------------- #
    def forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run all tokens of ``ctx``; return float32 logits ``[R, V]`` for ``logit_rows`` (int32
        token indices), or None when no logits are wanted (the cache is still written)."""
        if ctx.dependent_launch:
            with F.dependent_launch(True):
                return self._forward(ctx, logit_rows)
        return self._forward(ctx, logit_rows)

    def _forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        hidden = self.embedding.forward(ctx.token_ids)
        pending = None
        schedule = self.spec.schedule
        for pos, e in enumerate(schedule):
            layer = self.layers[e.layer]
            if not layer.block.accepts_deferred:
                pending = resolve(pending)
            if ctx.prefetch is not None:
                # what the layer after this one reads first, for this layer's last part to ask L2 for
                ctx.prefetch_upcoming = None
                if pos + 1 < len(schedule):
                    nxt, nxt_caches = self.layers[schedule[pos + 1].layer], self.bindings[pos + 1]
                    ctx.prefetch_upcoming = lambda n=nxt, c=nxt_caches: n.block.prefetch_layer(n, ctx, c)
            pending = layer.block.forward(layer, hidden, pending, ctx, self.bindings[pos])
            if self.layer_observer is not None:
                # the addition of a part's output is left to the next norm's kernel; form it here
                self.layer_observer(pos, hidden if pending is None else hidden + resolve(pending))
        if ctx.prefetch is not None:
            ctx.prefetch.join()
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        x = apply_norm(self.final_norm, hidden, pending, rows=logit_rows)
        return self.lm_head.forward(x)


def declared_tensors(spec: ModelSpec) -> List[TensorDecl]:
    return Model(spec).tensor_decls()
