"""The step function: one batch of (request, its next tokens) through the model.

A batch may hold portions of prompts beside single decoded tokens, cut
anywhere; the step runs only the tokens it is given, as one flat batch of
``T = sum(len(tokens))`` rows, reads everything older from the cache, and
returns logits at the wanted places only.

Reference: ``forward_paged_batched`` (src/model/transformer_model.h:128-143)
takes a rectangle ``[B, S]`` that is either all prompts padded to a bucket or
all single tokens (src/scheduler/scheduler.cpp:206-209, :298-300), needs the
caller to have grown the block tables (src/layers/attention.h:106-108), and
re-uploads the tables in every layer (src/layers/attention.cpp:783-814).  Here
the batch is ragged, pages are reserved by the step itself (all or nothing),
and the metadata crosses to the device once per step.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..parts.base import KVGroupView, Runtime, StepContext
from .model import Model


@dataclass
class StepEntry:
    """The next tokens of one request, and the places among them whose logits are wanted."""

    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepResult:
    """``logits [R, V]`` float32 on the device (None if nothing was wanted); ``index[r]`` is
    ``(request, place among its tokens of this step)`` of row ``r``."""

    logits: Optional[torch.Tensor]
    index: List[Tuple[Hashable, int]]
    num_tokens: int


class StepError(ValueError):
    """The batch was refused before anything ran."""


class WeightPrefetcher:
    """Runs L2 prefetch requests on a stream of its own: a request starts once the kernels queued on the
    calling stream so far have finished, beside whatever is queued next.  ``join`` ties the stream back
    in (a captured pass has to end with every forked stream joined)."""

    def __init__(self, device):
        self.stream = torch.cuda.Stream(device=device)
        self.forked = False

    def __call__(self, what) -> None:
        from ..ops import functional as F
        if what is None:
            return
        if not callable(what):
            what = [t for t in what if t is not None]
            if not what:
                return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            if callable(what):
                what()
            else:
                for t in what:
                    F.l2_prefetch(t)
        self.forked = True

    def join(self) -> None:
        if self.forked:
            torch.cuda.current_stream().wait_stream(self.stream)
            self.forked = False


class ModelRunner:
    """Owns the device side of the cache and runs steps.

    ``num_pages`` pages of ``page_size`` tokens per cache group; at most
    ``max_requests`` live requests (state slots), ``max_tokens_per_step`` rows per
    step, ``max_context`` tokens per request.
    """

    def __init__(self, model: Model, rt: Runtime, *, page_size: int, num_pages: int, max_requests: int,
                 max_tokens_per_step: int, max_context: int, cuda_graphs: bool = True, graph_chunk_tokens: int = 0):
        if rt.device.type != "cuda":
            raise RuntimeError("ModelRunner: the engine runs on a CUDA device only; there is no CPU path")
        self.model = model
        self.rt = rt
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_tokens = int(max_tokens_per_step)
        self.max_context = int(max_context)
        self.vocab_size = model.spec.vocab_size
        groups = model.kv_groups
        dev, act = rt.device, rt.act
        # Pages per group: the budget times the need's own share; a group behind a window never holds more
        # than its window and one step's tokens per request, so it is not given more than that.
        pages = []
        for g in groups:
            n = max(1, int(num_pages * float(g.need.pages_fraction)))
            if g.window > 0:
                per_request = -(-(g.window + self.max_tokens) // self.page_size) + 2
                n = min(n, max_requests * min(per_request, -(-self.max_context // self.page_size)))
            pages.append(n)
        self.cache = CacheManager(groups, pages, page_size, max_requests)
        # the tensors every group's need names: [layers of the group, pages, *shape of one page]
        self.kv_tensors: List[Dict[str, torch.Tensor]] = []
        for g, n in zip(groups, pages):
            self.kv_tensors.append({name: torch.zeros((g.num_layers, n) + tuple(shape), dtype=dtype or act, device=dev)
                                    for name, shape, dtype in g.need.tensors(page_size)})
        # (one slot more than requests: the rows that only fill a captured batch up write their state there)
        self.state_tensors = [torch.zeros((max_requests + 1,) + tuple(need.shape), dtype=need.dtype or torch.float32,
                                          device=dev) for _, need in model.state_needs]
        self.scratch = {k: torch.empty(n, dtype=torch.float32, device=dev)
                        for k, n in model.scratch_need(max_requests, max_context).items()}
        self.max_pages = -(-self.max_context // self.page_size)
        self._layout_staging()
        # Decode steps (one token per request, logits wanted for each) are launch-bound: their
        # forward pass is captured once per batch size as a CUDA graph and replayed.  Parts that
        # read host-side data of the step, or were not written with replay in mind, switch this off
        # by not declaring ``graph_safe``; a part with a state of its own may declare it (its state
        # tensor is static memory that a captured pass updates in place).
        self.cuda_graphs = bool(cuda_graphs) and all(getattr(p, "graph_safe", False) for p in model.all_parts())
        # steps of exactly this many tokens of one request (the scheduler's full prompt portions) are replayed
        # from a captured pass as well (0: only decode steps are)
        self.graph_chunk_tokens = int(graph_chunk_tokens)
        self._graphs: Dict[tuple, tuple] = {}
        self._prefetcher = WeightPrefetcher(rt.device)
        # parts with settings that change what a captured pass launches, or that leave side outputs
        from ..parts.base import Part
        self._keyed_parts = [p for p in model.all_parts() if type(p).capture_key is not Part.capture_key
                             or type(p).side_outputs is not Part.side_outputs]
        self._graph_pool = None
        self.graph_replays = 0
        self.graph_kernel_launches = 0      # kernels of this library launched through graph replays

    # ------------------------------------------------------------------ #
    # staging: one pinned buffer, one copy per step
    # ------------------------------------------------------------------ #
    def _layout_staging(self) -> None:
        T, B, G = self.max_tokens, self.max_requests, len(self.model.kv_groups)
        off = 0
        self._sec: Dict[str, Tuple[int, int]] = {}

        def sec(name, n):
            nonlocal off
            self._sec[name] = (off, n)
            off += (n + 3) // 4 * 4      # keep every section 16-byte aligned

        for name in ("token_ids", "positions", "req_of_token", "logit_rows"):
            sec(name, T)
        sec("q_start", B + 1)
        for name in ("kv_len", "state_slot", "fresh"):
            sec(name, B)
        for g in range(G):
            sec(f"slot_mapping{g}", T)
            sec(f"block_table{g}", B * self.max_pages)
        self._host = torch.zeros(off, dtype=torch.int32).pin_memory()
        self._host_np = self._host.numpy()          # the same pinned memory, for whole-array writes
        self.host_prepare_seconds = 0.0             # host time spent validating, reserving and staging
        self._dev = torch.zeros(off, dtype=torch.int32, device=self.rt.device)
        self._copied = torch.cuda.Event()
        self._copied.record()

    def _hview_np(self, name: str, n: int) -> np.ndarray:
        o, cap = self._sec[name]
        return self._host_np[o:o + n]

    def _dview(self, name: str, n: int) -> torch.Tensor:
        o, cap = self._sec[name]
        return self._dev[o:o + n]

    # ------------------------------------------------------------------ #
    # requests
    # ------------------------------------------------------------------ #
    def add_request(self, rid: Hashable) -> None:
        slot = self.cache.add_request(rid)
        for st in self.state_tensors:
            st[slot].zero_()

    def release(self, rid: Hashable) -> None:
        self.cache.release(rid)

    def has_request(self, rid: Hashable) -> bool:
        return self.cache.has_request(rid)

    def num_tokens(self, rid: Hashable) -> int:
        return self.cache.num_tokens(rid)

    # ------------------------------------------------------------------ #
    # the step
    # ------------------------------------------------------------------ #
    def validate(self, entries: Sequence[StepEntry]) -> List[np.ndarray]:
        """Refuse a bad batch before anything runs.  Returns every entry's token ids as an int64 array."""
        if not entries:
            raise StepError("step: empty batch")
        if len(entries) > self.max_requests:
            raise StepError(f"step: {len(entries)} requests exceed the limit {self.max_requests}")
        seen = set()
        total = 0
        arrays = []
        for e in entries:
            if e.rid in seen:
                raise StepError(f"step: request {e.rid!r} appears twice in one batch")
            seen.add(e.rid)
            if not self.cache.has_request(e.rid):
                raise StepError(f"step: unknown request {e.rid!r}")
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"step: request {e.rid!r} brings no tokens")
            total += n
            if self.cache.num_tokens(e.rid) + n > self.max_context:
                raise StepError(f"step: request {e.rid!r} would reach {self.cache.num_tokens(e.rid) + n} "
                                f"tokens, the context limit is {self.max_context}")
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.ndim != 1:
                raise StepError(f"step: the tokens of request {e.rid!r} are not a flat list")
            if int(toks.min()) < 0 or int(toks.max()) >= self.vocab_size:
                bad = int(toks[(toks < 0) | (toks >= self.vocab_size)][0])
                raise StepError(f"step: token id {bad} of request {e.rid!r} outside [0, {self.vocab_size})")
            arrays.append(toks)
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"step: wanted place {w} of request {e.rid!r} outside its {n} tokens")
        if total > self.max_tokens:
            raise StepError(f"step: {total} tokens exceed the budget {self.max_tokens}")
        return arrays

    def prepare(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
                ahead: bool = False, pad_to: int = 0) -> Tuple[StepContext, Optional[torch.Tensor], List]:
        """Validate, reserve pages (all entries or none), stage and upload the metadata.

        ``pad_to`` (decode steps that are replayed from a captured pass): the batch is filled up to this many
        rows with rows of no request (see :meth:`_stage`).

        With ``device_tokens`` (int32, one per row, on the device) the token ids of ``entries`` are
        placeholders and the step reads the given ones; ``ahead`` reserves through
        :meth:`CacheManager.reserve_ahead`.  Whatever goes wrong after pages were reserved, every
        reservation of the step is undone before the error leaves."""
        t_begin = time.perf_counter()
        arrays = self.validate(entries)
        starts = []
        done = []
        try:
            for e in entries:
                starts.append(self.cache.reserve_ahead(e.rid, len(e.tokens)) if ahead
                              else self.cache.reserve(e.rid, len(e.tokens)))
                done.append(e.rid)
            staged = self._stage(entries, arrays, starts, device_tokens, pad_to)
        except BaseException:
            for rid in done:
                self.cache.cancel(rid)
            raise
        self.host_prepare_seconds += time.perf_counter() - t_begin
        return staged

    def _stage(self, entries, arrays, starts, device_tokens, pad_to=0):
        """Fill the pinned staging buffer (whole arrays at a time, no per-token work on the host) and
        queue its one copy to the device.

        With ``pad_to`` above the number of entries, rows of no request follow the entries' rows, one
        token each: token 0 at position 0, written nowhere (slot -1), attending to the one key at the start
        of page 0 (finite data whatever it is), state in the spare slot, logits wanted so that the shapes
        are those of a full batch.  Every kernel works row by row, so the entries' results are what they
        would be without them; the caller drops the extra rows of logits."""
        B_real = len(entries)
        extra = max(0, int(pad_to) - B_real)
        B = B_real + extra
        counts = np.fromiter((a.shape[0] for a in arrays), dtype=np.int64, count=B_real)
        starts_np = np.asarray(starts, dtype=np.int64)
        T_real = int(counts.sum())
        if extra:
            counts = np.concatenate([counts, np.ones(extra, dtype=np.int64)])
            starts_np = np.concatenate([starts_np, np.zeros(extra, dtype=np.int64)])
            arrays = list(arrays) + [np.zeros(extra, dtype=np.int64)]
        T = int(counts.sum())
        self._copied.synchronize()      # the previous step's upload has left the pinned buffer
        h = self._hview_np
        first = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(counts, out=first[1:])
        req_of_token = np.repeat(np.arange(B, dtype=np.int64), counts)
        positions = np.arange(T, dtype=np.int64) - first[req_of_token] + starts_np[req_of_token]
        kv_len = starts_np + counts
        slots = np.fromiter((self.cache.slot_of(e.rid) for e in entries), dtype=np.int64, count=B_real)
        if extra:
            slots = np.concatenate([slots, np.full(extra, self.max_requests, dtype=np.int64)])
        h("token_ids", T)[:] = np.concatenate(arrays)
        h("positions", T)[:] = positions
        h("req_of_token", T)[:] = req_of_token
        h("q_start", B + 1)[:] = first
        h("kv_len", B)[:] = kv_len
        h("state_slot", B)[:] = slots
        h("fresh", B)[:] = starts_np == 0
        index: List[Tuple[Hashable, int]] = []
        row_l: List[int] = []
        for b, e in enumerate(entries):
            for w in e.want:
                row_l.append(int(first[b]) + int(w))
                index.append((e.rid, int(w)))
        row_l.extend(range(T_real, T))
        R = len(row_l)
        if R:
            h("logit_rows", R)[:] = row_l
        ps = self.page_size
        for g in range(len(self.model.kv_groups)):
            bt = h(f"block_table{g}", B * self.max_pages).reshape(B, self.max_pages)
            bt.fill(-1)
            for b, e in enumerate(entries):
                table = self.cache.block_table(g, e.rid)
                bt[b, :len(table)] = table
            bt[B_real:, 0] = 0
            pages = bt[req_of_token, positions // ps]
            if pages.size and int(pages[:T_real].min()) < 0:
                t = int(np.argmin(pages[:T_real]))
                raise RuntimeError(f"step: position {int(positions[t])} of request {entries[int(req_of_token[t])].rid!r} "
                                   f"lies in a released page of cache group {g}")
            h(f"slot_mapping{g}", T)[:] = pages.astype(np.int64) * ps + positions % ps
            h(f"slot_mapping{g}", T)[T_real:] = -1
        self._dev.copy_(self._host, non_blocking=True)
        self._copied.record()
        d = self._dview
        if device_tokens is not None:
            d("token_ids", T_real).copy_(device_tokens[:T_real], non_blocking=True)
        views = []
        for g in range(len(self.model.kv_groups)):
            views.append(KVGroupView(
                block_table=d(f"block_table{g}", B * self.max_pages).view(B, self.max_pages),
                slot_mapping=d(f"slot_mapping{g}", T), page_size=self.page_size, tensors=self.kv_tensors[g]))
        max_q, max_kv = int(counts.max()), int(kv_len.max())
        ctx = StepContext(
            num_tokens=T, num_requests=B, max_q_len=max_q, max_kv_len=max_kv, all_decode=(max_q == 1),
            token_ids=d("token_ids", T), positions=d("positions", T), q_start=d("q_start", B + 1),
            kv_len=d("kv_len", B), req_of_token=d("req_of_token", T), state_slot=d("state_slot", B),
            fresh=d("fresh", B), kv_groups=views, states=self.state_tensors, scratch=self.scratch,
            host_q_start=first.tolist(), host_kv_len=kv_len.tolist(), host_state_slot=slots.tolist())
        ctx.rows_of_no_request = extra
        single = counts == 1
        lead = B if bool(single.all()) else int(np.argmin(single))
        ctx.num_leading_decodes = lead
        ctx.leading_decodes_max_kv_len = int(kv_len[:lead].max()) if lead else 0
        from ..parts.tuning import TUNING
        if self.rt.act == torch.bfloat16 and T <= TUNING.l2_prefetch_max_tokens:
            ctx.prefetch = self._prefetcher
        ctx.dependent_launch = self.rt.act == torch.bfloat16 and T <= TUNING.dependent_launch_max_tokens
        logit_rows = d("logit_rows", R) if R else None
        return ctx, logit_rows, index

    def _graphs_allowed(self) -> bool:
        if not self.cuda_graphs or self.model.layer_observer is not None:
            return False
        from ..ops import functional as F
        return not F.DEBUG_BOUNDS    # the debug checks read indices back on the host: not inside a capture

    def _graph_eligible(self, entries: Sequence[StepEntry]) -> bool:
        """A decode step: one token per request, logits wanted for each."""
        return self._graphs_allowed() and not any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries)

    def _chunk_graph_eligible(self, entries: Sequence[StepEntry]) -> bool:
        """A full portion of one prompt: with chunked prefill every full chunk of a long prompt has the same
        shape (one request, ``graph_chunk_tokens`` tokens, logits at the last place or nowhere), and how
        much context lies before it is device data, so its forward pass is captured once and replayed: the
        gaps between the dependent launches of an eager pass shrink to a graph's."""
        if self.graph_chunk_tokens <= 0 or len(entries) != 1 or not self._graphs_allowed():
            return False
        e = entries[0]
        n = len(e.tokens)
        return n == self.graph_chunk_tokens and list(e.want) in ([], [n - 1])

    def _graph_batch(self, num_requests: int) -> int:
        """The batch size whose captured pass a decode step of ``num_requests`` requests is replayed from:
        the next size of the tuning's ladder, so that a batch that grows and shrinks by single requests does
        not capture a pass per size."""
        from ..parts.tuning import TUNING
        return min(TUNING.decode_graph_batch(num_requests), self.max_requests, self.max_tokens)

    def _decode_with_graph(self, ctx: StepContext, logit_rows: Optional[torch.Tensor],
                           chunk: bool = False) -> Optional[torch.Tensor]:
        """Replay (or first capture) the forward pass for this batch size and context-length bucket.
        The captured pass reads the same staging views every time and is launched for the longest
        context of its bucket, so only the data in the staging buffer changes between replays."""
        B = ctx.num_requests
        if chunk:
            # no launch shape of a prompt portion follows the context length
            ctx.max_kv_len = self.max_context
        else:
            # launch shapes that follow the context length (the splits of the decode attention) are captured
            # for the next power of two, at least 1024: a few graphs per batch size, and a short context is
            # not launched with the grid of the longest one
            bucket = 1024
            while bucket < ctx.max_kv_len:
                bucket *= 2
            ctx.max_kv_len = min(bucket, self.max_context)
        parts = self._keyed_parts
        key = (B, ctx.max_kv_len, tuple(p.capture_key() for p in parts),
               (ctx.num_tokens, logit_rows is not None) if chunk else None)
        if key not in self._graphs:
            # The warm-up pass (library workspaces, lazy initialisation) runs the step for real: what it
            # writes into the paged caches is written again by the replay, but a per-request state would
            # be advanced twice, so states are put back after it.
            kept = [st.clone() for st in self.state_tensors]
            side = torch.cuda.Stream(device=self.rt.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.model.forward(ctx, logit_rows)
            torch.cuda.current_stream().wait_stream(side)
            for st, old in zip(self.state_tensors, kept):
                st.copy_(old)
            torch.cuda.synchronize(self.rt.device)
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            from ..ops.library import launch_count
            before = launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self._graph_pool):
                out = self.model.forward(ctx, logit_rows)
            self._graphs[key] = (g, out, launch_count() - before, [p.side_outputs() for p in parts])
        g, out, kernels, side = self._graphs[key]
        g.replay()
        for p, outputs in zip(parts, side):
            if outputs is not None:
                p.adopt_side_outputs(outputs)
        self.graph_replays += 1
        self.graph_kernel_launches += kernels
        if out is not None and ctx.rows_of_no_request:
            out = out[:out.shape[0] - ctx.rows_of_no_request]
        return out

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry]) -> StepResult:
        decode_graph = self._graph_eligible(entries)
        ctx, logit_rows, index = self.prepare(entries, pad_to=self._graph_batch(len(entries)) if decode_graph else 0)
        # What a failed step wrote into the paged caches lies beyond every request's committed tokens and
        # is written again; a per-request state is updated in place, so the entries' slots are kept aside
        # and put back if the forward pass fails.
        saved = None
        if self.state_tensors:
            slots = torch.as_tensor(ctx.host_state_slot, dtype=torch.long, device=self.rt.device)
            saved = (slots, [st.index_select(0, slots) for st in self.state_tensors])
        try:
            if decode_graph:
                logits = self._decode_with_graph(ctx, logit_rows)
            elif self._chunk_graph_eligible(entries):
                logits = self._decode_with_graph(ctx, logit_rows, chunk=True)
                from ..ops.functional import check_tc_status
                check_tc_status()
            else:
                logits = self.model.forward(ctx, logit_rows)
                from ..ops.functional import check_tc_status
                check_tc_status()
        except Exception:
            for e in entries:
                self.cache.cancel(e.rid)
            if saved is not None:
                for st, rows in zip(self.state_tensors, saved[1]):
                    st.index_copy_(0, saved[0], rows)
            raise
        for e in entries:
            self.cache.commit(e.rid)
        return StepResult(logits, index, ctx.num_tokens - ctx.rows_of_no_request)

    # ------------------------------------------------------------------ #
    # a decode step launched ahead of the scheduler's decision
    # ------------------------------------------------------------------ #
    def can_step_ahead(self, rids: Sequence[Hashable]) -> bool:
        """A step of one token per request can be launched ahead only as a graph replay, and only by a
        model without per-request state: a dropped step's cache writes lie beyond the committed tokens
        and are overwritten, but a state updated in place could not be taken back."""
        if self.state_tensors:
            return False
        return self._graph_eligible([StepEntry(r, [0], [0]) for r in rids])

    @torch.no_grad()
    def step_ahead(self, rids: Sequence[Hashable], device_tokens: torch.Tensor) -> torch.Tensor:
        """Launch the decode step that feeds request ``rids[b]`` the token ``device_tokens[b]``
        (still being computed on the device) and return its logits ``[B, V]``.  Pages are held
        through :meth:`CacheManager.reserve_ahead`; the caller settles the step with
        :meth:`adopt_ahead` or :meth:`drop_ahead`.  Raises :class:`OutOfPages` and changes nothing
        if a request cannot grow."""
        entries = [StepEntry(r, [0], [0]) for r in rids]
        ctx, logit_rows, _ = self.prepare(entries, device_tokens=device_tokens, ahead=True,
                                          pad_to=self._graph_batch(len(entries)))
        try:
            return self._decode_with_graph(ctx, logit_rows)
        except Exception:
            self.drop_ahead(rids)
            raise

    def adopt_ahead(self, rids: Sequence[Hashable]) -> None:
        """The step launched ahead was the one decided: its tokens are in the cache."""
        for r in rids:
            self.cache.adopt_ahead(r)
            self.cache.commit(r)

    def drop_ahead(self, rids: Sequence[Hashable]) -> None:
        """The step launched ahead is void (what it wrote lies beyond every request's cached tokens
        and is overwritten by the step that is decided instead)."""
        for r in rids:
            if self.cache.has_ahead(r):
                self.cache.cancel(r)
