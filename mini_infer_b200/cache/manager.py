"""The cache manager: paged keys and values in groups, block tables per request,
state slots.

A *group* is a set of layers whose caches have the same geometry and the same
retention rule (all keys, or a window of them).  Every group has a page pool
and block tables of its own; one page id addresses the same page in every
layer of its group, as in the reference, where all layers share one pool
(src/core/allocator.h:60-78) and there is a single kind of layer.  A request's
block table lists its pages by logical index (token position // page size);
once a window has passed a page, the page goes back to the pool and its entry
becomes -1.  Beside the pages, every live request holds one *state slot*, the
index under which mixers with a fixed-size state keep theirs.

Reference behaviour kept: pages are taken one per ``page_size`` tokens as a
request grows (src/scheduler/paged_kv_cache.cpp:62-80) and all returned when it
ends (:44-51).  Changed: growth is all-or-nothing for a whole portion
(:meth:`reserve`), across all groups, so a step never starts half-provisioned.

This module is host-only and has no dependency on CUDA; the device tensors
that the page ids index are owned by the engine.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .needs import KVNeed, PagedCacheNeed
from .pages import OutOfPages, OutOfSlots, PagePool, SlotPool


@dataclass(frozen=True)
class CacheGroupSpec:
    """One group: what its layers keep per token (``need``: tensors per page, retention, share of the
    page budget) and the cache owners it serves (``entries``: anything hashable, the engine uses
    ``(schedule position, role)``)."""

    need: PagedCacheNeed
    entries: Tuple[Hashable, ...] = ()

    @property
    def num_layers(self) -> int:
        return len(self.entries)

    @property
    def window(self) -> int:
        return int(self.need.window)

    def __getattr__(self, name):
        # geometry of the need (num_kv_heads, head_dim, ...) read through the group
        if name in ("need", "entries"):
            raise AttributeError(name)
        return getattr(self.need, name)


def KVGroupSpec(num_kv_heads: int, head_dim: int, window: int = 0, entries: Tuple[Hashable, ...] = ()) -> CacheGroupSpec:
    """A group of key/value layers (the common case), as a :class:`CacheGroupSpec`."""
    return CacheGroupSpec(KVNeed(num_kv_heads, head_dim, window), tuple(entries))


@dataclass
class _Request:
    slot: int
    num_tokens: int = 0                       # tokens whose keys are in the cache
    reserved: int = 0                         # tokens reserved beyond num_tokens for the running step
    ahead: int = 0                            # tokens reserved for a step launched before it was decided
    tables: List[List[int]] = field(default_factory=list)   # per group: page id by logical index


class CacheManager:
    def __init__(self, groups: Sequence[CacheGroupSpec], num_pages: Sequence[int], page_size: int,
                 num_slots: int):
        if page_size < 1 or page_size & (page_size - 1):
            raise ValueError(f"CacheManager: page size {page_size} must be a power of two")
        if len(groups) != len(num_pages):
            raise ValueError("CacheManager: one page count per group")
        self.groups = list(groups)
        self.page_size = int(page_size)
        self.pools = [PagePool(n) for n in num_pages]
        self.slots = SlotPool(num_slots)
        self._req: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------------ #
    # requests
    # ------------------------------------------------------------------ #
    def add_request(self, rid: Hashable) -> int:
        """Register ``rid`` and give it a state slot.  Raises :class:`OutOfSlots`."""
        if rid in self._req:
            raise ValueError(f"CacheManager: request {rid!r} is already live")
        slot = self.slots.alloc()
        self._req[rid] = _Request(slot=slot, tables=[[] for _ in self.groups])
        return slot

    def has_request(self, rid: Hashable) -> bool:
        return rid in self._req

    def live_requests(self) -> List[Hashable]:
        return list(self._req)

    def num_tokens(self, rid: Hashable) -> int:
        return self._req[rid].num_tokens

    def slot_of(self, rid: Hashable) -> int:
        return self._req[rid].slot

    def release(self, rid: Hashable) -> None:
        """Give back every page and the slot of ``rid``."""
        r = self._req.pop(rid)
        for g, table in enumerate(r.tables):
            for p in table:
                if p >= 0:
                    self.pools[g].free(p)
        self.slots.free(r.slot)

    # ------------------------------------------------------------------ #
    # growth
    # ------------------------------------------------------------------ #
    def pages_needed(self, rid: Hashable, n_new: int) -> List[int]:
        """Pages each group must add so that ``rid`` can take ``n_new`` more tokens."""
        r = self._req[rid]
        end = r.num_tokens + r.reserved + n_new
        want = -(-end // self.page_size)
        return [max(0, want - len(t)) for t in r.tables]

    def can_reserve(self, rid: Hashable, n_new: int) -> bool:
        return all(n <= pool.num_free for n, pool in zip(self.pages_needed(rid, n_new), self.pools))

    def reserve(self, rid: Hashable, n_new: int) -> int:
        """Provide pages for the next ``n_new`` tokens of ``rid`` in every group, or raise
        :class:`OutOfPages` and change nothing.  Returns the position of the first new token."""
        if n_new < 1:
            raise ValueError("CacheManager.reserve: a portion has at least one token")
        r = self._req[rid]
        if r.ahead:
            raise ValueError("CacheManager.reserve: a step launched ahead is unsettled (adopt or cancel it)")
        need = self.pages_needed(rid, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].num_free:
                raise OutOfPages(f"group {g}: {n} pages wanted for request {rid!r}, "
                                 f"{self.pools[g].num_free} free")
        for g, n in enumerate(need):
            r.tables[g].extend(self.pools[g].alloc_many(n))
        start = r.num_tokens + r.reserved
        r.reserved += n_new
        return start

    def reserve_ahead(self, rid: Hashable, n_new: int) -> int:
        """:meth:`reserve` for a step that is launched before the scheduler has decided it (its
        tokens are still being sampled).  The pages are held, but :meth:`pages_needed` keeps
        answering for the committed tokens, so planning the very same step finds its pages in
        place.  Settled by :meth:`adopt_ahead` (then :meth:`commit`) or :meth:`cancel`."""
        r = self._req[rid]
        if r.reserved or r.ahead:
            raise ValueError("CacheManager.reserve_ahead: another step of this request is unsettled")
        start = self.reserve(rid, n_new)
        r.reserved, r.ahead = 0, n_new
        return start

    def adopt_ahead(self, rid: Hashable) -> None:
        """The step launched ahead is the one that was decided: its tokens count as reserved."""
        r = self._req[rid]
        r.reserved, r.ahead = r.ahead, 0

    def has_ahead(self, rid: Hashable) -> bool:
        return rid in self._req and self._req[rid].ahead > 0

    def cancel(self, rid: Hashable) -> None:
        """Undo :meth:`reserve` calls that no step followed (and a step launched ahead that was not
        adopted): pages beyond the cached tokens go back."""
        r = self._req[rid]
        keep = -(-r.num_tokens // self.page_size)
        for g, table in enumerate(r.tables):
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    self.pools[g].free(p)
        r.reserved = 0
        r.ahead = 0

    def commit(self, rid: Hashable) -> None:
        """The step that wrote the reserved tokens is done: count them, and give back the
        pages that every future query's window has passed."""
        r = self._req[rid]
        r.num_tokens += r.reserved
        r.reserved = 0
        for g, spec in enumerate(self.groups):
            if spec.window > 0:
                first_needed = r.num_tokens - spec.window + 1     # oldest key the next query reads
                dead = max(0, first_needed) // self.page_size      # pages wholly below it
                table = r.tables[g]
                for i in range(min(dead, len(table))):
                    if table[i] >= 0:
                        self.pools[g].free(table[i])
                        table[i] = -1

    def truncate(self, rid: Hashable, num_tokens: int) -> None:
        """Forget the tokens beyond ``num_tokens`` (pages past the new end are given back).
        Counterpart of the reference's ``rollback`` (src/scheduler/paged_kv_cache.cpp:82-107)."""
        r = self._req[rid]
        if r.reserved or r.ahead:
            raise ValueError("CacheManager.truncate: a step is in flight")
        if not 0 <= num_tokens <= r.num_tokens:
            raise ValueError("CacheManager.truncate: cannot grow")
        keep = -(-num_tokens // self.page_size)
        # a window group has given back the pages its window had passed; going back further than that
        # would leave the next query attending over keys that are gone
        for g, spec in enumerate(self.groups):
            if spec.window > 0 and num_tokens < r.num_tokens:
                first_needed = max(0, num_tokens - spec.window + 1) // self.page_size
                if any(p < 0 for p in r.tables[g][first_needed:keep]):
                    raise ValueError(f"CacheManager.truncate: group {g} (window {spec.window}) has released pages "
                                     f"that a query at position {num_tokens} would read; a request can go back "
                                     f"only as far as its window has not moved on")
        for g, table in enumerate(r.tables):
            while len(table) > keep:
                p = table.pop()
                if p >= 0:
                    self.pools[g].free(p)
        r.num_tokens = num_tokens

    # ------------------------------------------------------------------ #
    # what a step uploads
    # ------------------------------------------------------------------ #
    def block_table(self, group: int, rid: Hashable) -> List[int]:
        return self._req[rid].tables[group]

    def slot_mapping(self, group: int, rid: Hashable, start: int, n: int) -> List[int]:
        """Flat cache slot (``page * page_size + offset``) of tokens ``start .. start+n-1``."""
        table = self._req[rid].tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + n):
            page = table[pos // ps]
            if page < 0:
                raise RuntimeError(f"CacheManager: position {pos} of request {rid!r} lies in a released page")
            out.append(page * ps + pos % ps)
        return out

    def max_pages_per_request(self) -> int:
        return max((len(t) for r in self._req.values() for t in r.tables), default=0)

    # ------------------------------------------------------------------ #
    # diagnostics
    # ------------------------------------------------------------------ #
    def free_pages(self) -> List[int]:
        return [p.num_free for p in self.pools]

    def used_pages(self) -> List[int]:
        return [p.num_used for p in self.pools]

    def check_invariants(self) -> None:
        """No page lost, none held twice: pages in tables + free pages = the pool."""
        for g, pool in enumerate(self.pools):
            held = [p for r in self._req.values() for p in r.tables[g] if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {g}: a page is held twice")
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise AssertionError(f"group {g}: a page is on the free list twice")
            if free & set(held):
                raise AssertionError(f"group {g}: a held page is on the free list")
            if len(held) + len(free) != pool.num_pages:
                raise AssertionError(f"group {g}: {pool.num_pages - len(held) - len(free)} pages lost")
        slots = [r.slot for r in self._req.values()]
        if len(slots) != len(set(slots)):
            raise AssertionError("a state slot is held twice")
        if len(slots) + self.slots.num_free != self.slots.num_slots:
            raise AssertionError("a state slot is lost")


def plan_groups(needs: Sequence[Tuple[Hashable, PagedCacheNeed]]) -> Tuple[List[CacheGroupSpec], Dict[Hashable, Tuple[int, int]]]:
    """Sort cache owners into groups.

    ``needs``: (owner, need) for everything that owns a paged cache.  Owners whose needs have the same
    ``group_key()`` (tensors, window, share of the budget) share a group.  Returns the groups and
    ``owner -> (group index, layer slot)``.
    """
    keyed: Dict[tuple, Tuple[PagedCacheNeed, List[Hashable]]] = {}
    for owner, need in needs:
        keyed.setdefault(need.group_key(), (need, []))[1].append(owner)
    groups, where = [], {}
    for gi, (need, owners) in enumerate(keyed.values()):
        groups.append(CacheGroupSpec(need, tuple(owners)))
        for li, owner in enumerate(owners):
            where[owner] = (gi, li)
    return groups, where
