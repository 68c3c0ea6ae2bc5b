"""What a part asks the cache for: pages per token, or a fixed-size state per request.

A part's ``cache_need()`` returns one of these (or None).  A *paged* need says which tensors it keeps per
page and how long a token's entry must stay (``window``); the engine allocates exactly those tensors for
every group of layers with the same need, and the cache manager hands out the pages.  The built-in
attention keeps a key and a value row per token (:class:`KVNeed`); a part that keeps something else per
token (one latent row, say) subclasses :class:`PagedCacheNeed` and describes its own tensors, and nothing
in the engine has to change for it.

The reference has one kind of cache, keys and values of one geometry for all layers
(src/scheduler/paged_kv_cache.h:46-53, src/core/allocator.h:60-78).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

# (name, shape of one page, dtype or None for the model's activation dtype)
PageTensor = Tuple[str, Tuple[int, ...], Optional[object]]


class PagedCacheNeed:
    """Per-token entries kept in pages.

    ``window = 0`` keeps every token's entry, ``window = W`` only the last ``W`` (older pages are given
    back).  ``pages_fraction`` is the share of the engine's page budget that the group of this need gets
    (1.0 = as many pages as a full-history group)."""

    window: int = 0
    pages_fraction: float = 1.0

    def tensors(self, page_size: int) -> List[PageTensor]:
        """The tensors of one layer, per page of ``page_size`` tokens."""
        raise NotImplementedError

    def geometry(self) -> tuple:
        """What two needs must share for one to read the other's cache."""
        return tuple((n, tuple(s), str(d)) for n, s, d in self.tensors(1))

    def group_key(self) -> tuple:
        """Layers whose needs have the same key share a page pool and a block table per request."""
        return (type(self).__name__, self.geometry(), int(self.window), float(self.pages_fraction))

    def bytes_per_page(self, page_size: int, act_itemsize: int) -> int:
        total = 0
        for _, shape, dtype in self.tensors(page_size):
            n = 1
            for s in shape:
                n *= int(s)
            total += n * (act_itemsize if dtype is None else dtype.itemsize)
        return total


@dataclass(frozen=True)
class KVNeed(PagedCacheNeed):
    """Keys and values per token: ``k`` and ``v`` pages of ``[num_kv_heads, page_size, head_dim]``."""

    num_kv_heads: int
    head_dim: int
    window: int = 0
    pages_fraction: float = 1.0

    def tensors(self, page_size: int) -> List[PageTensor]:
        shape = (self.num_kv_heads, page_size, self.head_dim)
        return [("k", shape, None), ("v", shape, None)]


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request (``shape`` per slot), zeroed when a request starts."""

    shape: Tuple[int, ...]
    dtype: Optional[object] = None      # None: float32
