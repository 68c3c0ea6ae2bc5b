"""The cache manager on the host: no page lost, held twice or freed twice, windows give pages
back, reservation is all-or-nothing, under random orders of requests (CPU)."""

import random

import pytest

from mini_infer_b200.cache import CacheManager, KVGroupSpec, OutOfPages, OutOfSlots, PagePool, SlotPool


def test_pool_order_and_reuse():
    p = PagePool(4)
    assert [p.alloc() for _ in range(4)] == [0, 1, 2, 3]        # page 0 first (src/core/allocator.cpp:85-89)
    with pytest.raises(OutOfPages):
        p.alloc()
    p.free(2)
    p.free(0)
    assert p.alloc() == 0 and p.alloc() == 2                      # LIFO
    assert p.high_water == 4 and p.num_free == 0


def test_pool_refuses_double_free_and_bad_ids():
    p = PagePool(2)
    a = p.alloc()
    p.free(a)
    with pytest.raises(ValueError, match="already free"):
        p.free(a)
    with pytest.raises(ValueError, match="outside"):
        p.free(7)
    b = p.alloc()
    p.ref(b)
    p.free(b)
    assert p.num_free == 1                                        # still referenced once
    p.free(b)
    assert p.num_free == 2
    with pytest.raises(OutOfPages):
        p.alloc_many(3)
    assert p.num_free == 2                                        # all or nothing


def test_slots():
    s = SlotPool(2)
    a, b = s.alloc(), s.alloc()
    assert (a, b) == (0, 1)
    with pytest.raises(OutOfSlots):
        s.alloc()
    s.free(a)
    with pytest.raises(ValueError):
        s.free(a)
    assert s.alloc() == a


def _mgr(pages=(8,), windows=(0,), page_size=4, slots=3):
    groups = [KVGroupSpec(2, 8, w, (i,)) for i, w in enumerate(windows)]
    return CacheManager(groups, list(pages), page_size, slots)


def test_growth_tables_and_slot_mapping():
    m = _mgr()
    m.add_request("a")
    assert m.reserve("a", 6) == 0
    assert m.block_table(0, "a") == [0, 1]
    assert m.slot_mapping(0, "a", 0, 6) == [0, 1, 2, 3, 4, 5]
    m.commit("a")
    m.add_request("b")
    assert m.reserve("b", 1) == 0 and m.block_table(0, "b") == [2]
    m.commit("b")
    assert m.reserve("a", 3) == 6                                 # crosses into a third page
    assert m.block_table(0, "a") == [0, 1, 3]
    assert m.slot_mapping(0, "a", 6, 3) == [6, 7, 12]
    m.commit("a")
    assert m.num_tokens("a") == 9
    m.check_invariants()
    m.release("a")
    assert m.free_pages() == [7]
    m.add_request("c")
    m.reserve("c", 4)
    assert m.block_table(0, "c") == [3]                           # the page freed last is used again first
    m.check_invariants()


def test_reserve_is_all_or_nothing_across_groups():
    m = _mgr(pages=(8, 2), windows=(0, 0))
    m.add_request("a")
    with pytest.raises(OutOfPages):
        m.reserve("a", 12)                                        # group 1 has 2 pages, 3 are needed
    assert m.free_pages() == [8, 2] and m.block_table(0, "a") == []
    assert not m.can_reserve("a", 12) and m.can_reserve("a", 8)
    m.reserve("a", 8)
    m.cancel("a")
    assert m.free_pages() == [8, 2] and m.num_tokens("a") == 0
    m.check_invariants()


def test_window_gives_pages_back():
    m = _mgr(pages=(16, 4), windows=(0, 6), page_size=4)
    m.add_request("a")
    held = []
    for step in range(40):
        m.reserve("a", 1)
        m.commit("a")
        held.append(m.used_pages()[1])
        m.check_invariants()
        n = m.num_tokens("a")
        table = m.block_table(1, "a")
        first_needed = max(0, n - 6 + 1)
        for i, p in enumerate(table):
            if (i + 1) * 4 <= first_needed:
                assert p == -1, (n, table)
            else:
                assert p >= 0, (n, table)
    assert max(held) <= 3                                         # window 6 with pages of 4: at most 3 pages
    assert m.used_pages()[0] == 10                                # the full-history group keeps everything
    with pytest.raises(RuntimeError, match="released page"):
        m.slot_mapping(1, "a", 0, 1)
    m.release("a")
    assert m.free_pages() == [16, 4]


def test_a_step_launched_ahead_holds_pages_without_changing_what_planning_sees():
    m = CacheManager([KVGroupSpec(1, 8, 0, (0,))], [3], 4, 2)
    m.add_request("a")
    assert m.reserve("a", 4) == 0
    m.commit("a")                                   # 4 tokens: one full page
    assert m.reserve_ahead("a", 1) == 4             # the next token needs a second page
    assert m.free_pages() == [1] and m.has_ahead("a")
    assert m.pages_needed("a", 1) == [0]            # planning the same token finds its page in place
    with pytest.raises(ValueError, match="unsettled"):
        m.reserve("a", 1)
    with pytest.raises(ValueError, match="unsettled"):
        m.reserve_ahead("a", 1)
    with pytest.raises(ValueError, match="in flight"):
        m.truncate("a", 2)
    m.check_invariants()
    m.adopt_ahead("a")
    m.commit("a")
    assert m.num_tokens("a") == 5 and not m.has_ahead("a") and m.free_pages() == [1]
    assert m.reserve_ahead("a", 1) == 5             # same page, nothing taken
    assert m.free_pages() == [1]
    m.cancel("a")                                   # dropped: nothing lost, nothing counted
    assert m.num_tokens("a") == 5 and not m.has_ahead("a") and m.free_pages() == [1]
    for _ in range(3):
        m.reserve("a", 1)
        m.commit("a")                               # 8 tokens: two full pages
    m.reserve_ahead("a", 1)
    assert m.free_pages() == [0]
    m.cancel("a")                                   # the page taken ahead goes back
    assert m.free_pages() == [1]
    m.reserve_ahead("a", 1)
    m.release("a")                                  # a request that ends gives back that page too
    assert m.free_pages() == [3]
    m.check_invariants()
    m.add_request("b")
    m.reserve("b", 12)
    m.commit("b")
    with pytest.raises(OutOfPages):
        m.reserve_ahead("b", 1)
    assert not m.has_ahead("b") and m.free_pages() == [0]
    m.check_invariants()


def test_errors():
    m = _mgr()
    m.add_request("a")
    with pytest.raises(ValueError, match="already live"):
        m.add_request("a")
    with pytest.raises(KeyError):
        m.reserve("zz", 1)
    with pytest.raises(ValueError, match="power of two"):
        CacheManager([KVGroupSpec(1, 8)], [4], 6, 1)
    m.reserve("a", 5)
    m.commit("a")
    m.truncate("a", 2)
    assert m.block_table(0, "a") == [0] and m.num_tokens("a") == 2
    with pytest.raises(ValueError, match="cannot grow"):
        m.truncate("a", 3)


def test_truncate_cannot_reach_into_pages_a_window_released():
    """A window group gives pages back as the window moves on; going back to a length whose window needs
    one of them is refused, going back inside what is still held is not."""
    m = CacheManager([KVGroupSpec(1, 8, 0), KVGroupSpec(1, 8, 6)], [16, 16], 4, 2)
    m.add_request("a")
    m.reserve("a", 20)
    m.commit("a")                                # window 6 at 20 tokens: keys from 15, pages 0..2 released
    assert m.block_table(1, "a")[:3] == [-1, -1, -1] and m.block_table(1, "a")[3] >= 0
    with pytest.raises(ValueError, match="released pages"):
        m.truncate("a", 14)                      # a query at 14 reads keys 9..14: page 2 is gone
    assert m.num_tokens("a") == 20
    m.truncate("a", 18)                          # reads keys 13..18 -> from page 3 on: fine
    assert m.num_tokens("a") == 18
    m.check_invariants()
    m.release("a")
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    windows = (0, rng.choice([5, 9, 17]))
    m = _mgr(pages=(24, 12), windows=windows, page_size=4, slots=4)
    live = {}
    next_id = 0
    for it in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{next_id}"
            next_id += 1
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 11])
            if m.can_reserve(rid, n):
                start = m.reserve(rid, n)
                assert start == live[rid]
                if rng.random() < 0.1:
                    m.cancel(rid)
                else:
                    sm = m.slot_mapping(0, rid, start, n)
                    assert len(set(sm)) == n
                    m.commit(rid)
                    live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            assert m.num_tokens(rid) == n
            assert len(m.block_table(0, rid)) == -(-n // 4)
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.free_pages() == [24, 12] and m.slots.num_free == 4
