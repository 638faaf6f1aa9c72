"""The cache manager on the host: no page lost, held twice or freed twice, under random orders
of requests; all-or-nothing reservation; pages of a window group given back as the window
passes; state slots; borrowed caches."""
import random

import pytest

from llmengine_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from llmengine_b200.parts.base import PagedKVSpec, StateSpec

FULL = (PagedKVSpec(2, 16, 0), None)
WIN = (PagedKVSpec(2, 16, 20), None)


def test_page_pool_is_lifo_and_catches_double_free():
    p = PagePool(4)
    assert p.alloc(2) == [0, 1]                      # page 0 first (src/runtime/cache/paged_kv_cache.cpp:48-52)
    p.free([0])
    assert p.alloc(1) == [0]                         # the page freed last comes back first
    with pytest.raises(OutOfPages):
        p.alloc(3)
    assert p.free_count == 2                         # a failed request changes nothing
    p.free([1])
    with pytest.raises(CacheError):
        p.free([1])
    with pytest.raises(CacheError):
        p.free([7])


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager([FULL, WIN, FULL], page_size=8, max_cached_tokens=64, max_requests=4, max_request_len=256)
    assert len(m.groups) == 2 and m.groups[0].runs == [0, 2] and m.groups[1].runs == [1]
    m.add_request("a")
    m.reserve("a", 40)
    m.advance("a", 40)
    m.add_request("b")
    free = [g.pool.free_count for g in m.groups]
    with pytest.raises(OutOfPages):
        m.reserve("b", 50)                           # fits the window group, not the full one
    assert [g.pool.free_count for g in m.groups] == free and m.requests["b"].blocks == [[], []]
    m.check_invariants()
    with pytest.raises(CacheError):
        m.reserve("b", 257)                          # beyond the length limit
    with pytest.raises(CacheError):
        m.add_request("a")


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([WIN], page_size=8, max_cached_tokens=64, max_requests=2, max_request_len=512)
    m.add_request("a")
    held = []
    for length in range(1, 200):
        m.reserve("a", length)
        m.advance("a", length)
        blocks = m.requests["a"].blocks[0]
        first_needed = max(0, length - 20 + 1) // 8   # the next query (position `length`) sees keys > length - 20
        assert all(p < 0 for p in blocks[:first_needed]) and all(p >= 0 for p in blocks[first_needed:])
        held.append(sum(p >= 0 for p in blocks))
        m.check_invariants()
    assert max(held) <= 4                             # never more than the window's pages, though 199 tokens went by
    assert (m.tables[0][m.requests["a"].slot][: len(blocks)] == blocks).all()
    m.free_request("a")
    assert m.groups[0].pool.free_count == 8


def test_slots_and_block_tables():
    m = CacheManager([FULL, (StateSpec((4,)), None)], page_size=4, max_cached_tokens=32, max_requests=2, max_request_len=32)
    a = m.add_request("a").slot
    b = m.add_request("b").slot
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages):
        m.add_request("c")
    m.reserve("a", 9)
    assert list(m.slot_mapping("a", 0, 3, 6)) == [m.requests["a"].blocks[0][p // 4] * 4 + p % 4 for p in range(3, 9)]
    with pytest.raises(Exception):
        m.slot_mapping("a", 0, 10, 4)                # positions without a page
    m.free_request("a")
    assert (m.tables[0][a] == -1).all()
    assert m.add_request("c").slot == a              # the slot is used again
    with pytest.raises(CacheError):
        m.free_request("a")


def test_borrowed_caches_need_the_same_layout():
    CacheManager([FULL, (PagedKVSpec(2, 16, 0), 0)], 8, 64, 2, 64)
    with pytest.raises(CacheError, match="differs"):
        CacheManager([FULL, (PagedKVSpec(4, 16, 0), 0)], 8, 64, 2, 64)


def test_admission_budget():
    m = CacheManager([FULL, WIN], page_size=8, max_cached_tokens=80, max_requests=4, max_request_len=512)
    assert m.groups[0].peak_pages(100, 16) == 13 and m.groups[1].peak_pages(100, 16) == 6   # ceil((19+16)/8)+1
    assert not m.fits_at_all(100, 16) and m.fits_at_all(80, 16)
    m.add_request("a")
    assert m.try_commit("a", 50, 16)                 # 7 of 10 pages
    m.add_request("b")
    assert not m.try_commit("b", 30, 16)             # 4 more would be 11
    assert m.try_commit("b", 24, 16)
    m.free_request("a")
    assert m.groups[0].committed == 3


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_lose_nothing(seed):
    rng = random.Random(seed)
    specs = [FULL, WIN, (StateSpec((3,)), None), (PagedKVSpec(2, 16, 0), 0)]
    m = CacheManager(specs, page_size=rng.choice([1, 4, 16]), max_cached_tokens=rng.choice([96, 256]),
                     max_requests=5, max_request_len=200)
    live, counter = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            counter += 1
            m.add_request(counter)
            live[counter] = 0
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            new = live[r] + rng.choice([1, 1, 1, 2, 7, 33])
            try:
                m.reserve(r, new)
                m.advance(r, new)
                live[r] = new
            except (OutOfPages, CacheError):
                pass                                  # refused: nothing may have changed
        elif live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
        m.check_invariants()
        for r, n in live.items():
            assert m.length(r) == n
            if n:
                m.slot_mapping(r, 0, n - 1, 1)        # the newest position always has a page in the full group
    for r in list(live):
        m.free_request(r)
    m.check_invariants()
    assert all(g.pool.free_count == g.pool.num_pages for g in m.groups) and m.free_slots == 5
