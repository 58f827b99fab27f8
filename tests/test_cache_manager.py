"""The cache manager and its allocator: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; groups move together."""

import random

import pytest
import torch

from atomserve_b200.cache import BlockAllocator, CacheManager, OutOfBlocksError, StateSlots, block_hash, blocks_for_tokens
from atomserve_b200.parts import KVCacheSpec, StateSpec

FULL = KVCacheSpec(2, 16, None)
WINDOWED = KVCacheSpec(2, 16, 24)


def test_blocks_for_tokens():
    assert [blocks_for_tokens(n, 16) for n in (0, 1, 16, 17, 32)] == [0, 1, 1, 2, 2]


def test_allocator_all_or_nothing_and_double_free():
    a = BlockAllocator(4)
    got = a.allocate(3)
    assert got == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfBlocksError):
        a.allocate(2)
    assert a.num_free == 1
    a.free(got)
    with pytest.raises(ValueError):
        a.free([1])
    with pytest.raises(ValueError):
        a.free([9])
    assert a.num_free == 4


def test_allocator_prefix_cache_rules():
    a = BlockAllocator(3)
    h1 = block_hash(b"", [1, 2])
    h2 = block_hash(h1, [3, 4])
    assert h1 != h2 and block_hash(b"", [3, 4]) != h2  # chained
    b = a.allocate(2)
    a.register(b[0], h1)
    a.register(b[1], h2)
    a.free(b)  # later page freed first, so it is evicted first
    assert a.num_free == 3 and a.lookup(h1) == b[0] and a.num_cached == 2
    a.acquire(b[0])  # revive
    assert a.num_free == 2 and a.refcount(b[0]) == 1
    a.acquire(b[0])
    assert a.refcount(b[0]) == 2
    taken = a.allocate(2)  # the untouched page first (oldest), then the cached later page
    assert taken == [2, b[1]] and a.lookup(h2) is None and a.lookup(h1) == b[0]
    other = taken[0]
    a.register(other, h1)  # first copy wins
    assert a.lookup(h1) == b[0]


def test_state_slots_zero_on_reuse():
    s = StateSlots(2)
    buf = s.register("x", (3,), torch.float32)
    a = s.take()
    buf[a] = 7.0
    s.give_back(a)
    with pytest.raises(ValueError):
        s.give_back(a)
    b, c = s.take(), s.take()
    assert {b, c} == {0, 1} and float(buf.abs().sum()) == 0
    with pytest.raises(RuntimeError):
        s.take()


def audit(cache: CacheManager, live: list) -> None:
    """Every page is either free or held by exactly the requests whose tables name it."""
    for gi, g in enumerate(cache.groups):
        held = {}
        for rc in live:
            for b in rc.block_tables[gi]:
                if b >= 0:
                    held[b] = held.get(b, 0) + 1
        for b in range(cache.num_blocks):
            assert g.allocator.refcount(b) == held.get(b, 0), f"group {gi} page {b}"
        assert g.allocator.num_free == cache.num_blocks - len(held)
    slots = [rc.state_slot for rc in live if rc.state_slot >= 0]
    assert len(slots) == len(set(slots)) and cache.state.num_free == cache.state.num_slots - len(slots)


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    reqs = [(FULL, []), (WINDOWED, []), (None, []), (WINDOWED, [StateSpec("s", (4,))]), (FULL, [])]
    cache = CacheManager(reqs, block_size=8, num_blocks=40, num_state_slots=6)
    assert len(cache.groups) == 2 and cache.groups[0].entries == [0, 4] and cache.groups[1].entries == [1, 3]
    assert not cache.supports_prefix_caching
    live = []  # (rc, position)
    for _ in range(600):
        action = rng.random()
        if action < 0.3 and len(live) < 6:
            rc = cache.new_request()
            assert cache.admit(rc)
            live.append([rc, 0])
        elif action < 0.85 and live:
            item = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 13, 40])
            before = [list(t) for t in item[0].block_tables]
            if cache.reserve(item[0], item[1], n):
                item[1] += n
                for t in item[0].block_tables:
                    assert len(t) == blocks_for_tokens(item[1], 8)
                # the windowed group holds only what its window and this step need
                w = item[0].block_tables[1]
                assert sum(b >= 0 for b in w) <= blocks_for_tokens(24 + n, 8) + 1
            else:  # all or nothing: only passed window pages may have gone
                for t0, t1 in zip(before, item[0].block_tables):
                    assert len(t0) == len(t1) and all(b == a or b == -1 for a, b in zip(t0, t1))
        elif live:
            item = live.pop(rng.randrange(len(live)))
            cache.free(item[0])
            assert item[0].block_tables == [[], []] and item[0].state_slot == -1
        audit(cache, [rc for rc, _ in live])
    for rc, _ in live:
        cache.free(rc)
    audit(cache, [])


def test_window_pages_come_back_and_full_pages_stay():
    cache = CacheManager([(FULL, []), (WINDOWED, [])], block_size=8, num_blocks=32, num_state_slots=2)
    rc = cache.new_request()
    cache.admit(rc)
    pos = 0
    for n in [20, 1, 1, 30, 1, 1, 1, 1, 1, 1, 1, 1, 1]:
        assert cache.reserve(rc, pos, n)
        pos += n
    full, win = rc.block_tables
    assert all(b >= 0 for b in full) and len(full) == blocks_for_tokens(pos, 8)
    first_needed = max(0, (pos - 1) - 24 + 1) // 8  # for the step that started at pos - 1
    assert all(b == -1 for b in win[:first_needed]) and all(b >= 0 for b in win[first_needed:])
    cache.free(rc)
    assert cache.num_free_blocks == 32


def test_reservation_is_all_groups_or_none():
    cache = CacheManager([(FULL, []), (KVCacheSpec(1, 8, None), [])], block_size=4, num_blocks=4, num_state_slots=2)
    a, b = cache.new_request(), cache.new_request()
    assert cache.reserve(a, 0, 12)  # 3 pages in each group
    cache.groups[1].allocator.allocate(1)  # somebody takes the other group's last page
    assert not cache.reserve(b, 0, 4)
    assert b.block_tables == [[], []] and cache.groups[0].allocator.num_free == 1


def test_prefix_cache_through_the_manager():
    cache = CacheManager([(FULL, []), (FULL, [])], block_size=4, num_blocks=8, num_state_slots=2)
    assert cache.supports_prefix_caching and len(cache.groups) == 1
    tokens = list(range(11))
    a = cache.new_request()
    assert cache.use_cached_prefix(a, tokens) == 0
    cache.reserve(a, 0, 11)
    cache.register_full_blocks(a, tokens, 10)  # two full pages computed
    assert len(a.block_hashes) == 2
    b = cache.new_request()
    assert cache.use_cached_prefix(b, tokens[:9] + [99]) == 8  # shares both full pages
    assert b.block_tables[0] == a.block_tables[0][:2]
    c = cache.new_request()
    assert cache.use_cached_prefix(c, tokens[:8]) == 4  # always leaves a token to compute
    cache.free(a)
    cache.free(b)
    cache.free(c)
    assert cache.num_free_blocks == 8 and cache.groups[0].allocator.num_cached == 2


def test_bytes_per_block():
    reqs = [(FULL, []), (WINDOWED, []), (None, [])]
    assert CacheManager.bytes_per_block(reqs, 16, torch.bfloat16) == 2 * (2 * 2 * 16) * 16 * 2
