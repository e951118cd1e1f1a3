"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (CPU)."""
import random

import pytest

from moe_b200.cache import PAGE_TOKENS, CacheError, CacheLedger, pages_for
from pools import PagePool, SlotPool


def test_slots_are_unique_and_reused():
    p = SlotPool(4)
    got = [p.acquire() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and p.num_free == 0
    with pytest.raises(CacheError):
        p.acquire()
    p.release(got[1])
    with pytest.raises(CacheError):
        p.release(got[1])                 # freed twice
    with pytest.raises(CacheError):
        p.release(17)                     # never existed
    assert p.acquire() == got[1]          # given back, used again
    assert p.num_held == 4


def test_pages_never_include_the_scratch_page():
    p = PagePool(5)
    got = p.alloc(4)
    assert sorted(got) == [1, 2, 3, 4]
    with pytest.raises(CacheError):
        p.alloc(1)
    p.free(got[:2])
    with pytest.raises(CacheError):
        p.free(got[:1])                   # freed twice
    with pytest.raises(CacheError):
        p.free([0])                       # the scratch page is nobody's
    assert p.num_free == 2


def test_pages_for_rounds_up_and_rings_are_bounded():
    assert [pages_for(n) for n in (0, 1, 64, 65, 128, 129)] == [0, 1, 1, 2, 2, 3]
    assert pages_for(1000, ring_pages=2) == 2 and pages_for(10, ring_pages=2) == 1


def test_ledger_extend_release_and_budget():
    led = CacheLedger(num_slots=3, group_pages=[5, 3], group_ring_pages=[0, 1])   # 4 + 2 usable pages
    a, b = led.acquire(), led.acquire()
    up = led.extend(a, 70)                       # 2 pages in the full group, 1 in the ring
    assert sorted((g, s, i) for g, s, i, _ in up) == [(0, a, 0), (0, a, 1), (1, a, 0)]
    assert led.extend(a, 128) == []              # still inside its pages
    led.extend(b, 64)
    assert led.tokens_held() == 128 + 64
    with pytest.raises(CacheError):
        led.extend(b, 64 * 3)                    # would need 2 more full pages, 1 free
    assert led.length[b] == 64                   # a refused extend changes nothing
    assert led.groups[0].pool.num_free == 1
    led.release(a)
    assert led.groups[0].pool.num_free == 3 and led.groups[1].pool.num_free == 1
    with pytest.raises(CacheError):
        led.release(a)                           # released twice
    led.extend(b, 64 * 3)                        # now it fits
    led.release(b)
    assert led.groups[0].pool.num_free == 4 and led.groups[1].pool.num_free == 2 and led.slots.num_free == 3


def test_truncate_rules():
    led = CacheLedger(2, [9, 3], [0, 2])
    s = led.acquire()
    led.extend(s, 100)
    led.truncate(s, 40)
    assert led.length[s] == 40
    with pytest.raises(CacheError):
        led.truncate(s, 50)
    led.extend(s, 300)                           # ring of 128 tokens has wrapped: it holds positions 172..299
    with pytest.raises(CacheError):
        led.truncate(s, 250)                     # the window is not told: refused
    with pytest.raises(CacheError):
        led.truncate(s, 250, [0, 100])           # position 250 looks back to 151, which is gone
    assert led.length[s] == 300
    led.truncate(s, 271, [0, 100])               # position 271 looks back to 172: just still there
    assert led.length[s] == 271
    led.truncate(s, 271, [0, 100])               # to the same length: nothing to do, always allowed
    led.extend(s, 280)
    assert led.length[s] == 280


def test_random_walk_keeps_every_invariant():
    rng = random.Random(7)
    led = CacheLedger(8, [40, 17], [0, 2])
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and led.slots.num_free:
            live[led.acquire()] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            led.release(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = live[s] + rng.randint(1, 150)
            try:
                led.extend(s, n)
                live[s] = n
            except CacheError:
                pass
        # invariants: lengths as told; pages held exactly once; counts add up
        assert {s: led.length[s] for s in live} == live
        for g in led.groups:
            held = [p for s in live for p in g.pages[s]]
            assert len(held) == len(set(held)) and 0 not in held
            assert len(held) + g.pool.num_free == g.pool.num_pages - 1
            for s in live:
                assert len(g.pages[s]) == pages_for(live[s], g.ring_pages)
        assert led.slots.num_held == len(live)
        assert led.tokens_held() == sum(-(-n // PAGE_TOKENS) * PAGE_TOKENS for n in live.values())
    for s in list(live):
        led.release(s)
    assert all(g.pool.num_free == g.pool.num_pages - 1 for g in led.groups) and led.slots.num_free == 8


def test_check_says_what_reserve_would_and_changes_nothing():
    led = CacheLedger(2, [5, 5], [0, 2])
    a, b = led.acquire(), led.acquire()
    led.check([a, b], [100, 100], [4, 0])                    # 2 + 2 pages of the 4 free in either group
    with pytest.raises(CacheError):
        led.check([a, b], [100, 200], [4, 0])                # 2 + 4 pages: more than the 4 free
    with pytest.raises(CacheError):
        led.check([a], [300], [4, 0])                        # 5 pages: more than the page table holds
    with pytest.raises(ValueError):
        led.check([a, a], [1, 1], [4, 0])
    assert led.length[a] == 0 and led.length[b] == 0 and led.groups[0].pool.num_free == 4
    starts, upd = led.reserve([a, b], [100, 100], [4, 0])
    assert starts == [0, 0] and led.groups[0].pool.num_free == 0
