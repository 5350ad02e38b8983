"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from friday_inference_engine_b200.cache import PAGE, Cache, CacheError, CacheFull, FreeList
from friday_inference_engine_b200.parts.base import KVRequest, StateRequest


def test_free_list_never_loses_or_doubles():
    fl = FreeList(5, "slot")
    held = [fl.take() for _ in range(5)]
    assert sorted(held) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        fl.take()
    fl.give(3)
    with pytest.raises(CacheError):
        fl.give(3)                       # freed twice
    with pytest.raises(CacheError):
        fl.give(7)                       # never taken
    assert fl.take() == 3                # used again
    rnd = random.Random(0)
    held = set(held)
    for _ in range(2000):
        if held and (rnd.random() < 0.5 or fl.free_count == 0):
            s = rnd.choice(sorted(held))
            fl.give(s)
            held.remove(s)
        else:
            s = fl.take()
            assert s not in held         # never handed out twice
            held.add(s)
        assert fl.free_count + fl.held_count == 5 and fl.held_count == len(held)


def _cache(window=None, max_tokens=8 * PAGE, max_seq=4 * PAGE, slots=4, two_groups=False):
    reqs = {0: KVRequest(2, 8, window), 1: KVRequest(2, 8, window)}
    if two_groups:
        reqs[2] = KVRequest(2, 8, 70)
    reqs[9] = StateRequest((3,), torch.float32)
    return Cache(reqs, max_tokens, max_seq, torch.float32, "cpu", max_slots=slots)


def test_groups_by_need_and_shapes():
    c = _cache(two_groups=True)
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.entries == [0, 1] and win.entries == [2] and win.window == 70
    assert tuple(full.k_pool.shape) == (2, 8, PAGE, 2, 8)
    assert c.group_of[1] is full and c.group_of[2] is win
    assert tuple(c.states[9].shape) == (4, 3)


def test_pages_follow_lengths_and_come_back():
    c = _cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([a, b], [70, 1])
    c.commit([a, b], [70, 1])
    g = c.groups[0]
    assert len(g.held_pages(a)) == 2 and len(g.held_pages(b)) == 1 and c.lens[a] == 70
    assert set(g.held_pages(a)).isdisjoint(g.held_pages(b))
    for _ in range(58):
        c.reserve([a], [1])
        c.commit([a], [1])
    assert c.lens[a] == 128 and len(g.held_pages(a)) == 2
    c.reserve([a], [1])                                   # token 129 opens the third page
    c.commit([a], [1])
    assert len(g.held_pages(a)) == 3
    c.free_slot(a)
    assert g.pages.held_count == 1 and (g.table[a] == -1).all()
    with pytest.raises(CacheError):
        c.free_slot(a)
    c.free_slot(b)
    assert g.pages.held_count == 0 and c.slots.held_count == 0


def test_full_cache_refuses_and_holds_nothing_new():
    c = _cache(max_tokens=3 * PAGE)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([a], [2 * PAGE])
    c.commit([a], [2 * PAGE])
    before = c.groups[0].pages.held_count
    with pytest.raises(CacheFull):
        c.reserve([a, b], [1, PAGE + 1])                  # needs 1 + 2 pages, 1 is free
    assert c.groups[0].pages.held_count == before and c.groups[0].held_pages(b) == []
    with pytest.raises(CacheError):
        c.reserve([a], [3 * PAGE])                        # beyond one sequence's limit (4 pages of 64)


def test_window_group_gives_pages_back_early():
    c = _cache(window=70, max_tokens=64 * PAGE, max_seq=64 * PAGE)
    s = c.alloc_slot()
    g = c.groups[0]
    c.reserve([s], [300])
    assert len(g.held_pages(s)) == 5                      # held during the pass
    c.commit([s], [300])
    # a query at position >= 300 reaches back to 231: pages 0..2 (positions < 192) are gone
    assert [int(p) >= 0 for p in g.table[s][:6]] == [False, False, False, True, True, False]
    for _ in range(500):
        c.reserve([s], [1])
        c.commit([s], [1])
        assert len(g.held_pages(s)) <= 3
    c.free_slot(s)
    assert g.pages.held_count == 0


def test_state_is_zero_for_a_new_sequence():
    c = _cache()
    s = c.alloc_slot()
    c.states[9][s] += 5.0
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and float(c.states[9][s2].abs().sum()) == 0.0


def test_random_traffic_keeps_the_books():
    rnd = random.Random(1)
    c = _cache(max_tokens=16 * PAGE, max_seq=6 * PAGE, slots=6, two_groups=True)
    live = {}
    for _ in range(600):
        r = rnd.random()
        if live and r < 0.25:
            s = rnd.choice(sorted(live))
            c.free_slot(s)
            del live[s]
        elif r < 0.5 and c.slots.free_count:
            live[c.alloc_slot()] = 0
        elif live:
            s = rnd.choice(sorted(live))
            q = rnd.choice([1, 1, 1, 17, 90])
            if live[s] + q > 6 * PAGE:
                continue
            try:
                c.reserve([s], [q])
            except CacheFull:
                continue
            c.commit([s], [q])
            live[s] += q
        for g in c.groups:
            held = [p for s in range(6) for p in g.held_pages(s)]
            assert len(held) == len(set(held)) == g.pages.held_count          # no page held twice or lost
            assert g.pages.held_count + g.pages.free_count == g.n_pages
            for s in range(6):
                if s not in live:
                    assert g.held_pages(s) == []
        assert all(c.lens[s] == n for s, n in live.items())
