"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (no GPU).  The book is the
library's own Cache (cache/cache.cpp) built without device memory."""
import random

import pytest

from friday_inference_engine_b200.cache import PAGE, CacheBook, CacheError, CacheFull, kv_request, state_request


def test_slots_never_lost_or_doubled():
    c = CacheBook({0: kv_request(1, 8)}, 5 * PAGE, PAGE, max_slots=5)
    held = [c.alloc_slot() for _ in range(5)]
    assert sorted(held) == [0, 1, 2, 3, 4]
    with pytest.raises(CacheFull):
        c.alloc_slot()
    c.free_slot(3)
    with pytest.raises(CacheError):
        c.free_slot(3)                   # freed twice
    with pytest.raises(CacheError):
        c.free_slot(7)                   # never taken
    assert c.alloc_slot() == 3           # used again
    rnd = random.Random(0)
    held = set(held)
    for _ in range(2000):
        info = None
        if held and (rnd.random() < 0.5 or len(held) == 5):
            s = rnd.choice(sorted(held))
            c.free_slot(s)
            held.remove(s)
        else:
            s = c.alloc_slot()
            assert s not in held         # never handed out twice
            held.add(s)
        if rnd.random() < 0.05:
            info = c.info()
            assert info["slots_free"] + info["slots_held"] == 5 and info["slots_held"] == len(held)
            assert [i for i, h in enumerate(info["held"]) if h] == sorted(held)


def _cache(window=None, max_tokens=8 * PAGE, max_seq=4 * PAGE, slots=4, two_groups=False):
    reqs = {0: kv_request(2, 8, window), 1: kv_request(2, 8, window)}
    if two_groups:
        reqs[2] = kv_request(2, 8, 70)
    reqs[9] = state_request((3,))
    return CacheBook(reqs, max_tokens, max_seq, max_slots=slots)


def test_groups_by_need_and_shapes():
    info = _cache(two_groups=True).info()
    assert len(info["groups"]) == 2
    full, win = info["groups"]
    assert full["entries"] == [0, 1] and win["entries"] == [2] and win["window"] == 70 and full["window"] == 0
    assert full["pool_shape"] == [2, 8, PAGE, 2, 8]
    assert info["group_of"] == {"0": 0, "1": 0, "2": 1}
    assert info["states"] == {"9": [4, 3]}


def test_pages_follow_lengths_and_come_back():
    c = _cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([a, b], [70, 1])
    c.commit([a, b], [70, 1])
    assert len(c.held_pages(0, a)) == 2 and len(c.held_pages(0, b)) == 1 and c.info()["lens"][a] == 70
    assert set(c.held_pages(0, a)).isdisjoint(c.held_pages(0, b))
    for _ in range(58):
        c.reserve([a], [1])
        c.commit([a], [1])
    assert c.info()["lens"][a] == 128 and len(c.held_pages(0, a)) == 2
    c.reserve([a], [1])                                   # token 129 opens the third page
    c.commit([a], [1])
    assert len(c.held_pages(0, a)) == 3
    c.free_slot(a)
    g = c.info()["groups"][0]
    assert g["pages_held"] == 1 and all(p == -1 for p in g["table"][a])
    with pytest.raises(CacheError):
        c.free_slot(a)
    c.free_slot(b)
    info = c.info()
    assert info["groups"][0]["pages_held"] == 0 and info["slots_held"] == 0


def test_full_cache_refuses_and_holds_nothing_new():
    c = _cache(max_tokens=3 * PAGE)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([a], [2 * PAGE])
    c.commit([a], [2 * PAGE])
    before = c.info()["groups"][0]["pages_held"]
    with pytest.raises(CacheFull):
        c.reserve([a, b], [1, PAGE + 1])                  # needs 1 + 2 pages, 1 is free
    assert c.info()["groups"][0]["pages_held"] == before and c.held_pages(0, b) == []
    with pytest.raises(CacheError):
        c.reserve([a], [3 * PAGE])                        # beyond one sequence's limit (4 pages of 64; 3 here)


def test_window_group_gives_pages_back_early():
    c = _cache(window=70, max_tokens=64 * PAGE, max_seq=64 * PAGE)
    s = c.alloc_slot()
    c.reserve([s], [300])
    assert len(c.held_pages(0, s)) == 5                   # held during the pass
    c.commit([s], [300])
    # a query at position >= 300 reaches back to 231: pages 0..2 (positions < 192) are gone
    assert [p >= 0 for p in c.info()["groups"][0]["table"][s][:6]] == [False, False, False, True, True, False]
    for i in range(500):
        c.reserve([s], [1])
        c.commit([s], [1])
        if i % 25 == 0:
            assert len(c.held_pages(0, s)) <= 3
    c.free_slot(s)
    assert c.info()["groups"][0]["pages_held"] == 0


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
        elif r < 0.5 and len(live) < 6:
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
        info = c.info()
        for g in info["groups"]:
            held = [p for s in range(6) for p in g["table"][s] if p >= 0]
            assert len(held) == len(set(held)) == g["pages_held"]            # no page held twice or lost
            assert g["pages_held"] + g["pages_free"] == g["n_pages"]
            for s in range(6):
                if s not in live:
                    assert all(p < 0 for p in g["table"][s])
        assert all(info["lens"][s] == n for s, n in live.items())
