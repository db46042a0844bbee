import random

import pytest
import torch

import citlali_b200 as cb
from citlali_b200.cache import KVRequirement, PageAllocator, SequenceCache, SlotAllocator, StateRequirement


def test_slots_no_loss_no_double_hold_no_double_free():
    a = SlotAllocator(4)
    got = [a.acquire() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and a.free_count == 0
    with pytest.raises(cb.CitlaliError, match="in use"):
        a.acquire()
    a.release(2)
    with pytest.raises(cb.CitlaliError, match="not held"):
        a.release(2)
    with pytest.raises(cb.CitlaliError, match="not held"):
        a.release(7)
    assert a.acquire() == 2                      # a slot given back is used again
    rng = random.Random(0)
    held = set(a.held)
    for _ in range(2000):
        if held and (rng.random() < 0.5 or len(held) == 4):
            s = rng.choice(sorted(held)); a.release(s); held.remove(s)
        else:
            s = a.acquire(); assert s not in held; held.add(s)
        assert set(a.held) == held and a.free_count + len(held) == 4


def test_pages_no_loss_no_double_free():
    p = PageAllocator(10)
    x = p.allocate(4); y = p.allocate(6)
    assert sorted(x + y) == list(range(10))
    with pytest.raises(cb.CitlaliError, match="cache is full"):
        p.allocate(1)
    p.free(x)
    with pytest.raises(cb.CitlaliError, match="not held"):
        p.free([x[0]])
    assert p.free_count == 4 and p.held_count == 6
    assert sorted(p.allocate(4)) == sorted(x)


def _cache(window=None, slots=3, capacity=64 * 8, seq=64 * 6):
    reqs = [KVRequirement(2, 16, None), KVRequirement(2, 16, None), KVRequirement(2, 16, window) if window else None,
            StateRequirement((4, 3))]
    return SequenceCache(reqs, slots, capacity, seq, torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    c = _cache(window=70)
    assert len(c.kv_groups) == 2 and len(c.state_groups) == 1
    full = c.kv_groups[0]
    assert full.steps == [0, 1] and tuple(full.keys.shape) == (2, 8, 2, 64, 16)
    assert c.kv_groups[1].steps == [2] and c.kv_groups[1].requirement.window == 70
    v0, v1 = c.view(0), c.view(1)
    assert v0.keys.data_ptr() != v1.keys.data_ptr() and v0.page_table.data_ptr() == v1.page_table.data_ptr()
    assert tuple(c.view(3).storage.shape) == (3, 4, 3)
    assert not c.has_view(7)


def test_growth_release_and_reuse():
    c = _cache()
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 65); c.commit(a, 65)
    c.reserve(b, 64); c.commit(b, 64)
    g = c.kv_groups[0]
    assert len(g.held[a]) == 2 and len(g.held[b]) == 1 and g.pages.held_count == 3
    assert set(g.held[a].values()).isdisjoint(g.held[b].values())
    assert g.table_host[a, 0].item() == g.held[a][0] and g.table[a, 1].item() == g.held[a][1]
    c.reserve(a, 128); c.commit(a, 128)
    assert len(g.held[a]) == 2                                   # no new page until position 128
    c.reserve(a, 129)
    assert len(g.held[a]) == 3
    with pytest.raises(cb.CitlaliError, match="exceeds the cache's limit"):
        c.reserve(a, 64 * 6 + 1)
    c.release(a)
    assert g.pages.held_count == 1 and c.slots.free_count == 2
    with pytest.raises(cb.CitlaliError, match="not held"):
        c.release(a)
    with pytest.raises(cb.CitlaliError, match="not held"):
        c.reserve(a, 3)
    again = c.acquire()
    assert again == a and c.length(again) == 0


def test_full_pool_is_an_error_and_takes_nothing():
    c = _cache(capacity=64 * 3)
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 128)
    with pytest.raises(cb.CitlaliError, match="cache is full"):
        c.reserve(b, 129)
    assert c.kv_groups[0].pages.held_count == 2 and c.kv_groups[0].held[b] == {}
    c.reserve(b, 64)
    assert c.pages_held() == 3


def test_state_is_zeroed_on_acquire():
    c = _cache()
    s = c.acquire()
    c.view(3).storage[s] += 5.0
    c.release(s)
    assert c.acquire() == s and float(c.view(3).storage[s].abs().sum()) == 0.0


def test_window_group_gives_pages_back():
    c = _cache(window=70, capacity=64 * 8, seq=64 * 8)
    s = c.acquire()
    full, win = c.kv_groups
    c.reserve(s, 300); c.commit(s, 300)          # a prompt: every page while the step runs, then the window's
    assert len(full.held[s]) == 5
    assert sorted(win.held[s]) == [3, 4]         # first visible position 231 -> page 3
    for n in range(301, 400):
        c.reserve(s, n); c.commit(s, n)
    assert sorted(win.held[s]) == [5, 6] and len(full.held[s]) == 7
    c.release(s)
    assert win.pages.held_count == 0 and full.pages.held_count == 0


def test_random_traffic_keeps_the_books():
    rng = random.Random(1)
    c = _cache(window=100, slots=4, capacity=64 * 12, seq=64 * 6)
    live = {}
    for _ in range(600):
        if live and (rng.random() < 0.3 or len(live) == 4):
            s = rng.choice(sorted(live)); c.release(s); del live[s]
        elif len(live) < 4 and rng.random() < 0.5:
            live[c.acquire()] = 0
        elif live:
            s = rng.choice(sorted(live))
            n = min(live[s] + rng.choice([1, 1, 1, 40, 90]), 64 * 6)
            try:
                c.reserve(s, n)
            except cb.CitlaliError:
                continue
            c.commit(s, n); live[s] = n
        for g in c.kv_groups:
            pages = [p for s in g.held for p in g.held[s].values()]
            assert len(pages) == len(set(pages)) == g.pages.held_count      # nothing held twice or lost
            assert g.pages.held_count + g.pages.free_count == g.pages.num_pages
            assert set(g.held) == set(live)
        for s, n in live.items():
            assert c.length(s) == n
            assert set(range((n + 63) // 64)) == set(c.kv_groups[0].held[s])


def test_rewind_keeps_pages_and_lowers_the_length():
    import torch
    from citlali_b200.cache import KVRequirement, SequenceCache
    c = SequenceCache([KVRequirement(2, 16)], 2, 64 * 8, 64 * 4, torch.float32, "cpu")
    s = c.acquire()
    c.reserve(s, 200); c.commit(s, 200)
    held = c.pages_held()
    c.rewind(s, 70)
    assert c.length(s) == 70 and c.pages_held() == held
    c.reserve(s, 200); c.commit(s, 200)
    assert c.pages_held() == held
    with pytest.raises(cb.CitlaliError, match="cannot be rewound"):
        c.rewind(s, 201)
    w = SequenceCache([KVRequirement(2, 16, window=32)], 1, 64 * 8, 64 * 4, torch.float32, "cpu")
    t = w.acquire()
    w.reserve(t, 100); w.commit(t, 100)
    with pytest.raises(cb.CitlaliError, match="windowed"):
        w.rewind(t, 50)
