"""Slots and pages: nothing lost, nothing held twice, nothing freed twice (no GPU)."""
import random

import numpy as np
import pytest
import torch

from llama_rs_metal_b200.cache import Cache, FreeList
from llama_rs_metal_b200.errors import CacheMemoryError, ContextError, InvalidError
from llama_rs_metal_b200.parts.base import KeyValueRequest, StateRequest

FULL = KeyValueRequest(kv_heads=2, head_dim=16)
WINDOW = KeyValueRequest(kv_heads=1, head_dim=32, window=100)
STATE = StateRequest(shape=(3, 4))


def make(requests=(FULL, FULL), max_tokens=1024, max_slots=4, max_sequence=512):
    return Cache(list(requests), torch.float32, torch.device("cpu"), max_tokens, max_slots, max_sequence)


def test_free_list_hands_out_lowest_first_and_rejects_double_free():
    f = FreeList(3, "slot")
    assert f.take(2) == [0, 1]
    f.give_back([0])
    assert f.take(1) == [0]                  # given back, used again at once
    with pytest.raises(CacheMemoryError):
        f.take(3)
    f.give_back([1])
    with pytest.raises(InvalidError, match="freed twice"):
        f.give_back([1])
    with pytest.raises(InvalidError):
        f.give_back([2])                      # never taken
    assert f.available + f.held == 3


def test_layers_with_equal_requests_share_a_group_with_storage_of_its_own():
    cache = make(requests=(FULL, WINDOW, FULL, STATE, None))
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1
    full = next(g for g in cache.kv_groups if g.request == FULL)
    assert full.entries == [0, 2]
    assert cache.view(0).k.data_ptr() != cache.view(2).k.data_ptr()
    assert cache.view(0).page_table.data_ptr() == cache.view(2).page_table.data_ptr()
    assert cache.view(1).page_table.data_ptr() != cache.view(0).page_table.data_ptr()
    assert cache.view(1).window == 100 and cache.view(0).window is None
    assert cache.view(3).state.shape == (4, 3, 4)
    assert cache.view(4) is None


def test_pages_follow_each_sequence_own_length():
    cache = make()
    a, b = cache.open_slot(), cache.open_slot()
    cache.grow([(a, 5), (b, 130)])
    cache.commit([(a, 5), (b, 130)])
    table = cache.kv_groups[0].table_host
    assert (table[a] >= 0).sum() == 1 and (table[b] >= 0).sum() == 3
    assert cache.length(a) == 5 and cache.length(b) == 130
    cache.grow([(a, 64), (b, 192)])          # still inside the pages they hold
    assert cache.held_pages() == [4]
    cache.grow([(a, 65), (b, 193)])
    assert cache.held_pages() == [6]
    held = np.concatenate([table[a][table[a] >= 0], table[b][table[b] >= 0]])
    assert len(set(held.tolist())) == 6      # no page held twice


def test_a_step_that_does_not_fit_changes_nothing():
    cache = make(max_tokens=256, max_sequence=200)
    a, b = cache.open_slot(), cache.open_slot()
    cache.grow([(a, 100)])
    before = cache.kv_groups[0].table_host.copy()
    with pytest.raises(CacheMemoryError):
        cache.grow([(a, 128), (b, 129)])     # 2 + 3 pages wanted, 4 exist
    with pytest.raises(ContextError):
        cache.grow([(a, 201)])
    assert np.array_equal(before, cache.kv_groups[0].table_host) and cache.held_pages() == [2]


def test_closed_slots_and_their_pages_are_used_again():
    cache = make(max_tokens=512, max_slots=2)
    a, b = cache.open_slot(), cache.open_slot()
    with pytest.raises(CacheMemoryError):
        cache.open_slot()
    cache.grow([(a, 256), (b, 256)])
    pages_a = set(cache.kv_groups[0].table_host[a][:4].tolist())
    cache.close_slot(a)
    with pytest.raises(InvalidError):
        cache.close_slot(a)                   # freed twice
    with pytest.raises(InvalidError):
        cache.length(a)
    c = cache.open_slot()
    assert c == a and cache.length(c) == 0
    cache.grow([(c, 200)])
    assert set(cache.kv_groups[0].table_host[c][:4].tolist()) == pages_a


def test_window_group_returns_pages_that_left_the_window():
    cache = make(requests=(WINDOW,), max_tokens=640, max_sequence=640)
    s = cache.open_slot()
    cache.grow([(s, 300)])                    # a prompt of 300: positions 200..299 stay visible
    row = cache.kv_groups[0].table_host[s]
    assert [i for i in range(10) if row[i] >= 0] == [3, 4]
    for n in range(301, 641):
        cache.grow([(s, n)])
        kept = [i for i in range(10) if row[i] >= 0]
        assert kept == list(range((n - 100) // 64, (n - 1) // 64 + 1))
        assert cache.held_pages() == [len(kept)]
    cache.close_slot(s)
    assert cache.held_pages() == [0]


def test_state_is_zeroed_when_a_slot_is_taken():
    cache = make(requests=(STATE,))
    s = cache.open_slot()
    cache.view(0).state[s] += 5.0
    cache.close_slot(s)
    assert cache.open_slot() == s
    assert torch.all(cache.view(0).state[s] == 0)


def test_random_walk_keeps_the_books():
    rng = random.Random(0)
    cache = make(requests=(FULL, WINDOW), max_tokens=2048, max_slots=6, max_sequence=700)
    live = {}
    for _ in range(2000):
        roll = rng.random()
        if roll < 0.2 and len(live) < 6:
            live[cache.open_slot()] = 0
        elif roll < 0.3 and live:
            slot = rng.choice(list(live))
            cache.close_slot(slot)
            del live[slot]
        elif live:
            slot = rng.choice(list(live))
            new = live[slot] + rng.choice([1, 1, 1, 37, 64])
            try:
                cache.grow([(slot, new)])
                cache.commit([(slot, new)])
                live[slot] = new
            except (CacheMemoryError, ContextError):
                pass
        for group in cache.kv_groups:
            held = group.table_host[group.table_host >= 0].tolist()
            assert len(held) == len(set(held)) == group.pool.held          # none twice, none lost
            assert group.pool.held + group.pool.available == group.pool.count
            rows_in_use = {int(r) for r in np.nonzero((group.table_host >= 0).any(axis=1))[0]}
            assert rows_in_use <= set(live)
        assert cache.slots.held == len(live)
        for slot, n in live.items():
            assert cache.length(slot) == n
    for slot in list(live):
        cache.close_slot(slot)
    assert cache.held_pages() == [0, 0] and cache.slots.held == 0


def test_destination_rows_follow_the_page_table_and_skip_dropped_positions():
    cache = make(requests=(FULL, WINDOW), max_tokens=1024, max_sequence=512)
    a, b = cache.open_slot(), cache.open_slot()
    cache.grow([(a, 70), (b, 300)])
    full, window = cache.destination_rows([a, b], [0, 0], [70, 300])
    assert len(full) == len(window) == 370
    tf = cache.kv_groups[0].table_host
    assert full[0] == tf[a][0] * 64 and full[69] == tf[a][1] * 64 + 5
    assert full[70 + 299] == tf[b][4] * 64 + 299 % 64
    assert (full >= 0).all()
    tw = cache.kv_groups[1].table_host
    assert (window[70:70 + 192] == -1).all()              # positions 0..191 of b lie in dropped pages
    assert window[70 + 192] == tw[b][3] * 64 and window[-1] == tw[b][4] * 64 + 299 % 64
    cache.commit([(a, 70), (b, 300)])
    cache.grow([(a, 71), (b, 301)])
    full, _ = cache.destination_rows([a, b], [70, 300], [1, 1])
    assert full.tolist() == [tf[a][1] * 64 + 6, tf[b][4] * 64 + 300 % 64]


def test_grow_by_one_does_what_grow_does_for_a_decode_step():
    a, b = make(requests=(FULL, FULL), max_tokens=1024), make(requests=(FULL, FULL), max_tokens=1024)
    for cache in (a, b):
        for n in (63, 64, 5):
            s = cache.open_slot()
            cache.grow([(s, n)])
            cache.commit([(s, n)])
    slots = np.array([2, 0, 1])
    for _ in range(70):
        before, rows = a.grow_by_one(slots)
        a.commit_lengths(slots, before + 1)
        growth = [(int(s), b.length(int(s)) + 1) for s in slots]
        b.grow(growth)
        want = b.destination_rows([int(s) for s in slots], [n - 1 for _, n in growth], [1, 1, 1])
        b.commit(growth)
        assert np.array_equal(a.kv_groups[0].table_host, b.kv_groups[0].table_host)
        assert [r.tolist() for r in rows] == [w.tolist() for w in want]
        assert a.lengths.tolist() == b.lengths.tolist()
    tight = make(requests=(FULL,), max_tokens=128, max_slots=2)
    s, t = tight.open_slot(), tight.open_slot()
    tight.grow([(s, 64), (t, 64)])
    tight.commit([(s, 64), (t, 64)])
    table = tight.kv_groups[0].table_host.copy()
    with pytest.raises(CacheMemoryError):
        tight.grow_by_one(np.array([s, t]))               # both need a new page, none is free
    assert np.array_equal(table, tight.kv_groups[0].table_host)
    assert make(requests=(WINDOW,)).grow_by_one(np.array([], dtype=np.int64)) is None
