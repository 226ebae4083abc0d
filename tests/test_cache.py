"""The cache's bookkeeping on the CPU: no slot or block lost, held twice or freed twice."""
import numpy as np
import pytest
import torch

from cretif_b200.cache import (BlockPool, CacheError, CacheFull, KVRequest, SequenceCache,
                               SlotSet, StateRequest)


def test_block_pool_strictness():
    pool = BlockPool(5)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.free_count == 2 and pool.held_count == 3
    with pytest.raises(CacheFull):
        pool.take(3)
    assert pool.free_count == 2                       # a refused request changes nothing
    pool.give_back([1])
    with pytest.raises(CacheError, match="not held"):
        pool.give_back([1])                           # freed twice
    with pytest.raises(CacheError, match="twice"):
        pool.give_back([0, 0])
    with pytest.raises(CacheError, match="does not belong"):
        pool.give_back([9])
    assert pool.take(1) == [1]                        # lowest free block first: reuse
    pool.check()


def test_slot_set_strictness():
    slots = SlotSet(2)
    s0, s1 = slots.take(), slots.take()
    assert (s0, s1) == (0, 1)
    with pytest.raises(CacheFull):
        slots.take()
    slots.give_back(0)
    with pytest.raises(CacheError, match="not in use"):
        slots.give_back(0)
    with pytest.raises(CacheError, match="does not exist"):
        slots.give_back(7)
    assert slots.take() == 0 and slots.live() == [0, 1]
    slots.check()


def make_cache(max_tokens=512, **kw):
    reqs = {0: KVRequest(2, 16), 1: KVRequest(2, 16), 2: KVRequest(1, 32, window=100),
            3: StateRequest((4, 3)), 4: None}
    return SequenceCache(reqs, max_tokens, torch.float32, "cpu", **kw)


def test_groups_have_storage_of_their_own():
    cache = make_cache()
    st = cache.stats()
    assert st["blocks"] == 8 and st["block_tokens"] == 64
    groups = {(g["num_kv_heads"], g["head_dim"], g["window"]): g["layers"] for g in st["groups"]}
    assert groups == {(2, 16, 0): 2, (1, 32, 100): 1}
    v0, v1, v2 = cache.kv_view(0), cache.kv_view(1), cache.kv_view(2)
    assert tuple(v0.k.shape) == (8, 2, 64, 16) and tuple(v2.k.shape) == (8, 1, 64, 32)
    assert v0.table is v1.table and v0.table is not v2.table
    assert v0.k.data_ptr() != v1.k.data_ptr()
    assert v2.window == 100 and cache.has_state(3) and not cache.has_kv(3)
    assert tuple(cache.state_view(3).shape) == (cache.max_slots, 4, 3)
    assert not cache.has_kv(4) and not cache.has_state(4)


def test_steps_lengths_and_reuse():
    cache = make_cache()
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.begin_step([(a, 70), (b, 5)])
    cache.end_step([(a, 70), (b, 5)])
    assert cache.length(a) == 70 and cache.length(b) == 5
    full = cache._kv_groups[0]
    assert full.pool.held_count == 3                  # 2 blocks for 70 tokens, 1 for 5
    rows = full.table.numpy()
    assert (rows[a, :2] >= 0).all() and rows[a, 2] == -1 and rows[b, 0] >= 0
    for _ in range(59):
        cache.begin_step([(b, 1)])
        cache.end_step([(b, 1)])
    assert cache.length(b) == 64 and full.pool.held_count == 3
    cache.begin_step([(b, 1)])                         # crosses into a second block
    cache.end_step([(b, 1)])
    assert full.pool.held_count == 4
    cache.check()
    held = set(full.table_host[a][full.table_host[a] >= 0].tolist())
    cache.free_slot(a)
    assert full.pool.held_count == 2
    with pytest.raises(CacheError):
        cache.free_slot(a)                             # freed twice
    with pytest.raises(CacheError):
        cache.length(a)
    c = cache.alloc_slot()
    assert c == a and cache.length(c) == 0             # the slot is handed out again, empty
    cache.begin_step([(c, 100)])
    cache.end_step([(c, 100)])
    assert held <= set(full.table_host[c][:2].tolist())    # and so are its blocks
    cache.check()


def test_step_checks_change_nothing_when_refused():
    cache = make_cache(max_tokens=256)                 # 4 blocks
    a, b = cache.alloc_slot(), cache.alloc_slot()
    with pytest.raises(CacheError, match="twice"):
        cache.begin_step([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="not in use"):
        cache.begin_step([(5, 1)])
    with pytest.raises(CacheError, match="at least one token"):
        cache.begin_step([(a, 0)])
    with pytest.raises(CacheFull, match="cache blocks"):
        cache.begin_step([(a, 130), (b, 130)])         # 3 + 3 blocks > 4
    assert all(g.pool.held_count == 0 for g in cache._kv_groups)
    with pytest.raises(CacheFull, match="longest sequence"):
        cache.begin_step([(a, 257)])
    cache.begin_step([(a, 130)])
    cache.end_step([(a, 130)])
    cache.check()


def test_window_group_gives_blocks_back():
    cache = make_cache(max_tokens=1024)
    s = cache.alloc_slot()
    win = cache._kv_groups[1]
    assert win.request.window == 100
    cache.begin_step([(s, 300)])
    assert win.pool.held_count == 5                    # the whole prompt is needed for its step
    cache.end_step([(s, 300)])
    # the next query sits at 300 and reads keys 201..300: blocks 0..2 are done with
    assert win.pool.held_count == 2 and int(win.first_block[s]) == 3
    assert (win.table_host[s, :3] == -1).all() and (win.table_host[s, 3:5] >= 0).all()
    assert cache._kv_groups[0].pool.held_count == 5    # the full group keeps everything
    cache.check()
    cache.free_slot(s)
    assert win.pool.held_count == 0
    cache.check()


def test_state_is_zeroed_when_a_slot_is_taken():
    cache = make_cache()
    s = cache.alloc_slot()
    cache.state_view(3)[s] += 5.0
    cache.free_slot(s)
    t = cache.alloc_slot()
    assert t == s and cache.state_view(3)[t].abs().sum().item() == 0.0


def test_reserve_is_all_or_nothing():
    cache = make_cache(max_tokens=256)
    a, b = cache.alloc_slot(), cache.alloc_slot()
    cache.reserve(a, 150)                              # 3 of 4 blocks
    full = cache._kv_groups[0]
    assert full.pool.held_count == 3
    with pytest.raises(CacheFull):
        cache.reserve(b, 100)
    assert full.pool.held_count == 3
    cache.begin_step([(a, 150)])                       # already mapped: takes nothing more
    assert full.pool.held_count == 3
    cache.end_step([(a, 150)])
    cache.check()


def test_many_random_batches_lose_nothing():
    rng = np.random.default_rng(0)
    cache = make_cache(max_tokens=2048, max_slots=6)
    live = {}
    for _ in range(300):
        if live and rng.random() < 0.3:
            s = int(rng.choice(list(live)))
            cache.free_slot(s)
            del live[s]
        elif len(live) < 6 and rng.random() < 0.5:
            s = cache.alloc_slot()
            n = int(rng.integers(1, 200))
            try:
                cache.begin_step([(s, n)])
                cache.end_step([(s, n)])
                live[s] = n
            except CacheFull:
                cache.free_slot(s)
        elif live:
            entries = [(s, 1) for s in live]
            try:
                cache.begin_step(entries)
                cache.end_step(entries)
                for s in live:
                    live[s] += 1
            except CacheFull:
                pass
        cache.check()
        for s, n in live.items():
            assert cache.length(s) == n
    for s in list(live):
        cache.free_slot(s)
    cache.check()
    assert all(g.pool.held_count == 0 for g in cache._kv_groups)
