"""The sequence cache's bookkeeping on a CPU device: no slot or page is lost, held twice
or freed twice; groups and state; windows give pages back (no GPU)."""
import random

import pytest
import torch

from cpp_minilamma_b200.cache import PAGE, CacheError, CacheFull, PagePool, SequenceCache
from cpp_minilamma_b200.parts.base import CacheNeed, KVNeed, StateNeed


def make(max_tokens=PAGE * 8, n_slots=4, max_positions=1024, needs=None):
    needs = needs or [(0, None, CacheNeed(kv=KVNeed(2, 16))), (1, None, CacheNeed(kv=KVNeed(2, 16)))]
    return SequenceCache(needs, max_tokens, n_slots, max_positions, torch.float32, "cpu")


def test_page_pool():
    pool = PagePool(5)
    a = pool.take(3)
    assert len(set(a)) == 3 and pool.n_free == 2
    with pytest.raises(CacheFull):
        pool.take(3)
    assert pool.n_free == 2  # nothing changed
    pool.give_back(a[:1])
    with pytest.raises(CacheError, match="twice"):
        pool.give_back(a[:1])
    with pytest.raises(CacheError, match="does not exist"):
        pool.give_back([7])
    pool.check()


def test_slots_are_reused_and_never_held_twice():
    cache = make()
    first = cache.acquire(4)
    assert sorted(first) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        cache.acquire(1)
    cache.release(first[1])
    with pytest.raises(CacheError, match="not live"):
        cache.release(first[1])
    with pytest.raises(CacheError, match="does not exist"):
        cache.release(9)
    again = cache.acquire(1)
    assert again == [first[1]]
    cache.check()


def test_growth_is_all_or_nothing():
    cache = make(max_tokens=PAGE * 4)
    a, b = cache.acquire(2)
    cache.reserve([(a, PAGE + 1), (b, 1)])        # 2 + 1 pages
    assert cache.seq_len[a] == PAGE + 1 and cache.free_pages() == 1
    with pytest.raises(CacheFull):
        cache.reserve([(a, PAGE), (b, PAGE)])     # needs 1 + 1 pages, 1 free
    assert cache.seq_len[a] == PAGE + 1 and cache.seq_len[b] == 1 and cache.free_pages() == 1
    cache.reserve([(b, PAGE - 1)])                # fills b's page exactly: no new page
    assert cache.free_pages() == 1
    with pytest.raises(CacheError, match="twice in one step"):
        cache.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError, match="at least one token"):
        cache.reserve([(a, 0)])
    cache.check()
    cache.release(a)
    assert cache.free_pages() == 3
    cache.check()


def test_position_limit():
    cache = make(max_positions=100)
    s, = cache.acquire(1)
    cache.reserve([(s, 100)])
    with pytest.raises(CacheFull, match="positions"):
        cache.reserve([(s, 1)])


def test_block_tables_and_views():
    cache = make()
    a, b = cache.acquire(2)
    cache.reserve([(a, 70), (b, 3)])
    cache.flush()
    group = cache.groups[0]
    assert len(cache.groups) == 1 and group.entries == [0, 1]           # equal needs share a group
    assert group.k.shape == (2, 8 + 1, 2, PAGE, 16)                      # 8 pages to hand out and the padding slot's
    table = group.table_dev
    assert table.shape[0] == cache.n_slots + 1 and cache.pad_slot == cache.n_slots
    assert int(table[cache.pad_slot, 0]) == 8 and int(table[cache.pad_slot, 1]) == -1
    with pytest.raises(CacheError):
        cache.reserve([(cache.pad_slot, 1)])                            # never handed out, never grown
    pages_a = [int(p) for p in table[a, :2]]
    assert pages_a == group.pages[a] and int(table[a, 2]) == -1
    assert not set(pages_a) & {int(table[b, 0])}
    v0, v1 = cache.view(0), cache.view(1)
    assert v0.k.data_ptr() != v1.k.data_ptr() and v0.block_table is v1.block_table
    cache.release(a)
    # a slot that is not live has an empty row on the host; nobody reads its row on the device, which is
    # replaced when the slot is handed out again and grows
    assert int(group.table_host[a, 0]) == -1 and cache.take_table_updates() == []
    again, = cache.acquire(1)
    assert again == a
    cache.reserve([(a, 5)])
    (g, rows), = cache.take_table_updates()
    assert g is group and rows.shape == (1, 1 + group.max_blocks)
    assert int(rows[0, 0]) == a and int(rows[0, 1]) == group.pages[a][0] and int(rows[0, 2]) == -1
    assert cache.take_table_updates() == []


def test_groups_with_different_needs_have_storage_of_their_own():
    needs = [(0, None, CacheNeed(kv=KVNeed(2, 16))),
             (1, None, CacheNeed(kv=KVNeed(1, 32, window=100))),
             (2, 0, CacheNeed(kv=KVNeed(2, 16))),                       # reads entry 0's cache
             (3, None, CacheNeed(state=StateNeed((("sum", (8,)), ("count", (1,))))))]
    cache = make(max_tokens=PAGE * 16, needs=needs)
    assert len(cache.groups) == 2
    full, window = cache.groups
    assert full.entries == [0] and window.entries == [1]
    assert cache.view(2).k.data_ptr() == cache.view(0).k.data_ptr() and not cache.view(2).owns_kv
    assert cache.view(3).k is None and cache.view(3).state["sum"].shape == (cache.n_slots + 1, 8)  # and the padding slot
    s, = cache.acquire(1)
    cache.reserve([(s, 3 * PAGE)])
    assert window.pool.n_free == full.pool.n_free == 13
    cache.reserve([(s, 1)])     # query at 192 reads keys > 92: page 0 (0..63) is out of reach
    assert window.pool.n_free == 13 and full.pool.n_free == 12
    assert window.pages[s][0] is None and window.table_host[s, 0] == -1
    for _ in range(PAGE * 4):
        cache.reserve([(s, 1)])
    assert sum(p is not None for p in window.pages[s]) <= 3             # the window keeps about 100 tokens
    cache.check()
    cache.release(s)
    assert window.pool.n_free == full.pool.n_free == 16
    cache.check()


def test_state_is_zeroed_when_a_slot_is_handed_out():
    needs = [(0, None, CacheNeed(state=StateNeed((("sum", (4,)),))))]
    cache = make(needs=needs)
    s, = cache.acquire(1)
    cache.view(0).state["sum"][s] = 5.0
    cache.release(s)
    t, = cache.acquire(1)
    assert t == s and float(cache.view(0).state["sum"][t].abs().sum()) == 0.0


def test_cache_of_must_point_backwards():
    with pytest.raises(CacheError, match="runs later"):
        make(needs=[(0, 1, CacheNeed(kv=KVNeed(2, 16))), (1, None, CacheNeed(kv=KVNeed(2, 16)))])


def test_random_traffic_keeps_invariants():
    rng = random.Random(0)
    cache = make(max_tokens=PAGE * 12, n_slots=5)
    live = []
    for _ in range(600):
        op = rng.random()
        if op < 0.3 and cache.n_free_slots:
            live += cache.acquire(1)
        elif op < 0.5 and live:
            cache.release(live.pop(rng.randrange(len(live))))
        elif live:
            batch = rng.sample(live, rng.randint(1, len(live)))
            try:
                cache.reserve([(s, rng.choice([1, 1, 1, 5, 64, 130])) for s in batch])
            except CacheFull:
                pass
        cache.check()
    for s in live:
        cache.release(s)
    cache.check()
    assert cache.n_free_slots == 5 and cache.free_pages() == 12
