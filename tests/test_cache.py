"""The cache's bookkeeping on the host: no slot or page is lost, held twice or
freed twice; growth is all or nothing; windows give pages back; state is zeroed."""
import random

import pytest
import torch

from zlm_b200.cache import CacheBookkeepingError, CacheFull, FreeList, KVCache, pages_for
from zlm_b200.config import ScheduleEntry
from zlm_b200.parts.base import CacheRequest, StateRequest


def make(max_tokens=64 * 10, max_slots=4, max_seq_len=64 * 6, window=0, states=False, entries=3):
    sched = [ScheduleEntry(i) for i in range(entries)]
    reqs = [CacheRequest(2, 16, window if i % 2 else 0) for i in range(entries)]
    sts = [StateRequest((3, 5)) if states and i == 1 else None for i in range(entries)]
    return KVCache(sched, reqs, sts, max_tokens, max_slots, max_seq_len, torch.float32, "cpu")


def test_free_list_never_hands_a_number_out_twice():
    f = FreeList(5, "page")
    a = f.take(3)
    assert a == [0, 1, 2] and f.available == 2 and f.held == 3
    with pytest.raises(CacheFull, match="2 free pages, 3 are needed"):
        f.take(3)
    f.give([1])
    with pytest.raises(CacheBookkeepingError, match="page 1 is returned but is not held"):
        f.give([1])
    with pytest.raises(CacheBookkeepingError, match="page 4"):
        f.give([4])
    assert f.take(1) == [1]            # lowest first: reuse is deterministic
    f.check()


def test_slots_and_pages_come_back():
    c = make()
    s0, s1 = c.alloc_slot(), c.alloc_slot()
    c.reserve([(s0, 70), (s1, 5)])
    c.commit([(s0, 70), (s1, 5)])
    assert c.length(s0) == 70 and c.groups[0].pages.held == 3
    c.check()
    c.free_slot(s0)
    with pytest.raises(CacheBookkeepingError, match="slot 0 is freed but is not held"):
        c.free_slot(s0)
    assert c.groups[0].pages.held == 1 and c.slots.held == 1
    s2 = c.alloc_slot()
    assert s2 == s0 and c.length(s2) == 0       # the slot is used again, empty
    c.reserve([(s2, 64)])
    assert c.groups[0].slot_pages[s2] == [0]     # and so is its first page
    c.check()
    with pytest.raises(CacheBookkeepingError, match="slot 3 is not held"):
        c.reserve([(3, 1)])


def test_growth_is_all_or_nothing():
    c = make(max_tokens=64 * 4)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 100)])
    c.commit([(a, 100)])
    held = c.groups[0].pages.held
    with pytest.raises(CacheFull, match="needs 4 more pages"):
        c.reserve([(a, 29), (b, 129)])           # a would need 1, b 3; only 2 are free
    assert c.groups[0].pages.held == held and c.groups[0].slot_pages.get(b, []) == []
    with pytest.raises(CacheFull, match="longest"):
        c.reserve([(a, 64 * 6)])
    c.check()


def test_no_more_slots_than_asked_for():
    c = make(max_slots=2)
    c.alloc_slot(), c.alloc_slot()
    with pytest.raises(CacheFull, match="0 free slots"):
        c.alloc_slot()


def test_block_table_follows_the_pages():
    c = make()
    s = c.alloc_slot()
    c.reserve([(s, 65)])
    g = c.groups[0]
    assert g.block_table[s, :2].tolist() == g.slot_pages[s]
    c.commit([(s, 65)])
    c.reserve([(s, 64)])                          # 65 + 64 = 129 tokens: a third page
    assert len(g.slot_pages[s]) == 3 and g.block_table[s, 2].item() == g.slot_pages[s][2]


def test_groups_have_storage_of_their_own_and_windows_give_pages_back():
    c = make(window=70, max_tokens=64 * 8, max_seq_len=64 * 8)
    assert len(c.groups) == 2
    full = next(g for g in c.groups if g.window == 0)
    win = next(g for g in c.groups if g.window == 70)
    assert full.pool.data_ptr() != win.pool.data_ptr() and len(full.entries) == 2 and len(win.entries) == 1
    s = c.alloc_slot()
    c.reserve([(s, 300)])
    assert win.pages.held == full.pages.held == 5   # a long step needs all its keys while it runs
    c.commit([(s, 300)])
    # the next query sits at 300 and reads keys >= 231: pages 0..2 (keys < 192) are gone
    assert win.slot_pages[s][:3] == [-1, -1, -1] and win.pages.held == 2 and full.pages.held == 5
    c.check()
    c.free_slot(s)
    assert win.pages.held == 0 and full.pages.held == 0
    c.check()


def test_state_is_zeroed_when_a_slot_is_taken():
    c = make(states=True)
    st = c.ios[1].state
    assert st.shape == (4, 3, 5) and c.ios[0].state is None
    s = c.alloc_slot()
    st[s] += 7
    c.free_slot(s)
    assert c.alloc_slot() == s and float(st[s].abs().sum()) == 0.0


def test_an_entry_may_read_another_entrys_cache():
    sched = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)]
    reqs = [CacheRequest(2, 16), CacheRequest(2, 16), CacheRequest(2, 16)]
    c = KVCache(sched, reqs, [None] * 3, 640, 2, 640, torch.float32, "cpu")
    assert c.groups[0].entries == [0, 1]
    assert c.ios[2].cache.pool.data_ptr() == c.ios[0].cache.pool.data_ptr()
    assert c.ios[0].cache.writes and not c.ios[2].cache.writes


def test_random_traffic_keeps_the_books():
    rnd = random.Random(0)
    c = make(max_tokens=64 * 12, max_slots=5, max_seq_len=64 * 5, window=40)
    live = {}
    for _ in range(400):
        op = rnd.random()
        if op < 0.3 and c.slots.available:
            live[c.alloc_slot()] = 0
        elif op < 0.8 and live:
            s = rnd.choice(list(live))
            n = rnd.randint(1, 90)
            try:
                c.reserve([(s, n)])
                c.commit([(s, n)])
                live[s] += n
            except CacheFull:
                pass
        elif live:
            s = rnd.choice(list(live))
            c.free_slot(s)
            del live[s]
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            for g in c.groups:
                have = g.slot_pages.get(s, [])
                assert len(have) == pages_for(n)
                first = max(0, n + 1 - g.window) // 64 if g.window else 0
                assert all((p >= 0) == (i >= first) for i, p in enumerate(have))
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pages.held == 0 for g in c.groups) and c.slots.held == 0


def test_a_request_with_a_record_of_its_own_gets_its_own_paged_pool():
    """A mixer may keep something other than keys and values per token: the pool then has the
    record's shape and element type, in a group of its own, paged and freed like the others."""
    from zlm_b200.parts.base import CacheRequest
    sched = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)]
    reqs = [CacheRequest(2, 16), CacheRequest(1, 24, token_shape=(24,), dtype=torch.float32),
            CacheRequest(1, 24, token_shape=(24,), dtype=torch.float32)]
    c = KVCache(sched, reqs, [None] * 3, 64 * 6, 3, 256, torch.bfloat16, "cpu")
    assert len(c.groups) == 2
    kv, latent = c.ios[0].cache, c.ios[1].cache
    assert tuple(kv.pool.shape) == (6, 2, 2, 64, 16) and kv.pool.dtype == torch.bfloat16
    assert tuple(latent.pool.shape) == (6, 64, 24) and latent.pool.dtype == torch.float32
    assert c.ios[2].cache.block_table is latent.block_table and c.ios[2].cache.pool is not latent.pool
    assert c.bytes_per_token() == 2 * 2 * 16 * 2 + 2 * 24 * 4
    s = c.alloc_slot()
    c.reserve([(s, 130)])
    c.commit([(s, 130)])
    assert all(g.pages.held == 3 for g in c.groups)
    c.free_slot(s)
    c.check()
    assert all(g.pages.held == 0 for g in c.groups)
