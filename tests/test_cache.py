"""The cache's bookkeeping (no GPU): no slot or block lost, held twice or freed twice."""
import random

import pytest
import torch

from hymt2sharp_b200.cache import CacheBook, CacheError, CacheFull, GroupSpec, PagedCache

FULL = GroupSpec("full", kv_heads=2, head_dim=16, planes=2)
WIN = GroupSpec("window", kv_heads=1, head_dim=16, planes=1, window=100)


def test_slots_and_blocks_come_back():
    book = CacheBook([FULL], blocks_per_group=8, block_tokens=64, max_slots=3)
    a, b = book.alloc_slot(), book.alloc_slot()
    book.reserve([(a, 130), (b, 64)])
    book.commit(a, 130); book.commit(b, 64)
    assert book.length(a) == 130 and len(book.sequences[a].blocks[0]) == 3 and len(book.sequences[b].blocks[0]) == 1
    book.reserve([(b, 1)])  # crossing the block's end takes one more
    book.commit(b, 1)
    assert len(book.sequences[b].blocks[0]) == 2
    book.audit()
    book.free_slot(a)
    assert book.pools[0].free_count == 6
    c = book.alloc_slot()
    assert c == a  # the slot is used again
    book.reserve([(c, 64 * 6)])
    book.commit(c, 64 * 6)
    book.audit()
    assert book.pools[0].free_count == 0


def test_errors_change_nothing():
    book = CacheBook([FULL, WIN], blocks_per_group=4, block_tokens=64, max_slots=2)
    a, b = book.alloc_slot(), book.alloc_slot()
    with pytest.raises(CacheFull):
        book.alloc_slot()
    book.reserve([(a, 100)])
    book.commit(a, 100)
    before = (book.pools[0].free_count, book.pools[1].free_count)
    with pytest.raises(CacheFull):
        book.reserve([(a, 30), (b, 129)])  # 1 + 3 > 2 free: nothing of it may stay
    assert (book.pools[0].free_count, book.pools[1].free_count) == before
    with pytest.raises(CacheError):
        book.reserve([(a, 1), (a, 1)])
    with pytest.raises(CacheError):
        book.commit(b, 5)  # not reserved
    assert book.length(b) == 0
    book.free_slot(b)
    with pytest.raises(CacheError):
        book.free_slot(b)  # freed twice
    with pytest.raises(CacheError):
        book.length(7)
    book.audit()


def test_window_group_gives_old_blocks_back():
    book = CacheBook([FULL, WIN], blocks_per_group=8, block_tokens=64, max_slots=1)
    s = book.alloc_slot()
    book.reserve([(s, 300)])
    assert book.pools[1].free_count == 3  # a prompt needs all its blocks while it runs
    dropped = book.commit(s, 300)
    # the next step's first token (position 300) sees keys from 201 on: blocks 0..2 go back
    assert [(g, i) for g, i, p in dropped] == [(1, 0), (1, 1), (1, 2)]
    assert book.sequences[s].blocks[1][:3] == [-1, -1, -1] and book.pools[1].free_count == 6
    assert book.pools[0].free_count == 3  # the full group keeps everything
    for _ in range(200):
        book.reserve([(s, 1)])
        book.commit(s, 1)
        book.audit()
    assert book.pools[1].n - book.pools[1].free_count <= 3
    with pytest.raises(CacheError):
        book.truncate(s, 250)  # would need keys that are gone
    book.truncate(s, 499)
    book.free_slot(s)
    book.audit()
    assert book.pools[1].free_count == 8 and book.pools[0].free_count == 8


def test_truncate_and_reset():
    book = CacheBook([FULL], blocks_per_group=8, block_tokens=64, max_slots=1)
    s = book.alloc_slot()
    book.reserve([(s, 200)]); book.commit(s, 200)
    book.truncate(s, 65)
    assert book.length(s) == 65 and book.pools[0].free_count == 6
    book.truncate(s, 0)
    assert book.pools[0].free_count == 8
    with pytest.raises(CacheError):
        book.truncate(s, 1)


def test_random_traffic_loses_nothing():
    rng = random.Random(3)
    book = CacheBook([FULL, WIN], blocks_per_group=40, block_tokens=64, max_slots=6)
    live = []
    for step in range(2000):
        r = rng.random()
        if r < 0.15 and book.slots.free_count:
            live.append(book.alloc_slot())
        elif r < 0.25 and live:
            book.free_slot(live.pop(rng.randrange(len(live))))
        elif live:
            plan = [(s, rng.choice([1, 1, 1, 7, 70, 200])) for s in rng.sample(live, rng.randint(1, len(live)))]
            try:
                book.reserve(plan)
            except CacheFull:
                book.audit()
                continue
            for s, n in plan:
                book.commit(s, n)
        if step % 50 == 0:
            book.audit()
    for s in live:
        book.free_slot(s)
    book.audit()
    assert all(p.free_count == p.n for p in book.pools) and book.slots.free_count == 6


def test_device_side_on_cpu_tensors():
    """The tables and the state area follow the bookkeeping (tensors on the CPU here)."""
    cache = PagedCache([FULL, WIN], torch.float32, "cpu", capacity_tokens=64 * 12, max_slots=2, state_bytes=24)
    assert cache.storage[0].shape == (2, 2, 12, 2, 64, 16) and cache.storage[1].shape == (1, 2, 12, 1, 64, 16)
    assert cache.bytes_per_token() == (2 * 2 * 2 * 16 + 2 * 1 * 1 * 16) * 4
    slots = cache.alloc_slots(2)
    cache.state[slots[0]] = 7
    cache.begin_step([(slots[0], 70), (slots[1], 3)])
    cache.end_step([(slots[0], 70), (slots[1], 3)])
    assert cache.tables[0][slots[0], :2].tolist() == cache.host_tables[0][slots[0], :2].tolist()
    assert (cache.host_tables[0][slots[0], :2] >= 0).all() and cache.host_tables[0][slots[0], 2] == -1
    more = cache.alloc_slots(3)  # grows the tables and the state area
    assert cache.max_slots >= 5 and cache.state.shape[0] >= 5 and cache.layout_version == 1
    assert cache.tables[0][slots[0], :2].tolist() == cache.host_tables[0][slots[0], :2].tolist()
    assert int(cache.state[slots[0]].sum()) == 7 * 24
    cache.free_slots([slots[0]])
    again = cache.alloc_slots(1)
    assert again == [slots[0]] and int(cache.state[again[0]].sum()) == 0  # zeroed when handed out
    with pytest.raises(CacheFull):
        cache.begin_step([(more[0], 64 * 13)])
    cache.begin_step([(more[0], 64 * 9)])  # more columns than the table had
    assert cache.table_cols >= 9
    cache.end_step([(more[0], 64 * 9)])
    cache.free_slots(slots[1:] + more + again)
    cache.book.audit()
    assert cache.free_tokens() == 64 * 12
