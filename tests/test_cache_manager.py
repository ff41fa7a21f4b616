"""The cache manager on the host: no page lost, held twice or freed twice, under random orders."""

import random

import numpy as np
import pytest
import torch

from torchllms_b200.cache.manager import FREED, CacheError, CacheManager, OutOfPages, PageAllocator
from torchllms_b200.parts.base import CacheNeed, StateNeed

FULL = CacheNeed("full", 2, 16)
WIN = CacheNeed("window", 1, 32, window=20)


def manager(needs=((FULL, None, None), (FULL, None, None)), page_size=4, pool_tokens=64, max_num_seqs=4, max_len=48, **kw):
    return CacheManager(list(needs), page_size=page_size, pool_tokens=pool_tokens, max_num_seqs=max_num_seqs,
                        max_len=max_len, dtype=torch.float32, device="cpu", **kw)


def test_growth_is_lazy_and_by_whole_pages():
    m = manager()
    h = m.claim()
    assert m.length(h) == 0 and m.pages_of(h) == []
    assert m.extend_many([(h, 1)]) == [0] and len(m.pages_of(h)) == 1
    assert m.extend_many([(h, 3)]) == [1] and len(m.pages_of(h)) == 1          # still inside the first page
    assert m.extend_many([(h, 1)]) == [4] and len(m.pages_of(h)) == 2
    assert m.extend_many([(h, 9)]) == [5] and len(m.pages_of(h)) == 4 and m.length(h) == 14
    m.check_invariants()


def test_layers_of_one_need_share_one_group_and_one_table():
    m = manager()
    assert len(m.groups) == 1 and m.groups[0].runs == [0, 1]
    assert m.groups[0].k_pages.shape == (2, 16, 2, 4, 16)                      # [run, page, kv head, slot, head_dim]


def test_freed_pages_are_used_again_first():
    m = manager(pool_tokens=12)                                                # 3 pages
    a, b = m.claim(), m.claim()
    m.extend_many([(a, 8), (b, 4)])
    pa = m.pages_of(a)
    with pytest.raises(OutOfPages):
        m.extend_many([(b, 1)])
    m.release(a)
    m.extend_many([(b, 4)])
    assert m.pages_of(b)[1] == pa[-1]                                          # the page freed last goes out first
    m.check_invariants()


def test_extension_is_all_or_nothing():
    m = manager(pool_tokens=16)                                                # 4 pages
    a, b = m.claim(), m.claim()
    m.extend_many([(a, 6)])
    assert not m.can_extend([(a, 4), (b, 8)])
    with pytest.raises(OutOfPages):
        m.extend_many([(a, 4), (b, 8)])                                        # a alone would fit; together they do not
    assert m.length(a) == 6 and m.length(b) == 0 and m.free_pages() == 2
    assert m.can_extend([(a, 2), (b, 8)])
    m.extend_many([(a, 2), (b, 8)])
    assert m.free_pages() == 0
    m.check_invariants()


def test_room_for():
    m = manager(pool_tokens=16)
    a, b = m.claim(), m.claim()
    m.extend_many([(a, 6)])
    assert m.room_for(a) == 2 + 8 and m.room_for(b) == 8
    assert m.room_for(b, [(a, 3)]) == 4
    assert m.room_for(a, [(b, 8)]) == 2


def test_handles_are_never_reused_but_slots_are():
    m = manager(max_num_seqs=2)
    a, b = m.claim(), m.claim()
    assert not m.has_free_slot()
    with pytest.raises(CacheError):
        m.claim()
    slot_a = m.slot(a)
    m.release(a)
    c = m.claim()
    assert c not in (a, b) and m.slot(c) == slot_a
    with pytest.raises(CacheError):
        m.release(a)                                                           # freed twice
    with pytest.raises(CacheError):
        m.length(a)


def test_misuse_is_refused():
    m = manager()
    h = m.claim()
    with pytest.raises(CacheError):
        m.extend_many([(h, 2), (h, 1)])                                        # one request twice in a batch
    with pytest.raises(CacheError):
        m.extend_many([(h, 0)])
    with pytest.raises(CacheError):
        m.extend_many([(h, 49)])                                               # beyond the longest sequence
    assert not m.can_extend([(h, 49)])
    with pytest.raises(CacheError):
        m.extend_many([(99, 1)])
    alloc = PageAllocator(2)
    p = alloc.alloc(1)[0]
    alloc.release(p)
    with pytest.raises(CacheError):
        alloc.release(p)


def test_truncate_gives_trailing_pages_back():
    m = manager()
    h = m.claim()
    m.extend_many([(h, 14)])
    m.truncate(h, 5)
    assert m.length(h) == 5 and len(m.pages_of(h)) == 2 and m.free_pages() == 14
    m.truncate(h, 0)
    assert m.pages_of(h) == [] and m.free_pages() == 16
    m.check_invariants()


def test_slot_mapping_and_block_table_rows():
    m = manager()
    a, b = m.claim(), m.claim()
    m.extend_many([(a, 6), (b, 3)])
    pages = m.pages_of(a)
    sm = m.slot_mapping(0, a, 2, 4)
    assert sm.tolist() == [pages[0] * 4 + 2, pages[0] * 4 + 3, pages[1] * 4 + 0, pages[1] * 4 + 1]
    rows = m.block_table_rows(0, [m.slot(b), m.slot(a)])
    assert rows.shape == (2, 12) and rows[1, :2].tolist() == pages and (rows[1, 2:] == FREED).all()
    assert rows[0, 0] == m.pages_of(b)[0]


def test_window_group_gives_pages_back_behind_the_window():
    m = manager(needs=((FULL, None, None), (WIN, None, None)), page_size=4, pool_tokens=200, max_len=200)
    assert len(m.groups) == 2
    win = [g.index for g in m.groups if g.need.kind == "window"][0]
    full = 1 - win
    h = m.claim()
    m.extend_many([(h, 30)])
    assert m.pass_window(h) == 2           # next query at 30 reads keys 11..30: blocks 0 and 1 (keys 0..7) are dead
    assert m.pages_of(h, win)[:2] == [FREED, FREED] and FREED not in m.pages_of(h, full)
    m.check_invariants()
    for _ in range(40):
        m.extend_many([(h, 1)])
        m.pass_window(h)
        m.check_invariants()
    live = [p for p in m.pages_of(h, win) if p != FREED]
    assert len(live) <= 20 // 4 + 2        # about a window's worth of pages stays
    assert len(m.pages_of(h, full)) == -(-70 // 4) and FREED not in m.pages_of(h, full)
    with pytest.raises(CacheError):
        m.slot_mapping(win, h, 0, 4)       # those tokens' pages are gone
    with pytest.raises(CacheError):
        m.truncate(h, 20)                  # would need keys the window group gave back
    m.release(h)
    m.check_invariants()
    assert all(g.allocator.n_free == g.allocator.n_pages for g in m.groups)


def test_a_run_may_read_another_runs_cache():
    needs = [(FULL, None, None), (FULL, None, 0), (None, StateNeed((3,)), None)]
    m = manager(needs=needs)
    assert m.groups[0].runs == [0]                     # the borrowing run owns no pages
    bt, sm = [torch.zeros(1, 12, dtype=torch.int32)], [torch.zeros(1, dtype=torch.int32)]
    v0, v1, v2 = (m.run_view(i, bt, sm) for i in range(3))
    assert v0.writes and not v1.writes and v1.k_pages.data_ptr() == v0.k_pages.data_ptr()
    assert v2.k_pages is None and v2.state.shape == (4, 3)
    with pytest.raises(ValueError):
        manager(needs=[(None, None, None), (FULL, None, 0)])


def test_state_rows_are_zeroed_on_claim():
    m = manager(needs=[(None, StateNeed((2, 3)), None)])
    assert m.groups == []
    h = m.claim()
    m.state[0][m.slot(h)] += 5
    slot = m.slot(h)
    m.release(h)
    h2 = m.claim()
    assert m.slot(h2) == slot and (m.state[0][slot] == 0).all()
    assert m.extend_many([(h2, 7)]) == [0] and m.length(h2) == 7         # lengths are tracked without pages too


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_every_invariant(seed):
    rng = random.Random(seed)
    needs = ((FULL, None, None), (WIN, None, None), (FULL, None, 0)) if seed % 2 else ((FULL, None, None),)
    m = manager(needs=needs, page_size=rng.choice([1, 4, 8]), pool_tokens=rng.choice([40, 96, 160]),
                max_num_seqs=5, max_len=80)
    live = []
    for _ in range(400):
        op = rng.random()
        if op < 0.2 and m.has_free_slot():
            live.append(m.claim())
        elif op < 0.3 and live:
            m.release(live.pop(rng.randrange(len(live))))
        elif op < 0.37 and live:
            h = rng.choice(live)
            try:
                m.truncate(h, rng.randint(0, m.length(h)))
            except CacheError:
                pass                                       # behind a window
        elif live:
            batch = rng.sample(live, rng.randint(1, len(live)))
            wants = [(h, rng.randint(1, 24)) for h in batch]
            ok = m.can_extend(wants)
            before = [m.length(h) for h, _ in wants]
            try:
                starts = m.extend_many(wants)
                assert ok and starts == before
                for h, n in wants:
                    m.slot_mapping(0, h, m.length(h) - n, n)
                    m.pass_window(h)
            except OutOfPages:
                assert not ok and [m.length(h) for h, _ in wants] == before
            except CacheError:
                assert not ok                              # beyond max_len
        m.check_invariants()
    for h in live:
        m.release(h)
    m.check_invariants()
    assert all(g.allocator.n_free == g.allocator.n_pages for g in m.groups)
