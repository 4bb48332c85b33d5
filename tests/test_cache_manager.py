"""Cache manager on the CPU: pages are never lost, held twice or freed twice, under
random orders of requests; windowed groups give pages back; state slots."""
import random

import pytest
import torch

from sparseengine_b200.cache.manager import CacheManager
from sparseengine_b200.cache.pages import OutOfPages, PagePool
from sparseengine_b200.engine.model import CacheLayout, EntryCache
from sparseengine_b200.parts.base import KVRequest, StateRequest


def layout(windows=(None,), layers=(2,), states=()):
    groups = tuple((KVRequest(2, 16, w), n) for w, n in zip(windows, layers))
    entries = tuple(EntryCache(g, i, True, None) for g, (_, n) in enumerate(groups) for i in range(n))
    return CacheLayout(groups, tuple(states), entries)


def test_pool_lifo_and_books():
    p = PagePool(4)
    a = p.take(3)
    assert a == [0, 1, 2] and p.free == 1
    p.give([1])
    assert p.take(1) == [1]          # last given back is taken first
    assert p.reused_total == 1
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.free == 1               # a failed take takes nothing
    with pytest.raises(ValueError):
        p.give([3])                  # not held
    p.give([0])
    with pytest.raises(ValueError):
        p.give([0])                  # freed twice
    p.check()


def test_reserve_commit_release_and_block_table():
    cm = CacheManager(layout(), page_size=4, num_pages=6, max_rows=2, max_seq_len=40, allocate=False)
    row = cm.admit("a")
    cm.reserve("a", 5)               # positions 0..4 -> 2 pages
    assert cm.free_pages() == 4 and cm.length("a") == 0
    ups = cm.drain_updates(0)
    assert [(r, i) for r, i, _ in ups] == [(row, 0), (row, 1)]
    cm.commit("a", 5)
    cm.reserve("a", 3)               # positions 5..7 still fit page 1
    assert cm.free_pages() == 4 and cm.drain_updates(0) == []
    cm.commit("a", 3)
    cm.reserve("a", 1)               # position 8 -> a third page
    assert cm.free_pages() == 3
    cm.commit("a", 1)
    assert cm.length("a") == 9
    assert list(cm.groups[0].table_host[row, :3]) == [u[2] for u in ups] + [cm.drain_updates(0)[0][2]]
    cm.check()
    cm.release("a")
    assert cm.free_pages() == 6 and cm.free_rows == 2
    with pytest.raises(ValueError):
        cm.release("a")              # released twice
    cm.check()


def test_reserve_is_all_or_nothing_over_groups_and_cancel():
    cm = CacheManager(layout(windows=(None, 8), layers=(1, 1)), page_size=4, num_pages=[8, 2], max_rows=2,
                      max_seq_len=64, allocate=False)
    cm.admit("a")
    with pytest.raises(OutOfPages):
        cm.reserve("a", 12)          # group 1 has 2 pages, 3 are needed
    assert cm.free_pages(0) == 8 and cm.free_pages(1) == 2
    cm.reserve("a", 8)
    cm.cancel("a")
    assert cm.free_pages(0) == 8 and cm.free_pages(1) == 2 and cm.drain_updates(0) == []
    cm.check()
    with pytest.raises(ValueError):
        cm.reserve("a", 100)         # beyond max_seq_len


def test_window_group_gives_pages_back():
    cm = CacheManager(layout(windows=(None, 6), layers=(1, 1)), page_size=4, num_pages=[16, 4], max_rows=1,
                      max_seq_len=64, allocate=False)
    cm.admit("a")
    for _ in range(10):
        cm.reserve("a", 4)
        cm.commit("a", 4)
        # the next query (position = length) sees keys length-5 .. length: pages before that are back
        first_needed = cm.length("a") - 6 + 1
        held = sorted(cm._requests["a"].pages[1])
        assert all((i + 1) * 4 > first_needed for i in held)
        assert len(held) <= 3
        cm.check()
    assert cm.free_pages(0) == 16 - 10
    assert cm.groups[1].pool.reused_total > 0
    cm.release("a")
    assert cm.free_pages(1) == 4
    cm.check()


def test_state_slots_zeroed_on_admission():
    lay = CacheLayout((), (StateRequest((3,), torch.float32),), (EntryCache(None, None, False, 0),))
    cm = CacheManager(lay, page_size=4, num_pages=[], max_rows=2, max_seq_len=16, device="cpu")
    r = cm.admit("a")
    cm.states[0][r] += 5
    cm.release("a")
    r2 = cm.admit("b")
    assert r2 == r and float(cm.states[0][r2].abs().sum()) == 0.0
    slot = cm.slot_for(lay.entries[0])
    assert slot.state is cm.states[0] and slot.kv is None


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_double_book_a_page(seed):
    rng = random.Random(seed)
    windows = (None, rng.choice([5, 9, 16]))
    cm = CacheManager(layout(windows=windows, layers=(2, 1)), page_size=rng.choice([2, 4, 8]),
                      num_pages=[rng.randint(6, 20), rng.randint(6, 20)], max_rows=3, max_seq_len=60,
                      allocate=False)
    live = {}
    nxt = 0
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and cm.free_rows:
            cm.admit(nxt)
            live[nxt] = 0
            nxt += 1
        elif op < 0.8 and live:
            sid = rng.choice(list(live))
            n = rng.randint(1, 9)
            if live[sid] + n > 60:
                continue
            ok = cm.can_reserve([(sid, n)])
            try:
                cm.reserve(sid, n)
            except OutOfPages:
                assert not ok
                cm.check()
                continue
            assert ok
            if rng.random() < 0.15:
                cm.cancel(sid)
            else:
                cm.commit(sid, n)
                live[sid] += n
                assert cm.length(sid) == live[sid]
        elif live:
            sid = rng.choice(list(live))
            cm.release(sid)
            del live[sid]
        cm.check()
        # every position a later query can see has a page
        for sid, length in live.items():
            r = cm._requests[sid]
            for gi, g in enumerate(cm.groups):
                lo = 0 if g.window is None else max(0, length - g.window + 1)
                for pos in range(lo, length):
                    assert pos // cm.page_size in r.pages[gi]
    for sid in list(live):
        cm.release(sid)
    assert all(g.pool.free == g.pool.num_pages for g in cm.groups) and cm.free_rows == 3
    cm.check()


def test_reserved_state_slot_is_zeroed_at_admission():
    """The per-request slot that no part of the dense-cache path uses: fixed size, one per
    row, clean for every new request."""
    m = CacheManager(layout(), page_size=4, num_pages=8, max_rows=2, max_seq_len=32, reserved_state_bytes=24)
    assert m.reserved_state.shape == (2, 24) and m.reserved_state.dtype == torch.uint8
    row = m.admit("a")
    m.reserved_state[row].fill_(7)
    m.release("a")
    assert m.admit("b") == row and int(m.reserved_state[row].sum()) == 0
    assert CacheManager(layout(), page_size=4, num_pages=8, max_rows=2, max_seq_len=32).reserved_state is None
