"""Cache manager bookkeeping (no GPU): no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; reserve is all-or-nothing."""
import numpy as np
import pytest
import torch

from glint_b200.cache import CacheManager, PagedKVNeed, PagePool, SlotStateNeed
from glint_b200.errors import GlintError, PagePoolExhausted, SlotsExhausted


def manager(num_pages=12, num_slots=4, window=8, page=16, max_pos=256):
    needs = [PagedKVNeed(1, 8, window), PagedKVNeed(1, 8, None), PagedKVNeed(1, 8, window),
             SlotStateNeed((3,), torch.float32), None]
    return CacheManager(needs, [None] * 5, num_slots, num_pages, page, max_pos, torch.float32, "cpu")


def test_groups_by_need():
    m = manager()
    assert sorted(g.name for g in m.groups) == ["kv1x8/all", "kv1x8/window8"]
    win = next(g for g in m.groups if g.need.window == 8)
    assert win.members == [0, 2] and win.storage[0].shape == (2, 12, 1, 16, 8)
    assert m.views[0].k.data_ptr() != m.views[2].k.data_ptr()
    assert m.views[3] is None and m.states[3].shape == (4, 3) and m.states[4] is None


def test_pool_take_give_and_double_free():
    p = PagePool("g", 3)
    a = p.take(2)
    assert p.live == 2 and p.available == 1
    with pytest.raises(PagePoolExhausted) as e:
        p.take(2)
    assert (e.value.needed, e.value.available, e.value.capacity) == (2, 1, 3)
    assert p.live == 2                                  # nothing was taken
    p.give(a)
    with pytest.raises(GlintError, match="not owned"):
        p.give([a[0]])
    assert sorted(p.take(3)) == [0, 1, 2] and p.reuses == 2


def test_pages_only_on_boundaries_and_window_release():
    m = manager()
    s = m.alloc_slot()
    full = next(g for g in m.groups if g.need.window is None)
    win = next(g for g in m.groups if g.need.window == 8)
    m.reserve([(s, 16)]); m.advance([(s, 16)])
    assert full.pool.live == 1 and win.pool.live == 1
    m.reserve([(s, 1)]); m.advance([(s, 1)])
    assert full.pool.live == 2 and win.pool.live == 2
    for _ in range(23):                                # up to 40 tokens
        m.reserve([(s, 1)]); m.advance([(s, 1)])
    # next query at position 40 reads keys from 33: pages 0 and 1 of the window group are gone
    m.reserve([(s, 1)])
    assert full.pool.live == 3 and win.pool.live == 1
    assert list(win.table[s, :3]) == [-1, -1, win.table[s, 2]] and win.table[s, 2] >= 0
    m.check_consistency()
    m.free_slot(s)
    assert full.pool.live == 0 and win.pool.live == 0
    with pytest.raises(GlintError, match="not in use"):
        m.free_slot(s)


def test_reserve_is_all_or_nothing_and_reports_shortfall():
    m = manager(num_pages=4)
    a, b = m.alloc_slot(), m.alloc_slot()
    m.reserve([(a, 40)]); m.advance([(a, 40)])          # 3 pages
    before = m.stats()
    assert m.pages_short([(a, 1), (b, 17)]) is not None
    with pytest.raises(PagePoolExhausted) as e:
        m.reserve([(a, 1), (b, 17)])
    assert e.value.needed == 2 and e.value.available == 1 and e.value.capacity == 4
    assert {k: v["live"] for k, v in m.stats().items() if k.endswith("all")} == \
           {k: v["live"] for k, v in before.items() if k.endswith("all")}
    m.check_consistency()
    m.reserve([(b, 16)])                                 # what fits still fits
    m.check_consistency()


def test_context_limit_and_slots():
    m = manager(max_pos=32)
    s = m.alloc_slot()
    with pytest.raises(GlintError, match="context length"):
        m.reserve([(s, 33)])
    for _ in range(3):
        m.alloc_slot()
    with pytest.raises(SlotsExhausted):
        m.alloc_slot()


def test_state_rows_are_zeroed_at_admission():
    m = manager()
    s = m.alloc_slot()
    m.states[3][s] = 7.0
    m.free_slot(s)
    s2 = m.alloc_slot()
    assert s2 == s and float(m.states[3][s2].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = np.random.default_rng(seed)
    m = manager(num_pages=10, num_slots=4, window=int(rng.choice([8, 16, 40])), max_pos=200)
    live = {}
    for _ in range(400):
        op = rng.random()
        if op < 0.15 and m.free_slots:
            live[m.alloc_slot()] = 0
        elif op < 0.3 and live:
            s = list(live)[int(rng.integers(len(live)))]
            m.free_slot(s)
            del live[s]
        elif live:
            k = int(rng.integers(1, len(live) + 1))
            chosen = [list(live)[i] for i in rng.permutation(len(live))[:k]]
            rows = [(s, int(rng.integers(1, 30))) for s in chosen if live[s] < 150]
            if not rows:
                continue
            try:
                m.reserve(rows)
                m.advance(rows)
                for s, n in rows:
                    live[s] += n
            except PagePoolExhausted:
                pass
        m.check_consistency()
        for g in m.groups:                               # every key a next query needs has a page
            for s, n in live.items():
                lo = 0 if g.need.window is None else max(0, n - g.need.window + 1)
                for p in range(lo // 16, (n + 15) // 16):
                    assert g.table[s, p] >= 0, (g.name, s, n, p)
    for s in list(live):
        m.free_slot(s)
    assert all(v["live"] == 0 for v in m.stats().values())
