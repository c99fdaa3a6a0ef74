"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; exhaustion takes nothing."""

import random

import numpy as np
import pytest
import torch

from shiso_llm_b200.cache import BlockTable, CacheManager, OutOfPages, PagePool, SlotPool
from shiso_llm_b200.parts import FixedState, PagedKV


def manager(num_pages=12, page=4, slots=3, needs=None, max_blocks=None):
    needs = needs or [FixedState((2, 8)), PagedKV(2, 16), None, FixedState((3, 8)), PagedKV(1, 32)]
    return CacheManager(needs, page, num_pages, slots, torch.float32, "cpu", max_blocks)


def test_pool_is_fifo_and_refuses_double_free():
    pool = PagePool(4)
    assert pool.take(3) == [0, 1, 2]
    pool.give_back(1)
    assert pool.take(2) == [3, 1]  # the page free longest goes first
    with pytest.raises(OutOfPages):
        pool.take(1)
    pool.give_back(0)
    with pytest.raises(RuntimeError):
        pool.give_back(0)
    pool.check()


def test_claims_are_all_or_nothing():
    pool = PagePool(3)
    table = BlockTable(4)
    table.grow(pool, 5)
    assert len(table.pages) == 2
    with pytest.raises(OutOfPages):
        table.grow(pool, 16)
    assert len(table.pages) == 2 and pool.free_pages == 1


def test_slots():
    slots = SlotPool(2)
    a, b = slots.take(), slots.take()
    with pytest.raises(OutOfPages):
        slots.take()
    slots.give_back(a)
    with pytest.raises(RuntimeError):
        slots.give_back(a)
    assert slots.take() == a
    slots.check()


def test_layout_groups_and_state_views():
    m = manager()
    assert len(m.groups) == 1  # both paged entries keep all keys: one group, one block table
    assert m.view(1).k.shape == (12, 4, 2, 16) and m.view(4).k.shape == (12, 4, 1, 32)
    assert m.view(2) is None
    s0, s3 = m.view(0).state, m.view(3).state
    assert s0.shape == (3, 2, 8) and s3.shape == (3, 3, 8)
    assert m.bytes_per_slot == 4 * (16 + 24) and s0.stride(0) == 40 and s3.stride(0) == 40 and s0.dtype == torch.float32
    assert m.view(1, owner=False).owner is False and m.view(1).owner is True
    windowed = manager(needs=[PagedKV(2, 16), PagedKV(2, 16, window=6), PagedKV(2, 16, window=6)])
    assert len(windowed.groups) == 2 and windowed.view(1).group == windowed.view(2).group != windowed.view(0).group


def test_entries_may_name_their_own_widths_and_element_types():
    """Values narrower than keys, a cache in another element type than the compute type, and
    fixed state that is not float32: each entry's view has what it asked for, ranges of one slot
    do not overlap, and one fill zeroes a slot."""
    needs = [FixedState((3, 5), torch.bfloat16), PagedKV(2, 24, v_head_dim=8, dtype=torch.float16),
             FixedState((7,), torch.int32), PagedKV(1, 16), FixedState((2, 2))]
    m = manager(needs=needs)
    assert m.view(1).k.shape == (12, 4, 2, 24) and m.view(1).v.shape == (12, 4, 2, 8)
    assert m.view(1).k.dtype == m.view(1).v.dtype == torch.float16 and m.view(3).k.dtype == torch.float32
    a, b, c = m.view(0).state, m.view(2).state, m.view(4).state
    assert (a.shape, a.dtype) == ((3, 3, 5), torch.bfloat16) and (b.shape, b.dtype) == ((3, 7), torch.int32)
    assert (c.shape, c.dtype) == ((3, 2, 2), torch.float32)
    assert m.bytes_per_slot == 32 + 32 + 16  # 30, 28 and 16 bytes, each range 16-byte aligned
    a.fill_(1.0), b.fill_(2), c.fill_(3.0)
    assert (a == 1.0).all() and (b == 2).all() and (c == 3.0).all()  # no range reaches into another
    m.append("r", 1)
    slot = m.slot_of("r")
    assert (a[slot] == 0).all() and (b[slot] == 0).all() and (c[slot] == 0).all() and (a[1 - slot if slot < 2 else 0] == 1.0).all()
    page_bytes, state_bytes = m.costs(needs, 4, torch.float32)
    assert page_bytes == 4 * 2 * (24 + 8) * 2 + 4 * 1 * 32 * 4 and state_bytes == 80


def test_append_commit_release_and_zeroed_slot():
    m = manager()
    m.state.view(torch.float32).fill_(7.0)
    assert m.append("a", 5) == 0
    floats = m.state.view(torch.float32)
    assert (floats[m.slot_of("a")] == 0).all() and (floats == 7.0).sum() == 2 * 40
    m.commit("a")
    assert m.length("a") == 5 and m.block_table("a", 0) == [0, 1]
    assert m.append("a", 3) == 5  # still fits page 1
    with pytest.raises(RuntimeError):
        m.append("a", 1)  # twice in one step
    m.commit("a")
    assert m.block_table("a", 0) == [0, 1]
    assert m.append("b", 9) == 0
    m.commit("b")
    out = np.zeros((2, 4), dtype=np.int32)
    m.fill_block_tables(["b", "a"], 0, out)
    assert out.tolist() == [[2, 3, 4, -1], [0, 1, -1, -1]]
    m.release("a")
    with pytest.raises(KeyError):
        m.release("a")
    m.check()
    assert m.free_pages() == [12 - 3]


def test_exhaustion_takes_nothing():
    m = manager(num_pages=4, slots=2)
    m.append("a", 12)
    m.commit("a")
    assert not m.can_append("b", 8) and m.can_append("b", 4)
    with pytest.raises(OutOfPages):
        m.append("b", 8)
    assert not m.has("b") and m.slots.free_slots == 1 and m.free_pages() == [1]
    m.append("b", 4)
    m.commit("b")
    with pytest.raises(OutOfPages):
        m.append("c", 1)  # no state slot left
    with pytest.raises(OutOfPages):
        m.append("a", 5)  # one more page than there is
    assert m.length("a") == 12
    m.check()


def test_blocks_per_request_limit():
    m = manager(num_pages=12, max_blocks=2)
    m.append("a", 8)
    m.commit("a")
    with pytest.raises(OutOfPages):
        m.append("a", 1)


def test_window_pages_come_back_and_are_used_again():
    m = manager(num_pages=6, page=4, needs=[PagedKV(1, 16, window=6), PagedKV(1, 16)])
    win = [g.index for g in m.groups if g.window == 6][0]
    full = 1 - win
    for step in range(5):
        m.append("a", 4)
        m.commit("a")
    # 20 positions: the next query (position 20) reads positions 15..20 -> pages 3.. stay
    assert m.block_table("a", win) == [-1, -1, -1, 3, 4]
    assert m.block_table("a", full) == [0, 1, 2, 3, 4]
    assert m.free_pages()[win] == 4 and m.free_pages()[full] == 1
    m.append("a", 4)
    m.commit("a")
    assert m.block_table("a", win)[-1] == 5 and m.block_table("a", win)[3] == -1
    m.append("b", 1) if m.can_append("b", 1) else None
    m.check()
    m.release("a")
    m.check()


def test_random_orders_keep_the_books_straight():
    rng = random.Random(3)
    m = manager(num_pages=24, page=4, slots=4,
                needs=[PagedKV(1, 16), FixedState((2, 4)), PagedKV(1, 16, window=9)])
    live, next_id = {}, 0
    for _ in range(3000):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            rid = f"r{next_id}"
            next_id += 1
            n = rng.randint(1, 30)
            if m.can_append(rid, n):
                m.append(rid, n)
                m.commit(rid)
                live[rid] = n
            else:
                with pytest.raises(OutOfPages):
                    m.append(rid, n)
                assert not m.has(rid)
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 13])
            if m.can_append(rid, n):
                assert m.append(rid, n) == live[rid]
                if rng.random() < 0.05:
                    m.cancel(rid)  # the step failed: nothing moves forward
                else:
                    m.commit(rid)
                    live[rid] += n
            else:
                before = (m.free_pages(), m.length(rid))
                with pytest.raises(OutOfPages):
                    m.append(rid, n)
                assert (m.free_pages(), m.length(rid)) == before
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.length(rid) == n
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(f == 24 for f in m.free_pages()) and m.slots.free_slots == 4
