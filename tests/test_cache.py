"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of requests;
groups with a window give pages back as the window passes them; state slots."""
import random

import pytest
import torch

from zedinfer_b200.cache import (CacheManager, OutOfPages, PagedKVNeed, PagePool, StateNeed, StateSlotPool)


def test_pool_is_lifo_and_guards_misuse():
    p = PagePool(4)
    a, b = p.allocate(), p.allocate()
    assert (a, b) == (0, 1) and p.num_free == 2 and p.num_used == 2
    p.free(a)
    assert p.allocate() == a                      # the page just given back is handed out next
    with pytest.raises(ValueError, match="twice"):
        p.free(3)                                 # never handed out
    p.free(b)
    with pytest.raises(ValueError, match="twice"):
        p.free(b)
    with pytest.raises(ValueError, match="not of this pool"):
        p.free(9)
    p.allocate_many(3)
    with pytest.raises(OutOfPages):
        p.allocate()
    with pytest.raises(OutOfPages):
        p.allocate_many(1)
    p.check()


def test_state_slots():
    s = StateSlotPool(2)
    a, b = s.acquire_slot(), s.acquire_slot()
    assert s.num_free_slots == 0
    with pytest.raises(OutOfPages):
        s.acquire_slot()
    s.release_slot(a)
    with pytest.raises(ValueError):
        s.release_slot(a)
    assert s.acquire_slot() == a
    s.check()
    assert StateSlotPool(0).num_free_slots == 0


def manager(page_size=4, pages=16, window=None, max_requests=4):
    needs = [(0, PagedKVNeed(2, 16, None)), (1, PagedKVNeed(2, 16, window)), (2, PagedKVNeed(2, 16, None))]
    m = CacheManager(needs, page_size, max_requests=max_requests)
    m.set_num_pages(pages)
    return m


def test_groups_follow_page_shape_and_window():
    m = manager(window=None)
    assert len(m.groups) == 1 and m.groups[0].calls == [0, 1, 2]
    m = manager(window=8)
    assert len(m.groups) == 2 and m.groups[0].calls == [0, 2] and m.groups[1].calls == [1]
    v0, v1 = m.view_for_call(0), m.view_for_call(1)
    assert (v0.group, v1.group) == (0, 1) and v1.window == 8 and v0.window is None
    assert v0.page_stride == 2 * 2 * 2 * 4 * 16 and v0.kv_stride == 2 * 4 * 16
    assert m.view_for_call(7).kind == "none"


def test_ensure_is_all_or_nothing_and_close_returns_everything():
    m = manager(pages=5, window=8)
    a = m.open("a")
    m.ensure(a, 10)                               # 3 pages in each group
    assert [len(t) for t in a.tables] == [3, 3] and m.free_pages() == [2, 2]
    b = m.open("b")
    with pytest.raises(OutOfPages):
        m.ensure(b, 9)                            # would need 3
    assert b.tables == [[], []] and m.free_pages() == [2, 2]
    m.ensure(b, 8)
    m.check()
    assert m.pages_needed(a, 13) == [1, 1] and not m.can_ensure(a, 13)
    m.close(a)
    assert m.free_pages() == [3, 3] and m.can_ensure(b, 13)
    with pytest.raises(ValueError, match="twice"):
        m.close(a)
    with pytest.raises(RuntimeError, match="closed"):
        m.ensure(a, 4)
    m.close(b)
    assert m.free_pages() == [5, 5] and m.num_live == 0
    m.check()


def test_window_gives_pages_back_as_it_passes():
    m = manager(page_size=4, pages=32, window=6)
    r = m.open("r")
    m.ensure(r, 20)
    m.commit(r, 20)
    # the next query sits at position >= 20 and reads keys from 15 on: blocks 0..2 (tokens 0..11) are dead
    assert r.tables[1][:3] == [-1, -1, -1] and all(p >= 0 for p in r.tables[1][3:])
    assert all(p >= 0 for p in r.tables[0])                       # the full-attention group keeps everything
    assert m.free_pages() == [32 - 5, 32 - 2]
    m.ensure(r, 21)
    m.commit(r, 21)                                               # first needed token 16 -> block 3 now dead too
    assert r.tables[1][:4] == [-1] * 4 and len(r.tables[1]) == 6
    m.check()
    m.close(r)
    assert m.free_pages() == [32, 32]


def test_state_slots_limit_admission():
    needs = [(0, PagedKVNeed(1, 16, None)), (1, StateNeed((3, 5)))]
    m = CacheManager(needs, 4, max_requests=2)
    m.set_num_pages(8)
    a, b = m.open("a"), m.open("b")
    assert {a.slot, b.slot} == {0, 1} and not m.can_open()
    with pytest.raises(OutOfPages):
        m.open("c")
    slot_of_a = a.slot
    m.close(a)
    assert m.can_open() and m.open("c").slot == slot_of_a
    assert m.view_for_call(1).kind == "state"
    with pytest.raises(ValueError, match="already live"):
        m.open("c")


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    m = manager(page_size=rng.choice([2, 4, 8]), pages=rng.choice([6, 13, 40]), window=rng.choice([None, 5, 17]),
                max_requests=5)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            live[next_id] = m.open(next_id)
            next_id += 1
        elif op < 0.8 and live:
            rc = live[rng.choice(list(live))]
            new_len = rc.length + rng.choice([1, 1, 1, 2, 5, 9, 23])
            try:
                m.ensure(rc, new_len)
                m.commit(rc, new_len)
            except OutOfPages:
                before = [list(t) for t in rc.tables]
                assert before == rc.tables
        elif live:
            rid = rng.choice(list(live))
            m.close(live.pop(rid))
        m.check()
        for g in m.groups:
            assert g.pool.num_free + g.pool.num_used == g.pool.num_pages
    for rc in live.values():
        m.close(rc)
    m.check()
    assert all(g.pool.num_used == 0 for g in m.groups) and m.num_live == 0


def test_budget_to_pages():
    m = CacheManager([(i, PagedKVNeed(2, 128, None)) for i in range(28)], 16)
    per_page = 28 * 2 * 2 * 16 * 128 * 2
    assert m.bytes_per_page_all_groups(torch.bfloat16) == per_page
    assert m.pages_for_budget(per_page * 101, torch.bfloat16) == 100      # one page is the scratch page


def test_a_reopened_request_id_is_another_request():
    """Captured decode steps skip the upload of a row's block table while (request id, serial, version) is unchanged.
    An id that is closed and opened again (preemption does that) starts at version 0 again, so the serial must
    differ, or the row would keep the old request's pages."""
    m = CacheManager([(0, PagedKVNeed(2, 16))], page_size=4)
    m.set_num_pages(8)
    a = m.open("x")
    m.ensure(a, 6)
    first = (a.request_id, a.serial, a.version)
    m.close(a)
    b = m.open("x")
    m.ensure(b, 6)
    assert (b.request_id, b.version) == (first[0], first[2]) and b.serial != first[1]
    assert (b.request_id, b.serial, b.version) != first


def test_state_can_be_reset_and_copied_between_requests():
    m = CacheManager([(0, StateNeed((3,), torch.float32)), (2, StateNeed((2, 2), torch.float32))], page_size=4, max_requests=3)
    m.allocate_device(4, torch.float32, "cpu")
    a, b = m.open("a"), m.open("b")
    va, vb = m.view_for_call(0).tensor, m.view_for_call(2).tensor
    va[a.slot] += 5.0
    vb[a.slot] += 7.0
    m.copy_state(a, b)
    assert float(va[b.slot].sum()) == 15.0 and float(vb[b.slot].sum()) == 28.0
    m.reset_state(a)
    assert float(va[a.slot].abs().sum()) == 0.0 and float(vb[a.slot].abs().sum()) == 0.0
    assert float(va[b.slot].sum()) == 15.0
    m.close(a)
    c = m.open("c")                      # takes a's slot: zeroed when it opens
    assert c.slot == 0 or float(va[c.slot].abs().sum()) == 0.0
    m.check()


def test_a_group_with_a_window_gets_a_smaller_pool_when_steps_are_bounded():
    """With a bound on the tokens a step adds to a request, a group of layers with a window holds at most window + bound
    tokens of a request, so max_requests requests can never fill more than that many pages: its pool is cut to that,
    its scratch page is its own, and a byte budget buys the other groups more pages."""
    needs = [(0, PagedKVNeed(2, 16, None)), (1, PagedKVNeed(2, 16, 32)), (2, PagedKVNeed(2, 16, None))]
    m = CacheManager(needs, 8, max_requests=3, max_step_tokens=16)
    per_request = (32 + 16 + 8 - 2) // 8 + 1                       # 7 pages: 47 tokens starting anywhere in a page
    m.set_num_pages(100)
    assert [g.num_pages for g in m.groups] == [100, 3 * per_request] and m.scratch_pages == [100, 21]
    assert m.free_pages() == [100, 21]
    m.set_num_pages(10)                                            # never more than the others
    assert [g.num_pages for g in m.groups] == [10, 10]
    unbounded = CacheManager(needs, 8, max_requests=3)
    unbounded.set_num_pages(100)
    assert [g.num_pages for g in unbounded.groups] == [100, 100]
    # the budget: the largest count whose pools (one scratch page each) fit
    for budget in (10_000, 123_456, 5_000_000):
        n = m.pages_for_budget(budget, torch.bfloat16)
        assert m.pool_bytes(n, torch.bfloat16) <= budget < m.pool_bytes(n + 1, torch.bfloat16)
        assert n >= unbounded.pages_for_budget(budget, torch.bfloat16)
    assert m.pages_for_budget(5_000_000, torch.bfloat16) > unbounded.pages_for_budget(5_000_000, torch.bfloat16)


@pytest.mark.parametrize("seed", range(5))
def test_the_smaller_pool_of_a_windowed_group_never_runs_out_first(seed):
    """Random requests in random portions of at most max_step_tokens, max_requests at a time: whenever a step is
    refused for lack of pages, it is the group that keeps all keys that ran out."""
    rng = random.Random(seed)
    page, window, bound, live_max = 4, 10, 7, 3
    m = CacheManager([(0, PagedKVNeed(1, 8, None)), (1, PagedKVNeed(1, 8, window))], page, max_requests=live_max,
                     max_step_tokens=bound)
    m.set_num_pages(60)
    assert m.groups[1].num_pages < 60
    live, serial = {}, 0
    for _ in range(600):
        if len(live) < live_max and rng.random() < 0.3:
            serial += 1
            live[serial] = (m.open(serial), rng.randrange(1, 120))
        if not live:
            continue
        rid = rng.choice(list(live))
        rc, total = live[rid]
        n = min(rng.randrange(1, bound + 1), total - rc.length)
        needed = m.pages_needed(rc, rc.length + n)
        if m.can_ensure(rc, rc.length + n):
            m.ensure(rc, rc.length + n)
            m.commit(rc, rc.length + n)
        else:
            assert needed[0] > m.groups[0].pool.num_free and needed[1] <= m.groups[1].pool.num_free
            m.close(rc)
            del live[rid]
            continue
        if rc.length == total:
            m.close(rc)
            del live[rid]
        m.check()
    for rc, _ in list(live.values()):
        m.close(rc)
    assert m.free_pages() == [60, m.groups[1].num_pages]


def test_a_windowed_group_under_a_step_bound_takes_pages_only_as_far_as_the_next_step_reaches():
    """A whole prompt reserved at admission takes all its pages in the groups that keep all keys, and in a group with
    a window only those that the next step can write; the rest come step by step as the window gives pages back."""
    m = CacheManager([(0, PagedKVNeed(1, 8, None)), (1, PagedKVNeed(1, 8, 12))], 4, max_requests=2, max_step_tokens=8)
    m.set_num_pages(50)
    assert [g.num_pages for g in m.groups] == [50, 2 * ((12 + 8 + 2) // 4 + 1)]       # 12 pages for the window's group
    rc = m.open("long")
    assert m.pages_needed(rc, 100) == [25, 2] and m.can_ensure(rc, 100)
    m.ensure(rc, 100)                                   # far more tokens than the windowed pool could ever hold
    assert [len(t) for t in rc.tables] == [25, 2]
    done = 0
    while done < 100:                                   # the prompt in steps of 8, each asking for its own tokens
        n = min(8, 100 - done)
        m.ensure(rc, done + n)
        assert all(len(t) * 4 >= done + n for t in rc.tables)
        m.commit(rc, done + n)
        done += n
        assert sum(1 for p in rc.tables[1] if p >= 0) <= (12 + 8 + 2) // 4 + 1
        m.check()
    other = m.open("second")
    m.ensure(other, 8)
    with pytest.raises(RuntimeError, match="2 requests are live"):
        m.open("third")
    m.close(rc), m.close(other)
    assert m.free_pages() == [50, 12]
