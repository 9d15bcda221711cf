"""CPU tests of the page allocator and the incremental decode lease.  They pin the behaviours the
reference's tests pin (tests/test_cache_layout.py:13-68, tests/test_prepared_layout.py:6-30):
atomic planning, stale plans, LIFO page reuse, page math for non-dividing sizes, and equivalence of
the incremental lease with the transactional allocator."""
import pytest

from moba_opt.cache_layout import IncrementalLayout, PageAllocator


def snapshot(a):
    return a.tables, a.lengths, a.free_pages, a.version


def test_planning_is_side_effect_free_and_commit_is_versioned():
    a = PageAllocator(2, 17, 3, 12, 4)
    before = snapshot(a)
    plan = a.plan_append([1, 0], [5, 7])
    assert snapshot(a) == before
    assert plan.token_sequences == (1,) * 5 + (0,) * 7
    assert plan.token_positions == tuple(range(5)) + tuple(range(7))
    assert plan.completed_chunks == ((1, 0), (0, 0))
    a.commit(plan)
    assert a.lengths == (7, 5)
    assert a.tables[1][:2] == (0, 1) and a.tables[0][:3] == (2, 3, 4)   # page 0 is handed out first
    with pytest.raises(RuntimeError, match="stale"):
        a.commit(plan)


def test_released_pages_are_reused_last_in_first_out():
    a = PageAllocator(3, 12, 3, 4, 4)
    a.commit(a.plan_append([0, 1], [6, 3]))
    a.reset([0])
    a.commit(a.plan_append([2], [6]))
    assert a.tables[2][:2] == (1, 0)
    assert a.tables[1][0] == 2
    assert len(a.free_pages) == 1


@pytest.mark.parametrize("ids,counts", [([1], [1]), ([0], [20]), ([0, 0], [1, 1]), ([2], [1]), ([0], [0]), ([0], [True]),
                                        ([0.5], [1]), ([], [])])
def test_rejected_appends_leave_state_untouched(ids, counts):
    a = PageAllocator(2, 12, 3, 2, 4)
    a.commit(a.plan_append([0], [4]))
    before = snapshot(a)
    with pytest.raises(ValueError):
        a.plan_append(ids, counts)
    assert snapshot(a) == before


def test_pool_exhaustion_message():
    a = PageAllocator(2, 12, 3, 2, 4)
    a.commit(a.plan_append([0], [4]))
    with pytest.raises(ValueError, match="pool exhausted"):
        a.plan_append([1], [1])
    with pytest.raises(ValueError, match="max_seq_len"):
        a.plan_append([0], [20])


def test_completed_chunks_follow_logical_positions():
    a = PageAllocator(1, 20, 3, 7, 4)
    a.commit(a.plan_append([0], [3]))
    p = a.plan_append([0], [6])
    assert p.completed_chunks == ((0, 0), (0, 1))
    a.commit(p)
    assert a.plan_append([0], [1]).completed_chunks == ()


@pytest.mark.parametrize("page", [1, 3, 7, 16, 31, 48])
def test_page_accounting_for_sizes_that_do_not_divide(page):
    a = PageAllocator(2, 65, page, 2 * ((65 + page - 1) // page), 24)
    a.commit(a.plan_append([0, 1], [65, 33]))
    owned = [x for row in a.tables for x in row if x >= 0]
    assert len(owned) == len(set(owned))
    assert len(owned) + len(a.free_pages) == a.num_pages
    a.reset([0, 1])
    assert len(a.free_pages) == a.num_pages and a.lengths == (0, 0)


def test_int32_capacity_guard():
    with pytest.raises(ValueError, match="int32"):
        PageAllocator(1, 2 ** 30, 16, 4, 8)
    with pytest.raises(ValueError, match="int32"):
        PageAllocator(1, 64, 2 ** 16, 2 ** 15, 8)


@pytest.mark.parametrize("page", [1, 3, 7, 16])
def test_incremental_lease_equals_transactional_allocator(page):
    old = PageAllocator(3, 41, page, 3 * ((41 + page - 1) // page), 8)
    old.commit(old.plan_append([1, 0], [5, 7]))
    old.reset([1])
    fast = IncrementalLayout(old, [2, 0, 1])
    for _ in range(30):
        plan = fast.plan()
        before = (tuple(map(tuple, fast.tables)), tuple(fast.lengths), tuple(fast.free))
        assert fast.plan() == plan
        assert before == (tuple(map(tuple, fast.tables)), tuple(fast.lengths), tuple(fast.free))
        fast.commit(plan)
        old.commit(old.plan_append([2, 0, 1], [1, 1, 1]))
        assert tuple(map(tuple, fast.tables)) == old.tables
        assert tuple(fast.lengths) == old.lengths and tuple(fast.free) == old.free_pages
    fast.publish(old)
    assert old.lengths == (37, 30, 30)
    with pytest.raises(RuntimeError, match="stale"):
        fast.commit(plan)


def test_incremental_failures_do_not_mutate():
    old = PageAllocator(2, 4, 2, 1, 2)
    old.commit(old.plan_append([0], [2]))
    fast = IncrementalLayout(old, [0, 1])
    with pytest.raises(ValueError, match="pool exhausted"):
        fast.plan()
    assert fast.lengths == [2, 0] and fast.free == []
    old = PageAllocator(1, 1, 1, 1, 1)
    old.commit(old.plan_append([0], [1]))
    with pytest.raises(ValueError, match="max_seq_len"):
        IncrementalLayout(old, [0]).plan()


@pytest.mark.parametrize("page", [3, 4, 7])
def test_plan_without_token_lists_is_the_same_plan(page):
    """A whole-prompt append (append_prefill) plans without the per-token (sequence, position) lists; everything else
    of the plan - tables, lengths, pool, completed chunks - is what the full plan gives."""
    a = PageAllocator(3, 40, page, 40, 8)
    a.commit(a.plan_append([2], [5]))
    full = a.plan_append([0, 2, 1], [13, 9, 1])
    light = a.plan_append([0, 2, 1], [13, 9, 1], tokens=False)
    assert light.token_sequences == () and light.token_positions == ()
    assert len(full.token_sequences) == 23
    for field in ("version", "tables", "lengths", "free_pages", "completed_chunks"):
        assert getattr(full, field) == getattr(light, field)
    a.commit(light)
    assert a.lengths == (13, 1, 14)
