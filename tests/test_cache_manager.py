"""Cache manager accounting without a GPU: no page lost, held twice or freed twice, under
random orders of requests; windows give pages back; out-of-pages changes nothing.
Mirrors pulsar-core/tests/runtime/test_scheduler.cpp:103-188 (allocator accounting, page
boundary append, out of memory, slot mapping) and extends it to groups and windows."""
import random

import pytest

from pulsar_b200.cache import CacheError, CacheManager, CacheNeed, OutOfPages, PageAllocator


def manager(pages=8, page=4, window=None, max_requests=4, two_groups=False):
    needs = [CacheNeed.paged_kv(2, 16), CacheNeed.paged_kv(2, 16)]
    if two_groups:
        needs += [CacheNeed.paged_kv(2, 16, window), CacheNeed.paged_kv(2, 16, window)]
    elif window is not None:
        needs = [CacheNeed.paged_kv(2, 16, window)]
    return CacheManager(needs, page, pages, max_requests)


def test_allocator_is_lifo_and_refuses_double_free():
    a = PageAllocator(3)
    assert [a.take(), a.take(), a.take()] == [0, 1, 2]        # a fresh pool yields 0, 1, 2
    with pytest.raises(OutOfPages):
        a.take()
    a.give(1)
    a.give(0)
    assert a.take() == 0 and a.take() == 1                    # most recently freed first
    a.give(2)
    with pytest.raises(CacheError, match="freed twice"):
        a.give(2)
    with pytest.raises(CacheError):
        a.give(7)


def test_groups_are_formed_by_equal_needs():
    m = manager(two_groups=True, window=8)
    assert len(m.groups) == 2 and m.groups[0].entries == [0, 1] and m.groups[1].entries == [2, 3]
    assert m.group_of_entry == {0: 0, 1: 0, 2: 1, 3: 1}
    m2 = CacheManager([CacheNeed.paged_kv(2, 16), CacheNeed.state((3, 5)), CacheNeed.none(), CacheNeed.paged_kv(4, 16)], 4,
                      [8, 6], 2)
    assert [g.allocator.n for g in m2.groups] == [8, 6]
    with pytest.raises(CacheError):
        CacheManager([CacheNeed.paged_kv(2, 16)], 4, [8, 6], 2)


def test_append_across_page_boundaries_and_slots():
    m = manager(pages=8, page=4)
    m.open("a")
    assert m.append("a", 3) == 0 and m.table("a", 0) == [0]
    assert m.pages_to_append("a", 1) == [0] and m.pages_to_append("a", 2) == [1]
    assert m.append("a", 2) == 3 and m.table("a", 0) == [0, 1] and m.length("a") == 5
    m.open("b")
    m.append("b", 9)
    assert m.table("b", 0) == [2, 3, 4]
    assert m.slots("a", 0, 2, 3) == [2, 3, 4] and m.slots("b", 0, 7, 2) == [3 * 4 + 3, 4 * 4 + 0]
    m.check_consistency()
    m.close("a")
    m.open("c")
    m.append("c", 5)
    assert m.table("c", 0) == [1, 0]          # freed pages are used again, most recently freed first
    m.check_consistency()


def test_out_of_pages_changes_nothing():
    m = manager(pages=3, page=4)
    m.open("a")
    m.append("a", 8)
    m.open("b")
    before = (m.n_free_pages(), m.length("b"), list(m.table("b", 0)))
    assert not m.can_append("b", 5) and m.can_append("b", 4)
    with pytest.raises(OutOfPages):
        m.append("b", 5)
    assert (m.n_free_pages(), m.length("b"), list(m.table("b", 0))) == before
    m.append("b", 4)
    assert m.n_free_pages() == [0] and not m.can_admit(1)
    m.check_consistency()


def test_state_slots_run_out_and_come_back():
    m = manager(max_requests=2)
    assert m.open("a") == 0 and m.open("b") == 1
    with pytest.raises(OutOfPages, match="state slot"):
        m.open("c")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    m.close("a")
    assert m.open("c") == 0
    with pytest.raises(CacheError, match="unknown"):
        m.close("zzz")


def test_window_gives_pages_back_once_every_query_has_passed_them():
    m = manager(pages=6, page=4, window=6)
    m.open("a")
    m.append("a", 4)                         # keys 0..3 in page 0
    m.append("a", 4)                         # length 8: the next query (position 8) sees keys 3..8: page 0 still needed
    assert m.table("a", 0) == [0, 1] and m.n_free_pages() == [4]
    m.append("a", 1)                         # length 9; before growing, position 8's window starts at key 3
    assert m.table("a", 0)[0] == 0
    m.append("a", 1)                         # now length 9 -> next query 9 sees keys 4..9: page 0 is passed
    assert m.table("a", 0)[0] == -1 and m.n_free_pages() == [4]    # gave one back, took none (page 2 has room)
    with pytest.raises(CacheError, match="released"):
        m.slots("a", 0, 2, 1)
    for _ in range(30):                      # a long decode never holds more than window/page + 2 pages
        m.append("a", 1)
        assert sum(p >= 0 for p in m.table("a", 0)) <= 6 // 4 + 2
        m.check_consistency()
    m.close("a")
    assert m.n_free_pages() == [6]


def test_groups_with_and_without_window_share_one_request():
    m = manager(pages=10, page=4, window=5, two_groups=True)
    m.open("a")
    m.append("a", 20)
    m.append("a", 1)
    assert sum(p >= 0 for p in m.table("a", 0)) == 6 and sum(p >= 0 for p in m.table("a", 1)) < 6
    m.check_consistency()
    m.close("a")
    assert m.n_free_pages() == [10, 10]


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 7])
def test_random_orders_of_requests(seed, window):
    rng = random.Random(seed)
    m = manager(pages=12, page=4, window=window, max_requests=5, two_groups=window is not None)
    live, next_id, shadow = [], 0, {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{next_id}"
            next_id += 1
            m.open(rid)
            live.append(rid)
            shadow[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(live)
            n = rng.randint(1, 9)
            if m.can_append(rid, n):
                assert m.append(rid, n) == shadow[rid]
                shadow[rid] += n
                # the newest positions always have slots, and no two live tokens share one
                for g in range(len(m.groups)):
                    assert len(m.slots(rid, g, shadow[rid] - n, n)) == n
            else:
                before = m.n_free_pages()
                with pytest.raises(OutOfPages):
                    m.append(rid, n)
                assert m.n_free_pages() == before
        elif live:
            rid = live.pop(rng.randrange(len(live)))
            m.close(rid)
            del shadow[rid]
        m.check_consistency()
        for g in range(len(m.groups)):
            slots = [s for rid in live for s in m.slots(rid, g, max(0, shadow[rid] - 3), min(3, shadow[rid]))]
            assert len(slots) == len(set(slots))
    for rid in live:
        m.close(rid)
    m.check_consistency()
    assert all(f == 12 for f in m.n_free_pages()) and m.n_free_slots() == 5
