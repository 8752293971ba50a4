"""The cache manager's books (no GPU): pages, block tables, groups, windows, state slots."""
import random

import pytest

from sglang_rs_b200.cache import CacheManager, OutOfPages, OutOfStateSlots, PageAllocator
from sglang_rs_b200.parts import PagedKV, RequestState

FULL = ("kv", None)


def manager(needs=None, page_size=4, max_tokens=32, max_requests=4, **kw):
    needs = needs if needs is not None else [PagedKV(2, 16), PagedKV(2, 16)]
    return CacheManager(needs, page_size=page_size, max_tokens=max_tokens, max_requests=max_requests, device=None, **kw)


def test_allocator_reuses_returned_pages_first_and_refuses_double_free():
    pages = PageAllocator(4)
    got = pages.allocate(3)
    assert got == [0, 1, 2] and pages.free_count == 1
    assert pages.release(1) is True
    assert pages.allocate(1) == [1]                       # a page that came back is used again first
    with pytest.raises(OutOfPages) as error:
        pages.allocate(2)
    assert (error.value.requested, error.value.available) == (2, 1) and pages.free_count == 1   # nothing consumed
    pages.retain(0)
    assert pages.release(0) is False and pages.release(0) is True
    with pytest.raises(RuntimeError, match="freed twice"):
        pages.release(0)


def test_requests_never_share_a_partly_filled_page_and_fill_their_tail_first():
    cache = manager()
    a, b = cache.open("a"), cache.open("b")
    cache.reserve(a, 5); cache.commit(a, 5)               # 2 pages, the second holds one token
    cache.reserve(b, 1); cache.commit(b, 1)
    assert len(a.tables[FULL]) == 2 and len(b.tables[FULL]) == 1
    assert not set(a.tables[FULL]) & set(b.tables[FULL])
    before = list(a.tables[FULL])
    cache.reserve(a, 3); cache.commit(a, 3)               # fills the tail page, takes no new one
    assert a.tables[FULL] == before
    cache.reserve(a, 1); cache.commit(a, 1)
    assert len(a.tables[FULL]) == 3
    assert cache.slot_of(a, FULL, 5) == a.tables[FULL][1] * 4 + 1
    cache.check_invariants()


def test_failed_reservation_changes_nothing_and_close_returns_everything():
    cache = manager(max_tokens=16)                         # 4 pages
    a, b = cache.open("a"), cache.open("b")
    cache.reserve(a, 9); cache.commit(a, 9)                # 3 pages
    with pytest.raises(OutOfPages):
        cache.reserve(b, 8)
    assert b.tables[FULL] == [] and cache.free_pages()[FULL] == 1
    assert cache.can_reserve(b, 4) and not cache.can_reserve(b, 5)
    cache.close(a)
    assert cache.free_pages()[FULL] == 4
    with pytest.raises(RuntimeError, match="ended twice"):
        cache.close(a)
    cache.reserve(b, 16); cache.commit(b, 16)
    cache.check_invariants()


def test_trim_gives_back_what_a_step_that_did_not_run_had_reserved():
    cache = manager()
    a = cache.open("a")
    cache.reserve(a, 6); cache.commit(a, 6)
    cache.reserve(a, 10)
    assert len(a.tables[FULL]) == 4
    cache.trim_reservation(a)
    assert len(a.tables[FULL]) == 2 and a.length == 6
    cache.check_invariants()


def test_window_group_has_its_own_pages_and_gives_them_back_as_the_window_passes():
    needs = [PagedKV(2, 16), PagedKV(2, 16, window=6), PagedKV(1, 32, window=6), PagedKV(2, 16)]
    cache = manager(needs, page_size=4, max_tokens=64)
    window = ("kv", 6)
    assert set(cache.allocators) == {FULL, window}
    assert cache.layer_caches[1].group == window and cache.layer_caches[3].group == FULL
    a = cache.open("a")
    for step in range(10):
        cache.reserve(a, 3); cache.commit(a, 3)
        kept_from = max(0, a.length - 6 + 1)
        table = a.tables[window]
        for logical, page in enumerate(table):
            assert (page == -1) == ((logical + 1) * 4 <= kept_from), (step, logical)
        assert all(page >= 0 for page in a.tables[FULL])
        cache.check_invariants()
    assert cache.free_pages()[window] == 16 - 2            # only the pages the window still touches
    with pytest.raises(RuntimeError, match="given back"):
        cache.slot_of(a, window, 0)
    cache.close(a)
    assert cache.free_pages() == {FULL: 16, window: 16}


def test_state_slots_and_live_limit():
    """The slots of the cache manager's own books (C++), through the manager: one per live request, the one
    given back last is handed out next, a request cannot end twice, and under random openings and
    closings no slot is ever held by two live requests or lost."""
    cache = manager([RequestState((3, 5)), PagedKV(2, 16)], max_requests=2)
    a, b = cache.open("a"), cache.open("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(OutOfStateSlots):
        cache.open("c")
    with pytest.raises(ValueError, match="already live"):
        cache.open("a")
    cache.close(a)
    with pytest.raises(RuntimeError, match="ended twice"):
        cache.close(a)
    assert cache.state_pool.free_count == 1
    c = cache.open("c")
    assert c.state_slot == a.state_slot
    cache.check_invariants()
    cache.close(b); cache.close(c)
    assert cache.state_pool.free_count == cache.state_pool.capacity == 2

    import random
    rng = random.Random(4)
    cache = manager([RequestState((2,)), PagedKV(2, 16)], max_requests=5)
    live = {}
    for step in range(400):
        if live and (len(live) == 5 or rng.random() < 0.45):
            name = rng.choice(sorted(live))
            cache.close(live.pop(name))
        else:
            live[f"r{step}"] = cache.open(f"r{step}")
        slots = [handle.state_slot for handle in live.values()]
        assert len(set(slots)) == len(slots) and all(0 <= slot < 5 for slot in slots)
        assert cache.state_pool.free_count == 5 - len(live)
    cache.check_invariants()


def test_shared_prefix_pages_are_counted():
    cache = manager(max_tokens=32)
    a = cache.open("a")
    cache.reserve(a, 10); cache.commit(a, 10)
    b = cache.open("b")
    cache.adopt_prefix(b, FULL, a.tables[FULL][:2])
    assert b.length == 8 and b.shared_prefix_pages == 2
    cache.reserve(b, 3); cache.commit(b, 3)
    assert b.tables[FULL][2] != a.tables[FULL][2]          # the partly filled page is private
    cache.check_invariants()
    cache.close(a)
    assert cache.allocators[FULL].refcount(b.tables[FULL][0]) == 1
    cache.check_invariants()
    cache.close(b)
    assert cache.free_pages()[FULL] == 8


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    needs = [PagedKV(2, 16), PagedKV(2, 16, window=10), RequestState((4,))]
    cache = manager(needs, page_size=4, max_tokens=rng.choice([24, 40, 64]), max_requests=4)
    live = {}
    counter = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            counter += 1
            live[counter] = cache.open(counter)
        elif action < 0.85 and live:
            handle = live[rng.choice(list(live))]
            tokens = rng.choice([1, 1, 1, 2, 3, 7, 13])
            try:
                cache.reserve(handle, tokens)
            except OutOfPages:
                victim = rng.choice(list(live))
                cache.close(live.pop(victim))
            else:
                if rng.random() < 0.1:
                    cache.trim_reservation(handle)         # the step did not run
                else:
                    cache.commit(handle, tokens)
        elif live:
            cache.close(live.pop(rng.choice(list(live))))
        cache.check_invariants()
    for handle in list(live.values()):
        cache.close(handle)
    cache.check_invariants()
    assert all(a.free_count == a.num_pages for a in cache.allocators.values())
    assert cache.state_pool.free_count == 4
