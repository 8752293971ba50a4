"""The prefix tree and its use by the cache manager and the scheduler (no GPU)."""
import random

import pytest

from sglang_rs_b200.cache import CacheManager, PageAllocator, PrefixTree
from sglang_rs_b200.parts import PagedKV, RequestState
from test_scheduler import drain, expected_output, make, request, run_step

FULL = ("kv", None)


def test_match_is_by_whole_pages_and_leaves_a_token_to_compute():
    pages = PageAllocator(16)
    tree = PrefixTree(4, pages)
    tokens = list(range(100, 114))                        # 14 tokens: 3 full pages
    mine = pages.allocate(4)
    assert tree.insert(tokens, mine) == 3                 # the partly filled fourth page stays private
    assert tree.pages_held == 3 and pages.refcount(mine[0]) == 2 and pages.refcount(mine[3]) == 1
    assert tree.match(tokens) == mine[:3]
    assert tree.match(tokens[:12]) == mine[:2]            # all 12 are known: one page is computed again
    assert tree.match(tokens[:13]) == mine[:3]
    assert tree.match(tokens[:5] + [7] + tokens[6:]) == mine[:1]
    assert tree.match([1, 2, 3]) == [] and tree.match(tokens[:4]) == []
    # the same tokens under other page ids are not taken twice
    again = pages.allocate(3)
    assert tree.insert(tokens, again) == 0 and pages.refcount(again[0]) == 1


def test_eviction_takes_unshared_leaves_least_recently_used_first():
    pages = PageAllocator(16)
    tree = PrefixTree(2, pages)
    a, b = pages.allocate(3), pages.allocate(2)
    tree.insert([1, 2, 3, 4, 5, 6], a)
    tree.insert([1, 2, 9, 9], [a[0], b[1]])               # shares the first page, adds one
    for page in a + b:
        pages.release(page)                               # the requests have ended
    assert pages.free_count == 16 - 4 and tree.evictable() == 4
    tree.match([1, 2, 3, 4, 5, 6, 0])                      # touches the first branch
    assert tree.evict(1) == 1 and b[1] not in tree.pages()      # the branch used longer ago goes first
    held = pages.allocate(1)                               # somebody takes a page: unrelated
    pages.retain(a[1])                                     # a request holds the middle page of the branch
    assert tree.evict(10) == 1                             # only the leaf can go; its parent is held, the root page is a parent
    assert set(tree.pages()) == {a[0], a[1]}
    pages.release(a[1])
    assert tree.evict(10) == 2 and tree.pages() == [] and pages.free_count == 15
    pages.release(held[0])
    tree.clear()
    assert pages.free_count == 16


def test_manager_reclaims_cached_pages_before_it_refuses():
    cache = CacheManager([PagedKV(2, 16)], page_size=4, max_tokens=32, max_requests=4, device=None)
    tree = cache.enable_prefix_reuse()
    a = cache.open("a")
    cache.reserve(a, 24); cache.commit(a, 24)
    tree.insert(list(range(24)), a.tables[FULL])
    cache.close(a)
    assert cache.allocators[FULL].free_count == 2 and cache.free_pages()[FULL] == 8
    cache.check_invariants()
    b = cache.open("b")
    assert cache.can_reserve(b, 30)
    cache.reserve(b, 30); cache.commit(b, 30)              # needs all 8 pages: the cached ones are evicted
    assert tree.pages_held == 0
    cache.check_invariants()
    cache.close(b)
    with pytest.raises(ValueError):
        CacheManager([PagedKV(2, 16, window=8)], page_size=4, max_tokens=32, max_requests=2, device=None).enable_prefix_reuse()
    assert not CacheManager([PagedKV(2, 16), RequestState((4,))], page_size=4, max_tokens=32, max_requests=2,
                            device=None).prefix_reuse_possible()


def test_scheduler_reuses_prefixes_counts_them_and_keeps_the_tokens_right():
    scheduler, cache = make(max_tokens=256, page_size=8, budget=16)
    cache.enable_prefix_reuse()
    base = list(range(40))
    first = request("first", base, max_new_tokens=4)
    scheduler.add_request(first)
    drain(scheduler, cache)
    second = request("second", base[:24] + [90, 91, 92, 93, 94], max_new_tokens=4)
    whole = request("whole", base, max_new_tokens=4)
    scheduler.add_request(second)
    scheduler.add_request(whole)
    log = []
    drain(scheduler, cache, log=log)
    assert (first.cached_tokens, second.cached_tokens, whole.cached_tokens) == (0, 24, 32)
    assert log[0] == [("second", 5, True), ("whole", 8, True)]      # only what is not cached is computed
    for r in (first, second, whole):
        assert r.output_ids == expected_output(r.prompt, 4)
    cache.check_invariants()
    assert cache.prefix_tree.pages_held == 5 + 0 and cache.free_pages()[FULL] == 32
    # 27 pages are free and the tree could give up its 5: 32 can be taken, 33 cannot
    assert cache.allocators[FULL].free_count == 27
    assert cache.can_take(27) and cache.can_take(32) and not cache.can_take(33)


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_with_shared_prefixes_and_a_small_pool(seed):
    rng = random.Random(seed)
    scheduler, cache = make(max_tokens=rng.choice([64, 96, 160]), page_size=4, budget=rng.choice([7, 16, 40]),
                            max_running=rng.choice([2, 4]))
    cache.enable_prefix_reuse()
    stems = [[rng.randrange(97) for _ in range(rng.randrange(4, 24))] for _ in range(3)]
    requests, step = [], 0
    arrivals = sorted(rng.randrange(80) for _ in range(16))
    while arrivals or scheduler.has_work:
        while arrivals and arrivals[0] <= step:
            arrivals.pop(0)
            prompt = rng.choice(stems) + [rng.randrange(97) for _ in range(rng.randrange(0, 12))]
            r = request(len(requests), prompt, max_new_tokens=rng.randrange(1, 10))
            requests.append(r)
            scheduler.add_request(r)
        run_step(scheduler, cache)
        step += 1
        assert step < 5000
    for r in requests:
        assert r.finished and r.output_ids == expected_output(r.prompt, r.sampling.max_new_tokens)
        assert r.cached_tokens % 4 == 0 and r.cached_tokens < len(r.prompt)
    assert any(r.cached_tokens for r in requests)
    cache.prefix_tree.clear()
    assert cache.allocators[FULL].free_count == cache.allocators[FULL].num_pages


def test_evictable_count_is_kept_without_a_walk():
    """Two requests compute the same prompt at the same time; the second publishes a page below nodes that
    hold the first one's pages.  When the first ends, its pages have no other holder but cannot be freed
    while the page below them is in use: the count that the tree keeps says so, and a walk agrees."""
    cache = CacheManager([PagedKV(2, 16)], page_size=4, max_tokens=64, max_requests=4, device=None)
    tree = cache.enable_prefix_reuse()
    tokens = list(range(16))
    a, b = cache.open("a"), cache.open("b")
    for handle, count in ((a, 12), (b, 16)):
        cache.reserve(handle, count); cache.commit(handle, count)
    assert tree.insert(tokens[:12], a.tables[FULL]) == 3
    assert tree.insert(tokens, b.tables[FULL]) == 1                  # three nodes exist already, one is new
    assert tree.evictable() == 0
    cache.check_invariants()
    cache.close(a)
    assert tree.evictable() == 0                                      # b's page below keeps a's three from eviction
    cache.check_invariants()
    c = cache.open("c")
    cache.adopt_prefix(c, FULL, tree.match(tokens + [99]))
    assert c.length == 16
    cache.close(b)
    assert tree.evictable() == 0                                      # c holds the whole path now
    cache.check_invariants()
    cache.close(c)
    assert tree.evictable() == 4
    cache.check_invariants()
    assert tree.evict(1) == 1 and tree.evictable() == 3
    cache.check_invariants()
    tree.clear()
    assert tree.evictable() == 0 and cache.allocators[FULL].free_count == 16
    cache.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_tree_books_under_random_orders_of_holders(seed):
    """Requests publish, adopt, end and come back in random order, eviction takes pages in between: after
    every move the count of evictable pages and the list of idle leaves equal a walk over the tree, and no
    page is lost or held by a node that is gone."""
    rng = random.Random(seed)
    page_size, num_pages = 2, 48
    cache = CacheManager([PagedKV(2, 16)], page_size=page_size, max_tokens=num_pages * page_size, max_requests=8, device=None)
    tree = cache.enable_prefix_reuse()
    stems = [[rng.randrange(5) for _ in range(rng.randrange(2, 9))] for _ in range(3)]
    live = {}
    for move in range(300):
        kind = rng.random()
        if kind < 0.45 and len(live) < 8:
            tokens = rng.choice(stems) + [rng.randrange(5) for _ in range(rng.randrange(0, 9))]
            handle = cache.open(f"r{move}")
            matched = tree.match(tokens)
            if matched:
                cache.adopt_prefix(handle, FULL, matched)
            rest = len(tokens) - handle.length
            if not cache.can_reserve(handle, rest):
                cache.close(handle)
                continue
            cache.reserve(handle, rest); cache.commit(handle, rest)
            live[handle.request_id] = (handle, tokens)
            if rng.random() < 0.8:
                tree.insert(tokens, handle.tables[FULL])
        elif kind < 0.8 and live:
            handle, _ = live.pop(rng.choice(sorted(live)))
            cache.close(handle)
        elif kind < 0.95:
            before = tree.evictable()
            freed = tree.evict(rng.randrange(1, 6))
            assert freed <= before and tree.evictable() == before - freed
        else:
            tree.match(rng.choice(stems) + [0, 1])                    # a look-up alone moves stamps
        cache.check_invariants()
    for handle, _ in live.values():
        cache.close(handle)
    cache.check_invariants()
    assert tree.evictable() == tree.pages_held
    held = tree.pages_held
    assert tree.evict(10 ** 6) == held and tree.pages_held == 0 and tree.evictable() == 0
    tree.clear()
    cache.check_invariants()
    assert cache.allocators[FULL].free_count == num_pages
