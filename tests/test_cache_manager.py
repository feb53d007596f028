"""The cache manager: no page lost, held twice or freed twice, under random orders of requests;
windowed groups hand pages back while a request lives; state slots."""
from __future__ import annotations

import random

import numpy as np
import pytest

from kvcore_b200.cache import (
    CacheGroupSpec, KVManager, PagePool, PagePoolError, StateSlotError, StateSlotPool,
)


def manager(num_pages=9, page_size=4, windows=(None,), max_num_seqs=4, max_model_len=64):
    groups = [CacheGroupSpec(i, (i,), 2, 2, 16, w) for i, w in enumerate(windows)]
    return KVManager(groups, num_pages=num_pages, page_size=page_size, max_num_seqs=max_num_seqs,
                     max_model_len=max_model_len)


def test_pool_null_page_order_and_double_free():
    pool = PagePool(5)
    assert pool.num_free == 4 and pool.num_usable == 4
    pages = pool.allocate(3)
    assert pages == [1, 2, 3] and 0 not in pages
    with pytest.raises(PagePoolError):
        pool.allocate(2)
    pool.free(reversed(pages))
    assert pool.free_pages() == [4, 3, 2, 1]  # freed pages queue behind the never-used one
    with pytest.raises(PagePoolError, match="twice"):
        pool.free([2])
    with pytest.raises(PagePoolError, match="null"):
        pool.free([0])
    with pytest.raises(PagePoolError):
        pool.free([9])
    assert pool.allocate(2) == [4, 3]


def test_allocate_advance_free_and_tables():
    kv = manager()
    assert kv.can_fit("a", 9) and kv.allocate_slots("a", 9)  # 3 pages
    assert kv.block_ids("a") == ((1, 2, 3),)
    assert kv.pages_needed("a", 9) == [0] and kv.pages_needed("a", 13) == [1]
    kv.advance("a", 9)
    assert kv.num_computed("a") == 9
    assert kv.allocate_slots("a", 3)  # fits in the third page
    assert kv.block_ids("a") == ((1, 2, 3),)
    kv.advance("a", 3)
    assert kv.allocate_slots("a", 1) and kv.block_ids("a") == ((1, 2, 3, 4),)
    assert kv.allocate_slots("b", 16) and kv.block_ids("b") == ((5, 6, 7, 8),)
    assert not kv.can_fit("c", 1) and not kv.allocate_slots("c", 1)
    assert not kv.has_request("c")
    row = kv.tables[0][kv.state_slot("b")]
    assert row[:4].tolist() == [5, 6, 7, 8] and not row[4:].any()
    kv.check_invariants()
    kv.free("a")
    assert kv.pools[0].free_pages() == [4, 3, 2, 1]  # reverse order: tail pages first
    assert kv.allocate_slots("c", 5) and kv.block_ids("c") == ((4, 3),)
    kv.free("b"); kv.free("c"); kv.free("c")
    kv.check_invariants()
    assert kv.num_free_pages() == [8] and not kv.live_requests()


def test_advance_beyond_pages_is_an_error():
    kv = manager()
    kv.allocate_slots("a", 4)
    with pytest.raises(Exception, match="holds pages"):
        kv.advance("a", 5)


def test_max_model_len_and_slots_limit():
    kv = manager(num_pages=100, max_num_seqs=2, max_model_len=10)
    assert not kv.can_fit("a", 11) and kv.allocate_slots("a", 10)
    assert kv.allocate_slots("b", 1)
    assert not kv.can_fit("c", 1)  # no state slot left
    kv.free("a")
    assert kv.allocate_slots("c", 1) and kv.state_slot("c") == 0
    assert kv.take_fresh_slots() == [1, 0] and kv.take_fresh_slots() == []


def test_window_group_hands_pages_back_while_the_request_lives():
    kv = manager(num_pages=6, page_size=4, windows=(None, 6), max_model_len=40)
    assert kv.allocate_slots("a", 10)
    kv.advance("a", 10)  # next query at 10 sees keys >= 5: page 0 (positions 0..3) is passed
    assert kv.block_ids("a") == ((1, 2, 3), (0, 2, 3))
    assert kv.num_free_pages() == [2, 3]
    for _ in range(10):
        assert kv.allocate_slots("a", 1)
        kv.advance("a", 1)
        kv.check_invariants()
    # 20 tokens: the full group would need 5 pages; the windowed one never holds more than 3
    assert kv.num_free_pages()[1] >= 2 and kv.block_ids("a")[1][:3] == (0, 0, 0)
    assert not kv.can_fit("a", 1)  # the full group is exhausted
    kv.free("a")
    kv.check_invariants()
    assert kv.num_free_pages() == [5, 5]


def test_window_never_releases_a_page_a_later_query_can_see():
    page, window = 4, 6
    kv = manager(num_pages=50, page_size=page, windows=(window,), max_model_len=100)
    rng = random.Random(0)
    done = 0
    while done < 90:
        n = rng.choice([1, 1, 2, 5, 9])
        assert kv.allocate_slots("a", n)
        # every key the portion's queries can see must still have a page
        first_visible = max(0, done - window + 1)
        row = kv.tables[0][kv.state_slot("a")]
        for pos in range(first_visible, done + n):
            assert row[pos // page] != 0, (done, n, pos)
        kv.advance("a", n)
        done += n
    assert kv.pools[0].num_usable - kv.pools[0].num_free <= -(-(window + 9) // page) + 1


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    kv = manager(num_pages=24, page_size=4, windows=(None, 7), max_num_seqs=5, max_model_len=48)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.35 and len(live) < 5:
            counter += 1
            rid = f"r{counter}"
            n = rng.randint(1, 20)
            if kv.allocate_slots(rid, n):
                kv.advance(rid, n)
                live[rid] = n
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 3, 8])
            before = kv.num_free_pages()
            if kv.allocate_slots(rid, n):
                kv.advance(rid, n)
                live[rid] += n
            else:
                assert kv.num_free_pages() == before  # a refused allocation changes nothing
        elif live:
            rid = rng.choice(list(live))
            kv.free(rid)
            del live[rid]
        kv.check_invariants()
        for rid, n in live.items():
            assert kv.num_computed(rid) == n
        slots = [kv.state_slot(r) for r in live]
        assert len(set(slots)) == len(slots)
    for rid in list(live):
        kv.free(rid)
    kv.check_invariants()
    assert kv.num_free_pages() == [23, 23] and kv.slots.num_free == 5
    assert not any(np.any(t) for t in kv.tables)


# ---- prefix reuse ----------------------------------------------------------------------------------
def test_pool_shared_pages_and_registered_contents():
    pool = PagePool(6)
    a, b = pool.allocate(2)
    assert pool.register(a, "ka") and not pool.register(b, "ka") and pool.lookup("ka") == a
    pool.share(a)
    assert pool.ref_count(a) == 2
    pool.free([a])
    assert pool.is_held(a) and not pool.is_queued(a)
    pool.free([a])                                   # last holder: to the tail, still findable
    assert pool.is_queued(a) and pool.lookup("ka") == a and pool.free_pages()[-1] == a
    pool.share(a)                                    # taken over again, out of the queue
    assert not pool.is_queued(a) and pool.ref_count(a) == 1
    pool.free([a])
    with pytest.raises(PagePoolError, match="twice"):
        pool.free([a])
    with pytest.raises(PagePoolError, match="registered"):
        pool.share(b)
    taken = pool.allocate(pool.num_free)             # the queue hands the page out again: key dropped
    assert a in taken and pool.lookup("ka") is None


def prefix_manager(**kw):
    return KVManager([CacheGroupSpec(0, (0, 1), 2, 2, 16, None)], num_pages=kw.pop("num_pages", 17), page_size=4,
                     max_num_seqs=4, max_model_len=64, enable_prefix_caching=True, **kw)


def test_prefix_pages_are_taken_over_by_a_later_request():
    kv = prefix_manager()
    first = list(range(100, 114))                    # 14 tokens: 3 full pages and a half
    assert kv.find_prefix(first) == []
    assert kv.allocate_slots("a", 14)
    kv.advance("a", 14)
    kv.register_full_pages("a", first)
    a_pages = kv.block_ids("a")[0]
    second = first[:9] + [7, 8, 9]                   # shares two full pages (8 tokens)
    hit = kv.find_prefix(second)
    assert hit == [(page,) for page in a_pages[:2]]
    assert kv.allocate_slots("b", len(second) - 8, hit)
    assert kv.num_computed("b") == 8 and kv.block_ids("b")[0][:2] == a_pages[:2]
    assert kv.block_ids("b")[0][2] not in a_pages
    kv.check_invariants()
    kv.free("a")                                      # shared pages stay with b
    kv.check_invariants()
    assert all(kv.pools[0].is_held(p) for (p,) in hit)
    kv.advance("b", len(second) - 8)
    kv.register_full_pages("b", second)
    kv.free("b")
    kv.check_invariants()
    assert kv.num_free_pages() == [16]
    # everything is free, yet still findable: a third request takes pages over out of the queue
    again = kv.find_prefix(first)
    assert again == [(page,) for page in a_pages[:3]]
    assert kv.can_fit("c", 2, again) and kv.allocate_slots("c", 2, again)
    assert kv.num_computed("c") == 12 and kv.num_prefix_hits == 5
    kv.check_invariants()


def test_the_last_token_of_a_prompt_is_always_left_to_compute():
    kv = prefix_manager()
    tokens = list(range(8))
    assert kv.allocate_slots("a", 8)
    kv.advance("a", 8)
    kv.register_full_pages("a", tokens)
    assert len(kv.find_prefix(tokens)) == 1           # 8 tokens = 2 full pages, but only 1 may be taken
    assert len(kv.find_prefix(tokens + [9])) == 2


def test_taken_over_pages_in_the_queue_count_against_the_free_pages():
    kv = prefix_manager(num_pages=5)                 # 4 usable pages
    tokens = list(range(12))
    assert kv.allocate_slots("a", 12)
    kv.advance("a", 12)
    kv.register_full_pages("a", tokens)
    kv.free("a")
    hit = kv.find_prefix(tokens + [1, 2, 3, 4, 5])   # 3 pages, all in the queue now
    assert len(hit) == 3
    assert not kv.can_fit("b", 8, hit)               # 5 pages in all > 4
    assert kv.can_fit("b", 4, hit) and kv.allocate_slots("b", 4, hit)
    kv.check_invariants()
    assert kv.num_free_pages() == [0]


def test_prefix_reuse_is_off_without_the_flag_and_with_windows():
    plain = manager()
    assert not plain.prefix_caching and plain.find_prefix(list(range(20))) == []
    windowed = KVManager([CacheGroupSpec(0, (0,), 2, 2, 16, 8)], num_pages=9, page_size=4, max_num_seqs=2,
                         max_model_len=64, enable_prefix_caching=True)
    assert not windowed.prefix_caching


def test_prefix_reuse_over_two_groups_counts_only_what_both_still_hold():
    """Two groups that keep every key (say, layers with different head sizes): a prefix is taken over in
    both tables, and only as far as both pools still have the page."""
    kv = KVManager([CacheGroupSpec(0, (0,), 2, 2, 16, None), CacheGroupSpec(1, (1,), 1, 1, 24, None)], num_pages=[17, 17],
                   page_size=4, max_num_seqs=4, max_model_len=64, enable_prefix_caching=True)
    assert kv.prefix_caching
    tokens = list(range(50, 63))                     # 13 tokens: 3 full pages
    assert kv.allocate_slots("a", 13)
    kv.advance("a", 13)
    kv.register_full_pages("a", tokens)
    a_pages = kv.block_ids("a")
    hit = kv.find_prefix(tokens)
    assert hit == [(a_pages[0][i], a_pages[1][i]) for i in range(3)]
    assert kv.allocate_slots("b", 2, hit[:2])
    assert kv.num_computed("b") == 8
    assert kv.block_ids("b")[0][:2] == a_pages[0][:2] and kv.block_ids("b")[1][:2] == a_pages[1][:2]
    kv.check_invariants()
    kv.free("a")
    kv.free("b")
    kv.check_invariants()
    # the second group's queue hands its pages out again: the prefix is gone in that group, so it is gone
    taken = kv.pools[1].allocate(kv.pools[1].num_free)
    assert kv.find_prefix(tokens) == []
    kv.pools[1].free(taken)
    kv.check_invariants()


@pytest.mark.parametrize("seed", range(4))
def test_random_orders_with_shared_prefixes_keep_every_page_accounted(seed):
    rng = random.Random(100 + seed)
    kv = prefix_manager(num_pages=30)
    stems = [[rng.randint(0, 50) for _ in range(24)] for _ in range(3)]
    live: dict[str, list[int]] = {}
    counter = 0
    for _ in range(500):
        action = rng.random()
        if action < 0.4 and len(live) < 4:
            counter += 1
            rid = f"r{counter}"
            tokens = rng.choice(stems)[: rng.randint(1, 24)] + [rng.randint(60, 90) for _ in range(rng.randint(1, 6))]
            hit = kv.find_prefix(tokens)
            n = len(tokens) - 4 * len(hit)
            if kv.allocate_slots(rid, n, hit):
                assert kv.num_computed(rid) == 4 * len(hit)
                kv.advance(rid, n)
                kv.register_full_pages(rid, tokens)
                live[rid] = tokens
        elif action < 0.7 and live:
            rid = rng.choice(list(live))
            if kv.allocate_slots(rid, 1):
                kv.advance(rid, 1)
                live[rid] = live[rid] + [rng.randint(60, 90)]
                kv.register_full_pages(rid, live[rid])
        elif live:
            rid = rng.choice(list(live))
            kv.free(rid)
            del live[rid]
        kv.check_invariants()
    for rid in list(live):
        kv.free(rid)
    kv.check_invariants()
    assert kv.num_free_pages() == [29] and kv.num_prefix_hits > 0


def test_state_slots():
    pool = StateSlotPool(2)
    a, b = pool.allocate("a"), pool.allocate("b")
    assert (a, b) == (0, 1) and pool.owner(1) == "b"
    with pytest.raises(StateSlotError):
        pool.allocate("c")
    pool.free(a)
    with pytest.raises(StateSlotError):
        pool.free(a)
    assert pool.allocate("c") == 0


def test_released_pages_are_reported_once_when_tracking_is_on():
    """The debug fill of freed pages reads this list: every page that lost its last holder (a finished
    request's pages, pages behind a window) appears once, and nothing is kept without the switch."""
    kv = KVManager([CacheGroupSpec(0, (0,), 2, 2, 16, None), CacheGroupSpec(1, (1,), 2, 2, 16, 8)], num_pages=[9, 9],
                   page_size=4, max_num_seqs=2, max_model_len=32, track_released_pages=True)
    assert kv.allocate_slots("a", 16)
    held = kv.block_ids("a")
    kv.advance("a", 16)                       # the windowed group hands back pages behind the window
    released = kv.take_released_pages()
    assert released[0] == [] and released[1] == list(held[1][:2])
    assert kv.take_released_pages() == [[], []]
    kv.free("a")
    released = kv.take_released_pages()
    assert sorted(released[0]) == sorted(held[0]) and sorted(released[1]) == sorted(held[1][2:])
    kv.check_invariants()
    silent = KVManager([CacheGroupSpec(0, (0,), 2, 2, 16, None)], num_pages=9, page_size=4, max_num_seqs=2,
                       max_model_len=32)
    assert silent.allocate_slots("a", 8)
    silent.free("a")
    assert silent.take_released_pages() == [[]]
