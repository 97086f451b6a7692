"""The cache manager: pages, prefix hashes, windows, state slots (no GPU)."""

from __future__ import annotations

import random

import pytest

from mini_engine_b200.cache import NULL_PAGE, CacheManager, GroupSpec, SlotGroupSpec, hash_page

FULL = [GroupSpec("full")]


def computed(mgr, req, tokens, count):
    mgr.register_computed(req, tokens, count)


def test_hashes_chain():
    a = hash_page(b"", [1, 2, 3, 4])
    assert a == hash_page(b"", [1, 2, 3, 4]) and len(a) == 16
    assert hash_page(a, [5, 6, 7, 8]) != hash_page(b"", [5, 6, 7, 8])


def test_allocate_free_round_trip_and_all_or_nothing():
    mgr = CacheManager(FULL, num_blocks=4, block_size=4, max_num_seqs=2)
    a, b = mgr.new_request(), mgr.new_request()
    assert mgr.try_allocate(a, 9) and len(a.block_tables[0]) == 3 and a.state_slot >= 0
    assert not mgr.try_allocate(b, 8)  # two pages wanted, one free: nothing changes
    assert b.block_tables == [[]] and b.state_slot == -1 and mgr.num_free_blocks == 1
    mgr.check_invariants([a, b])
    mgr.free(a)
    assert mgr.num_free_blocks == 4 and a.holds_nothing()
    mgr.check_invariants([])
    with pytest.raises(AssertionError):
        mgr.pools[0].release(0)  # freed twice


def test_prefix_sharing_counts_references_and_always_leaves_a_token():
    mgr = CacheManager(FULL, num_blocks=8, block_size=4, max_num_seqs=4)
    tokens = list(range(12))
    a = mgr.new_request()
    assert mgr.try_allocate(a, 12)
    computed(mgr, a, tokens, 12)
    hits = mgr.match_prefix(tokens)  # 12 tokens: only the first two pages are eligible
    assert hits == [a.block_tables[0][:2]]
    b = mgr.new_request()
    assert mgr.try_allocate(b, 12, hits)
    assert b.block_tables[0][:2] == a.block_tables[0][:2] and b.block_tables[0][2] != a.block_tables[0][2]
    assert [mgr.pools[0].ref_counts[p] for p in hits[0]] == [2, 2]
    mgr.check_invariants([a, b])
    mgr.free(a)
    mgr.free(b)
    mgr.check_invariants([])
    assert mgr.match_prefix(tokens + [99]) != [[]]  # freed pages stay cached


def test_eviction_takes_unhashed_pages_first_then_least_recently_freed():
    mgr = CacheManager(FULL, num_blocks=4, block_size=2, max_num_seqs=4)
    a, b = mgr.new_request(), mgr.new_request()
    assert mgr.try_allocate(a, 4) and mgr.try_allocate(b, 3)
    computed(mgr, a, [1, 2, 3, 4], 4)
    computed(mgr, b, [5, 6, 7], 3)  # b's second page is not full: unhashed
    b_tail = b.block_tables[0][1]
    a_pages = list(a.block_tables[0])
    mgr.free(a)
    mgr.free(b)
    c = mgr.new_request()
    assert mgr.try_allocate(c, 2) and c.block_tables[0] == [b_tail] and mgr.num_evictions == 0
    d = mgr.new_request()
    assert mgr.try_allocate(d, 2)
    assert d.block_tables[0] == [a_pages[1]] and mgr.num_evictions == 1  # a's tail before a's head
    mgr.check_invariants([c, d])


def test_reviving_cached_pages_counts_against_capacity():
    mgr = CacheManager(FULL, num_blocks=3, block_size=2, max_num_seqs=4)
    a = mgr.new_request()
    tokens = [1, 2, 3, 4, 5]
    assert mgr.try_allocate(a, 5)
    computed(mgr, a, tokens, 5)
    mgr.free(a)
    b = mgr.new_request()
    assert mgr.try_allocate(b, 2)  # takes the unhashed third page
    c = mgr.new_request()
    hits = mgr.match_prefix(tokens)
    assert len(hits[0]) == 2
    assert not mgr.try_allocate(c, 6, hits)  # 2 revived + 1 fresh > 2 free
    assert mgr.try_allocate(c, 4, hits)
    mgr.check_invariants([b, c])


def test_duplicate_content_is_not_registered_twice_and_reset():
    mgr = CacheManager(FULL, num_blocks=4, block_size=2, max_num_seqs=4)
    a, b = mgr.new_request(), mgr.new_request()
    assert mgr.try_allocate(a, 2) and mgr.try_allocate(b, 2)
    computed(mgr, a, [1, 2], 2)
    computed(mgr, b, [1, 2], 2)
    assert mgr.pools[0].page_hash[b.block_tables[0][0]] is None
    mgr.check_invariants([a, b])
    mgr.reset_prefix_cache()
    assert mgr.match_prefix([1, 2, 3]) == [[]]


def test_prefix_caching_disabled_or_unsound():
    off = CacheManager(FULL, 4, 2, 2, enable_prefix_caching=False)
    a = off.new_request()
    assert off.try_allocate(a, 4)
    computed(off, a, [1, 2, 3, 4], 4)
    assert off.match_prefix([1, 2, 3, 4, 5]) == [[]] and a.page_hashes == []
    # a group says by itself that what it holds cannot be found again by content: a slot of state
    # (no snapshots), or a page group that declares it; one such group and every request starts at 0
    assert not CacheManager(FULL, 4, 2, 2, slot_groups=[SlotGroupSpec("state")]).enable_prefix_caching
    assert not CacheManager([GroupSpec("full"), GroupSpec("odd", shareable=False)], 4, 2, 2).enable_prefix_caching
    assert CacheManager(FULL, 4, 2, 2, slot_groups=[SlotGroupSpec("snapshotted", shareable=True)]).enable_prefix_caching
    assert CacheManager([GroupSpec("w", window=8)], 4, 2, 2).enable_prefix_caching


def test_prefix_hits_with_a_window_need_only_the_pages_the_window_reaches():
    """A group with a window shares the pages that its window still reaches from the end of the
    shared prefix; earlier ones may be long gone and stand as NULL_PAGE in the new table."""
    groups = [GroupSpec("full"), GroupSpec("win", window=6)]
    mgr = CacheManager(groups, num_blocks=12, block_size=4, max_num_seqs=3)
    tokens = list(range(100, 120))
    first = mgr.new_request()
    assert mgr.try_allocate(first, 20)
    computed(mgr, first, tokens, 20)
    assert mgr.release_behind_window(first, 20) == 3  # next query at 20 reads keys > 14: pages 0..2 are passed
    # a second request with the same 20 tokens and 5 more: 5 whole pages could be shared; the window at
    # position 20 needs page 3 on (keys 15..19 lie in pages 3 and 4), which `first` still holds
    hits = mgr.match_prefix(tokens + [1, 2, 3, 4, 5])
    assert hits[0] == first.block_tables[0][:5]
    assert hits[1][:3] == [NULL_PAGE] * 3 and hits[1][3:] == first.block_tables[1][3:5]
    second = mgr.new_request()
    assert mgr.try_allocate(second, 25, hits)
    assert second.block_tables[1][:3] == [NULL_PAGE] * 3 and len(second.block_tables[1]) == 7
    mgr.check_invariants([first, second])
    # the passed pages of the window group went back hashed; once they are evicted nothing changes for a
    # hit at this length, but a shorter prefix (12 tokens: window needs pages 1..2) cannot be served
    # by the window group when those pages have been overwritten
    taker = mgr.new_request()
    assert mgr.try_allocate(taker, 12)  # takes three fresh pages in each group
    short = mgr.match_prefix(tokens[:12] + [9])
    served = len(short[0])
    assert served in (0, 3)
    if served:
        assert NULL_PAGE not in short[1][mgr._first_needed_page(groups[1], 12) : 3]
    mgr.free(first), mgr.free(second), mgr.free(taker)
    mgr.check_invariants([])
    assert mgr.pools[0].num_free == 12 and mgr.pools[1].num_free == 12


def test_groups_have_pools_of_their_own_size():
    groups = [GroupSpec("full"), GroupSpec("win", window=6, num_blocks=5)]
    mgr = CacheManager(groups, num_blocks=16, block_size=4, max_num_seqs=2, enable_prefix_caching=False)
    assert [p.num_pages for p in mgr.pools] == [16, 5] and mgr.smallest_pool == 16
    req = mgr.new_request()
    assert not mgr.try_allocate(req, 24) and req.holds_nothing()  # six pages at once: the window group has five
    assert mgr.try_allocate(req, 16)
    mgr.release_behind_window(req, 16)
    assert mgr.try_allocate(req, 28)  # 7 pages of the full group; the window group holds pages 2..6 only
    assert mgr.num_free_blocks == 0
    mgr.check_invariants([req])
    mgr.free(req)
    mgr.check_invariants([])


def test_window_group_gives_pages_back_while_the_request_runs():
    groups = [GroupSpec("full"), GroupSpec("win", window=6)]
    mgr = CacheManager(groups, num_blocks=8, block_size=4, max_num_seqs=2)
    req = mgr.new_request()
    assert mgr.try_allocate(req, 16)
    assert mgr.release_behind_window(req, 16) == 2  # next query at 16 reads keys > 10: pages 0 and 1 are passed
    assert req.block_tables[1][:2] == [NULL_PAGE, NULL_PAGE] and NULL_PAGE not in req.block_tables[0]
    assert mgr.pools[1].num_free == 6 and mgr.pools[0].num_free == 4
    assert mgr.release_behind_window(req, 16) == 0
    mgr.check_invariants([req])
    assert mgr.try_allocate(req, 20) and len(req.block_tables[1]) == 5
    mgr.free(req)
    mgr.check_invariants([])
    assert mgr.pools[1].num_free == 8


def test_state_slots_run_out_and_come_back():
    mgr = CacheManager(FULL, num_blocks=16, block_size=4, max_num_seqs=2, slot_groups=[SlotGroupSpec("state")])
    reqs = [mgr.new_request() for _ in range(3)]
    assert mgr.try_allocate(reqs[0], 1) and mgr.try_allocate(reqs[1], 1)
    assert not mgr.try_allocate(reqs[2], 1) and reqs[2].holds_nothing()
    assert reqs[0].state_slot != reqs[1].state_slot
    mgr.free(reqs[0])
    assert mgr.try_allocate(reqs[2], 1)
    mgr.check_invariants(reqs[1:])


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    """Requests arrive, grow, share prefixes, pass windows and end in random order; after every
    operation no page is lost, held twice without a count, or free while held."""
    rng = random.Random(seed)
    groups = [GroupSpec("full")] if seed % 2 == 0 else [GroupSpec("full"), GroupSpec("win", window=5)]
    mgr = CacheManager(groups, num_blocks=12, block_size=4, max_num_seqs=5)
    live: list[dict] = []
    prefixes = [[rng.randrange(50) for _ in range(8)] for _ in range(2)]
    for _ in range(400):
        action = rng.random()
        if action < 0.35 and len(live) < 6:
            tokens = list(rng.choice(prefixes)) + [rng.randrange(50) for _ in range(rng.randrange(1, 20))]
            req = mgr.new_request()
            hits = mgr.match_prefix(tokens)
            cached = len(hits[0]) * 4
            take = rng.randrange(1, len(tokens) - cached + 1)
            if mgr.try_allocate(req, cached + take, hits):
                live.append({"req": req, "tokens": tokens, "done": cached, "alloc": cached + take})
            else:
                assert req.holds_nothing()
        elif action < 0.8 and live:
            item = rng.choice(live)
            item["done"] = item["alloc"]
            mgr.register_computed(item["req"], item["tokens"], item["done"])
            mgr.release_behind_window(item["req"], item["done"])
            if item["done"] == len(item["tokens"]):
                item["tokens"].append(rng.randrange(50))
            grow = min(len(item["tokens"]), item["done"] + rng.randrange(1, 6))
            if mgr.try_allocate(item["req"], grow):
                item["alloc"] = grow
        elif live:
            item = live.pop(rng.randrange(len(live)))
            mgr.free(item["req"])
        mgr.check_invariants([i["req"] for i in live])
    for item in live:
        mgr.free(item["req"])
    mgr.check_invariants([])
    assert all(pool.num_free == 12 for pool in mgr.pools)


def test_pages_that_a_memory_budget_holds():
    import torch

    from mini_engine_b200.cache.storage import blocks_for_budget, bytes_per_token
    from mini_engine_b200.parts.base import PagedCacheSpec, StateSpec

    full, window = PagedCacheSpec(2, 16), PagedCacheSpec(4, 32, window=8)
    # three owners and one entry that reads the first entry's cache (it holds nothing itself)
    needs = [(full, None, None), (window, None, None), (full, None, 0), (None, StateSpec((4,)), None), (full, None, None)]
    per_token = 2 * (2 * 16 + 4 * 32 + 2 * 16)
    assert bytes_per_token(needs, torch.bfloat16) == per_token * 2
    assert bytes_per_token(needs, torch.float32) == per_token * 4
    page = per_token * 2 * 8
    assert blocks_for_budget(needs, torch.bfloat16, 8, 10 * page) == 9  # one page is the spare
    assert blocks_for_budget(needs, torch.bfloat16, 8, 10 * page + page - 1) == 9
    with pytest.raises(ValueError, match="hold no KV page"):
        blocks_for_budget(needs, torch.bfloat16, 8, 2 * page - 1)
    assert blocks_for_budget([(None, StateSpec((4,)), None)], torch.float32, 8, 0) == 1


def test_version_tells_when_a_copy_of_the_tables_is_stale():
    manager = CacheManager([GroupSpec("full", None), GroupSpec("window", 8)], 16, 4, 4, enable_prefix_caching=False)
    a, b = manager.new_request(), manager.new_request()
    assert a.serial != b.serial
    seen = a.version
    assert manager.try_allocate(a, 3) and a.version > seen
    seen = a.version
    assert manager.try_allocate(a, 4) and a.version == seen  # still one page: nothing changed
    assert manager.try_allocate(a, 20) and a.version > seen
    seen = a.version
    assert manager.release_behind_window(a, 20) > 0 and a.version > seen  # the window group gave pages back
    seen = a.version
    assert manager.release_behind_window(a, 20) == 0 and a.version == seen
    manager.free(a)
    assert a.version > seen
    manager.check_invariants([b])
