"""The cache manager's bookkeeping (no GPU): no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; slots; groups."""

import random

import pytest

from rapid_llm_b200.cache import CacheError, CacheManager, PagePool, plan_groups
from rapid_llm_b200.parts.base import CacheNeed

FULL = CacheNeed("full", 2, 16)
WIN = CacheNeed("window", 2, 16, 40)


def manager(needs=(FULL, FULL), pages=12, page=16, seqs=4, seq_len=256):
    groups, _ = plan_groups(list(needs))
    return CacheManager(groups, page_size=page, num_pages=pages, max_num_seqs=seqs, max_seq_len=seq_len)


def test_pool_all_or_nothing_and_double_free():
    pool = PagePool(4)
    assert pool.allocate(5) is None and pool.num_free == 4
    pages = pool.allocate(3)
    assert sorted(pages) == [1, 2, 3] and 0 not in pages
    pool.free(pages[:1])
    with pytest.raises(CacheError, match="freed twice"):
        pool.free(pages[:1])
    with pytest.raises(CacheError, match="does not belong"):
        pool.free([9])
    assert pool.allocate(1) == pages[:1]            # a freed page is the next handed out
    pool.check()


def test_a_refused_free_changes_nothing():
    pool = PagePool(4)
    pages = pool.allocate(3)
    for bad in ([pages[0], pages[0]], [pages[1], 9], [pages[2], 4]):      # twice in one call, foreign, not held
        with pytest.raises(CacheError):
            pool.free(bad)
        assert pool.num_free == 1
        pool.check()
    pool.free(pages)
    assert pool.num_free == 4


def test_groups_by_need():
    groups, entry_group = plan_groups([FULL, WIN, None, FULL, WIN, CacheNeed("full", 1, 32)])
    assert [g.entries for g in groups] == [(0, 3), (1, 4), (5,)]
    assert entry_group == [0, 1, None, 0, 1, 2]
    assert [g.window for g in groups] == [0, 40, 0]


def test_reserve_grow_release_and_table():
    cache = manager()
    assert cache.admit("a") == 0 and cache.admit("b") == 1
    assert cache.reserve("a", 17) and cache.num_tokens("a") == 17
    assert cache.pages_of("a")[0] == list(cache.block_tables[0][0, :2])
    assert cache.reserve("a", 32) and len(cache.pages_of("a")[0]) == 2      # same pages, no growth
    assert cache.reserve("a", 33) and len(cache.pages_of("a")[0]) == 3
    dest = cache.kv_destinations(0, 0, 15, 3)
    pages = cache.pages_of("a")[0]
    assert dest.tolist() == [pages[0] * 16 + 15, pages[1] * 16, pages[1] * 16 + 1]
    assert not cache.reserve("b", 16 * 10) and cache.pages_of("b") == [[]]  # all or nothing
    held = cache.pages_of("a")[0]
    cache.release("a")
    assert not cache.block_tables[0][0].any()
    with pytest.raises(CacheError):
        cache.release("a")
    assert cache.reserve("b", 40)
    assert set(cache.pages_of("b")[0]) & set(held), "freed pages are used again"
    cache.check()


def test_slots_run_out_and_come_back():
    cache = manager(seqs=2)
    assert cache.admit("a") is not None and cache.admit("b") is not None
    assert cache.admit("c") is None
    with pytest.raises(CacheError):
        cache.admit("a")
    cache.release("a")
    assert cache.admit("c") == 0
    cache.check()


def test_window_pages_are_given_back_and_full_pages_stay():
    cache = manager(needs=(FULL, WIN), pages=20, seq_len=320)
    cache.admit("w")
    for upto in range(16, 305, 16):
        assert cache.reserve("w", upto)
        cache.release_passed("w")
        full, windowed = cache.pages_of("w")
        assert all(full) and len(full) == upto // 16
        oldest = max(upto - 40 + 1, 0)
        assert [bool(p) for p in windowed] == [index >= oldest // 16 for index in range(upto // 16)]
        cache.check()
    assert cache.pools[1].num_held <= 40 // 16 + 2
    cache.release("w")
    assert cache.pools[0].num_free == 20 and cache.pools[1].num_free == 20


def test_cannot_shrink_or_outgrow():
    cache = manager(seq_len=64)
    cache.admit("a")
    cache.reserve("a", 20)
    with pytest.raises(CacheError, match="shrink"):
        cache.reserve("a", 10)
    with pytest.raises(CacheError, match="max_seq_len"):
        cache.reserve("a", 65)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    cache = manager(needs=(FULL, WIN, FULL), pages=[30, 14], page=8, seqs=5, seq_len=200)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            name = f"r{counter}"
            counter += 1
            assert cache.admit(name) is not None
            live[name] = 0
        elif action < 0.8 and live:
            name = rng.choice(list(live))
            upto = min(200, live[name] + rng.choice([1, 1, 1, 2, 7, 13, 40]))
            if upto > live[name] and cache.reserve(name, upto):
                live[name] = upto
                cache.release_passed(name)
        elif live:
            name = rng.choice(list(live))
            cache.release(name)
            del live[name]
        cache.check()
        for name, tokens in live.items():
            assert cache.num_tokens(name) == tokens
            full = cache.pages_of(name)[0]
            assert len(full) == -(-tokens // 8) and all(full)
            row = cache.block_tables[0][cache.slot_of(name)]
            assert row[: len(full)].tolist() == full and not row[len(full):].any()
    for name in list(live):
        cache.release(name)
    assert [pool.num_free for pool in cache.pools] == [30, 14]
    assert all(not table.any() for table in cache.block_tables)


def test_dirty_rows_are_reported_once():
    cache = manager()
    cache.admit("a")
    cache.reserve("a", 5)
    assert cache.take_dirty(0) == [0] and cache.take_dirty(0) == []
    cache.reserve("a", 6)
    assert cache.take_dirty(0) == []            # same page: the row did not change
    cache.reserve("a", 17)
    assert cache.take_dirty(0) == [0]


def test_pages_sized_from_free_memory():
    """The pool takes the given share of free memory after the largest step's buffers are set aside,
    is capped by what the slots can hold, and is never empty."""
    from rapid_llm_b200.engine.runner import pages_that_fit

    gib = 1 << 30
    page = 36 * 2 * 8 * 128 * 16 * 2                       # a page of 16 tokens over 36 layers of 8 x 128 keys and values
    assert pages_that_fit(100 * gib, 0.9, page, reserve=4 * gib, cap=10**9) == (90 * gib - 4 * gib) // page
    assert pages_that_fit(100 * gib, 0.9, page, reserve=4 * gib, cap=1000) == 1000
    assert pages_that_fit(1 * gib, 0.5, page, reserve=2 * gib, cap=1000) == 1      # nothing left: one page, and the step fails loudly
    assert pages_that_fit(100 * gib, 1.0, 0, reserve=0, cap=77) == 77               # no mixer keeps pages


def test_a_cache_need_with_a_row_of_its_own_per_token():
    from rapid_llm_b200.cache.manager import plan_groups
    from rapid_llm_b200.parts.base import CacheNeed

    keys_and_values = CacheNeed("full", 2, 64)
    latent = CacheNeed("full", token_shape=(72,))
    assert keys_and_values.page_shape(16) == (2, 2, 16, 64) and keys_and_values.elements_per_token() == 256
    assert latent.page_shape(16) == (16, 72) and latent.elements_per_token() == 72
    groups, entry_group = plan_groups([keys_and_values, latent, None, latent, keys_and_values])
    assert entry_group == [0, 1, None, 1, 0] and [g.entries for g in groups] == [(0, 4), (1, 3)]
    import pytest
    with pytest.raises(ValueError, match="token's row"):
        plan_groups([CacheNeed("full")])
