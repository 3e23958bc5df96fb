"""Radix prefix cache (KV half): match / insert / split / lock / LRU eviction invariants, after
the reference's tests (crates/warp34-host/src/radix.rs:1402-1742,
crates/warp34-host/tests/radix_cache_and_scheduler.rs:15-85)."""
import pytest

from warp34_b200.kv import PagePool, PrefixCache, Sequence


@pytest.fixture(autouse=True)
def _libs(native_libs):
    return native_libs


def _seq_with(pool, n_tokens):
    s = Sequence(pool)
    assert s.reserve(n_tokens) >= 0
    s.commit(n_tokens)
    return s


def test_insert_match_and_page_alignment():
    pool = PagePool(64)
    cache = PrefixCache(pool)
    a = _seq_with(pool, 64)
    toks = list(range(100, 164))
    assert cache.insert(toks, a.pages) == (0, 1)
    assert cache.sanity_check() == 0
    assert all(pool.refcount(p) == 2 for p in a.pages)
    # full match, partial match inside a page (rounded down), miss
    assert cache.match_prefix(toks)[:2] == (a.pages, 64)
    pages, matched, node = cache.match_prefix(toks[:40] + [7] * 24)
    assert matched == 32 and pages == a.pages[:2] and node != 0
    assert cache.match_prefix(toks[:15]) == ([], 0, 0)
    assert cache.match_prefix([5] * 64) == ([], 0, 0)
    assert cache.sanity_check() == 0
    # the partial match split the node at the page boundary: 2 nodes now
    assert cache.stats()["nodes"] == 2 and cache.stats()["cached"] == 4


def test_insert_shares_the_common_prefix_and_reports_duplicates():
    pool = PagePool(64)
    cache = PrefixCache(pool)
    a = _seq_with(pool, 48)
    b = _seq_with(pool, 64)
    ta = list(range(48))
    tb = list(range(32)) + list(range(900, 932))
    assert cache.insert(ta, a.pages)[0] == 0
    already, node_b = cache.insert(tb, b.pages)
    assert already == 32                       # b's first two pages duplicate cached content
    assert cache.stats()["cached"] == 3 + 2     # a's three pages + b's two new ones
    assert [pool.refcount(p) for p in b.pages] == [1, 1, 2, 2]
    pages, matched, _ = cache.match_prefix(tb)
    assert matched == 64 and pages == a.pages[:2] + b.pages[2:]
    assert cache.insert(tb, b.pages)[0] == 64   # inserting again stores nothing new
    assert cache.sanity_check() == 0


def test_locks_protect_paths_and_eviction_is_lru_over_unlocked_leaves():
    pool = PagePool(64)
    cache = PrefixCache(pool)
    seqs, toks, nodes = {}, {}, {}
    for i, name in enumerate("ABC"):
        seqs[name] = _seq_with(pool, 32)
        toks[name] = [1000 * (i + 1) + t for t in range(32)]
        nodes[name] = cache.insert(toks[name], seqs[name].pages)[1]
    for s in seqs.values():
        s.close()                                # the cache is now the only owner
    assert pool.free_count == 64 - 6
    cache.match_prefix(toks["A"])                # touch A: B is now least recently used
    assert cache.lock(nodes["C"]) == 0
    assert cache.stats()["protected"] == 2
    freed = cache.evict(1)
    assert len(freed) == 2 and cache.match_prefix(toks["B"])[1] == 0
    freed = cache.evict(10)                       # A goes, C is locked
    assert len(freed) == 2 and cache.match_prefix(toks["C"])[1] == 32
    assert cache.evict(1) == []
    assert cache.unlock(nodes["C"]) == 0
    assert cache.unlock(nodes["C"]) < 0           # unbalanced
    assert len(cache.evict(1)) == 2
    assert pool.free_count == 64 and cache.stats()["nodes"] == 0
    assert cache.sanity_check() == 0


def test_prefix_hit_feeds_a_sequence_and_rollback_keeps_shared_pages():
    pool = PagePool(64)
    cache = PrefixCache(pool)
    donor = _seq_with(pool, 80)
    toks = list(range(80))
    cache.insert(toks, donor.pages)
    donor.close()
    prompt = toks[:70] + [9999] * 20
    pages, matched, node = cache.match_prefix(prompt[:-1])
    assert matched == 64 and len(pages) == 4
    cache.lock(node)
    req = Sequence(pool)
    assert req.attach_prefix(pages, matched) == 0
    assert req.reserve(len(prompt) + 4) >= 0      # speculative headroom
    req.commit(len(prompt) - matched)
    freed = req.rollback()
    assert all(p not in pages for p in freed)
    assert req.protected_pages == 4 and req.pages[:4] == pages
    assert cache.evict(100) == [] or all(p not in pages for p in cache.evict(0))
    req.close()
    cache.unlock(node)
    cache.close()
    assert pool.free_count == 64
