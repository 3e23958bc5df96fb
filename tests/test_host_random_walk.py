"""Seeded random walks over the host page manager (pool + sequences + prefix cache) against a small
Python model of who holds which page.  Invariants after every operation, in the spirit of the
reference's page-accounting tests (crates/warp34-host/src/radix.rs:1402-1742,
crates/warp34-host/src/cache.rs:396-416):

  * a page's reference count equals the number of holders the model knows (sequences that list it,
    plus one if the cache holds it);
  * free pages + pages with holders = capacity, and no sequence lists a free page;
  * a sequence's pages cover its committed tokens, after a rollback exactly (or its protected prefix);
  * rollback returns only pages nobody else holds and never a protected (shared-prefix) page;
  * the cache's own consistency check passes, and when everything is closed and evicted the pool is
    whole again.
"""
import random

import pytest

from warp34_b200.kv import PagePool, PrefixCache, Sequence


@pytest.fixture(autouse=True)
def _libs(native_libs):
    return native_libs


PAGE = 16


class Model:
    def __init__(self, pool, cache):
        self.pool, self.cache = pool, cache
        self.seqs = []          # dicts: seq, tokens (ids of committed tokens), reserved
        self.cached = set()     # pages the cache holds

    def holders(self):
        h = {}
        for s in self.seqs:
            for p in s["seq"].pages:
                h[p] = h.get(p, 0) + 1
        for p in self.cached:
            h[p] = h.get(p, 0) + 1
        return h

    def check(self):
        h = self.holders()
        cap = self.pool.num_pages
        for p, n in h.items():
            assert self.pool.refcount(p) == n, (p, self.pool.refcount(p), n)
        assert self.pool.free_count + len(h) == cap
        for s in self.seqs:
            q = s["seq"]
            assert q.committed_len == len(s["tokens"])
            assert q.num_pages * PAGE >= q.committed_len
            assert q.protected_pages <= q.num_pages
        assert self.cache.sanity_check() == 0


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_walk_keeps_page_accounting_exact(seed):
    rng = random.Random(seed)
    pool = PagePool(96)
    cache = PrefixCache(pool)
    m = Model(pool, cache)
    vocab = 50
    docs = [[rng.randrange(vocab) for _ in range(96)] for _ in range(3)]   # prompts start as one of these
    hits = 0
    for step in range(400):
        op = rng.choice(["new", "new", "grow", "grow", "grow", "spec", "finish", "evict"])
        if op == "new" and len(m.seqs) < 10:
            prompt = rng.choice(docs)[:rng.randrange(1, 90)] + [rng.randrange(vocab) for _ in range(rng.randrange(0, 20))]
            pages, matched, node = cache.match_prefix(prompt[:-1])
            hits += matched > 0
            seq = Sequence(pool)
            if matched:
                cache.lock(node)
                assert seq.attach_prefix(pages, matched) == 0
                assert set(pages) <= m.cached
            if seq.reserve(len(prompt)) < 0:      # pool exhausted: nothing may have changed
                assert seq.num_pages == len(pages) if matched else seq.num_pages == 0
                seq.close()
                if matched:
                    cache.unlock(node)
                m.check()
                continue
            cow = seq.prepare_append()
            assert cow is None                    # prefixes from the cache are page aligned
            seq.commit(len(prompt) - matched)
            m.seqs.append(dict(seq=seq, tokens=list(prompt), node=node if matched else None))
        elif op == "grow" and m.seqs:
            s = rng.choice(m.seqs)
            n = rng.randrange(1, 20)
            if s["seq"].reserve(len(s["tokens"]) + n) >= 0:
                s["seq"].commit(n)
                s["tokens"] += [rng.randrange(vocab) for _ in range(n)]
        elif op == "spec" and m.seqs:
            s = rng.choice(m.seqs)
            before = set(s["seq"].pages)
            protected = set(s["seq"].pages[:s["seq"].protected_pages])
            draft = rng.randrange(1, 40)
            if s["seq"].reserve(len(s["tokens"]) + draft) >= 0:
                accepted = rng.randrange(0, draft + 1)
                s["seq"].commit(accepted)
                s["tokens"] += [rng.randrange(vocab) for _ in range(accepted)]
                freed = s["seq"].rollback()
                assert not (set(freed) & protected)
                assert all(pool.refcount(p) == 0 for p in freed)
                assert s["seq"].num_pages == (len(s["tokens"]) + PAGE - 1) // PAGE or \
                    s["seq"].num_pages == s["seq"].protected_pages
                assert set(s["seq"].pages) <= before | set(s["seq"].pages)
        elif op == "finish" and m.seqs:
            s = m.seqs.pop(rng.randrange(len(m.seqs)))
            full_pages = len(s["tokens"]) // PAGE
            if full_pages and rng.random() < 0.8:
                toks = s["tokens"][:full_pages * PAGE]
                cache.insert(toks, s["seq"].pages[:full_pages])
                pages, matched, _ = cache.match_prefix(toks)
                assert matched == len(toks)
                m.cached |= set(pages)
            s["seq"].close()
            if s["node"] is not None:
                cache.unlock(s["node"])
        elif op == "evict":
            gone = cache.evict(rng.randrange(0, 12))
            assert set(gone) <= m.cached
            in_use = set()
            for s in m.seqs:
                in_use |= set(s["seq"].pages)
            assert not (set(gone) & in_use)       # locked paths are never evicted
            m.cached -= set(gone)
        m.check()
    for s in m.seqs:
        s["seq"].close()
        if s["node"] is not None:
            cache.unlock(s["node"])
    m.seqs = []
    m.cached -= set(cache.evict(10 ** 6))
    m.check()
    assert not m.cached
    assert hits >= 10   # the walk did share prefixes
    cache.close()
    assert pool.free_count == pool.num_pages


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_persistent_step_arena_always_equals_a_fresh_pack(seed):
    """StepIo packs into a persistent arena and uploads only what changed (lengths and slots every
    step, block tables up to the last changed entry).  Over a random walk of growing, rolled-back
    and replaced sequences the device-side copy must always equal what a from-scratch pack of the
    same step produces (graph_io.rs:109-195, :368-420)."""
    from warp34_b200 import kv
    rng = random.Random(seed)
    pool = PagePool(512)
    n, max_q, max_blocks = 6, 4, 24
    seqs = [Sequence(pool) for _ in range(n)]
    for s in seqs:
        c = rng.randrange(1, 200)
        assert s.reserve(c + max_q) >= 0
        s.commit(c)
    io = kv.StepIo(n, n * max_q, max_blocks, device="cpu")
    full_bytes = 0
    for step in range(120):
        q_lens = [rng.randrange(1, max_q + 1) for _ in range(n)]
        for s, q in zip(seqs, q_lens):
            if s.reserve(s.committed_len + q) < 0 or s.num_pages > max_blocks:
                # start over as a fresh short request in the same row
                s.rollback()
                s.set_committed(0)
                s.rollback()
                assert s.reserve(rng.randrange(1, 40) + q) >= 0
                s.commit(s.num_pages * PAGE - PAGE if s.num_pages > 1 else 0)
                assert s.reserve(s.committed_len + q) >= 0
        io.pack(seqs, q_lens, 0.0625)
        full_bytes -= io.upload()
        fresh = kv.build_step(seqs, q_lens, max_blocks, 0.0625, device="cpu")
        total = sum(q_lens)
        d = io.desc
        assert (d.num_reqs, d.total_tokens, d.max_q_len) == (n, total, max(q_lens))
        assert d.max_seq_len == fresh.desc.max_seq_len
        arena, offs = io.dev.numpy(), io._offs   # the device-side copy after the partial upload
        got = {"query_start_loc": arena[offs[0]:offs[0] + n + 1], "context_lens_before": arena[offs[1]:offs[1] + n],
               "seq_lens_after": arena[offs[2]:offs[2] + n], "write_slot_mapping": arena[offs[3]:offs[3] + total],
               "block_tables": arena[offs[4]:offs[4] + n * max_blocks].reshape(n, max_blocks)}
        for key in ("query_start_loc", "context_lens_before", "seq_lens_after", "write_slot_mapping"):
            assert (got[key] == fresh.host[key]).all(), key
        # live part of every block-table row; entries past a row's pages are never read
        for r, s in enumerate(seqs):
            assert (got["block_tables"][r, :s.num_pages] == fresh.host["block_tables"][r, :s.num_pages]).all()
        full_bytes += io.nbytes
        # accept a random part of the step's tokens, hand the rest back
        for s, q in zip(seqs, q_lens):
            s.commit(rng.randrange(0, q + 1))
            s.rollback()
    assert full_bytes > 0   # the partial uploads moved fewer bytes than full ones would have
    for s in seqs:
        s.close()
    assert pool.free_count == pool.num_pages
