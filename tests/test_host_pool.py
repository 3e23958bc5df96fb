"""Host page manager: allocator order, idempotent free, policies, rollback, sharing, COW and the
step-metadata builder.  The numeric expectations are the reference's own unit tests
(crates/warp34-host/src/cache.rs:628-745, :783-810; radix.rs:1558-1567;
crates/warp34-host/tests/tq4_vision_and_moe.rs:35-80)."""
import ctypes as C

import pytest

from warp34_b200 import ffi
from warp34_b200.kv import PagePool, Sequence, resolve_layer


@pytest.fixture(autouse=True)
def _libs(native_libs):
    return native_libs


def test_row_bytes():
    h = ffi.host()
    exp256 = {ffi.KV_FORMAT_FP16: 512, ffi.KV_FORMAT_BF16: 512, ffi.KV_FORMAT_TQ4: 132,
              ffi.KV_FORMAT_Q8_0: 272, ffi.KV_FORMAT_FP8_E4M3: 264}
    exp128 = {ffi.KV_FORMAT_FP16: 256, ffi.KV_FORMAT_BF16: 256, ffi.KV_FORMAT_TQ4: 66,
              ffi.KV_FORMAT_Q8_0: 136, ffi.KV_FORMAT_FP8_E4M3: 132}
    for f, b in exp256.items():
        assert h.w34_kv_format_row_bytes(f, 256) == b
    for f, b in exp128.items():
        assert h.w34_kv_format_row_bytes(f, 128) == b


def test_policy_layers_and_byte_budgets():
    h = ffi.host()
    tq4 = (ffi.KV_FORMAT_TQ4, ffi.KV_FORMAT_TQ4, 1, 1)
    for layer in range(16):
        assert resolve_layer(ffi.POLICY_FP16, layer, 16) == (0, 0, 0, 0)
        assert resolve_layer(ffi.POLICY_TQ4_ALL, layer, 16) == tq4
        want = tq4 if layer < 12 else (ffi.KV_FORMAT_Q8_0, ffi.KV_FORMAT_Q8_0, 0, 0)
        assert resolve_layer(ffi.POLICY_TQ4, layer, 16) == want
        want8 = tq4 if layer < 12 else (ffi.KV_FORMAT_FP8_E4M3, ffi.KV_FORMAT_FP8_E4M3, 0, 0)
        assert resolve_layer(ffi.POLICY_TQ4, layer, 16, supports_fp8=True) == want8
    assert h.w34_kv_policy_bytes_per_token(ffi.POLICY_TQ4_ALL, 16, 8, 256, 0) == 33792
    # 27B: 16 full-attention layers x 4 kv heads x d256
    assert h.w34_kv_policy_bytes_per_token(ffi.POLICY_FP16, 16, 4, 256, 0) == 65536
    assert h.w34_kv_policy_bytes_per_token(ffi.POLICY_Q8_0, 16, 4, 256, 0) == 34816
    assert h.w34_kv_policy_bytes_per_token(ffi.POLICY_TQ4, 16, 4, 256, 0) == 21376
    assert h.w34_kv_policy_bytes_per_token(ffi.POLICY_TQ4_ALL, 16, 4, 256, 0) == 16896


def test_layout_strides():
    lay = ffi.KvLayerLayout()
    f = (C.c_int32 * 4)(2, 2, 1, 1)
    kb, vb = C.c_uint64(), C.c_uint64()
    assert ffi.host().w34_kv_layout_init(C.byref(lay), 4096, 8192, 0, 3, 4, 256, 16, f, 100,
                                         C.byref(kb), C.byref(vb)) == 0
    assert (lay.k_token_stride_bytes, lay.k_head_stride_bytes, lay.k_page_stride_bytes) == (132, 2112, 8448)
    assert (lay.v_token_stride_bytes, lay.v_head_stride_bytes, lay.v_page_stride_bytes) == (132, 2112, 8448)
    assert kb.value == vb.value == 100 * 8448
    assert lay.layer_id == 3 and lay.block_size == 16 and lay.head_dim == 256


def test_bitmap_ascending_coalescing_and_idempotent_free():
    bm = PagePool(130)
    assert bm.free_count == 130
    for expected in range(130):
        assert bm.alloc_page() == expected
    assert bm.alloc_page() is None and bm.free_count == 0
    for p in (129, 64, 65, 3, 2, 1, 0, 128, 63):
        bm.free_page(p)
    bm.free_page(64)
    bm.free_page(-1)
    bm.free_page(130)
    assert bm.free_count == 9
    assert [bm.alloc_page() for _ in range(9)] == [0, 1, 2, 3, 63, 64, 65, 128, 129]
    assert bm.alloc_page() is None
    bm.reset()
    assert bm.free_count == 130 and bm.alloc_page() == 0


def test_truncate_pages_resets():
    p = PagePool(100)
    for _ in range(10):
        p.alloc_page()
    p.truncate(40)
    assert p.num_pages == 40 and p.free_count == 40
    p.truncate(80)  # growing is ignored
    assert p.num_pages == 40


def test_rollback_frees_uncommitted_tail_but_not_protected_pages():
    pool = PagePool(256)
    for _ in range(120):
        pool.alloc_page()
    req = Sequence(pool)
    req.set_pages_unchecked(list(range(100, 116)), protected_pages=4)
    req.set_committed(200)  # 13 pages needed of the 16 reserved
    assert req.rollback() == [113, 114, 115]
    assert req.num_pages == 13
    assert req.rollback() == []
    req.set_committed(10)  # fewer pages than the protected prefix: keep 4
    freed = req.rollback()
    assert freed == list(range(104, 113)) and req.num_pages == 4


def test_shuffled_free_list_is_seeded_and_withholds_page0():
    a, b, c = PagePool(500), PagePool(500), PagePool(500)
    assert a.shuffle_free_list(7) == 499 and b.shuffle_free_list(7) == 499 and c.shuffle_free_list(8) == 499
    xa = [a.alloc_page() for _ in range(499)]
    xb = [b.alloc_page() for _ in range(499)]
    xc = [c.alloc_page() for _ in range(499)]
    assert xa == xb and xa != xc
    assert sorted(xa) == list(range(1, 500)) and xa != sorted(xa)
    assert a.alloc_page() is None
    a.free_page(xa[10])
    assert a.alloc_page() == xa[10]


def test_reserve_is_all_or_nothing_and_exhaustion_is_an_error_code():
    pool = PagePool(8)
    s = Sequence(pool)
    assert s.reserve(16 * 5) == 5
    assert s.reserve(16 * 5) == 0
    t = Sequence(pool)
    assert t.reserve(16 * 4) == ffi.W34_ERR_EXHAUSTED
    assert pool.free_count == 3 and t.num_pages == 0
    assert t.reserve(16 * 3 - 5) == 3
    assert pool.free_count == 0


def test_prefix_sharing_refcounts_and_release():
    pool = PagePool(64)
    donor = Sequence(pool)
    donor.reserve(64)
    donor.commit(64)
    shared = donor.pages
    readers = [Sequence(pool) for _ in range(3)]
    for r in readers:
        assert r.attach_prefix(shared, 64) == 0
        assert r.protected_pages == 4 and r.committed_len == 64
    assert all(pool.refcount(p) == 4 for p in shared)
    assert pool.stats()["shared"] == 4
    # page-aligned prefix: no copy before the first append, and the new page is private
    r0 = readers[0]
    assert r0.prepare_append() is None
    assert r0.reserve(64 + 20) == 2
    assert all(pool.refcount(p) == 1 for p in r0.pages[4:])
    # speculative tail is rolled back, shared pages survive
    r0.commit(3)
    assert len(r0.rollback()) == 1
    assert r0.num_pages == 5
    for r in readers:
        r.close()
    assert all(pool.refcount(p) == 1 for p in shared)
    donor.close()
    assert pool.free_count == 64


def test_copy_on_write_of_a_shared_partial_tail_page():
    """docs/contracts/cache-layout.md:106-110: a prefix hit that ends inside a shared page gets a
    private copy of that page before new tokens are written."""
    pool = PagePool(32)
    donor = Sequence(pool)
    donor.reserve(4100)  # pool too small: error code, nothing changes
    assert donor.num_pages == 0
    donor.reserve(16 * 4 + 4)
    donor.commit(16 * 4 + 4)  # 5 pages, the last holds 4 rows
    pages = donor.pages
    a = Sequence(pool)
    assert a.attach_prefix(pages, 68) == 0
    assert pool.refcount(pages[4]) == 2
    cow = a.prepare_append()
    assert cow is not None
    src, dst, rows = cow
    assert src == pages[4] and rows == 4 and dst not in pages
    assert a.pages[:4] == pages[:4] and a.pages[4] == dst
    assert pool.refcount(pages[4]) == 1 and pool.refcount(dst) == 1
    assert a.protected_pages == 4
    assert a.prepare_append() is None  # now private
    # the donor, sole owner again, appends in place
    assert donor.prepare_append() is None
    a.close()
    donor.close()
    assert pool.free_count == 32


def test_step_metadata_slots_and_block_tables():
    from warp34_b200.kv import build_step
    pool = PagePool(64)
    pool.shuffle_free_list(3)
    seqs = [Sequence(pool) for _ in range(3)]
    ctx, ql = [37, 0, 16], [1, 5, 4]
    for s, c, q in zip(seqs, ctx, ql):
        assert s.reserve(c + q) >= 0
        s.commit(c)
    b = build_step(seqs, ql, max_blocks_per_req=4, sm_scale=0.0625, device="cpu")
    h = b.host
    assert h["query_start_loc"].tolist() == [0, 1, 6, 10]
    assert h["context_lens_before"].tolist() == ctx
    assert h["seq_lens_after"].tolist() == [38, 5, 20]
    assert b.desc.max_q_len == 5 and b.desc.max_seq_len == 38 and b.desc.total_tokens == 10
    tok = 0
    for i, s in enumerate(seqs):
        pages = s.pages
        assert h["block_tables"][i, :len(pages)].tolist() == pages
        assert (h["block_tables"][i, len(pages):] == 0).all()
        for t in range(ql[i]):
            pos = ctx[i] + t
            assert h["write_slot_mapping"][tok] == pages[pos // 16] * 16 + pos % 16
            tok += 1
    with pytest.raises(RuntimeError):
        build_step(seqs, ql, max_blocks_per_req=2, sm_scale=0.0625, device="cpu")


def test_speculative_batch_commits_accepted_tokens_and_frees_rejected_pages(native_libs):
    """1 + 3 draft tokens per step; a rejected suffix gives its pages back (radix.rs:1234-1245)."""
    from warp34_b200 import kv
    pool = kv.PagePool(64, 16)
    seqs = [kv.Sequence(pool) for _ in range(3)]
    for s, c in zip(seqs, (14, 16, 31)):
        assert s.reserve(c) >= 0
        s.commit(c)
    spec = kv.SpeculativeBatch(seqs)
    free0 = pool.free_count
    added = spec.reserve_ahead(4)           # positions 14..17 | 16..19 | 31..34
    assert added == 1 + 1 + 1
    assert [s.num_pages for s in seqs] == [2, 2, 3]
    freed = spec.commit_and_rollback([1, 4, 1])   # 15 | 20 | 32 committed tokens
    assert [s.committed_len for s in seqs] == [15, 20, 32]
    assert [s.num_pages for s in seqs] == [1, 2, 2]
    assert len(freed) == 2 and pool.free_count == free0 - 1
    # exhaustion is all-or-nothing over the batch
    hog = kv.Sequence(pool)
    assert hog.reserve(16 * (pool.free_count - 1)) >= 0
    before = [s.num_pages for s in seqs]
    with pytest.raises(RuntimeError):
        spec.reserve_ahead(40)
    assert [s.num_pages for s in seqs] == before


def test_step_io_upload_stops_at_the_last_changed_block_table_entry(native_libs):
    """Lengths and slots travel every step; of the block tables only what lies before the last
    changed entry (graph_io.rs:109-195).  Runs on the CPU: both arenas are host tensors."""
    from warp34_b200 import kv
    pool = kv.PagePool(256, 16)
    seqs = [kv.Sequence(pool) for _ in range(4)]
    for s, c in zip(seqs, (15, 16, 40, 100)):
        assert s.reserve(c + 1) >= 0
        s.commit(c)
    io = kv.StepIo(4, 4, 16, device="cpu")
    io.pack(seqs, [1, 1, 1, 1], 0.0625)
    first = io.upload()
    assert first == io.nbytes                      # nothing uploaded before: everything
    assert torch_equal(io.dev, io.host)
    for s in seqs:
        s.commit(1)
        assert s.reserve(s.committed_len + 1) >= 0
    io.pack(seqs, [1, 1, 1, 1], 0.0625)
    second = io.upload()
    head_bytes = 4 * int(io._offs[4])
    # sequence 0 went from 16 to 17 reserved positions (a second page), sequence 1 already had two pages:
    # the copy ends right after entry 1 of row 0
    assert second == head_bytes + 4 * 2
    assert torch_equal(io.dev, io.host)
    for s in seqs:
        s.commit(1)
        assert s.reserve(s.committed_len + 1) >= 0
    io.pack(seqs, [1, 1, 1, 1], 0.0625)
    assert io.upload() == head_bytes             # no table entry changed
    assert torch_equal(io.dev, io.host)


def torch_equal(a, b):
    import torch
    return bool(torch.equal(a, b))
