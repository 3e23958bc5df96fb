"""GPU parity tests, all through the C ABI (include/warp34_b200.h).

Append: packed codes, scales and untouched bytes are compared bit-for-bit with the golden fixture
written by the reference's kernels, and with the reference library itself when
oracle/_ref/libwarp34_ref.so travelled with the repository.  Attention: |a-b| <= 2e-3 + 1e-2|b|
against the reference's scalar dequant-then-attend output (fixture) and the CPU oracle.
The relational tests follow the reference's own (page-permutation invariance:
crates/warp34-host/tests/backbone_and_collectives.rs:453-572; masks and sentinels:
crates/warp34-host/src/cuda/tests.rs:538-572, tests/paged_fa2.rs:521-691)."""
import ctypes as C
import os

import numpy as np
import pytest

from util import GOLDEN, f16, fast_parity, host_layout, parity_stats, plain_parity, tq4_rows_equal_up_to_scale_ulp, within_tol

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

HAVE_GOLDEN = os.path.exists(GOLDEN)


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    ex = kv.Executor(64 << 20)
    return dict(ffi=ffi, kv=kv, synth=synth, ex=ex, lib=native_libs[0])


@pytest.fixture(scope="module")
def ref_lib(env):
    import oracle
    p = oracle.ref_lib_path()
    if p is None:
        pytest.skip("reference kernels not built (oracle/_ref)")
    return env["ffi"].bind_kernel_abi(p)


def _golden_workload(env, fx, fill=0x5A):
    """Rebuilds the fixture's pool geometry: same pages, same slots."""
    kv, synth = env["kv"], env["synth"]
    layer = kv.KvLayer(int(fx["num_pages"]), int(fx["hkv"]), fill=fill)
    return layer


def _batch(env, fx, tag, slots=None, **kw):
    kv = env["kv"]
    if tag == "app":
        return kv.StepBatch(fx["app_qsl"], fx["app_ctx"], fx["app_seq"], fx["app_bt"], fx["app_slots"],
                            fx["app_bt"].shape[1], 0.0625, **kw)
    n = int(fx[f"{tag}_query_start_loc"][-1])
    return kv.StepBatch(fx[f"{tag}_query_start_loc"], fx[f"{tag}_context_lens_before"],
                        fx[f"{tag}_seq_lens_after"], fx[f"{tag}_block_tables"],
                        np.full(n, -1, np.int32) if slots is None else slots,
                        fx[f"{tag}_block_tables"].shape[1], 0.0625, **kw)


@pytest.mark.skipif(not HAVE_GOLDEN, reason="golden fixture missing")
def test_append_is_bit_exact_with_reference_fixture(env):
    fx = np.load(GOLDEN)
    kv = env["kv"]
    layer = _golden_workload(env, fx)
    b = _batch(env, fx, "app")
    k = torch.from_numpy(fx["k_in"].view(np.float16)).cuda()
    v = torch.from_numpy(fx["v_in"].view(np.float16)).cuda()
    kv.kv_cache_write(env["ex"], layer, b, k, v)
    torch.cuda.synchronize()
    assert (layer.k.cpu().numpy() == fx["k_pool"]).all()
    assert (layer.v.cpu().numpy() == fx["v_pool"]).all()


def test_append_is_bit_exact_with_reference_kernels_cfg0(env, ref_lib):
    """Config 0 of the benchmark: 4 sequences, contexts in [1024, 4096], 4 KV heads, shuffled pages."""
    kv, synth = env["kv"], env["synth"]
    ctx = synth.context_lengths(4, 1024, 4096, 0)
    T = int(ctx.sum())
    k, v = synth.make_kv(T, 4, 0)
    kd, vd = k.cuda(), v.cuda()
    pools = []
    for lib in (None, ref_lib):
        wl = synth.PagedWorkload([0] * 4, [int(c) for c in ctx], 4, seed=0, fill=0xA5)
        kv.kv_cache_write(env["ex"], wl.layer, wl.step(), kd, vd, lib=lib)
        torch.cuda.synchronize()
        pools.append((wl.layer.k.cpu().numpy(), wl.layer.v.cpu().numpy(), wl))
    assert (pools[0][0] == pools[1][0]).all() and (pools[0][1] == pools[1][1]).all()
    # and the CPU oracle agrees except for rare last-place differences of the fp16 scales
    import oracle
    wl = pools[0][2]
    hk, hv = np.full_like(pools[0][0], 0xA5), np.full_like(pools[0][1], 0xA5)
    lay = host_layout(wl.layer.layout, hk, hv)
    assert oracle.kv_cache_write(lay, wl.step().host_desc(), k.numpy().view(np.uint16),
                                 v.numpy().view(np.uint16), 1024, 1024, nthreads=8) == 0
    for got, want in ((hk, pools[0][0]), (hv, pools[0][1])):
        code_mism, scale_mism, ulp = tq4_rows_equal_up_to_scale_ulp(got, want)
        assert code_mism <= 2 and ulp <= 1 and scale_mism <= got.size // 66 // 2000 + 2


def test_append_masks_strides_and_sentinels(env):
    """valid_token_mask / valid_req_mask / negative slots have no side effects, K and V may be
    column slices of one packed activation, and bytes outside written rows are untouched."""
    kv, synth, ffi = env["kv"], env["synth"], env["ffi"]
    hkv, T = 2, 37
    packed = torch.zeros(T, 3 * hkv * 256 + 64, dtype=torch.float16)
    k, v = synth.make_kv(T, hkv, 77)
    packed[:, 512:512 + hkv * 256] = k
    packed[:, 512 + hkv * 256:512 + 2 * hkv * 256] = v
    pd = packed.cuda()
    kview, vview = pd[:, 512:512 + hkv * 256], pd[:, 512 + hkv * 256:512 + 2 * hkv * 256]
    qsl = [0, 10, 10, 30, 37]
    slots = np.array([16 * (5 + t // 16) + t % 16 for t in range(T)], np.int32)
    slots[3] = -1
    vtm = np.ones(T, np.uint8)
    vtm[7] = 0
    vrm = np.array([1, 1, 1, 0], np.uint8)  # last request (tokens 30..36) masked
    bt = np.zeros((4, 4), np.int32)

    def run(masked):
        layer = kv.KvLayer(12, hkv, fill=0x55)
        b = kv.StepBatch(qsl, [0, 0, 0, 0], [10, 0, 20, 7], bt, slots, 4, 0.0625,
                         valid_token_mask=vtm if masked else None, valid_req_mask=vrm if masked else None)
        kv.kv_cache_write(env["ex"], layer, b, kview, vview, k_row_stride=pd.stride(0), v_row_stride=pd.stride(0))
        torch.cuda.synchronize()
        return layer.k.cpu().numpy().reshape(12, hkv, 16, 132), layer.v.cpu().numpy().reshape(12, hkv, 16, 132)

    km, vm = run(True)
    # contiguous inputs give the same bytes as the strided views
    layer2 = kv.KvLayer(12, hkv, fill=0x55)
    s2 = slots.copy()
    b2 = kv.StepBatch(qsl, [0] * 4, [10, 0, 20, 7], bt, s2, 4, 0.0625)
    kv.kv_cache_write(env["ex"], layer2, b2, k.cuda(), v.cuda())
    torch.cuda.synchronize()
    kc = layer2.k.cpu().numpy().reshape(12, hkv, 16, 132)
    vc = layer2.v.cpu().numpy().reshape(12, hkv, 16, 132)
    for t in range(T):
        page, off = 5 + t // 16, t % 16
        skipped = t == 3 or t == 7 or t >= 30
        for h in range(hkv):
            if skipped:
                assert (km[page, h, off] == 0x55).all() and (vm[page, h, off] == 0x55).all()
            else:
                assert (km[page, h, off] == kc[page, h, off]).all() and (vm[page, h, off] == vc[page, h, off]).all()
    untouched = np.ones(12, bool)
    untouched[5:8] = False
    assert (km[untouched] == 0x55).all() and (vm[untouched] == 0x55).all()
    assert (km[7, :, 5:] == 0x55).all()  # rows past the last token of page 7
    # stride below heads * 256 is rejected
    rc = env["lib"].warp34_kv_cache_write_strided(C.byref(env["ex"].ex), C.byref(layer2.layout), C.byref(b2.desc),
                                                  k.cuda().data_ptr(), v.cuda().data_ptr(), 256, 512)
    assert rc == ffi.CUDA_ERROR_INVALID_VALUE


@pytest.mark.skipif(not HAVE_GOLDEN, reason="golden fixture missing")
@pytest.mark.parametrize("tag", ["dec", "ver"])
@pytest.mark.parametrize("scalar", [False, True])
def test_attention_matches_reference_dequant_then_attend(env, tag, scalar):
    fx = np.load(GOLDEN)
    kv = env["kv"]
    layer = _golden_workload(env, fx)
    layer.k.copy_(torch.from_numpy(fx["k_pool"]))
    layer.v.copy_(torch.from_numpy(fx["v_pool"]))
    b = _batch(env, fx, tag)
    q = torch.from_numpy(fx[f"q_{tag}"].view(np.float16)).cuda()
    out = torch.zeros_like(q)
    kv.paged_attention(env["ex"], layer, b, q, out, int(fx["hq"]), scalar=scalar)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    want = f16(fx[f"out_{tag}"])
    if scalar:
        ok = within_tol(got, want)
        assert ok.all(), f"{(~ok).sum()} of {ok.size} outside tolerance, max abs {np.abs(got - want).max()}"
    else:
        ok, msg = plain_parity(got, want)
        assert ok, msg
        # the fast build stays at least as close to dequant-then-attend as the reference's own
        # tensor-core kernel, whose output on the same inputs is in the fixture
        fast = kv.Executor(64 << 20)
        fast.ex.flags = env["ffi"].EXEC_FLAG_FAST_ATTENTION
        out_f = torch.zeros_like(q)
        kv.paged_attention(fast, layer, b, q, out_f, int(fx["hq"]))
        torch.cuda.synchronize()
        ref_viol, ref_worst = parity_stats(f16(fx[f"out_{tag}_prod"]), want)
        my_viol, my_worst = parity_stats(out_f.float().cpu().numpy(), want)
        assert my_viol <= ref_viol + 2 and my_worst <= max(1.0, 1.25 * ref_worst), (my_viol, my_worst, ref_viol, ref_worst)


def _decode_case(env, ctx, hq, hkv, seed, q_lens=None, shuffle=True, fill=None):
    kv, synth = env["kv"], env["synth"]
    q_lens = q_lens or [1] * len(ctx)
    wl = synth.PagedWorkload([0] * len(ctx), [int(c) for c in ctx], hkv, seed=seed, shuffle=shuffle, fill=fill)
    k, v = synth.make_kv(int(sum(ctx)), hkv, seed)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c, ql in zip(wl.seqs, ctx, q_lens):
        s.commit(int(c) - ql)
    q = synth.make_q(sum(q_lens), hq, seed)
    return wl, q


def _oracle_attention(wl, batch, q, hq, nthreads=8):
    import oracle
    hk, hv = wl.layer.k.cpu().numpy(), wl.layer.v.cpu().numpy()
    lay = host_layout(wl.layer.layout, hk, hv)
    out = np.zeros((q.shape[0], hq, 256), np.uint16)
    assert oracle.paged_attention(lay, batch.host_desc(), q.numpy().view(np.uint16), out, hq, nthreads=nthreads) == 0
    return f16(out)


@pytest.mark.parametrize("hq,hkv,q_len", [(16, 4, 1), (24, 4, 1), (24, 4, 4), (8, 8, 1), (20, 2, 3)])
def test_attention_matches_cpu_oracle_on_ragged_batches(env, hq, hkv, q_len):
    kv = env["kv"]
    ctx = [1, 15, 16, 17, 250, 1000, 33]
    ctx = [max(c, q_len) for c in ctx]
    wl, q = _decode_case(env, ctx, hq, hkv, seed=100 + hq + q_len, q_lens=[q_len] * len(ctx))
    b = wl.step(q_lens=[q_len] * len(ctx))
    out = torch.full((q.shape[0], hq, 256), 9.0, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
    torch.cuda.synchronize()
    want = _oracle_attention(wl, b, q, hq)
    got = out.float().cpu().numpy()
    ok, msg = plain_parity(got, want)
    assert ok, msg
    status = int(env["ex"].scratch[:4].cpu().numpy().view(np.int32)[0])
    assert status == 0
    # the fp32 path, selected by the exec flag, meets the plain elementwise bound
    precise = kv.Executor(1 << 20)
    precise.ex.flags = env["ffi"].EXEC_FLAG_PRECISE_ATTENTION
    out2 = torch.zeros_like(out)
    kv.paged_attention(precise, wl.layer, b, q.cuda(), out2, hq)
    torch.cuda.synchronize()
    ok2 = within_tol(out2.float().cpu().numpy(), want)
    assert ok2.all(), f"fp32 path: {(~ok2).sum()} of {ok2.size} outside tolerance"


def test_page_permutation_invariance_is_zero_ulp(env):
    """Same tokens at pages [1,2,3,...] and at a shuffled placement: identical output bits."""
    kv = env["kv"]
    ctx, hq, hkv = [40, 700], 8, 2
    outs = []
    for shuffle in (False, True):
        wl, q = _decode_case(env, ctx, hq, hkv, seed=9, shuffle=shuffle)
        b = wl.step(q_lens=[1, 1])
        out = torch.zeros(2, hq, 256, dtype=torch.float16, device="cuda")
        kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy().view(np.uint16))
        pages = [s.pages for s in wl.seqs]
    assert pages[0] != sorted(pages[0])
    assert (outs[0] == outs[1]).all()


def test_masks_windows_and_untouched_rows(env):
    """Masked tokens / requests leave their output rows untouched; sliding window and the
    non-causal window mode agree with the CPU oracle."""
    kv = env["kv"]
    ctx, hq, hkv, ql = [90, 41, 300], 8, 2, 3
    wl, q = _decode_case(env, ctx, hq, hkv, seed=21, q_lens=[ql] * 3)
    sentinel = np.float16(0.0).view(np.uint16) + 0x5500
    for mode, window in ((0, 0), (0, 33), (1, 50), (1, 0)):
        vtm = np.ones(9, np.uint8)
        vtm[4] = 0
        vrm = np.array([1, 1, 0], np.uint8)
        b = wl.step(q_lens=[ql] * 3, mask_mode=mode, sliding_window=window, valid_token_mask=vtm, valid_req_mask=vrm)
        out = torch.from_numpy(np.full((9, hq, 256), sentinel, np.uint16).view(np.float16)).cuda()
        kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
        torch.cuda.synchronize()
        got_bits = out.cpu().numpy().view(np.uint16)
        assert (got_bits[4] == sentinel).all() and (got_bits[6:] == sentinel).all()
        want = _oracle_attention(wl, b, q, hq)
        live = [0, 1, 2, 3, 5]
        ok, msg = plain_parity(f16(got_bits[live]), want[live])
        assert ok, (mode, window, msg)


def test_block_table_entries_past_the_sequence_are_never_used(env):
    """Entries beyond ceil(seq_len / 16) point at a page whose scales are NaN: any use of them
    would poison the output (the reference's tight-block-table test, tests/paged_fa2.rs:521-616)."""
    kv = env["kv"]
    ctx, hq, hkv = [37, 64], 8, 2
    wl, q = _decode_case(env, ctx, hq, hkv, seed=31)
    poison = wl.pool.alloc_page()
    kview = wl.layer.k.view(wl.num_pages, -1)
    vview = wl.layer.v.view(wl.num_pages, -1)
    kview[poison] = 0x7E
    vview[poison] = 0x7E  # fp16 0x7e7e is NaN
    b = wl.step(q_lens=[1, 1])
    bt = b.host["block_tables"].copy()
    for i, c in enumerate(ctx):
        bt[i, (c + 15) // 16:] = poison
    b2 = kv.StepBatch(b.host["query_start_loc"], b.host["context_lens_before"], b.host["seq_lens_after"], bt,
                      b.host["write_slot_mapping"], bt.shape[1], 0.0625)
    out = torch.zeros(2, hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b2, q.cuda(), out, hq)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    ok, msg = plain_parity(got, _oracle_attention(wl, b, q, hq))
    assert ok, msg


def test_small_scratch_and_odd_strides_fall_back_to_the_scalar_kernel(env):
    kv, ffi = env["kv"], env["ffi"]
    ctx, hq, hkv = [100, 20], 8, 2
    wl, q = _decode_case(env, ctx, hq, hkv, seed=41)
    b = wl.step(q_lens=[1, 1])
    want = _oracle_attention(wl, b, q, hq)
    tiny = kv.Executor(4096)
    out = torch.zeros(2, hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(tiny, wl.layer, b, q.cuda(), out, hq)
    torch.cuda.synchronize()
    assert within_tol(out.float().cpu().numpy(), want).all()
    # empty batch: success, nothing launched, output untouched
    empty = ffi.AttentionBatch()
    rc = env["lib"].warp34_paged_attention_f16(C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(empty),
                                               q.cuda().data_ptr(), out.data_ptr(), hq)
    assert rc == 0


def test_split_partitioning_does_not_change_the_result_beyond_tolerance(env):
    """The same step with scratch for 12 worker warps and for the full grid: different
    cuts of the KV stream, same answer (merge algebra of op_paged_attn.cu:1168-1202)."""
    kv = env["kv"]
    ctx, hq, hkv = [5000, 1234, 16, 9000], 24, 4
    wl, q = _decode_case(env, ctx, hq, hkv, seed=51)
    b = wl.step(q_lens=[1] * 4)
    outs = []
    need_min = 4096 + (12 + 4 * 8) * (8 * 256 + 16) * 4 + (24 * 2064 * 4)
    for ex in (env["ex"], kv.Executor(need_min)):
        out = torch.zeros(4, hq, 256, dtype=torch.float16, device="cuda")
        kv.paged_attention(ex, wl.layer, b, q.cuda(), out, hq)
        torch.cuda.synchronize()
        outs.append(out.float().cpu().numpy())
    want = _oracle_attention(wl, b, q, hq)
    for o in outs:
        ok, msg = plain_parity(o, want)
        assert ok, msg
    assert np.abs(outs[0] - outs[1]).max() <= 2e-3 + 1e-2 * np.abs(want).max()


@pytest.mark.parametrize("case", ["many_short_requests_2mib", "decode_batch_8mib", "draft_tokens_masks_4mib", "fast_flag_4mib"])
def test_a_workspace_too_small_for_the_batch_serves_it_in_several_passes(env, case):
    """A workspace that cannot hold a partial slot and the query fragments of every (request, kv head) next to
    a useful number of worker slots (the reference's engine guarantees 8 MiB, op_paged_attn.cu:1301-1315) is
    used for some of the requests at a time: plan, stream and merge per part.  Same bound as one pass; the
    status word shows that the split-KV kernels ran and the plan header that the last pass held fewer items
    than the batch."""
    kv, ffi = env["kv"], env["ffi"]
    rng = np.random.default_rng(77)
    hq, hkv = 24, 4
    if case == "many_short_requests_2mib":
        ctx, q_lens, scratch, flags, kw = [int(x) for x in rng.integers(1, 200, size=400)], None, 2 << 20, 0, {}
    elif case == "decode_batch_8mib":
        ctx, q_lens, scratch, flags, kw = [int(x) for x in rng.integers(500, 3000, size=64)], None, 8 << 20, 0, {}
    elif case == "draft_tokens_masks_4mib":
        q_lens = [int(x) for x in rng.integers(1, 4, size=90)]           # 1 to 3 tokens: up to 18 rows per kv head
        ctx = [int(q + rng.integers(0, 700)) for q in q_lens]
        vtm = (rng.random(sum(q_lens)) > 0.2).astype(np.uint8)
        vrm = (rng.random(90) > 0.1).astype(np.uint8)
        scratch, flags, kw = 4 << 20, 0, dict(valid_token_mask=vtm, valid_req_mask=vrm, sliding_window=300)
    else:
        q_lens = [4] * 40                                                 # fast flag: four-warp teams, 24 rows per item
        ctx = [int(4 + rng.integers(0, 900)) for _ in q_lens]
        scratch, flags, kw = 4 << 20, ffi.EXEC_FLAG_FAST_ATTENTION, {}
    wl, q = _decode_case(env, ctx, hq, hkv, seed=61, q_lens=q_lens)
    b = wl.step(q_lens=q_lens or [1] * len(ctx), **kw)
    T = q.shape[0]
    outs = {}
    for name, ex, fl in (("small", kv.Executor(scratch), flags), ("fp32", kv.Executor(1 << 20), ffi.EXEC_FLAG_PRECISE_ATTENTION)):
        ex.ex.flags = fl
        ex.scratch[:16].fill_(0x7f)
        out = torch.full((T, hq, 256), 0, dtype=torch.int16, device="cuda")
        out.fill_(0x5500)
        kv.paged_attention(ex, wl.layer, b, q.cuda(), out.view(torch.float16), hq)
        torch.cuda.synchronize()
        outs[name] = out.cpu().numpy().view(np.uint16)
        if name == "small":
            hdr = ex.scratch[:16].cpu().numpy().view(np.int32)
            assert hdr[0] == 0, "status: the split-KV kernels did not run or reported a failure"
            whole = hkv * sum(-(-(ql * (hq // hkv)) // (24 if flags else 8)) for ql in (q_lens or [1] * len(ctx)))
            assert 0 < hdr[1] < whole, (int(hdr[1]), whole)      # items of the last pass < items of the batch
    untouched = (outs["fp32"] == 0x5500).all(axis=(1, 2))
    assert ((outs["small"] == 0x5500).all(axis=(1, 2)) == untouched).all(), "masked rows differ"
    got, want = f16(outs["small"][~untouched]), f16(outs["fp32"][~untouched])
    ok, msg = (fast_parity if flags else plain_parity)(got, want)
    assert ok, (case, msg)


@pytest.mark.parametrize("q_len,flag", [(1, None), (4, None), (4, "EXEC_FLAG_FAST_ATTENTION"), (60, None),
                                        (60, "EXEC_FLAG_FAST_ATTENTION"), (1, "EXEC_FLAG_PRECISE_ATTENTION")])
def test_context_lens_before_may_be_null(env, q_len, flag):
    """The descriptor's context_lens_before is optional (the context is then seq_lens_after minus the query
    length, op_paged_attn.cu:266-280): every kernel family gives the same bits with and without it."""
    kv, ffi = env["kv"], env["ffi"]
    ctx, hq, hkv = [300, 77, 1200], 24, 4
    wl, q = _decode_case(env, ctx, hq, hkv, seed=71, q_lens=[q_len] * 3)
    b = wl.step(q_lens=[q_len] * 3)
    ex = kv.Executor(64 << 20)
    ex.ex.flags = getattr(ffi, flag) if flag else 0
    outs = []
    for null in (False, True):
        if null:
            b.desc.context_lens_before = None
        out = torch.zeros(3 * q_len, hq, 256, dtype=torch.float16, device="cuda")
        kv.paged_attention(ex, wl.layer, b, q.cuda(), out, hq)
        torch.cuda.synchronize()
        outs.append(out.view(torch.int16).cpu())
    assert outs[0].numpy().any()
    assert torch.equal(outs[0], outs[1])


def test_understated_max_q_len_is_reported_and_the_declared_rows_stay_right(env):
    """batch.max_q_len sizes the store of prepared query fragments.  A request with more query
    tokens than it declares keeps its first row group (8 rows: 2 tokens x 4 heads here), the rest
    is dropped and bit 2 of the status word at the head of the scratch says so."""
    kv = env["kv"]
    hq, hkv = 8, 2
    wl, q = _decode_case(env, [300, 200], hq, hkv, seed=83, q_lens=[3, 1])
    honest = wl.step(q_lens=[3, 1])
    want = _oracle_attention(wl, honest, q, hq)
    lied = wl.step(q_lens=[3, 1], max_q_len=1)
    out = torch.full((4, hq, 256), 7.0, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, lied, q.cuda(), out, hq)
    torch.cuda.synchronize()
    status = int(env["ex"].scratch[:4].cpu().numpy().view(np.int32)[0])
    assert status & 4
    got = out.float().cpu().numpy()
    for tok in (0, 1, 3):   # the first group of request 0, and request 1
        ok, msg = plain_parity(got[tok:tok + 1], want[tok:tok + 1])
        assert ok, (tok, msg)
    assert (got[2] == 7.0).all()
    # declared honestly the same batch is complete and the status clear
    kv.paged_attention(env["ex"], wl.layer, honest, q.cuda(), out, hq)
    torch.cuda.synchronize()
    assert int(env["ex"].scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
    ok, msg = plain_parity(out.float().cpu().numpy(), want)
    assert ok, msg


def test_page_sharded_partials_merge_to_the_unsharded_result(env):
    """One sequence cut into page ranges (as the GPUs of the 256K configuration hold it): every
    shard emits un-normalised (acc, m, l) triples, the merge reproduces single-pass attention."""
    kv = env["kv"]
    ctx, hq, hkv = [3000], 16, 4
    wl, q = _decode_case(env, ctx, hq, hkv, seed=61)
    b = wl.step(q_lens=[1])
    whole = torch.zeros(1, hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), whole, hq)
    pages = wl.seqs[0].pages
    cuts = [0, 64, 65, len(pages)]  # three shards of 64, 1 and the remaining pages
    triples = torch.zeros(3, 1 * hq, 258, dtype=torch.float32, device="cuda")
    for g in range(3):
        p0, p1 = cuts[g], cuts[g + 1]
        n_tok = min(ctx[0], p1 * 16) - p0 * 16
        bt = np.zeros((1, len(pages)), np.int32)
        bt[0, :p1 - p0] = pages[p0:p1]
        sb = kv.StepBatch([0, 1], [n_tok - 1], [n_tok], bt, [-1], len(pages), 0.0625)
        kv.paged_attention_partial(env["ex"], wl.layer, sb, q.cuda(), triples[g], hq)
    merged = torch.zeros(1, hq, 256, dtype=torch.float16, device="cuda")
    kv.merge_shards(env["ex"], triples, merged)
    torch.cuda.synchronize()
    want = _oracle_attention(wl, b, q, hq)
    ok, msg = plain_parity(merged.float().cpu().numpy(), want)
    assert ok, msg
    diff = np.abs(merged.float().cpu().numpy() - whole.float().cpu().numpy())
    assert diff.max() <= 2e-3 + 1e-2 * np.abs(want).max()
    # a shard without keys contributes nothing
    triples2 = torch.cat([triples, torch.zeros(1, hq, 258, device="cuda")])
    merged2 = torch.zeros_like(merged)
    kv.merge_shards(env["ex"], triples2, merged2)
    torch.cuda.synchronize()
    assert (merged2.cpu().numpy().view(np.uint16) == merged.cpu().numpy().view(np.uint16)).all()


def test_masked_rows_stay_untouched_through_the_sharded_path(env):
    """A masked request's rows carry "no keys" triples out of every shard, and the cross-shard
    merge leaves its output rows as they were."""
    kv = env["kv"]
    ctx, hq, hkv = [700, 400], 16, 4
    wl, q = _decode_case(env, ctx, hq, hkv, seed=62)
    vrm = np.array([1, 0], np.uint8)
    b = wl.step(q_lens=[1, 1], valid_req_mask=vrm)
    triples = torch.full((2, 2 * hq, 258), 7.0, dtype=torch.float32, device="cuda")   # stale contents
    for g in range(2):
        kv.paged_attention_partial(env["ex"], wl.layer, b, q.cuda(), triples[g], hq)
    merged = torch.full((2, hq, 256), 0, dtype=torch.int16, device="cuda")
    merged.fill_(0x5500)
    kv.merge_shards(env["ex"], triples, merged.view(torch.float16))
    torch.cuda.synchronize()
    t = triples.cpu().numpy().reshape(2, 2, hq, 258)
    assert (t[:, 1, :, 257] == 0).all() and (t[:, 1, :, :256] == 0).all()
    bits = merged.cpu().numpy().view(np.uint16)
    assert (bits[1] == 0x5500).all(), "masked request's rows were written"
    # two identical shards merge to the single-pass result of the live request
    want = _oracle_attention(wl, b, q, hq)
    ok, msg = plain_parity(f16(bits[0:1]), want[0:1])
    assert ok, msg


def _mailbox_views(kv, buf, world, max_rows):
    n_in = 2 * world * max_rows * 258 * 4
    inbox = buf[:n_in].view(torch.float32).view(2, world, max_rows, 258)
    flags = buf[n_in:n_in + world * max_rows * 4].view(torch.int32).view(world, max_rows)
    return inbox, flags


def test_exchange_merge_over_mailboxes_equals_the_gathered_merge(env):
    """Three ranks played one after another on one device (kernels that wait on one another never
    run side by side on one GPU): before rank r runs, the host plays the stores of the ranks that
    have not run yet; ranks that have run delivered theirs through the kernel.  Rank 2's inbox is
    filled by kernels only.  Every rank's output must equal the merge of the gathered triples
    bit for bit, over several steps (both mailbox parities, the device-side step counter)."""
    kv = env["kv"]
    world, rows, max_rows = 3, 10, 12
    g = torch.Generator(device="cuda")
    g.manual_seed(99)
    bufs = [torch.zeros(kv.PeerExchange.mailbox_bytes(world, max_rows), dtype=torch.uint8, device="cuda")
            for _ in range(world)]
    px = [kv.PeerExchange.over_buffers(r, max_rows, bufs, wait_limit=2000) for r in range(world)]
    for step in range(1, 5):
        triples = torch.randn(world, rows, 258, generator=g, device="cuda")
        triples[:, :, 256] = torch.randn(world, rows, generator=g, device="cuda") * 4.0  # m
        triples[:, :, 257] = torch.rand(world, rows, generator=g, device="cuda") + 0.1   # l > 0
        if step == 3:
            triples[1, :, 257] = 0.0  # a shard without keys
        want = torch.zeros(rows, 256, dtype=torch.float16, device="cuda")
        kv.merge_shards(env["ex"], triples, want)
        for r in range(world):
            inbox, flags = _mailbox_views(kv, bufs[r], world, max_rows)
            for w in range(r + 1, world):  # peers that have not run this step yet
                inbox[step & 1, w, :rows] = triples[w]
                flags[w, :rows] = step
            out = torch.full((rows, 256), 7.0, dtype=torch.float16, device="cuda")
            px[r].exchange_merge(env["ex"], triples[r].contiguous(), out)
            torch.cuda.synchronize()
            assert px[r].status() == 0
            assert torch.equal(out.view(torch.int16), want.view(torch.int16)), (step, r)
        # what the kernels delivered is what the host would have stored
        for r in range(world):
            inbox, flags = _mailbox_views(kv, bufs[r], world, max_rows)
            for w in range(world):
                if w != r:
                    assert torch.equal(inbox[step & 1, w, :rows], triples[w])
                    assert (flags[w, :rows] == step).all() and (flags[w, rows:] == 0).all()
        assert (px[0].private[:rows] == step).all()


def test_exchange_merge_wait_runs_out_with_a_status(env):
    """A flag that nothing sets: the bounded wait gives up, reports through the status word, leaves
    the output alone and still counts the step, so the next step (its peer delivered) is right."""
    kv = env["kv"]
    world, rows = 2, 5
    bufs = [torch.zeros(kv.PeerExchange.mailbox_bytes(world, rows), dtype=torch.uint8, device="cuda")
            for _ in range(world)]
    px = kv.PeerExchange.over_buffers(0, rows, bufs, wait_limit=300)
    triples = torch.rand(world, rows, 258, device="cuda") + 0.5
    out = torch.full((rows, 256), 7.0, dtype=torch.float16, device="cuda")
    px.exchange_merge(env["ex"], triples[0].contiguous(), out)
    torch.cuda.synchronize()
    assert px.status() == 1
    assert (out == 7.0).all()
    inbox, flags = _mailbox_views(kv, bufs[0], world, rows)
    inbox[0, 1] = triples[1]   # step 2 uses parity 0
    flags[1] = 2
    px.exchange_merge(env["ex"], triples[0].contiguous(), out)
    torch.cuda.synchronize()
    want = torch.zeros(rows, 256, dtype=torch.float16, device="cuda")
    kv.merge_shards(env["ex"], triples, want)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert px.status() == 1  # sticky
    with pytest.raises(Exception):
        px.exchange_merge(env["ex"], torch.zeros(rows + 1, 258, device="cuda"), out)  # more rows than the mailbox holds


def test_copy_on_write_tail_page_gives_the_unshared_result(env):
    """A request attaches a 68-token prefix whose last page is shared and partial, gets a private
    copy of that page (w34_seq_prepare_append + warp34_kv_page_copy), appends 9 tokens: its
    attention output is bit-identical to a request that owns all its pages, and the donor's
    page is untouched (docs/contracts/cache-layout.md:106-110)."""
    kv, synth = env["kv"], env["synth"]
    hq, hkv, n_pre, n_new = 8, 2, 68, 9
    k, v = synth.make_kv(n_pre + n_new, hkv, 71)
    q = synth.make_q(1, hq, 71)
    pool = kv.PagePool(40)
    pool.shuffle_free_list(5)
    layer = kv.KvLayer(40, hkv, fill=0x11)
    ex = env["ex"]

    def append(seq, lo, hi):
        assert seq.reserve(hi) >= 0
        b = kv.build_step([seq], [hi - lo], 8, 0.0625)
        kv.kv_cache_write(ex, layer, b, k[lo:hi].cuda(), v[lo:hi].cuda())
        seq.commit(hi - lo)

    donor = kv.Sequence(pool)
    append(donor, 0, n_pre)
    torch.cuda.synchronize()
    donor_tail = donor.pages[-1]
    before = layer.k.view(40, -1)[donor_tail].cpu().numpy().copy()

    sharer = kv.Sequence(pool)
    assert sharer.attach_prefix(donor.pages, n_pre) == 0
    cow = sharer.prepare_append()
    assert cow is not None and cow[0] == donor_tail and cow[2] == n_pre % 16
    kv.kv_page_copy(ex, layer, cow[0], cow[1], cow[2])
    append(sharer, n_pre, n_pre + n_new)

    owner = kv.Sequence(pool)
    append(owner, 0, n_pre + n_new)

    outs = []
    for seq in (sharer, owner):
        seq.set_committed(n_pre + n_new - 1)
        b = kv.build_step([seq], [1], 8, 0.0625)
        out = torch.zeros(1, hq, 256, dtype=torch.float16, device="cuda")
        kv.paged_attention(ex, layer, b, q.cuda(), out, hq)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy().view(np.uint16))
    assert (outs[0] == outs[1]).all()
    assert (layer.k.view(40, -1)[donor_tail].cpu().numpy() == before).all()
    assert sharer.pages[:4] == donor.pages[:4] and sharer.pages[4] != donor_tail


def test_bf16_activations_match_the_fp16_entry_points(env):
    """warp34_tq4_kv_cache_write_strided_bf16 / warp34_tq4_paged_attention_bf16: inputs on the grid
    bf16 and fp16 share give bit-identical TQ4 bytes; the attention output is the bf16 rounding of
    the same result; bf16 values beyond the fp16 range are accepted."""
    kv, synth, lib = env["kv"], env["synth"], env["lib"]
    hq, hkv, ctx = 8, 2, [75, 300]
    T = sum(ctx)
    k, v = synth.make_kv(T, hkv, 81)
    q = synth.make_q(2, hq, 81)
    pools, outs = [], []
    for bf16 in (False, True):
        wl = synth.PagedWorkload([0] * 2, ctx, hkv, seed=81, fill=0x22)
        b = wl.step()
        kd, vd = (k.to(torch.bfloat16).cuda(), v.to(torch.bfloat16).cuda()) if bf16 else (k.cuda(), v.cuda())
        fn = lib.warp34_tq4_kv_cache_write_strided_bf16 if bf16 else lib.warp34_kv_cache_write_strided
        assert fn(C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(b.desc), kd.data_ptr(), vd.data_ptr(),
                  hkv * 256, hkv * 256) == 0
        for s, c in zip(wl.seqs, ctx):
            s.commit(c - 1)
        d = wl.step(q_lens=[1, 1])
        qd = q.to(torch.bfloat16).cuda() if bf16 else q.cuda()
        out = torch.zeros_like(qd)
        fn = lib.warp34_tq4_paged_attention_bf16 if bf16 else lib.warp34_paged_attention_f16
        assert fn(C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(d.desc), qd.data_ptr(), out.data_ptr(), hq) == 0
        torch.cuda.synchronize()
        pools.append((wl.layer.k.cpu().numpy(), wl.layer.v.cpu().numpy()))
        outs.append(out.float().cpu().numpy())
    assert (pools[0][0] == pools[1][0]).all() and (pools[0][1] == pools[1][1]).all()
    # same fp32 result rounded to fp16 / bf16: they differ by at most one bf16 ulp
    assert (np.abs(outs[0] - outs[1]) <= 2.0 ** -8 * np.abs(outs[0]) + 1e-6).all()
    # a bf16 row far outside the fp16 range still encodes (scales saturate to +inf like any overflow)
    wl = synth.PagedWorkload([0], [16], hkv, seed=82, fill=0)
    big = torch.full((16, hkv * 256), 3.0e38, dtype=torch.bfloat16).cuda()
    b = wl.step()
    assert lib.warp34_tq4_kv_cache_write_strided_bf16(C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(b.desc),
                                                      big.data_ptr(), big.data_ptr(), hkv * 256, hkv * 256) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("hq", [16, 24])
@pytest.mark.parametrize("q_len,ctx_before", [(64, 0), (65, 19), (137, 128), (256, 200)])
def test_chunked_prefill_matches_cpu_oracle(env, hq, q_len, ctx_before):
    """Prefill chunks through the default prefill kernel, on the shapes the reference uses to compare its
    16- / 64- / 128-row kernels (crates/warp34-host/src/cuda/tests.rs:111-576): a chunk of q_len
    tokens after ctx_before cached tokens, causal inside the chunk."""
    kv, synth = env["kv"], env["synth"]
    hkv = 4
    total = ctx_before + q_len
    wl = synth.PagedWorkload([0], [total], hkv, seed=200 + q_len)
    k, v = synth.make_kv(total, hkv, 200 + q_len)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    wl.seqs[0].commit(ctx_before)
    b = wl.step(q_lens=[q_len])
    q = synth.make_q(q_len, hq, 200 + q_len)
    out = torch.full((q_len, hq, 256), 5.0, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
    torch.cuda.synchronize()
    want = _oracle_attention(wl, b, q, hq)
    ok, msg = plain_parity(out.float().cpu().numpy(), want)
    assert ok, msg


def test_mixed_prefill_and_decode_batch_with_masks(env):
    """Three requests in one call (a prefill chunk, a decode token, a second chunk with a sliding
    window), one masked token and sentinels in the output (cuda/tests.rs:538-572)."""
    kv, synth = env["kv"], env["synth"]
    hq, hkv = 16, 4
    ctx_before, q_lens = [40, 300, 7], [50, 1, 90]
    totals = [c + q for c, q in zip(ctx_before, q_lens)]
    wl = synth.PagedWorkload([0] * 3, totals, hkv, seed=300)
    k, v = synth.make_kv(sum(totals), hkv, 300)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c in zip(wl.seqs, ctx_before):
        s.commit(c)
    q = synth.make_q(sum(q_lens), hq, 300)
    sentinel = np.uint16(0x5500)
    for window in (0, 33):
        vtm = np.ones(sum(q_lens), np.uint8)
        vtm[60] = 0
        b = wl.step(q_lens=q_lens, sliding_window=window, valid_token_mask=vtm)
        out = torch.from_numpy(np.full((sum(q_lens), hq, 256), sentinel, np.uint16).view(np.float16)).cuda()
        kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
        torch.cuda.synchronize()
        bits = out.cpu().numpy().view(np.uint16)
        assert (bits[60] == sentinel).all()
        live = np.array([i for i in range(sum(q_lens)) if i != 60])
        want = _oracle_attention(wl, b, q, hq)
        ok, msg = plain_parity(f16(bits[live]), want[live])
        assert ok, (window, msg)


def _logical_rows(layer, seq, n_tokens, hkv):
    """K and V rows of a sequence in position order, read through its block table."""
    lay = layer.layout
    kp, vp = layer.k.cpu().numpy(), layer.v.cpu().numpy()
    pages = seq.pages
    ks, vs = [], []
    for pos in range(n_tokens):
        page, off = pages[pos // 16], pos % 16
        for h in range(hkv):
            o = page * lay.k_page_stride_bytes + h * lay.k_head_stride_bytes + off * lay.k_token_stride_bytes
            ks.append(kp[o:o + 132])
            o = page * lay.v_page_stride_bytes + h * lay.v_head_stride_bytes + off * lay.v_token_stride_bytes
            vs.append(vp[o:o + 132])
    return np.stack(ks), np.stack(vs)


def test_speculative_steps_with_rollback_leave_the_cache_as_if_only_accepted_tokens_were_appended(env):
    """Three verify steps of 1 + 3 draft tokens with rejected suffixes (pages truncated and reused):
    the cache then holds, position by position, the bytes of a plain append of the accepted tokens,
    and the next verify pass agrees with the CPU oracle."""
    kv, synth = env["kv"], env["synth"]
    hq, hkv, ql = 24, 4, 4
    ctx = [13, 30, 64]
    wl = synth.PagedWorkload(ctx, [ql] * 3, hkv, seed=41, slack_pages=16)
    kept = wl.fill_context(env["ex"], 41, keep=True)
    spec = kv.SpeculativeBatch(wl.seqs)
    accepted_rows = [[kept[i][0], kept[i][1]] for i in range(3)]       # fp16 K, V of every accepted token
    plan = [[2, 4, 1], [1, 3, 4], [4, 1, 2]]
    for step_i, accepted in enumerate(plan):
        spec.reserve_ahead(ql)
        k, v = synth.make_kv(3 * ql, hkv, 500 + step_i)
        b = wl.step(q_lens=[ql] * 3)
        kv.kv_cache_write(env["ex"], wl.layer, b, k.cuda(), v.cuda())
        torch.cuda.synchronize()
        for i, a in enumerate(accepted):
            accepted_rows[i][0] = torch.cat([accepted_rows[i][0], k[i * ql:i * ql + a]])
            accepted_rows[i][1] = torch.cat([accepted_rows[i][1], v[i * ql:i * ql + a]])
        spec.commit_and_rollback(accepted)
    lens = [c + sum(p[i] for p in plan) for i, c in enumerate(ctx)]
    assert [s.committed_len for s in wl.seqs] == lens
    assert [s.num_pages for s in wl.seqs] == [(n + 15) // 16 for n in lens]
    # reference cache: the accepted tokens appended in one go
    ref = synth.PagedWorkload([0] * 3, lens, hkv, seed=77)
    kk = torch.cat([r[0] for r in accepted_rows]).cuda()
    vv = torch.cat([r[1] for r in accepted_rows]).cuda()
    kv.kv_cache_write(env["ex"], ref.layer, ref.step(), kk, vv)
    torch.cuda.synchronize()
    for i in range(3):
        a_k, a_v = _logical_rows(wl.layer, wl.seqs[i], lens[i], hkv)
        b_k, b_v = _logical_rows(ref.layer, ref.seqs[i], lens[i], hkv)
        assert (a_k == b_k).all() and (a_v == b_v).all()
    # one more verify pass over the rolled-back cache
    spec.reserve_ahead(ql)
    k, v = synth.make_kv(3 * ql, hkv, 900)
    q = synth.make_q(3 * ql, hq, 900)
    b = wl.step(q_lens=[ql] * 3)
    kv.kv_cache_write(env["ex"], wl.layer, b, k.cuda(), v.cuda())
    out = torch.zeros(3 * ql, hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
    torch.cuda.synchronize()
    want = _oracle_attention(wl, b, q, hq)
    ok, msg = plain_parity(out.float().cpu().numpy(), want)
    assert ok, msg


@pytest.mark.parametrize("selector", [0, 1, 2])
@pytest.mark.parametrize("hq", [16, 24])
def test_forced_kernel_variants_on_the_reference_shapes(env, hq, selector):
    """warp34_paged_attention_f16_force_kernel_for_test on the shapes of the reference's
    variant-equality test (crates/warp34-host/src/cuda/tests.rs:111-576): four requests with
    (q_len, cached) = (64, 0), (65, 19), (137, 128), (256, 200) in one call, one masked token whose
    output row must keep its sentinel 0x5500.  The reference compares its variants at 0 ULP because
    they share their arithmetic; these do not, so each is compared with the oracle: selectors 0 and 1
    inside the plain bound on every element, selector 2 (tcgen05, single fp16 operands) inside the
    bound of the fast build."""
    kv, synth, ffi = env["kv"], env["synth"], env["ffi"]
    hkv = 4
    shapes = [(64, 0), (65, 19), (137, 128), (256, 200)]
    q_lens = [s[0] for s in shapes]
    totals = [s[0] + s[1] for s in shapes]
    wl = synth.PagedWorkload([0] * 4, totals, hkv, seed=700 + hq)
    k, v = synth.make_kv(sum(totals), hkv, 700 + hq)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, (ql, c) in zip(wl.seqs, shapes):
        s.commit(c)
    n = sum(q_lens)
    vtm = np.ones(n, np.uint8)
    vtm[70] = 0                                   # a token of the second request
    b = wl.step(q_lens=q_lens, valid_token_mask=vtm)
    q = synth.make_q(n, hq, 701)
    out = torch.full((n, hq, 256), 0, dtype=torch.int16, device="cuda")
    out.fill_(0x5500)
    rc = env["lib"].warp34_paged_attention_f16_force_kernel_for_test(
        C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(b.desc), q.cuda().data_ptr(), out.data_ptr(), hq, selector)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(env["ex"].scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
    bits = out.cpu().numpy().view(np.uint16)
    assert (bits[70] == 0x5500).all(), "masked row was written"
    live = vtm.astype(bool)
    want = _oracle_attention(wl, b, q, hq)
    ok, msg = (fast_parity if selector == 2 else plain_parity)(f16(bits[live]), want[live])
    assert ok, (selector, msg)


def test_forced_kernel_selector_validates_like_the_reference(env):
    ffi = env["ffi"]
    lay, b = ffi.KvLayerLayout(), ffi.AttentionBatch()
    fn = env["lib"].warp34_paged_attention_f16_force_kernel_for_test
    assert fn(None, C.byref(lay), C.byref(b), 1, 1, 16, 0) == ffi.CUDA_ERROR_INVALID_VALUE
    assert fn(C.byref(env["ex"].ex), C.byref(lay), C.byref(b), 1, 1, 16, 1) == 0      # empty batch: no launch
    b.total_tokens, b.num_reqs = 1, 1
    lay.head_dim, lay.block_size, lay.local_kv_heads = 128, 16, 4                      # head_dim other than 256
    assert fn(C.byref(env["ex"].ex), C.byref(lay), C.byref(b), 1, 1, 16, 2) == ffi.CUDA_ERROR_INVALID_VALUE


@pytest.mark.parametrize("mode", ["default", "short_chunk", "verify", "fast", "fast_short_chunk", "fast_verify", "verify_flag"])
def test_prefill_dispatch_paths_agree_with_the_oracle(env, mode):
    """Default: the register-MMA prefill kernel with value + residual operands (also with partly
    filled 128-row tiles) and 8-row items for a verify batch, held to the plain bound.  With the
    fast flag: the tcgen05 kernel and the four-warp team kernel, held to the bound of the fast build."""
    kv, synth, ffi = env["kv"], env["synth"], env["ffi"]
    hkv = 4
    shape = {"default": (16, 200, 333), "short_chunk": (16, 20, 100), "verify": (24, 4, 1500)}
    hq, q_len, ctx_before = shape[mode.replace("fast_", "").replace("_flag", "").replace("fast", "default")]
    flags = ffi.EXEC_FLAG_FAST_ATTENTION if mode.startswith("fast") else 0
    if mode == "verify_flag":
        flags = ffi.EXEC_FLAG_TCGEN05_VERIFY
    total = ctx_before + q_len
    wl = synth.PagedWorkload([0, 0], [total, total // 2 + q_len], hkv, seed=610, fill=0xFF)
    lens = [total, total // 2 + q_len]
    k, v = synth.make_kv(sum(lens), hkv, 610)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, n in zip(wl.seqs, lens):
        s.commit(n - q_len)
    b = wl.step(q_lens=[q_len, q_len])
    q = synth.make_q(2 * q_len, hq, 611)
    ex = kv.Executor(8 << 20)
    ex.scratch[:16].zero_()          # the status word; only the tcgen05 kernel writes it on this path
    ex.ex.flags = flags
    out = torch.full((2 * q_len, hq, 256), 5.0, dtype=torch.float16, device="cuda")
    kv.paged_attention(ex, wl.layer, b, q.cuda(), out, hq)
    torch.cuda.synchronize()
    assert int(ex.scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
    want = _oracle_attention(wl, b, q, hq)
    ok, msg = (plain_parity if flags == 0 else fast_parity)(out.float().cpu().numpy(), want)
    assert ok, (mode, msg)


def test_graph_replayed_steps_match_eager_steps(env):
    """DecodeStep.run(graph=True) replays one captured CUDA graph per step (uploads, append,
    attention, download) with the block-table changes copied in front of it: over steps in which
    sequences grow across page boundaries its outputs and cache bytes equal the eager path's."""
    kv, synth = env["kv"], env["synth"]
    hq, hkv = 16, 4
    ctx = [14, 15, 16, 31, 100]
    outs, pools = [], []
    for use_graph in (False, True):
        wl = synth.PagedWorkload(ctx, [1] * len(ctx), hkv, seed=71, slack_pages=16)
        ex0 = kv.Executor(8 << 20)
        wl.fill_context(ex0, 71)
        step = kv.DecodeStep(wl.layer, wl.seqs, hq, max_q_len=1, scratch_bytes=8 << 20, extra_blocks=2)
        res = []
        for it in range(6):
            for s in wl.seqs:
                assert s.reserve(s.committed_len + 1) >= 0
            k, v = synth.make_kv(len(ctx), hkv, 800 + it)
            q = synth.make_q(len(ctx), hq, 800 + it)
            step.k_host.copy_(k); step.v_host.copy_(v); step.q_host.copy_(q)
            out = step.run([1] * len(ctx), graph=use_graph)
            res.append(out.clone())
            for s in wl.seqs:
                s.commit(1)
        outs.append(res)
        pools.append([_logical_rows(wl.layer, s, s.committed_len, hkv) for s in wl.seqs])
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    for (ak, av), (bk, bv) in zip(pools[0], pools[1]):
        assert (ak == bk).all() and (av == bv).all()
