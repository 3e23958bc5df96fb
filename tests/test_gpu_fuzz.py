"""Seeded random geometries through the C ABI: the default (tensor-core) path of every storage format
against this library's fp32 dequant-then-attend kernels (WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION), which
the other GPU tests pin against the reference's scalar kernel.  Head counts with GQA groups from 1 to 12,
ragged contexts from one token to a few hundred, decode / draft / chunk query lengths, causal and symmetric
sliding windows, masked tokens and requests, the fused output epilogue (gate, gate + Hadamard-64), pools
pre-filled with 0xFF bytes; for the query-sparse entry point random
selected lists with skipped, invisible and partly visible groups.  Bound: 2e-3 + 1e-2 |b| on every output,
masked rows bit-identical (untouched, or zeros for the query-sparse entry point)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-2
FORMATS = {"tq4": (2, 1), "fp8": (4, 0), "q8": (3, 0)}
HEADS = [(4, 4), (8, 4), (16, 4), (24, 4), (8, 1), (24, 2), (6, 3)]


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    return dict(ffi=ffi, kv=kv, synth=synth, lib=native_libs[0])


def _close(got_bits, want_bits, sentinel):
    untouched = (want_bits == sentinel).all(axis=(1, 2))
    assert ((got_bits == sentinel).all(axis=(1, 2)) == untouched).all(), "masked rows differ"
    g = got_bits.view(np.float16).astype(np.float32)[~untouched]
    w = want_bits.view(np.float16).astype(np.float32)[~untouched]
    assert np.isfinite(g).all() and np.isfinite(w).all()
    d = np.abs(g - w)
    assert np.all(d <= ATOL + RTOL * np.abs(w)), float((d / (ATOL + RTOL * np.abs(w))).max())
    return g.size


@pytest.mark.parametrize("fmt_name", ["tq4", "fp8", "q8"])
@pytest.mark.parametrize("seed", range(8))
def test_random_batches_default_path_against_the_fp32_kernel(env, fmt_name, seed):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    rng = np.random.default_rng(1000 * seed + len(fmt_name))
    fmt, tr = FORMATS[fmt_name]
    hq, hkv = HEADS[int(rng.integers(len(HEADS)))]
    if fmt_name != "tq4" and hq // hkv > 8:     # the fp32 kernel of the 8-bit layers serves groups of up to 8 heads
        hq, hkv = 16, 2
    n = int(rng.integers(1, 6))
    mode = ["decode", "draft", "chunk"][int(rng.integers(3))]
    q_lens = {"decode": [1] * n, "draft": [int(rng.integers(1, 6)) for _ in range(n)],
              "chunk": [int(rng.integers(20, 90)) for _ in range(n)]}[mode]
    ctx = [int(q + rng.integers(0, 500)) for q in q_lens]            # tokens after the step
    window = int(rng.integers(8, 200)) if rng.random() < 0.3 else 0
    wl = synth.PagedWorkload([0] * n, ctx, hkv, seed=seed, fill=0xFF, formats=(fmt, fmt, tr, tr))
    ex = kv.Executor(64 << 20)
    k, v = synth.make_kv(sum(ctx), hkv, seed)
    if rng.random() < 0.3:      # rows of zeros and of fp16 subnormals among the tokens (padding, dead channels)
        for buf in (k, v):
            kinds = rng.random(buf.shape[0])
            buf[torch.from_numpy(kinds < 0.12)] = 0.0
            tiny = torch.from_numpy((kinds >= 0.12) & (kinds < 0.2))
            buf[tiny] = (buf[tiny].float() * 3e-6).to(buf.dtype)
    kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c, ql in zip(wl.seqs, ctx, q_lens):
        s.commit(c - ql)
    T = sum(q_lens)
    kw = {}
    if rng.random() < 0.5:
        vtm = (rng.random(T) > 0.2).astype(np.uint8)
        kw["valid_token_mask"] = vtm
    if n > 1 and rng.random() < 0.3:
        vrm = np.ones(n, np.uint8)
        vrm[int(rng.integers(n))] = 0
        kw["valid_req_mask"] = vrm
    if window:
        kw["sliding_window"] = window
        if rng.random() < 0.5:
            kw["mask_mode"] = ffi.ATTN_MASK_SYMMETRIC_WINDOW
    b = wl.step(q_lens=q_lens, **kw)
    q = synth.make_q(T, hq, seed + 1).cuda()
    # a third of the cases go through the entry point with the fused output epilogue (gate, gate + Hadamard-64)
    epilogue = int(rng.integers(3)) if rng.random() < 0.33 else 0
    gate = (torch.randn(T, hq, 256, generator=torch.Generator().manual_seed(seed)) * 2).to(torch.float16).cuda()
    # the default path also runs with workspaces too small for the batch in one pass (several passes, or the
    # kernel without a workspace when not even one request fits)
    small = kv.Executor(int(rng.choice([64 << 20, 1 << 20, 300 << 10])))
    outs = []
    fill_ex = ex
    for flags in (0, ffi.EXEC_FLAG_PRECISE_ATTENTION):
        ex = small if flags == 0 else fill_ex
        ex.ex.flags = flags
        out = torch.full((T, hq, 256), 0, dtype=torch.int16, device="cuda")
        out.fill_(0x5500)
        if epilogue:
            kv.paged_attention_gated(ex, wl.layer, b, q, gate, out.view(torch.float16), hq, hadamard64=(epilogue == 2))
        else:
            kv.paged_attention(ex, wl.layer, b, q, out.view(torch.float16), hq)
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy().view(np.uint16))
    ex.ex.flags = 0
    if epilogue == 2:
        # The Hadamard-64 epilogue mixes 64 gated values g_i into each output (sum of +-g_i / 8): what the
        # bound on every g_i implies for an output is the sum of their tolerances / 8, whatever the output's
        # own size, plus its fp16 rounding.  The g_i are recovered by rotating the fp32 kernel's result back
        # (the transform is its own inverse).
        untouched = (outs[1] == 0x5500).all(axis=(1, 2))
        assert ((outs[0] == 0x5500).all(axis=(1, 2)) == untouched).all(), "masked rows differ"
        h64 = np.array([[1.0 if bin(i & j).count("1") % 2 == 0 else -1.0 for j in range(64)] for i in range(64)], np.float32) / 8.0
        got, want = (o.view(np.float16).astype(np.float32)[~untouched].reshape(-1, hq, 4, 64) for o in outs)
        assert np.isfinite(got).all()
        gated = want @ h64
        tol = (ATOL + RTOL * np.abs(gated)).sum(axis=-1, keepdims=True) / 8.0 + 2.0 ** -10 * np.abs(want)
        d = np.abs(got - want)
        assert np.all(d <= tol), float((d / tol).max())
    else:
        _close(outs[0], outs[1], 0x5500)


@pytest.mark.parametrize("fmt_name", ["tq4", "fp8", "q8"])
@pytest.mark.parametrize("seed", range(8))
def test_random_selected_lists_stream_kernel_against_the_fp32_kernel(env, seed, fmt_name):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    rng = np.random.default_rng(77 + seed)
    fmt, tr = FORMATS[fmt_name]
    hq, hkv = HEADS[int(rng.integers(len(HEADS)))]
    n = int(rng.integers(1, 4))
    ctx = [int(rng.integers(1, 700)) for _ in range(n)]
    wl = synth.PagedWorkload([0] * n, ctx, hkv, seed=seed, fill=0xFF, formats=(fmt, fmt, tr, tr))
    ex = kv.Executor(64 << 20)
    k, v = synth.make_kv(sum(ctx), hkv, seed)
    kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
    T = int(rng.integers(1, 9))
    select_k = int(rng.integers(1, 70))
    phys = np.full((T, select_k), -1, np.int32)
    logical = np.zeros((T, select_k), np.int32)
    n_sel = np.zeros(T, np.int32)
    pos = np.zeros(T, np.int32)
    for t in range(T):
        s = int(rng.integers(n))
        pos[t] = int(rng.integers(ctx[s]))
        groups = (ctx[s] + 3) // 4
        pick = rng.permutation(groups)[:select_k]              # any group of the sequence: some lie beyond pos
        pages = np.asarray(wl.seqs[s].pages)
        logical[t, :len(pick)] = pick
        phys[t, :len(pick)] = pages[pick // 4] * 4 + pick % 4
        phys[t, :len(pick)][rng.random(len(pick)) < 0.15] = -1
        n_sel[t] = int(rng.integers(0, len(pick) + 1))
    vtm = (rng.random(T) > 0.2).astype(np.uint8)
    dev = [torch.from_numpy(a).cuda() for a in (phys, logical, n_sel, pos, vtm)]
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, hq, 256, generator=g).to(torch.float16).cuda()
    gate = (torch.randn(T, hq, 256, generator=g) * 2).to(torch.float16).cuda()
    hadamard = bool(rng.integers(2))
    fn = getattr(env["lib"], "warp34_qsa_sparse_paged_attn_hadamard_f16" if hadamard else "warp34_qsa_sparse_paged_attn_f16")
    outs = []
    for flags in (0, ffi.EXEC_FLAG_PRECISE_ATTENTION):
        ex.ex.flags = flags
        out = torch.full((T, hq, 256), 0, dtype=torch.int16, device="cuda")
        out.fill_(0x5500)
        assert fn(C.addressof(ex.ex), q.data_ptr(), gate.data_ptr(), C.addressof(wl.layer.layout), dev[0].data_ptr(),
                  dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), dev[4].data_ptr(), out.data_ptr(), T, hq,
                  select_k, 0.0625) == 0
        torch.cuda.synchronize()
        if flags == 0:
            assert int(ex.scratch[:4].cpu().numpy().view(np.int32)[0]) & 3 == 0
        outs.append(out.cpu().numpy().view(np.uint16))
    ex.ex.flags = 0
    assert not (outs[1] == 0x5500).any(), "the query-sparse entry point writes every row"
    assert (outs[0][vtm == 0] == 0).all() and (outs[1][vtm == 0] == 0).all()
    g0 = outs[0].view(np.float16).astype(np.float32)
    g1 = outs[1].view(np.float16).astype(np.float32)
    assert np.isfinite(g0).all() and np.isfinite(g1).all()
    assert np.all(np.abs(g0 - g1) <= ATOL + RTOL * np.abs(g1)), float(np.abs(g0 - g1).max())


@pytest.mark.parametrize("fmt_name,q_hi,flag", [("tq4", 1, None), ("tq4", 1, "EXEC_FLAG_FAST_ATTENTION"), ("tq4", 4, None),
                                                ("tq4", 4, "EXEC_FLAG_FAST_ATTENTION"), ("fp8", 1, None), ("q8", 3, None)])
def test_thousands_of_short_requests_with_idle_ones_between(env, fmt_name, q_hi, flag):
    """3000 requests in one batch, contexts of 1 to 90 tokens, every seventh request with no new token
    in this step (equal neighbours in query_start_loc): plan, work split and merge at a request count far
    above the benchmark's, against the fp32 kernels."""
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    rng = np.random.default_rng(9000 + q_hi)
    fmt, tr = FORMATS[fmt_name]
    hq, hkv = (24, 4) if fmt_name == "tq4" else (16, 4)
    n = 3000
    q_lens = [0 if i % 7 == 3 else int(rng.integers(1, q_hi + 1)) for i in range(n)]
    ctx = [int(max(q, 1) + rng.integers(0, 90)) for q in q_lens]          # tokens after the step
    wl = synth.PagedWorkload([0] * n, ctx, hkv, seed=5, fill=0xFF, formats=(fmt, fmt, tr, tr))
    ex = kv.Executor(128 << 20)
    k, v = synth.make_kv(sum(ctx), hkv, 5)
    kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c, ql in zip(wl.seqs, ctx, q_lens):
        s.commit(c - ql)
    T = sum(q_lens)
    b = wl.step(q_lens=q_lens)
    assert (np.diff(b.host["query_start_loc"]) == 0).sum() >= n // 7
    # a slot and a set of query fragments per (request, kv head, row group): far more workspace than a
    # benchmark batch needs; with less the call would run the kernel without a workspace instead
    need = env["lib"].warp34_paged_attention_scratch_bytes(C.byref(wl.layer.layout), C.byref(b.desc), hq)
    assert (64 << 20) < need < (1 << 30), need
    ex = kv.Executor(int(need))
    q = synth.make_q(T, hq, 6).cuda()
    outs = []
    for flags in (getattr(ffi, flag) if flag else 0, ffi.EXEC_FLAG_PRECISE_ATTENTION):
        ex.ex.flags = flags
        out = torch.full((T, hq, 256), 0, dtype=torch.int16, device="cuda")
        out.fill_(0x5500)
        ex.scratch[:4].fill_(0x7f)                 # the plan of the split-KV path rewrites the status word
        kv.paged_attention(ex, wl.layer, b, q, out.view(torch.float16), hq)
        torch.cuda.synchronize()
        status = int(ex.scratch[:4].cpu().numpy().view(np.int32)[0])
        assert status == (0x7f7f7f7f if flags == ffi.EXEC_FLAG_PRECISE_ATTENTION else 0), hex(status)
        outs.append(out.cpu().numpy().view(np.uint16))
    ex.ex.flags = 0
    if flag is None:
        assert _close(outs[0], outs[1], 0x5500) == T * hq * 256
    else:   # single fp16 operands: that build's own, wider bound (99.9 % inside the plain one, capped outliers)
        from util import f16, fast_parity
        ok, msg = fast_parity(f16(outs[0]), f16(outs[1]))
        assert ok, msg


@pytest.fixture(scope="module")
def ref_lib(env):
    import oracle
    p = oracle.ref_lib_path()
    if p is None:
        pytest.skip("reference kernels not built (oracle/_ref)")
    return env["ffi"].bind_kernel_abi(p)


def _append_case(env, ref_lib, fmt_name, seed):
    """Random tokens, heads, slots, masks, row strides and value ranges through the append entry point of this
    library and of the reference's own kernels: the two pools must hold the same bytes."""
    ffi, kv = env["ffi"], env["kv"]
    rng = np.random.default_rng(31000 + seed)
    fmt, tr = FORMATS[fmt_name]
    hkv = int(rng.choice([1, 2, 3, 4, 8]))
    T = int(rng.integers(1, 200))
    num_pages = 40
    g = torch.Generator().manual_seed(seed)
    pad = int(rng.choice([0, 4, 8, 64]))        # 4 halves: every other row starts off a 16-byte boundary
    width = hkv * 256 + pad
    kbuf = torch.randn(T, width, generator=g)
    vbuf = torch.randn(T, width, generator=g)
    # value ranges per token: ordinary, outlier channels, huge, tiny (fp16 subnormals), exact zeros, one hot
    kind = rng.integers(0, 6, size=T)
    for t in range(T):
        for buf in (kbuf, vbuf):
            if kind[t] == 1:
                buf[t, rng.integers(0, hkv * 256, size=6)] *= 25.0
            elif kind[t] == 2:
                buf[t] *= 9000.0
            elif kind[t] == 3:
                buf[t] *= 3e-6
            elif kind[t] == 4:
                buf[t] = 0.0
            elif kind[t] == 5:
                buf[t] = 0.0
                buf[t, int(rng.integers(0, hkv * 256))] = float(rng.choice([1.0, -300.0, 6e-5]))
    kbuf, vbuf = kbuf.clamp(-65000, 65000).to(torch.float16).cuda(), vbuf.clamp(-65000, 65000).to(torch.float16).cuda()
    # requests of random lengths; distinct random slots, some skipped
    cuts = np.sort(rng.choice(np.arange(1, T), size=min(int(rng.integers(0, 5)), T - 1), replace=False)) if T > 1 else np.array([], int)
    qsl = np.concatenate([[0], cuts, [T]]).astype(np.int32)
    n = len(qsl) - 1
    slots = rng.permutation(np.arange(16, num_pages * 16))[:T].astype(np.int32)
    slots[rng.random(T) < 0.1] = -1
    kw = {}
    if rng.random() < 0.5:
        kw["valid_token_mask"] = (rng.random(T) > 0.15).astype(np.uint8)
    if rng.random() < 0.3:
        kw["valid_req_mask"] = (rng.random(n) > 0.3).astype(np.uint8)
    bt = np.zeros((n, 4), np.int32)
    lens = np.diff(qsl)
    pools = []
    for lib in (env["lib"], ref_lib):
        layer = kv.KvLayer(num_pages, hkv, formats=(fmt, fmt, tr, tr), fill=0x3C)
        b = kv.StepBatch(qsl, [0] * n, lens.tolist(), bt, slots, 4, 0.0625, **kw)
        ex = kv.Executor(1 << 20)
        kv.kv_cache_write(ex, layer, b, kbuf, vbuf, k_row_stride=width, v_row_stride=width, lib=lib)
        torch.cuda.synchronize()
        pools.append((layer.k.cpu().numpy(), layer.v.cpu().numpy()))
    assert np.array_equal(pools[0][0], pools[1][0]), ("K pool", fmt_name, seed, int((pools[0][0] != pools[1][0]).sum()))
    assert np.array_equal(pools[0][1], pools[1][1]), ("V pool", fmt_name, seed, int((pools[0][1] != pools[1][1]).sum()))
    assert (pools[0][0] != 0x3C).any() or (slots < 0).all() or "valid_token_mask" in kw or "valid_req_mask" in kw


@pytest.mark.parametrize("fmt_name", ["tq4", "fp8", "q8"])
@pytest.mark.parametrize("seed", range(6))
def test_random_appends_give_the_reference_kernels_bytes(env, ref_lib, fmt_name, seed):
    _append_case(env, ref_lib, fmt_name, seed)
