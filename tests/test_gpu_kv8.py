"""GPU parity of the unrotated 8-bit boundary-layer formats (Q8_0 and FP8 E4M3 rows), through the
C ABI.  Append: bit-exact against the reference's own kernels when oracle/_ref travelled with the
repository, and against the CPU restatement (oracle/kv8.py) up to one quantisation step on a few
codes (the restatement divides exactly, the kernels use the fast reciprocal).  Attention:
|a-b| <= 2e-3 + 1e-2|b| against the reference's own scalar dequant-then-attend kernel
(warp34_paged_attention_scalar_f16 -> paged_attention_kernel<__half> with read_kv_elem,
op_kv_cache.cu:288-322, :373-792, :1244) run on the same pool, which also pins the float64
restatement of the decode (oracle/kv8.py).  The reference's tensor-core dispatcher
(warp34_paged_attention_f16, op_paged_attn.cu:1266) is NOT called on these layers: in an earlier run
it returned non-finite output and, for one geometry, an illegal memory access, and reading its
dispatcher, row decoder and 16-row kernel against the descriptors passed here did not show why.
Formats and policies: crates/warp34-host/src/cache.rs:62-108."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    return dict(ffi=ffi, kv=kv, synth=synth, ex=kv.Executor(16 << 20), lib=native_libs[0])


@pytest.fixture(scope="module")
def ref_lib(env):
    import oracle
    p = oracle.ref_lib_path()
    if p is None:
        pytest.skip("reference kernels not built (oracle/_ref)")
    return env["ffi"].bind_kernel_abi(p)


def _formats(ffi, fmt):
    return (fmt, fmt, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY)


def _workload(env, fmt, ctx, hkv, seed, fill=0x11):
    synth, ffi = env["synth"], env["ffi"]
    wl = synth.PagedWorkload([0] * len(ctx), [int(c) for c in ctx], hkv, seed=seed, fill=fill,
                             formats=_formats(ffi, fmt))
    return wl


def _pool_rows(layer, fmt_bytes, hkv):
    """[pages, hkv, 16, row bytes] views of the K and V slabs."""
    k = layer.k.cpu().numpy().reshape(layer.num_pages, hkv, 16, fmt_bytes)
    v = layer.v.cpu().numpy().reshape(layer.num_pages, hkv, 16, fmt_bytes)
    return k, v


@pytest.mark.parametrize("fmt_name", ["q8_0", "fp8_e4m3"])
def test_append_8bit_rows_bit_exact_with_reference_and_close_to_the_restatement(env, fmt_name, request):
    from oracle import kv8
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    fmt = ffi.KV_FORMAT_Q8_0 if fmt_name == "q8_0" else ffi.KV_FORMAT_FP8_E4M3
    hkv, ctx = 2, [70, 33, 129, 24]
    T = sum(ctx)
    k, v = synth.make_kv(T, hkv, 31)
    edge = T - 24   # the last request carries edge rows
    k[edge] = 0
    v[edge + 1] = 0
    k[edge + 2] = 6.1e-5
    v[edge + 3] = 1000.0
    k[edge + 4] = 0
    k[edge + 4, 17] = 3.0
    v[edge + 5, :256] = 0
    k[edge + 6] = 60000.0
    v[edge + 7] = -1.0
    pools = {}
    for name in ("ours", "ref"):
        if name == "ref":
            try:
                lib = request.getfixturevalue("ref_lib")
            except pytest.skip.Exception:
                continue
        else:
            lib = None
        wl = _workload(env, fmt, ctx, hkv, seed=31)
        kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda(), lib=lib)
        torch.cuda.synchronize()
        pools[name] = (wl, wl.layer.k.cpu().numpy(), wl.layer.v.cpu().numpy())
    wl, pk, pv = pools["ours"]
    if "ref" in pools:
        assert (pk == pools["ref"][1]).all() and (pv == pools["ref"][2]).all()
    # against the CPU restatement, row by row through the block tables
    rb = kv8.ROW_BYTES[fmt]
    kr, vr = _pool_rows(wl.layer, rb, hkv)
    start = 0
    worst, differing, total = 0, 0, 0
    for s, c in zip(wl.seqs, ctx):
        pages = s.pages
        for h in range(hkv):
            for src, pool in ((k, kr), (v, vr)):
                x = src[start:start + c, 256 * h:256 * h + 256].float().numpy()
                want = kv8.encode_rows(x, fmt)
                got = np.stack([pool[pages[t // 16], h, t % 16] for t in range(c)])
                if fmt == ffi.KV_FORMAT_Q8_0:
                    sc_g = np.concatenate([got[:, 68 * b:68 * b + 4] for b in range(4)], axis=1)
                    sc_w = np.concatenate([want[:, 68 * b:68 * b + 4] for b in range(4)], axis=1)
                else:
                    sc_g, sc_w = got[:, 256:], want[:, 256:]
                # scales: fast division may differ in the last place
                dg, dw = sc_g.copy().view(np.float32), sc_w.copy().view(np.float32)
                assert np.all(np.abs(dg - dw) <= 2.0 ** -22 * np.abs(dw))
                cg, cw = kv8.codes(got, fmt), kv8.codes(want, fmt)
                worst = max(worst, int(np.abs(cg - cw).max()))
                differing += int((cg != cw).sum())
                total += cg.size
        start += c
    assert worst <= 1, worst
    assert differing <= total * 0.01, (differing, total)
    # bytes of pages nobody wrote keep the fill pattern
    used = {p for s in wl.seqs for p in s.pages}
    free = [p for p in range(wl.layer.num_pages) if p not in used]
    assert free and (kr[free] == 0x11).all() and (vr[free] == 0x11).all()


def _dequant_then_attend(env, wl, fmt, ctx, q_lens, q, hq, hkv):
    from oracle import kv8
    rb = kv8.ROW_BYTES[fmt]
    kr, vr = _pool_rows(wl.layer, rb, hkv)
    g = hq // hkv
    out = np.zeros((sum(q_lens), hq, 256))
    t0 = 0
    for s, c, ql in zip(wl.seqs, ctx, q_lens):
        pages = s.pages
        for h in range(hkv):
            kd = kv8.decode_rows(np.stack([kr[pages[t // 16], h, t % 16] for t in range(c)]), fmt)
            vd = kv8.decode_rows(np.stack([vr[pages[t // 16], h, t % 16] for t in range(c)]), fmt)
            for j in range(ql):
                n_vis = c - ql + j + 1
                qq = q[t0 + j, h * g:(h + 1) * g].float().numpy()
                out[t0 + j, h * g:(h + 1) * g] = kv8.attention(kd[:n_vis], vd[:n_vis], qq, 1.0 / 16.0)
        t0 += ql
    return out


@pytest.mark.parametrize("fmt_name", ["q8_0", "fp8_e4m3"])
@pytest.mark.parametrize("hq,hkv,q_len", [(24, 4, 1), (16, 4, 3), (8, 8, 1)])
def test_attention_over_8bit_rows_matches_dequant_then_attend(env, fmt_name, hq, hkv, q_len, request):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    fmt = ffi.KV_FORMAT_Q8_0 if fmt_name == "q8_0" else ffi.KV_FORMAT_FP8_E4M3
    ctx = [257, 40, 16, 1000]
    q_lens = [q_len] * len(ctx)
    T = sum(ctx)
    k, v = synth.make_kv(T, hkv, 47)
    wl = _workload(env, fmt, ctx, hkv, seed=47)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c, ql in zip(wl.seqs, ctx, q_lens):
        s.commit(c - ql)
    b = wl.step(q_lens=q_lens)
    q = synth.make_q(sum(q_lens), hq, 47)
    out = torch.zeros(sum(q_lens), hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out, hq)
    torch.cuda.synchronize()
    # the stream kernel's status word (no bounded wait gave up)
    assert int(env["ex"].scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
    got = out.float().cpu().numpy()
    want = _dequant_then_attend(env, wl, fmt, ctx, q_lens, q, hq, hkv)
    assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want)), float(np.abs(got - want).max())
    # the scalar entry point is the fp32 dequant-then-attend kernel; the default path is the tensor-core
    # stream kernel (exact operands, P as value + residual)
    out2 = torch.zeros_like(out)
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out2, hq, scalar=True)
    torch.cuda.synchronize()
    g2 = out2.float().cpu().numpy()
    assert np.all(np.abs(g2 - want) <= ATOL + RTOL * np.abs(want)), float(np.abs(g2 - want).max())
    assert not torch.equal(out.view(torch.int16), out2.view(torch.int16)), "the default path did not take the stream kernel"
    # The pin: the reference's scalar kernel (fp32, read_kv_elem) over the same bytes.  This library's
    # output must sit inside the plain bound of it, and so must the float64 restatement, which the
    # tests of the 8-bit path lean on when the reference library is absent.
    try:
        ref = request.getfixturevalue("ref_lib")
    except pytest.skip.Exception:
        return
    out3 = torch.zeros_like(out)
    kv.paged_attention(env["ex"], wl.layer, b, q.cuda(), out3, hq, lib=ref, scalar=True)
    torch.cuda.synchronize()
    r = out3.float().cpu().numpy()
    assert np.isfinite(r).all()
    assert np.all(np.abs(got - r) <= ATOL + RTOL * np.abs(r)), float(np.abs(got - r).max())
    # the restatement against the reference, fp16 output rounding aside
    assert np.all(np.abs(want - r) <= 2.0 ** -10 * np.abs(r) + 2e-4), float(np.abs(want - r).max())


def test_8bit_layers_refuse_what_they_do_not_cover(env):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    rotated = (ffi.KV_FORMAT_Q8_0, ffi.KV_FORMAT_Q8_0, ffi.KV_TRANSFORM_RADEMACHER_WHT256,
               ffi.KV_TRANSFORM_RADEMACHER_WHT256)
    wl = synth.PagedWorkload([0], [20], 2, seed=3, formats=rotated)
    k, v = synth.make_kv(20, 2, 3)
    rc = env["lib"].warp34_kv_cache_write(C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(wl.step().desc),
                                          k.cuda().data_ptr(), v.cuda().data_ptr())
    assert rc == ffi.CUDA_ERROR_NOT_SUPPORTED


@pytest.mark.parametrize("fmt_name", ["fp8_e4m3", "q8_0"])
@pytest.mark.parametrize("case", ["verify_gqa6", "chunk", "window", "masked_rows", "long_few_rows", "bf16_io"])
def test_8bit_stream_kernel_geometries_against_the_fp32_kernel(env, case, fmt_name, request):
    """The tensor-core path of the 8-bit layers against this library's fp32 dequant-then-attend kernel (itself
    pinned above) and, when it travelled, the reference's scalar kernel: draft tokens with 24 query
    rows per kv head, a prefill chunk, a sliding window, masked tokens and requests, one long sequence
    cut into many shares, bf16 activations.  The pool is pre-filled with 0xFF bytes (NaN as e4m3 codes
    and as scales), so a key past a row's last visible position that leaked into a product would show."""
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    fmt = ffi.KV_FORMAT_Q8_0 if fmt_name == "q8_0" else ffi.KV_FORMAT_FP8_E4M3
    hq, hkv = 24, 4
    ctx, q_len, kw = {
        "verify_gqa6": ([300, 1000, 17, 64], 4, {}),
        "chunk": ([90, 260], 70, {}),
        "window": ([700, 130, 2000], 2, dict(sliding_window=128)),
        "masked_rows": ([500, 40, 260], 3, {}),
        "long_few_rows": ([40000], 1, {}),
        "bf16_io": ([700, 31], 1, {}),
    }[case]
    n = len(ctx)
    wl = _workload(env, fmt, ctx, hkv, seed=61, fill=0xFF)
    k, v = synth.make_kv(sum(ctx), hkv, 61)
    ex = env["kv"].Executor(64 << 20)
    kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c in zip(wl.seqs, ctx):
        s.commit(c - q_len)
    if case == "masked_rows":
        vtm = np.ones(n * q_len, np.uint8)
        vtm[1] = 0
        vtm[-1] = 0
        kw = dict(valid_token_mask=vtm, valid_req_mask=np.asarray([1, 0, 1], np.uint8))
    b = wl.step(q_lens=[q_len] * n, **kw)
    q = synth.make_q(n * q_len, hq, 62).cuda()
    if case == "bf16_io":
        # bf16 activations (warp34_tq4_paged_attention_bf16): stream kernel against the fp32 kernel
        fn = env["lib"].warp34_tq4_paged_attention_bf16
        qb = q.to(torch.bfloat16)
        res = []
        for flags in (0, ffi.EXEC_FLAG_PRECISE_ATTENTION):
            ex.ex.flags = flags
            o = torch.zeros(n * q_len, hq, 256, dtype=torch.bfloat16, device="cuda")
            assert fn(C.byref(ex.ex), C.byref(wl.layer.layout), C.byref(b.desc), qb.data_ptr(), o.data_ptr(), hq) == 0
            torch.cuda.synchronize()
            res.append(o.float().cpu().numpy())
        ex.ex.flags = 0
        assert np.isfinite(res[0]).all() and np.abs(res[1]).max() > 0.1
        assert np.all(np.abs(res[0] - res[1]) <= ATOL + RTOL * np.abs(res[1])), float(np.abs(res[0] - res[1]).max())
        return
    out = torch.full((n * q_len, hq, 256), 0, dtype=torch.int16, device="cuda")
    out.fill_(0x5500)
    kv.paged_attention(ex, wl.layer, b, q, out.view(torch.float16), hq)
    torch.cuda.synchronize()
    assert int(ex.scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
    want = torch.full_like(out, 0)
    want.fill_(0x5500)
    ex.ex.flags = ffi.EXEC_FLAG_PRECISE_ATTENTION
    kv.paged_attention(ex, wl.layer, b, q, want.view(torch.float16), hq)
    ex.ex.flags = 0
    torch.cuda.synchronize()
    gb, wb = out.cpu().numpy().view(np.uint16), want.cpu().numpy().view(np.uint16)
    untouched = (wb == 0x5500).all(axis=(1, 2))
    if case == "masked_rows":
        assert untouched.sum() == 5                # token 1, the last token, request 1's three tokens
    assert ((gb == 0x5500).all(axis=(1, 2)) == untouched).all(), "masked rows differ"
    g, w = gb.view(np.float16).astype(np.float32)[~untouched], wb.view(np.float16).astype(np.float32)[~untouched]
    assert np.isfinite(g).all() and np.isfinite(w).all()
    assert np.all(np.abs(g - w) <= ATOL + RTOL * np.abs(w)), float(np.abs(g - w).max())
    try:
        ref = request.getfixturevalue("ref_lib")
    except pytest.skip.Exception:
        return
    if case in ("window",):
        return   # the reference's scalar kernel has no window argument of its own to compare here
    r = torch.zeros(n * q_len, hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(ex, wl.layer, b, q, r, hq, lib=ref, scalar=True)
    torch.cuda.synchronize()
    rr = r.float().cpu().numpy()[~untouched]
    assert np.isfinite(rr).all()
    assert np.all(np.abs(g - rr) <= ATOL + RTOL * np.abs(rr)), float(np.abs(g - rr).max())


@pytest.mark.parametrize("fmt_name", ["fp8_e4m3", "q8_0"])
def test_8bit_layers_serve_a_batch_in_several_passes_when_the_workspace_is_small(env, fmt_name):
    """300 decode requests on an 8-bit layer with 2 MiB of workspace (a slot per (request, kv head) alone
    is 9.9 MB): the tensor-core stream kernel runs over part of the requests at a time instead of
    leaving the batch to the fp32 kernel.  The status word shows which kernels ran, the plan header that
    the last pass held fewer items than the batch."""
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    fmt = {"q8_0": ffi.KV_FORMAT_Q8_0, "fp8_e4m3": ffi.KV_FORMAT_FP8_E4M3}[fmt_name]
    rng = np.random.default_rng(5)
    hq, hkv, n = 24, 4, 300
    ctx = [int(x) for x in rng.integers(1, 400, size=n)]
    wl = _workload(env, fmt, ctx, hkv, seed=9)
    fill = kv.Executor(16 << 20)
    k, v = synth.make_kv(sum(ctx), hkv, 9)
    kv.kv_cache_write(fill, wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c in zip(wl.seqs, ctx):
        s.commit(c - 1)
    vtm = (rng.random(n) > 0.1).astype(np.uint8)
    b = wl.step(q_lens=[1] * n, valid_token_mask=vtm)
    q = synth.make_q(n, hq, 10).cuda()
    outs = {}
    for name, ex, flags in (("small", kv.Executor(2 << 20), 0), ("fp32", kv.Executor(1 << 20), ffi.EXEC_FLAG_PRECISE_ATTENTION)):
        ex.ex.flags = flags
        ex.scratch[:16].fill_(0x7f)
        out = torch.full((n, hq, 256), 0, dtype=torch.int16, device="cuda")
        out.fill_(0x5500)
        kv.paged_attention(ex, wl.layer, b, q, out.view(torch.float16), hq)
        torch.cuda.synchronize()
        outs[name] = out.cpu().numpy().view(np.uint16)
        if name == "small":
            hdr = ex.scratch[:16].cpu().numpy().view(np.int32)
            assert hdr[0] == 0, "status: the stream kernel did not run or reported a failure"
            assert 0 < hdr[1] < n * hkv, int(hdr[1])
    untouched = (outs["fp32"] == 0x5500).all(axis=(1, 2))
    assert (untouched == (vtm == 0)).all()
    assert ((outs["small"] == 0x5500).all(axis=(1, 2)) == untouched).all(), "masked rows differ"
    got = outs["small"][~untouched].view(np.float16).astype(np.float32)
    want = outs["fp32"][~untouched].view(np.float16).astype(np.float32)
    d = np.abs(got - want)
    assert np.all(d <= ATOL + RTOL * np.abs(want)), float((d / (ATOL + RTOL * np.abs(want))).max())
