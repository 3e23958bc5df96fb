"""The bounds-checked build of the kernel library (-DW34_BOUNDS, libwarp34_b200_bounds.so): the stand-in
for the reference's sanitizer runs of this path (tools/check_cuda_sanitizer.py:77-102).

 * every kernel family runs its small cases under it with the pool's page count stated: no violation
   is recorded and the results equal the regular build's bit for bit;
 * descriptors that point outside what the host declared are caught: the record names what, where,
   the value and its limit, the access is redirected (reads) or skipped (writes).  The violating
   values are only outside the DECLARED extent (a pool declared smaller than the one allocated, a
   block table declared narrower than the array behind it), so nothing can reach unowned memory in
   either build."""
import ctypes as C
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import build, ffi, kv, synth
    path = build.build_bounds()
    assert os.path.exists(path)
    return dict(ffi=ffi, kv=kv, synth=synth, ex=kv.Executor(64 << 20), lib=native_libs[0],
                blib=ffi.bind_kernel_abi(path))


def _report(blib, reset=True):
    out = (C.c_int32 * 4)()
    assert blib.warp34_bounds_report(out, 1 if reset else 0) == 0
    return dict(what=out[0] & 255, where=out[0] >> 8, value=out[1], limit=out[2], count=out[3])


def test_regular_build_has_no_checks(env):
    out = (C.c_int32 * 4)()
    assert env["lib"].warp34_bounds_set_pool_pages(16) == 801
    assert env["lib"].warp34_bounds_report(out, 0) == 801


CASES = {
    # name: (contexts, q_len, flags name, formats)
    "decode": ([700, 31, 2000, 16], 1, None, None),
    "verify": ([300, 1000], 4, None, None),
    "verify_team": ([300, 1000], 4, "EXEC_FLAG_FAST_ATTENTION", None),
    "chunk": ([90, 260], 70, None, None),
    "chunk_tcgen05": ([90, 260], 70, "EXEC_FLAG_FAST_ATTENTION", None),
    "fp32": ([500, 40], 1, "EXEC_FLAG_PRECISE_ATTENTION", None),
    "bf16": ([400, 33], 1, None, "bf16"),
    "fp8": ([400, 33], 1, None, "fp8"),
    "q8": ([400, 33], 1, None, "q8"),
}


@pytest.mark.parametrize("name", list(CASES))
def test_small_cases_run_clean_and_equal_the_regular_build(env, name):
    kv, synth, ffi, blib = env["kv"], env["synth"], env["ffi"], env["blib"]
    ctx, q_len, flag, fmt = CASES[name]
    code = {None: None, "bf16": ffi.KV_FORMAT_BF16, "fp8": ffi.KV_FORMAT_FP8_E4M3, "q8": ffi.KV_FORMAT_Q8_0}[fmt]
    formats = None if code is None else (code, code, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY)
    hq, hkv, n = 24, 4, len(ctx)
    outs, pools = [], []
    for lib in (env["lib"], blib):
        wl = synth.PagedWorkload([c - q_len for c in ctx], [q_len] * n, hkv, seed=77, formats=formats)
        if lib is blib:
            assert blib.warp34_bounds_set_pool_pages(wl.num_pages) == 0
            _report(blib)
        ex = kv.Executor(64 << 20)
        wl.fill_context(ex, 77, lib=lib)
        b = wl.step()
        k, v = synth.make_kv(n * q_len, hkv, 78, device="cuda")
        q = synth.make_q(n * q_len, hq, 79).cuda()
        ex.ex.flags = getattr(ffi, flag) if flag else 0
        if fmt == "bf16":
            k, v, q = k.to(torch.bfloat16), v.to(torch.bfloat16), q.to(torch.bfloat16)
            out = torch.zeros(n * q_len, hq, 256, dtype=torch.bfloat16, device="cuda")
            kv.kv_cache_write_bf16(ex, wl.layer, b, k, v, lib=lib)
            kv.paged_attention_bf16kv(ex, wl.layer, b, q, out, hq, lib=lib)
        else:
            out = torch.zeros(n * q_len, hq, 256, dtype=torch.float16, device="cuda")
            kv.kv_cache_write(ex, wl.layer, b, k, v, lib=lib)
            kv.paged_attention(ex, wl.layer, b, q, out, hq, lib=lib)
        torch.cuda.synchronize()
        outs.append(out.view(torch.int16).cpu())
        pools.append((wl.layer.k.cpu(), wl.layer.v.cpu()))
    r = _report(blib)
    assert r["count"] == 0 and r["what"] == 0, r
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(pools[0][0], pools[1][0]) and torch.equal(pools[0][1], pools[1][1])
    assert outs[0].numpy().any()


def _decode_case(env, lib, seed=5):
    kv, synth = env["kv"], env["synth"]
    wl = synth.PagedWorkload([200, 90], [1, 1], 4, seed=seed, slack_pages=64)
    ex = kv.Executor(64 << 20)
    wl.fill_context(ex, seed, lib=lib)
    return wl, ex


def test_page_id_outside_the_declared_pool_is_recorded_and_redirected(env):
    kv, synth, ffi, blib = env["kv"], env["synth"], env["ffi"], env["blib"]
    assert blib.warp34_bounds_set_pool_pages(0) == 0
    wl, ex = _decode_case(env, blib)
    b = wl.step()
    k, v = synth.make_kv(2, 4, 6, device="cuda")
    kv.kv_cache_write(ex, wl.layer, b, k, v, lib=blib)
    q = synth.make_q(2, 24, 7).cuda()
    used = sorted({int(p) for s in wl.seqs for p in s.pages})
    declared = used[len(used) // 2]          # every page id >= declared is now "outside the pool"
    outside = [p for p in used if p >= declared]
    _report(blib)
    assert blib.warp34_bounds_set_pool_pages(declared) == 0
    for flags, where in ((0, 3), (ffi.EXEC_FLAG_PRECISE_ATTENTION, 2)):
        ex.ex.flags = flags
        out = torch.zeros(2, 24, 256, dtype=torch.float16, device="cuda")
        assert kv.paged_attention(ex, wl.layer, b, q, out, 24, lib=blib) in (0, None)
        torch.cuda.synchronize()
        r = _report(blib)
        assert r["what"] == 2 and r["where"] == where and r["limit"] == declared and r["value"] in outside, r
        assert r["count"] >= len(outside)
        assert torch.isfinite(out.float()).all()
    assert blib.warp34_bounds_set_pool_pages(0) == 0


def test_write_slot_outside_the_declared_pool_is_recorded_and_skipped(env):
    kv, synth, blib = env["kv"], env["synth"], env["blib"]
    wl, ex = _decode_case(env, blib, seed=9)
    b = wl.step()
    slots = b.host["write_slot_mapping"]
    declared = int(slots.max()) // 16            # the page of the larger slot is outside, the other inside
    assert int(slots.min()) // 16 < declared
    assert blib.warp34_bounds_set_pool_pages(declared) == 0
    _report(blib)
    before = (wl.layer.k.clone(), wl.layer.v.clone())
    k, v = synth.make_kv(2, 4, 10, device="cuda")
    kv.kv_cache_write(ex, wl.layer, b, k, v, lib=blib)
    torch.cuda.synchronize()
    r = _report(blib)
    assert r["what"] == 3 and r["where"] == 1 and r["value"] == int(slots.max()) and r["limit"] == declared * 16, r
    page_bytes = wl.layer.k.numel() // wl.num_pages
    kb, ka = before[0].view(torch.uint8).view(wl.num_pages, page_bytes), wl.layer.k.view(torch.uint8).view(wl.num_pages, page_bytes)
    changed = (kb != ka).any(dim=1).nonzero().flatten().tolist()
    assert changed == [int(slots.min()) // 16], changed
    assert blib.warp34_bounds_set_pool_pages(0) == 0


def test_block_table_index_beyond_the_declared_width_is_recorded(env):
    kv, synth, ffi, blib = env["kv"], env["synth"], env["ffi"], env["blib"]
    wl, ex = _decode_case(env, blib, seed=11)
    s = wl.seqs[0]
    n_tok = 200                                   # all of them appended by the fill
    pages = list(s.pages)                         # 13 pages behind the row
    bt = np.asarray([pages], np.int32)
    # the descriptor declares a 4-entry row while the sequence is 200 tokens long: entries 4..12 are
    # outside the declared width (and inside the array that is really there)
    b = kv.StepBatch([0, 1], [n_tok - 1], [n_tok], bt, [-1], 4, 0.0625, max_seq_len=64)
    _report(blib)
    ex.ex.flags = ffi.EXEC_FLAG_PRECISE_ATTENTION
    q = synth.make_q(1, 24, 12).cuda()
    out = torch.zeros(1, 24, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(ex, wl.layer, b, q, out, 24, lib=blib)
    torch.cuda.synchronize()
    r = _report(blib)
    assert r["what"] == 1 and r["where"] == 2 and r["limit"] == 4 and 4 <= r["value"] <= 12, r
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("scratch", [True, False])
def test_query_sparse_lists_run_clean_under_the_checks(env, scratch):
    """The selected-group lists of the query-sparse entry point carry page ids of their own: both of its
    kernels (stream kernel with a workspace, fp32 kernel without) check them against the declared pool."""
    kv, synth, blib = env["kv"], env["synth"], env["blib"]
    ctx = [300, 90]
    wl = synth.PagedWorkload([0, 0], ctx, 4, seed=21)
    assert blib.warp34_bounds_set_pool_pages(wl.num_pages) == 0
    _report(blib)
    ex = kv.Executor(32 << 20 if scratch else 0)
    fill = kv.Executor(8 << 20)
    k, v = synth.make_kv(sum(ctx), 4, 21)
    kv.kv_cache_write(fill, wl.layer, wl.step(), k.cuda(), v.cuda(), lib=blib)
    select_k, T = 16, 2
    phys = np.full((T, select_k), -1, np.int32)
    logical = np.zeros((T, select_k), np.int32)
    for t in range(T):
        groups = np.arange(min(select_k, (ctx[t] + 3) // 4))
        logical[t, :len(groups)] = groups
        phys[t, :len(groups)] = np.asarray(wl.seqs[t].pages)[groups // 4] * 4 + groups % 4
    dev = [torch.from_numpy(a).cuda() for a in (phys, logical, np.full(T, select_k, np.int32), np.asarray(ctx, np.int32) - 1)]
    q = synth.make_q(T, 24, 22).cuda()
    out = torch.zeros_like(q)
    fn = blib.warp34_qsa_sparse_paged_attn_f16
    assert fn(C.addressof(ex.ex), q.data_ptr(), None, C.addressof(wl.layer.layout), dev[0].data_ptr(), dev[1].data_ptr(),
              dev[2].data_ptr(), dev[3].data_ptr(), None, out.data_ptr(), T, 24, select_k, 0.0625) == 0
    torch.cuda.synchronize()
    r = _report(blib)
    assert r["count"] == 0, r
    assert torch.isfinite(out.float()).all() and out.float().abs().max() > 0.01
    # declare a pool that ends below the highest page the lists use: recorded, redirected, no fault
    top = int(phys.max()) // 4
    assert blib.warp34_bounds_set_pool_pages(top) == 0
    assert fn(C.addressof(ex.ex), q.data_ptr(), None, C.addressof(wl.layer.layout), dev[0].data_ptr(), dev[1].data_ptr(),
              dev[2].data_ptr(), dev[3].data_ptr(), None, out.data_ptr(), T, 24, select_k, 0.0625) == 0
    torch.cuda.synchronize()
    r = _report(blib)
    assert r["what"] == 2 and r["where"] in (3, 9) and r["value"] == top and r["limit"] == top, r
    assert blib.warp34_bounds_set_pool_pages(0) == 0


@pytest.mark.parametrize("fmt", [None, "fp8"])
def test_a_batch_served_in_several_passes_runs_clean_under_the_checks(env, fmt):
    """120 decode requests with 1 MiB of workspace: the launcher serves them a few at a time, every pass
    with block-table rows and request arrays offset into the batch's; no index leaves its declared range
    and the result equals the regular build's bit for bit."""
    kv, synth, ffi, blib = env["kv"], env["synth"], env["ffi"], env["blib"]
    code = None if fmt is None else ffi.KV_FORMAT_FP8_E4M3
    formats = None if code is None else (code, code, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY)
    rng = np.random.default_rng(3)
    n, hq, hkv = 120, 24, 4
    ctx = [int(x) for x in rng.integers(2, 300, size=n)]
    outs = []
    for lib in (env["lib"], blib):
        wl = synth.PagedWorkload([c - 1 for c in ctx], [1] * n, hkv, seed=91, formats=formats)
        if lib is blib:
            assert blib.warp34_bounds_set_pool_pages(wl.num_pages) == 0
            _report(blib)
        fill = kv.Executor(64 << 20)
        wl.fill_context(fill, 91, lib=lib)
        b = wl.step()
        k, v = synth.make_kv(n, hkv, 92, device="cuda")
        kv.kv_cache_write(fill, wl.layer, b, k, v, lib=lib)
        q = synth.make_q(n, hq, 93).cuda()
        ex = kv.Executor(1 << 20)
        ex.scratch[:16].fill_(0x7f)
        out = torch.zeros(n, hq, 256, dtype=torch.float16, device="cuda")
        kv.paged_attention(ex, wl.layer, b, q, out, hq, lib=lib)
        torch.cuda.synchronize()
        hdr = ex.scratch[:16].cpu().numpy().view(np.int32)
        assert hdr[0] == 0 and 0 < hdr[1] < n * hkv, hdr[:2]        # split-KV kernels, last pass smaller than the batch
        outs.append(out.view(torch.int16).cpu())
    r = _report(blib)
    assert r["count"] == 0 and r["what"] == 0, r
    assert torch.equal(outs[0], outs[1]) and outs[0].numpy().any()
    assert blib.warp34_bounds_set_pool_pages(0) == 0
