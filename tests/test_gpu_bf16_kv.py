"""GPU parity tests of the uncompressed BF16 KV path (warp34_kv_cache_write[_strided]_bf16,
warp34_paged_attention_bf16), through the C ABI.

Append: stored rows are the input rows bit for bit, everything else keeps its fill byte; compared
with the reference's kernels as well when oracle/_ref travelled.  Attention: |a-b| <= 2e-3 +
1e-2|b| against a float64 dequant-free attention over the same rows (the bf16 result rounding,
2^-9 relative, sits inside the relative term), and against the reference's kernel."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    return dict(ffi=ffi, kv=kv, synth=synth, ex=kv.Executor(64 << 20), lib=native_libs[0])


@pytest.fixture(scope="module")
def ref_lib(env):
    import oracle
    p = oracle.ref_lib_path()
    if p is None:
        pytest.skip("reference kernels not built (oracle/_ref)")
    return env["ffi"].bind_kernel_abi(p)


def _workload(env, ctx, q_lens, hkv, seed, fill=None):
    kv, synth = env["kv"], env["synth"]
    wl = synth.PagedWorkload(ctx, q_lens, hkv, seed, fill=fill, formats=kv.BF16_KV_FORMATS)
    kept = wl.fill_context(env["ex"], seed, keep=True)
    return wl, kept


def _reference_attention(kept, new_kv, q, ctx, q_lens, hq, hkv, sm_scale, window=0, symmetric=False):
    """float64 softmax(q k^T * scale) v per request; rows follow the kernel's mask rules
    (op_kv_cache.cu:916-931): keys [max(0, pos - window + 1), pos] with pos = ctx + offset, or up
    to the end of the sequence in the symmetric mode."""
    g = hq // hkv
    out = np.zeros((q.shape[0], hq, 256), np.float64)
    t0 = 0
    for i, (c, ql) in enumerate(zip(ctx, q_lens)):
        k_all = torch.cat([x for x in (kept[i][0], new_kv[0][t0:t0 + ql]) if x is not None]).double().numpy()
        v_all = torch.cat([x for x in (kept[i][1], new_kv[1][t0:t0 + ql]) if x is not None]).double().numpy()
        k_all = k_all.reshape(-1, hkv, 256)
        v_all = v_all.reshape(-1, hkv, 256)
        for off in range(ql):
            pos = c + off
            hi = (c + ql - 1) if symmetric else pos
            lo = max(0, pos - window + 1) if window > 0 else 0
            if lo > hi:
                continue
            for h in range(hq):
                s = (k_all[lo:hi + 1, h // g] @ q[t0 + off, h].double().numpy()) * sm_scale
                w = np.exp(s - s.max())
                out[t0 + off, h] = (w / w.sum()) @ v_all[lo:hi + 1, h // g]
        t0 += ql
    return out


def _assert_close(got, want, what):
    bad = np.abs(got - want) > ATOL + RTOL * np.abs(want)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outside tolerance, max err {np.abs(got - want).max():.3e}"


def test_append_stores_rows_bit_for_bit_and_touches_nothing_else(env):
    kv, synth = env["kv"], env["synth"]
    hkv, ctx = 4, [0, 0, 0]
    q_lens = [37, 1, 16]
    wl = synth.PagedWorkload(ctx, q_lens, hkv, 5, fill=0xA5, formats=kv.BF16_KV_FORMATS)
    T = sum(q_lens)
    k, v = synth.make_kv(T, hkv, 3)
    k, v = k.to(torch.bfloat16), v.to(torch.bfloat16)
    # packed [K | V] activations: one buffer, row stride 2 * heads * 256 elements
    packed = torch.cat([k, v], dim=1).cuda().contiguous()
    vtm = np.ones(T, np.uint8); vtm[5] = 0
    vrm = np.array([1, 0, 1], np.uint8)
    b = wl.step(valid_token_mask=vtm, valid_req_mask=vrm)
    slots = b.host["write_slot_mapping"].copy()
    slots[40] = -1
    b2 = kv.StepBatch(b.host["query_start_loc"], b.host["context_lens_before"], b.host["seq_lens_after"],
                      b.host["block_tables"], slots, wl.max_blocks, 0.0625, valid_token_mask=vtm, valid_req_mask=vrm)
    kv.kv_cache_write_bf16(env["ex"], wl.layer, b2, packed[:, :hkv * 256], packed[:, hkv * 256:],
                           row_stride_elems=2 * hkv * 256)
    torch.cuda.synchronize()
    lay = wl.layer.layout
    kp = wl.layer.k.cpu().numpy()
    vp = wl.layer.v.cpu().numpy()
    want_k = np.full_like(kp, 0xA5)
    want_v = np.full_like(vp, 0xA5)
    kb = k.view(torch.int16).numpy().view(np.uint8).reshape(T, hkv, 512)
    vb = v.view(torch.int16).numpy().view(np.uint8).reshape(T, hkv, 512)
    qsl = b.host["query_start_loc"]
    for t in range(T):
        r = int(np.searchsorted(qsl, t, side="right") - 1)
        if not vtm[t] or not vrm[r] or slots[t] < 0:
            continue
        page, off = divmod(int(slots[t]), 16)
        for h in range(hkv):
            o = page * lay.k_page_stride_bytes + h * lay.k_head_stride_bytes + off * lay.k_token_stride_bytes
            want_k[o:o + 512] = kb[t, h]
            o = page * lay.v_page_stride_bytes + h * lay.v_head_stride_bytes + off * lay.v_token_stride_bytes
            want_v[o:o + 512] = vb[t, h]
    assert (kp == want_k).all()
    assert (vp == want_v).all()
    # unaligned source (odd element offset): the 2-byte path must give the same bytes
    wl2 = synth.PagedWorkload(ctx, q_lens, hkv, 5, fill=0xA5, formats=kv.BF16_KV_FORMATS)
    shifted = torch.zeros(packed.numel() + 1, dtype=torch.bfloat16, device="cuda")
    shifted[1:] = packed.reshape(-1)
    view = shifted[1:].view(T, 2 * hkv * 256)
    b3 = kv.StepBatch(b.host["query_start_loc"], b.host["context_lens_before"], b.host["seq_lens_after"],
                      b.host["block_tables"], slots, wl2.max_blocks, 0.0625, valid_token_mask=vtm, valid_req_mask=vrm)
    kv.kv_cache_write_bf16(env["ex"], wl2.layer, b3, view[:, :hkv * 256], view[:, hkv * 256:],
                           row_stride_elems=2 * hkv * 256)
    torch.cuda.synchronize()
    assert (wl2.layer.k.cpu().numpy() == want_k).all()
    assert (wl2.layer.v.cpu().numpy() == want_v).all()


def test_wrong_descriptor_is_rejected(env):
    kv, synth = env["kv"], env["synth"]
    wl = synth.PagedWorkload([0], [4], 2, 1)          # TQ4 layer
    k, v = synth.make_kv(4, 2, 1)
    with pytest.raises(RuntimeError):
        kv.kv_cache_write_bf16(env["ex"], wl.layer, wl.step(), k.to(torch.bfloat16).cuda(), v.to(torch.bfloat16).cuda())
    q = torch.zeros(4, 4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        kv.paged_attention_bf16kv(env["ex"], wl.layer, wl.step(), q, torch.zeros_like(q), 4)


@pytest.mark.parametrize("hq,hkv,q_len", [(16, 4, 1), (24, 4, 1), (24, 4, 4), (8, 8, 1), (20, 2, 3), (16, 4, 9)])
def test_attention_matches_float64_reference_on_ragged_batches(env, hq, hkv, q_len):
    kv, synth = env["kv"], env["synth"]
    ctx = [max(c, 0) for c in [0, 15, 16, 17, 250, 1000, 33]]
    q_lens = [q_len] * len(ctx)
    wl, kept = _workload(env, ctx, q_lens, hkv, seed=300 + hq + q_len, fill=0xFF)   # 0xFFFF = a bf16 NaN
    T = sum(q_lens)
    k_new, v_new = synth.make_kv(T, hkv, 77)
    q = synth.make_q(T, hq, 78)
    b = wl.step()
    kv.kv_cache_write_bf16(env["ex"], wl.layer, b, k_new.to(torch.bfloat16).cuda(), v_new.to(torch.bfloat16).cuda())
    out = torch.full((T, hq, 256), 9.0, dtype=torch.bfloat16, device="cuda")
    kv.paged_attention_bf16kv(env["ex"], wl.layer, b, q.to(torch.bfloat16).cuda(), out, hq)
    torch.cuda.synchronize()
    want = _reference_attention(kept, (k_new, v_new), q, ctx, q_lens, hq, hkv, 0.0625)
    _assert_close(out.float().cpu().numpy().astype(np.float64), want, "bf16 KV attention")
    assert int(env["ex"].scratch[:4].cpu().numpy().view(np.int32)[0]) == 0


def test_windows_masks_and_small_scratch(env):
    kv, synth = env["kv"], env["synth"]
    hq, hkv, ql = 8, 2, 3
    ctx, q_lens = [90, 41, 300], [ql] * 3
    wl, kept = _workload(env, ctx, q_lens, hkv, seed=21)
    T = sum(q_lens)
    k_new, v_new = synth.make_kv(T, hkv, 5)
    q = synth.make_q(T, hq, 6)
    kv.kv_cache_write_bf16(env["ex"], wl.layer, wl.step(), k_new.to(torch.bfloat16).cuda(), v_new.to(torch.bfloat16).cuda())
    qd = q.to(torch.bfloat16).cuda()
    small = kv.Executor(1 << 20)      # a few CTAs' worth of partial slots: the grid shrinks
    for window, symmetric in [(0, False), (32, False), (7, False), (40, True)]:
        vtm = np.ones(T, np.uint8); vtm[4] = 0
        vrm = np.array([1, 1, 0], np.uint8)
        b = wl.step(sliding_window=window, mask_mode=1 if symmetric else 0, valid_token_mask=vtm, valid_req_mask=vrm)
        want = _reference_attention(kept, (k_new, v_new), q, ctx, q_lens, hq, hkv, 0.0625, window, symmetric)
        for ex in (env["ex"], small):
            out = torch.full((T, hq, 256), 9.0, dtype=torch.bfloat16, device="cuda")
            kv.paged_attention_bf16kv(ex, wl.layer, b, qd, out, hq)
            torch.cuda.synchronize()
            got = out.float().cpu().numpy().astype(np.float64)
            live = np.ones(T, bool); live[4] = False; live[6:] = False
            _assert_close(got[live], want[live], f"window {window} symmetric {symmetric}")
            assert (got[~live] == 9.0).all(), "masked rows must stay untouched"


def test_matches_the_reference_kernels(env, ref_lib):
    kv, synth = env["kv"], env["synth"]
    hq, hkv = 24, 4
    ctx, q_lens = [700, 64, 2049, 5], [1, 1, 1, 1]
    wl, kept = _workload(env, ctx, q_lens, hkv, seed=8)
    T = sum(q_lens)
    k_new, v_new = synth.make_kv(T, hkv, 9)
    q = synth.make_q(T, hq, 10).to(torch.bfloat16).cuda()
    b = wl.step()
    kb, vb = k_new.to(torch.bfloat16).cuda(), v_new.to(torch.bfloat16).cuda()
    kv.kv_cache_write_bf16(env["ex"], wl.layer, b, kb, vb)
    torch.cuda.synchronize()
    mine_k, mine_v = wl.layer.k.clone(), wl.layer.v.clone()
    # the reference's append over the same descriptor writes the same bytes
    kv.kv_cache_write_bf16(env["ex"], wl.layer, b, kb, vb, lib=ref_lib)
    torch.cuda.synchronize()
    assert torch.equal(mine_k, wl.layer.k) and torch.equal(mine_v, wl.layer.v)
    out = torch.zeros(T, hq, 256, dtype=torch.bfloat16, device="cuda")
    ref = torch.zeros_like(out)
    kv.paged_attention_bf16kv(env["ex"], wl.layer, b, q, out, hq)
    kv.paged_attention_bf16kv(env["ex"], wl.layer, b, q, ref, hq, lib=ref_lib)
    torch.cuda.synchronize()
    got, theirs = out.float().cpu().numpy().astype(np.float64), ref.float().cpu().numpy().astype(np.float64)
    want = _reference_attention(kept, (k_new, v_new), q.float().cpu(), ctx, q_lens, hq, hkv, 0.0625)
    _assert_close(got, want, "bf16 KV attention")
    # The reference rounds the softmax weights to bf16 before P.V (8 mantissa bits), so it sits
    # further from the exact result than this path does: the two are compared with a term of
    # 2^-7 x the largest |V| of the channel on top of the usual bound.
    vmax = np.zeros((hkv, 256))
    for kk, vv in kept:
        vmax = np.maximum(vmax, np.abs(vv.double().numpy()).reshape(-1, hkv, 256).max(axis=0))
    ch = np.repeat(vmax, hq // hkv, axis=0)[None]
    bad = np.abs(got - theirs) > ATOL + RTOL * np.abs(theirs) + 2.0 ** -7 * ch
    assert not bad.any(), f"vs reference bf16 kernel: {bad.sum()} of {bad.size}"
    assert np.abs(got - want).max() <= np.abs(theirs - want).max()
