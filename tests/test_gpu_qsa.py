"""GPU parity of the query-sparse paged attention entry points (warp34_qsa_sparse_paged_attn_f16 /
_hadamard_f16), through the C ABI, against the reference's own kernels (op_qsa.cu compiled unmodified
into oracle/_ref) run on the same pool, lists and queries, against the committed fixture of those
kernels' outputs, and against the float64 restatement (oracle/qsa.py).  Bound: 2e-3 + 1e-2 |b| on
every element; masked tokens must come out as exact zeros."""
import ctypes as C
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-2
FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qsa_ref_sm100a.npz")


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    import oracle
    p = oracle.ref_lib_path()
    ref = C.CDLL(p) if p else None
    return dict(ffi=ffi, kv=kv, synth=synth, lib=native_libs[0], ref=ref)


def _call(lib, name, ex, q, gate, layer, phys, logical, n_sel, pos, mask, out, hq, select_k, num_tokens=None):
    fn = getattr(lib, name)
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 10 + [C.c_int, C.c_int, C.c_int, C.c_float]
    return fn(C.addressof(ex.ex), q.data_ptr(), None if gate is None else gate.data_ptr(), C.addressof(layer.layout),
              phys.data_ptr(), logical.data_ptr(), n_sel.data_ptr(), pos.data_ptr(),
              None if mask is None else mask.data_ptr(), out.data_ptr(), q.shape[0] if num_tokens is None else num_tokens,
              hq, select_k, 0.0625)


def _lists(wl, ctx, tokens, select_k, rng, drop=True):
    """tokens: (sequence, position) per token.  Random groups of the sequence plus the token's own."""
    T = len(tokens)
    phys = np.full((T, select_k), -1, np.int32)
    logical = np.zeros((T, select_k), np.int32)
    n_sel = np.zeros(T, np.int32)
    for t, (s, pos) in enumerate(tokens):
        pages = wl.seqs[s].pages
        groups = (ctx[s] + 3) // 4
        own = pos // 4
        pick = [own] + [int(g) for g in rng.permutation(groups) if g != own][:select_k - 1]
        for i, g in enumerate(pick):
            logical[t, i] = g
            phys[t, i] = pages[g // 4] * 4 + (g % 4)
        n_sel[t] = len(pick)
        if drop and len(pick) > 3:
            phys[t, 1] = -1
    return phys, logical, n_sel


FORMATS = {"tq4": (2, 1), "fp8": (4, 0), "q8": (3, 0)}


@pytest.mark.parametrize("fmt_name", ["tq4", "fp8", "q8"])
@pytest.mark.parametrize("hq,hkv", [(24, 4), (16, 4), (8, 8), (20, 2)])
@pytest.mark.parametrize("variant", ["plain", "gated", "hadamard"])
def test_sparse_attention_matches_the_reference_kernel(env, fmt_name, hq, hkv, variant):
    if env["ref"] is None:
        pytest.skip("reference kernels not built (oracle/_ref)")
    kv, synth = env["kv"], env["synth"]
    fmt, tr = FORMATS[fmt_name]
    ctx = [700, 130, 2000]
    select_k = 96
    wl = synth.PagedWorkload([0] * 3, ctx, hkv, seed=71, fill=0xFF, formats=(fmt, fmt, tr, tr))
    ex = kv.Executor(32 << 20)
    k, v = synth.make_kv(sum(ctx), hkv, 71)
    kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
    rng = np.random.default_rng(5)
    tokens = [(0, 699), (0, 350), (1, 129), (2, 1999), (2, 3), (1, 64), (2, 1000)]
    phys, logical, n_sel = _lists(wl, ctx, tokens, select_k, rng)
    n_sel[5] = 0
    T = len(tokens)
    vtm = np.ones(T, np.uint8)
    vtm[6] = 0
    g = torch.Generator().manual_seed(9)
    q = torch.randn(T, hq, 256, generator=g).to(torch.float16).cuda()
    gate = (torch.randn(T, hq, 256, generator=g) * 2).to(torch.float16).cuda()
    dev = [torch.from_numpy(a).cuda() for a in (phys, logical, n_sel, np.asarray([p for _, p in tokens], np.int32), vtm)]
    name = "warp34_qsa_sparse_paged_attn_hadamard_f16" if variant == "hadamard" else "warp34_qsa_sparse_paged_attn_f16"
    gt = None if variant == "plain" else gate
    outs = {}
    precise = kv.Executor(32 << 20)
    precise.ex.flags = env["ffi"].EXEC_FLAG_PRECISE_ATTENTION
    for who, lib, scratch in (("ours", env["lib"], True), ("unsplit", env["lib"], False), ("fp32", env["lib"], None),
                              ("ref", env["ref"], True)):
        e = precise if scratch is None else ex if scratch else kv.Executor(0)
        out = torch.full((T, hq, 256), 0, dtype=torch.int16, device="cuda")
        out.fill_(0x5500)
        assert _call(lib, name, e, q, gt, wl.layer, *dev, out, hq, select_k) == 0
        torch.cuda.synchronize()
        if who == "ours":
            # lists with a workspace run on the tensor-core stream kernels: their status word stays clear
            assert int(e.scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
        outs[who] = out.cpu().numpy().view(np.uint16)
    want = outs["ref"].view(np.float16).astype(np.float32)
    assert np.isfinite(want).all() and np.abs(want).max() > 0.05
    for who in ("ours", "unsplit", "fp32"):
        got = outs[who].view(np.float16).astype(np.float32)
        # the masked token is written as zero bits; the token without entries comes out as (signed) zeros
        assert (outs[who][6] == 0).all() and (got[5] == 0).all(), "masked / empty token is not zero"
        assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want)), (who, float(np.abs(got - want).max()))


@pytest.mark.parametrize("fmt_name", ["tq4", "fp8"])
@pytest.mark.parametrize("variant", ["plain", "gated", "hadamard"])
def test_sparse_attention_reproduces_the_committed_fixture(env, fmt_name, variant):
    if not os.path.exists(FIXTURE):
        pytest.skip("fixture not generated yet")
    kv, ffi = env["kv"], env["ffi"]
    fx = dict(np.load(FIXTURE))
    fmt, tr = FORMATS[fmt_name]
    kp, vp = fx[f"{fmt_name}_k_pool"], fx[f"{fmt_name}_v_pool"]
    pages, hkv = kp.shape[0], kp.shape[1]
    layer = kv.KvLayer(pages, hkv, formats=(fmt, fmt, tr, tr))
    layer.k.copy_(torch.from_numpy(kp.reshape(-1)))
    layer.v.copy_(torch.from_numpy(vp.reshape(-1)))
    q = torch.from_numpy(fx["q"].view(np.int16)).cuda()
    gate = torch.from_numpy(fx["gate"].view(np.int16)).cuda()
    T, hq = q.shape[0], q.shape[1]
    dev = [torch.from_numpy(fx[n]).cuda() for n in ("sel_phys", "sel_logical", "num_selected", "seq_pos", "valid_token_mask")]
    name = "warp34_qsa_sparse_paged_attn_hadamard_f16" if variant == "hadamard" else "warp34_qsa_sparse_paged_attn_f16"
    out = torch.full((T, hq, 256), 0, dtype=torch.int16, device="cuda")
    out.fill_(0x5500)
    ex = kv.Executor(8 << 20)
    assert _call(env["lib"], name, ex, q, None if variant == "plain" else gate, layer, *dev, out, hq,
                 fx["sel_phys"].shape[1]) == 0
    torch.cuda.synchronize()
    got_bits = out.cpu().numpy().view(np.uint16)
    want_bits = fx[f"{fmt_name}_out_{variant}"]
    got, want = got_bits.view(np.float16).astype(np.float32), want_bits.view(np.float16).astype(np.float32)
    assert (got_bits[3] == 0).all() and (got[2] == 0).all()
    assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want)), float(np.abs(got - want).max())
    # and the float64 restatement on the same inputs
    from oracle import qsa
    r = qsa.sparse_attention(kp, vp, fmt, fmt, fx["q"].view(np.float16).astype(np.float32),
                             None if variant == "plain" else fx["gate"].view(np.float16).astype(np.float32),
                             fx["sel_phys"], fx["sel_logical"], fx["num_selected"], fx["seq_pos"],
                             fx["valid_token_mask"], hq, hkv, 0.0625, variant == "hadamard")
    assert np.all(np.abs(got - r) <= ATOL + RTOL * np.abs(r)), float(np.abs(got - r).max())


def test_sparse_attention_validates_like_the_reference(env):
    kv, ffi = env["kv"], env["ffi"]
    layer = kv.KvLayer(4, 2)
    ex = kv.Executor(1 << 20)
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    q = torch.zeros(1, 4, 256, dtype=torch.float16, device="cuda")
    out = torch.zeros_like(q)
    name = "warp34_qsa_sparse_paged_attn_f16"
    assert _call(env["lib"], name, ex, q, None, layer, z, z, z, z, None, out, 3, 4) == 1      # 3 q heads on 2 kv heads
    assert _call(env["lib"], name, ex, q, None, layer, z, z, z, z, None, out, 4, -1) == 1     # negative list width
    fp16 = kv.KvLayer(4, 2)
    fp16.layout.k_format = ffi.KV_FORMAT_FP16
    assert _call(env["lib"], name, ex, q, None, fp16, z, z, z, z, None, out, 4, 4) == ffi.CUDA_ERROR_NOT_SUPPORTED
    assert _call(env["lib"], name, ex, q, None, layer, z, z, z, z, None, out, 4, 4, num_tokens=0) == 0   # no tokens
