"""The attention output epilogue of the reference's layer, fused into the attention kernels
(warp34_paged_attention_gated_f16) and as stand-alone steps with the reference's own names
(warp34_apply_attn_output_gate_f16 / _hadamard_f16, crates/warp34-host/src/model/forward.rs:1192-1211,
crates/warp34-kernels/csrc/ops/op_norms_rope_act.cu:742-764, :805-851).

Oracle: attention by the CPU oracle, then the gate (and the Hadamard-64 per 64 columns) in numpy with
the two-kernel sequence's roundings.  The stand-alone steps are also compared with the reference's
own kernels when oracle/_ref holds them (oracle/build_ref.sh compiles op_norms_rope_act.cu as well)."""
import ctypes as C

import numpy as np
import pytest

from util import f16, host_layout, plain_parity

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _h64(x):
    """Normalised 64-point Hadamard over every 64 consecutive columns (x 1/8), fp32."""
    h = np.array([[1.0]], np.float32)
    while h.shape[0] < 64:
        h = np.block([[h, h], [h, -h]])
    shape = x.shape
    return ((x.reshape(-1, 64) @ h) * np.float32(0.125)).reshape(shape)


def _gate_oracle(attn_f16, gate_f16, hadamard):
    a = attn_f16.astype(np.float32)
    g = gate_f16.astype(np.float32)
    y = (a * (1.0 / (1.0 + np.exp(-g)))).astype(np.float16)
    if hadamard:
        y = _h64(y.astype(np.float32).reshape(y.shape[0], -1)).reshape(y.shape).astype(np.float16)
    return y.astype(np.float32)


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    return dict(ffi=ffi, kv=kv, synth=synth, ex=kv.Executor(64 << 20), lib=native_libs[0])


def _oracle_attention(wl, batch, q, hq):
    import oracle
    hk, hv = wl.layer.k.cpu().numpy(), wl.layer.v.cpu().numpy()
    lay = host_layout(wl.layer.layout, hk, hv)
    out = np.zeros((q.shape[0], hq, 256), np.uint16)
    assert oracle.paged_attention(lay, batch.host_desc(), q.numpy().view(np.uint16), out, hq, nthreads=8) == 0
    return out.view(np.float16)


@pytest.mark.parametrize("hadamard", [False, True])
@pytest.mark.parametrize("shape", ["decode", "verify", "chunk", "chunk_fast", "fp32"])
def test_fused_epilogue_matches_attention_then_gate(env, shape, hadamard):
    kv, synth, ffi = env["kv"], env["synth"], env["ffi"]
    hq, hkv = 24, 4
    ctx, q_len = {"decode": ([700, 31, 2000], 1), "verify": ([300, 1000], 4), "chunk": ([90, 260], 70),
                  "chunk_fast": ([90, 260], 70), "fp32": ([500, 40], 1)}[shape]
    flags = {"chunk_fast": ffi.EXEC_FLAG_FAST_ATTENTION, "fp32": ffi.EXEC_FLAG_PRECISE_ATTENTION}.get(shape, 0)
    n = len(ctx)
    wl = synth.PagedWorkload([0] * n, ctx, hkv, seed=900)
    k, v = synth.make_kv(sum(ctx), hkv, 900)
    kv.kv_cache_write(env["ex"], wl.layer, wl.step(), k.cuda(), v.cuda())
    for s, c in zip(wl.seqs, ctx):
        s.commit(c - q_len)
    vtm = np.ones(n * q_len, np.uint8)
    vtm[-1] = 0
    b = wl.step(q_lens=[q_len] * n, valid_token_mask=vtm)
    q = synth.make_q(n * q_len, hq, 901)
    gate = synth.make_q(n * q_len, hq, 902) * 2.0
    out = torch.full((n * q_len, hq, 256), 0, dtype=torch.int16, device="cuda")
    out.fill_(0x5500)
    ex = kv.Executor(64 << 20)
    ex.ex.flags = flags
    kv.paged_attention_gated(ex, wl.layer, b, q.cuda(), gate.cuda(), out.view(torch.float16), hq, hadamard64=hadamard)
    torch.cuda.synchronize()
    bits = out.cpu().numpy().view(np.uint16)
    assert (bits[-1] == 0x5500).all(), "masked row was written"
    live = vtm.astype(bool)
    attn = _oracle_attention(wl, b, q, hq)
    want = _gate_oracle(attn, gate.numpy(), hadamard)
    got = f16(bits)
    if shape == "chunk_fast":
        d = np.abs(got[live] - want[live])
        assert (d <= 2e-3 + 1e-2 * np.abs(want[live])).mean() >= 0.999 and d.max() < 0.2
    else:
        ok, msg = plain_parity(got[live], want[live])
        assert ok, (shape, hadamard, msg)


@pytest.mark.parametrize("hadamard", [False, True])
@pytest.mark.parametrize("total_dim", [6144, 320])
def test_stand_alone_gate_steps(env, hadamard, total_dim):
    lib, synth = env["lib"], env["synth"]
    t = 37
    g = torch.Generator().manual_seed(5)
    attn = (torch.randn(t, total_dim, generator=g) * 3).to(torch.float16)
    gate = (torch.randn(t, total_dim, generator=g) * 2).to(torch.float16)
    vtm = np.ones(t, np.uint8)
    vtm[5] = 0
    mask = torch.from_numpy(vtm).cuda()
    out = torch.full((t, total_dim), 0, dtype=torch.int16, device="cuda")
    out.fill_(0x5500)
    fn = lib.warp34_apply_attn_output_gate_hadamard_f16 if hadamard else lib.warp34_apply_attn_output_gate_f16
    a_dev, g_dev = attn.cuda(), gate.cuda()
    assert fn(C.byref(env["ex"].ex), a_dev.data_ptr(), g_dev.data_ptr(), out.data_ptr(), mask.data_ptr(), t, total_dim) == 0
    torch.cuda.synchronize()
    bits = out.cpu().numpy().view(np.uint16)
    assert (bits[5] == 0x5500).all()
    want = _gate_oracle(attn.numpy(), gate.numpy(), hadamard)
    live = vtm.astype(bool)
    d = np.abs(f16(bits)[live] - want[live])
    # one fp16 step of the result: the sigmoid uses the fast exponential
    assert (d <= 2e-3 + 2.0 ** -10 * np.abs(want[live])).all(), d.max()
    # in place
    assert fn(C.byref(env["ex"].ex), a_dev.data_ptr(), g_dev.data_ptr(), a_dev.data_ptr(), None, t, total_dim) == 0
    torch.cuda.synchronize()
    d2 = np.abs(a_dev.float().cpu().numpy()[live] - want[live])
    assert (d2 <= 2e-3 + 2.0 ** -10 * np.abs(want[live])).all()
    if hadamard:
        assert fn(C.byref(env["ex"].ex), a_dev.data_ptr(), g_dev.data_ptr(), out.data_ptr(), None, t, 100) == 1
    # the reference's own kernels on the same inputs (when its unit was built into oracle/_ref): the same bits
    # (the sigmoid is ex2.approx and rcp.approx, as its -use_fast_math build lowers expf and the division)
    import oracle
    path = oracle.ref_lib_path()
    ref = C.CDLL(path) if path else None
    name = "warp34_apply_attn_output_gate_hadamard_f16" if hadamard else "warp34_apply_attn_output_gate_f16"
    if ref is None or not hasattr(ref, name):
        return
    rfn = getattr(ref, name)
    rfn.restype = C.c_int
    rfn.argtypes = [C.c_void_p] * 5 + [C.c_int, C.c_int]
    out_r = torch.full((t, total_dim), 0, dtype=torch.int16, device="cuda")
    out_r.fill_(0x5500)
    a2 = attn.cuda()
    assert rfn(C.addressof(env["ex"].ex), a2.data_ptr(), g_dev.data_ptr(), out_r.data_ptr(), mask.data_ptr(), t, total_dim) == 0
    torch.cuda.synchronize()
    rb = out_r.cpu().numpy().view(np.uint16)
    assert (rb[5] == 0x5500).all()
    assert (bits[live] == rb[live]).all(), int((bits[live] != rb[live]).sum())
