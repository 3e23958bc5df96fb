"""K-norm + RoPE + TQ4 append in one kernel (warp34_fused_k_rmsnorm_rope_kv_cache_write_f16) against the
reference's two-kernel sequence run on the same inputs: warp34_fused_qk_rmsnorm_rope_gate_strided_f16
(op_norms_rope_act.cu:524-680, :1201-1246) followed by warp34_kv_cache_write_strided, both from the
reference's own sources in oracle/_ref.  The packed bytes of the pool must be identical
(call site: crates/warp34-host/src/model/forward.rs:1109-1149)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import oracle
    from warp34_b200 import ffi, kv, synth
    p = oracle.ref_lib_path()
    if p is None:
        pytest.skip("reference kernels not built (oracle/_ref)")
    ref = C.CDLL(p)
    if not hasattr(ref, "warp34_fused_qk_rmsnorm_rope_gate_strided_f16"):
        pytest.skip("oracle/_ref was built without the reference's producer unit")
    return dict(ffi=ffi, kv=kv, synth=synth, ex=kv.Executor(16 << 20), lib=native_libs[0], ref=ref,
                ref_abi=ffi.bind_kernel_abi(p))


@pytest.mark.parametrize("hq,hkv,rotary_dim,sections", [(24, 4, 64, (11, 11, 10)), (16, 4, 64, (8, 12, 12)),
                                                       (8, 2, 128, (24, 20, 20)), (8, 2, 256, (44, 42, 42)),
                                                       # a token's heads share their sines only when four rows of a warp
                                                       # are one token's and rotary_dim / 16 is a multiple of 4
                                                       (8, 8, 128, (22, 21, 21)), (3, 3, 64, (12, 10, 10)),
                                                       (4, 1, 32, (6, 5, 5)), (8, 4, 96, (16, 16, 16))])
def test_fused_producer_append_is_bit_identical_to_the_two_kernel_sequence(env, hq, hkv, rotary_dim, sections):
    ffi, kv, synth, lib, ref = env["ffi"], env["kv"], env["synth"], env["lib"], env["ref"]
    ctx = [37, 300, 1, 16]
    n_tok = sum(ctx)
    g = torch.Generator().manual_seed(11 + hq)
    qgd, kd = hq * 256 * 2, hkv * 256
    stride = qgd + 2 * kd                                  # packed [q|gate per head, k, v] rows (forward.rs:1088-1090)
    qkv = (torch.randn(n_tok, stride, generator=g) * 1.5).to(torch.float16)
    for h in range(hkv):                                   # outlier channels in K and V
        qkv[:, qgd + h * 256 + 7] *= 20
        qkv[:, qgd + kd + h * 256 + 100] *= 20
    k_norm_w = (torch.randn(256, generator=g) * 0.2).to(torch.float16)
    q_norm_w = (torch.randn(256, generator=g) * 0.2).to(torch.float16)
    # three position planes (text tokens carry the same value in all three; a few differ as for images)
    pos = torch.cat([torch.arange(c) for c in ctx]).to(torch.int32)
    planes = torch.stack([pos, pos + (pos % 5), pos + (pos % 3) * 2]).contiguous()
    vtm = np.ones(n_tok, np.uint8)
    vtm[40] = 0

    def pool():
        wl = synth.PagedWorkload([0] * len(ctx), ctx, hkv, seed=21, fill=0x3C)
        return wl, wl.step(valid_token_mask=vtm)

    dev = lambda t: t.cuda()  # noqa: E731
    qkv_d, kw_d, qw_d, planes_d = dev(qkv), dev(k_norm_w), dev(q_norm_w), dev(planes)
    k_in = qkv_d.data_ptr() + 2 * qgd
    v_in = qkv_d.data_ptr() + 2 * (qgd + kd)
    ex = env["ex"]
    # ---- the reference's two kernels --------------------------------------------------------------
    wl_r, b_r = pool()
    q_out = torch.zeros(n_tok, hq, 256, dtype=torch.float16, device="cuda")
    gate_out = torch.zeros_like(q_out)
    k_out = torch.zeros(n_tok, hkv, 256, dtype=torch.float16, device="cuda")
    f = ref.warp34_fused_qk_rmsnorm_rope_gate_strided_f16
    f.restype = C.c_int
    f.argtypes = [C.c_void_p] * 10 + [C.c_int] * 11 + [C.c_float, C.c_float]
    mask_d = torch.from_numpy(vtm).cuda()
    rc = f(C.addressof(ex.ex), qkv_d.data_ptr(), k_in, qw_d.data_ptr(), kw_d.data_ptr(), planes_d.data_ptr(),
           mask_d.data_ptr(), q_out.data_ptr(), k_out.data_ptr(), gate_out.data_ptr(), n_tok, n_tok, hq, hkv, 256,
           rotary_dim, sections[0], sections[1], sections[2], stride, stride, 1.0e6, 1e-6)
    assert rc == 0
    rc = env["ref_abi"].warp34_kv_cache_write_strided(C.byref(ex.ex), C.byref(wl_r.layer.layout), C.byref(b_r.desc),
                                                      k_out.data_ptr(), v_in, kd, stride)
    assert rc == 0
    # ---- one kernel -----------------------------------------------------------------------------------
    wl_f, b_f = pool()
    rc = lib.warp34_fused_k_rmsnorm_rope_kv_cache_write_f16(
        C.byref(ex.ex), C.byref(wl_f.layer.layout), C.byref(b_f.desc), k_in, v_in, kw_d.data_ptr(), planes_d.data_ptr(),
        n_tok, rotary_dim, sections[0], sections[1], sections[2], stride, stride, 1.0e6, 1e-6)
    assert rc == 0
    torch.cuda.synchronize()
    kr, kf = wl_r.layer.k.cpu().numpy(), wl_f.layer.k.cpu().numpy()
    vr, vf = wl_r.layer.v.cpu().numpy(), wl_f.layer.v.cpu().numpy()
    assert (vr == vf).all()
    assert (kr == kf).all(), f"{int((kr != kf).sum())} of {kr.size} K bytes differ"
    assert (kf != 0x3C).any()


def test_fused_producer_refuses_what_it_does_not_cover(env):
    ffi, synth, lib = env["ffi"], env["synth"], env["lib"]
    wl = synth.PagedWorkload([0], [4], 2, seed=3)
    b = wl.step()
    x = torch.zeros(4, 2048, dtype=torch.float16, device="cuda")
    w = torch.zeros(256, dtype=torch.float16, device="cuda")
    pos = torch.zeros(3, 4, dtype=torch.int32, device="cuda")
    args = (C.byref(env["ex"].ex), C.byref(wl.layer.layout), C.byref(b.desc), x.data_ptr(), x.data_ptr(), w.data_ptr(),
            pos.data_ptr(), 4)
    fn = lib.warp34_fused_k_rmsnorm_rope_kv_cache_write_f16
    assert fn(*args, 40, 7, 7, 6, 512, 512, 1e6, 1e-6) == ffi.CUDA_ERROR_NOT_SUPPORTED      # rotary_dim / 2 not a multiple of 8
    assert fn(*args[:5], None, *args[6:], 64, 11, 11, 10, 512, 512, 1e6, 1e-6) == ffi.CUDA_ERROR_INVALID_VALUE
    assert fn(*args, 64, 11, 11, 10, 100, 512, 1e6, 1e-6) == ffi.CUDA_ERROR_INVALID_VALUE     # K row stride too small
