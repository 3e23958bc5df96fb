"""How far beyond the benchmark's value distribution the default (value + residual) kernels keep every
output inside 2e-3 + 1e-2 |b|, measured against float64 dequant-then-attend over the stored bytes
(oracle/tq4_oracle.c decodes the rows; the attention is numpy float64).

The benchmark's distribution is K, V ~ N(0, 1) with 4 outlier channels x20 and Q ~ N(0, 1).  The sweep
goes to K outliers x30, V outliers x60, 8 outlier channels, a query scale of 2 and a V pattern whose
outlier channels alternate in sign from key to key (so that large terms cancel in the output), over
contexts of 1 to 299 tokens, where a softmax has few keys and every rounding shows.  The fp32 kernel is
held to the same bound on the same cases (it sits below a tenth of it)."""
import itertools

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def env(native_libs, oracle_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    from oracle import qsa
    return dict(ffi=ffi, kv=kv, synth=synth, oracle=oracle_lib, h256=qsa._H256, signs=qsa.signs())


def _grid(x):
    x = x.to(torch.bfloat16).to(torch.float32)
    x = torch.where(x.abs() < 2.0 ** -14, torch.zeros_like(x), x)
    return x.to(torch.float16)


def _float64_attention(env, wl, ctx, q, hq, hkv):
    oracle, H, sg = env["oracle"], env["h256"], env["signs"]
    kp = wl.layer.k.cpu().numpy().reshape(wl.num_pages, hkv, 16, 132)
    vp = wl.layer.v.cpu().numpy().reshape(wl.num_pages, hkv, 16, 132)
    out = np.zeros((len(ctx), hq, 256))
    g = hq // hkv
    for i, (s, c) in enumerate(zip(wl.seqs, ctx)):
        pages = s.pages
        for h in range(hkv):
            kd = np.stack([oracle.decode_row(kp[pages[t // 16], h, t % 16]) for t in range(c)]).astype(np.float64)
            vd = np.stack([oracle.decode_row(vp[pages[t // 16], h, t % 16]) for t in range(c)]).astype(np.float64)
            for j in range(g):
                qq = H @ (sg * q[i, h * g + j].astype(np.float64)) * 0.0625
                sc = kd @ qq
                p = np.exp(sc - sc.max())
                out[i, h * g + j] = sg * (H @ ((p / p.sum()) @ vd))
    return out


@pytest.mark.parametrize("ctx", [[1, 2, 3, 5, 8, 13, 17, 31, 40], [100, 150, 299]])
def test_default_kernels_hold_the_bound_beyond_the_benchmark_distribution(env, ctx):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    hq, hkv, n = 24, 4, len(ctx)
    worst = {"default": 0.0, "fp32": 0.0}
    for sk, sv, nout, qs, cancel in itertools.product([20, 30], [20, 60], [4, 8], [1.0, 2.0], [False, True]):
        g = torch.Generator().manual_seed(7)
        T = sum(ctx)
        k = torch.randn(T, hkv, 256, generator=g)
        v = torch.randn(T, hkv, 256, generator=g)
        for h in range(hkv):
            idx = torch.randperm(256, generator=g)[:nout]
            k[:, h, idx] *= sk
            v[:, h, idx] *= sv
            if cancel:
                sign = (torch.arange(T) % 2 * 2 - 1).float()
                v[:, h, idx[:2]] = sv * 3.0 * sign[:, None] * (1 + 0.01 * torch.randn(T, 2, generator=g))
        k, v = _grid(k).reshape(T, -1).contiguous(), _grid(v).reshape(T, -1).contiguous()
        wl = synth.PagedWorkload([0] * n, ctx, hkv, seed=7)
        ex = kv.Executor(64 << 20)
        kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
        for s, c in zip(wl.seqs, ctx):
            s.commit(c - 1)
        b = wl.step(q_lens=[1] * n)
        q = _grid(torch.randn(n, hq, 256, generator=g) * qs)
        want = _float64_attention(env, wl, ctx, q.float().numpy(), hq, hkv)
        tol = ATOL + RTOL * np.abs(want)
        for name, flags in (("default", 0), ("fp32", ffi.EXEC_FLAG_PRECISE_ATTENTION)):
            ex.ex.flags = flags
            out = torch.zeros(n, hq, 256, dtype=torch.float16, device="cuda")
            kv.paged_attention(ex, wl.layer, b, q.cuda(), out, hq)
            torch.cuda.synchronize()
            r = float((np.abs(out.float().cpu().numpy() - want) / tol).max())
            worst[name] = max(worst[name], r)
            assert r <= 1.0, (name, sk, sv, nout, qs, cancel, r)
    print(f"[margin] contexts up to {ctx[-1]}: default kernels worst {worst['default']:.2f} x the bound, fp32 kernel {worst['fp32']:.2f}")
    assert worst["fp32"] < 0.2
