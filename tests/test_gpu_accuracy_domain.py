"""How far beyond the benchmark's value distribution the default (value + residual) kernels keep every
output inside 2e-3 + 1e-2 |b|, measured against float64 dequant-then-attend over the stored bytes
(oracle/tq4_oracle.c decodes the rows; the attention is numpy float64).

The benchmark's distribution is K, V ~ N(0, 1) with 4 outlier channels x20 and Q ~ N(0, 1).  The sweep
goes to K outliers x30, V outliers x60, 8 outlier channels, a query scale of 2 and a V pattern whose
outlier channels alternate in sign from key to key at three times the outlier scale (so that large terms
cancel in the output), over contexts of 1 to 300 tokens, where a softmax has few keys and every rounding
shows.  Asserted: inside the bound everywhere except the corner "x60 V outliers AND the alternating
pattern" (|v| = 180, nine times the benchmark's outliers), where outputs of about 0.05 are what +-180
terms leave over and a few per million of a prefill chunk reach the bound (measured 1.06x; held to 1.5x;
the same with the V-centroid pass or the residual of P x d_v taken on every page).  The fp32 kernel is held to the bound on all cases (it sits below a
tenth of it)."""
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


def _float64_attention(env, wl, ctx, q, hq, hkv, q_len=1):
    """ctx[i] tokens after the step, the last q_len of them the query tokens (causal among themselves)."""
    oracle, H, sg = env["oracle"], env["h256"], env["signs"]
    kp = wl.layer.k.cpu().numpy().reshape(wl.num_pages, hkv, 16, 132)
    vp = wl.layer.v.cpu().numpy().reshape(wl.num_pages, hkv, 16, 132)
    out = np.zeros((len(ctx) * q_len, hq, 256))
    g = hq // hkv
    for i, (s, c) in enumerate(zip(wl.seqs, ctx)):
        pages = s.pages
        for h in range(hkv):
            kd = np.stack([oracle.decode_row(kp[pages[t // 16], h, t % 16]) for t in range(c)]).astype(np.float64)
            vd = np.stack([oracle.decode_row(vp[pages[t // 16], h, t % 16]) for t in range(c)]).astype(np.float64)
            for t in range(q_len):
                vis = c - q_len + t + 1
                for j in range(g):
                    qq = H @ (sg * q[i * q_len + t, h * g + j].astype(np.float64)) * 0.0625
                    sc = kd[:vis] @ qq
                    p = np.exp(sc - sc.max())
                    out[i * q_len + t, h * g + j] = sg * (H @ ((p / p.sum()) @ vd[:vis]))
    return out


@pytest.mark.parametrize("ctx,q_len", [([1, 2, 3, 5, 8, 13, 17, 31, 40], 1), ([100, 150, 299], 1),
                                       ([64, 300], 4), ([90, 260], 70)])
def test_default_kernels_hold_the_bound_beyond_the_benchmark_distribution(env, ctx, q_len):
    """Decode (stream kernel), draft tokens (three 8-row items per kv head) and a prefill chunk (128-row kernel)."""
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    hq, hkv, n = 24, 4, len(ctx)
    worst = {"default": 0.0, "fp32": 0.0}
    by_v = {}
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
            s.commit(c - q_len)
        b = wl.step(q_lens=[q_len] * n)
        q = _grid(torch.randn(n * q_len, hq, 256, generator=g) * qs)
        want = _float64_attention(env, wl, ctx, q.float().numpy(), hq, hkv, q_len)
        tol = ATOL + RTOL * np.abs(want)
        for name, flags in (("default", 0), ("fp32", ffi.EXEC_FLAG_PRECISE_ATTENTION)):
            ex.ex.flags = flags
            out = torch.zeros(n * q_len, hq, 256, dtype=torch.float16, device="cuda")
            kv.paged_attention(ex, wl.layer, b, q.cuda(), out, hq)
            torch.cuda.synchronize()
            r = float((np.abs(out.float().cpu().numpy() - want) / tol).max())
            worst[name] = max(worst[name], r)
            if name == "default":
                by_v[(sv, cancel)] = max(by_v.get((sv, cancel), 0.0), r)
    print(f"[margin] contexts up to {ctx[-1]}, {q_len} query token(s): default kernels worst {worst['default']:.2f} x the bound, fp32 kernel {worst['fp32']:.2f}")
    print("[margin] by (V outlier scale, alternating pattern):", {k: round(x, 2) for k, x in sorted(by_v.items())})
    assert worst["fp32"] < 0.2
    for (sv, cancel), r in by_v.items():
        assert r <= (1.5 if (sv == 60 and cancel) else 1.0), (sv, cancel, r)
