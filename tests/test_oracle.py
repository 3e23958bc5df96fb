"""The CPU oracle (oracle/tq4_oracle.c) against (a) its own algebraic properties and (b) the
golden fixture produced by the reference's kernels (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from util import GOLDEN, canonical_layout, f16, host_batch, tq4_rows_equal_up_to_scale_ulp, within_tol


def test_half_conversions_match_numpy(oracle_lib):
    L = oracle_lib.lib()
    bits = np.arange(0, 65536, dtype=np.uint32).astype(np.uint16)
    vals = bits.view(np.float16).astype(np.float32)
    for i in range(0, 65536, 97):
        f = L.w34o_half_to_float(int(bits[i]))
        assert (np.isnan(f) and np.isnan(vals[i])) or f == vals[i]
    rng = np.random.RandomState(0)
    xs = np.concatenate([rng.randn(2000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 300.0, 7e4)])
    xs = np.concatenate([xs, np.float32([0.0, -0.0, 65504.0, 65520.0, 6e-8, 2.98e-8, 3.0e-8])])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([L.w34o_float_to_half(float(x)) for x in xs], np.uint16)
    assert (got == want).all()


def test_wht_is_an_orthonormal_involution(oracle_lib):
    L = oracle_lib.lib()
    x = np.random.RandomState(1).randn(256).astype(np.float32)
    y = x.copy()
    L.w34o_wht256(y.ctypes.data)
    assert abs(np.dot(y, y) - np.dot(x, x)) < 1e-3 * np.dot(x, x)
    z = y.copy()
    L.w34o_wht256(z.ctypes.data)
    assert np.abs(z - x).max() < 1e-5
    e = np.zeros(256, np.float32)
    e[0] = 1.0
    L.w34o_wht256(e.ctypes.data)
    assert (e == 0.0625).all()


def test_encode_layout_and_edge_rows(oracle_lib):
    zero = np.zeros(256, np.float16).view(np.uint16)
    row, amb, rot = oracle_lib.encode_row(zero)
    assert (row[[0, 1, 66, 67]] == 0).all()           # +0 scales (0 + (-0) = +0)
    assert (row[2:66] == 0x77).all() and (row[68:] == 0x77).all()  # 0 > b_i for i < 7 -> code 7
    x = np.random.RandomState(2).randn(256).astype(np.float16)
    row, amb, rot = oracle_lib.encode_row(x.view(np.uint16))
    dec = oracle_lib.decode_row(row)
    assert np.corrcoef(rot, dec)[0, 1] > 0.99
    # low nibble = even rotated coordinate
    L = oracle_lib.lib()
    d0 = float(row[:2].copy().view(np.float16)[0])
    assert dec[0] == np.float32(d0) * np.float32(L.w34o_centroid(int(row[2]) & 15))
    assert dec[1] == np.float32(d0) * np.float32(L.w34o_centroid(int(row[2]) >> 4))
    # scaling the input by a power of two scales d and leaves the codes alone
    row2, _, _ = oracle_lib.encode_row((x * np.float16(4)).view(np.uint16))
    assert (row2[2:66] == row[2:66]).all() and (row2[68:] == row[68:]).all()
    assert float(row2[:2].copy().view(np.float16)[0]) == 4 * d0


needs_golden = pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden fixture not generated yet")


@needs_golden
def test_oracle_append_matches_reference_kernels(oracle_lib):
    fx = np.load(GOLDEN)
    hkv = int(fx["hkv"])
    lay = canonical_layout(hkv)
    k_pool = np.full_like(fx["k_pool"], 0x5A)
    v_pool = np.full_like(fx["v_pool"], 0x5A)
    lay.k_base, lay.v_base = k_pool.ctypes.data, v_pool.ctypes.data
    b, keep = host_batch(fx["app_qsl"], fx["app_ctx"], fx["app_seq"], fx["app_bt"], fx["app_slots"])
    k_in, v_in = np.ascontiguousarray(fx["k_in"]), np.ascontiguousarray(fx["v_in"])
    assert oracle_lib.kv_cache_write(lay, b, k_in, v_in, hkv * 256, hkv * 256, nthreads=2) == 0
    # untouched slots keep the fill pattern in both
    for got, want in ((k_pool, fx["k_pool"]), (v_pool, fx["v_pool"])):
        code_mism, scale_mism, ulp = tq4_rows_equal_up_to_scale_ulp(got, want)
        assert code_mism == 0
        assert ulp <= 1 and scale_mism <= 1 + got.size // 66 // 500


@needs_golden
@pytest.mark.parametrize("tag", ["dec", "ver"])
def test_oracle_attention_matches_reference_scalar_kernel(oracle_lib, tag):
    fx = np.load(GOLDEN)
    hq, hkv = int(fx["hq"]), int(fx["hkv"])
    lay = canonical_layout(hkv)
    k_pool, v_pool = np.ascontiguousarray(fx["k_pool"]), np.ascontiguousarray(fx["v_pool"])
    lay.k_base, lay.v_base = k_pool.ctypes.data, v_pool.ctypes.data
    b, keep = host_batch(fx[f"{tag}_query_start_loc"], fx[f"{tag}_context_lens_before"],
                         fx[f"{tag}_seq_lens_after"], fx[f"{tag}_block_tables"])
    q = np.ascontiguousarray(fx[f"q_{tag}"])
    out = np.zeros_like(fx[f"out_{tag}"])
    assert oracle_lib.paged_attention(lay, b, q, out, hq, nthreads=2) == 0
    want = f16(fx[f"out_{tag}"])
    got = f16(out)
    # same algorithm, fp32 on both sides: far tighter than the path's tolerance
    assert np.abs(got - want).max() <= 1e-3 + 2e-3 * np.abs(want).max()
    assert within_tol(got, want).all()


def test_oracle_masks_and_windows(oracle_lib):
    """Causal bound, sliding window and the non-causal window mode
    (op_kv_cache.cu:405-422) on a hand-checkable case: V rows are one-hot in the rotated
    domain is not expressible, so compare against a direct numpy softmax over dequantised rows."""
    rng = np.random.RandomState(5)
    hkv, hq, T = 1, 2, 40
    lay = canonical_layout(hkv)
    k_pool = np.zeros(4 * 2112, np.uint8)
    v_pool = np.zeros(4 * 2112, np.uint8)
    lay.k_base, lay.v_base = k_pool.ctypes.data, v_pool.ctypes.data
    kin = rng.randn(T, 256).astype(np.float16)
    vin = rng.randn(T, 256).astype(np.float16)
    pages = [2, 0, 3]
    slots = [pages[t // 16] * 16 + t % 16 for t in range(T)]
    b, keep = host_batch([0, T], [0], [T], [pages], slots)
    assert oracle_lib.kv_cache_write(lay, b, kin.view(np.uint16), vin.view(np.uint16), 256, 256) == 0
    L = oracle_lib.lib()
    sign = np.array([L.w34o_sign(i) for i in range(256)], np.float32)

    def unrot(x):
        y = np.ascontiguousarray(x, np.float32).copy()
        L.w34o_wht256(y.ctypes.data)
        return y * sign

    kd = np.stack([unrot(oracle_lib.decode_row(k_pool[slots[t] * 132:slots[t] * 132 + 132])) for t in range(T)])
    vd = np.stack([unrot(oracle_lib.decode_row(v_pool[slots[t] * 132:slots[t] * 132 + 132])) for t in range(T)])
    q = rng.randn(3, hq, 256).astype(np.float16)
    for mode, window in ((0, 0), (0, 7), (1, 9), (1, 0)):
        bq, keep2 = host_batch([0, 3], [T - 3], [T], [pages], None, mask_mode=mode, window=window)
        out = np.zeros((3, hq, 256), np.uint16)
        assert oracle_lib.paged_attention(lay, bq, q.view(np.uint16), out, hq) == 0
        for t in range(3):
            pos = T - 3 + t
            hi = T - 1 if mode == 1 else pos
            lo = max(0, pos - window + 1) if window > 0 else 0
            for h in range(hq):
                s = kd[lo:hi + 1] @ q[t, h].astype(np.float32) * 0.0625
                p = np.exp(s - s.max())
                want = (p[:, None] * vd[lo:hi + 1]).sum(0) / p.sum()
                assert np.abs(f16(out[t, h]) - want).max() < 3e-3
