"""CPU checks of the 8-bit row restatement (oracle/kv8.py): known answers worked out by hand from the
row definitions (crates/warp34-kernels/csrc/tq/tq4_kv_common.cuh:29-46, op_kv_cache.cu:32-151), size
and layout of the rows (cache.rs:161-162: 272 and 264 bytes at head_dim 256), and the error bound of a
round trip."""
import numpy as np

from oracle import kv8


def test_row_sizes_and_known_answers():
    x = np.zeros((3, 256), np.float32)
    x[0] = 1.0
    x[1, :64] = -2.0          # only the first Q8 block / first FP8 half is non-zero
    x[2, 200] = 0.5
    q8 = kv8.encode_rows(x, kv8.Q8_0)
    f8 = kv8.encode_rows(x, kv8.FP8_E4M3)
    assert q8.shape == (3, 272) and f8.shape == (3, 264)
    # all ones: d = 1/127, every code 127; fp8: d = 1/448, every code 0x7E (= 448)
    assert np.allclose(q8[0, 0:4].copy().view(np.float32), 1.0 / 127.0, rtol=1e-7)
    assert (q8[0, 4:68].view(np.int8) == 127).all() and (q8[0, 72:136].view(np.int8) == 127).all()
    assert (f8[0, :256] == 0x7E).all()
    assert np.allclose(f8[0, 256:264].copy().view(np.float32), 1.0 / 448.0, rtol=1e-7)
    # a block of -2 then zeros: first block codes -127, the other three blocks all zero with d = 0
    assert (q8[1, 4:68].view(np.int8) == -127).all()
    assert (q8[1, 68:] == 0).all()
    assert (f8[1, :64] == 0xFE).all() and (f8[1, 64:256] == 0).all()
    assert f8[1, 260:264].copy().view(np.float32)[0] == 0.0
    # a single spike lands in Q8 block 3 (columns 192..255) at offset 8, and in FP8 half 1
    assert q8[2, 68 * 3 + 4 + 8].view(np.int8) == 127 and int((kv8.codes(q8[2:3], kv8.Q8_0) != 0).sum()) == 1
    assert (q8[2, :68 * 3] == 0).all()
    assert f8[2, 200] == 0x7E and (np.delete(f8[2, :256], 200) == 0).all()
    for fmt, rows in ((kv8.Q8_0, q8), (kv8.FP8_E4M3, f8)):
        assert np.allclose(kv8.decode_rows(rows, fmt), x, rtol=1e-6, atol=0)


def test_round_trip_error_bounds():
    rng = np.random.RandomState(5)
    x = (rng.randn(200, 256) * rng.uniform(0.01, 30, size=(200, 1))).astype(np.float16).astype(np.float32)
    y = kv8.decode_rows(kv8.encode_rows(x, kv8.Q8_0), kv8.Q8_0)
    for sb in range(4):
        amax = np.abs(x[:, 64 * sb:64 * sb + 64]).max(axis=1, keepdims=True)
        assert np.all(np.abs(y - x)[:, 64 * sb:64 * sb + 64] <= amax / 127.0 * 0.5 * (1 + 1e-5))
    y = kv8.decode_rows(kv8.encode_rows(x, kv8.FP8_E4M3), kv8.FP8_E4M3)
    # e4m3 keeps 3 mantissa bits: relative error 2^-4 for normal codes, absolute 2^-10 d below them
    for h in range(2):
        sl = slice(128 * h, 128 * h + 128)
        d = np.abs(x[:, sl]).max(axis=1, keepdims=True) / 448.0
        assert np.all(np.abs(y - x)[:, sl] <= np.maximum(np.abs(x[:, sl]) * 2.0 ** -4, d * 2.0 ** -10) * (1 + 1e-5))
    assert kv8.code_steps_apart(kv8.encode_rows(x, kv8.Q8_0), kv8.encode_rows(x * (1 + 1e-7), kv8.Q8_0), kv8.Q8_0) <= 1
