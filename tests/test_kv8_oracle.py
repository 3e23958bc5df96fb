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


def _edge_and_random_rows():
    rng = np.random.RandomState(9)
    x = (rng.randn(300, 256) * rng.uniform(1e-3, 40, size=(300, 1))).astype(np.float16)
    x[0] = 0
    x[1] = 6.1e-5
    x[2] = 60000.0
    x[3, ::2] = 0
    x[4] = 0
    x[4, 17] = 3.0
    x[5, :128] = 0
    x[6] = -1.0
    x[7] = np.float16(1.0) * np.where(np.arange(256) % 3 == 0, 448, 1)   # values on fp8 grid points after scaling
    return x


def test_the_c_restatement_and_the_numpy_one_write_the_same_bytes(oracle_lib):
    """Two independent restatements of the row definitions: the C one used by the attention oracle and
    the numpy / torch one.  Both divide exactly, so every byte must agree, fp8 rounding ties included."""
    x = _edge_and_random_rows()
    bits = x.view(np.uint16)
    for fmt in (kv8.Q8_0, kv8.FP8_E4M3):
        want = kv8.encode_rows(x.astype(np.float32), fmt)
        got = np.zeros_like(want)
        for r in range(len(x)):
            oracle_lib.lib().w34o_kv8_encode_row(bits[r].ctypes.data, fmt, got[r].ctypes.data)
        assert (got == want).all(), (fmt, np.argwhere(got != want)[:5])
        # decode: the C one rounds d * code to fp16 as the reference's readers do
        dec = np.zeros((len(x), 256), np.float32)
        for r in range(len(x)):
            oracle_lib.lib().w34o_kv8_decode_row(want[r].ctypes.data, fmt, dec[r].ctypes.data)
        ref = kv8.decode_rows(want, fmt)
        with np.errstate(over="ignore"):
            assert np.array_equal(dec, ref.astype(np.float16).astype(np.float32))


def test_every_e4m3_code_survives_a_round_trip_through_the_c_conversion(oracle_lib):
    """A row whose largest magnitude is 448 has scale 1, so encoding the value of a code must give the
    code back (NaN codes left out; -0 comes back as 0x80, which the comparison expects too)."""
    vals = kv8._E4M3_VALUES
    for start in (0, 128):
        codes = np.arange(start, start + 127, dtype=np.uint8)
        keep = ~np.isnan(vals[codes])
        row = np.zeros(256, np.float16)
        row[:127] = np.where(keep, vals[codes], 0).astype(np.float16)
        row[127] = 448.0     # pins the scale of the first half to 1
        out = np.zeros(264, np.uint8)
        oracle_lib.lib().w34o_kv8_encode_row(row.view(np.uint16).ctypes.data, kv8.FP8_E4M3, out.ctypes.data)
        assert out[256:260].copy().view(np.float32)[0] == 1.0
        want = np.where(keep, codes, 0)
        assert (out[:127] == want).all(), np.argwhere(out[:127] != want)[:5]


def test_c_oracle_attention_over_8bit_pages_matches_float64(oracle_lib):
    """The C oracle's paged attention over host slabs of 8-bit rows against the numpy float64
    dequant-then-attend, through real block tables (CPU only)."""
    import ctypes as C

    from warp34_b200 import ffi
    rng = np.random.RandomState(3)
    hq, hkv, pages_total = 4, 2, 12
    ctx = [37, 16]
    for fmt in (kv8.Q8_0, kv8.FP8_E4M3):
        rb = kv8.ROW_BYTES[fmt]
        kpool = np.zeros((pages_total, hkv, 16, rb), np.uint8)
        vpool = np.zeros_like(kpool)
        lay = ffi.KvLayerLayout()
        f = (C.c_int32 * 4)(fmt, fmt, 0, 0)
        kb, vb = C.c_uint64(), C.c_uint64()
        assert ffi.host().w34_kv_layout_init(C.byref(lay), 0, 0, 0, 0, hkv, 256, 16, f, pages_total, C.byref(kb), C.byref(vb)) == 0
        assert kb.value == kpool.nbytes
        lay.k_base, lay.v_base = kpool.ctypes.data, vpool.ctypes.data
        perm = rng.permutation(np.arange(1, pages_total))
        bt = np.zeros((2, 4), np.int32)
        bt[0, :3] = perm[:3]
        bt[1, :1] = perm[3:4]
        kf = (rng.randn(sum(ctx), hkv, 256) * 2).astype(np.float16)
        vf = (rng.randn(sum(ctx), hkv, 256) * 2).astype(np.float16)
        slots = np.concatenate([[bt[r, t // 16] * 16 + t % 16 for t in range(c)] for r, c in enumerate(ctx)]).astype(np.int32)
        qsl = np.array([0, ctx[0], sum(ctx)], np.int32)
        zeros, seq = np.zeros(2, np.int32), np.array(ctx, np.int32)
        b = ffi.AttentionBatch()
        b.query_start_loc, b.context_lens_before, b.seq_lens_after = qsl.ctypes.data, zeros.ctypes.data, seq.ctypes.data
        b.block_tables, b.write_slot_mapping = bt.ctypes.data, slots.ctypes.data
        b.num_reqs, b.total_tokens, b.max_blocks_per_req, b.max_q_len, b.max_seq_len = 2, sum(ctx), 4, max(ctx), max(ctx)
        b.sm_scale = 0.0625
        kflat, vflat = kf.reshape(sum(ctx), -1), vf.reshape(sum(ctx), -1)
        assert oracle_lib.lib().w34o_kv_cache_write_strided(C.byref(lay), C.byref(b), kflat.view(np.uint16).ctypes.data,
                                                      vflat.view(np.uint16).ctypes.data, hkv * 256, hkv * 256, 2) == 0
        # the pool now holds what the numpy restatement encodes
        want_rows = kv8.encode_rows(kf[:, 1].astype(np.float32), fmt)
        got_rows = np.stack([kpool[slots[t] // 16, 1, slots[t] % 16] for t in range(sum(ctx))])
        assert (got_rows == want_rows).all()
        # decode step: one query token per request attends its whole context
        qsl2 = np.array([0, 1, 2], np.int32)
        ctx_before = np.array([c - 1 for c in ctx], np.int32)
        b.query_start_loc, b.context_lens_before = qsl2.ctypes.data, ctx_before.ctypes.data
        b.total_tokens, b.max_q_len = 2, 1
        q = rng.randn(2, hq, 256).astype(np.float16)
        out = np.zeros((2, hq, 256), np.uint16)
        assert oracle_lib.lib().w34o_paged_attention_f16(C.byref(lay), C.byref(b), q.view(np.uint16).ctypes.data,
                                                   out.ctypes.data, hq, 2) == 0
        got = out.view(np.float16).astype(np.float64)
        start = 0
        for r, c in enumerate(ctx):
            for h in range(hkv):
                rows = [(bt[r, t // 16], t % 16) for t in range(c)]
                kd = kv8.decode_rows(np.stack([kpool[p, h, o] for p, o in rows]), fmt)
                vd = kv8.decode_rows(np.stack([vpool[p, h, o] for p, o in rows]), fmt)
                want = kv8.attention(kd, vd, q[r, 2 * h:2 * h + 2].astype(np.float32), 0.0625)
                assert np.all(np.abs(got[r, 2 * h:2 * h + 2] - want) <= 2e-3 + 1e-2 * np.abs(want))
            start += c
