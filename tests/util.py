"""Helpers shared by the parity tests."""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "tq4_ref_sm100a.npz")

# Attention tolerance of this path: |a - b| <= 2e-3 + 1e-2 |b|, a and b as fp16 outputs
# compared in fp32 (the dequant-then-attend result is b).
ATOL, RTOL = 2e-3, 1e-2


def within_tol(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return np.abs(a - b) <= ATOL + RTOL * np.abs(b)


# The tensor-core kernel feeds fp16 operands (rotated Q, codebook values, softmax weights) to
# the MMAs, like the reference's production kernel (op_paged_attn.cu:357, :470, :47-50).  Rounding
# the rotated query to fp16 perturbs a score by about 2^-12 |q||k| sm_scale, i.e. a softmax weight
# by up to 1e-3 relative when K has x20 outlier channels, and that moves an output channel by
# eps * |V value|, not by eps * |average|: where an outlier channel of two dominant keys
# cancels, the output is near zero while the error scales with the V values that were averaged.
# No fp16-operand kernel, the reference's included, meets 2e-3 + 1e-2|b| on those few elements
# (the fixture test compares against the reference's production kernel).
# So for this kernel: the plain bound must hold for at least 99.95 % of the elements, and every
# element must be inside the bound widened by CHANNEL_TERM * (largest |V| of that request, kv
# head and channel).  The fp32 kernel (WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION,
# warp34_paged_attention_scalar_f16) meets the plain bound everywhere.
CHANNEL_TERM = 2e-3
MIN_FRACTION_WITHIN = 0.9995


def channel_scale(v_rows, req_token_ranges, q_lens, hq, hkv):
    """max |V| per (query token, q head, channel): v_rows is fp16/fp32 [T_kv, hkv*256] holding the
    requests' keys back to back, req_token_ranges[i] = (first, last+1) row range of request i."""
    v = np.abs(np.asarray(v_rows, np.float32)).reshape(len(v_rows), hkv, 256)
    out = []
    g = hq // hkv
    for (lo, hi), ql in zip(req_token_ranges, q_lens):
        m = v[lo:hi].max(axis=0) if hi > lo else np.zeros((hkv, 256), np.float32)  # [hkv, 256]
        per_head = np.repeat(m, g, axis=0)                                          # [hq, 256]
        out.extend([per_head] * ql)
    return np.stack(out)


def parity_stats(a, b):
    """(violations of the plain bound, max error / plain bound) of a against b."""
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    d = np.abs(a - b)
    tol = ATOL + RTOL * np.abs(b)
    return int((d > tol).sum()), float((d / tol).max())


def tensor_core_parity(a, b, v_scale):
    """Returns (ok, message) for the fp16-operand kernel against dequant-then-attend."""
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    d = np.abs(a - b)
    plain = d <= ATOL + RTOL * np.abs(b)
    capped = d <= ATOL + RTOL * np.abs(b) + CHANNEL_TERM * np.asarray(v_scale, np.float32)
    frac = plain.mean()
    msg = (f"{(~plain).sum()} of {plain.size} outside 2e-3 + 1e-2|b| (fraction inside {frac:.6f}), "
           f"{(~capped).sum()} outside the channel-scaled bound, max abs {d.max():.3e}")
    for idx in np.argwhere(~capped)[:4]:
        i = tuple(idx)
        msg += f"; at {tuple(int(x) for x in i)}: got {a[i]:.5f} want {b[i]:.5f} channel max {v_scale[i]:.3f}"
    return bool(capped.all() and frac >= MIN_FRACTION_WITHIN), msg


def f16(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def host_layout(layer_layout, k_pool, v_pool):
    """A copy of a layer descriptor whose bases point at host slabs (for the CPU oracle)."""
    from warp34_b200 import ffi
    lay = ffi.KvLayerLayout()
    C.memmove(C.byref(lay), C.byref(layer_layout), C.sizeof(lay))
    lay.k_base = k_pool.ctypes.data
    lay.v_base = v_pool.ctypes.data
    return lay


def canonical_layout(hkv, num_pages=0):
    from warp34_b200 import ffi
    lay = ffi.KvLayerLayout()
    f = (C.c_int32 * 4)(2, 2, 1, 1)
    rc = ffi.host().w34_kv_layout_init(C.byref(lay), 0, 0, 0, 0, hkv, 256, 16, f, num_pages, None, None)
    assert rc == 0
    return lay


def host_batch(qsl, ctx, seq, bt, slots=None, sm_scale=0.0625, mask_mode=0, window=0, vtm=None, vrm=None):
    """warp34_attention_batch over host numpy arrays; returns (desc, keepalive)."""
    from warp34_b200 import ffi
    arrs = dict(qsl=np.ascontiguousarray(qsl, np.int32), ctx=np.ascontiguousarray(ctx, np.int32),
                seq=np.ascontiguousarray(seq, np.int32), bt=np.ascontiguousarray(bt, np.int32),
                slots=None if slots is None else np.ascontiguousarray(slots, np.int32),
                vtm=None if vtm is None else np.ascontiguousarray(vtm, np.uint8),
                vrm=None if vrm is None else np.ascontiguousarray(vrm, np.uint8))
    b = ffi.AttentionBatch()
    b.query_start_loc = arrs["qsl"].ctypes.data
    b.context_lens_before = arrs["ctx"].ctypes.data
    b.seq_lens_after = arrs["seq"].ctypes.data
    b.block_tables = arrs["bt"].ctypes.data
    b.write_slot_mapping = None if arrs["slots"] is None else arrs["slots"].ctypes.data
    b.valid_token_mask = None if arrs["vtm"] is None else arrs["vtm"].ctypes.data
    b.valid_req_mask = None if arrs["vrm"] is None else arrs["vrm"].ctypes.data
    b.num_reqs = len(arrs["qsl"]) - 1
    b.total_tokens = int(arrs["qsl"][-1])
    b.max_blocks_per_req = arrs["bt"].shape[1] if arrs["bt"].ndim == 2 else len(arrs["bt"])
    q = np.diff(arrs["qsl"])
    b.max_q_len = int(q.max()) if len(q) else 0
    b.max_seq_len = int(arrs["seq"].max()) if len(arrs["seq"]) else 0
    b.mask_mode = mask_mode
    b.sliding_window = window
    b.sm_scale = sm_scale
    return b, arrs


def tq4_rows_equal_up_to_scale_ulp(a, b):
    """Compares two TQ4 slabs: packed codes must be identical; fp16 scales may differ by one
    unit in the last place (IEEE division on the CPU against the GPU's approximate division).
    Returns (code_byte_mismatches, scale_mismatches, max_scale_ulp)."""
    a = np.asarray(a, np.uint8).reshape(-1, 66)
    b = np.asarray(b, np.uint8).reshape(-1, 66)
    code_mism = int((a[:, 2:] != b[:, 2:]).sum())
    sa = a[:, :2].copy().view(np.uint16).astype(np.int32).ravel()
    sb = b[:, :2].copy().view(np.uint16).astype(np.int32).ravel()
    diff = np.abs(sa - sb)
    return code_mism, int((diff != 0).sum()), int(diff.max()) if diff.size else 0
