"""CPU restatement (numpy / torch CPU) of the reference's unrotated 8-bit KV rows.  TEST INFRASTRUCTURE:
only tests may import it; the product never does.

Follows crates/warp34-kernels/csrc/ops/op_kv_cache.cu:32-151 (encode) and
crates/warp34-kernels/csrc/ops/op_paged_attn.cu:59-105 (decode), identity transform, head_dim 256:

  Q8_0      272 B = 4 x { float32 d; int8 qs[64] }; block sb = columns [64 sb, 64 sb + 64);
            d = max|x| / 127, q = clamp(round_half_away(x * (1 / d)), -127, 127); zeros when d <= 1e-12
  FP8_E4M3  264 B = { uint8 qs[256]; float32 d0; float32 d1 }; d_h = max|x| over half h * (1 / 448),
            qs = e4m3(x * (1 / d_h)), round to nearest even, saturating; zeros when d <= 1e-30

The reference is built with fast math (approximate reciprocal), this file divides exactly: a code may
differ by one step where x / d sits on a rounding boundary.  Parity of the bytes is therefore pinned
against the reference's own kernels (oracle/_ref) in the GPU tests, and this restatement is held to
"almost all bytes equal, none off by more than one step".  The attention function below is plain
float64 dequant-then-attend over stored bytes: parity unpinned against the reference's attention
output for these layers (its kernels did not return finite output on them where this was tried).
"""
import numpy as np
import torch

Q8_0, FP8_E4M3 = 3, 4
ROW_BYTES = {Q8_0: 272, FP8_E4M3: 264}

_E4M3_VALUES = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()


def encode_rows(x, fmt):
    """x: float32 [n, 256] (fp16-representable values).  Returns uint8 [n, ROW_BYTES[fmt]]."""
    x = np.ascontiguousarray(x, np.float32)
    n = x.shape[0]
    out = np.zeros((n, ROW_BYTES[fmt]), np.uint8)
    if fmt == Q8_0:
        for sb in range(4):
            blk = x[:, 64 * sb:64 * sb + 64]
            d = (np.abs(blk).max(axis=1) / np.float32(127.0)).astype(np.float32)
            inv = np.where(d > 1e-12, np.float32(1.0) / np.where(d > 0, d, 1), 0).astype(np.float32)
            t = blk * inv[:, None]
            q = np.clip(np.sign(t) * np.floor(np.abs(t) + np.float32(0.5)), -127, 127).astype(np.int8)
            out[:, 68 * sb:68 * sb + 4] = d.view(np.uint8).reshape(n, 4)
            out[:, 68 * sb + 4:68 * sb + 68] = q.view(np.uint8)
        return out
    for h in range(2):
        half = x[:, 128 * h:128 * h + 128]
        d = (np.abs(half).max(axis=1) * np.float32(1.0 / 448.0)).astype(np.float32)
        inv = np.where(d > 1e-30, np.float32(1.0) / np.where(d > 0, d, 1), 0).astype(np.float32)
        t = np.clip(half * inv[:, None], -448.0, 448.0).astype(np.float32)
        q = torch.from_numpy(t).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        out[:, 128 * h:128 * h + 128] = q
        out[:, 256 + 4 * h:260 + 4 * h] = d.view(np.uint8).reshape(n, 4)
    return out


def decode_rows(rows, fmt):
    """uint8 [n, ROW_BYTES[fmt]] -> float32 [n, 256]."""
    rows = np.ascontiguousarray(rows, np.uint8)
    n = rows.shape[0]
    out = np.zeros((n, 256), np.float32)
    if fmt == Q8_0:
        for sb in range(4):
            d = rows[:, 68 * sb:68 * sb + 4].copy().view(np.float32).reshape(n)
            q = rows[:, 68 * sb + 4:68 * sb + 68].copy().view(np.int8).astype(np.float32)
            out[:, 64 * sb:64 * sb + 64] = q * d[:, None]
        return out
    for h in range(2):
        d = rows[:, 256 + 4 * h:260 + 4 * h].copy().view(np.float32).reshape(n)
        out[:, 128 * h:128 * h + 128] = _E4M3_VALUES[rows[:, 128 * h:128 * h + 128]] * d[:, None]
    return out


def codes(rows, fmt):
    """The 256 codes of every row as signed integers that order like the values they stand for."""
    if fmt == Q8_0:
        return np.concatenate([rows[:, 68 * s + 4:68 * s + 68] for s in range(4)], axis=1).copy().view(np.int8).astype(np.int32)
    q = rows[:, :256].astype(np.int32)   # e4m3: sign bit 7, magnitude bits 0..6 order like |value|
    return np.where(q & 0x80, -(q & 0x7f), q & 0x7f)


def code_steps_apart(a, b, fmt):
    """Largest distance, in quantisation steps, between the codes of two row arrays."""
    return int(np.abs(codes(a, fmt) - codes(b, fmt)).max())


def attention(k_rows, v_rows, q, sm_scale):
    """Dequant-then-attend in float64 for ONE (request, kv head): k_rows / v_rows float32 [n_keys, 256]
    already decoded, q float32 [rows, 256] with per-row visible key counts given by the caller
    through slicing.  Returns float64 [rows, 256]."""
    s = (q.astype(np.float64) @ k_rows.astype(np.float64).T) * sm_scale
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    return p @ v_rows.astype(np.float64)
