#!/usr/bin/env python3
"""Generates tests/golden/tq4_ref_sm100a.npz from the REFERENCE's own kernels.

Needs a CUDA device and oracle/_ref/libwarp34_ref.so (the reference's op_kv_cache.cu /
op_paged_attn.cu compiled unmodified for sm_100a by oracle/build_ref.sh).  The fixture holds
seeded inputs and what the reference kernels produced for them:

  k_in, v_in           fp16 bits [T, Hkv*256]   inputs of the append (with edge rows)
  slots, block tables  step metadata of the append and of the two attention steps
  k_pool, v_pool       uint8 slabs written by warp34_kv_cache_write_strided   (bit-exact pin)
  q_dec, out_dec       decode step (1 token / request): reference scalar dequant-then-attend
  out_dec_prod         same step through the reference's production dispatcher (mma path)
  q_ver, out_ver       MTP-style verify step (4 tokens / request, causal), scalar path

Run:  python tests/golden/make_golden.py   (on a GPU box, from the repository root)
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from warp34_b200 import ffi, kv, synth  # noqa: E402

HQ, HKV = 8, 2
CTX = [70, 33, 129]   # requests the attention steps read: benchmark value distribution
EDGE = 24             # a fourth, append-only request that carries the edge rows
SEED = 20240


def edge_rows(k, v):
    """Rows the reference tests single out: all-zero rows, subnormal-ish and large magnitudes,
    a single spike, channel-0 / channel-128 outliers.  k, v are views of the edge request."""
    k[0] = 0
    v[1] = 0
    k[2] = 6.1e-5
    v[3] = 1000.0
    k[4] = 0
    k[4, 17] = 3.0
    v[5, 0] *= 50
    v[5, 128] *= 50
    k[6, :256] = -k[6, :256].abs()
    v[7, 256:] = 0
    k[8] = 60000.0      # scale overflows fp16: the stored scale is +inf in both implementations
    v[9] = -1.0
    k[10, ::2] = 0
    v[11] = v[11].abs() * 1e-3


def main(out_path):
    dev = "cuda"
    ref = ffi.bind_kernel_abi(oracle.ref_lib_path())
    T = sum(CTX) + EDGE
    k, v = synth.make_kv(T, HKV, SEED)
    edge_rows(k[sum(CTX):], v[sum(CTX):])
    wl = synth.PagedWorkload([0] * 4, CTX + [EDGE], HKV, seed=SEED, device=dev, slack_pages=3, fill=0x5A)
    ex = kv.Executor(16 << 20)
    app = wl.step()
    kv.kv_cache_write(ex, wl.layer, app, k.to(dev), v.to(dev), lib=ref)
    torch.cuda.synchronize()
    fx = dict(hq=HQ, hkv=HKV, ctx=np.array(CTX), num_pages=wl.num_pages,
              k_in=k.numpy().view(np.uint16), v_in=v.numpy().view(np.uint16),
              app_qsl=app.host["query_start_loc"], app_ctx=app.host["context_lens_before"],
              app_seq=app.host["seq_lens_after"], app_bt=app.host["block_tables"],
              app_slots=app.host["write_slot_mapping"],
              k_pool=wl.layer.k.cpu().numpy(), v_pool=wl.layer.v.cpu().numpy())

    def attend(q_lens, tag, seed):
        for s, c, ql in zip(wl.seqs, CTX, q_lens):
            s.set_committed(c - ql)
        b = kv.build_step(wl.seqs[:3], q_lens, wl.max_blocks, 1.0 / 16.0, device=dev)
        q = synth.make_q(sum(q_lens), HQ, seed)
        fx[f"q_{tag}"] = q.numpy().view(np.uint16)
        for nm in ("query_start_loc", "context_lens_before", "seq_lens_after", "block_tables"):
            fx[f"{tag}_{nm}"] = b.host[nm]
        for scalar, suffix in ((True, ""), (False, "_prod")):
            out = torch.zeros(sum(q_lens), HQ, 256, dtype=torch.float16, device=dev)
            kv.paged_attention(ex, wl.layer, b, q.to(dev), out, HQ, lib=ref, scalar=scalar)
            torch.cuda.synchronize()
            fx[f"out_{tag}{suffix}"] = out.cpu().numpy().view(np.uint16)

    attend([1, 1, 1], "dec", SEED + 1)
    attend([4, 4, 4], "ver", SEED + 2)
    np.savez_compressed(out_path, **fx)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "tq4_ref_sm100a.npz"))
