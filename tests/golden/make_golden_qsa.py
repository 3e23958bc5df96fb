#!/usr/bin/env python3
"""Generates tests/golden/qsa_ref_sm100a.npz from the REFERENCE's own kernels.

Needs a CUDA device and oracle/_ref/libwarp34_ref.so (the reference's op_kv_cache.cu and op_qsa.cu
compiled unmodified for sm_100a by oracle/build_ref.sh).  For a TQ4 pool and an FP8 E4M3 pool, both
filled by the reference's append kernel, the fixture holds seeded queries, gates and selected-group lists
and what warp34_qsa_sparse_paged_attn_f16 / _hadamard_f16 of the reference produced for them:

  <fmt>_k_pool, <fmt>_v_pool   uint8 [pages, kv heads, 16, row bytes]
  q, gate                      fp16 bits [T, HQ, 256]
  sel_phys, sel_logical        int32 [T, SELECT_K]; num_selected, seq_pos int32 [T]; valid_token_mask uint8 [T]
  <fmt>_out_plain              no gate, no Hadamard     (fp16 bits [T, HQ, 256])
  <fmt>_out_gated              sigmoid gate
  <fmt>_out_hadamard           sigmoid gate + Hadamard-64

The lists carry the cases the reference's kernel distinguishes: a negative (skipped) entry, a group that
is entirely beyond the token's position, the token's own partly visible group, fewer entries than
SELECT_K, a token with no entry at all and a masked token.

Run:  python tests/golden/make_golden_qsa.py   (on a GPU box, from the repository root)
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from warp34_b200 import ffi, kv, synth  # noqa: E402

HQ, HKV, SELECT_K, SEED = 12, 2, 12, 4242
CTX = [61, 38]                 # two sequences; tokens 0-2 read the first, tokens 3-4 the second
TOK_SEQ = [0, 0, 0, 1, 1]
TOK_POS = [60, 37, 9, 37, 20]  # token_seq_pos


def build_lists(wl, rng):
    T = len(TOK_SEQ)
    phys = np.full((T, SELECT_K), -1, np.int32)
    logical = np.zeros((T, SELECT_K), np.int32)
    n_sel = np.zeros(T, np.int32)
    for t, (s, pos) in enumerate(zip(TOK_SEQ, TOK_POS)):
        pages = wl.seqs[s].pages
        groups = (CTX[s] + 3) // 4
        own = pos // 4
        pick = [own] + [int(g) for g in rng.permutation(groups) if g != own][:SELECT_K - 3]
        if own + 1 < groups:
            pick.append(own + 1)            # entirely beyond the token's position
        for i, g in enumerate(pick):
            logical[t, i] = g
            phys[t, i] = pages[g // 4] * 4 + (g % 4)
        n_sel[t] = len(pick)
    phys[0, 2] = -1                          # a skipped entry
    n_sel[2] = 0                             # a token without any entry
    n_sel[4] = 3                             # fewer entries than the list holds
    return phys, logical, n_sel


def main(out_path):
    ref = C.CDLL(oracle.ref_lib_path())
    refabi = ffi.bind_kernel_abi(oracle.ref_lib_path())
    rng = np.random.default_rng(SEED)
    T = len(TOK_SEQ)
    g = torch.Generator().manual_seed(SEED)
    q = torch.randn(T, HQ, 256, generator=g).to(torch.float16)
    gate = (torch.randn(T, HQ, 256, generator=g) * 2).to(torch.float16)
    vtm = np.ones(T, np.uint8)
    vtm[3] = 0
    fixture = dict(q=q.numpy().view(np.uint16), gate=gate.numpy().view(np.uint16), valid_token_mask=vtm,
                   seq_pos=np.asarray(TOK_POS, np.int32), ctx=np.asarray(CTX, np.int32),
                   tok_seq=np.asarray(TOK_SEQ, np.int32))
    lists = None
    for name, fmt, row in (("tq4", ffi.KV_FORMAT_TQ4, 132), ("fp8", ffi.KV_FORMAT_FP8_E4M3, 264)):
        tr = ffi.KV_TRANSFORM_RADEMACHER_WHT256 if fmt == ffi.KV_FORMAT_TQ4 else ffi.KV_TRANSFORM_IDENTITY
        wl = synth.PagedWorkload([0, 0], CTX, HKV, seed=SEED, slack_pages=1, fill=0x5A, formats=(fmt, fmt, tr, tr))
        ex = kv.Executor(8 << 20)
        k, v = synth.make_kv(sum(CTX), HKV, SEED)
        kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda(), lib=refabi)
        torch.cuda.synchronize()
        if lists is None:
            lists = build_lists(wl, rng)
            fixture.update(sel_phys=lists[0], sel_logical=lists[1], num_selected=lists[2])
            first_pages = [list(s.pages) for s in wl.seqs]
        assert [list(s.pages) for s in wl.seqs] == first_pages   # same seed, same page placement
        phys, logical, n_sel = (torch.from_numpy(a).cuda() for a in lists)
        pos, mask = torch.from_numpy(fixture["seq_pos"]).cuda(), torch.from_numpy(vtm).cuda()
        qd, gd = q.cuda(), gate.cuda()
        for label, fn, gptr in (("plain", ref.warp34_qsa_sparse_paged_attn_f16, None),
                                ("gated", ref.warp34_qsa_sparse_paged_attn_f16, gd.data_ptr()),
                                ("hadamard", ref.warp34_qsa_sparse_paged_attn_hadamard_f16, gd.data_ptr())):
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p] * 10 + [C.c_int, C.c_int, C.c_int, C.c_float]
            out = torch.full((T, HQ, 256), 0, dtype=torch.int16, device="cuda")
            out.fill_(0x5500)
            rc = fn(C.addressof(ex.ex), qd.data_ptr(), gptr, C.addressof(wl.layer.layout), phys.data_ptr(),
                    logical.data_ptr(), n_sel.data_ptr(), pos.data_ptr(), mask.data_ptr(), out.data_ptr(), T, HQ,
                    SELECT_K, 0.0625)
            assert rc == 0, rc
            torch.cuda.synchronize()
            fixture[f"{name}_out_{label}"] = out.cpu().numpy().view(np.uint16)
        fixture[f"{name}_k_pool"] = wl.layer.k.cpu().numpy().view(np.uint8).reshape(wl.num_pages, HKV, 16, row)
        fixture[f"{name}_v_pool"] = wl.layer.v.cpu().numpy().view(np.uint8).reshape(wl.num_pages, HKV, 16, row)
    np.savez_compressed(out_path, **fixture)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "qsa_ref_sm100a.npz"))
