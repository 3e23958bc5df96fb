"""Pools larger than 4 GiB per tensor: page offsets that do not fit 32 bits.

A serving process that gives most of a 180 GB device to the KV pool holds several GiB per layer and
side; page id x page stride then exceeds 2^32.  Each case runs the same sequences (same seeds, so the
same rows) once in a small pool and once in a pool whose shuffled free list spreads their pages over
more than 4 GiB, through every kernel family.  Page ids change nothing but addresses: appended rows and
attention outputs must be equal bit for bit."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

FOUR_GIB = 1 << 32
# name: (storage, contexts after the step, q_len, flag, heads)
CASES = {
    "tq4_decode": ("tq4", [700, 31, 2000], 1, None, (24, 4)),
    "tq4_decode_fast": ("tq4", [700, 31, 2000], 1, "EXEC_FLAG_FAST_ATTENTION", (24, 4)),
    "tq4_fp32": ("tq4", [300, 40], 1, "EXEC_FLAG_PRECISE_ATTENTION", (24, 4)),
    "tq4_verify": ("tq4", [300, 1000], 4, None, (24, 4)),
    "tq4_verify_team": ("tq4", [300, 1000], 4, "EXEC_FLAG_FAST_ATTENTION", (24, 4)),
    "tq4_chunk": ("tq4", [200, 400], 100, None, (16, 4)),
    "tq4_chunk_tcgen05": ("tq4", [200, 400], 100, "EXEC_FLAG_FAST_ATTENTION", (16, 4)),
    "fp8_decode": ("fp8", [700, 31], 1, None, (24, 4)),
    "q8_decode": ("q8", [700, 31], 1, None, (24, 4)),
    "bf16_decode": ("bf16", [700, 31], 1, None, (24, 4)),
}


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    free, _ = torch.cuda.mem_get_info()
    assert free > (24 << 30), "these cases hold about 10 GiB of pool"
    return dict(ffi=ffi, kv=kv, synth=synth, lib=native_libs[0])


def _formats(ffi, storage):
    if storage == "tq4":
        return None
    code = {"fp8": ffi.KV_FORMAT_FP8_E4M3, "q8": ffi.KV_FORMAT_Q8_0, "bf16": ffi.KV_FORMAT_BF16}[storage]
    return (code, code, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY)


def _page_bytes(wl):
    return wl.layer.k.numel() * wl.layer.k.element_size() // wl.num_pages


def _run(env, storage, ctx, q_len, flag, heads, slack_pages):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    hq, hkv = heads
    n = len(ctx)
    wl = synth.PagedWorkload([c - q_len for c in ctx], [q_len] * n, hkv, seed=61, slack_pages=slack_pages,
                             formats=_formats(ffi, storage))
    ex = kv.Executor(64 << 20)
    wl.fill_context(ex, 61)
    b = wl.step()
    k, v = synth.make_kv(n * q_len, hkv, 62, device="cuda")
    q = synth.make_q(n * q_len, hq, 63).cuda()
    ex.ex.flags = getattr(ffi, flag) if flag else 0
    if storage == "bf16":
        k, v, q = k.to(torch.bfloat16), v.to(torch.bfloat16), q.to(torch.bfloat16)
        out = torch.zeros(n * q_len, hq, 256, dtype=torch.bfloat16, device="cuda")
        kv.kv_cache_write_bf16(ex, wl.layer, b, k, v)
        kv.paged_attention_bf16kv(ex, wl.layer, b, q, out, hq)
    else:
        out = torch.zeros(n * q_len, hq, 256, dtype=torch.float16, device="cuda")
        kv.kv_cache_write(ex, wl.layer, b, k, v)
        kv.paged_attention(ex, wl.layer, b, q, out, hq)
    torch.cuda.synchronize()
    # the rows of every sequence, gathered page by page in sequence order
    pb = _page_bytes(wl)
    kpool = wl.layer.k.view(torch.uint8).view(wl.num_pages, pb)
    vpool = wl.layer.v.view(torch.uint8).view(wl.num_pages, pb)
    rows = []
    for s in wl.seqs:
        idx = torch.as_tensor(np.asarray(s.pages, np.int64), device="cuda")
        rows.append((kpool[idx].cpu(), vpool[idx].cpu()))
    top = max(int(p) for s in wl.seqs for p in s.pages)
    return out.view(torch.int16).cpu(), rows, (top + 1) * pb


@pytest.mark.parametrize("name", list(CASES))
def test_pages_beyond_4_gib_give_the_same_bits(env, name):
    storage, ctx, q_len, flag, heads = CASES[name]
    # pages per 4 GiB: 508 400 (TQ4, 8448 B), 254 200 (FP8), 246 723 (Q8_0), 131 072 (BF16)
    slack = {"tq4": 560000, "fp8": 290000, "q8": 280000, "bf16": 150000}[storage]
    small = _run(env, storage, ctx, q_len, flag, heads, 64)
    big = _run(env, storage, ctx, q_len, flag, heads, slack)
    assert big[2] > FOUR_GIB, "the large pool's sequences do not reach beyond 4 GiB"
    assert small[0].numpy().any()
    assert torch.equal(small[0], big[0]), "attention output depends on the page addresses"
    # Only the rows' own bytes are compared: the tail of a sequence's last page is whatever the pool held.
    for (ks, vs), (kb, vb), c in zip(small[1], big[1], ctx):
        full = c // 16
        assert torch.equal(ks[:full], kb[:full]) and torch.equal(vs[:full], vb[:full])


def test_query_sparse_lists_over_pages_beyond_4_gib(env):
    """Physical group ids (page * 4 + group) up to 2.2 million; same lists by logical group in both pools."""
    kv, synth, lib = env["kv"], env["synth"], env["lib"]
    outs = []
    tops = []
    for slack in (64, 560000):
        ctx = [1200, 333]
        wl = synth.PagedWorkload([0, 0], ctx, 4, seed=71, slack_pages=slack)
        ex = kv.Executor(64 << 20)
        k, v = synth.make_kv(sum(ctx), 4, 71)
        kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
        rng = np.random.default_rng(4)
        T, select_k = 4, 40
        phys = np.full((T, select_k), -1, np.int32)
        logical = np.zeros((T, select_k), np.int32)
        pos = np.zeros(T, np.int32)
        for t in range(T):
            s = t % 2
            pos[t] = ctx[s] - 1 - t
            pick = rng.permutation((ctx[s] + 3) // 4)[:select_k]
            logical[t, :len(pick)] = pick
            phys[t, :len(pick)] = np.asarray(wl.seqs[s].pages)[pick // 4] * 4 + pick % 4
        tops.append((int(phys.max()) // 4 + 1) * _page_bytes(wl))
        dev = [torch.from_numpy(a).cuda() for a in (phys, logical, np.full(T, select_k, np.int32), pos)]
        q = synth.make_q(T, 24, 72).cuda()
        for scratch in (ex, kv.Executor(0)):                  # stream kernel, then the kernel without a workspace
            out = torch.zeros(T, 24, 256, dtype=torch.float16, device="cuda")
            rc = lib.warp34_qsa_sparse_paged_attn_f16(
                C.addressof(scratch.ex), q.data_ptr(), None, C.addressof(wl.layer.layout), dev[0].data_ptr(),
                dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), None, out.data_ptr(), T, 24, select_k, 0.0625)
            assert rc == 0
            torch.cuda.synchronize()
            outs.append(out.view(torch.int16).cpu())
    assert tops[1] > FOUR_GIB
    assert outs[0].numpy().any()
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
