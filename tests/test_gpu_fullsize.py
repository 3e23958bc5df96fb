"""GPU parity at the benchmark's full sizes, through the C ABI, against the reference's own scalar
dequant-then-attend kernel (warp34_paged_attention_scalar_f16, op_kv_cache.cu:1244, compiled
unmodified into oracle/_ref) run on the same pool bytes: every output of the default kernels must be
inside 2e-3 + 1e-2 |b|.  Without that library the fp32 kernel of this library stands in (it is held
to the same bound against the fixture and the CPU oracle in test_gpu_parity.py).

  config 0   4 sequences, contexts U[1024, 4096], 16 / 4 heads: append everything, one decode step
  config 1   64 sequences, contexts U[8192, 32768], 24 / 4 heads, one decode step
  config 3   128 sequences x 4 query tokens (causal among the drafts), contexts U[2048, 16384]
  config 4   one sequence of 262 144 tokens: single pass, and 8 page shards merged on one GPU
  config 2   one 2048-token chunk after 14 336 cached tokens, 16 / 4 heads
  beyond     one sequence of 1 048 576 tokens (four times config 4)
plus page-permutation invariance at config 1's size (0 ULP, the reference's own relational test,
crates/warp34-host/tests/backbone_and_collectives.rs:453-572)."""
import numpy as np
import pytest

from util import fast_parity, plain_parity

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import oracle
    from warp34_b200 import ffi, kv, sharding, synth
    p = oracle.ref_lib_path()
    ref = ffi.bind_kernel_abi(p) if p is not None else None
    return dict(ffi=ffi, kv=kv, synth=synth, sharding=sharding, ex=kv.Executor(128 << 20), ref=ref)


def _dequant_then_attend(env, wl, b, q, hq):
    """The reference's scalar kernel on this pool (or this library's fp32 kernel when the reference
    library did not travel)."""
    kv = env["kv"]
    out = torch.zeros(q.shape[0], hq, 256, dtype=torch.float16, device="cuda")
    kv.paged_attention(env["ex"], wl.layer, b, q, out, hq, lib=env["ref"], scalar=True)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


def _workload(env, name, seed_shift=0, ctx=None, q_len=None, hq=None):
    kv, synth = env["kv"], env["synth"]
    c_hq, hkv, batch, lo, hi, c_ql, seed = synth.CONFIGS[name]
    hq = hq or c_hq
    q_len = q_len or c_ql
    ctx = ctx if ctx is not None else [int(c) for c in synth.context_lengths(batch, lo, hi, seed)]
    wl = synth.PagedWorkload(ctx, [q_len] * len(ctx), hkv, seed=seed + seed_shift)
    wl.fill_context(env["ex"], seed, chunk_tokens=32768)
    b = wl.step()
    k, v = synth.make_kv(len(ctx) * q_len, hkv, seed + 17, device="cuda")
    kv.kv_cache_write(env["ex"], wl.layer, b, k, v)
    q = synth.make_q(len(ctx) * q_len, hq, seed + 17).cuda()
    return wl, b, q, hq


def _run(env, wl, b, q, hq, flags=0):
    kv = env["kv"]
    ex = env["ex"]
    ex.ex.flags = flags
    try:
        out = torch.zeros(q.shape[0], hq, 256, dtype=torch.float16, device="cuda")
        kv.paged_attention(ex, wl.layer, b, q, out, hq)
        torch.cuda.synchronize()
        assert int(ex.scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
    finally:
        ex.ex.flags = 0
    return out


@pytest.mark.parametrize("name", ["cfg0_single_layer", "cfg1_batched_decode", "cfg3_mtp_verify"])
def test_full_size_step_is_inside_the_plain_bound_on_every_output(env, name):
    wl, b, q, hq = _workload(env, name)
    want = _dequant_then_attend(env, wl, b, q, hq)
    assert np.isfinite(want).all() and np.abs(want).max() > 0.1
    got = _run(env, wl, b, q, hq).float().cpu().numpy()
    ok, msg = plain_parity(got, want)
    print(f"[margin] {name} default kernels: {msg}")
    assert ok, (name, msg)
    # the opt-in single-operand build stays within its own, wider bound on the same step
    fast = _run(env, wl, b, q, hq, flags=env["ffi"].EXEC_FLAG_FAST_ATTENTION).float().cpu().numpy()
    ok, msg = fast_parity(fast, want)
    assert ok, (name, "fast build", msg)


def test_full_size_decode_is_invariant_under_page_permutation(env):
    outs, pages = [], []
    for shift in (0, 12345):                 # same tokens, two different physical page placements
        wl, b, q, hq = _workload(env, "cfg1_batched_decode", seed_shift=shift)
        outs.append(_run(env, wl, b, q, hq))
        pages.append(list(wl.seqs[0].pages))
        del wl
    assert pages[0] != pages[1]
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_long_context_single_pass_and_eight_page_shards(env):
    kv, sharding = env["kv"], env["sharding"]
    wl, b, q, hq = _workload(env, "cfg4_long_context")
    n_tok = wl.ctx[0] + 1
    want = _dequant_then_attend(env, wl, b, q, hq)
    whole = _run(env, wl, b, q, hq).float().cpu().numpy()
    ok, msg = plain_parity(whole, want)
    print(f"[margin] cfg4 single pass: {msg}")
    assert ok, ("single pass", msg)
    pages = wl.seqs[0].pages
    world = 8
    triples = torch.zeros(world, hq, 258, dtype=torch.float32, device="cuda")
    for g in range(world):
        lo, hi = sharding.split_pages(n_tok, world, g)
        bt = np.zeros((1, len(pages)), np.int32)
        bt[0, :(hi - lo + 15) // 16] = pages[lo // 16:(hi + 15) // 16]
        # the last shard holds the query's own token, so every shard's keys are all visible
        sb = kv.StepBatch([0, 1], [hi - lo - 1], [hi - lo], bt, [-1], len(pages), 0.0625)
        kv.paged_attention_partial(env["ex"], wl.layer, sb, q, triples[g], hq)
    merged = torch.zeros(1, hq, 256, dtype=torch.float16, device="cuda")
    kv.merge_shards(env["ex"], triples, merged)
    torch.cuda.synchronize()
    ok, msg = plain_parity(merged.float().cpu().numpy(), want)
    print(f"[margin] cfg4 eight page shards: {msg}")
    assert ok, ("8 shards", msg)


def test_one_million_token_sequence(env):
    """Four times config 4: one sequence of 1 048 576 tokens (a 65 536-entry block table row, 262 144
    (page, kv head) units, 296 partials per row through the wide merge)."""
    wl, b, q, hq = _workload(env, "cfg4_long_context", ctx=[(1 << 20) - 1])
    assert wl.seqs[0].num_pages == 65536
    want = _dequant_then_attend(env, wl, b, q, hq)
    assert np.isfinite(want).all() and np.abs(want).max() > 0
    got = _run(env, wl, b, q, hq).float().cpu().numpy()
    ok, msg = plain_parity(got, want)
    print(f"[margin] one sequence of 1 048 576 tokens: {msg}")
    assert ok, msg
    fast = _run(env, wl, b, q, hq, flags=env["ffi"].EXEC_FLAG_FAST_ATTENTION).float().cpu().numpy()
    ok, msg = fast_parity(fast, want)
    assert ok, ("fast build", msg)


def test_prefill_chunk_after_14k_cached_tokens(env):
    kv, synth = env["kv"], env["synth"]
    hq, hkv, ctx_before, q_len, seed = 16, 4, 14336, 2048, 2
    wl = synth.PagedWorkload([ctx_before], [q_len], hkv, seed=seed)
    wl.fill_context(env["ex"], seed, chunk_tokens=32768)
    b = wl.step()
    k, v = synth.make_kv(q_len, hkv, seed + 17, device="cuda")
    kv.kv_cache_write(env["ex"], wl.layer, b, k, v)
    q = synth.make_q(q_len, hq, seed + 17).cuda()
    want = _dequant_then_attend(env, wl, b, q, hq)
    got = _run(env, wl, b, q, hq).float().cpu().numpy()
    ok, msg = plain_parity(got, want)
    print(f"[margin] 2048-token chunk after 14336 tokens: {msg}")
    assert ok, msg
    fast = _run(env, wl, b, q, hq, flags=env["ffi"].EXEC_FLAG_FAST_ATTENTION).float().cpu().numpy()
    ok, msg = fast_parity(fast, want)
    assert ok, ("tcgen05 build", msg)
