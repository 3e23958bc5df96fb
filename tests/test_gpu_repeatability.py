"""Run-to-run repeatability of every kernel family through the C ABI: the same step launched many
times, with the workspace overwritten by garbage between launches, returns the same bits every time.

The partials of the split-KV kernels are merged in slot order and the plan depends on the batch
geometry alone, so nothing in a result may depend on which warp finished first, on what an earlier
launch left in the workspace or in the staging rings, or on the output buffer's previous contents.  A
difference between two launches would mean a race (a staging slot reused before its last reader, a
partial read before it was written) that the parity tolerances could hide."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REPEATS = 12
# name: (context lengths after the step, query length, exec flag name, storage format, heads)
CASES = {
    "decode": ([3000, 17, 811, 4096, 260, 1], 1, None, "tq4", (24, 4)),
    "decode_fast": ([3000, 17, 811, 4096, 260, 1], 1, "EXEC_FLAG_FAST_ATTENTION", "tq4", (24, 4)),
    "decode_one_long_row": ([40000], 1, None, "tq4", (16, 4)),
    "verify": ([900, 2100, 64], 4, None, "tq4", (24, 4)),
    "verify_team": ([900, 2100, 64], 4, "EXEC_FLAG_FAST_ATTENTION", "tq4", (24, 4)),
    "chunk": ([700, 300], 150, None, "tq4", (16, 4)),
    "chunk_tcgen05": ([700, 300], 150, "EXEC_FLAG_FAST_ATTENTION", "tq4", (16, 4)),
    "fp32": ([500, 90], 1, "EXEC_FLAG_PRECISE_ATTENTION", "tq4", (24, 4)),
    "fp8": ([3000, 17, 811], 1, None, "fp8", (24, 4)),
    "q8": ([3000, 17, 811], 1, None, "q8", (24, 4)),
}


@pytest.fixture(scope="module")
def env(native_libs):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from warp34_b200 import ffi, kv, synth
    return dict(ffi=ffi, kv=kv, synth=synth, lib=native_libs[0])


def _formats(ffi, name):
    if name == "tq4":
        return None
    code = {"fp8": ffi.KV_FORMAT_FP8_E4M3, "q8": ffi.KV_FORMAT_Q8_0}[name]
    return (code, code, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY)


@pytest.mark.parametrize("name", list(CASES))
def test_attention_is_repeatable_over_a_garbage_workspace(env, name):
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    ctx, q_len, flag, fmt, (hq, hkv) = CASES[name]
    n = len(ctx)
    wl = synth.PagedWorkload([c - q_len for c in ctx], [q_len] * n, hkv, seed=31, formats=_formats(ffi, fmt))
    ex = kv.Executor(96 << 20)
    wl.fill_context(ex, 31)
    b = wl.step()
    k, v = synth.make_kv(n * q_len, hkv, 32, device="cuda")
    kv.kv_cache_write(ex, wl.layer, b, k, v)
    q = synth.make_q(n * q_len, hq, 33).cuda()
    ex.ex.flags = getattr(ffi, flag) if flag else 0
    gen = torch.Generator(device="cuda").manual_seed(5)
    first = None
    for it in range(REPEATS):
        # the workspace holds whatever the previous user left there: random bytes, NaN patterns included
        ex.scratch.view(torch.int32).random_(-2**31, 2**31 - 1, generator=gen)
        out = torch.empty(n * q_len, hq, 256, dtype=torch.int16, device="cuda")
        out.fill_(0x7e00 if it % 2 else 0x5500)
        kv.paged_attention(ex, wl.layer, b, q, out.view(torch.float16), hq)
        torch.cuda.synchronize()
        if flag != "EXEC_FLAG_PRECISE_ATTENTION":      # the fp32 kernel has no workspace and no status word
            assert int(ex.scratch[:4].cpu().numpy().view(np.int32)[0]) == 0, "kernel status"
        bits = out.cpu().numpy()
        if first is None:
            first = bits
            assert np.isfinite(bits.view(np.float16).astype(np.float32)).all()
            assert (bits != 0x5500).any()
        else:
            assert np.array_equal(first, bits), f"launch {it} differs from launch 0 in {(first != bits).sum()} values"
    ex.ex.flags = 0


def test_append_is_repeatable_and_touches_only_its_rows(env):
    """The same 3000-token append into two pools pre-filled with different bytes: the written rows are
    equal bit for bit and every other byte keeps its fill."""
    kv, synth = env["kv"], env["synth"]
    pools = []
    for fill in (0x00, 0xFF):
        wl = synth.PagedWorkload([0, 0, 0], [1500, 1, 1499], 4, seed=41, fill=fill)
        ex = kv.Executor(16 << 20)
        k, v = synth.make_kv(3000, 4, 42, device="cuda")
        for _ in range(3):
            kv.kv_cache_write(ex, wl.layer, wl.step(), k, v)
        torch.cuda.synchronize()
        pools.append((wl.layer.k.view(torch.uint8).cpu().numpy().ravel(), wl.layer.v.view(torch.uint8).cpu().numpy().ravel()))
    for a, b_ in zip(pools[0], pools[1]):
        written = ~((a == 0x00) & (b_ == 0xFF))
        assert np.array_equal(a[written], b_[written])
        assert written.sum() >= 3000 * 4 * 130            # 132-byte rows: at most two bytes of a row may equal both fills
        assert (a[~written] == 0x00).all() and (b_[~written] == 0xFF).all()


@pytest.mark.parametrize("fmt", ["tq4", "fp8"])
def test_query_sparse_lists_are_repeatable(env, fmt):
    import ctypes as C
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    ctx = [2000, 333]
    wl = synth.PagedWorkload([0, 0], ctx, 4, seed=51, formats=_formats(ffi, fmt))
    ex = kv.Executor(64 << 20)
    k, v = synth.make_kv(sum(ctx), 4, 51)
    kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
    rng = np.random.default_rng(3)
    T, select_k = 6, 48
    phys = np.full((T, select_k), -1, np.int32)
    logical = np.zeros((T, select_k), np.int32)
    pos = np.zeros(T, np.int32)
    for t in range(T):
        s = t % 2
        pos[t] = ctx[s] - 1 - t
        pick = rng.permutation((ctx[s] + 3) // 4)[:select_k]
        logical[t, :len(pick)] = pick
        phys[t, :len(pick)] = np.asarray(wl.seqs[s].pages)[pick // 4] * 4 + pick % 4
    dev = [torch.from_numpy(a).cuda() for a in (phys, logical, np.full(T, select_k, np.int32), pos)]
    q = synth.make_q(T, 24, 52).cuda()
    gen = torch.Generator(device="cuda").manual_seed(6)
    first = None
    for it in range(REPEATS):
        ex.scratch.view(torch.int32).random_(-2**31, 2**31 - 1, generator=gen)
        out = torch.empty(T, 24, 256, dtype=torch.int16, device="cuda")
        out.fill_(0x7e00)
        rc = env["lib"].warp34_qsa_sparse_paged_attn_f16(
            C.addressof(ex.ex), q.data_ptr(), None, C.addressof(wl.layer.layout), dev[0].data_ptr(), dev[1].data_ptr(),
            dev[2].data_ptr(), dev[3].data_ptr(), None, out.data_ptr(), T, 24, select_k, 0.0625)
        assert rc == 0
        torch.cuda.synchronize()
        bits = out.cpu().numpy()
        if first is None:
            first = bits
            assert np.isfinite(bits.view(np.float16).astype(np.float32)).all()
        else:
            assert np.array_equal(first, bits), f"launch {it} differs"


def test_two_host_threads_on_two_streams_with_their_own_workspaces(env):
    """The library keeps no mutable device state between calls besides the caller's workspace: two host
    threads, each with a stream, a workspace and a pool of its own, run append + attention steps at the
    same time (ctypes releases the interpreter lock inside the calls) and get the bits a lone thread gets."""
    import threading
    ffi, kv, synth = env["ffi"], env["kv"], env["synth"]
    hq, hkv = 24, 4
    jobs = [([3000, 17, 811, 4096], 1), ([900, 2100, 64], 4)]

    def run(job, stream, rounds, sink):
        ctx, q_len = job
        n = len(ctx)
        with torch.cuda.stream(stream):
            wl = synth.PagedWorkload([c - q_len for c in ctx], [q_len] * n, hkv, seed=81)
            ex = kv.Executor(96 << 20, stream=stream)
            wl.fill_context(ex, 81)
            b = wl.step()
            k, v = synth.make_kv(n * q_len, hkv, 82, device="cuda")
            q = synth.make_q(n * q_len, hq, 83).cuda()
            outs = []
            for _ in range(rounds):
                out = torch.zeros(n * q_len, hq, 256, dtype=torch.float16, device="cuda")
                kv.kv_cache_write(ex, wl.layer, b, k, v)
                kv.paged_attention(ex, wl.layer, b, q, out, hq)
                outs.append(out)
            stream.synchronize()
            assert int(ex.scratch[:4].cpu().numpy().view(np.int32)[0]) == 0
            sink.append([o.view(torch.int16).cpu() for o in outs])

    alone = []
    for job in jobs:
        run(job, torch.cuda.Stream(), 1, alone)
    together = [[], []]
    errors = []

    def guarded(i):
        try:
            run(jobs[i], torch.cuda.Stream(), 25, together[i])
        except Exception as e:  # surfaced in the main thread below
            errors.append(e)

    threads = [threading.Thread(target=guarded, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i in range(2):
        assert len(together[i][0]) == 25
        for o in together[i][0]:
            assert torch.equal(o, alone[i][0])
