"""The entry point that brings its own workspace (warp34_paged_attention_f16_static_scratch).

Hosts that cannot pass a scratch buffer and may not call an allocator -- an engine that has
handed all of its device memory to the KV pool, a plugin that only sees tensors and a stream --
call this variant; its split-KV workspace is an array inside the library.  The test drives it
through the C ABI twice in a row (the second call finds the first call's leftovers in the shared
array) and checks both results against the ordinary entry point.  This file sorts last on purpose:
a run that stops at the first failure has then already covered every other test."""
import ctypes as C

import numpy as np
import pytest

from util import ATOL, RTOL

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_the_ordinary_one_twice(native_libs):
    assert torch.cuda.is_available()
    from warp34_b200 import ffi, kv, synth
    lib = native_libs[0]
    hq, hkv = 24, 4
    ex = kv.Executor(64 << 20)
    stream = torch.cuda.current_stream().cuda_stream

    def case(ctx, q_len, seed):
        wl = synth.PagedWorkload([0] * len(ctx), ctx, hkv, seed=seed)
        k, v = synth.make_kv(sum(ctx), hkv, seed)
        kv.kv_cache_write(ex, wl.layer, wl.step(), k.cuda(), v.cuda())
        for s, c in zip(wl.seqs, ctx):
            s.commit(c - q_len)
        b = wl.step(q_lens=[q_len] * len(ctx))
        q = synth.make_q(q_len * len(ctx), hq, seed).cuda()
        want = torch.zeros_like(q)
        kv.paged_attention(ex, wl.layer, b, q, want, hq)
        return wl, b, q, want

    # different batches back to back, each over the previous one's leftovers: decode, verify, and a
    # prefill chunk (which takes the 128-row kernel and needs the status word only)
    for ctx, q_len, seed in (([900, 17, 2500, 64], 1, 5), ([300, 33], 4, 6), ([500, 140], 70, 7)):
        wl, b, q, want = case(ctx, q_len, seed)
        got = torch.full_like(q, 3.0)
        needed = C.c_size_t(0)
        rc = lib.warp34_paged_attention_f16_static_scratch(stream, C.byref(wl.layer.layout), C.byref(b.desc),
                                                           q.data_ptr(), got.data_ptr(), hq, C.byref(needed))
        assert rc == 0 and 0 < needed.value <= (16 << 20)
        assert (needed.value == 16) == (q_len == 70)
        torch.cuda.synchronize()
        a, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert (np.abs(a - w) <= ATOL + RTOL * np.abs(w)).all()
        status = C.c_int32(-1)
        assert lib.warp34_static_scratch_status(C.byref(status)) == 0 and status.value == 0

    # A decode batch beyond the built-in workspace is refused before anything is launched.  (Only the
    # sizes are inflated: had the call gone through, the kernels would have read past the two requests'
    # metadata, so the descriptor is a decode one, whose size the entry point checks.)
    big = ffi.AttentionBatch()
    C.memmove(C.byref(big), C.byref(b.desc), C.sizeof(big))
    big.total_tokens, big.num_reqs, big.max_q_len = 4096, 4096, 1
    sentinel = got.clone()
    needed = C.c_size_t(0)
    rc = lib.warp34_paged_attention_f16_static_scratch(stream, C.byref(wl.layer.layout), C.byref(big), q.data_ptr(),
                                                       got.data_ptr(), hq, C.byref(needed))
    torch.cuda.synchronize()
    assert rc == ffi.CUDA_ERROR_INVALID_VALUE and needed.value > (16 << 20)
    assert torch.equal(got, sentinel)
    # malformed arguments do not report a size
    needed = C.c_size_t(7)
    assert lib.warp34_paged_attention_f16_static_scratch(stream, None, None, None, None, hq, C.byref(needed)) == 1
    assert needed.value == 0
