"""Where the decode kernel's time goes, warp by warp (a development aid, not a benchmark).

    python -m warp34_b200.stream_profile [cfg1_batched_decode] [cfg4_long_context] ...

Builds a second copy of the CUDA library with -DW34_STREAM_PROFILE (libwarp34_b200_sprof.so, next
to the product library), in which every warp of tq4_attention_stream_kernel writes %globaltimer
stamps at the ends of its phases to the scratch buffer at offset 48 MiB, runs one attention call
of the named workload geometry (page tables and lengths as in the benchmark; the pool holds a
constant byte pattern, which is enough for timing) and prints the phase durations over all warps.
"""
import sys

import numpy as np
import torch

from . import build, ffi, kv, synth

PROFILE_OFFSET = 48 << 20
WARPS = 148 * 12


def profile(cfg, lib):
    hq, hkv, batch, lo, hi, q_len, seed = synth.CONFIGS[cfg]
    ctx = synth.context_lengths(batch, lo, hi, seed)
    wl = synth.PagedWorkload([int(c) for c in ctx], [q_len] * batch, hkv, seed=seed, device="cuda",
                             slack_pages=64, fill=0x3C)
    for sq, c in zip(wl.seqs, ctx):
        sq.commit(int(c))
    ex = kv.Executor(64 << 20)
    b = wl.step()
    q = synth.make_q(batch * q_len, hq, 3).cuda()
    out = torch.zeros_like(q)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stamps = ex.scratch[PROFILE_OFFSET:PROFILE_OFFSET + WARPS * 64]
    for _ in range(6):
        stamps.zero_()
        e0.record()
        kv.paged_attention(ex, wl.layer, b, q, out, hq, lib=lib)
        e1.record()
    torch.cuda.synchronize()
    raw = stamps.cpu().numpy().view(np.int64).reshape(WARPS, 8)
    act = raw[:, 0] > 0
    r = raw[act].astype(np.float64)
    t0 = r[:, 0].min()
    print(f"{cfg}: attention call {e0.elapsed_time(e1):.4f} ms, {int(act.sum())} active warps, "
          f"{r[:, 7].mean():.2f} items per warp")

    def line(name, x):
        print(f"  {name:34s} mean {x.mean() / 1e3:8.2f} us  min {x.min() / 1e3:8.2f}  "
              f"p50 {np.median(x) / 1e3:8.2f}  max {x.max() / 1e3:8.2f}")

    line("table + barrier", r[:, 1] - r[:, 0])
    line("request look-up", r[:, 2] - r[:, 1])
    line("query fragments (first item)", r[:, 3] - r[:, 2])
    line("first page arrives", r[:, 4] - r[:, 3])
    line("page loop (all items)", r[:, 5] - r[:, 4])
    line("last partial written", r[:, 6] - r[:, 5])
    line("warp total", r[:, 6] - r[:, 0])
    print(f"  kernel span {(r[:, 6].max() - t0) / 1e3:.1f} us")
    items = raw[act][:, 7]
    total = r[:, 6] - r[:, 0]
    for k in sorted(set(items.tolist())):
        m = items == k
        print(f"  warps with {k} item(s): {int(m.sum())}, total mean {total[m].mean() / 1e3:.1f} us, "
              f"max {total[m].max() / 1e3:.1f}")


def main(argv):
    path = build.build_cuda(extra_defines=["-DW34_STREAM_PROFILE"], out_name="libwarp34_b200_sprof.so")
    lib = ffi.bind_kernel_abi(path)
    for cfg in argv or ["cfg1_batched_decode"]:
        profile(cfg, lib)


if __name__ == "__main__":
    main(sys.argv[1:])
