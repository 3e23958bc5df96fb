#!/usr/bin/env python3
"""Benchmark of the TQ4 paged-KV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (config.workload): batched decode at the 27B-class full-attention layer shape --
24 Q heads, 4 KV heads, head_dim 256, 64 sequences with contexts uniform in [8192, 32768],
TQ4 pages of 16 tokens placed by a seeded shuffled free list.  A step appends one token per
sequence (quantize-and-append) and runs one decode attention pass.  Inputs are synthetic and
seeded; the KV read per step (about 1.34 GB) is far larger than L2.

Metric: compressed-KV GB/s = sum(ctx_len) * Hkv * 264 B per step / step time.  With N > 1
every rank runs its own 64-sequence batch (weak scaling, no data-path collective); the value
is all ranks' bytes over the slowest rank's time.  The K-step loop is timed five times; the
median is reported.  The line also carries the count of the step's outputs outside
2e-3 + 1e-2 |b| of dequant-then-attend (`parity`), the numbers of the opt-in single-operand
build (`fast_build`) and, in `sharded`, the strong-scaling cases: the same 64 sequences split by
KV head (and batch halves at 8 GPUs), and one 262 144-token sequence split by pages.

`--impl reference` runs the same steps through the reference's own kernels compiled for
sm_100a (oracle/_ref), or, when that library is absent, through the CPU oracle.
"""
import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "tq4_paged_decode_attention_kv_gbps"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def measured_traffic_ratio(kernel):
    """DRAM bytes per algorithmic byte of `kernel`, from the small JSON that sits beside its ncu
    summary (written when the capture is taken; carries the capture's date and workload).  None when
    there is no capture of the kernel as it is built now."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        rec = json.load(open(p)).get(kernel)
        return float(rec["dram_bytes"]) / float(rec["algorithmic_bytes"]), rec
    except Exception:
        return None, None


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


class ClockSampler(threading.Thread):
    """Polls NVML (read-only) for SM clock and clock-event reasons while the benchmark runs."""

    def __init__(self, index, period_s=0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples = []  # (t, sm_mhz, reasons_bitmask)
        self.stop_flag = False
        self.max_mhz = None
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def summary(self, t0, t1):
        names = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        scope = "timed_region"
        if not inside:
            inside, scope = self.samples, "whole_run"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "scope": "unavailable"}
        mask = 0
        for s in inside:
            mask |= s[2]
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in names.items() if mask & b], "samples": len(inside), "scope": scope}


def init_dist(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return rank, local, world


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x, world):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def cpu_baseline(wl, hq, q_host, k_new, v_new, step_host_desc, budget_s=20.0, q_len=1):
    """The CPU oracle (a restatement of the reference's algorithm; the reference has no CPU
    implementation of this path) on the host cores: the same step on a bounded sample of the
    batch.  Returns the cpu_baseline object."""
    import oracle
    from warp34_b200 import ffi
    cores = os.cpu_count() or 1
    hk, hv = wl.layer.k.cpu().numpy(), wl.layer.v.cpu().numpy()
    lay = ffi.KvLayerLayout()
    C.memmove(C.byref(lay), C.byref(wl.layer.layout), C.sizeof(lay))
    lay.k_base, lay.v_base = hk.ctypes.data, hv.ctypes.data
    nreq = step_host_desc.num_reqs
    # size the sample from a one-sequence probe
    def run(n):
        b = ffi.AttentionBatch()
        C.memmove(C.byref(b), C.byref(step_host_desc), C.sizeof(b))
        b.num_reqs, b.total_tokens = n, n * q_len
        out = np.zeros((n * q_len, hq, 256), np.uint16)
        t0 = time.perf_counter()
        oracle.kv_cache_write(lay, b, k_new, v_new, k_new.shape[1], v_new.shape[1], nthreads=cores)
        oracle.paged_attention(lay, b, q_host, out, hq, nthreads=cores)
        return time.perf_counter() - t0
    t1 = run(1)
    n = int(max(1, min(nreq, budget_s / max(t1, 1e-4))))
    dt = run(n)
    kv_bytes = sum(wl.ctx[i] + q_len for i in range(n)) * wl.num_kv_heads * 264
    return {"value": kv_bytes / dt / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"one full step (append + attention) over the first {n} of {nreq} sequences, {dt:.2f} s"}


def host_step_batch(kv, step, batch, n_tok):
    """The step's metadata as a host-side StepBatch (keeps the arrays alive for the oracle)."""
    io = step.io
    o = io._offs
    # arena order: query_start_loc | context_lens_before | seq_lens_after | write_slot_mapping | block_tables
    return kv.StepBatch(io._np[o[0]:o[0] + batch + 1], io._np[o[1]:o[1] + batch], io._np[o[2]:o[2] + batch],
                        io._np[o[4]:o[4] + batch * io.max_blocks].reshape(batch, -1), io._np[o[3]:o[3] + n_tok],
                        io.max_blocks, 1.0 / 16.0, device="cpu")


def strong_scaling_cases(args, world, rank, dev, headline):
    """The sharded configurations with the TOTAL work fixed (strong scaling), device-resident, one CUDA
    graph replay per step, timed like the headline (K steps, five times, median, max over ranks):

      cfg1_by_kv_head  the same 64 sequences of config 1 on every N: kv heads split over 1 / 2 / 4 GPUs
                       (4 / 2 / 1 local kv heads with their 6 q heads each, the reference's TP split,
                       forward.rs:1085-1086); at 8 GPUs one kv head and one half of the batch per GPU.
                       No collective.
      cfg4_by_pages    one sequence of 262 144 tokens, pages split in contiguous ranges; every GPU runs
                       partial attention over its range, the (m, l, acc) triples are exchanged and
                       merged by one kernel over peer-mapped mailboxes (NCCL all-gather + merge kernel
                       when no peer mapping is available).
    """
    from warp34_b200 import kv, sharding, synth
    import torch.distributed as dist
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    REPS = 5

    def timed_graph(body, ex):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ex.set_stream()
            body()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(g):
            ex.set_stream()
            body()
        ex.set_stream()
        for _ in range(3):
            g.replay()
        out = []
        for _ in range(REPS):
            barrier(world)
            e0.record()
            for _ in range(args.steps):
                g.replay()
            e1.record()
            barrier(world)
            out.append(max_over_ranks(e0.elapsed_time(e1), world) / args.steps)
        return float(np.median(out)), [float(min(out)), float(max(out))]

    res = {}
    # ---- config 1, strong: kv heads (and batch halves at 8 GPUs) --------------------------------
    hq, hkv, batch, lo, hi, q_len, seed = synth.CONFIGS["cfg1_batched_decode"]
    ctx_all = [int(c) for c in synth.context_lengths(batch, lo, hi, seed)]
    if world == 1:
        res["cfg1_by_kv_head"] = {"partition": "4 kv heads x 64 sequences on 1 GPU (the headline's workload)",
                                  "ms_per_step": headline["ms_per_step"], "value": headline["value"], "unit": UNIT,
                                  "kv_bytes_total": headline["kv_bytes"]}
    elif world in (2, 4, 8):
        (h0, h1), _, batch_split = sharding.split_kv_heads(hkv, hq, world, rank)
        b0, b1 = sharding.split_batch(batch, batch_split, rank % batch_split)
        ctx = ctx_all[b0:b1]
        lh = h1 - h0
        lq = lh * (hq // hkv)
        wl = synth.PagedWorkload(ctx, [q_len] * len(ctx), lh, seed=seed + 1000 * rank, device=dev)
        ex = kv.Executor(64 << 20, device=dev)
        wl.fill_context(ex, seed + 1000 * rank, chunk_tokens=32768)
        b = wl.step()
        k_new, v_new = synth.make_kv(len(ctx) * q_len, lh, seed + 17, device=dev)
        q = synth.make_q(len(ctx) * q_len, lq, seed + 17).to(dev)
        out = torch.zeros_like(q)

        def body():
            kv.kv_cache_write(ex, wl.layer, b, k_new, v_new)
            kv.paged_attention(ex, wl.layer, b, q, out, lq)

        ms, span = timed_graph(body, ex)
        total = sum_over_ranks(float(wl.algorithmic_kv_bytes()), world)
        status = int(max_over_ranks(float(int(ex.scratch[:4].cpu().numpy().view(np.int32)[0])), world))
        res["cfg1_by_kv_head"] = {"partition": f"{lh} kv head(s) x {len(ctx)} sequences per GPU, no collective",
                                  "ms_per_step": ms, "ms_per_step_min_max": span, "value": total / (ms * 1e-3) / 1e9,
                                  "unit": UNIT, "kv_bytes_total": total, "kernel_status": status}
        del wl, ex
    # ---- config 4, strong: pages of one sequence --------------------------------------------------
    hq, hkv, batch, lo, hi, q_len, seed = synth.CONFIGS["cfg4_long_context"]
    n_local = (hi // world) // 16 * 16
    wl = synth.PagedWorkload([n_local - q_len], [q_len], hkv, seed=seed + 1000 * rank, device=dev)
    ex = kv.Executor(64 << 20, device=dev)
    wl.fill_context(ex, seed + 1000 * rank, chunk_tokens=32768)
    b = wl.step()
    k_new, v_new = synth.make_kv(q_len, hkv, seed + 17, device=dev)
    q = synth.make_q(q_len, hq, seed + 17).to(dev)
    out = torch.zeros_like(q)
    rows = q_len * hq
    mode, px, equal = "single GPU", None, None
    if world > 1:
        triples = torch.zeros(rows, 258, dtype=torch.float32, device=dev)
        gathered = torch.zeros(world * rows, 258, dtype=torch.float32, device=dev)
        try:
            px = kv.PeerExchange.symmetric(dist.group.WORLD, rows, dev)
        except Exception as exc:
            sys.stderr.write(f"rank {rank}: peer mailboxes unavailable ({exc}); using the NCCL all-gather\n")
        have = torch.tensor([1 if px is not None else 0], device=dev)
        dist.all_reduce(have, op=dist.ReduceOp.MIN)
        if int(have.item()) == 0:
            px = None
        mode = ("peer-mapped mailboxes: exchange + merge in one kernel" if px is not None
                else "NCCL all-gather + merge kernel")

    def gather_merge():
        dist.all_gather_into_tensor(gathered, triples)
        kv.merge_shards(ex, gathered.view(world, -1, 258), out)

    def body4():
        kv.kv_cache_write(ex, wl.layer, b, k_new, v_new)
        if world == 1:
            kv.paged_attention(ex, wl.layer, b, q, out, hq)
            return
        kv.paged_attention_partial(ex, wl.layer, b, q, triples, hq)
        if px is not None:
            px.exchange_merge(ex, triples, out)
        else:
            gather_merge()

    if px is not None:     # once: the fused exchange must reproduce all-gather + merge bit for bit
        barrier(world)
        body4()
        fused = out.clone()
        gather_merge()
        torch.cuda.synchronize()
        equal = bool(torch.equal(fused.view(torch.int16), out.view(torch.int16)) and px.status() == 0)
    ms, span = timed_graph(body4, ex)
    total = sum_over_ranks(float(wl.algorithmic_kv_bytes()), world)
    res["cfg4_by_pages"] = {"partition": f"{n_local} tokens of one {n_local * world}-token sequence per GPU; {mode}",
                            "ms_per_step": ms, "ms_per_step_min_max": span, "value": total / (ms * 1e-3) / 1e9, "unit": UNIT,
                            "kv_bytes_total": total,
                            **({"exchange_equals_allgather_merge": equal, "exchange_status": px.status()} if px is not None else {})}
    return res


def run_chunked_prefill(args):
    """Config 2: 8 sequences x 16384 tokens prefilled in 2048-token chunks (quantize-and-append,
    then causal chunk attention over everything cached so far); the first 4096 tokens are one
    shared, reference-counted prefix that only the first sequence computes.  Sequences are split
    over the ranks (strong scaling), each rank keeps its own copy of the shared prefix."""
    import oracle  # noqa: F401  (reference arm only)
    from warp34_b200 import ffi, kv, sharding, synth
    reference = args.impl == "reference"
    ref_path = oracle.ref_lib_path() if reference else None
    if reference and ref_path is None:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference kernels not built (oracle/_ref missing)"}))
        return
    rank, local, world = init_dist(args.gpus)
    dev = f"cuda:{local}"
    lib = ffi.bind_kernel_abi(ref_path) if ref_path else ffi.kernels()
    hq, hkv, n_seq, seq_len, chunk, prefix = 16, 4, 8, 16384, 2048, args.prefix_tokens
    lo, hi = sharding.split_batch(n_seq, world, rank)
    my_seqs = max(hi - lo, 0)
    pages_needed = my_seqs * (seq_len // 16) + 64
    pool = kv.PagePool(pages_needed + 1)
    pool.shuffle_free_list(2 + rank)
    layer = kv.KvLayer(pages_needed + 1, hkv, device=dev)
    cache = kv.PrefixCache(pool)
    ex = kv.Executor(64 << 20, device=dev)
    kc1, vc1 = synth.make_kv(chunk, hkv, 2, device=dev)
    qc1 = synth.make_q(chunk, hq, 2, device=dev)
    reps = max(my_seqs, 1)
    kc, vc, qc = kc1.repeat(reps, 1), vc1.repeat(reps, 1), qc1.repeat(reps, 1, 1)   # the same chunk for every sequence
    out = torch.zeros(reps * chunk, hq, 256, dtype=torch.float16, device=dev)
    max_blocks = seq_len // 16
    tokens = list(range(seq_len))           # every sequence has the same first `prefix` tokens

    def run_job(timed):
        """The scheduler's order: the first sequence prefills the shared prefix alone; the others
        attach to it; from then on every step carries one 2048-token chunk of every sequence."""
        flops, n_tok = 0.0, 0
        evs = []

        cow_copies = 0

        def step(seqs, start, chunk=chunk):
            nonlocal flops, n_tok, cow_copies
            n = len(seqs)
            for s in seqs:
                assert s.reserve(start + chunk) >= 0
                cow = s.prepare_append()     # a shared, partly filled tail page is copied before the first write
                if cow is not None:
                    kv.kv_page_copy(ex, layer, *cow)
                    cow_copies += 1
            b = kv.build_step(seqs, [chunk] * n, max_blocks, 1.0 / 16.0, device=dev)
            if timed:
                e = tuple(torch.cuda.Event(enable_timing=True) for _ in range(3))
                e[0].record()
            kv.kv_cache_write(ex, layer, b, kc[:n * chunk], vc[:n * chunk], lib=lib)
            if timed:
                e[1].record()
            kv.paged_attention(ex, layer, b, qc[:n * chunk], out[:n * chunk], hq, lib=lib)
            if timed:
                e[2].record()
                evs.append(e)
            for s in seqs:
                s.commit(chunk)
            # causal: token t of a chunk sees start + t + 1 keys
            flops += n * 4.0 * hq * 256 * (chunk * start + chunk * (chunk + 1) / 2)
            n_tok += n * chunk

        pool_seqs = [kv.Sequence(pool) for _ in range(my_seqs)]
        if my_seqs > 0:
            # the first sequence prefills the shared prefix (its last piece may be shorter than a chunk)
            for start in range(0, prefix, chunk):
                step(pool_seqs[:1], start, min(chunk, prefix - start))
            whole = prefix // 16 * 16            # the radix cache works in whole pages
            cache.insert(tokens[:whole], pool_seqs[0].pages[:whole // 16])
            for s in pool_seqs[1:]:
                pages, matched, node = cache.match_prefix(tokens[:whole])
                assert matched == whole
                if prefix > whole:               # share the partly filled tail page as well: copy-on-write later
                    pages = pages + [pool_seqs[0].pages[whole // 16]]
                s.attach_prefix(pages, prefix)
            for start in range(prefix, seq_len, chunk):
                step(pool_seqs, start, min(chunk, seq_len - start))
        torch.cuda.synchronize()
        for s in pool_seqs:
            s.close()
        freed = cache.evict(10 ** 9)
        return flops, n_tok, evs, len(freed), cow_copies

    run_job(False)                            # warm-up pass over the whole job
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.start()
    t_begin = time.perf_counter()
    e0.record()
    flops, n_tok, evs, shared_pages, cow_copies = run_job(True)
    e1.record()
    barrier(world)
    t_end = time.perf_counter()
    sampler.stop_flag = True
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    attn_ms = sum(b.elapsed_time(c) for a, b, c in evs)
    app_ms = sum(a.elapsed_time(b) for a, b, c in evs)
    tot_flops = sum_over_ranks(flops, world)
    tot_tok = sum_over_ranks(float(n_tok), world)
    fast_build = None
    if not reference:
        # the same job with the opt-in single-operand build: chunks take the tcgen05 + TMEM kernel
        ex.ex.flags = ffi.EXEC_FLAG_FAST_ATTENTION
        run_job(False)
        barrier(world)
        e0.record()
        f_flops, _, f_evs, _, _ = run_job(True)
        e1.record()
        barrier(world)
        ex.ex.flags = 0
        f_ms = max_over_ranks(e0.elapsed_time(e1), world)
        f_attn_ms = sum(b.elapsed_time(c) for a, b, c in f_evs)
        fast_build = {"flag": "WARP34_B200_EXEC_FLAG_FAST_ATTENTION", "kernel": "tq4_attention_prefill_tc_kernel (tcgen05, 128-row CTAs)",
                      "ms_per_step": f_ms, "value": tot_flops / (f_ms * 1e-3) / 1e12,
                      "attention_tflops_rank0": f_flops / (f_attn_ms * 1e-3) / 1e12 if f_attn_ms > 0 else None}
    if rank != 0:
        return
    peaks, kind = measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    achieved = flops / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else 0.0
    line = {"metric": "tq4_chunked_prefill_attention_tflops", "value": tot_flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": 1, "warmup": 1, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "cfg2_chunked_prefill: 8 seqs x 16384 tokens, 2048-token chunks, first 4096 tokens a "
                                   "shared refcounted prefix computed once, then one chunk of every sequence per call; "
                                   "16 q heads / 4 kv heads, d256; a step is the whole job",
                       "l2": "each chunk re-reads its sequence's cached KV (up to 17 MB): L2-resident by design of the workload",
                       "parallelism": f"sequences split over {world} rank(s), no collective", "shared_prefix_pages": shared_pages,
                       "shared_prefix_tokens": prefix, "copy_on_write_tail_pages": cow_copies},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_kind": f"of {kind} (sustained bf16)",
                         "kernel": "tq4_attention_prefill_exact_kernel (register MMAs, value + residual operands, 128-row CTAs)", "traffic": None,
                         "attention_ms_rank0": attn_ms},
            "append_tokens_per_s": n_tok / (app_ms * 1e-3) if app_ms > 0 else None,
            "prefill_tokens_per_s": tot_tok / (ms * 1e-3), "gpu_launches": 2 * len(evs),
            "clocks": sampler.summary(t_begin, t_end)}
    if fast_build is not None:
        fast_build["roofline_frac"] = (fast_build["attention_tflops_rank0"] or 0.0) / peak
        line["fast_build"] = fast_build
    if reference:
        line["impl"] = "reference"
        line["roofline"]["kernel"] = "reference paged_attention_prefill_mma_f16_kernel<64>"
    print(json.dumps(line))


def run_fused_steps(args):
    """`--config fused_steps`: what the two fusions around the path save, on one GPU.
    (1) K producer in front of the append: per-head RMS norm + interleaved 3-D mRoPE + TQ4 append of
    `--append-tokens` tokens in one kernel, against the append alone on already normalised K (the difference
    is the whole cost of the fused producer; a separate producer kernel writes and re-reads 2 x 2048 B per
    token on top) and, when the reference's kernels were built, against its norm/RoPE kernel + its append.
    (2) Output gate (+ Hadamard-64) behind the attention: config 1's decode step through the gated entry
    point, against the plain entry point followed by the stand-alone gate kernel."""
    import ctypes as C
    import oracle
    from warp34_b200 import ffi, kv, synth
    lib = ffi.kernels()
    ref_path = oracle.ref_lib_path()
    ex = kv.Executor(64 << 20)
    ex.set_stream()
    hq, hkv = 24, 4
    n_tok = int(args.append_tokens)
    reps = max(5, min(args.steps, 50))

    def timed(fn, flush=None):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for a, b in evs:
            if flush is not None:
                flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return float(np.median([a.elapsed_time(b) for a, b in evs]))

    # ---- (1) producer + append ------------------------------------------------------------------------
    g = torch.Generator().manual_seed(5)
    qgd, kd = hq * 256 * 2, hkv * 256
    stride = qgd + 2 * kd
    qkv = (torch.randn(n_tok, stride, generator=g) * 1.5).to(torch.float16).cuda()
    k_norm_w = (torch.randn(256, generator=g) * 0.2).to(torch.float16).cuda()
    q_norm_w = (torch.randn(256, generator=g) * 0.2).to(torch.float16).cuda()
    pos = torch.arange(n_tok, dtype=torch.int32)
    planes = torch.stack([pos, pos, pos]).contiguous().cuda()
    wl = synth.PagedWorkload([0], [n_tok], hkv, seed=5)
    b = wl.step()
    k_in = qkv.data_ptr() + 2 * qgd
    v_in = qkv.data_ptr() + 2 * (qgd + kd)
    rot, sec = 64, (11, 11, 10)

    def fused():
        rc = lib.warp34_fused_k_rmsnorm_rope_kv_cache_write_f16(
            C.byref(ex.ex), C.byref(wl.layer.layout), C.byref(b.desc), k_in, v_in, k_norm_w.data_ptr(), planes.data_ptr(),
            n_tok, rot, sec[0], sec[1], sec[2], stride, stride, 1.0e6, 1e-6)
        assert rc == 0, rc

    def plain():
        rc = lib.warp34_kv_cache_write_strided(C.byref(ex.ex), C.byref(wl.layer.layout), C.byref(b.desc), k_in, v_in, stride, stride)
        assert rc == 0, rc

    producer = {"tokens": n_tok, "fused_norm_rope_append_ms": timed(fused), "append_alone_ms": timed(plain)}
    if ref_path is not None:
        ref = C.CDLL(ref_path)
        ref_abi = ffi.bind_kernel_abi(ref_path)
        if hasattr(ref, "warp34_fused_qk_rmsnorm_rope_gate_strided_f16"):
            f = ref.warp34_fused_qk_rmsnorm_rope_gate_strided_f16
            f.restype = C.c_int
            f.argtypes = [C.c_void_p] * 10 + [C.c_int] * 11 + [C.c_float, C.c_float]
            q_out = torch.zeros(n_tok, hq, 256, dtype=torch.float16, device="cuda")
            gate_out = torch.zeros_like(q_out)
            k_out = torch.zeros(n_tok, hkv, 256, dtype=torch.float16, device="cuda")

            def ref_norm():
                rc = f(C.addressof(ex.ex), qkv.data_ptr(), k_in, q_norm_w.data_ptr(), k_norm_w.data_ptr(), planes.data_ptr(), None,
                       q_out.data_ptr(), k_out.data_ptr(), gate_out.data_ptr(), n_tok, n_tok, hq, hkv, 256, rot, sec[0], sec[1],
                       sec[2], stride, stride, 1.0e6, 1e-6)
                assert rc == 0, rc

            def ref_append():
                rc = ref_abi.warp34_kv_cache_write_strided(C.byref(ex.ex), C.byref(wl.layer.layout), C.byref(b.desc),
                                                           k_out.data_ptr(), v_in, kd, stride)
                assert rc == 0, rc

            producer["reference_qk_norm_rope_gate_ms"] = timed(ref_norm)
            producer["reference_append_ms"] = timed(ref_append)
            producer["note"] = "the reference's norm kernel also produces Q and the gate (24 heads); its K half cannot be timed alone"
    del qkv, wl

    # ---- (2) attention + output gate ------------------------------------------------------------------
    _, _, batch, lo, hi, _, seed = synth.CONFIGS["cfg1_batched_decode"]
    if args.batch > 0:
        batch = args.batch
    ctx = [int(c) for c in synth.context_lengths(batch, lo, hi, seed)]
    wl = synth.PagedWorkload(ctx, [1] * batch, hkv, seed=seed)
    wl.fill_context(ex, seed, chunk_tokens=32768)
    b = wl.step()
    k1, v1 = synth.make_kv(batch, hkv, 99, device="cuda")
    kv.kv_cache_write(ex, wl.layer, b, k1, v1)
    q = synth.make_q(batch, hq, seed + 17).cuda()
    gate = (synth.make_q(batch, hq, seed + 18) * 2).cuda()
    out = torch.zeros_like(q)
    epilogue = {"workload": f"config 1 decode step, {batch} sequences", "tokens_in_cache": int(sum(ctx)) + batch}
    for name, had in (("gate", False), ("gate_hadamard64", True)):
        standalone = lib.warp34_apply_attn_output_gate_hadamard_f16 if had else lib.warp34_apply_attn_output_gate_f16

        def fused_call():
            kv.paged_attention_gated(ex, wl.layer, b, q, gate, out, hq, hadamard64=had)

        def two_calls():
            kv.paged_attention(ex, wl.layer, b, q, out, hq)
            rc = standalone(C.byref(ex.ex), out.data_ptr(), gate.data_ptr(), out.data_ptr(), None, batch, hq * 256)
            assert rc == 0, rc

        epilogue[name] = {"fused_ms": timed(fused_call), "attention_then_gate_kernel_ms": timed(two_calls)}
    epilogue["attention_alone_ms"] = timed(lambda: kv.paged_attention(ex, wl.layer, b, q, out, hq))
    print(json.dumps({"metric": "fused_steps_ms", "unit": "ms", "n_gpus": 1, "steps": reps, "warmup": 3, "higher_is_better": False,
                      "data": "synthetic", "dtype": "f16", "producer_append": producer, "attention_output_gate": epilogue}))


def run_qsa_sparse(args):
    """`--config qsa_sparse_decode`: query-sparse paged attention over TQ4 pages, one decode step of
    config 1's geometry: every token attends to 256 selected 4-token groups (1024 keys) of its sequence.
    `--impl reference` times the reference's own kernel (oracle/_ref) on the same lists."""
    import ctypes as C
    import oracle
    from warp34_b200 import ffi, kv, synth
    reference = args.impl == "reference"
    ref_path = oracle.ref_lib_path() if reference else None
    if reference and ref_path is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference kernels not built (oracle/_ref missing)"}))
        return
    lib = C.CDLL(ref_path) if reference else ffi.kernels()
    hq, hkv, batch, lo, hi, _, seed = synth.CONFIGS["cfg1_batched_decode"]
    if args.batch > 0:
        batch = args.batch
    select_k = 256
    ctx = [int(c) for c in synth.context_lengths(batch, lo, hi, seed)]
    wl = synth.PagedWorkload(ctx, [0] * batch, hkv, seed=seed)
    ex = kv.Executor(64 << 20)
    wl.fill_context(ex, seed, chunk_tokens=32768)
    rng = np.random.default_rng(seed)
    phys = np.full((batch, select_k), -1, np.int32)
    logical = np.zeros((batch, select_k), np.int32)
    for t, c in enumerate(ctx):
        pages = wl.seqs[t].pages
        own = (c - 1) // 4
        pick = np.concatenate([[own], rng.choice(own, select_k - 1, replace=False)])
        logical[t] = pick
        phys[t] = np.asarray(pages, np.int64)[pick // 4] * 4 + pick % 4
    dev = [torch.from_numpy(a).cuda() for a in (phys, logical, np.full(batch, select_k, np.int32),
                                                np.asarray(ctx, np.int32) - 1)]
    q = synth.make_q(batch, hq, seed + 17).cuda()
    gate = synth.make_q(batch, hq, seed + 18).cuda()
    out = torch.zeros_like(q)
    fn = lib.warp34_qsa_sparse_paged_attn_f16
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p] * 10 + [C.c_int, C.c_int, C.c_int, C.c_float]
    ex.set_stream()

    def one():
        rc = fn(C.addressof(ex.ex), q.data_ptr(), gate.data_ptr(), C.addressof(wl.layer.layout), dev[0].data_ptr(),
                dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), None, out.data_ptr(), batch, hq, select_k, 0.0625)
        assert rc == 0, rc

    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(args.warmup):
        one()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t_begin = time.perf_counter()
    for a, b in evs:
        flush.zero_()              # the selected rows of a step fit in L2: evict them between steps
        a.record()
        one()
        b.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    sampler.stop_flag = True
    ms = float(np.median([a.elapsed_time(b) for a, b in evs]))
    kv_bytes = batch * hkv * select_k * 4 * 264
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    achieved = kv_bytes / (ms * 1e-3) / 1e9
    line = {"metric": "qsa_sparse_attention_kv_gbps", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32" if reference else "f16", "data": "synthetic",
            "config": {"workload": f"qsa_sparse_decode: {batch} tokens x {select_k} selected 4-token groups of contexts "
                                   f"U[{lo},{hi}], {hq} q heads / {hkv} kv heads, d256, TQ4 pages, sigmoid gate",
                       "kv_bytes_per_step": kv_bytes, "l2": "a 256 MB buffer is written between timed steps"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "kernel": "tq4_attention_stream_kernel, query-sparse instantiation (+ plan and merge launches, timed together)", "launch_ms": ms,
                         "traffic": None},
            "gpu_launches": 3 * args.steps, "clocks": sampler.summary(t_begin, t_end)}
    if reference:
        line["impl"] = "reference"
        line["roofline"]["kernel"] = "reference qsa_sparse_paged_attn_gqa_f16_kernel (+ merge)"
        line["gpu_launches"] = None
    print(json.dumps(line))


def run_other_kv(args):
    """The same decode step over another storage format of the reference, device-resident, one GPU:
    `--kv bf16` uncompressed BF16 pages (1024 B per token and KV head instead of 264; the comparison
    arm), `--kv fp8` / `--kv q8` the unrotated 8-bit rows of the boundary layers (528 / 544 B).
    `--impl reference` runs the reference's own kernels when they were built: its bf16 kernels, and on
    the 8-bit layers its scalar dequant-then-attend entry point (its tensor-core dispatcher faulted on
    these layers here and is not run again)."""
    import oracle
    from warp34_b200 import ffi, kv, synth
    reference = args.impl == "reference"
    bf16 = args.kv == "bf16"
    ref_path = oracle.ref_lib_path() if reference else None
    if reference and ref_path is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference kernels not built (oracle/_ref missing)"}))
        return
    lib = ffi.bind_kernel_abi(ref_path) if ref_path else ffi.kernels()
    hq, hkv, batch, lo, hi, q_len, seed = synth.CONFIGS[args.config]
    if args.batch > 0:
        batch = args.batch
    ctx = synth.context_lengths(batch, lo, hi, seed)
    if bf16:
        formats, act = kv.BF16_KV_FORMATS, torch.bfloat16
        append, attend = kv.kv_cache_write_bf16, kv.paged_attention_bf16kv
        kernel, label = "bf16kv_attention_stream_kernel (+ plan and merge)", "uncompressed BF16 pages"
    else:
        fmt = ffi.KV_FORMAT_FP8_E4M3 if args.kv == "fp8" else ffi.KV_FORMAT_Q8_0
        formats, act = (fmt, fmt, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY), torch.float16
        append = kv.kv_cache_write
        attend = ((lambda *a, **k: kv.paged_attention(*a, scalar=True, **k)) if reference else kv.paged_attention)
        kernel = "kv8_attention_stream_kernel (+ plan and merge)"
        label = "unrotated FP8 E4M3 rows" if args.kv == "fp8" else "unrotated Q8_0 rows"
    wl = synth.PagedWorkload([int(c) for c in ctx], [q_len] * batch, hkv, seed=seed, formats=formats)
    ex = kv.Executor(64 << 20)
    wl.fill_context(ex, seed, chunk_tokens=32768)
    n_tok = batch * q_len
    k_new, v_new = (x.to(act).cuda() for x in synth.make_kv(n_tok, hkv, seed + 17))
    q = synth.make_q(n_tok, hq, seed + 17).to(act).cuda()
    out = torch.zeros_like(q)
    b = wl.step()
    ex.set_stream()

    def one(ev=None):
        append(ex, wl.layer, b, k_new, v_new, lib=lib)
        if ev is not None:
            ev[0].record()
        attend(ex, wl.layer, b, q, out, hq, lib=lib)
        if ev is not None:
            ev[1].record()

    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(args.warmup):
        one()
    torch.cuda.synchronize()
    evs = [tuple(torch.cuda.Event(enable_timing=True) for _ in range(2)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        one(evs[i])
    e1.record()
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    sampler.stop_flag = True
    ms = e0.elapsed_time(e1) / args.steps
    attn_ms = float(np.mean([a.elapsed_time(c) for a, c in evs]))
    kv_bytes = wl.algorithmic_kv_bytes()
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    achieved = kv_bytes / (attn_ms * 1e-3) / 1e9
    line = {"metric": f"{args.kv}_kv_decode_GBps", "value": kv_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if bf16 else "f32", "data": "synthetic",
            "config": {"workload": f"{args.config} over {label}: {batch} seqs x ctx U[{lo},{hi}], "
                                   f"{hq} q heads / {hkv} kv heads, d256, step = append {q_len} token/seq + decode attention",
                       "kv_bytes_per_step": kv_bytes, "l2": "KV read per step is larger than L2; no flush needed"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "kernel": kernel, "launch_ms": attn_ms, "traffic": None},
            "attended_tokens_per_s": float(sum(wl.ctx) + n_tok) / (attn_ms * 1e-3),
            "gpu_launches": 4 * args.steps, "clocks": sampler.summary(t_begin, t_end)}
    if reference:
        line["impl"] = "reference"
        line["roofline"]["kernel"] = ("reference paged_attention_gqa_bf16_kernel" if bf16 else
                                      "reference warp34_paged_attention_scalar_f16 (fp32 dequant-then-attend)")
        line["gpu_launches"] = None
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="page-sharded long context: all-gather over NCCL + merge, or one kernel over peer-mapped mailboxes")
    ap.add_argument("--config", default="cfg1_batched_decode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true", help="skip the strong-scaling cases of the `sharded` object")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the number of sequences of the configuration (a smaller case of the same "
                         "kernels for profiler captures; not a benchmark value)")
    ap.add_argument("--append-tokens", type=int, default=32768, help="tokens of the bulk-append measurement")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches only (no CUDA graph replay)")
    ap.add_argument("--prefix-tokens", type=int, default=4096,
                    help="cfg2: shared prefix length; 4100 leaves a partly filled shared tail page (copy-on-write)")
    ap.add_argument("--kv", default="tq4", choices=["tq4", "bf16", "fp8", "q8"],
                    help="bf16: the uncompressed-storage comparison arm of the same decode step; fp8 / q8: the "
                         "unrotated 8-bit rows of the boundary layers (one GPU each)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.config == "qsa_sparse_decode":
        return run_qsa_sparse(args)
    if args.config == "fused_steps":
        return run_fused_steps(args)
    if args.kv != "tq4":
        return run_other_kv(args)
    if args.config == "cfg2_chunked_prefill":
        return run_chunked_prefill(args)

    import oracle  # only for the reference arm and the cpu_baseline leg
    from warp34_b200 import ffi, kv, synth

    reference = args.impl == "reference"
    ref_path = oracle.ref_lib_path() if reference else None
    if reference and int(os.environ.get("RANK", "0")) != 0 and ref_path is None:
        return  # the CPU fallback of the reference arm runs on rank 0 only
    rank, local, world = init_dist(args.gpus)
    dev = f"cuda:{local}"
    lib = ffi.bind_kernel_abi(ref_path) if ref_path else ffi.kernels()

    hq, hkv, batch, lo, hi, q_len, seed = synth.CONFIGS[args.config]
    if args.batch > 0:
        batch = args.batch
    sharded = args.config == "cfg4_long_context" and world > 1 and not reference
    if sharded:
        # one sequence, pages split across ranks: rank r holds tokens [r L / N, (r + 1) L / N)
        lo = hi = (hi // world) // 16 * 16
    ctx = synth.context_lengths(batch, lo, hi, seed + 1000 * rank)
    if sharded:
        ctx = ctx - q_len  # every shard plays "context + the query token" so all its keys are visible
    speculative = q_len > 1      # MTP verify: the end-to-end loop commits accepted tokens and rolls back the rest
    grow_pages = 56 if speculative else 0   # 200 steps x at most 4 tokens
    wl = synth.PagedWorkload([int(c) for c in ctx], [q_len] * batch, hkv, seed=seed + 1000 * rank, device=dev,
                             slack_pages=64 + batch * grow_pages)
    step = kv.DecodeStep(wl.layer, wl.seqs, hq, max_q_len=q_len, scratch_bytes=64 << 20, device=dev,
                         extra_blocks=grow_pages)
    triples = gathered = peer_px = None
    exchange_ok = True
    if sharded:
        import torch.distributed as dist
        triples = torch.zeros(batch * q_len * hq, 258, dtype=torch.float32, device=dev)
        gathered = torch.zeros(world * batch * q_len * hq, 258, dtype=torch.float32, device=dev)  # rank-major
        if args.exchange == "peer":
            # mailboxes in symmetric memory: the exchange and the merge are one kernel over NVLink
            try:
                peer_px = kv.PeerExchange.symmetric(dist.group.WORLD, batch * q_len * hq, dev)
            except Exception as exc:  # no peer mapping on this box: every rank falls back together
                sys.stderr.write(f"rank {rank}: peer mailboxes unavailable ({exc}); using the NCCL all-gather\n")
            have = torch.tensor([1 if peer_px is not None else 0], device=dev)
            dist.all_reduce(have, op=dist.ReduceOp.MIN)
            if int(have.item()) == 0:
                peer_px = None
    wl.fill_context(step.ex, seed + 1000 * rank, chunk_tokens=32768, lib=lib)  # untimed: KV pool resident in HBM
    n_tok = batch * q_len
    k_new, v_new = synth.make_kv(n_tok, hkv, seed + 17)
    q_new = synth.make_q(n_tok, hq, seed + 17)
    step.k_host.copy_(k_new)
    step.v_host.copy_(v_new)
    step.q_host.copy_(q_new)
    q_lens = [q_len] * batch
    kv_bytes = wl.algorithmic_kv_bytes()

    if reference and ref_path is None:
        # CPU arm: the oracle port on the host cores, each step a bounded sample.
        step.run(q_lens)
        hb = host_step_batch(kv, step, batch, n_tok)
        cb = cpu_baseline(wl, hq, q_new.numpy().view(np.uint16), k_new.numpy().view(np.uint16),
                          v_new.numpy().view(np.uint16), hb.host_desc(), budget_s=8.0, q_len=q_len)
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": args.config}, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    # ---- device-resident timing: inputs already in HBM -------------------------------------
    step.io.pack(wl.seqs, q_lens, 1.0 / 16.0)
    step.io.upload()
    step.k_dev.copy_(step.k_host)
    step.v_dev.copy_(step.v_host)
    step.q_dev.copy_(step.q_host)
    torch.cuda.synchronize()
    desc = kv._DescOnly(step.io.desc)
    step.ex.set_stream()

    def attend(desc_):
        if sharded:
            kv.paged_attention_partial(step.ex, wl.layer, desc_, step.q_dev, triples, hq)
            if peer_px is not None:
                peer_px.exchange_merge(step.ex, triples, step.out_dev)
            else:
                dist.all_gather_into_tensor(gathered, triples)
                kv.merge_shards(step.ex, gathered.view(world, -1, 258), step.out_dev)
        else:
            kv.paged_attention(step.ex, wl.layer, desc_, step.q_dev, step.out_dev, hq, lib=lib)

    def device_step(ev=None):
        if ev is not None:
            ev[0].record()
        kv.kv_cache_write(step.ex, wl.layer, desc, step.k_dev, step.v_dev, lib=lib)
        if ev is not None:
            ev[1].record()
        attend(desc)
        if ev is not None:
            ev[2].record()

    if peer_px is not None:
        # one step each way: the fused exchange must reproduce the all-gather + merge bit for bit
        barrier(world)
        device_step()
        fused = step.out_dev.clone()
        saved, peer_px = peer_px, None
        attend(desc)
        peer_px = saved
        torch.cuda.synchronize()
        if not torch.equal(fused.view(torch.int16), step.out_dev.view(torch.int16)) or peer_px.status() != 0:
            exchange_ok = False   # reported in the JSON line; the run goes on so that every rank leaves in step
            sys.stderr.write(f"rank {rank}: fused exchange differs from all-gather + merge (status {peer_px.status()})\n")
    REPS = 5     # the K-step loop is timed this many times; the median is reported, the extremes kept beside it

    def timed_reps(fn):
        out = []
        for _ in range(REPS):
            barrier(world)
            e0.record()
            for i in range(args.steps):
                fn(i)
            e1.record()
            barrier(world)
            out.append(max_over_ranks(e0.elapsed_time(e1), world) / args.steps)
        return out

    def capture(body):
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step.ex.set_stream()
            body()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(g):
            step.ex.set_stream()
            body()
        step.ex.set_stream()
        for _ in range(3):
            g.replay()
        return g

    sampler = ClockSampler(local)
    sampler.start()
    barrier(world)
    for _ in range(args.warmup):
        device_step()
    barrier(world)
    evs = [tuple(torch.cuda.Event(enable_timing=True) for _ in range(3)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    eager_reps = timed_reps(lambda i: device_step(evs[i]))     # the events keep the last repetition's stamps
    rep_ms = eager_reps
    eager_ms_per_step = float(np.median(eager_reps))
    # The same K steps replayed from one CUDA graph (how the reference's engine runs a decode step,
    # crates/warp34-host/src/model/graphs.rs:199-259): launch gaps between the four kernels go away.
    # The page-sharded case captures its exchange in the same graph.  Not for the reference arm.
    graph_used = False
    if not args.no_graph and not reference:
        try:
            g = capture(device_step)
            rep_ms = timed_reps(lambda i: g.replay())
            graph_used = True
        except Exception as exc:  # keep the eager numbers
            step.ex.set_stream()
            sys.stderr.write(f"CUDA graph replay unavailable: {exc}\n")
    ms_per_step = float(np.median(rep_ms))
    t_end = time.perf_counter()
    append_ms = float(np.mean([a.elapsed_time(b) for a, b, c in evs]))
    attn_ms = float(np.mean([b.elapsed_time(c) for a, b, c in evs]))
    clocks = sampler.summary(t_begin, t_end)
    all_bytes = sum_over_ranks(float(kv_bytes), world)
    value = all_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: host buffers in, host result out, every step ----------------------------
    use_graph = not args.no_graph and not sharded       # both arms: one graph replay per step
    if sharded:
        attend_e2e = attend
    else:
        attend_e2e = None                               # the plain attention call: eligible for the graph
    for _ in range(3):
        step.run(q_lens, lib=lib, attend=attend_e2e, graph=use_graph)
    barrier(world)
    e2e_steps = max(3, min(args.steps, 200))
    rollback = None
    h2d_before = step.h2d_bytes_total
    if speculative:
        # Each step: pages for 1 + 3 draft tokens, append + verify, then a seeded-random suffix of
        # 0..3 draft tokens is rejected: the accepted ones are committed, pages that only held
        # rejected tokens go back to the pool.  Sequences grow, so the bytes are summed per step.
        spec = kv.SpeculativeBatch(wl.seqs)
        rng = np.random.RandomState(seed + 99 + rank)
        freed_pages, e2e_bytes, accepted_total = 0, 0.0, 0
        cached_tokens = sum(s.committed_len for s in wl.seqs)     # kept up to date from the accepted counts
        e0.record()
        for _ in range(e2e_steps):
            spec.reserve_ahead(q_len)
            e2e_bytes += float(cached_tokens + batch * q_len) * hkv * 264
            step.run(q_lens, lib=lib, sync=True, attend=attend_e2e, graph=use_graph)
            accepted = q_len - rng.randint(0, q_len, size=batch)
            freed_pages += len(spec.commit_and_rollback(accepted))
            accepted_total += int(accepted.sum())
            cached_tokens += int(accepted.sum())
        e1.record()
        barrier(world)
        e2e_ms = max_over_ranks(e0.elapsed_time(e1), world) / e2e_steps
        e2e_value = sum_over_ranks(e2e_bytes / e2e_steps, world) / (e2e_ms * 1e-3) / 1e9
        rollback = {"accepted_tokens_per_step": accepted_total / e2e_steps, "pages_freed_per_step": freed_pages / e2e_steps}
    else:
        e0.record()
        for _ in range(e2e_steps):
            step.run(q_lens, lib=lib, sync=True, attend=attend_e2e, graph=use_graph)
        e1.record()
        barrier(world)
        e2e_ms = max_over_ranks(e0.elapsed_time(e1), world) / e2e_steps
        e2e_value = all_bytes / (e2e_ms * 1e-3) / 1e9
    sampler.stop_flag = True

    status = int(step.ex.scratch[:4].cpu().numpy().view(np.int32)[0]) if not reference else 0

    # ---- the step's own outputs against dequant-then-attend, and the opt-in fast build ------------
    parity = fast_build = None
    if not reference and not sharded:
        check_path = oracle.ref_lib_path()
        check_lib = ffi.bind_kernel_abi(check_path) if check_path else None
        want = torch.zeros_like(step.out_dev)
        kv.paged_attention(step.ex, wl.layer, desc, step.q_dev, want, hq, lib=check_lib, scalar=True)
        torch.cuda.synchronize()
        w = want.float()

        def outside(flags):
            step.ex.ex.flags = flags
            kv.paged_attention(step.ex, wl.layer, desc, step.q_dev, step.out_dev, hq)
            torch.cuda.synchronize()
            step.ex.ex.flags = 0
            d = (step.out_dev.float() - w).abs()
            tol = 2e-3 + 1e-2 * w.abs()
            return int((d > tol).sum().item()), float((d / tol).max().item())

        n_out, worst = outside(0)
        parity = {"against": ("the reference's scalar dequant-then-attend kernel (oracle/_ref) on the same pool" if check_path
                              else "this library's fp32 dequant-then-attend kernel on the same pool"),
                  "outputs": int(w.numel()), "outside_2e-3_plus_1e-2_rel": n_out, "worst_error_over_bound": worst}
        if not args.no_graph:
            n_fast, worst_fast = outside(ffi.EXEC_FLAG_FAST_ATTENTION)
            step.ex.ex.flags = ffi.EXEC_FLAG_FAST_ATTENTION
            try:
                gf = capture(device_step)
                fast_ms = float(np.median(timed_reps(lambda i: gf.replay())))
                ev_f = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ev_f[0].record()
                for _ in range(20):
                    attend(desc)
                ev_f[1].record()
                torch.cuda.synchronize()
                fast_attn_ms = ev_f[0].elapsed_time(ev_f[1]) / 20
                fast_build = {"flag": "WARP34_B200_EXEC_FLAG_FAST_ATTENTION", "ms_per_step": fast_ms,
                              "value": all_bytes / (fast_ms * 1e-3) / 1e9, "attention_ms": fast_attn_ms,
                              "roofline_frac": kv_bytes / (fast_attn_ms * 1e-3) / 1e9 / float(measured_peaks()[0].get("hbm_gbs", FALLBACK_HBM_GBS)),
                              "outside_2e-3_plus_1e-2_rel": n_fast, "worst_error_over_bound": worst_fast}
            finally:
                step.ex.ex.flags = 0
                step.ex.set_stream()

    # ---- bulk append (prefill-sized): the "appended tokens/s" half of the metric ----------------
    bulk_tokens = args.append_tokens
    wl2 = synth.PagedWorkload([0], [bulk_tokens], hkv, seed=seed + 5 + 1000 * rank, device=dev)
    kb, vb = synth.make_kv(bulk_tokens, hkv, seed + 5, device=dev)   # 2 x 67 MB at 32768 tokens: > L2 together with the pool
    b2 = wl2.step()
    for _ in range(3):
        kv.kv_cache_write(step.ex, wl2.layer, b2, kb, vb, lib=lib)
    barrier(world)
    n_bulk = 20
    e0.record()
    for _ in range(n_bulk):
        kv.kv_cache_write(step.ex, wl2.layer, b2, kb, vb, lib=lib)
    e1.record()
    barrier(world)
    bulk_ms = max_over_ranks(e0.elapsed_time(e1), world) / n_bulk
    bulk_tok_s = world * bulk_tokens / (bulk_ms * 1e-3)

    sharded_cases = None
    if args.config == "cfg1_batched_decode" and not reference and not args.no_sharded and args.batch == 0:
        try:
            sharded_cases = strong_scaling_cases(args, world, rank, dev,
                                                 {"ms_per_step": ms_per_step, "value": value, "kv_bytes": all_bytes})
        except Exception as exc:     # every rank raises or none: the collectives inside are entered by all
            sharded_cases = {"error": repr(exc)}
    if rank != 0:
        return
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    achieved = kv_bytes / (attn_ms * 1e-3) / 1e9
    traffic_ratio, traffic_rec = (None, None) if reference else measured_traffic_ratio("tq4_attention_stream_kernel<exact>")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if sharded else "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"{args.config}: {batch} seqs x ctx U[{lo},{hi}], {hq} q heads / {hkv} kv heads, "
                               f"d256, TQ4 pages of 16, step = append {q_len} token/seq + decode attention",
                   "kv_bytes_per_step_per_gpu": kv_bytes, "tokens_in_cache_per_gpu": int(sum(wl.ctx)),
                   "l2": "KV read per step (>1.3 GB) is larger than L2; no flush needed",
                   "per_gpu_batch": batch, "parallelism": ((f"pages of one sequence sharded x{world}, (m, l, acc) triples exchanged and merged by one kernel over peer-mapped memory"
                                    if peer_px is not None else
                                    f"pages of one sequence sharded x{world}, (m, l, acc) triples all-gathered over NCCL")
                                   if sharded else f"batch-sharded x{world}, no collective")},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
                     "kernel": "tq4_attention_stream_kernel, exact build (+ plan and merge launches, timed together)",
                     "launch_ms": attn_ms,
                     # DRAM bytes of one stream-kernel launch: the ratio measured by ncu on a smaller case of
                     # the same kernel (recorded with its date and workload) times this run's bytes
                     "traffic": (kv_bytes * traffic_ratio if traffic_ratio is not None and not sharded else None),
                     **({"traffic_source": traffic_rec} if traffic_rec is not None and not sharded else {})},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": (step.h2d_bytes_total - h2d_before) / e2e_steps,
                "d2h_bytes_per_step": step.d2h_bytes, "cuda_graph_replay": use_graph,
                **({"speculative_rollback": rollback} if rollback else {})},
        **({"exchange": "peer", "exchange_equals_allgather_merge": bool(exchange_ok and peer_px.status() == 0)}
           if peer_px is not None else {}),
        "gpu_launches": 4 * args.steps, "cuda_graph_replay": graph_used, "eager_ms_per_step": eager_ms_per_step,
        "repeats": REPS, "ms_per_step_min_max": [float(min(rep_ms)), float(max(rep_ms))],
        **({"parity": parity} if parity is not None else {}),
        **({"sharded": sharded_cases} if sharded_cases is not None else {}),
        **({"fast_build": fast_build} if fast_build is not None else {}),
        "clocks": clocks,
        "append_tokens_per_s": n_tok / (append_ms * 1e-3), "append_ms": append_ms,
        "append_bulk": {"tokens": bulk_tokens, "ms": bulk_ms, "tokens_per_s": bulk_tok_s,
                        "algorithmic_GBps": bulk_tok_s * hkv * 1288 / 1e9,
                        "frac_of_peak": bulk_tok_s * hkv * 1288 / 1e9 / (world * float(measured_peaks()[0].get("hbm_gbs", FALLBACK_HBM_GBS)))},
        "attention_steps_per_s": 1e3 / attn_ms, "kernel_status": status,
    }
    if reference:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": value, "unit": UNIT, "cores": 0, "kind": "reference",
                                "sample": "the reference's CUDA kernels (op_kv_cache.cu, op_paged_attn.cu) built "
                                          "unmodified for sm_100a, run on the GPU: the reference has no CPU path"}
        line["gpu_launches"] = None
        line["roofline"]["kernel"] = "reference paged_attention_gqa_mma_f16_kernel"
    elif not args.no_cpu_baseline:
        b = host_step_batch(kv, step, batch, n_tok)
        line["cpu_baseline"] = cpu_baseline(wl, hq, q_new.numpy().view(np.uint16), k_new.numpy().view(np.uint16),
                                            v_new.numpy().view(np.uint16), b.host_desc(), q_len=q_len)
    print(json.dumps(line))


if __name__ == "__main__":
    try:
        main()
    finally:
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            import torch.distributed as _dist
            if _dist.is_initialized():
                _dist.destroy_process_group()
