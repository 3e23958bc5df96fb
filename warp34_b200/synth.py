"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (no dataset is involved).

Values: K, V ~ N(0,1) rounded to bf16, four fixed channels per head scaled x20, then moved to
the grid that bf16 and fp16 share (|x| < 2^-14 flushed to zero), so the fp16 kernels see exactly
the reals a bf16 producer would emit.  Q ~ N(0,1) on the same grid.  Page tables come from a
seeded shuffled free list with page 0 kept as the trash sink.
"""
import numpy as np
import torch

from . import ffi
from . import kv as kvmod

HEAD_DIM = 256
PAGE = 16

CONFIGS = {
    # name: (num_q_heads, num_kv_heads, batch, ctx_lo, ctx_hi, q_len, seed)
    "cfg0_single_layer": (16, 4, 4, 1024, 4096, 1, 0),
    "cfg1_batched_decode": (24, 4, 64, 8192, 32768, 1, 1),
    "cfg3_mtp_verify": (24, 4, 128, 2048, 16384, 4, 3),
    "cfg4_long_context": (16, 4, 1, 262144, 262144, 1, 4),
}


def _grid(x_bf16):
    x = x_bf16.to(torch.float32)
    x = torch.where(x.abs() < 2.0 ** -14, torch.zeros_like(x), x)
    return x.to(torch.float16)


def outlier_channels(num_heads, seed):
    g = np.random.RandomState((seed + 7919) % (1 << 32))  # numpy seeds are 32-bit; per-rank seeds exceed that
    return np.stack([np.sort(g.choice(HEAD_DIM, 4, replace=False)) for _ in range(num_heads)])


def make_kv(num_tokens, num_heads, seed, device="cpu", outliers=None):
    """fp16 K and V, each [num_tokens, num_heads * 256]."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    outs = outlier_channels(num_heads, seed) if outliers is None else outliers
    res = []
    for _ in range(2):
        x = torch.randn(num_tokens, num_heads, HEAD_DIM, generator=gen, device=device, dtype=torch.float32)
        x = x.to(torch.bfloat16).to(torch.float32)
        for h in range(num_heads):
            idx = torch.as_tensor(outs[h], device=device, dtype=torch.long)
            x[:, h, idx] *= 20.0
        res.append(_grid(x.to(torch.bfloat16)).reshape(num_tokens, num_heads * HEAD_DIM).contiguous())
    return res[0], res[1]


def make_q(num_tokens, num_q_heads, seed, device="cpu"):
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 104729)
    x = torch.randn(num_tokens, num_q_heads, HEAD_DIM, generator=gen, device=device, dtype=torch.float32)
    return _grid(x.to(torch.bfloat16)).contiguous()


def context_lengths(batch, lo, hi, seed):
    g = np.random.RandomState(seed % (1 << 32))
    return g.randint(lo, hi + 1, size=batch).astype(np.int64)


class PagedWorkload:
    """A pool, one sequence per request, and the metadata of a step with q_len new tokens each.

    ctx[i] tokens are already committed for sequence i; the step appends q_lens[i] tokens and
    attends over ctx[i] + q_lens[i] keys (causal among the new tokens).
    """

    def __init__(self, ctx, q_lens, num_kv_heads, seed, device="cuda", slack_pages=64,
                 shuffle=True, fill=None, formats=None):
        self.ctx = [int(c) for c in ctx]
        self.q_lens = [int(q) for q in q_lens]
        n = len(self.ctx)
        need = sum((c + q + PAGE - 1) // PAGE for c, q in zip(self.ctx, self.q_lens))
        self.num_pages = need + slack_pages + 1
        self.pool = kvmod.PagePool(self.num_pages, PAGE)
        if shuffle:
            self.pool.shuffle_free_list(seed, reserve_page0=True)
        else:
            assert self.pool.alloc_page() == 0  # keep page 0 as the trash sink
        self.seqs = [kvmod.Sequence(self.pool) for _ in range(n)]
        for s, c, q in zip(self.seqs, self.ctx, self.q_lens):
            rc = s.reserve(c + q)
            assert rc >= 0, rc
        self.bf16_storage = formats is not None and tuple(formats) == tuple(kvmod.BF16_KV_FORMATS)
        extra = {} if formats is None else {"formats": tuple(formats)}
        self.layer = kvmod.KvLayer(self.num_pages, num_kv_heads, device=device, fill=fill, **extra)
        self.num_kv_heads = num_kv_heads
        self.device = device
        self.max_blocks = max(s.num_pages for s in self.seqs)

    def step(self, q_lens=None, sm_scale=1.0 / 16.0, **kw):
        return kvmod.build_step(self.seqs, q_lens if q_lens is not None else self.q_lens,
                                self.max_blocks, sm_scale, device=self.device, **kw)

    def prefill_batches(self, chunk_tokens):
        """Yields (seq_index, start, n) pieces that cover every sequence's ctx tokens."""
        for i, c in enumerate(self.ctx):
            for start in range(0, c, chunk_tokens):
                yield i, start, min(chunk_tokens, c - start)

    def fill_context(self, ex, seed, chunk_tokens=65536, lib=None, keep=False):
        """Appends ctx[i] synthetic tokens to every sequence through the append entry point and
        commits them.  Returns (K, V) fp16 host copies per sequence when keep=True."""
        kept = []
        for i, s in enumerate(self.seqs):
            ks, vs = [], []
            c = self.ctx[i]
            start = 0
            while start < c:
                n = min(chunk_tokens, c - start)
                k, v = make_kv(n, self.num_kv_heads, seed * 1000003 + i * 1009 + start, device=self.device)
                batch = kvmod.build_step([s], [n], self.max_blocks, 1.0 / 16.0, device=self.device)
                if self.bf16_storage:
                    k, v = k.to(torch.bfloat16), v.to(torch.bfloat16)   # exact: values sit on the bf16 grid
                    kvmod.kv_cache_write_bf16(ex, self.layer, batch, k, v, lib=lib)
                else:
                    kvmod.kv_cache_write(ex, self.layer, batch, k, v, lib=lib)
                s.commit(n)
                if keep:
                    ks.append(k.cpu())
                    vs.append(v.cpu())
                start += n
            if keep:
                kept.append((torch.cat(ks) if ks else None, torch.cat(vs) if vs else None))
        if self.device != "cpu":
            torch.cuda.synchronize()
        return kept

    def algorithmic_kv_bytes(self):
        """KV bytes one decode / verify pass must read: sum(ctx+q) * Hkv * (K row + V row bytes):
        264 for TQ4 storage, 1024 for uncompressed BF16, 528 for FP8 E4M3 rows, 544 for Q8_0 rows."""
        lay = self.layer.layout
        row_pair = (ffi.host().w34_kv_format_row_bytes(lay.k_format, HEAD_DIM) +
                    ffi.host().w34_kv_format_row_bytes(lay.v_format, HEAD_DIM))
        return sum(c + q for c, q in zip(self.ctx, self.q_lens)) * self.num_kv_heads * row_pair
