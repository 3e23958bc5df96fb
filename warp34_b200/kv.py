"""Host-side mirror of the reference's KV cache interface for this path, over the C ABIs.

Reference counterparts: KvPool / PageBitmap / KvFormatPolicy (crates/warp34-host/src/cache.rs),
ReqRadixState page vectors and rollback (crates/warp34-host/src/radix.rs:1070-1245), the step
metadata packers (crates/warp34-host/src/model/graph_io.rs:368-420, execution.rs:7-127) and the
two kernel calls of run_attention_block (crates/warp34-host/src/model/forward.rs:1141-1188).

torch is used only to own device memory and streams.
"""
import ctypes as C
import os

import numpy as np
import torch

from . import ffi


class PagePool:
    """Logical page allocator (lowest-free-first, or a seeded shuffled free list)."""

    def __init__(self, num_pages, block_size=16):
        self._h = ffi.host()
        self.handle = self._h.w34_pool_create(num_pages, block_size)
        if not self.handle:
            raise ValueError("w34_pool_create failed")
        self.block_size = block_size

    def close(self):
        if self.handle:
            self._h.w34_pool_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    num_pages = property(lambda s: s._h.w34_pool_num_pages(s.handle))
    free_count = property(lambda s: s._h.w34_pool_free_count(s.handle))

    def alloc_page(self):
        p = self._h.w34_pool_alloc_page(self.handle)
        return None if p < 0 else p

    def free_page(self, page):
        return self._h.w34_pool_free_page(self.handle, int(page))

    def ref_page(self, page):
        return self._h.w34_pool_ref_page(self.handle, int(page))

    def refcount(self, page):
        return self._h.w34_pool_refcount(self.handle, int(page))

    def reset(self):
        self._h.w34_pool_reset(self.handle)

    def truncate(self, max_pages):
        self._h.w34_pool_truncate(self.handle, max_pages)

    def shuffle_free_list(self, seed, reserve_page0=True):
        return self._h.w34_pool_shuffle_free_list(self.handle, seed, 1 if reserve_page0 else 0)

    def stats(self):
        st = ffi.PoolStats()
        self._h.w34_pool_get_stats(self.handle, C.byref(st))
        return {"capacity": st.capacity, "free": st.free_pages, "shared": st.shared_pages,
                "active": st.active_pages}


class Sequence:
    """Block table and committed length of one request."""

    def __init__(self, pool):
        self._h = ffi.host()
        self.pool = pool
        self.handle = self._h.w34_seq_create(pool.handle)

    def close(self):
        if self.handle:
            self._h.w34_seq_destroy(self.handle)
            self.handle = None

    def attach_prefix(self, pages, num_tokens):
        arr = (C.c_int32 * len(pages))(*pages)
        return self._h.w34_seq_attach_prefix(self.handle, arr, len(pages), num_tokens)

    def reserve(self, total_tokens):
        return self._h.w34_seq_reserve(self.handle, total_tokens)

    def prepare_append(self):
        """Returns None, or (src_page, dst_page, rows) when a shared tail page must be copied."""
        s, d, r = C.c_int32(), C.c_int32(), C.c_int32()
        rc = self._h.w34_seq_prepare_append(self.handle, C.byref(s), C.byref(d), C.byref(r))
        if rc < 0:
            raise RuntimeError(f"w34_seq_prepare_append: {rc}")
        return (s.value, d.value, r.value) if rc == 1 else None

    def commit(self, n):
        return self._h.w34_seq_commit(self.handle, n)

    def set_committed(self, n):
        return self._h.w34_seq_set_committed(self.handle, n)

    def rollback(self):
        cap = max(self.num_pages, 1)
        buf = (C.c_int32 * cap)()
        n = self._h.w34_seq_rollback(self.handle, buf, cap)
        if n < 0:
            raise RuntimeError(f"w34_seq_rollback: {n}")
        return list(buf[:n])

    committed_len = property(lambda s: s._h.w34_seq_committed_len(s.handle))
    num_pages = property(lambda s: s._h.w34_seq_num_pages(s.handle))
    protected_pages = property(lambda s: s._h.w34_seq_protected_pages(s.handle))

    @property
    def pages(self):
        n = self.num_pages
        p = self._h.w34_seq_pages(self.handle)
        return [p[i] for i in range(n)]

    def set_pages_unchecked(self, pages, protected_pages=0):
        arr = (C.c_int32 * len(pages))(*pages)
        return self._h.w34_seq_set_pages_unchecked(self.handle, arr, len(pages), protected_pages)


class PrefixCache:
    """Page-aligned radix cache of token prefixes (KV half of the reference's MambaRadixCache)."""

    def __init__(self, pool):
        self._h = ffi.host()
        self.pool = pool
        self.handle = self._h.w34_radix_create(pool.handle)

    def close(self):
        if self.handle:
            self._h.w34_radix_destroy(self.handle)
            self.handle = None

    def match_prefix(self, tokens):
        """Returns (pages, matched_tokens, node)."""
        n = len(tokens)
        tok = (C.c_int32 * max(n, 1))(*tokens)
        cap = n // self.pool.block_size + 1
        out = (C.c_int32 * cap)()
        mt, node = C.c_int32(), C.c_int32()
        rc = self._h.w34_radix_match_prefix(self.handle, tok, n, out, cap, C.byref(mt), C.byref(node))
        if rc < 0:
            raise RuntimeError(f"w34_radix_match_prefix: {rc}")
        return list(out[:rc]), mt.value, node.value

    def insert(self, tokens, pages):
        """Returns (tokens already cached, node ending the sequence)."""
        tok = (C.c_int32 * max(len(tokens), 1))(*tokens)
        pg = (C.c_int32 * max(len(pages), 1))(*pages)
        node = C.c_int32()
        rc = self._h.w34_radix_insert(self.handle, tok, len(tokens), pg, len(pages), C.byref(node))
        if rc < 0:
            raise RuntimeError(f"w34_radix_insert: {rc}")
        return rc, node.value

    def lock(self, node):
        return self._h.w34_radix_lock(self.handle, node)

    def unlock(self, node):
        return self._h.w34_radix_unlock(self.handle, node)

    def evict(self, num_pages):
        cap = self.pool.num_pages
        buf = (C.c_int32 * cap)()
        n = self._h.w34_radix_evict(self.handle, num_pages, buf, cap)
        if n < 0:
            raise RuntimeError(f"w34_radix_evict: {n}")
        return list(buf[:n])

    def stats(self):
        st = ffi.RadixStats()
        self._h.w34_radix_get_stats(self.handle, C.byref(st))
        return {"nodes": st.nodes, "cached": st.cached_pages, "protected": st.protected_pages,
                "evictable": st.evictable_pages}

    def sanity_check(self):
        return self._h.w34_radix_sanity_check(self.handle)


class SpeculativeBatch:
    """The page bookkeeping of one speculative (draft + verify) step for a fixed set of sequences:
    reserve pages for `extra` tokens each, and after the verify pass commit the accepted tokens and
    hand back the pages that only held rejected ones (mtp/propose.rs, radix.rs:1197-1245)."""

    def __init__(self, seqs):
        self.seqs = list(seqs)
        n = len(self.seqs)
        self._handles = (C.c_void_p * n)(*[s.handle for s in self.seqs])
        self._accepted = (C.c_int32 * n)()
        self._freed = (C.c_int32 * max(4 * n, 1))()
        self._h = ffi.host()

    def reserve_ahead(self, extra_tokens):
        rc = self._h.w34_seqs_reserve_ahead(self._handles, len(self.seqs), extra_tokens)
        if rc < 0:
            raise RuntimeError(f"w34_seqs_reserve_ahead: {rc}")
        return rc

    def commit_and_rollback(self, accepted):
        n = len(self.seqs)
        self._accepted[:] = [int(a) for a in accepted]
        rc = self._h.w34_seqs_commit_and_rollback(self._handles, self._accepted, n, self._freed, len(self._freed))
        if rc < 0:
            raise RuntimeError(f"w34_seqs_commit_and_rollback: {rc}")
        return list(self._freed[:rc])


def resolve_layer(policy, ordinal, num_layers, supports_fp8=False):
    out = (C.c_int32 * 4)()
    rc = ffi.host().w34_kv_policy_resolve_layer(policy, ordinal, num_layers, int(supports_fp8), out)
    if rc != 0:
        raise ValueError("bad policy")
    return tuple(out)


class KvLayer:
    """One layer's K and V slabs plus its descriptor (KvLayerBuffer, cache.rs:168-177)."""

    def __init__(self, num_pages, local_kv_heads, head_dim=256, block_size=16,
                 formats=(ffi.KV_FORMAT_TQ4, ffi.KV_FORMAT_TQ4,
                          ffi.KV_TRANSFORM_RADEMACHER_WHT256, ffi.KV_TRANSFORM_RADEMACHER_WHT256),
                 device="cuda", namespace_id=0, layer_id=0, fill=None):
        self.layout = ffi.KvLayerLayout()
        f = (C.c_int32 * 4)(*formats)
        kb, vb = C.c_uint64(), C.c_uint64()
        rc = ffi.host().w34_kv_layout_init(C.byref(self.layout), 0, 0, namespace_id, layer_id,
                                           local_kv_heads, head_dim, block_size, f, num_pages,
                                           C.byref(kb), C.byref(vb))
        if rc != 0:
            raise ValueError("w34_kv_layout_init failed")
        if fill is None:
            self.k = torch.zeros(kb.value, dtype=torch.uint8, device=device)
            self.v = torch.zeros(vb.value, dtype=torch.uint8, device=device)
        else:
            self.k = torch.full((kb.value,), fill, dtype=torch.uint8, device=device)
            self.v = torch.full((vb.value,), fill, dtype=torch.uint8, device=device)
        self.layout.k_base = self.k.data_ptr()
        self.layout.v_base = self.v.data_ptr()
        self.num_pages = num_pages


class StepBatch:
    """Device-resident metadata of one step plus the warp34_attention_batch descriptor."""

    def __init__(self, query_start_loc, context_lens_before, seq_lens_after, block_tables,
                 write_slot_mapping, max_blocks_per_req, sm_scale, device="cuda", mask_mode=0,
                 sliding_window=0, valid_token_mask=None, valid_req_mask=None, max_q_len=None,
                 max_seq_len=None):
        i32 = lambda a: torch.as_tensor(np.ascontiguousarray(a, dtype=np.int32)).to(device)  # noqa: E731
        self.host = dict(query_start_loc=np.asarray(query_start_loc, np.int32),
                         context_lens_before=np.asarray(context_lens_before, np.int32),
                         seq_lens_after=np.asarray(seq_lens_after, np.int32),
                         block_tables=np.asarray(block_tables, np.int32),
                         write_slot_mapping=np.asarray(write_slot_mapping, np.int32),
                         valid_token_mask=None if valid_token_mask is None else np.asarray(valid_token_mask, np.uint8),
                         valid_req_mask=None if valid_req_mask is None else np.asarray(valid_req_mask, np.uint8))
        self.qsl = i32(query_start_loc)
        self.ctx = i32(context_lens_before)
        self.seq = i32(seq_lens_after)
        self.bt = i32(block_tables)
        self.slots = i32(write_slot_mapping)
        self.vtm = None if valid_token_mask is None else torch.as_tensor(np.asarray(valid_token_mask, np.uint8)).to(device)
        self.vrm = None if valid_req_mask is None else torch.as_tensor(np.asarray(valid_req_mask, np.uint8)).to(device)
        q = np.asarray(query_start_loc, np.int64)
        b = ffi.AttentionBatch()
        b.query_start_loc = self.qsl.data_ptr()
        b.context_lens_before = self.ctx.data_ptr()
        b.seq_lens_after = self.seq.data_ptr()
        b.block_tables = self.bt.data_ptr()
        b.write_slot_mapping = self.slots.data_ptr()
        b.valid_token_mask = None if self.vtm is None else self.vtm.data_ptr()
        b.valid_req_mask = None if self.vrm is None else self.vrm.data_ptr()
        b.num_reqs = len(q) - 1
        b.total_tokens = int(q[-1])
        b.max_blocks_per_req = int(max_blocks_per_req)
        b.max_q_len = int(max_q_len if max_q_len is not None else (np.diff(q).max() if len(q) > 1 else 0))
        b.max_seq_len = int(max_seq_len if max_seq_len is not None else (np.max(seq_lens_after) if len(q) > 1 else 0))
        b.mask_mode = mask_mode
        b.sliding_window = sliding_window
        b.sm_scale = sm_scale
        self.desc = b

    def host_desc(self):
        """The same descriptor over HOST arrays (for the CPU oracle)."""
        h = self.host
        b = ffi.AttentionBatch()
        C.memmove(C.byref(b), C.byref(self.desc), C.sizeof(b))
        b.query_start_loc = h["query_start_loc"].ctypes.data
        b.context_lens_before = h["context_lens_before"].ctypes.data
        b.seq_lens_after = h["seq_lens_after"].ctypes.data
        b.block_tables = h["block_tables"].ctypes.data
        b.write_slot_mapping = h["write_slot_mapping"].ctypes.data
        b.valid_token_mask = None if h["valid_token_mask"] is None else h["valid_token_mask"].ctypes.data
        b.valid_req_mask = None if h["valid_req_mask"] is None else h["valid_req_mask"].ctypes.data
        return b


def build_step(seqs, q_lens, max_blocks_per_req, sm_scale, device="cuda", **kw):
    """Packs the step metadata of `seqs` (each already reserved) through the C++ builder."""
    n = len(seqs)
    total = int(sum(q_lens))
    handles = (C.c_void_p * n)(*[s.handle for s in seqs])
    ql = (C.c_int32 * n)(*q_lens)
    qsl = np.zeros(n + 1, np.int32)
    ctx = np.zeros(n, np.int32)
    seq = np.zeros(n, np.int32)
    bt = np.zeros((n, max_blocks_per_req), np.int32)
    slots = np.zeros(max(total, 1), np.int32)
    mq, ms = C.c_int32(), C.c_int32()
    ip = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))  # noqa: E731
    rc = ffi.host().w34_build_step_metadata(handles, ql, n, max_blocks_per_req, ip(qsl), ip(ctx),
                                            ip(seq), ip(bt), ip(slots), C.byref(mq), C.byref(ms))
    if rc < 0:
        raise RuntimeError(f"w34_build_step_metadata: {rc}")
    kw.setdefault("max_q_len", mq.value)  # a caller may declare another bound (tests of the contract)
    return StepBatch(qsl, ctx, seq, bt, slots[:total], max_blocks_per_req, sm_scale, device=device,
                     max_seq_len=ms.value, **kw)


class Executor:
    """warp34_exec: a stream and a scratch buffer."""

    def __init__(self, scratch_bytes=64 << 20, device="cuda", stream=None):
        self.scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=device)
        self.ex = ffi.Exec()
        self.ex.scratch_ptr = self.scratch.data_ptr()
        self.ex.scratch_size = scratch_bytes
        self.ex.flags = 0
        self.set_stream(stream)

    def set_stream(self, stream=None):
        s = stream if stream is not None else torch.cuda.current_stream()
        self.ex.stream = s.cuda_stream


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUDA error {rc}")


def kv_cache_write(ex, layer, batch, k, v, k_row_stride=None, v_row_stride=None, lib=None):
    """warp34_kv_cache_write_strided: fp16 k/v [tokens, heads*256] (or strided views)."""
    lib = lib or ffi.kernels()
    ks = k_row_stride if k_row_stride is not None else k.stride(0)
    vs = v_row_stride if v_row_stride is not None else v.stride(0)
    rc = lib.warp34_kv_cache_write_strided(C.byref(ex.ex), C.byref(layer.layout), C.byref(batch.desc),
                                           k.data_ptr(), v.data_ptr(), ks, vs)
    _check(rc, "warp34_kv_cache_write_strided")


def paged_attention(ex, layer, batch, q, out, num_q_heads, lib=None, scalar=False):
    """warp34_paged_attention_f16 (or the scalar dequant-then-attend entry point)."""
    lib = lib or ffi.kernels()
    fn = lib.warp34_paged_attention_scalar_f16 if scalar else lib.warp34_paged_attention_f16
    rc = fn(C.byref(ex.ex), C.byref(layer.layout), C.byref(batch.desc), q.data_ptr(), out.data_ptr(),
            num_q_heads)
    _check(rc, "warp34_paged_attention_f16")


def paged_attention_gated(ex, layer, batch, q, gate, out, num_q_heads, hadamard64=False, lib=None):
    """warp34_paged_attention_gated_f16: attention, sigmoid output gate and (optionally) the
    Hadamard-64 pre-rotation of o_proj's input in one call."""
    lib = lib or ffi.kernels()
    rc = lib.warp34_paged_attention_gated_f16(C.byref(ex.ex), C.byref(layer.layout), C.byref(batch.desc), q.data_ptr(),
                                              gate.data_ptr(), out.data_ptr(), num_q_heads, 1 if hadamard64 else 0)
    _check(rc, "warp34_paged_attention_gated_f16")


BF16_KV_FORMATS = (ffi.KV_FORMAT_BF16, ffi.KV_FORMAT_BF16, ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_IDENTITY)


def kv_cache_write_bf16(ex, layer, batch, k, v, row_stride_elems=None, lib=None):
    """warp34_kv_cache_write_strided_bf16: bf16 k/v into a BF16-format layer (KvLayer(formats=BF16_KV_FORMATS))."""
    lib = lib or ffi.kernels()
    rs = row_stride_elems if row_stride_elems is not None else k.stride(0)
    rc = lib.warp34_kv_cache_write_strided_bf16(C.byref(ex.ex), C.byref(layer.layout), C.byref(batch.desc),
                                                k.data_ptr(), v.data_ptr(), rs)
    _check(rc, "warp34_kv_cache_write_strided_bf16")


def paged_attention_bf16kv(ex, layer, batch, q, out, num_q_heads, lib=None):
    """warp34_paged_attention_bf16: bf16 q / out over a BF16-format layer."""
    lib = lib or ffi.kernels()
    rc = lib.warp34_paged_attention_bf16(C.byref(ex.ex), C.byref(layer.layout), C.byref(batch.desc),
                                         q.data_ptr(), out.data_ptr(), num_q_heads)
    _check(rc, "warp34_paged_attention_bf16")


def paged_attention_partial(ex, layer, batch, q, triples, num_q_heads, lib=None):
    """warp34_paged_attention_partial_f16: triples is fp32 [tokens, heads, 258]."""
    lib = lib or ffi.kernels()
    rc = lib.warp34_paged_attention_partial_f16(C.byref(ex.ex), C.byref(layer.layout), C.byref(batch.desc),
                                                q.data_ptr(), triples.data_ptr(), num_q_heads)
    _check(rc, "warp34_paged_attention_partial_f16")


def merge_shards(ex, triples, out, lib=None):
    """warp34_paged_attention_merge_shards_f16: triples fp32 [shards, rows, 258] -> out fp16 [rows, 256]."""
    lib = lib or ffi.kernels()
    shards, rows = triples.shape[0], triples[0].numel() // 258
    rc = lib.warp34_paged_attention_merge_shards_f16(C.byref(ex.ex), triples.data_ptr(), shards, rows, out.data_ptr())
    _check(rc, "warp34_paged_attention_merge_shards_f16")


class PeerExchange:
    """Mailboxes of warp34_paged_attention_exchange_merge_f16: per rank one buffer
    [inbox fp32 [2][world][max_rows][258] | flags u32 [world][max_rows]] that every rank has mapped,
    plus this rank's private step counters and status word.

    `symmetric()` allocates the buffers in torch's symmetric memory (peer-mapped over NVLink) for a
    process group; `over_buffers()` takes addresses the caller mapped itself (tests hand it several
    buffers of one device to play the peers' parts)."""

    @staticmethod
    def mailbox_bytes(world, max_rows):
        return 2 * world * max_rows * 258 * 4 + world * max_rows * 4

    def __init__(self, world, rank, max_rows, base_addrs, device, wait_limit=0, keep=()):
        self.world, self.rank, self.max_rows = world, rank, max_rows
        self.private = torch.zeros(max_rows + 1, dtype=torch.int32, device=device)  # steps | status
        self._keep = keep
        mb = ffi.PeerMailboxes()
        mb.world, mb.rank, mb.max_rows, mb.wait_limit = world, rank, max_rows, wait_limit
        inbox_bytes = 2 * world * max_rows * 258 * 4
        for w in range(world):
            mb.inbox[w] = int(base_addrs[w])
            mb.flags[w] = int(base_addrs[w]) + inbox_bytes
        mb.steps = self.private.data_ptr()
        mb.status = self.private.data_ptr() + 4 * max_rows
        self.mb = mb

    @classmethod
    def over_buffers(cls, rank, max_rows, buffers, wait_limit=0):
        world = len(buffers)
        for b in buffers:
            assert b.dtype == torch.uint8 and b.numel() >= cls.mailbox_bytes(world, max_rows)
        return cls(world, rank, max_rows, [b.data_ptr() for b in buffers], buffers[rank].device,
                   wait_limit=wait_limit, keep=tuple(buffers))

    @classmethod
    def symmetric(cls, group, max_rows, device, wait_limit=0):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        # plain peer mappings only: the mailboxes are never bound to an NVSwitch multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        buf = symm.empty(cls.mailbox_bytes(world, max_rows), dtype=torch.uint8, device=device)
        buf.zero_()
        handle = symm.rendezvous(buf, group)
        torch.cuda.synchronize()
        dist.barrier(group)  # every mailbox is zeroed before anyone stores into it
        return cls(world, rank, max_rows, list(handle.buffer_ptrs), device, wait_limit=wait_limit,
                   keep=(buf, handle))

    def status(self):
        return int(self.private[self.max_rows].item())

    def exchange_merge(self, ex, triples, out, lib=None):
        """triples fp32 [rows, 258] of this rank -> out fp16 [rows, 256] merged over all ranks."""
        lib = lib or ffi.kernels()
        rows = triples.numel() // 258
        rc = lib.warp34_paged_attention_exchange_merge_f16(C.byref(ex.ex), C.byref(self.mb), triples.data_ptr(),
                                                           rows, out.data_ptr())
        _check(rc, "warp34_paged_attention_exchange_merge_f16")


def kv_page_copy(ex, layer, src_page, dst_page, rows, lib=None):
    lib = lib or ffi.kernels()
    _check(lib.warp34_kv_page_copy(C.byref(ex.ex), C.byref(layer.layout), src_page, dst_page, rows),
           "warp34_kv_page_copy")


class StepIo:
    """Persistent step-metadata buffers: one pinned host arena and one device arena (the reference
    packs tokens | slots | block tables | lengths into a single pinned upload,
    crates/warp34-host/src/model/execution.rs:38-93; graph_io.rs:368-420).  Each step uploads the
    small arrays (lengths, slots) in one copy and, of the block tables, only the row suffixes that
    changed since the last upload (graph_io.rs:109-195): a decode step adds a page to one sequence
    in sixteen."""

    def __init__(self, max_reqs, max_tokens, max_blocks_per_req, device="cuda"):
        self.max_reqs, self.max_tokens, self.max_blocks = max_reqs, max_tokens, max_blocks_per_req
        # arena order: query_start_loc | context_lens_before | seq_lens_after | write_slot_mapping | block_tables
        sizes = [max_reqs + 1, max_reqs, max_reqs, max_tokens, max_reqs * max_blocks_per_req]
        offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])
        self._offs, self._sizes = offs, sizes
        total = int(offs[-1])
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory() if device != "cpu" else torch.zeros(total, dtype=torch.int32)
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self._np = self.host.numpy()
        # per-row changed column ranges: of the last pack, and pending since the last upload
        self._lo = np.zeros(max_reqs, np.int32)
        self._hi = np.zeros(max_reqs, np.int32)
        self._pend_lo = np.full(max_reqs, max_blocks_per_req, np.int32)
        self._pend_hi = np.zeros(max_reqs, np.int32)
        self._uploaded_once = False
        self._packs_pending = 0
        self._arg_key = None
        ip = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))  # noqa: E731
        self._lo_p, self._hi_p = ip(self._lo), ip(self._hi)
        self._pack_fn = ffi.host().w34_build_step_metadata_delta
        self.desc = ffi.AttentionBatch()
        base = self.dev.data_ptr()
        self.desc.query_start_loc = base + 4 * int(offs[0])
        self.desc.context_lens_before = base + 4 * int(offs[1])
        self.desc.seq_lens_after = base + 4 * int(offs[2])
        self.desc.write_slot_mapping = base + 4 * int(offs[3])
        self.desc.block_tables = base + 4 * int(offs[4])
        self.desc.max_blocks_per_req = max_blocks_per_req
        self._arena_ptrs = (self._ptr(0), self._ptr(1), self._ptr(2), self._ptr(4), self._ptr(3))
        self.nbytes = total * 4          # a full upload
        self.last_upload_bytes = 0

    def _ptr(self, i):
        return C.cast(self._np.ctypes.data + 4 * int(self._offs[i]), C.POINTER(C.c_int32))

    def pack(self, seqs, q_lens, sm_scale, mask_mode=0, sliding_window=0):
        n = len(seqs)
        assert n <= self.max_reqs and sum(q_lens) <= self.max_tokens
        key = (tuple(id(s) for s in seqs), tuple(q_lens))
        if key != self._arg_key:          # the ctypes argument arrays are rebuilt only when the batch changes
            self._arg_key = key
            self._handles = (C.c_void_p * n)(*[s.handle for s in seqs])
            self._ql = (C.c_int32 * n)(*q_lens)
        handles, ql = self._handles, self._ql
        mq, ms = C.c_int32(), C.c_int32()
        # the packer writes the changed ranges of this pack; a second pack before an upload folds the
        # earlier ranges in
        if self._packs_pending:
            np.minimum(self._pend_lo, self._lo, out=self._pend_lo)
            np.maximum(self._pend_hi, self._hi, out=self._pend_hi)
        rc = self._pack_fn(handles, ql, n, self.max_blocks, *self._arena_ptrs, C.byref(mq), C.byref(ms),
                           self._lo_p, self._hi_p)
        if rc < 0:
            raise RuntimeError(f"w34_build_step_metadata_delta: {rc}")
        self._packs_pending += 1
        d = self.desc
        d.num_reqs, d.total_tokens = n, rc
        d.max_q_len, d.max_seq_len = mq.value, ms.value
        d.mask_mode, d.sliding_window, d.sm_scale = mask_mode, sliding_window, sm_scale
        return rc

    def upload(self, full=False, tables_only=False):
        """One copy of the arena up to the last block-table entry that changed since the previous
        upload (the length and slot arrays sit in front of the tables); returns the bytes copied.
        tables_only: the copy starts at the block tables (the caller uploads the front part itself,
        e.g. from a captured graph) and is skipped when no entry changed."""
        bt0, bt1 = int(self._offs[4]), int(self._offs[5])
        end = bt0
        if full or not self._uploaded_once:
            end = bt1
        else:
            lo, hi = self._lo, self._hi
            if self._packs_pending > 1:
                lo, hi = np.minimum(self._pend_lo, lo), np.maximum(self._pend_hi, hi)
            rows = np.flatnonzero(hi > lo)
            if len(rows):
                r = int(rows[-1])
                end = bt0 + r * self.max_blocks + int(hi[r])
        begin = bt0 if tables_only else 0
        if end > begin:
            self.dev[begin:end].copy_(self.host[begin:end], non_blocking=True)
        self._uploaded_once = True
        if self._packs_pending > 1:
            self._pend_lo[:] = self.max_blocks
            self._pend_hi[:] = 0
        self._packs_pending = 0
        self.last_upload_bytes = 4 * (end - begin)
        return self.last_upload_bytes

    @property
    def head_words(self):
        """Words in front of the block tables: lengths and slots."""
        return int(self._offs[4])


class _DescOnly:
    def __init__(self, desc):
        self.desc = desc


class DecodeStep:
    """The call a user of this path makes once per model step and layer: new K/V rows and Q in
    HOST memory in, attention output in HOST memory out (append then attend, forward.rs:1141-1188)."""

    def __init__(self, layer, seqs, num_q_heads, max_q_len=1, scratch_bytes=64 << 20, device="cuda", extra_blocks=0):
        self.layer, self.seqs, self.hq = layer, seqs, num_q_heads
        hkv = layer.layout.local_kv_heads
        n_tok = len(seqs) * max_q_len
        max_blocks = max(s.num_pages for s in seqs) + extra_blocks   # room for sequences that grow
        self.io = StepIo(len(seqs), n_tok, max_blocks, device=device)
        self.ex = Executor(scratch_bytes, device=device)
        pin = lambda *shape: torch.zeros(*shape, dtype=torch.float16).pin_memory()  # noqa: E731
        self.k_host, self.v_host = pin(n_tok, hkv * 256), pin(n_tok, hkv * 256)
        self.q_host, self.out_host = pin(n_tok, num_q_heads, 256), pin(n_tok, num_q_heads, 256)
        self.k_dev = torch.zeros_like(self.k_host, device=device)
        self.v_dev = torch.zeros_like(self.v_host, device=device)
        self.q_dev = torch.zeros_like(self.q_host, device=device)
        self.out_dev = torch.zeros_like(self.out_host, device=device)
        self.payload_bytes = 2 * self.k_host.numel() * 2 + self.q_host.numel() * 2
        self.h2d_bytes = self.io.nbytes + self.payload_bytes      # upper bound: a full metadata upload
        self.h2d_bytes_total = 0                                  # bytes actually copied by run() so far
        self._graphs = {}
        self.d2h_bytes = self.out_host.numel() * 2
        self._fence = None      # recorded after a step's last use of the pinned buffers when sync=False

    def _capture(self, lib):
        """Two CUDA graphs for the whole step (the reference replays its decode steps the same way,
        crates/warp34-host/src/model/graphs.rs:199-259): the first uploads K, V and Q from pinned
        memory and is launched before the host packs the step's metadata, so that the copies run
        while the CPU works; the second uploads lengths and slots, appends, attends and downloads
        the output.  Block tables are in neither: their changed part is copied between the two."""
        head = self.io.head_words
        b = _DescOnly(self.io.desc)

        def payload():
            self.k_dev.copy_(self.k_host, non_blocking=True)
            self.v_dev.copy_(self.v_host, non_blocking=True)
            self.q_dev.copy_(self.q_host, non_blocking=True)

        def body():
            self.ex.set_stream()
            self.io.dev[:head].copy_(self.io.host[:head], non_blocking=True)
            kv_cache_write(self.ex, self.layer, b, self.k_dev, self.v_dev, lib=lib)
            paged_attention(self.ex, self.layer, b, self.q_dev, self.out_dev, self.hq, lib=lib)
            self.out_host.copy_(self.out_dev, non_blocking=True)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            payload()
            body()                      # warm-up outside the capture (one-time attribute calls)
        torch.cuda.current_stream().wait_stream(side)
        graphs = []
        for fn in (payload, body):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            graphs.append(g)
        self.ex.set_stream()
        return tuple(graphs)

    def run(self, q_lens, sm_scale=1.0 / 16.0, lib=None, sync=True, attend=None, graph=False,
            mask_mode=0, sliding_window=0):
        """sync=False returns while the step is still running: the pinned K / V / Q / metadata
        buffers and out_host belong to the device until the NEXT run() (which waits for this step
        first) or until the caller synchronises the stream."""
        if self._fence is not None:     # the previous step may still be reading the pinned arena
            self._fence.synchronize()
            self._fence = None
        if graph and attend is None:
            # baked into the captured launches (the descriptors are passed by value): the geometry,
            # the softmax scale, the mask mode and the window, and the executor's flags
            key = (id(lib), len(self.seqs), int(sum(q_lens)), int(max(q_lens)), float(sm_scale),
                   int(mask_mode), int(sliding_window), int(self.ex.ex.flags))
            g = self._graphs.get(key)
            if g is not None:
                g[0].replay()           # K, V, Q on their way while the metadata is packed
            self.io.pack(self.seqs, q_lens, sm_scale, mask_mode, sliding_window)
            if g is None:
                self.io.upload(full=True)
                g = self._graphs[key] = self._capture(lib)
                g[0].replay()
            self.meta_bytes_last = self.io.upload(tables_only=True) + 4 * self.io.head_words
            self.h2d_bytes_total += self.meta_bytes_last + self.payload_bytes
            g[1].replay()
            self._finish(sync)
            return self.out_host
        self.io.pack(self.seqs, q_lens, sm_scale, mask_mode, sliding_window)
        self.meta_bytes_last = self.io.upload()
        self.h2d_bytes_total += self.meta_bytes_last + self.payload_bytes
        self.k_dev.copy_(self.k_host, non_blocking=True)
        self.v_dev.copy_(self.v_host, non_blocking=True)
        self.q_dev.copy_(self.q_host, non_blocking=True)
        self.ex.set_stream()
        b = _DescOnly(self.io.desc)
        kv_cache_write(self.ex, self.layer, b, self.k_dev, self.v_dev, lib=lib)
        if attend is not None:
            attend(b)  # e.g. partial attention + all-gather + merge when pages are sharded over GPUs
        else:
            paged_attention(self.ex, self.layer, b, self.q_dev, self.out_dev, self.hq, lib=lib)
        self.out_host.copy_(self.out_dev, non_blocking=True)
        self._finish(sync)
        return self.out_host

    def _finish(self, sync):
        if sync:
            torch.cuda.current_stream().synchronize()
        else:
            self._fence = torch.cuda.Event()
            self._fence.record()
