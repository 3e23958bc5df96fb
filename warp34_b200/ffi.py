"""ctypes bindings of the two C ABIs (include/warp34_b200.h, include/warp34_host.h).

The struct layouts mirror the reference FFI seam
(crates/warp34-kernels/csrc/warp34_cuda.h:50-101, crates/warp34-kernels/src/ffi.rs:15-110).
Loading fails loudly when a library has not been built: there is no fallback path.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(HERE, "lib")

# enums (warp34_cuda.h:20-48)
KV_FORMAT_FP16, KV_FORMAT_BF16, KV_FORMAT_TQ4, KV_FORMAT_Q8_0, KV_FORMAT_FP8_E4M3 = range(5)
KV_TRANSFORM_IDENTITY, KV_TRANSFORM_RADEMACHER_WHT256 = 0, 1
ATTN_MASK_CAUSAL, ATTN_MASK_SYMMETRIC_WINDOW = 0, 1
KV_NAMESPACE_TARGET_FULL_ATTN, KV_NAMESPACE_MTP_FULL_ATTN, KV_NAMESPACE_DFLASH_DRAFT_CTX = 0, 1, 2
POLICY_FP16, POLICY_BF16, POLICY_Q8_0, POLICY_FP8, POLICY_TQ4, POLICY_TQ4_ALL = range(6)

EXEC_FLAG_PRECISE_ATTENTION = 1 << 40
EXEC_FLAG_TCGEN05_VERIFY = 1 << 42
EXEC_FLAG_FAST_ATTENTION = 1 << 43
CUDA_ERROR_INVALID_VALUE = 1
CUDA_ERROR_NOT_SUPPORTED = 801
W34_ERR_INVALID, W34_ERR_EXHAUSTED, W34_ERR_PROTECTED, W34_ERR_CAPACITY = -1, -2, -3, -4


class Exec(C.Structure):
    _fields_ = [("stream", C.c_size_t), ("scratch_ptr", C.c_uint64),
                ("scratch_size", C.c_size_t), ("flags", C.c_uint64)]


class KvLayerLayout(C.Structure):
    _fields_ = [("k_base", C.c_uint64), ("v_base", C.c_uint64),
                ("k_page_stride_bytes", C.c_uint64), ("k_head_stride_bytes", C.c_uint64),
                ("k_token_stride_bytes", C.c_uint64), ("v_page_stride_bytes", C.c_uint64),
                ("v_head_stride_bytes", C.c_uint64), ("v_token_stride_bytes", C.c_uint64),
                ("namespace_id", C.c_int32), ("layer_id", C.c_int32),
                ("local_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("block_size", C.c_int32), ("k_format", C.c_int32), ("v_format", C.c_int32),
                ("k_transform", C.c_int32), ("v_transform", C.c_int32), ("reserved", C.c_int32)]


class AttentionBatch(C.Structure):
    _fields_ = [("query_start_loc", C.c_void_p), ("context_lens_before", C.c_void_p),
                ("seq_lens_after", C.c_void_p), ("block_tables", C.c_void_p),
                ("write_slot_mapping", C.c_void_p), ("valid_token_mask", C.c_void_p),
                ("valid_req_mask", C.c_void_p),
                ("num_reqs", C.c_int32), ("total_tokens", C.c_int32),
                ("max_blocks_per_req", C.c_int32), ("max_q_len", C.c_int32),
                ("max_seq_len", C.c_int32), ("mask_mode", C.c_int32),
                ("sliding_window", C.c_int32), ("sm_scale", C.c_float), ("reserved", C.c_int32)]


class RadixStats(C.Structure):
    _fields_ = [("nodes", C.c_int32), ("cached_pages", C.c_int32),
                ("protected_pages", C.c_int32), ("evictable_pages", C.c_int32)]


class PoolStats(C.Structure):
    _fields_ = [("capacity", C.c_int32), ("free_pages", C.c_int32),
                ("shared_pages", C.c_int32), ("active_pages", C.c_int32)]


class PeerMailboxes(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("max_rows", C.c_int64),
                ("inbox", C.c_uint64 * 8), ("flags", C.c_uint64 * 8),
                ("steps", C.c_uint64), ("status", C.c_uint64),
                ("wait_limit", C.c_uint32), ("reserved", C.c_uint32)]


assert C.sizeof(PeerMailboxes) == 168
assert C.sizeof(Exec) == 32 and C.sizeof(KvLayerLayout) == 104 and C.sizeof(AttentionBatch) == 96

_P = C.POINTER
_KERNEL_SIGS = {
    "warp34_kv_cache_write": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch), C.c_void_p, C.c_void_p]),
    "warp34_kv_cache_write_strided": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                 C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "warp34_paged_attention_f16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                              C.c_void_p, C.c_void_p, C.c_int]),
    "warp34_paged_attention_scalar_f16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                     C.c_void_p, C.c_void_p, C.c_int]),
    "warp34_paged_attention_f16_force_kernel_for_test": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                                    C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "warp34_tq4_kv_cache_write_strided_bf16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                          C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "warp34_tq4_paged_attention_bf16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                   C.c_void_p, C.c_void_p, C.c_int]),
    "warp34_paged_attention_partial_f16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                      C.c_void_p, C.c_void_p, C.c_int]),
    "warp34_paged_attention_merge_shards_f16": (C.c_int, [_P(Exec), C.c_void_p, C.c_int, C.c_int64, C.c_void_p]),
    "warp34_paged_attention_exchange_merge_f16": (C.c_int, [_P(Exec), _P(PeerMailboxes), C.c_void_p, C.c_int64,
                                                             C.c_void_p]),
    "warp34_paged_attention_f16_static_scratch": (C.c_int, [C.c_size_t, _P(KvLayerLayout), _P(AttentionBatch),
                                                             C.c_void_p, C.c_void_p, C.c_int, _P(C.c_size_t)]),
    "warp34_static_scratch_status": (C.c_int, [_P(C.c_int32)]),
    "warp34_qsa_sparse_paged_attn_f16": (C.c_int, [C.c_void_p] * 10 + [C.c_int, C.c_int, C.c_int, C.c_float]),
    "warp34_qsa_sparse_paged_attn_hadamard_f16": (C.c_int, [C.c_void_p] * 10 + [C.c_int, C.c_int, C.c_int, C.c_float]),
    "warp34_bounds_set_pool_pages": (C.c_int, [C.c_int32]),
    "warp34_bounds_report": (C.c_int, [_P(C.c_int32), C.c_int32]),
    "warp34_fused_k_rmsnorm_rope_kv_cache_write_f16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                                                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                                  C.c_float, C.c_float]),
    "warp34_paged_attention_gated_f16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "warp34_apply_attn_output_gate_f16": (C.c_int, [_P(Exec), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                     C.c_int, C.c_int]),
    "warp34_apply_attn_output_gate_hadamard_f16": (C.c_int, [_P(Exec), C.c_void_p, C.c_void_p, C.c_void_p,
                                                              C.c_void_p, C.c_int, C.c_int]),
    "warp34_kv_page_copy": (C.c_int, [_P(Exec), _P(KvLayerLayout), C.c_int32, C.c_int32, C.c_int32]),
    "warp34_paged_attention_scratch_bytes": (C.c_size_t, [_P(KvLayerLayout), _P(AttentionBatch), C.c_int]),
    "warp34_kv_cache_write_bf16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                             C.c_void_p, C.c_void_p]),
    "warp34_kv_cache_write_strided_bf16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                                     C.c_void_p, C.c_void_p, C.c_int]),
    "warp34_paged_attention_bf16": (C.c_int, [_P(Exec), _P(KvLayerLayout), _P(AttentionBatch),
                                              C.c_void_p, C.c_void_p, C.c_int]),
    "warp34_paged_attention_bf16_scratch_bytes": (C.c_size_t, [_P(KvLayerLayout), _P(AttentionBatch), C.c_int]),
    "warp34_b200_version": (C.c_char_p, []),
}

_HOST_SIGS = {
    "w34_kv_format_row_bytes": (C.c_int32, [C.c_int32, C.c_int32]),
    "w34_kv_policy_resolve_layer": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P(C.c_int32)]),
    "w34_kv_policy_bytes_per_token": (C.c_int64, [C.c_int32] * 5),
    "w34_kv_layout_init": (C.c_int32, [_P(KvLayerLayout), C.c_uint64, C.c_uint64, C.c_int32, C.c_int32,
                                        C.c_int32, C.c_int32, C.c_int32, _P(C.c_int32), C.c_int64,
                                        _P(C.c_uint64), _P(C.c_uint64)]),
    "w34_pool_create": (C.c_void_p, [C.c_int32, C.c_int32]),
    "w34_pool_destroy": (None, [C.c_void_p]),
    "w34_pool_num_pages": (C.c_int32, [C.c_void_p]),
    "w34_pool_block_size": (C.c_int32, [C.c_void_p]),
    "w34_pool_free_count": (C.c_int32, [C.c_void_p]),
    "w34_pool_alloc_page": (C.c_int32, [C.c_void_p]),
    "w34_pool_free_page": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_pool_ref_page": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_pool_refcount": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_pool_reset": (None, [C.c_void_p]),
    "w34_pool_truncate": (None, [C.c_void_p, C.c_int32]),
    "w34_pool_shuffle_free_list": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_int32]),
    "w34_pool_get_stats": (None, [C.c_void_p, _P(PoolStats)]),
    "w34_seq_create": (C.c_void_p, [C.c_void_p]),
    "w34_seq_destroy": (None, [C.c_void_p]),
    "w34_seq_attach_prefix": (C.c_int32, [C.c_void_p, _P(C.c_int32), C.c_int32, C.c_int32]),
    "w34_seq_reserve": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_seq_prepare_append": (C.c_int32, [C.c_void_p, _P(C.c_int32), _P(C.c_int32), _P(C.c_int32)]),
    "w34_seq_commit": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_seq_set_committed": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_seq_rollback": (C.c_int32, [C.c_void_p, _P(C.c_int32), C.c_int32]),
    "w34_seqs_reserve_ahead": (C.c_int32, [_P(C.c_void_p), C.c_int32, C.c_int32]),
    "w34_seqs_commit_and_rollback": (C.c_int32, [_P(C.c_void_p), _P(C.c_int32), C.c_int32, _P(C.c_int32), C.c_int32]),
    "w34_seq_committed_len": (C.c_int32, [C.c_void_p]),
    "w34_seq_num_pages": (C.c_int32, [C.c_void_p]),
    "w34_seq_protected_pages": (C.c_int32, [C.c_void_p]),
    "w34_seq_pages": (_P(C.c_int32), [C.c_void_p]),
    "w34_seq_set_pages_unchecked": (C.c_int32, [C.c_void_p, _P(C.c_int32), C.c_int32, C.c_int32]),
    "w34_radix_create": (C.c_void_p, [C.c_void_p]),
    "w34_radix_destroy": (None, [C.c_void_p]),
    "w34_radix_match_prefix": (C.c_int32, [C.c_void_p, _P(C.c_int32), C.c_int32, _P(C.c_int32), C.c_int32,
                                            _P(C.c_int32), _P(C.c_int32)]),
    "w34_radix_lock": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_radix_unlock": (C.c_int32, [C.c_void_p, C.c_int32]),
    "w34_radix_insert": (C.c_int32, [C.c_void_p, _P(C.c_int32), C.c_int32, _P(C.c_int32), C.c_int32, _P(C.c_int32)]),
    "w34_radix_evict": (C.c_int32, [C.c_void_p, C.c_int32, _P(C.c_int32), C.c_int32]),
    "w34_radix_get_stats": (None, [C.c_void_p, _P(RadixStats)]),
    "w34_radix_sanity_check": (C.c_int32, [C.c_void_p]),
    "w34_build_step_metadata": (C.c_int32, [_P(C.c_void_p), _P(C.c_int32), C.c_int32, C.c_int32] +
                                [_P(C.c_int32)] * 7),
    "w34_build_step_metadata_delta": (C.c_int32, [_P(C.c_void_p), _P(C.c_int32), C.c_int32, C.c_int32] +
                                      [_P(C.c_int32)] * 9),
}


def _bind(lib, sigs):
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)  # AttributeError when a declared symbol is missing
        fn.restype = res
        fn.argtypes = args
    return lib


def _load(name, sigs):
    path = os.path.join(LIB_DIR, name)
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m warp34_b200.build` "
            "(there is no CPU or eager fallback for this path)")
    return _bind(C.CDLL(path), sigs)


_kernels = None
_host = None


def kernels():
    """The CUDA library (libwarp34_b200.so)."""
    global _kernels
    if _kernels is None:
        _kernels = _load("libwarp34_b200.so", _KERNEL_SIGS)
    return _kernels


def host():
    """The host page-manager library (libwarp34_host.so)."""
    global _host
    if _host is None:
        _host = _load("libwarp34_host.so", _HOST_SIGS)
    return _host


def bind_kernel_abi(path):
    """Binds another library that exports the same kernel ABI (used by tests for the
    reference build)."""
    lib = C.CDLL(path)
    for name, (res, args) in _KERNEL_SIGS.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
    return lib
