"""The C ABI: struct sizes, enum values and exported symbols.

Mirrors the reference's own ABI checks (crates/warp34-kernels/src/lib.rs:27-81: sizes 32 / 104 /
96 and the enum constants)."""
import ctypes as C
import os
import re

from warp34_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions(header):
    txt = open(os.path.join(ROOT, "include", header)).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    names = re.findall(r"\b(w34_\w+|warp34_\w+)\s*\(", txt)
    return sorted(set(names))


def test_struct_sizes_match_reference_seam():
    assert C.sizeof(ffi.Exec) == 32
    assert C.sizeof(ffi.KvLayerLayout) == 104
    assert C.sizeof(ffi.AttentionBatch) == 96
    assert ffi.KvLayerLayout.k_token_stride_bytes.offset == 32
    assert ffi.KvLayerLayout.namespace_id.offset == 64
    assert ffi.AttentionBatch.num_reqs.offset == 56
    assert ffi.AttentionBatch.sm_scale.offset == 84


def test_enum_values():
    assert (ffi.KV_FORMAT_FP16, ffi.KV_FORMAT_BF16, ffi.KV_FORMAT_TQ4, ffi.KV_FORMAT_Q8_0,
            ffi.KV_FORMAT_FP8_E4M3) == (0, 1, 2, 3, 4)
    assert (ffi.KV_TRANSFORM_IDENTITY, ffi.KV_TRANSFORM_RADEMACHER_WHT256) == (0, 1)
    assert (ffi.ATTN_MASK_CAUSAL, ffi.ATTN_MASK_SYMMETRIC_WINDOW) == (0, 1)
    hdr = open(os.path.join(ROOT, "include", "warp34_b200.h")).read()
    for name, val in (("WARP34_KV_FORMAT_TQ4", 2), ("WARP34_KV_TRANSFORM_RADEMACHER_WHT256", 1),
                      ("WARP34_KV_FORMAT_FP8_E4M3", 4), ("WARP34_ATTN_MASK_SYMMETRIC_WINDOW", 1)):
        assert re.search(rf"{name}\s*=\s*{val}\b", hdr), name


def test_kernel_library_exports_every_declared_symbol(native_libs):
    kernels, _ = native_libs
    declared = _declared_functions("warp34_b200.h")
    assert "warp34_kv_cache_write_strided" in declared and "warp34_paged_attention_f16" in declared
    for name in declared:
        assert hasattr(kernels, name), f"{name} declared in warp34_b200.h but not exported"
    assert kernels.warp34_b200_version().decode().endswith("sm_100a")


def test_bounds_checked_build_exports_the_same_abi(native_libs):
    """The -DW34_BOUNDS build is the same library with range checks compiled in: same symbols; the
    regular build answers the two bounds calls with 801 (host-only returns, no GPU needed)."""
    import ctypes as C
    from warp34_b200 import build, ffi
    blib = ffi.bind_kernel_abi(build.build_bounds())
    for name in _declared_functions("warp34_b200.h"):
        assert hasattr(blib, name), f"{name} missing from the bounds-checked build"
    out = (C.c_int32 * 4)()
    assert native_libs[0].warp34_bounds_set_pool_pages(4) == 801
    assert native_libs[0].warp34_bounds_report(out, 0) == 801


def test_host_library_exports_every_declared_symbol(native_libs):
    _, host = native_libs
    declared = [n for n in _declared_functions("warp34_host.h") if n.startswith("w34_")]
    assert len(declared) > 25
    for name in declared:
        assert hasattr(host, name), f"{name} declared in warp34_host.h but not exported"


def test_argument_validation_needs_no_gpu(native_libs):
    """Null descriptors are rejected with cudaErrorInvalidValue before any CUDA call
    (op_kv_cache.cu:836-838, op_paged_attn.cu:1270-1272)."""
    kernels, _ = native_libs
    assert kernels.warp34_kv_cache_write_strided(None, None, None, None, None, 0, 0) == 1
    assert kernels.warp34_paged_attention_f16(None, None, None, None, None, 16) == 1
    assert kernels.warp34_kv_cache_write(None, None, None, None, None) == 1
    ex, lay, b = ffi.Exec(), ffi.KvLayerLayout(), ffi.AttentionBatch()
    # empty batch returns 0 without a launch (op_kv_cache.cu:843, op_paged_attn.cu:1277)
    lay.local_kv_heads = 4
    one = C.c_int(0)
    p = C.addressof(one)
    assert kernels.warp34_kv_cache_write_strided(C.byref(ex), C.byref(lay), C.byref(b), p, p, 1024, 1024) == 0
    assert kernels.warp34_paged_attention_f16(C.byref(ex), C.byref(lay), C.byref(b), p, p, 16) == 0
    # non-TQ4 layouts are refused loudly
    b.total_tokens = 1
    lay.head_dim, lay.block_size, lay.k_format, lay.v_format = 256, 16, ffi.KV_FORMAT_FP16, ffi.KV_FORMAT_FP16
    assert kernels.warp34_kv_cache_write_strided(C.byref(ex), C.byref(lay), C.byref(b), p, p, 1024, 1024) == 801
    # a row stride below heads * head_dim is invalid (op_kv_cache.cu:844-845)
    lay.k_format = lay.v_format = ffi.KV_FORMAT_TQ4
    lay.k_transform = lay.v_transform = ffi.KV_TRANSFORM_RADEMACHER_WHT256
    assert kernels.warp34_kv_cache_write_strided(C.byref(ex), C.byref(lay), C.byref(b), p, p, 512, 1024) == 1
    # the query-sparse entry points check their arguments like the reference's launcher (op_qsa.cu:1464-1470)
    qsa = kernels.warp34_qsa_sparse_paged_attn_f16
    assert qsa(None, p, None, C.addressof(lay), p, p, p, p, None, p, 1, 8, 4, 0.0625) == 1          # no exec
    assert qsa(C.addressof(ex), p, None, C.addressof(lay), p, p, p, p, None, p, 1, 6, 4, 0.0625) == 1   # 6 q heads / 4 kv heads
    assert qsa(C.addressof(ex), p, None, C.addressof(lay), p, p, p, p, None, p, -1, 8, 4, 0.0625) == 1  # negative token count
    lay.k_format = ffi.KV_FORMAT_FP16
    lay.k_base = lay.v_base = 4096
    assert qsa(C.addressof(ex), p, None, C.addressof(lay), p, p, p, p, None, p, 1, 8, 4, 0.0625) == 801  # FP16 rows
    lay.k_format = ffi.KV_FORMAT_TQ4
    lay.k_token_stride_bytes = lay.v_token_stride_bytes = 132
    lay.k_head_stride_bytes = lay.v_head_stride_bytes = 2112
    lay.k_page_stride_bytes = lay.v_page_stride_bytes = 8448
    assert qsa(C.addressof(ex), p, None, C.addressof(lay), p, p, p, p, None, p, 0, 8, 4, 0.0625) == 0    # no tokens: no launch
