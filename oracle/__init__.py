"""TEST INFRASTRUCTURE ONLY: ctypes loader of the CPU oracle (oracle/tq4_oracle.c) and of the
reference's own kernels when oracle/_ref/libwarp34_ref.so has been built.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may import
this package; the product (warp34_b200/) never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def build():
    subprocess.run(["make", "-s", "-C", HERE, "liboracle.so"], check=True)
    return os.path.join(HERE, "liboracle.so")


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        vp, i = C.c_void_p, C.c_int
        L.w34o_kv_cache_write_strided.restype = i
        L.w34o_kv_cache_write_strided.argtypes = [vp, vp, vp, vp, i, i, i]
        L.w34o_paged_attention_f16.restype = i
        L.w34o_paged_attention_f16.argtypes = [vp, vp, vp, vp, i, i]
        L.w34o_paged_attention_partial.restype = i
        L.w34o_paged_attention_partial.argtypes = [vp, vp, vp, vp, i, i]
        L.w34o_merge_shards.restype = i
        L.w34o_merge_shards.argtypes = [vp, i, C.c_long, vp]
        L.w34o_tq4_encode_row.restype = None
        L.w34o_tq4_encode_row.argtypes = [vp, vp, vp, vp]
        L.w34o_tq4_decode_row.restype = None
        L.w34o_tq4_decode_row.argtypes = [vp, vp]
        L.w34o_wht256.restype = None
        L.w34o_wht256.argtypes = [vp]
        L.w34o_kv8_encode_row.restype = None
        L.w34o_kv8_encode_row.argtypes = [vp, i, vp]
        L.w34o_kv8_decode_row.restype = None
        L.w34o_kv8_decode_row.argtypes = [vp, i, vp]
        for name in ("w34o_centroid", "w34o_boundary", "w34o_sign"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [i]
        L.w34o_half_to_float.restype = C.c_float
        L.w34o_half_to_float.argtypes = [C.c_uint16]
        L.w34o_float_to_half.restype = C.c_uint16
        L.w34o_float_to_half.argtypes = [C.c_float]
        _lib = L
    return _lib


def ref_lib_path():
    p = os.path.join(HERE, "_ref", "libwarp34_ref.so")
    return p if os.path.exists(p) else None


def encode_row(x_f16):
    """x_f16: uint16[256] (fp16 bits). Returns (row132 uint8, ambiguous uint8[256], rotated f32[256])."""
    x = np.ascontiguousarray(x_f16, dtype=np.uint16)
    out = np.zeros(132, np.uint8)
    amb = np.zeros(256, np.uint8)
    rot = np.zeros(256, np.float32)
    lib().w34o_tq4_encode_row(x.ctypes.data, out.ctypes.data, amb.ctypes.data, rot.ctypes.data)
    return out, amb, rot


def decode_row(row132):
    r = np.ascontiguousarray(row132, dtype=np.uint8)
    out = np.zeros(256, np.float32)
    lib().w34o_tq4_decode_row(r.ctypes.data, out.ctypes.data)
    return out


def kv_cache_write(layout, batch_host, k_f16, v_f16, k_stride, v_stride, nthreads=1):
    """layout.k_base / v_base must point to HOST slabs; batch_host holds host pointers."""
    return lib().w34o_kv_cache_write_strided(C.addressof(layout), C.addressof(batch_host),
                                             k_f16.ctypes.data, v_f16.ctypes.data, k_stride, v_stride,
                                             nthreads)


def paged_attention(layout, batch_host, q_f16, out_f16, num_q_heads, nthreads=1):
    return lib().w34o_paged_attention_f16(C.addressof(layout), C.addressof(batch_host),
                                          q_f16.ctypes.data, out_f16.ctypes.data, num_q_heads, nthreads)


def paged_attention_partial(layout, batch_host, q_f16, triples_f32, num_q_heads, nthreads=1):
    return lib().w34o_paged_attention_partial(C.addressof(layout), C.addressof(batch_host), q_f16.ctypes.data,
                                              triples_f32.ctypes.data, num_q_heads, nthreads)


def merge_shards(triples_f32, out_f16):
    shards, rows = triples_f32.shape[0], triples_f32[0].size // 258
    return lib().w34o_merge_shards(triples_f32.ctypes.data, shards, rows, out_f16.ctypes.data)
