// Shared device helpers for the TQ4 KV path: format tables, the 256-point
// Walsh-Hadamard rotation on one warp, and small PTX wrappers.
//
// TQ4 row (head_dim 256) = two 66-byte blocks {fp16 d; u8 qs[64]}; block b covers
// rotated coordinates [128 b, 128 b + 128); qs[i] = code[2i] | code[2i+1] << 4.
// (reference format: crates/warp34-kernels/csrc/tq/tq4_kv_common.cuh:21-26)
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/warp34_b200.h"
#include "tq4_tables.h"

namespace w34 {

constexpr int kHeadDim = 256;
constexpr int kPageTokens = 16;
constexpr int kTq4RowBytes = 132;
constexpr int kTq4BlockBytes = 66;
constexpr int kTq4PageHeadBytes = kPageTokens * kTq4RowBytes;  // 2112, a multiple of 16

__device__ __constant__ uint32_t c_centroid_bits[16] = W34_TQ4_CENTROID_BITS;
__device__ __constant__ uint32_t c_boundary_bits[15] = W34_TQ4_BOUNDARY_BITS;
__device__ __constant__ uint32_t c_sign_mask[8] = W34_TQ4_SIGN_MASK;

__device__ __forceinline__ float tq4_centroid(int i) { return __uint_as_float(c_centroid_bits[i]); }
__device__ __forceinline__ float tq4_boundary(int i) { return __uint_as_float(c_boundary_bits[i]); }

// x with the sign bit flipped where the diagonal entry for `col` is -1 (exact).
__device__ __forceinline__ float apply_sign(float x, int col) {
    const uint32_t neg = (c_sign_mask[col >> 5] >> (col & 31)) & 1u;
    return __uint_as_float(__float_as_uint(x) ^ (neg << 31));
}

// 256-point normalised WHT on one warp, element col = lane + 32 j held in v[j].
// Stage order h = 1..128, every stage computes (lower + upper, lower - upper), final
// scale 1/16: the same operation order as the reference's wht256_warp
// (tq4_kv_common.cuh:75-107), hence the same fp32 bits.
__device__ __forceinline__ void wht256_lanes(float (&v)[8], int lane) {
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
        const bool upper = (lane & h) != 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float o = __shfl_xor_sync(0xffffffffu, v[j], h);
            v[j] = upper ? __fsub_rn(o, v[j]) : __fadd_rn(v[j], o);
        }
    }
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if ((j & s) == 0) {
                const float a = v[j], b = v[j | s];
                v[j] = __fadd_rn(a, b);
                v[j | s] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], 0.0625f);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Binary search of tok in query_start_loc[0..num_reqs]; returns -1 when tok is outside.
__device__ __forceinline__ int find_request(const int32_t* __restrict__ qsl, int num_reqs, int tok) {
    if (num_reqs <= 0 || tok < qsl[0] || tok >= qsl[num_reqs]) return -1;
    int lo = 0, hi = num_reqs;  // invariant: qsl[lo] <= tok < qsl[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (qsl[mid] <= tok) lo = mid; else hi = mid;
    }
    return lo;
}

// ---- bounds-checked build (-DW34_BOUNDS) ----------------------------------------------------------
// Every index into a block table, every page id read from one and every write slot is range-checked
// before an address is formed from it.  The first violation is recorded in a device word (what, the
// value, its limit; a count of all violations beside it) that warp34_bounds_report() reads, and the
// access goes to entry 0 / page 0 / is skipped instead: nothing traps, the context stays usable.  The
// layer descriptor does not carry the pool's page count, so the host states it once with
// warp34_bounds_set_pool_pages().  Without the define these helpers cost nothing.
enum { kBoundsBlockIndex = 1, kBoundsPageId = 2, kBoundsWriteSlot = 3 };
enum { kInAppend = 1, kInScalar = 2, kInStream = 3, kInTeam = 4, kInPrefillExact = 5, kInPrefillTc = 6,
       kInBf16 = 7, kInKv8 = 8, kInSparse = 9 };
#ifdef W34_BOUNDS
struct BoundsWord { int what, value, limit, count; };
static __device__ BoundsWord g_bounds;       // one per translation unit; the report merges them
static __device__ int g_bounds_pool_pages;   // 0: not stated, page ids and slots are not checked
__device__ __forceinline__ bool bounds_ok(int v, int limit, int what, int where) {
    if ((unsigned)v < (unsigned)limit) return true;
    if (atomicAdd(&g_bounds.count, 1) == 0) {
        g_bounds.value = v;
        g_bounds.limit = limit;
        __threadfence();
        g_bounds.what = what | (where << 8);
    }
    return false;
}
__device__ __forceinline__ int block_table_page(const int32_t* __restrict__ blocks, int idx, int max_blocks, int where) {
    if (!bounds_ok(idx, max_blocks, kBoundsBlockIndex, where)) idx = 0;
    int page = blocks[idx];
    const int pages = g_bounds_pool_pages;
    if (pages > 0 && !bounds_ok(page, pages, kBoundsPageId, where)) page = 0;
    return page;
}
// false: the slot points outside the pool and the row must not be written
__device__ __forceinline__ bool write_slot_ok(int slot, int where) {
    const int pages = g_bounds_pool_pages;
    return pages <= 0 || bounds_ok(slot, pages * kPageTokens, kBoundsWriteSlot, where);
}
// a page id that did not come from a block table (a selected-block list)
__device__ __forceinline__ int pool_page(int page, int where) {
    const int pages = g_bounds_pool_pages;
    return (pages > 0 && !bounds_ok(page, pages, kBoundsPageId, where)) ? 0 : page;
}
#define W34_BOUNDS_HOST_HOOKS(tag)                                                                  \
    int bounds_fetch_##tag(int32_t* out, int reset) {                                               \
        BoundsWord w;                                                                               \
        if (cudaMemcpyFromSymbol(&w, g_bounds, sizeof(w)) != cudaSuccess) return 1;                 \
        out[0] = w.what; out[1] = w.value; out[2] = w.limit; out[3] = w.count;                      \
        if (reset) { w = BoundsWord{0, 0, 0, 0}; cudaMemcpyToSymbol(g_bounds, &w, sizeof(w)); }     \
        return 0;                                                                                   \
    }                                                                                               \
    int bounds_set_pages_##tag(int pages) {                                                         \
        return cudaMemcpyToSymbol(g_bounds_pool_pages, &pages, sizeof(int)) == cudaSuccess ? 0 : 1; \
    }
#else
__device__ __forceinline__ int block_table_page(const int32_t* __restrict__ blocks, int idx, int, int) { return blocks[idx]; }
__device__ __forceinline__ bool write_slot_ok(int, int) { return true; }
__device__ __forceinline__ int pool_page(int page, int) { return page; }
#define W34_BOUNDS_HOST_HOOKS(tag)
#endif

}  // namespace w34
