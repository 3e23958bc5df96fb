// Append for the unrotated 8-bit boundary-layer formats, head_dim 256.  Included by tq4_append.cu
// (same -use_fast_math build as the reference, so '/' and roundf() lower alike).
//
// Replaces the Q8_0 and FP8_E4M3 branches of the reference's write_kv_row
// (crates/warp34-kernels/csrc/ops/op_kv_cache.cu:32-151) for the identity transform, which is
// what every cache policy of the reference pairs with these formats
// (crates/warp34-host/src/cache.rs:62-108: the default policy stores the last four
// full-attention layers as FP8 E4M3 on sm_89 and later, as Q8_0 before).
//
//   Q8_0      272 B row = 4 x { float d; int8 qs[64] }, block sb holds columns [64 sb, 64 sb + 64):
//             d = max|x| / 127, q = clamp(roundf(x / d), -127, 127); d <= 1e-12 stores zeros.
//   FP8_E4M3  264 B row = { uint8 qs[256]; float d0; float d1 }, d_h = max|x| over half h / 448,
//             qs = e4m3(x / d_h) with saturation; d <= 1e-30 stores zeros.
//
// One warp per (token, kv head): its K row and its V row.
#pragma once

#include <cuda_fp8.h>

namespace w34 {

constexpr int kQ8BlockBytes = 68;
constexpr int kQ8RowBytes = 4 * kQ8BlockBytes;   // 272
constexpr int kFp8RowBytes = kHeadDim + 8;       // 264

__device__ __forceinline__ float warp_max_all(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// One row from eight fp16 values per lane (lane holds columns [8 lane, 8 lane + 8)).  Maxima do not depend
// on the order they are taken in and every code depends on its own value and the scale alone, so the bytes
// are those of kv8_encode_row_by_element() below.
__device__ __forceinline__ void kv8_encode_row_vec(const uint4 raw, uint8_t* dst, int format, int lane) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        v[2 * j] = __half2float(__ushort_as_half((unsigned short)(w[j] & 0xffffu)));
        v[2 * j + 1] = __half2float(__ushort_as_half((unsigned short)(w[j] >> 16)));
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    if (format == WARP34_KV_FORMAT_Q8_0) {
        // block sb = lane >> 3: columns [64 sb, 64 sb + 64) sit in eight lanes
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = amax / 127.0f;
        const float inv_d = (d > 1e-12f) ? (1.0f / d) : 0.0f;
        uint8_t* blk = dst + (lane >> 3) * kQ8BlockBytes;
        if ((lane & 7) == 0) *reinterpret_cast<float*>(blk) = d;
        uint32_t packed[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float q = fminf(127.0f, fmaxf(-127.0f, roundf(v[j] * inv_d)));
            packed[j >> 2] |= ((uint32_t)(int)q & 0xffu) << (8 * (j & 3));
        }
        uint32_t* qs = reinterpret_cast<uint32_t*>(blk + 4 + 8 * (lane & 7));   // 4-byte aligned like the row
        qs[0] = packed[0];
        qs[1] = packed[1];
        return;
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = amax * (1.0f / 448.0f);
    const float inv_d = (d > 1e-30f) ? (1.0f / d) : 0.0f;
    if (lane == 0) *reinterpret_cast<float*>(dst + kHeadDim) = d;
    if (lane == 16) *reinterpret_cast<float*>(dst + kHeadDim + 4) = d;
    const uint32_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv_d, v[1] * inv_d), __NV_SATFINITE, __NV_E4M3);
    const uint32_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv_d, v[3] * inv_d), __NV_SATFINITE, __NV_E4M3);
    const uint32_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(v[4] * inv_d, v[5] * inv_d), __NV_SATFINITE, __NV_E4M3);
    const uint32_t p3 = __nv_cvt_float2_to_fp8x2(make_float2(v[6] * inv_d, v[7] * inv_d), __NV_SATFINITE, __NV_E4M3);
    uint32_t* q = reinterpret_cast<uint32_t*>(dst + 8 * lane);
    if ((reinterpret_cast<uintptr_t>(q) & 7u) == 0u) {
        *reinterpret_cast<uint2*>(q) = make_uint2(p0 | (p1 << 16), p2 | (p3 << 16));
    } else {
        q[0] = p0 | (p1 << 16);
        q[1] = p2 | (p3 << 16);
    }
}

// The same row read element by element: any 2-byte-aligned source.
__device__ __forceinline__ void kv8_encode_row_by_element(const __half* src_row, uint8_t* dst, int format, int lane) {
    if (format == WARP34_KV_FORMAT_Q8_0) {
        // lane holds columns lane + 32 j; block sb takes j = 2 sb and 2 sb + 1
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __half2float(src_row[32 * j + lane]);
#pragma unroll
        for (int sb = 0; sb < 4; ++sb) {
            const float x0 = v[2 * sb], x1 = v[2 * sb + 1];
            const float amax = warp_max_all(fmaxf(fabsf(x0), fabsf(x1)));
            const float d = amax / 127.0f;
            const float inv_d = (d > 1e-12f) ? (1.0f / d) : 0.0f;
            uint8_t* blk = dst + sb * kQ8BlockBytes;
            if (lane == 0) *reinterpret_cast<float*>(blk) = d;
            const float q0 = fminf(127.0f, fmaxf(-127.0f, roundf(x0 * inv_d)));
            const float q1 = fminf(127.0f, fmaxf(-127.0f, roundf(x1 * inv_d)));
            reinterpret_cast<int8_t*>(blk + 4)[lane] = (int8_t)q0;
            reinterpret_cast<int8_t*>(blk + 4)[lane + 32] = (int8_t)q1;
        }
        return;
    }
    // FP8 E4M3: lane holds columns [8 lane, 8 lane + 8); lanes 0..15 are half 0, 16..31 half 1
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __half2float(src_row[8 * lane + j]);
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = amax * (1.0f / 448.0f);
    const float inv_d = (d > 1e-30f) ? (1.0f / d) : 0.0f;
    if (lane == 0) *reinterpret_cast<float*>(dst + kHeadDim) = d;
    if (lane == 16) *reinterpret_cast<float*>(dst + kHeadDim + 4) = d;
    const uint32_t p0 = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv_d, v[1] * inv_d), __NV_SATFINITE, __NV_E4M3);
    const uint32_t p1 = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv_d, v[3] * inv_d), __NV_SATFINITE, __NV_E4M3);
    const uint32_t p2 = __nv_cvt_float2_to_fp8x2(make_float2(v[4] * inv_d, v[5] * inv_d), __NV_SATFINITE, __NV_E4M3);
    const uint32_t p3 = __nv_cvt_float2_to_fp8x2(make_float2(v[6] * inv_d, v[7] * inv_d), __NV_SATFINITE, __NV_E4M3);
    uint32_t* q = reinterpret_cast<uint32_t*>(dst + 8 * lane);   // rows are 4-byte aligned (checked on the host)
    q[0] = p0 | (p1 << 16);
    q[1] = p2 | (p3 << 16);
}

// One warp per (token, kv head): its K row and its V row, both loads in flight before either is encoded.
// ALIGNED: the host has checked that every source row starts on a 16-byte boundary (base pointers and row
// strides), so the kernel holds the 128-bit path alone.
template <bool ALIGNED>
__global__ void __launch_bounds__(128) kv8_append_kernel(const AppendParams p) {
    const int lane = threadIdx.x & 31;
    const int heads = p.layout.local_kv_heads;
    const long long th_ll = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (2 * th_ll >= p.total_rows) return;
    const int th = (int)th_ll;
    const int tok = th / heads, head = th - tok * heads;
    if (p.batch.valid_token_mask != nullptr && p.batch.valid_token_mask[tok] == 0) return;
    if (p.batch.valid_req_mask != nullptr && p.batch.query_start_loc != nullptr && p.batch.num_reqs > 0) {
        const int req = find_request(p.batch.query_start_loc, p.batch.num_reqs, tok);
        if (req < 0 || p.batch.valid_req_mask[req] == 0) return;
    }
    const int slot = p.batch.write_slot_mapping[tok];
    if (slot < 0 || !write_slot_ok(slot, kInKv8)) return;
    const int page = slot >> 4, off = slot & 15;
    const __half* ksrc = reinterpret_cast<const __half*>(p.k_in + (size_t)tok * p.k_row_stride + (size_t)head * kHeadDim);
    const __half* vsrc = reinterpret_cast<const __half*>(p.v_in + (size_t)tok * p.v_row_stride + (size_t)head * kHeadDim);
    uint8_t* kdst = (uint8_t*)(uintptr_t)p.layout.k_base + (size_t)page * p.layout.k_page_stride_bytes +
                    (size_t)head * p.layout.k_head_stride_bytes + (size_t)off * p.layout.k_token_stride_bytes;
    uint8_t* vdst = (uint8_t*)(uintptr_t)p.layout.v_base + (size_t)page * p.layout.v_page_stride_bytes +
                    (size_t)head * p.layout.v_head_stride_bytes + (size_t)off * p.layout.v_token_stride_bytes;
    // Rows that start on a 16-byte boundary (the usual case: contiguous or packed activations) are read
    // with one 128-bit load per lane.
    if (ALIGNED || ((reinterpret_cast<uintptr_t>(ksrc) | reinterpret_cast<uintptr_t>(vsrc)) & 15u) == 0u) {
        const uint4 rk = *reinterpret_cast<const uint4*>(ksrc + 8 * lane);
        const uint4 rv = *reinterpret_cast<const uint4*>(vsrc + 8 * lane);
        kv8_encode_row_vec(rk, kdst, p.layout.k_format, lane);
        kv8_encode_row_vec(rv, vdst, p.layout.v_format, lane);
        return;
    }
    if (!ALIGNED) {
        kv8_encode_row_by_element(ksrc, kdst, p.layout.k_format, lane);
        kv8_encode_row_by_element(vsrc, vdst, p.layout.v_format, lane);
    }
}

// Formats this file handles: both sides 8-bit and unrotated.
static bool kv8_layout_ok(const warp34_kv_layer_layout* l) {
    const bool k8 = l->k_format == WARP34_KV_FORMAT_Q8_0 || l->k_format == WARP34_KV_FORMAT_FP8_E4M3;
    const bool v8 = l->v_format == WARP34_KV_FORMAT_Q8_0 || l->v_format == WARP34_KV_FORMAT_FP8_E4M3;
    return k8 && v8 && l->head_dim == kHeadDim && l->block_size == kPageTokens &&
           l->k_transform == WARP34_KV_TRANSFORM_IDENTITY && l->v_transform == WARP34_KV_TRANSFORM_IDENTITY;
}

}  // namespace w34
