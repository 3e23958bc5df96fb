// TQ4 quantize-and-append for sm_100a.
//
// Replaces kv_cache_write_kernel / write_kv_row of the reference
// (crates/warp34-kernels/csrc/ops/op_kv_cache.cu:152-218, :325-368) for
// head_dim 256, TQ4 storage and the sign-diagonal + WHT-256 rotation.
//
// Per (token, kv head) and per K / V row:
//   v = sign * x  ->  WHT-256  ->  per 128-half: s = sum v^2,
//   inv = 0.70710678 * rsqrt(s)  ->  code = #{i : v*inv > boundary_i}
//   ->  d = sum(v * c[code]) / sum(c[code]^2)  ->  fp16(d) + 64 packed bytes.
//
// The packed bytes and scales are bit-identical to the reference because every
// fp32 operation is issued in the same association order:
//   * the WHT is the same butterfly network (stage order 1..128);
//   * each of the 24 sums is the reference's 32-lane xor butterfly (levels over
//     column bits 4,3,2,1,0) followed by a sequential sum over the four
//     32-column groups of a half.
// The thread layout is different: 8 lanes hold one row (column bits 0..2 select
// the lane, bits 3..7 the register), so the first two butterfly levels and five
// of the eight WHT stages are register-only, and the three cross-lane levels of
// the eight per-group sums are done with a halving exchange (7 shuffles instead
// of 40 per quantity).  A warp encodes 4 rows at once.
//
// This translation unit is compiled with -use_fast_math like the reference
// build (crates/warp34-kernels/build.rs:56-59), so rsqrtf() and '/' lower to the
// same approximate instructions and denormals flush the same way.
#include "tq4_common.cuh"

#include <cuda_bf16.h>

namespace w34 {

// The reference computes warp_reduce_sum(a * b): the product is rounded, then summed by the
// butterfly, and nvcc does not contract the butterfly's first add with the product into an fma
// (all eight contracted / uncontracted combinations of the three sums were compared with the
// reference kernels built for sm_100a: only "none contracted" is bit-identical).  Products and adds
// below are therefore explicit __fmul_rn / __fadd_rn.

// code = #{i : rv > boundary_i} for the 15 ascending, symmetric boundaries (b[7] = 0), by a
// three-level binary search on |rv| in the integer domain.  bpos[k] = bits(boundary[8 + k]) > 0.
// For rv > 0 all of b[0..7] are below rv and the code is 8 + #{k : |rv| > B_k}; for rv <= 0 none
// of b[7..14] is, rv > -B  <=>  |rv| < B, and the code is 7 - #{k : |rv| >= B_k}.  Positive floats
// order like their bit patterns and ">= B" is "> B - 1 ulp", so both cases count
// #{k : bits(|rv|) + (rv > 0 ? 0 : 1) > bits(B_k)}.  NaN gives 0 and -0 gives 7, as the
// comparison chain does.
__device__ __forceinline__ int tq4_bucket(float rv, const uint32_t (&bpos)[7]) {
    const bool pos = rv > 0.0f;
    const uint32_t x = (__float_as_uint(rv) & 0x7fffffffu) + (pos ? 0u : 1u);
    const bool c1 = x > bpos[3];
    const bool c2 = x > (c1 ? bpos[5] : bpos[1]);
    const uint32_t t3 = c1 ? (c2 ? bpos[6] : bpos[4]) : (c2 ? bpos[2] : bpos[0]);
    const int c = (c1 ? 4 : 0) + (c2 ? 2 : 0) + ((x > t3) ? 1 : 0);
    return pos ? (8 + c) : (7 - c);
}

// One level of the halving exchange: the lane keeps the N/2 values whose index bit
// matches its own lane bit and adds the partner's copies of the same indices.
template <int N>
__device__ __forceinline__ void halve_level(float (&x)[8], int lane_bit_set, int xor_mask) {
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
        const float keep = lane_bit_set ? x[i + N / 2] : x[i];
        const float send = lane_bit_set ? x[i] : x[i + N / 2];
        const float got = __shfl_xor_sync(0xffffffffu, send, xor_mask);
        x[i] = __fadd_rn(keep, got);
    }
}

// Cross-lane part of eight butterfly sums at once.  In: x[j] = this lane's partial of
// group j after the register-only levels.  Out: total of group (lane & 7) for the
// lane's row, levels applied in the order column bit 2, 1, 0.
__device__ __forceinline__ float group_totals(float (&x)[8], int sub) {
    halve_level<8>(x, sub & 4, 4);
    halve_level<4>(x, sub & 2, 2);
    halve_level<2>(x, sub & 1, 1);
    return x[0];
}

// Sequential sum (((0 + t0) + t1) + t2) + t3 of the group totals held by lanes base+g0..g0+3.
__device__ __forceinline__ float seq4(float t, int lane_base, int g0) {
    // The reference starts from 0.0f (0 + (-0) = +0 matters for all-zero rows).
    float s = __fadd_rn(0.0f, __shfl_sync(0xffffffffu, t, lane_base + g0));
    s = __fadd_rn(s, __shfl_sync(0xffffffffu, t, lane_base + g0 + 1));
    s = __fadd_rn(s, __shfl_sync(0xffffffffu, t, lane_base + g0 + 2));
    s = __fadd_rn(s, __shfl_sync(0xffffffffu, t, lane_base + g0 + 3));
    return s;
}

// Register-only levels (column bits 4 then 3) of the butterfly over products a*b for one
// group; r indexes column bits 3,4 as (bit3 = r & 1, bit4 = r >> 1).
__device__ __forceinline__ void reg_levels(const float (&a)[4], const float (&b)[4], float& lo, float& hi) {
    float p[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) p[r] = __fmul_rn(a[r], b[r]);
    lo = __fadd_rn(__fadd_rn(p[0], p[2]), __fadd_rn(p[1], p[3]));
    hi = lo;
}

struct AppendParams {
    warp34_kv_layer_layout layout;
    warp34_attention_batch batch;
    const uint16_t* k_in;   // fp16 or bf16 bits, see the kernel's template argument
    const uint16_t* v_in;
    int k_row_stride;
    int v_row_stride;
    int total_rows;  // total_tokens * local_kv_heads * 2
    // producer fused in front of the K rows (PRODUCER builds only)
    const uint16_t* k_norm_w;   // fp16 [256]
    const int32_t* positions;   // [planes][pos_plane_stride]
    int pos_plane_stride;
    int rotary_dim;
    int mrope_s1, mrope_s2;
    float rope_theta;
    float rms_eps;
};

// Accurate libdevice routines, by name, as the reference's producer calls them
// (op_norms_rope_act.cu:14-16): -use_fast_math must not swap them for the approximate ones.
extern "C" __device__ float __nv_sinf(float);
extern "C" __device__ float __nv_cosf(float);
extern "C" __device__ float __nv_powf(float, float);

// The producer of the reference's layer, K half: per-head Gemma RMS norm (weight 1 + w) and partial
// interleaved 3-D mRoPE (fused_qk_rmsnorm_rope_gate_f16_kernel, op_norms_rope_act.cu:524-680), on a row
// held as x[r] = column sub + 8 r by the 8 lanes of a row group, returning the fp16 values that
// kernel would have written to k_out, so that the packed bytes are the same as those of the
// two-kernel sequence.  Arithmetic order is the reference's:
//  * sum of squares: its thread t adds the squares of columns 8 t .. 8 t + 7 in order, as a chain of
//    fused multiply-adds from 0, then a 32-wide xor butterfly (here: the row is transposed through
//    shared memory so that each lane runs four of the chains, and the butterfly's first two levels
//    stay in the lane);
//  * x * inv_rms, then * (1 + w), each rounded, then to fp16;
//  * angle = position * (1 / powf(theta, 2 i / rotary_dim)), sine and cosine rounded to fp16.
// Every lane of the warp takes part (the chain uses shuffles): the caller calls it for groups of four K
// rows.  rotary_dim / 2 must be a multiple of 8 so that both elements of a rotated pair sit in one lane.
__device__ __forceinline__ void k_producer(float (&x)[32], int sub, int lane_base, int tok, const AppendParams& p,
                                           const float* s_w1, const float* s_inv_freq, float* s_rows) {
    // The reference's thread t = sub + 8 j of this row sums columns 8 t .. 8 t + 7; this lane holds column
    // sub + 8 r in register r.  The row goes through shared memory (one 257-float line per row of the warp)
    // and comes back as the four 8-column runs of threads sub, sub + 8, sub + 16, sub + 24.
    float* line = s_rows + (lane_base >> 3) * 257;
#pragma unroll
    for (int r = 0; r < 32; ++r) line[sub + 8 * r] = x[r];
    __syncwarp();
    float part[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float* run = line + 8 * (sub + 8 * j);
        float acc = 0.0f;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc = __fmaf_rn(run[c], run[c], acc);
        part[j] = acc;
    }
    __syncwarp();   // the line is rewritten by the next group of rows
    // its 32-wide xor butterfly 16, 8, 4, 2, 1: thread bits 4 and 3 are j, bits 2..0 are sub
    float sum_sq = __fadd_rn(__fadd_rn(part[0], part[2]), __fadd_rn(part[1], part[3]));
#pragma unroll
    for (int h = 4; h > 0; h >>= 1) sum_sq = __fadd_rn(sum_sq, __shfl_xor_sync(0xffffffffu, sum_sq, h));
    const float inv_rms = rsqrtf(sum_sq / (float)kHeadDim + p.rms_eps);
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        const float v = __fmul_rn(x[r], inv_rms);
        x[r] = __half2float(__float2half(__fmul_rn(v, s_w1[sub + 8 * r])));
    }
    const int half_rot = p.rotary_dim >> 1;
    const int regs = half_rot >> 3;
    // sine and cosine of pair i = sub + 8 r at this row's token, rounded to fp16
    auto sincos_of = [&](int i, float& sin_a, float& cos_a) {
        int plane = 0;
        if ((i % 3) == 1 && i < p.mrope_s1 * 3) {
            plane = 1;
        } else if ((i % 3) == 2 && i < p.mrope_s2 * 3) {
            plane = 2;
        }
        const float pos = (float)p.positions[(size_t)plane * p.pos_plane_stride + tok];
        const float angle = pos * s_inv_freq[i];
        sin_a = __half2float(__float2half_rn(__nv_sinf(angle)));
        cos_a = __half2float(__float2half_rn(__nv_cosf(angle)));
    };
    // The four rows of a warp are usually the kv heads of one token: the angles are then the same in all
    // four, and row group g computes those of registers g, g + 4, ... for the others (a quarter of the calls).
    const int g = lane_base >> 3;
    const bool shared = ((regs & 3) == 0) && __all_sync(0xffffffffu, tok == __shfl_sync(0xffffffffu, tok, 0));
    float s_own[4] = {0.f, 0.f, 0.f, 0.f}, c_own[4] = {0.f, 0.f, 0.f, 0.f};
    if (shared) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (4 * k < regs) sincos_of(sub + 8 * (g + 4 * k), s_own[k], c_own[k]);
        }
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
        if (r < regs) {
            float sin_a, cos_a;
            if (shared) {
                sin_a = __shfl_sync(0xffffffffu, s_own[r >> 2], sub + 8 * (r & 3));
                cos_a = __shfl_sync(0xffffffffu, c_own[r >> 2], sub + 8 * (r & 3));
            } else {
                sincos_of(sub + 8 * r, sin_a, cos_a);
            }
            const float x1 = x[r];
            const float x2 = x[r + regs];
            x[r] = __half2float(__float2half(x1 * cos_a - x2 * sin_a));
            x[r + regs] = __half2float(__float2half(x2 * cos_a + x1 * sin_a));
        }
    }
}

constexpr int kAppendBlocksPerSm = 5;   // 4, 6 and 8 measured within 3 % of it on a 32 768-token append
constexpr int kProducerBlocksPerSm = 4;   // with the K producer in front: 128 registers (5 blocks of 96 registers measured the same, 3 of 168 slower)

// IN_BF16: activations are bf16 instead of fp16.  Values that both types can hold encode to the
// same bytes; bf16 values beyond the fp16 range are simply larger fp32 inputs.
// PRODUCER: K rows go through k_producer() first (fp16 activations only).
template <bool IN_BF16, bool PRODUCER>
__global__ void __launch_bounds__(128, PRODUCER ? kProducerBlocksPerSm : kAppendBlocksPerSm) tq4_append_kernel(const AppendParams p) {
    __shared__ float s_centroid[16];
    __shared__ float s_w1[PRODUCER ? kHeadDim : 1];
    __shared__ float s_inv_freq[PRODUCER ? kHeadDim / 2 : 1];
    __shared__ float s_rows[PRODUCER ? 4 * 4 * 257 : 1];   // one line per row of each of the four warps
    if (threadIdx.x < 16) s_centroid[threadIdx.x] = tq4_centroid(threadIdx.x);
    if (PRODUCER) {
        for (int i = threadIdx.x; i < kHeadDim; i += blockDim.x) {
            s_w1[i] = 1.0f + __half2float(__ushort_as_half(p.k_norm_w[i]));
        }
        for (int i = threadIdx.x; i < (p.rotary_dim >> 1); i += blockDim.x) {
            s_inv_freq[i] = __fdiv_rn(1.0f, __nv_powf(p.rope_theta, (float)(2 * i) / (float)p.rotary_dim));
        }
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int sub = lane & 7;
    const int lane_base = lane & ~7;
    // Per-lane constants, paid once per thread: the warp then loops over groups of 4 rows.
    uint32_t sign_word = 0;   // bit r = sign of column sub + 8 r
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        const int col = sub + 8 * r;
        sign_word |= ((c_sign_mask[col >> 5] >> (col & 31)) & 1u) << r;
    }
    uint32_t bpos[7];
#pragma unroll
    for (int k = 0; k < 7; ++k) bpos[k] = c_boundary_bits[8 + k];
    // butterfly direction of the three cross-lane WHT stages: upper lanes compute o - v
    const float dir1 = (sub & 1) ? -1.0f : 1.0f, dir2 = (sub & 2) ? -1.0f : 1.0f, dir4 = (sub & 4) ? -1.0f : 1.0f;

    const int heads = p.layout.local_kv_heads;
    const int warps_total = gridDim.x * 4;
    // A warp takes four rows at a time.  Plain append: rows 4 q .. 4 q + 3 of the list (token, head, K | V).
    // With the producer in front, a group holds four K rows or four V rows (groups alternate), so that the
    // norm and the rotation run for K groups only and not for the V rows that would share a warp with them.
    const int pairs = p.total_rows >> 1;                      // (token, head) pairs
    const int quads = PRODUCER ? 2 * ((pairs + 3) >> 2) : (p.total_rows + 3) >> 2;
#pragma unroll 1
    for (int quad = blockIdx.x * 4 + (threadIdx.x >> 5); quad < quads; quad += warps_total) {
    const int row_id = quad * 4 + (lane >> 3);

    // ---- resolve the row: (token, head, K or V), masks, destination ------------------
    const int which = PRODUCER ? (quad & 1) : (row_id & 1);
    const int th = PRODUCER ? ((quad >> 1) * 4 + (lane >> 3)) : (row_id >> 1);
    bool active = PRODUCER ? (th < pairs) : (row_id < p.total_rows);
    const int tok = active ? th / heads : 0;
    const int head = th - tok * heads;
    int slot = -1;
    if (active) {
        if (p.batch.valid_token_mask != nullptr && p.batch.valid_token_mask[tok] == 0) active = false;
    }
    if (active && p.batch.valid_req_mask != nullptr && p.batch.query_start_loc != nullptr &&
        p.batch.num_reqs > 0) {
        const int req = find_request(p.batch.query_start_loc, p.batch.num_reqs, tok);
        if (req < 0 || p.batch.valid_req_mask[req] == 0) active = false;
    }
    if (active) {
        slot = p.batch.write_slot_mapping[tok];
        if (slot < 0 || !write_slot_ok(slot, kInAppend)) active = false;
    }
    // All 8 lanes of a row agree on `active`; rows of a warp may differ, and every lane
    // still takes part in the shuffles below.
    const uint16_t* src = nullptr;
    uint8_t* dst = nullptr;
    if (active) {
        const int page = slot >> 4, off = slot & 15;
        if (which == 0) {
            src = p.k_in + (size_t)tok * p.k_row_stride + (size_t)head * kHeadDim;
            dst = (uint8_t*)(uintptr_t)p.layout.k_base + (size_t)page * p.layout.k_page_stride_bytes +
                  (size_t)head * p.layout.k_head_stride_bytes + (size_t)off * p.layout.k_token_stride_bytes;
        } else {
            src = p.v_in + (size_t)tok * p.v_row_stride + (size_t)head * kHeadDim;
            dst = (uint8_t*)(uintptr_t)p.layout.v_base + (size_t)page * p.layout.v_page_stride_bytes +
                  (size_t)head * p.layout.v_head_stride_bytes + (size_t)off * p.layout.v_token_stride_bytes;
        }
    }

    // ---- load: v[r] = sign * x[sub + 8 r] -------------------------------------------
    float v[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) {
        const uint16_t raw = active ? src[sub + 8 * r] : (uint16_t)0;
        const float x = IN_BF16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(__ushort_as_half(raw));
        v[r] = PRODUCER ? x : __uint_as_float(__float_as_uint(x) ^ ((sign_word << (31 - r)) & 0x80000000u));
    }
    if (PRODUCER) {
        if (which == 0) k_producer(v, sub, lane_base, tok, p, s_w1, s_inv_freq, s_rows + (threadIdx.x >> 5) * (4 * 257));   // warp-uniform: a group is all K or all V
#pragma unroll
        for (int r = 0; r < 32; ++r) v[r] = __uint_as_float(__float_as_uint(v[r]) ^ ((sign_word << (31 - r)) & 0x80000000u));
    }

    // ---- WHT-256: stages 1,2,4 across lanes, 8..128 in registers ----------------------
    // lower lane: v + o, upper lane: o - v; fma(+-1, v, o) is the same single rounding.
#pragma unroll
    for (int r = 0; r < 32; ++r) v[r] = __fmaf_rn(dir1, v[r], __shfl_xor_sync(0xffffffffu, v[r], 1));
#pragma unroll
    for (int r = 0; r < 32; ++r) v[r] = __fmaf_rn(dir2, v[r], __shfl_xor_sync(0xffffffffu, v[r], 2));
#pragma unroll
    for (int r = 0; r < 32; ++r) v[r] = __fmaf_rn(dir4, v[r], __shfl_xor_sync(0xffffffffu, v[r], 4));
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            if ((r & s) == 0) {
                const float a = v[r], b = v[r | s];
                v[r] = __fadd_rn(a, b);
                v[r | s] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 32; ++r) v[r] = __fmul_rn(v[r], 0.0625f);

    // ---- s_sq per half, in both lane classes -------------------------------------------
    float inv_lo[2], inv_hi[2];
    {
        float xl[8], xh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float a[4] = {v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]};
            reg_levels(a, a, xl[j], xh[j]);
        }
        const float tl = group_totals(xl, sub);
        const float s0l = seq4(tl, lane_base, 0), s1l = seq4(tl, lane_base, 4);
        inv_lo[0] = (s0l > 1e-20f) ? (0.7071067811865475f * rsqrtf(s0l)) : 0.0f;
        inv_lo[1] = (s1l > 1e-20f) ? (0.7071067811865475f * rsqrtf(s1l)) : 0.0f;
        inv_hi[0] = inv_lo[0];
        inv_hi[1] = inv_lo[1];
    }

    // ---- codes, centroids, least-squares sums ------------------------------------------
    uint32_t nib[4] = {0u, 0u, 0u, 0u};  // nibble r at nib[r >> 3] bits 4 (r & 7)
    float vcl[8], ccl[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float c[4];
        const float a[4] = {v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]};
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            const int r = 4 * j + q4;
            const float inv = (q4 & 2) ? inv_hi[j >> 2] : inv_lo[j >> 2];
            const int q = tq4_bucket(__fmul_rn(a[q4], inv), bpos);
            nib[r >> 3] += (uint32_t)q * (1u << (4 * (r & 7)));   // disjoint nibbles: add == or
            c[q4] = s_centroid[q];
        }
        float hi_unused;
        reg_levels(a, c, vcl[j], hi_unused);
        reg_levels(c, c, ccl[j], hi_unused);
    }
    // Only lane 0 of the reference warp (a lo-class lane) uses these sums.
    const float vct = group_totals(vcl, sub);
    const float cct = group_totals(ccl, sub);
    const float vc0 = seq4(vct, lane_base, 0), vc1 = seq4(vct, lane_base, 4);
    const float cc0 = seq4(cct, lane_base, 0), cc1 = seq4(cct, lane_base, 4);
    const float d0 = (cc0 > 1e-10f) ? (vc0 / cc0) : 0.0f;
    const float d1 = (cc1 > 1e-10f) ? (vc1 / cc1) : 0.0f;
    const uint32_t d0h = __half_as_ushort(__float2half_rn(d0));
    const uint32_t d1h = __half_as_ushort(__float2half_rn(d1));

    // ---- 8x8 nibble transpose inside the 8-lane group -----------------------------------
    // Before: lane `sub`, register m, nibble t  = code of column sub + 8 (8 m + t).
    // After : lane t,     register m, nibble s  = code of column s   + 8 (8 m + t),
    //         i.e. the 4 packed bytes of columns [8 (8 m + t), +8).
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        uint32_t w = nib[m];
        {
            const uint32_t o = __shfl_xor_sync(0xffffffffu, w, 4);
            w = (sub & 4) ? ((w & 0xffff0000u) | (o >> 16)) : ((w & 0x0000ffffu) | (o << 16));
        }
        {
            const uint32_t o = __shfl_xor_sync(0xffffffffu, w, 2);
            w = (sub & 2) ? ((w & 0xff00ff00u) | ((o >> 8) & 0x00ff00ffu))
                          : ((w & 0x00ff00ffu) | ((o << 8) & 0xff00ff00u));
        }
        {
            const uint32_t o = __shfl_xor_sync(0xffffffffu, w, 1);
            w = (sub & 1) ? ((w & 0xf0f0f0f0u) | ((o >> 4) & 0x0f0f0f0fu))
                          : ((w & 0x0f0f0f0fu) | ((o << 4) & 0xf0f0f0f0u));
        }
        nib[m] = w;
    }
    // Lane t now holds qs-words: block 0 words t (nib[0]) and 8 + t (nib[1]);
    // block 1 words t (nib[2]) and 8 + t (nib[3]).
    //
    // The row as 33 aligned 32-bit words W0..W32: W0 = d0 | qs0[0..1] << 16,
    // Wk = hi16(qs0 word k-1) | lo16(qs0 word k) << 16 (k = 1..15),
    // W16 = hi16(qs0 word 15) | d1 << 16, W(17 + k) = qs1 word k.
    const uint32_t a_prev = __shfl_sync(0xffffffffu, nib[0], lane_base + ((sub + 7) & 7));
    const uint32_t b_prev = __shfl_sync(0xffffffffu, nib[1], lane_base + ((sub + 7) & 7));
    if (active) {
        const bool word_ok = ((((uintptr_t)dst) & 3u) == 0u);
        if (word_ok) {
            uint32_t* w = reinterpret_cast<uint32_t*>(dst);
            const uint32_t w_a = (sub == 0) ? (d0h | (nib[0] << 16)) : ((a_prev >> 16) | (nib[0] << 16));
            const uint32_t prev_for_b = (sub == 0) ? a_prev : b_prev;  // lane 0: qs0 word 7 (from lane 7)
            const uint32_t w_b = (prev_for_b >> 16) | (nib[1] << 16);
            w[sub] = w_a;
            w[8 + sub] = w_b;
            w[17 + sub] = nib[2];
            w[25 + sub] = nib[3];
            if (sub == 7) w[16] = (nib[1] >> 16) | (d1h << 16);
        } else {
            // Row base not 4-byte aligned: 16-bit stores (rows are always 2-byte aligned).
            uint16_t* h = reinterpret_cast<uint16_t*>(dst);
            if (sub == 0) { h[0] = (uint16_t)d0h; h[33] = (uint16_t)d1h; }
            h[1 + 2 * sub] = (uint16_t)nib[0];
            h[2 + 2 * sub] = (uint16_t)(nib[0] >> 16);
            h[17 + 2 * sub] = (uint16_t)nib[1];
            h[18 + 2 * sub] = (uint16_t)(nib[1] >> 16);
            h[34 + 2 * sub] = (uint16_t)nib[2];
            h[35 + 2 * sub] = (uint16_t)(nib[2] >> 16);
            h[50 + 2 * sub] = (uint16_t)nib[3];
            h[51 + 2 * sub] = (uint16_t)(nib[3] >> 16);
        }
    }
    }  // row-quad loop
}

W34_BOUNDS_HOST_HOOKS(append)

}  // namespace w34

#include "kv8_append.cuh"

namespace w34 {
// Unrotated 8-bit layers: one warp per row.
static int launch_append_kv8(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                             const warp34_attention_batch* batch, const void* k_in, const void* v_in,
                             int k_row_stride, int v_row_stride) {
    const int min_stride = layout->local_kv_heads * layout->head_dim;
    if (k_row_stride < min_stride || v_row_stride < min_stride) return (int)cudaErrorInvalidValue;
    if (batch->write_slot_mapping == nullptr || layout->k_base == 0 || layout->v_base == 0) {
        return (int)cudaErrorInvalidValue;
    }
    // Scales are fp32 and the codes are stored as 32-bit words: every row must be 4-byte aligned
    // (the reference's row structs have the same alignment).
    if ((layout->k_base | layout->v_base | layout->k_page_stride_bytes | layout->k_head_stride_bytes |
         layout->k_token_stride_bytes | layout->v_page_stride_bytes | layout->v_head_stride_bytes |
         layout->v_token_stride_bytes) & 3u) {
        return (int)cudaErrorInvalidValue;
    }
    AppendParams p;
    p.layout = *layout;
    p.batch = *batch;
    p.k_in = static_cast<const uint16_t*>(k_in);
    p.v_in = static_cast<const uint16_t*>(v_in);
    p.k_row_stride = k_row_stride;
    p.v_row_stride = v_row_stride;
    const long long rows = 2ll * batch->total_tokens * layout->local_kv_heads;
    if (rows > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    p.total_rows = (int)rows;
    const bool aligned = ((((uintptr_t)k_in | (uintptr_t)v_in) & 15u) == 0u) && (k_row_stride & 7) == 0 && (v_row_stride & 7) == 0;
    const unsigned blocks8 = (unsigned)((rows / 2 + 3) / 4);   // a warp per (token, head)
    if (aligned) kv8_append_kernel<true><<<blocks8, 128, 0, (cudaStream_t)ex->stream>>>(p);
    else kv8_append_kernel<false><<<blocks8, 128, 0, (cudaStream_t)ex->stream>>>(p);
    return (int)cudaGetLastError();
}

struct KProducer {
    const void* k_norm_w;
    const int32_t* positions;
    int pos_plane_stride, rotary_dim, mrope_s1, mrope_s2;
    float rope_theta, rms_eps;
};

static int launch_append(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                         const warp34_attention_batch* batch, const void* k_in, const void* v_in,
                         int k_row_stride, int v_row_stride, bool in_bf16, const KProducer* producer = nullptr) {
    if (ex == nullptr || layout == nullptr || batch == nullptr || k_in == nullptr || v_in == nullptr) {
        return (int)cudaErrorInvalidValue;
    }
    if (producer != nullptr) {
        if (producer->k_norm_w == nullptr || producer->positions == nullptr) return (int)cudaErrorInvalidValue;
        // both elements of a rotated pair must sit in one lane: rotary_dim / 2 a multiple of 8
        if (producer->rotary_dim < 0 || producer->rotary_dim > kHeadDim || (producer->rotary_dim & 15) != 0) {
            return (int)cudaErrorNotSupported;
        }
    }
    if (batch->total_tokens <= 0 || layout->local_kv_heads <= 0) return 0;
    if (kv8_layout_ok(layout)) {
        if (in_bf16 || producer != nullptr) return (int)cudaErrorNotSupported;
        return launch_append_kv8(ex, layout, batch, k_in, v_in, k_row_stride, v_row_stride);
    }
    if (layout->head_dim != kHeadDim || layout->block_size != kPageTokens ||
        layout->k_format != WARP34_KV_FORMAT_TQ4 || layout->v_format != WARP34_KV_FORMAT_TQ4 ||
        layout->k_transform != WARP34_KV_TRANSFORM_RADEMACHER_WHT256 ||
        layout->v_transform != WARP34_KV_TRANSFORM_RADEMACHER_WHT256) {
        return (int)cudaErrorNotSupported;
    }
    const int min_stride = layout->local_kv_heads * layout->head_dim;
    if (k_row_stride < min_stride || v_row_stride < min_stride) return (int)cudaErrorInvalidValue;
    if (batch->write_slot_mapping == nullptr || layout->k_base == 0 || layout->v_base == 0) {
        return (int)cudaErrorInvalidValue;
    }
    // Scales are stored with 16-bit accesses: every row must be 2-byte aligned.
    if ((layout->k_base | layout->v_base | layout->k_page_stride_bytes | layout->k_head_stride_bytes |
         layout->k_token_stride_bytes | layout->v_page_stride_bytes | layout->v_head_stride_bytes |
         layout->v_token_stride_bytes) & 1u) {
        return (int)cudaErrorInvalidValue;
    }
    AppendParams p;
    p.layout = *layout;
    p.batch = *batch;
    p.k_in = static_cast<const uint16_t*>(k_in);
    p.v_in = static_cast<const uint16_t*>(v_in);
    p.k_row_stride = k_row_stride;
    p.v_row_stride = v_row_stride;
    const long long rows = 2ll * batch->total_tokens * layout->local_kv_heads;
    if (rows > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    p.total_rows = (int)rows;
    // 4 warps x 4 rows per block and pass; each warp then strides over the remaining row groups,
    // so per-thread constants are set up once.  The grid is what the GPU can hold at once.
    const long long blocks_needed = (rows + 15) / 16;
    static int sm_count_cache[64];
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
        if (sm_count_cache[dev] == 0) {
            int n = 0;
            if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) {
                sm_count_cache[dev] = n;
            }
        }
        if (sm_count_cache[dev] > 0) sms = sm_count_cache[dev];
    }
    const long long resident = (long long)sms * (producer != nullptr ? kProducerBlocksPerSm : kAppendBlocksPerSm);
    const unsigned blocks = (unsigned)(blocks_needed < resident ? blocks_needed : resident);
    p.k_norm_w = nullptr;
    p.positions = nullptr;
    p.pos_plane_stride = p.rotary_dim = p.mrope_s1 = p.mrope_s2 = 0;
    p.rope_theta = p.rms_eps = 0.0f;
    if (producer != nullptr) {
        if (in_bf16) return (int)cudaErrorNotSupported;
        p.k_norm_w = static_cast<const uint16_t*>(producer->k_norm_w);
        p.positions = producer->positions;
        p.pos_plane_stride = producer->pos_plane_stride;
        p.rotary_dim = producer->rotary_dim;
        p.mrope_s1 = producer->mrope_s1;
        p.mrope_s2 = producer->mrope_s2;
        p.rope_theta = producer->rope_theta;
        p.rms_eps = producer->rms_eps;
        tq4_append_kernel<false, true><<<blocks, 128, 0, (cudaStream_t)ex->stream>>>(p);
    } else if (in_bf16) {
        tq4_append_kernel<true, false><<<blocks, 128, 0, (cudaStream_t)ex->stream>>>(p);
    } else {
        tq4_append_kernel<false, false><<<blocks, 128, 0, (cudaStream_t)ex->stream>>>(p);
    }
    return (int)cudaGetLastError();
}
}  // namespace w34

extern "C" int warp34_kv_cache_write_strided(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                             const warp34_attention_batch* batch, const void* k_in,
                                             const void* v_in, int k_row_stride, int v_row_stride) {
    return w34::launch_append(ex, layout, batch, k_in, v_in, k_row_stride, v_row_stride, false);
}

// K-norm + RoPE + rotate / quantise / pack in one kernel: the K half of the reference's
// warp34_fused_qk_rmsnorm_rope_gate_strided_f16 followed by its warp34_kv_cache_write_strided
// (crates/warp34-host/src/model/forward.rs:1109-1149), without the fp16 K rows going through HBM.
extern "C" int warp34_fused_k_rmsnorm_rope_kv_cache_write_f16(
    const warp34_exec* ex, const warp34_kv_layer_layout* layout, const warp34_attention_batch* batch,
    const void* k_in, const void* v_in, const void* k_norm_w, const int32_t* positions, int pos_plane_stride,
    int rotary_dim, int mrope_s0, int mrope_s1, int mrope_s2, int k_row_stride, int v_row_stride, float rope_theta,
    float rms_eps) {
    (void)mrope_s0;   // the first section needs no bound: plane 0 is the default (op_norms_rope_act.cu:640-646)
    w34::KProducer pr;
    pr.k_norm_w = k_norm_w;
    pr.positions = positions;
    pr.pos_plane_stride = pos_plane_stride;
    pr.rotary_dim = rotary_dim;
    pr.mrope_s1 = mrope_s1;
    pr.mrope_s2 = mrope_s2;
    pr.rope_theta = rope_theta;
    pr.rms_eps = rms_eps;
    return w34::launch_append(ex, layout, batch, k_in, v_in, k_row_stride, v_row_stride, false, &pr);
}

extern "C" int warp34_kv_cache_write(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                     const warp34_attention_batch* batch, const void* k_in,
                                     const void* v_in) {
    if (layout == nullptr) return (int)cudaErrorInvalidValue;
    const int stride = layout->local_kv_heads * layout->head_dim;
    return w34::launch_append(ex, layout, batch, k_in, v_in, stride, stride, false);
}

extern "C" int warp34_tq4_kv_cache_write_strided_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                      const warp34_attention_batch* batch, const void* k_in,
                                                      const void* v_in, int k_row_stride, int v_row_stride) {
    return w34::launch_append(ex, layout, batch, k_in, v_in, k_row_stride, v_row_stride, true);
}
