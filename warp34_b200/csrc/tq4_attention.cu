// Paged attention over TQ4 pages for sm_100a: decode, MTP verify and (slowly) anything else
// the descriptor ABI can express.
//
// Replaces, for TQ4 + sign/WHT-256 layers, the reference's
//   paged_attention_gqa_mma_f16_kernel            (crates/warp34-kernels/csrc/ops/op_paged_attn.cu:186-588)
//   paged_attention_split_kv_reduce_f16_kernel    (op_paged_attn.cu:1132-1218)
//   warp34_paged_attention_f16 (dispatcher)       (op_paged_attn.cu:1266-1448)
//   paged_attention_kernel<__half> (scalar path)  (op_kv_cache.cu:373-461, :619-792)
//
// Three launches per call:
//   plan   : block 0: per request page range, item count and prefix sums -> scratch header;
//            blocks 1..: the rotated, scaled query rows of every (request, kv head) as the
//            stream kernel's MMA fragments (decode-sized batches).
//   stream : persistent grid, one CTA per SM.  The work list is the flattened sequence of
//            (request, kv head, row group, page) units, cut into equal contiguous shares, one
//            per warp.  A warp streams its pages through a private ring of shared-memory
//            stages filled by cp.async.bulk (one 2112-byte run for K and one for V per page
//            and head, completion on an mbarrier), dequantises the 4-bit codes in registers
//            through a conflict-free byte-pair lookup table, and runs S^T = K Q'^T and
//            O^T += V^T P^T as m16n8k16 tensor-core MMAs with fp32 accumulators (M = 16 keys or
//            16 channels, N = 8 query rows = GQA heads x query tokens of one row group).
//            Warps never synchronise with each other inside the page loop.
//   merge  : per (token, q head) combine the (m, l, acc[256]) partials of every warp share
//            that touched the row, one inverse WHT, sign diagonal, fp16 store.
//
// Scales never touch the operands: scores are d0 * (q . c)[0:128] + d1 * (q . c)[128:256]
// with one accumulator per 128-half, and P is multiplied by the V scales of its key before
// the PV product (the same factoring as op_kv_cache.cu:653-656 and :695-705).
#include "tq4_common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

namespace w34 {

// ---------------------------------------------------------------------------------------
// Request geometry shared by all kernels (op_paged_attn.cu:266-280 / op_kv_cache.cu:405-422)
// ---------------------------------------------------------------------------------------
struct ReqGeom {
    int q_start, q_len, ctx_before, seq_after;
    bool valid;
};

__device__ __forceinline__ ReqGeom load_req(const warp34_attention_batch& b, int r) {
    ReqGeom g;
    g.q_start = b.query_start_loc[r];
    g.q_len = b.query_start_loc[r + 1] - g.q_start;
    g.seq_after = b.seq_lens_after[r];
    g.ctx_before = (b.context_lens_before != nullptr) ? b.context_lens_before[r] : (g.seq_after - g.q_len);
    g.valid = g.q_len > 0 && (b.valid_req_mask == nullptr || b.valid_req_mask[r] != 0);
    return g;
}

__device__ __forceinline__ int row_max_kv(const warp34_attention_batch& b, const ReqGeom& g, int q_off) {
    int m = (b.mask_mode == WARP34_ATTN_MASK_SYMMETRIC_WINDOW) ? (g.seq_after - 1) : (g.ctx_before + q_off);
    if (m >= g.seq_after) m = g.seq_after - 1;
    return m;
}

__device__ __forceinline__ int row_min_kv(const warp34_attention_batch& b, const ReqGeom& g, int q_off) {
    int m = 0;
    if (b.sliding_window > 0) {
        const int w = g.ctx_before + q_off - b.sliding_window + 1;
        if (w > m) m = w;
    }
    return m;
}

// Activations are fp16 (the reference ABI) or bf16 (additive entry points): 16-bit loads and
// stores with the conversion picked at run time, outside the per-page loops.
__device__ __forceinline__ float load_act(const void* base, size_t idx, int bf16) {
    const uint16_t raw = static_cast<const uint16_t*>(base)[idx];
    return bf16 ? __uint_as_float((uint32_t)raw << 16) : __half2float(__ushort_as_half(raw));
}
__device__ __forceinline__ void store_act(void* base, size_t idx, float x, int bf16) {
    static_cast<uint16_t*>(base)[idx] = bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(x))
                                             : __half_as_ushort(__float2half_rn(x));
}

// ---------------------------------------------------------------------------------------
// Output epilogue.  The reference's layer multiplies the attention output by a sigmoid gate and,
// when its o_proj weights were rotated offline, applies a 64-point Hadamard to every 64 columns
// (warp34_apply_attn_output_gate_f16 / _hadamard_f16, op_norms_rope_act.cu:742-764, :805-851; call
// site crates/warp34-host/src/model/forward.rs:1192-1211).  Both steps round like the two-kernel
// sequence does: the attention output to the activation type first, the gated value again
// before the Hadamard.
// ---------------------------------------------------------------------------------------
struct OutputGate {
    const void* gate;   // [total_tokens, num_q_heads, 256] in the activation type, or null
    int mode;           // 0 none, 1 sigmoid gate, 2 sigmoid gate then Hadamard-64 (x 1/8) per 64 columns;
                        // + 4: the gate multiplies the un-rounded fp32 value (the query-sparse kernels'
                        // epilogue, op_qsa.cu:1040-1067) and may be absent (gate == nullptr)
};

// 1 / (1 + e^-g) as the reference's kernels compute it under -use_fast_math: ex2.approx of -g log2 e, then
// rcp.approx (op_norms_rope_act.cu:756, :841), not an IEEE division.
__device__ __forceinline__ float sigmoid_gate(float g) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + __expf(-g)));
    return r;
}

__device__ __forceinline__ float round_act(float x, int bf16) {
    return bf16 ? __bfloat162float(__float2bfloat16_rn(x)) : __half2float(__float2half_rn(x));
}

// Normalised 64-point Hadamard (x 1/8) over every 64 columns of a row held as v[j] = column
// lane + 32 j, on the values rounded to the activation type.
__device__ __forceinline__ void hadamard64_row(float (&v)[8], int lane, int io_bf16) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {   // block b = columns [64 b, 64 b + 64): index bits 0-4 = lane, bit 5 = register
        const float x0 = round_act(v[2 * b], io_bf16), x1 = round_act(v[2 * b + 1], io_bf16);
        float a0 = x0 + x1, a1 = x0 - x1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const float o0 = __shfl_xor_sync(0xffffffffu, a0, d), o1 = __shfl_xor_sync(0xffffffffu, a1, d);
            const float dir = (lane & d) ? -1.0f : 1.0f;   // upper lane: o - a, lower: a + o, one rounding either way
            a0 = __fmaf_rn(dir, a0, o0);
            a1 = __fmaf_rn(dir, a1, o1);
        }
        v[2 * b] = a0 * 0.125f;
        v[2 * b + 1] = a1 * 0.125f;
    }
}

// v[j] = column lane + 32 j of one 256-wide row (8 registers per lane of one warp).
__device__ __forceinline__ void apply_output_gate(float (&v)[8], const OutputGate& og, size_t row_base, int lane, int io_bf16) {
    if (og.mode == 0) return;
    if (og.gate != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float g = load_act(og.gate, row_base + lane + 32 * j, io_bf16);
            const float a = (og.mode & 4) ? v[j] : round_act(v[j], io_bf16);
            v[j] = a * sigmoid_gate(g);
        }
    }
    if ((og.mode & 3) != 2) return;
    hadamard64_row(v, lane, io_bf16);
}

// Stores one output row of a TQ4 layer: t[j] is column lane + 32 j after the inverse rotation,
// before the sign diagonal.
__device__ __forceinline__ void store_output_row(void* out, size_t row_base, float (&t)[8], int lane, int io_bf16,
                                                 const OutputGate& og) {
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = apply_sign(t[j], lane + 32 * j);
    apply_output_gate(t, og, row_base, lane, io_bf16);
#pragma unroll
    for (int j = 0; j < 8; ++j) store_act(out, row_base + lane + 32 * j, t[j], io_bf16);
}

// One 256-column chunk whose three rows start on 16-byte boundaries: lane holds columns [8 lane, 8 lane + 8).
template <int MODE, bool BF16>
__device__ __forceinline__ void gate_chunk_vec(uintptr_t pa, uintptr_t pg, uintptr_t po, int lane) {
    constexpr int mode = MODE;
    constexpr int io_bf16 = BF16 ? 1 : 0;
    const uint4 ra = reinterpret_cast<const uint4*>(pa)[lane];   // in place is fine: a lane writes the 16 bytes it read
    const uint4 rg = reinterpret_cast<const uint4*>(pg)[lane];
    const uint32_t wa[4] = {ra.x, ra.y, ra.z, ra.w}, wg[4] = {rg.x, rg.y, rg.z, rg.w};
    float x[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // two columns per 32-bit word
        float2 a, g;
        if (io_bf16) {
            a = make_float2(__uint_as_float(wa[i] << 16), __uint_as_float(wa[i] & 0xffff0000u));
            g = make_float2(__uint_as_float(wg[i] << 16), __uint_as_float(wg[i] & 0xffff0000u));
        } else {
            a = __half22float2(*reinterpret_cast<const __half2*>(&wa[i]));
            g = __half22float2(*reinterpret_cast<const __half2*>(&wg[i]));
        }
        x[2 * i] = a.x * sigmoid_gate(g.x);   // `a` is already a value of the activation type
        x[2 * i + 1] = a.y * sigmoid_gate(g.y);
    }
    if (mode == 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {   // the gated values rounded to the activation type, pairwise
            if (io_bf16) {
                const float2 r = __bfloat1622float2(__floats2bfloat162_rn(x[2 * i], x[2 * i + 1]));
                x[2 * i] = r.x;
                x[2 * i + 1] = r.y;
            } else {
                const float2 r = __half22float2(__floats2half2_rn(x[2 * i], x[2 * i + 1]));
                x[2 * i] = r.x;
                x[2 * i + 1] = r.y;
            }
        }
#pragma unroll
        for (int d = 1; d < 8; d <<= 1) {        // column bits 0-2: registers
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if ((i & d) == 0) {
                    const float lo = x[i], hi = x[i | d];
                    x[i] = lo + hi;
                    x[i | d] = lo - hi;
                }
            }
        }
#pragma unroll
        for (int d = 1; d < 8; d <<= 1) {        // column bits 3-5: lanes (upper lane: o - x, lower: x + o)
            const float dir = (lane & d) ? -1.0f : 1.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float o = __shfl_xor_sync(0xffffffffu, x[i], d);
                x[i] = __fmaf_rn(dir, x[i], o);   // one rounding, like the add or the subtraction
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] *= 0.125f;
    }
    uint32_t wo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (io_bf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            wo[i] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
            const __half2 h = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
            wo[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    reinterpret_cast<uint4*>(po)[lane] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
}

// The whole matrix in full, aligned chunks (known on the host): nothing but the vector path.
template <int MODE, bool BF16>
__global__ void __launch_bounds__(128) attn_output_gate_vec_kernel(const void* __restrict__ attn, const void* gate, void* out,
                                                                   const uint8_t* __restrict__ valid_token_mask, int num_tokens,
                                                                   int total_dim) {
    const int lane = threadIdx.x & 31;
    const int tok = (int)blockIdx.x, c = (int)blockIdx.y * 4 + (int)(threadIdx.x >> 5);
    if (tok >= num_tokens || c * 256 >= total_dim) return;
    if (valid_token_mask != nullptr && valid_token_mask[tok] == 0) return;
    const size_t off = 2 * ((size_t)tok * total_dim + (size_t)c * 256);
    gate_chunk_vec<MODE, BF16>(reinterpret_cast<uintptr_t>(attn) + off, reinterpret_cast<uintptr_t>(gate) + off,
                               reinterpret_cast<uintptr_t>(out) + off, lane);
}

// The two steps on their own (for layers whose attention kernel has no fused epilogue): one warp per
// 256 columns, in place or out of place.
template <int MODE, bool BF16>
__global__ void __launch_bounds__(128) attn_output_gate_kernel(const void* __restrict__ attn, const void* gate,
                                                               void* out, const uint8_t* __restrict__ valid_token_mask,
                                                               int num_tokens, int total_dim) {
    constexpr int mode = MODE;
    constexpr int io_bf16 = BF16 ? 1 : 0;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int chunks = (total_dim + 255) / 256;
    const int tok = (int)blockIdx.x, c = (int)blockIdx.y * 4 + wid;   // grid: (tokens, chunks / 4)
    if (tok >= num_tokens || c >= chunks) return;
    if (valid_token_mask != nullptr && valid_token_mask[tok] == 0) return;
    const size_t base = (size_t)tok * total_dim + (size_t)c * 256;
    const int cols = min(256, total_dim - c * 256);    // a multiple of 64 when mode == 2 (checked by the caller)
    // A full chunk whose three rows start on 16-byte boundaries: lane holds columns [8 lane, 8 lane + 8), one
    // 128-bit access per row; a 64-column Hadamard block is eight lanes (three levels in registers, three
    // across lanes: the transform is the same whatever the order of its levels).  (A grid-stride loop with
    // the next chunk's loads in flight measured slower than one chunk per warp.)
    const uintptr_t pa = reinterpret_cast<uintptr_t>(attn) + 2 * base, pg = reinterpret_cast<uintptr_t>(gate) + 2 * base;
    const uintptr_t po = reinterpret_cast<uintptr_t>(out) + 2 * base;
    if (cols == 256 && ((pa | pg | po) & 15u) == 0u) {
        gate_chunk_vec<MODE, BF16>(pa, pg, po, lane);
        return;
    }
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = (lane + 32 * j < cols) ? load_act(attn, base + lane + 32 * j, io_bf16) : 0.0f;
    OutputGate og;
    og.gate = gate;
    og.mode = mode;
    if (cols == 256) {
        apply_output_gate(v, og, base, lane, io_bf16);
    } else {   // ragged tail: the gate column by column; whole 64-blocks only reach the Hadamard
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (lane + 32 * j < cols) {
                const float g = load_act(gate, base + lane + 32 * j, io_bf16);
                v[j] = round_act(v[j], io_bf16) * sigmoid_gate(g);
            }
        }
        if (mode == 2) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float x0 = round_act(v[2 * b], io_bf16), x1 = round_act(v[2 * b + 1], io_bf16);
                float a0 = x0 + x1, a1 = x0 - x1;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const float o0 = __shfl_xor_sync(0xffffffffu, a0, d), o1 = __shfl_xor_sync(0xffffffffu, a1, d);
                    const bool up = (lane & d) != 0;
                    a0 = up ? (o0 - a0) : (a0 + o0);
                    a1 = up ? (o1 - a1) : (a1 + o1);
                }
                v[2 * b] = a0 * 0.125f;
                v[2 * b + 1] = a1 * 0.125f;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (lane + 32 * j < cols) store_act(out, base + lane + 32 * j, v[j], io_bf16);
    }
}

// ---------------------------------------------------------------------------------------
// Scalar dequant-then-attend: one block of four warps per (token, q head), fp32, any strides.
// ---------------------------------------------------------------------------------------
// One block of four warps per (token, q head): warp w takes the keys min_kv + w, + 4, ... (two per step, so
// that two rows are in flight), and the four online-softmax states are merged through shared memory.
__global__ void __launch_bounds__(128) tq4_attention_scalar_kernel(
    const warp34_kv_layer_layout layout, const warp34_attention_batch batch,
    const void* __restrict__ q_in, void* __restrict__ attn_out, int num_q_heads, int io_bf16, const OutputGate og) {
    __shared__ float s_x[4][kHeadDim];
    __shared__ float s_m[4], s_l[4];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long row = blockIdx.x;
    const int tok = (int)(row / num_q_heads), q_head = (int)(row % num_q_heads);
    if (batch.valid_token_mask != nullptr && batch.valid_token_mask[tok] == 0) return;   // block-uniform exits
    const int req = find_request(batch.query_start_loc, batch.num_reqs, tok);
    if (req < 0) return;
    const ReqGeom g = load_req(batch, req);
    if (!g.valid) return;
    const int gqa = num_q_heads / layout.local_kv_heads;
    const int kv_head = q_head / gqa;
    const int q_off = tok - g.q_start;
    const int max_kv = row_max_kv(batch, g, q_off);
    const int min_kv = row_min_kv(batch, g, q_off);

    const size_t row_base = ((size_t)tok * num_q_heads + q_head) * kHeadDim;

    // Q' = WHT(sign * q) (every warp computes it); then lane L owns rotated columns [8 L, 8 L + 8).
    float t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = apply_sign(load_act(q_in, row_base + lane + 32 * j, io_bf16), lane + 32 * j);
    wht256_lanes(t, lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) s_x[wid][lane + 32 * j] = t[j];
    __syncwarp();
    float qv[8], acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { qv[e] = s_x[wid][8 * lane + e]; acc[e] = 0.0f; }
    __syncwarp();

    const int blk = lane >> 4;                       // which 128-half this lane reads
    const int byte_off = kTq4BlockBytes * blk + 2 + 4 * (lane & 15);
    const int32_t* blocks = batch.block_tables + (size_t)req * batch.max_blocks_per_req;
    const uint8_t* k_head = (const uint8_t*)(uintptr_t)layout.k_base + (size_t)kv_head * layout.k_head_stride_bytes;
    const uint8_t* v_head = (const uint8_t*)(uintptr_t)layout.v_base + (size_t)kv_head * layout.v_head_stride_bytes;
    float m_i = -1e30f, l_i = 0.0f;
    for (int pos0 = min_kv + wid; pos0 <= max_kv; pos0 += 8) {
        // keys pos0 and pos0 + 4 of this warp; the second may lie past the row's last key
        const int pos1 = pos0 + 4;
        const bool two = pos1 <= max_kv;
        const uint8_t* kp[2];
        const uint8_t* vp[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int pos = (x == 0 || two) ? pos0 + 4 * x : pos0;
            const int page = block_table_page(blocks, pos >> 4, batch.max_blocks_per_req, kInScalar), off = pos & 15;
            kp[x] = k_head + (size_t)page * layout.k_page_stride_bytes + (size_t)off * layout.k_token_stride_bytes;
            vp[x] = v_head + (size_t)page * layout.v_page_stride_bytes + (size_t)off * layout.v_token_stride_bytes;
        }
        float dk[2], dv[2];
        uint32_t kw[2], vw[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            dk[x] = __half2float(*reinterpret_cast<const __half*>(kp[x] + kTq4BlockBytes * blk));
            kw[x] = (uint32_t)*reinterpret_cast<const uint16_t*>(kp[x] + byte_off) |
                    ((uint32_t)*reinterpret_cast<const uint16_t*>(kp[x] + byte_off + 2) << 16);
            dv[x] = __half2float(*reinterpret_cast<const __half*>(vp[x] + kTq4BlockBytes * blk));
            vw[x] = (uint32_t)*reinterpret_cast<const uint16_t*>(vp[x] + byte_off) |
                    ((uint32_t)*reinterpret_cast<const uint16_t*>(vp[x] + byte_off + 2) << 16);
        }
        float dot[2] = {0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            dot[0] += qv[e] * tq4_centroid((kw[0] >> (4 * e)) & 15u);
            dot[1] += qv[e] * tq4_centroid((kw[1] >> (4 * e)) & 15u);
        }
        dot[0] *= dk[0];
        dot[1] *= dk[1];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            dot[0] += __shfl_xor_sync(0xffffffffu, dot[0], off);
            dot[1] += __shfl_xor_sync(0xffffffffu, dot[1], off);
        }
        const float s0 = dot[0] * batch.sm_scale;
        const float s1 = two ? dot[1] * batch.sm_scale : -1e30f;
        const float m_new = fmaxf(m_i, fmaxf(s0, s1));
        const float alpha = __expf(m_i - m_new);
        const float p0 = __expf(s0 - m_new);
        const float p1 = two ? __expf(s1 - m_new) : 0.0f;
        l_i = l_i * alpha + p0 + p1;
        m_i = m_new;
        const float pd0 = p0 * dv[0], pd1 = p1 * dv[1];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            acc[e] = acc[e] * alpha + pd0 * tq4_centroid((vw[0] >> (4 * e)) & 15u) +
                     pd1 * tq4_centroid((vw[1] >> (4 * e)) & 15u);
        }
    }
    // ---- merge the four warps' states: warp 0 keeps the result ---------------------------------------
#pragma unroll
    for (int e = 0; e < 8; ++e) s_x[wid][8 * lane + e] = acc[e];
    if (lane == 0) { s_m[wid] = m_i; s_l[wid] = l_i; }
    __syncthreads();
    if (wid != 0) return;
    float m_tot = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float l_tot = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float wgt = (s_l[w] > 0.0f) ? __expf(s_m[w] - m_tot) : 0.0f;
        l_tot += s_l[w] * wgt;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += s_x[w][8 * lane + e] * wgt;
    }
    __syncwarp();
    const float inv_l = (l_tot > 0.0f) ? (1.0f / l_tot) : 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) s_x[0][8 * lane + e] = acc[e] * inv_l;
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = s_x[0][lane + 32 * j];
    wht256_lanes(t, lane);
    store_output_row(attn_out, row_base, t, lane, io_bf16, og);
}

// ---------------------------------------------------------------------------------------
// Split-KV streaming path
// ---------------------------------------------------------------------------------------
constexpr int kRowsPerGroup = 8;            // N of the MMA: query rows per work item
constexpr int kLutBytes = 256 * 256;         // byte-pair table: 256-byte entry stride, 32 lane copies each
constexpr int kPartialFloats = kRowsPerGroup * kHeadDim + 2 * kRowsPerGroup;
constexpr long long kWaitCycleLimit = 1ll << 31;  // about one second of SM clocks
constexpr int kMinUnitsPerWarp = 4;   // 8, 16 and 32 measured equal or slower on small batches
// The lookup table holds fp16(kLutScale * centroid).  fp16 rounding of the 8 centroid
// magnitudes is a systematic error of up to 3.7e-4 relative; with this common factor every one
// of them lands within 9.5e-5 of an fp16 grid point (found by exhaustive search over
// [0.5, 2)), and the factor itself is divided out exactly: 1/kLutScale is folded into Q' for
// the scores and into the final normalisation for the output.
constexpr float kLutScale = 0.954016f;

// Scratch header written by the plan kernel.
struct PlanHeader {
    int32_t status;        // 0 ok; bit 0: an mbarrier wait gave up; bit 1: shared-memory window too small;
                           // bit 2: a request's q_len exceeded batch.max_q_len (its extra rows were dropped)
    int32_t total_items;
    int32_t total_units;
    int32_t units_per_warp;
};
// Per request (num_reqs + 1 entries where it is a prefix sum), all int32, after the header:
//   unit_prefix[r], item_prefix[r], page_lo[r], npages[r], ngroups[r]
constexpr int kPlanArrays = 5;

__host__ __device__ inline size_t plan_bytes(int num_reqs) {
    size_t b = sizeof(PlanHeader) + (size_t)kPlanArrays * (size_t)(num_reqs + 1) * sizeof(int32_t);
    return (b + 255) & ~(size_t)255;
}

struct StreamParams {
    warp34_kv_layer_layout layout;
    warp34_attention_batch batch;
    const void* q_in;      // fp16 or bf16, see io_bf16
    void* attn_out;
    int io_bf16;
    float* triple_out;     // [total_tokens, num_q_heads, 258] when the merge stops before normalising
    uint8_t* scratch;      // plan header, arrays, then partial slots
    int num_q_heads;
    int gqa;
    int num_warps;         // worker warps over the whole grid
    int max_slots;
    uint32_t smem_bytes;   // dynamic shared memory given to the stream kernel
    int rows_per_group;    // query rows per work item: 8 (one warp per item) or 8 * NT (teams)
    float q_scale;         // sm_scale * log2(e) / kLutScale, folded into Q'
    int natural;           // partials are in natural (unrotated, unscaled) coordinates: uncompressed KV
    uint32_t* qfrag;       // rotated queries as MMA fragments, written by the plan launch (or null)
    int q_groups_max;      // row groups per (request, kv head) that qfrag has room for
    OutputGate og;         // applied by the merge kernel when it stores attn_out
    // Query-sparse mode (sel_phys != nullptr): request r is token r, its "pages" are units of four
    // selected 4-token groups (physical group id = page * 4 + group in page, logical group index for the
    // causal test against seq_pos[r]); rows of masked tokens are written as zeros.
    int q_floor = 0;       // query fragments for the exact build: hi rounded down, residual bytes 0..255
    int rows_from_first_token = 0;   // merge: block x is row x of the batch (0) or row x counted from the batch's first token (1)
    int keep_status = 0;             // plan: OR into the status word instead of clearing it (second and later passes)
    const int32_t* sel_phys = nullptr;
    const int32_t* sel_logical = nullptr;
    const int32_t* num_selected = nullptr;
    const int32_t* seq_pos = nullptr;
    int select_k = 0;
};

// Geometry of request r: from the batch descriptor, or in query-sparse mode one query token at
// position seq_pos[r].
__device__ __forceinline__ ReqGeom stream_req(const StreamParams& p, int r) {
    if (p.sel_phys == nullptr) return load_req(p.batch, r);
    ReqGeom g;
    g.q_start = r;
    g.q_len = 1;
    g.ctx_before = p.seq_pos[r];
    g.seq_after = g.ctx_before + 1;
    g.valid = true;
    return g;
}

__device__ __forceinline__ int32_t* plan_array(uint8_t* scratch, int which, int num_reqs) {
    return reinterpret_cast<int32_t*>(scratch + sizeof(PlanHeader)) + (size_t)which * (num_reqs + 1);
}

// Words per lane of one work item's query fragments: 16 k-steps x 2 B-fragment words of fp16(Q'),
// then 16 words holding the residual of Q' as bytes (four per k-step): Q' = hi + lo with hi the fp16
// value just below Q' (rounded towards minus infinity), so that 0 <= lo < 1 ulp; lo divided by the
// row's own step (largest lo of the row / 255) and rounded is an integer 0..255, which as the low
// byte of an fp16 word is the subnormal number integer x 2^-24: exact, and no arithmetic to widen it;
// then the steps of the lane's two rows (2 tig, 2 tig + 1), times 2^24, as floats.
constexpr int kQFragWords = 50;
__host__ __device__ inline size_t qfrag_item_bytes() { return (size_t)kQFragWords * 32 * sizeof(uint32_t); }
__device__ void qprep_block(const StreamParams& p, int idx);
constexpr int kPlanThreads = 32 * kRowsPerGroup;  // the query-fragment blocks use one warp per query row

// Block 0 plans the split.  Blocks 1.. (one-warp items only) each rotate and scale the query rows
// of one (request, kv head, row group) and store them as the B fragments of S^T = K Q'^T, so that
// the stream kernel's warps (several per item, and again for every further item a warp reaches)
// only load them.  The fragments are indexed without the plan, so both run side by side.
__global__ void __launch_bounds__(kPlanThreads) tq4_attention_plan_kernel(const StreamParams p) {
    if (blockIdx.x > 0) {
        qprep_block(p, (int)blockIdx.x - 1);
        return;
    }
    if (threadIdx.x >= 32) return;
    const int lane = threadIdx.x;
    const int R = p.batch.num_reqs;
    int32_t* unit_prefix = plan_array(p.scratch, 0, R);
    int32_t* item_prefix = plan_array(p.scratch, 1, R);
    int32_t* page_lo = plan_array(p.scratch, 2, R);
    int32_t* npages_a = plan_array(p.scratch, 3, R);
    int32_t* ngroups_a = plan_array(p.scratch, 4, R);
    const int hkv = p.layout.local_kv_heads;
    int unit_carry = 0, item_carry = 0;
    bool clamped = false;
    for (int base = 0; base < R; base += 32) {
        const int r = base + lane;
        int npages = 0, ngroups = 0, plo = 0;
        if (r < R && p.sel_phys != nullptr) {
            // query-sparse: a unit is four entries of the token's selected list; masked tokens have no items
            if (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[r] != 0) {
                int n_sel = p.num_selected[r];
                if (n_sel > p.select_k) n_sel = p.select_k;
                npages = n_sel > 0 ? (n_sel + 3) >> 2 : 0;
                ngroups = (p.gqa + p.rows_per_group - 1) / p.rows_per_group;
                if (p.qfrag != nullptr && ngroups > p.q_groups_max) { ngroups = p.q_groups_max; clamped = true; }
            }
        } else if (r < R) {
            const ReqGeom g = load_req(p.batch, r);
            if (g.valid) {
                const int lo = row_min_kv(p.batch, g, 0);
                const int hi = row_max_kv(p.batch, g, g.q_len - 1);
                if (hi >= lo) { plo = lo >> 4; npages = (hi >> 4) - plo + 1; }
                ngroups = (g.q_len * p.gqa + p.rows_per_group - 1) / p.rows_per_group;
                // a request longer than the batch's max_q_len has no room in the fragment store
                if (p.qfrag != nullptr && ngroups > p.q_groups_max) { ngroups = p.q_groups_max; clamped = true; }
            }
        }
        const int items = hkv * ngroups;
        int units = items * npages;
        int iu = units, ii = items;  // inclusive scans
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int a = __shfl_up_sync(0xffffffffu, iu, d);
            const int c = __shfl_up_sync(0xffffffffu, ii, d);
            if (lane >= d) { iu += a; ii += c; }
        }
        if (r < R) {
            unit_prefix[r] = unit_carry + iu - units;
            item_prefix[r] = item_carry + ii - items;
            page_lo[r] = plo;
            npages_a[r] = npages;
            ngroups_a[r] = ngroups;
        }
        unit_carry += __shfl_sync(0xffffffffu, iu, 31);
        item_carry += __shfl_sync(0xffffffffu, ii, 31);
    }
    const bool clamped_any = __any_sync(0xffffffffu, clamped);
    if (lane == 0) {
        unit_prefix[R] = unit_carry;
        item_prefix[R] = item_carry;
        page_lo[R] = 0; npages_a[R] = 0; ngroups_a[R] = 0;
        PlanHeader* h = reinterpret_cast<PlanHeader*>(p.scratch);
        // bit 2: a request's q_len exceeded batch.max_q_len, rows dropped.  A later part of a batch that runs in
        // several passes keeps what the earlier passes reported.
        h->status = (clamped_any ? 4 : 0) | (p.keep_status ? h->status : 0);
        h->total_items = item_carry;
        h->total_units = unit_carry;
        int per = (unit_carry + p.num_warps - 1) / (p.num_warps > 0 ? p.num_warps : 1);
        if (unit_carry > 0 && per < kMinUnitsPerWarp) per = kMinUnitsPerWarp;
        h->units_per_warp = per;
    }
}

// ---- PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; returns false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int spin = 0; spin < 256; ++spin) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (clock64() - t0 > kWaitCycleLimit) return false;
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// Schedulable shared-memory loads.  A volatile asm keeps its place among all other volatile
// asms, which chains every load and MMA of a page in source order.  These two are plain asms:
// the compiler may move and interleave them freely.
//  * lds32_lut: the lookup table never changes after the kernel's first barrier, and its address
//    always derives from a code word loaded in the same page iteration.
//  * lds32_dep: staged page data.  `token` is produced by page_token() right after the stage's
//    mbarrier wait, so the load cannot rise above the wait, and loads of different iterations are
//    different expressions; every result feeds an MMA of the same iteration, so it cannot sink
//    past the stage's release either.
__device__ __forceinline__ uint32_t lds32_lut(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
template <bool B> struct BoolTag { static constexpr bool value = B; };
__device__ __forceinline__ uint2 lds64_lut(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32_dep(uint32_t addr, uint32_t token) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1+0];  // dep %2" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint32_t page_token(int i) {
    uint32_t t;
    asm volatile("mov.u32 %0, %1;" : "=r"(t) : "r"(i) : "memory");
    return t;
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// First MMA of a chain: the accumulator input is the zero register, no clearing moves.
__device__ __forceinline__ void mma16816_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// A 132-byte row is 33 aligned words W0..W32.  Codes of the first 128-half sit at bytes 2..65,
// i.e. shifted by half a word.  "Virtual word" vw (0..15) of half 0 is W[vw] for vw >= 1 and the
// splice {bytes 2,3 | bytes 64,65} = (W0 >> 16) | (W16 << 16) for vw = 0; of half 1 it is
// W[17 + vw].  Rotated columns covered by virtual word vw, element e (0..7):
__device__ __forceinline__ int vword_col(int half, int vw, int e) {
    if (half == 1) return 128 + 8 * vw + e;
    if (vw == 0) return (e < 4) ? e : (120 + e);
    return 8 * vw - 4 + e;
}

// Shared-memory stage of one (page, kv head): each 2112-byte run is brought in as two
// 1056-byte halves (tokens 0-7, tokens 8-15) with 32 bytes of padding between them, so that
// token t sits at bank offset t (t < 8) or t + 8 (t >= 8).  With 33-word rows that makes every
// code load below hit 32 distinct banks:
//   K: one load covers tokens {0..3} u {8..11} (or {4..7} u {12..15}) x words {w, w+4, w+8, w+12};
//   V: one load covers tokens {k, k+2, k+8, k+10} x words {0,1,4,5,8,9,12,13} (+2).
constexpr int kHalfBytes = 8 * kTq4RowBytes;       // 1056
constexpr int kHalfStride = kHalfBytes + 32;       // 1088
constexpr int kRunStride = 2 * kHalfStride - 32;   // 2144: K run, then V run
constexpr int kStageStride = 2 * kRunStride;       // 4288

__device__ __forceinline__ uint32_t token_offset(int t) {  // byte offset of token row t in a run
    return (uint32_t)((t >> 3) * kHalfStride + (t & 7) * kTq4RowBytes);
}

// The streaming kernel comes in two builds.
//  * exact (default): every fp16 tensor-core operand that carries a rounding error of its own is
//    fed as value + residual: Q' (residual kept as one byte per element, widened in registers), the K
//    centroids (the lookup returns value pair and residual pair at once) and, on pages where some
//    weight is large enough to matter, P x d_v.  Three score MMAs per k-step instead of one.  With
//    fp16 operands alone a softmax weight is off by a few 1e-4 relative, which a x20 outlier channel
//    of V turns into several 1e-3 absolute where its large terms cancel.
//  * fast (WARP34_B200_EXEC_FLAG_FAST_ATTENTION): single fp16 operands, as the reference's own
//    tensor-core kernel computes (op_paged_attn.cu:357, :47-50, :470).
constexpr int kFastWarps = 12, kFastStages = 3;
constexpr int kExactWarps = 8, kExactStages = 4;
// A page is "peaked" when one of its keys holds more than this fraction of a row's softmax mass so
// far (an upper bound of the key's final weight: the mass only grows).  Only there does the rounding
// residual of the V centroids (1e-4 relative, but the same for every coordinate that holds the same
// code, so the inverse rotation can collect it on one channel) go through an extra product: a key
// below a quarter of the mass moves the output by less than a quarter of that.  (Gating the residual
// of P x d_v the same way, at 1/16 of the mass, measured no faster than carrying it on every page.)
constexpr float kPeakedWeight = 0.25f;
// The prefill kernel (tensor-bound) also gates the residual of P x d_v, at this fraction of the mass.
constexpr float kPResidualWeight = 1.0f / 64.0f;
// The prefill kernel takes the V-centroid residual pass from an eighth of the mass (its pages serve 16 rows
// per warp, and the pass costs it little).
constexpr float kPxPeakedWeight = 0.125f;
// Rounding residuals are 2^-12 of their values.  Those of the table's centroids (values 0.12 .. 2.6
// after the common factor; residuals at most 1e-3, at least a few hundred fp16 subnormal steps) are
// stored in this kernel's table times 2^11, as normal fp16 numbers, and their products scaled back in
// fp32: the MMA takes subnormal operands as they are (the prefill kernel's table holds the residuals
// unscaled and adds their product straight to the scores), but this kernel measured 1.4 % faster with
// the scaled table.  The residual of Q' is kept as one byte per element in units of a step of its own
// row (see the query-fragment block).
constexpr float kResidualScale = 2048.0f;

// Eight warps: the query fragments of item idx = (request * kv heads + kv head) * q_groups_max + group.
// Warp w rotates and scales query row w of the group into shared memory (fp32 [8 rows][256 rotated
// columns], times q_scale); after the barrier it builds the fragment words of step w.
__device__ void qprep_block(const StreamParams& p, int idx) {
    __shared__ float q_stage[kRowsPerGroup * kHeadDim];
    __shared__ float q_step[kRowsPerGroup];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const int hkv = p.layout.local_kv_heads;
    const int group = idx % p.q_groups_max;
    const int kv_head = (idx / p.q_groups_max) % hkv;
    const int r = idx / (p.q_groups_max * hkv);
    if (r >= p.batch.num_reqs || p.qfrag == nullptr) return;  // block-uniform
    const ReqGeom g = stream_req(p, r);
    const int rows_in_req = g.q_len * p.gqa;
    if (!g.valid || group * kRowsPerGroup >= rows_in_req) return;  // block-uniform
    {
        const int row8 = wid;
        const int row = group * kRowsPerGroup + row8;
        const int q_off = row / p.gqa;
        const int q_head = kv_head * p.gqa + (row - q_off * p.gqa);
        const bool ok = row < rows_in_req &&
                        (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
        float t[8];
        if (ok) {
            const size_t q_base = ((size_t)(g.q_start + q_off) * p.num_q_heads + q_head) * kHeadDim;
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = apply_sign(load_act(p.q_in, q_base + lane + 32 * j, p.io_bf16), lane + 32 * j);
            wht256_lanes(t, lane);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = 0.0f;
        }
        float rmax = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = t[j] * p.q_scale;
            q_stage[row8 * kHeadDim + lane + 32 * j] = f;
            if (p.q_floor) rmax = fmaxf(rmax, f - __half2float(__float2half_rd(f)));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, d));
        if (lane == 0) q_step[row8] = rmax * (1.0f / 255.0f);
    }
    __syncthreads();
    // B fragments of Q'^T: step s (0..7) covers half s >> 2, virtual word 4 tig + (s & 3);
    // k-step 2 s uses elements 0..3 of the word, k-step 2 s + 1 elements 4..7.
    // Q' = hi + lo: hi is fp16 (rounded down), lo >= 0 is kept as 4 bytes per k-step, integers in units
    // of the row's step, and widened to fp16 pairs (subnormals) by two PRMTs right before its MMA.
    const int s = wid;
    const int half = s >> 2, vw = 4 * tig + (s & 3);
    uint32_t* dst = p.qfrag + (size_t)idx * (kQFragWords * 32) + lane;
    const float step = q_step[gid];
    const float inv_step = step > 0.0f ? 1.0f / step : 0.0f;
    if (s == 0) {   // the steps of the rows whose scores this lane holds in the stream kernel
        dst[48 * 32] = __float_as_uint(q_step[2 * tig] * 16777216.0f);
        dst[49 * 32] = __float_as_uint(q_step[2 * tig + 1] * 16777216.0f);
    }
#pragma unroll
    for (int hk = 0; hk < 2; ++hk) {
        uint32_t lo_bytes = 0;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int e = 4 * hk + 2 * x;
            const float f0 = q_stage[gid * kHeadDim + vword_col(half, vw, e)];
            const float f1 = q_stage[gid * kHeadDim + vword_col(half, vw, e + 1)];
            const __half h0 = p.q_floor ? __float2half_rd(f0) : __float2half_rn(f0);
            const __half h1 = p.q_floor ? __float2half_rd(f1) : __float2half_rn(f1);
            dst[(2 * (2 * s + hk) + x) * 32] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
            // residuals in units of the row's step: integers 0..255
            const uint32_t b0 = (uint32_t)max(min(__float2int_rn((f0 - __half2float(h0)) * inv_step), 255), 0);
            const uint32_t b1 = (uint32_t)max(min(__float2int_rn((f1 - __half2float(h1)) * inv_step), 255), 0);
            lo_bytes |= (b0 & 0xffu) << (16 * x) | (b1 & 0xffu) << (16 * x + 8);
        }
        dst[(32 + 2 * s + hk) * 32] = lo_bytes;
    }
}

template <int STAGES, int WARPS, bool EXACT, bool SPARSE = false>
__global__ void __launch_bounds__(WARPS * 32, 1) tq4_attention_stream_kernel(const StreamParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    // The lookup table sits at the first 64 KB-aligned SHARED address inside the dynamic window,
    // so that (table address | code byte << 8 | lane << 2) is one PRMT.  Warp rings fill the
    // space below and above it; the mbarriers follow the last ring.
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int warps_per_cta = blockDim.x >> 5;
    const uint32_t win_lo = smem_u32(smem);
    const uint32_t win_hi = win_lo + p.smem_bytes;
    const uint32_t lut_addr = (win_lo + 0xffffu) & ~0xffffu;
    constexpr uint32_t kRingBytes = STAGES * kStageStride;
    const uint32_t warps_below = (lut_addr - win_lo) / kRingBytes;
    const uint32_t ring = ((uint32_t)wid < warps_below) ? (win_lo + (uint32_t)wid * kRingBytes)
                                                         : (lut_addr + kLutBytes + ((uint32_t)wid - warps_below) * kRingBytes);
    const uint32_t above = (uint32_t)warps_per_cta > warps_below ? (uint32_t)warps_per_cta - warps_below : 0u;
    const uint32_t bars_base = lut_addr + kLutBytes + above * kRingBytes;
    const uint32_t bars = bars_base + (uint32_t)wid * STAGES * 8u;
    PlanHeader* hdr = reinterpret_cast<PlanHeader*>(p.scratch);
    if (lut_addr + kLutBytes > win_hi || bars_base + (uint32_t)warps_per_cta * STAGES * 8u > win_hi) {
        if (threadIdx.x == 0) atomicOr(&hdr->status, 2);  // shared-memory window cannot hold the layout
        return;
    }
    uint8_t* ring_gen = smem + (ring - win_lo);

    // Byte-pair table: entry (byte, lane) at byte * 256 + lane * 4 holds
    // half2(s * centroid[byte & 15], s * centroid[byte >> 4]); bank = lane for any data.
    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
        const int byte = i >> 5, ln = i & 31;
        const float c0 = kLutScale * tq4_centroid(byte & 15), c1 = kLutScale * tq4_centroid(byte >> 4);
        if (EXACT) {
            // K table: (value pair, residual pair) in 16 copies of 8 bytes; V table: value pair in
            // 32 copies of 4 bytes, in the upper half of the same 256-byte entry
            const uint32_t hi = pack_half2(c0, c1);
            const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
            if (ln < 16) {
                sts32(lut_addr + (uint32_t)(byte * 256 + ln * 8), hi);
                sts32(lut_addr + (uint32_t)(byte * 256 + ln * 8 + 4),
                      pack_half2((c0 - hf.x) * kResidualScale, (c1 - hf.y) * kResidualScale));
            }
            sts32(lut_addr + (uint32_t)(byte * 256 + 128 + ln * 4), hi);
        } else {
            sts32(lut_addr + (uint32_t)(byte * 256 + ln * 4), pack_half2(c0, c1));
        }
    }
    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8u * s, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int R = p.batch.num_reqs;
    const int32_t* unit_prefix = plan_array(p.scratch, 0, R);
    const int32_t* item_prefix = plan_array(p.scratch, 1, R);
    const int32_t* page_lo_a = plan_array(p.scratch, 2, R);
    const int32_t* npages_a = plan_array(p.scratch, 3, R);
    const int32_t* ngroups_a = plan_array(p.scratch, 4, R);
    float* partials = reinterpret_cast<float*>(p.scratch + plan_bytes(R));

    // Worker index: consecutive workers sit on different SMs, so that a step with fewer shares
    // than warps spreads over the whole GPU instead of filling the first CTAs.
    const int w_global = wid * (int)gridDim.x + (int)blockIdx.x;
    const int per = hdr->units_per_warp;
    const int total_units = hdr->total_units;
    long long u_ll = (long long)w_global * per;
    if (per <= 0 || u_ll >= total_units) return;
    int u = (int)u_ll;
    const int u_end = min(u + per, total_units);

    const int gid = lane >> 2, tig = lane & 3;
    // MMA row m of S^T <-> token key(m) = (m & 3) + 8 ((m >> 2) & 1) + 4 (m >> 3) of the page.
    const int key_a = (gid & 3) + 8 * (gid >> 2);      // row gid; row gid + 8 is token key_a + 4
    // In the PV product thread tig owns tokens kv0 + {0, 1, 4, 5} (k positions 2tig, 2tig+1, +8, +9).
    const int kv0 = 2 * (tig & 1) + 8 * (tig >> 1);
    // byte 1 of these is zero: the code byte goes there
    const uint32_t lut_lane = EXACT ? lut_addr + 128u + 4u * lane : lut_addr + 4u * lane;   // V (and K) values
    const uint32_t lutk_lane = lut_addr + 8u * (lane & 15);                                      // K value + residual
    uint32_t phase_bits = 0;   // bit s = parity to wait for on stage s
    uint32_t pending = 0;      // bit s = a copy into stage s has been issued and not yet awaited
    bool failed = false;

    // locate the request containing unit u
    int r;
    {
        int lo = 0, hi = R;  // unit_prefix[lo] <= u < unit_prefix[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (unit_prefix[mid] <= u) lo = mid; else hi = mid;
        }
        r = lo;
    }

    while (u < u_end && !failed) {
        while (unit_prefix[r + 1] <= u) ++r;  // skips requests without units
        const int npages = npages_a[r];
        const int ngroups = ngroups_a[r];
        const int in_req = u - unit_prefix[r];
        const int item = in_req / npages;
        const int page_in_item = in_req - item * npages;
        const int n_here = min(u_end - u, npages - page_in_item);
        const int kv_head = item / ngroups;
        const int group = item - kv_head * ngroups;
        const int pg0 = page_lo_a[r] + page_in_item;  // first logical page of this segment
        const int slot = w_global + item_prefix[r] + item;
        const ReqGeom g = stream_req(p, r);
        const int rows_in_req = g.q_len * p.gqa;

        // ---- per-row limits for this lane's two query rows (2 tig, 2 tig + 1) ----------
        int rmax[2], rmin[2];
        bool rvalid[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int row = group * kRowsPerGroup + 2 * tig + x;
            const int q_off = row / p.gqa;
            rvalid[x] = row < rows_in_req &&
                        (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
            rmax[x] = rvalid[x] ? row_max_kv(p.batch, g, q_off) : -1;
            rmin[x] = rvalid[x] ? row_min_kv(p.batch, g, q_off) : 0x7fffffff;
        }
        // keys in [safe_lo, safe_hi] are visible to every valid row of the group
        int safe_hi = min(rvalid[0] ? rmax[0] : 0x7fffffff, rvalid[1] ? rmax[1] : 0x7fffffff);
        int safe_lo = max(rvalid[0] ? rmin[0] : 0, rvalid[1] ? rmin[1] : 0);
#pragma unroll
        for (int d = 1; d < 4; d <<= 1) {
            safe_hi = min(safe_hi, __shfl_xor_sync(0xffffffffu, safe_hi, d));
            safe_lo = max(safe_lo, __shfl_xor_sync(0xffffffffu, safe_lo, d));
        }

        // ---- Q' fragments of this item, prepared by the plan launch ---------------------------
        uint32_t qb[16][2];
        uint32_t qlo[16];
        float q_step[2] = {0.0f, 0.0f};
        {
            const uint32_t* qf = p.qfrag + ((size_t)(r * p.layout.local_kv_heads + kv_head) * p.q_groups_max + group) *
                                               (kQFragWords * 32) + lane;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                qb[i][0] = __ldg(qf + (2 * i) * 32);
                qb[i][1] = __ldg(qf + (2 * i + 1) * 32);
                qlo[i] = EXACT ? __ldg(qf + (32 + i) * 32) : 0u;
            }
            if (EXACT) {
                q_step[0] = __uint_as_float(__ldg(qf + 48 * 32));
                q_step[1] = __uint_as_float(__ldg(qf + 49 * 32));
            }
        }
        // ---- accumulators ----------------------------------------------------------------
        float o[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
        float m_run[2] = {-1e30f, -1e30f};
        float l_run[2] = {0.0f, 0.0f};

        // ---- page pipeline ---------------------------------------------------------------
        const int32_t* blocks = p.batch.block_tables + (size_t)r * p.batch.max_blocks_per_req;
        const uint8_t* k_head_base = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
        const uint8_t* v_head_base = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
        int32_t my_page = 0, next_page = 0;
        if (!SPARSE) {
            my_page = (lane < n_here) ? block_table_page(blocks, pg0 + lane, p.batch.max_blocks_per_req, kInStream) : 0;  // page ids of units [0, 32)
            next_page = (32 + lane < n_here) ? block_table_page(blocks, pg0 + 32 + lane, p.batch.max_blocks_per_req, kInStream) : 0;
        }
        // query-sparse: the token's selected list, its length and its position
        const int32_t* sel_phys = SPARSE ? p.sel_phys + (size_t)r * p.select_k : nullptr;
        const int32_t* sel_logical = SPARSE ? p.sel_logical + (size_t)r * p.select_k : nullptr;
        const int n_sel = SPARSE ? min(p.num_selected[r], p.select_k) : 0;

        fence_proxy_async();  // the staging writes above precede async-proxy writes to the ring
        auto issue = [&](int idx) {  // called by all lanes; lane 0 issues the four copies
            if (SPARSE) {
                // Unit idx = entries 4 (pg0 + idx) .. + 3 of the list.  Lane j < 4 takes entry j: a group of
                // four rows (528 bytes of K, 528 of V) lands at rows 4 j .. 4 j + 3 of the stage; a skipped
                // entry (negative id, past the list's end, or wholly after the token's position) copies
                // nothing and is masked below through the position word kept in the stage's padding.
                const int s = idx % STAGES;
                const uint32_t bar = bars + 8u * s;
                const uint32_t dst = ring + (uint32_t)s * kStageStride;
                const int gi = 4 * (pg0 + idx) + lane;
                int ph = -1, first_pos = 0x3fffffff;
                if (lane < 4 && gi < n_sel) {
                    ph = sel_phys[gi];
                    const int lg = sel_logical[gi];
                    if (ph >= 0 && 4 * lg <= g.ctx_before) first_pos = 4 * lg; else ph = -1;
                }
                const int n_valid = __popc(__ballot_sync(0xffffffffu, ph >= 0));
                pending |= 1u << s;
                if (lane == 0) mbar_expect_tx(bar, (uint32_t)n_valid * 8u * kTq4RowBytes);
                __syncwarp();
                if (lane < 4) {
                    sts32(dst + kHalfBytes + 4u * lane, (uint32_t)first_pos);
                    if (ph >= 0) {
                        const int page = pool_page(ph >> 2, kInStream);
                        const uint32_t row_off = (uint32_t)(ph & 3) * 4u * kTq4RowBytes;
                        bulk_g2s(dst + token_offset(4 * lane), k_head_base + (size_t)page * p.layout.k_page_stride_bytes + row_off,
                                 4u * kTq4RowBytes, bar);
                        bulk_g2s(dst + kRunStride + token_offset(4 * lane),
                                 v_head_base + (size_t)page * p.layout.v_page_stride_bytes + row_off, 4u * kTq4RowBytes, bar);
                    }
                }
                return;
            }
            const int32_t page = __shfl_sync(0xffffffffu, (idx & 32) ? next_page : my_page, idx & 31);
            pending |= 1u << (idx % STAGES);
            if (lane == 0) {
                const int s = idx % STAGES;
                const uint32_t bar = bars + 8u * s;
                const uint32_t dst = ring + (uint32_t)s * kStageStride;
                const uint8_t* ksrc = k_head_base + (size_t)page * p.layout.k_page_stride_bytes;
                const uint8_t* vsrc = v_head_base + (size_t)page * p.layout.v_page_stride_bytes;
                mbar_expect_tx(bar, 4 * kHalfBytes);
                bulk_g2s(dst, ksrc, kHalfBytes, bar);
                bulk_g2s(dst + kHalfStride, ksrc + kHalfBytes, kHalfBytes, bar);
                bulk_g2s(dst + kRunStride, vsrc, kHalfBytes, bar);
                bulk_g2s(dst + kRunStride + kHalfStride, vsrc + kHalfBytes, kHalfBytes, bar);
            }
        };
        // `my_page` holds ids for units [64 c, 64 c + 32), `next_page` for [64 c + 32, 64 c + 64).
#pragma unroll 1
        for (int i = 0; i < STAGES - 1 && i < n_here; ++i) issue(i);
        if (SPARSE) __syncwarp();   // the position words written by lanes 0-3 are read by all lanes

#pragma unroll 1
        for (int i = 0; i < n_here; ++i) {
            // refill page-id registers every 32 units, one window ahead
            if (!SPARSE && (i & 31) == 0 && i > 0) {
                const int base = i + 32;  // ids for [i+32, i+64) replace the window just consumed
                const int32_t fresh = (base + lane < n_here) ? block_table_page(blocks, pg0 + base + lane, p.batch.max_blocks_per_req, kInStream) : 0;
                if (i & 32) my_page = fresh; else next_page = fresh;
            }
            {
                const int ahead = i + STAGES - 1;
                if (ahead < n_here) issue(ahead);
            }
            const int s = i % STAGES;
            if (!mbar_wait(bars + 8u * s, (phase_bits >> s) & 1u)) { failed = true; break; }
            phase_bits ^= 1u << s;
            pending &= ~(1u << s);

            const uint32_t kst = ring + (uint32_t)s * kStageStride;
            const uint32_t vst = kst + kRunStride;
            const int kv_base = (pg0 + i) << 4;
            bool full = (kv_base >= safe_lo) && (kv_base + 15 <= safe_hi);
            const uint32_t ptok = page_token(i);
            // query-sparse: position of the first row of the two groups this lane's keys sit in
            int pos_a_sparse = 0, pos_b_sparse = 0;
            if (SPARSE) {
                const uint32_t pw = kst + kHalfBytes;
                const int f0 = (int)lds32_dep(pw, ptok), f1 = (int)lds32_dep(pw + 4, ptok);
                const int f2 = (int)lds32_dep(pw + 8, ptok), f3 = (int)lds32_dep(pw + 12, ptok);
                full = max(max(f0, f1), max(f2, f3)) + 3 <= safe_hi;
                pos_a_sparse = ((key_a >> 3) ? f2 : f0) + (key_a & 3);
                pos_b_sparse = ((key_a >> 3) ? f3 : f1) + (key_a & 3);
            }
#define W34_LDS(addr) lds32_dep(addr, ptok)
#define W34_LUT(word, k) lds32_lut(__byte_perm((word), lut_lane, 0x7604 + ((k) << 4)))
#define W34_LUTK(word, k) lds64_lut(__byte_perm((word), lutk_lane, 0x7604 + ((k) << 4)))

            // ---- S^T = K Q'^T, one accumulator per 128-half ------------------------------
            float sa[2][4], sl[2][4], sk[2][4];  // value, query-residual and key-residual chains are independent
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                sa[h][0] = sa[h][1] = sa[h][2] = sa[h][3] = 0.0f;
                sl[h][0] = sl[h][1] = sl[h][2] = sl[h][3] = 0.0f;
                sk[h][0] = sk[h][1] = sk[h][2] = sk[h][3] = 0.0f;
            }
            const uint32_t krow_a = kst + token_offset(key_a);
            const uint32_t krow_b = krow_a + 4u * kTq4RowBytes;
            const uint32_t ka0 = W34_LDS(krow_a), ka16 = W34_LDS(krow_a + 64);
            const uint32_t kb0 = W34_LDS(krow_b), kb16 = W34_LDS(krow_b + 64);
#pragma unroll
            for (int s8 = 0; s8 < 8; ++s8) {
                const int half = s8 >> 2;
                uint32_t wa, wb;
                if (half == 0) {
                    const uint32_t off = 4u * (4u * tig + (s8 & 3));
                    wa = W34_LDS(krow_a + off);
                    wb = W34_LDS(krow_b + off);
                    if ((s8 & 3) == 0 && tig == 0) {
                        wa = (ka0 >> 16) | (ka16 << 16);
                        wb = (kb0 >> 16) | (kb16 << 16);
                    }
                } else {
                    const uint32_t off = 4u * (17u + 4u * tig + (s8 & 3));
                    wa = W34_LDS(krow_a + off);
                    wb = W34_LDS(krow_b + off);
                }
#pragma unroll
                for (int hk = 0; hk < 2; ++hk) {
                    uint32_t a0, a1, a2, a3;
                    if (EXACT) {
                        const uint2 e0 = W34_LUTK(wa, 2 * hk), e1 = W34_LUTK(wb, 2 * hk);
                        const uint2 e2 = W34_LUTK(wa, 2 * hk + 1), e3 = W34_LUTK(wb, 2 * hk + 1);
                        a0 = e0.x; a1 = e1.x; a2 = e2.x; a3 = e3.x;
                        mma16816(sk[half], e0.y, e1.y, e2.y, e3.y, qb[2 * s8 + hk][0], qb[2 * s8 + hk][1]);
                    } else {
                        a0 = W34_LUT(wa, 2 * hk);
                        a1 = W34_LUT(wb, 2 * hk);
                        a2 = W34_LUT(wa, 2 * hk + 1);
                        a3 = W34_LUT(wb, 2 * hk + 1);
                    }
                    const uint32_t ql = qlo[2 * s8 + hk];
                    if ((s8 & 3) == 0 && hk == 0) {
                        mma16816_zero(sa[half], a0, a1, a2, a3, qb[2 * s8 + hk][0], qb[2 * s8 + hk][1]);
                    } else {
                        mma16816(sa[half], a0, a1, a2, a3, qb[2 * s8 + hk][0], qb[2 * s8 + hk][1]);
                    }
                    if (EXACT) {   // residual bytes -> fp16 pairs: byte b becomes the half 0x00bb = b x 2^-24
                        mma16816(sl[half], a0, a1, a2, a3, __byte_perm(ql, 0, 0x4140), __byte_perm(ql, 0, 0x4342));
                    }
                }
            }
            // scales of this lane's two keys
            const float dka0 = __half2float(__ushort_as_half((unsigned short)(ka0 & 0xffffu)));
            const float dka1 = __half2float(__ushort_as_half((unsigned short)(ka16 >> 16)));
            const float dkb0 = __half2float(__ushort_as_half((unsigned short)(kb0 & 0xffffu)));
            const float dkb1 = __half2float(__ushort_as_half((unsigned short)(kb16 >> 16)));
            // sc[0],sc[1]: token key_a, rows 2tig, 2tig+1;  sc[2],sc[3]: token key_a + 4
            if (EXACT) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) sa[h][x] += sl[h][x] * q_step[x & 1] + sk[h][x] * (1.0f / kResidualScale);
                }
            }
            float sc[4];
            sc[0] = dka0 * sa[0][0] + dka1 * sa[1][0];
            sc[1] = dka0 * sa[0][1] + dka1 * sa[1][1];
            sc[2] = dkb0 * sa[0][2] + dkb1 * sa[1][2];
            sc[3] = dkb0 * sa[0][3] + dkb1 * sa[1][3];

            const uint32_t vrow_a = vst + token_offset(key_a);  // V rows of the same two tokens
            const uint32_t va0 = W34_LDS(vrow_a), va16 = W34_LDS(vrow_a + 64);
            const uint32_t vb0 = W34_LDS(vrow_a + 4u * kTq4RowBytes), vb16 = W34_LDS(vrow_a + 4u * kTq4RowBytes + 64);
            float dva0 = __half2float(__ushort_as_half((unsigned short)(va0 & 0xffffu)));
            float dva1 = __half2float(__ushort_as_half((unsigned short)(va16 >> 16)));
            float dvb0 = __half2float(__ushort_as_half((unsigned short)(vb0 & 0xffffu)));
            float dvb1 = __half2float(__ushort_as_half((unsigned short)(vb16 >> 16)));

            bool msk[4] = {false, false, false, false};
            if (!full) {
                const int pos_a = SPARSE ? pos_a_sparse : kv_base + key_a, pos_b = SPARSE ? pos_b_sparse : pos_a + 4;
                msk[0] = !(pos_a >= rmin[0] && pos_a <= rmax[0]);
                msk[1] = !(pos_a >= rmin[1] && pos_a <= rmax[1]);
                msk[2] = !(pos_b >= rmin[0] && pos_b <= rmax[0]);
                msk[3] = !(pos_b >= rmin[1] && pos_b <= rmax[1]);
#pragma unroll
                for (int x = 0; x < 4; ++x) if (msk[x]) sc[x] = -1e30f;
            }
            // ---- online softmax over the 16 keys, per query row -----------------------------
            float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
            for (int d = 4; d < 32; d <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, d));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, d));
            }
            const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
            const bool grew = (mn0 > m_run[0]) || (mn1 > m_run[1]);
            if (__any_sync(0xffffffffu, grew)) {
                const float al0 = ex2(m_run[0] - mn0), al1 = ex2(m_run[1] - mn1);
                l_run[0] *= al0;
                l_run[1] *= al1;
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    o[t][0] *= al0; o[t][1] *= al1; o[t][2] *= al0; o[t][3] *= al1;
                }
                m_run[0] = mn0;
                m_run[1] = mn1;
            }
            float pr[4];
            pr[0] = ex2(sc[0] - mn0);
            pr[1] = ex2(sc[1] - mn1);
            pr[2] = ex2(sc[2] - mn0);
            pr[3] = ex2(sc[3] - mn1);
            if (!full) {
#pragma unroll
                for (int x = 0; x < 4; ++x) if (msk[x]) pr[x] = 0.0f;
                // a key no row can see may hold never-written bytes: keep its scale finite
                if (msk[0] && msk[1]) { dva0 = 0.0f; dva1 = 0.0f; }
                if (msk[2] && msk[3]) { dvb0 = 0.0f; dvb1 = 0.0f; }
            }
            bool peaked = false;
            if (EXACT) {
                // the exact build keeps the row totals (every lane of a row holds the same l) for the test
                float ps0 = pr[0] + pr[2], ps1 = pr[1] + pr[3];
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    ps0 += __shfl_xor_sync(0xffffffffu, ps0, d);
                    ps1 += __shfl_xor_sync(0xffffffffu, ps1, d);
                }
                l_run[0] += ps0;
                l_run[1] += ps1;
                // (rows that do not exist score 0 against their zero query; they must not count as peaks)
                const bool pk0 = rvalid[0] && fmaxf(pr[0], pr[2]) > kPeakedWeight * l_run[0];
                const bool pk1 = rvalid[1] && fmaxf(pr[1], pr[3]) > kPeakedWeight * l_run[1];
                peaked = __any_sync(0xffffffffu, pk0 || pk1);
            } else {
                l_run[0] += pr[0] + pr[2];
                l_run[1] += pr[1] + pr[3];
            }
            // P * d_v per half as B fragments (k = key, n = query row); the exact build adds the fp16
            // rounding residual of P * d_v as a second fragment.
            uint32_t pb[2][2], pl[2][2] = {{0u, 0u}, {0u, 0u}};
            const float pd[2][4] = {{pr[0] * dva0, pr[1] * dva0, pr[2] * dvb0, pr[3] * dvb0},
                                    {pr[0] * dva1, pr[1] * dva1, pr[2] * dvb1, pr[3] * dvb1}};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const __half2 hi = __floats2half2_rn(pd[h][2 * x], pd[h][2 * x + 1]);
                    pb[h][x] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hi));
                    if (EXACT) {
                        const float2 hf = __half22float2(hi);
                        const __half2 lo = __floats2half2_rn(pd[h][2 * x] - hf.x, pd[h][2 * x + 1] - hf.y);
                        pl[h][x] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&lo));
                    }
                }
            }

            // ---- O^T += V^T P^T -----------------------------------------------------------
            // step i4: half i4 >> 1, virtual word 4 (gid >> 1) + (gid & 1) + 2 (i4 & 1);
            // tokens kv0 + {0, 1, 4, 5}
            const uint32_t vr = vst + token_offset(kv0);
            const uint32_t vwb = 4u * (uint32_t)(gid >> 1) + (uint32_t)(gid & 1);
            // Every page: V P + V P_residual.  A peaked page then adds V_residual P in a second pass over
            // its V codes (the K table holds the residuals).
            // The second pass is a branch of its own so that the common pass stays one basic block
            // with the softmax above it, whose latencies its loads and look-ups fill.
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                const int half = i4 >> 1;
                uint32_t w[4];
                const uint32_t off = 4u * ((half ? 17u : 0u) + vwb + 2u * (i4 & 1));
                w[0] = W34_LDS(vr + off);
                w[1] = W34_LDS(vr + kTq4RowBytes + off);
                w[2] = W34_LDS(vr + 4u * kTq4RowBytes + off);
                w[3] = W34_LDS(vr + 5u * kTq4RowBytes + off);
                if (i4 == 0 && gid == 0) {  // virtual word 0 of half 0: splice (W0 >> 16) | (W16 << 16)
                    w[0] = (w[0] >> 16) | (W34_LDS(vr + 64) << 16);
                    w[1] = (w[1] >> 16) | (W34_LDS(vr + kTq4RowBytes + 64) << 16);
                    w[2] = (w[2] >> 16) | (W34_LDS(vr + 4u * kTq4RowBytes + 64) << 16);
                    w[3] = (w[3] >> 16) | (W34_LDS(vr + 5u * kTq4RowBytes + 64) << 16);
                }
                // byte t of lo_ab -> (V[ka][e=2t], V[kb][e=2t]); of hi_ab -> e = 2t+1
                const uint32_t lo_ab = (w[0] & 0x0f0f0f0fu) | ((w[1] << 4) & 0xf0f0f0f0u);
                const uint32_t hi_ab = ((w[0] >> 4) & 0x0f0f0f0fu) | (w[1] & 0xf0f0f0f0u);
                const uint32_t lo_cd = (w[2] & 0x0f0f0f0fu) | ((w[3] << 4) & 0xf0f0f0f0u);
                const uint32_t hi_cd = ((w[2] >> 4) & 0x0f0f0f0fu) | (w[3] & 0xf0f0f0f0u);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const uint32_t a0 = W34_LUT(lo_ab, t);
                    const uint32_t a1 = W34_LUT(hi_ab, t);
                    const uint32_t a2 = W34_LUT(lo_cd, t);
                    const uint32_t a3 = W34_LUT(hi_cd, t);
                    mma16816(o[4 * i4 + t], a0, a1, a2, a3, pb[half][0], pb[half][1]);
                    if (EXACT) mma16816(o[4 * i4 + t], a0, a1, a2, a3, pl[half][0], pl[half][1]);
                }
            }
            if (peaked) {
                // P * d_v / kResidualScale, the partner of the scaled centroid residuals
                uint32_t ps[2][2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const __half2 sc2 = __floats2half2_rn(pd[h][2 * x] * (1.0f / kResidualScale),
                                                              pd[h][2 * x + 1] * (1.0f / kResidualScale));
                        ps[h][x] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&sc2));
                    }
                }
                auto pv_fix = [&]() {
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const int half = i4 >> 1;
                        uint32_t w[4];
                        const uint32_t off = 4u * ((half ? 17u : 0u) + vwb + 2u * (i4 & 1));
                        w[0] = W34_LDS(vr + off);
                        w[1] = W34_LDS(vr + kTq4RowBytes + off);
                        w[2] = W34_LDS(vr + 4u * kTq4RowBytes + off);
                        w[3] = W34_LDS(vr + 5u * kTq4RowBytes + off);
                        if (i4 == 0 && gid == 0) {
                            w[0] = (w[0] >> 16) | (W34_LDS(vr + 64) << 16);
                            w[1] = (w[1] >> 16) | (W34_LDS(vr + kTq4RowBytes + 64) << 16);
                            w[2] = (w[2] >> 16) | (W34_LDS(vr + 4u * kTq4RowBytes + 64) << 16);
                            w[3] = (w[3] >> 16) | (W34_LDS(vr + 5u * kTq4RowBytes + 64) << 16);
                        }
                        const uint32_t lo_ab = (w[0] & 0x0f0f0f0fu) | ((w[1] << 4) & 0xf0f0f0f0u);
                        const uint32_t hi_ab = ((w[0] >> 4) & 0x0f0f0f0fu) | (w[1] & 0xf0f0f0f0u);
                        const uint32_t lo_cd = (w[2] & 0x0f0f0f0fu) | ((w[3] << 4) & 0xf0f0f0f0u);
                        const uint32_t hi_cd = ((w[2] >> 4) & 0x0f0f0f0fu) | (w[3] & 0xf0f0f0f0u);
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint2 e0 = W34_LUTK(lo_ab, t), e1 = W34_LUTK(hi_ab, t);
                            const uint2 e2 = W34_LUTK(lo_cd, t), e3 = W34_LUTK(hi_cd, t);
                            mma16816(o[4 * i4 + t], e0.y, e1.y, e2.y, e3.y, ps[half][0], ps[half][1]);
                        }
                    }
                };
                pv_fix();
            }
#undef W34_LUT
#undef W34_LUTK
#undef W34_LDS
            __syncwarp();  // every lane is done with stage s before it is refilled
        }

        // ---- drain: nothing of this segment may still be in flight ------------------------
        // (every issued stage was waited for above unless a wait gave up)
        if (failed) {
            // wait, bounded, for copies already issued so the CTA does not exit under them
            for (int s = 0; s < STAGES; ++s) {
                if (pending & (1u << s)) (void)mbar_wait(bars + 8u * s, (phase_bits >> s) & 1u);
            }
            if (lane == 0) atomicOr(&hdr->status, 1);
            break;
        }

        // ---- write the partial: natural column order, through the idle ring ------------------
        // l: add the 8 lanes (gid) that share a query row (the exact build already holds row totals)
        if (!EXACT) {
#pragma unroll
            for (int d = 4; d < 32; d <<= 1) {
                l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
                l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
            }
        }
        float* stage_o = reinterpret_cast<float*>(ring_gen);  // [8 rows][256]
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const int half = i4 >> 1, vw = 4 * (gid >> 1) + (gid & 1) + 2 * (i4 & 1);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int ca = vword_col(half, vw, 2 * t), cb = vword_col(half, vw, 2 * t + 1);
                stage_o[(2 * tig) * kHeadDim + ca] = o[4 * i4 + t][0];
                stage_o[(2 * tig + 1) * kHeadDim + ca] = o[4 * i4 + t][1];
                stage_o[(2 * tig) * kHeadDim + cb] = o[4 * i4 + t][2];
                stage_o[(2 * tig + 1) * kHeadDim + cb] = o[4 * i4 + t][3];
            }
        }
        __syncwarp();
        if (slot < p.max_slots) {
            float* dst = partials + (size_t)slot * kPartialFloats;
            const float4* src4 = reinterpret_cast<const float4*>(stage_o);
            float4* dst4 = reinterpret_cast<float4*>(dst);
#pragma unroll
            for (int k = 0; k < (kRowsPerGroup * kHeadDim / 4) / 32; ++k) dst4[k * 32 + lane] = src4[k * 32 + lane];
            if (gid == 0) {
                dst[kRowsPerGroup * kHeadDim + 2 * tig] = m_run[0];
                dst[kRowsPerGroup * kHeadDim + 2 * tig + 1] = m_run[1];
                dst[kRowsPerGroup * kHeadDim + kRowsPerGroup + 2 * tig] = l_run[0];
                dst[kRowsPerGroup * kHeadDim + kRowsPerGroup + 2 * tig + 1] = l_run[1];
            }
        }
        __syncwarp();
        u += n_here;
    }
}

// ---------------------------------------------------------------------------------------
// Team kernel: 8 * NT query rows (GQA heads x draft tokens of a verify step) share ONE pass
// over the KV pages.  A team is four warps; warp t owns a quarter of the 256 channels (half
// t >> 1 of the row, every other pair of 8-channel words), for the score product and for the
// output alike, so every code is looked up once per page however many query rows read it and
// each looked-up fragment feeds NT MMAs.  The team meets once per page, after the partial
// scores: they are summed through shared memory by the warp that owns an 8-row tile, which
// runs its online softmax and publishes P fragments and rescale factors (double-buffered);
// the output product of a page runs after the next meeting, so one page's softmax overlaps the
// next page's score product.  Three teams per CTA, one CTA per SM, each team with its own ring.
// ---------------------------------------------------------------------------------------
constexpr int kTeams = 3;
constexpr int kTeamWarps = 4;
constexpr int kTeamStages = 8;

__device__ __forceinline__ void team_barrier(int team) {
    asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(kTeamWarps * 32) : "memory");
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128f(uint32_t addr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts64f(uint32_t addr, float2 v) {
    asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(addr), "f"(v.x), "f"(v.y) : "memory");
}

// Carves [lo, hi) minus the 64 KB table at `lut` into chunks: first fit below the table, then above.
struct SmemCarver {
    uint32_t a_cur, a_end, b_cur, b_end;
    bool ok;
    __device__ SmemCarver(uint32_t lo, uint32_t lut, uint32_t hi)
        : a_cur(lo), a_end(lut), b_cur(lut + kLutBytes), b_end(hi), ok(lut + kLutBytes <= hi) {}
    __device__ uint32_t take(uint32_t bytes, uint32_t align) {
        uint32_t a = (a_cur + align - 1) & ~(align - 1);
        if (a + bytes <= a_end) { a_cur = a + bytes; return a; }
        uint32_t b = (b_cur + align - 1) & ~(align - 1);
        if (b + bytes <= b_end) { b_cur = b + bytes; return b; }
        ok = false;
        return b_end >= bytes ? b_end - bytes : 0;
    }
};

template <int NT>
__global__ void __launch_bounds__(kTeams * kTeamWarps * 32, 1) tq4_attention_team_kernel(const StreamParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int RG = 8 * NT;
    constexpr int PARTIAL = RG * kHeadDim + 2 * RG;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int team = wid >> 2, t = wid & 3;     // warp t of its team
    const int half = t >> 1, cset = t & 1;      // 128-half and word set owned by this warp
    const uint32_t win_lo = smem_u32(smem);
    const uint32_t win_hi = win_lo + p.smem_bytes;
    const uint32_t lut_addr = (win_lo + 0xffffu) & ~0xffffu;
    PlanHeader* hdr = reinterpret_cast<PlanHeader*>(p.scratch);

    SmemCarver carve(win_lo, lut_addr, win_hi);
    uint32_t ring = 0, sx = 0, px = 0, ax = 0, bars = 0;
    for (int tm = 0; tm < kTeams; ++tm) {
        const uint32_t r_ = carve.take(kTeamStages * kStageStride, 128);
        if (tm == team) ring = r_;
    }
    for (int tm = 0; tm < kTeams; ++tm) {
        // all three are double-buffered by page parity
        const uint32_t s_ = carve.take(2 * kTeamWarps * NT * 512, 16);   // partial scores [buf][warp][tile][lane] float4
        const uint32_t p_ = carve.take(2 * NT * 2 * 2 * 128, 16);         // P fragments [buf][tile][half][reg][lane]
        const uint32_t a_ = carve.take(2 * NT * 4 * 8, 8);                // rescale factors [buf][tile][tig] float2
        const uint32_t b_ = carve.take(kTeamStages * 8, 8);
        if (tm == team) { sx = s_; px = p_; ax = a_; bars = b_; }
    }
    if (!carve.ok) {
        if (threadIdx.x == 0) atomicOr(&hdr->status, 2);
        return;
    }
    uint8_t* ring_gen = smem + (ring - win_lo);

    for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
        const int byte = i >> 5, ln = i & 31;
        sts32(lut_addr + (uint32_t)(byte * 256 + ln * 4),
              pack_half2(kLutScale * tq4_centroid(byte & 15), kLutScale * tq4_centroid(byte >> 4)));
    }
    if (t == 0 && lane == 0) {
        for (int s = 0; s < kTeamStages; ++s) mbar_init(bars + 8u * s, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int R = p.batch.num_reqs;
    const int32_t* unit_prefix = plan_array(p.scratch, 0, R);
    const int32_t* item_prefix = plan_array(p.scratch, 1, R);
    const int32_t* page_lo_a = plan_array(p.scratch, 2, R);
    const int32_t* npages_a = plan_array(p.scratch, 3, R);
    const int32_t* ngroups_a = plan_array(p.scratch, 4, R);
    float* partials = reinterpret_cast<float*>(p.scratch + plan_bytes(R));

    const int worker = blockIdx.x * kTeams + team;
    const int per = hdr->units_per_warp;
    const int total_units = hdr->total_units;
    const long long u_ll = (long long)worker * per;
    if (per <= 0 || u_ll >= total_units) return;   // whole team leaves together
    int u = (int)u_ll;
    const int u_end = min(u + per, total_units);

    const int gid = lane >> 2, tig = lane & 3;
    const int key_a = (gid & 3) + 8 * (gid >> 2);
    const int kv0 = 2 * (tig & 1) + 8 * (tig >> 1);
    const uint32_t lut_lane = lut_addr + 4u * lane;
    // Softmax owners are rotated from team to team so that the schedulers, which each host one
    // warp of every team, share the softmax work evenly.
    const int tile = (t + 4 - (team & 3)) & 3;   // query tile this warp owns, if < NT
    const bool owner = tile < NT;
    uint32_t phase_bits = 0, pending = 0;
    bool failed = false;

    int r;
    {
        int lo = 0, hi = R;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (unit_prefix[mid] <= u) lo = mid; else hi = mid;
        }
        r = lo;
    }

    while (u < u_end) {
        while (unit_prefix[r + 1] <= u) ++r;
        const int npages = npages_a[r];
        const int ngroups = ngroups_a[r];
        const int in_req = u - unit_prefix[r];
        const int item = in_req / npages;
        const int page_in_item = in_req - item * npages;
        const int n_here = min(u_end - u, npages - page_in_item);
        const int kv_head = item / ngroups;
        const int group = item - kv_head * ngroups;
        const int pg0 = page_lo_a[r] + page_in_item;
        const int slot = worker + item_prefix[r] + item;
        const ReqGeom g = load_req(p.batch, r);
        const int rows_in_req = g.q_len * p.gqa;

        // ---- limits: this lane's two rows of the tile it owns, and the group-wide safe range ----
        int rmax[2] = {-1, -1}, rmin[2] = {0x7fffffff, 0x7fffffff};
        int safe_hi = 0x7fffffff, safe_lo = 0;
        for (int row = group * RG + lane; row < group * RG + RG; row += 32) {   // RG <= 32: one pass
            const int q_off = row / p.gqa;
            const bool ok = row < rows_in_req &&
                            (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
            if (ok) {
                safe_hi = row_max_kv(p.batch, g, q_off);
                safe_lo = row_min_kv(p.batch, g, q_off);
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            safe_hi = min(safe_hi, __shfl_xor_sync(0xffffffffu, safe_hi, d));
            safe_lo = max(safe_lo, __shfl_xor_sync(0xffffffffu, safe_lo, d));
        }
        if (owner) {
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int row = group * RG + 8 * tile + 2 * tig + x;
                const int q_off = row / p.gqa;
                const bool ok = row < rows_in_req &&
                                (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
                if (ok) { rmax[x] = row_max_kv(p.batch, g, q_off); rmin[x] = row_min_kv(p.batch, g, q_off); }
            }
        }

        // ---- stage Q' (fp16 [RG][256], pre-scaled) in the idle ring; warp t rotates rows t, t+4, ...
        __half* q_stage = reinterpret_cast<__half*>(ring_gen);
        for (int row8 = t; row8 < RG; row8 += kTeamWarps) {
            const int row = group * RG + row8;
            const int q_off = row / p.gqa;
            const int q_head = kv_head * p.gqa + (row - q_off * p.gqa);
            const bool ok = row < rows_in_req &&
                            (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
            float tv[8];
            if (ok) {
                const size_t q_base = ((size_t)(g.q_start + q_off) * p.num_q_heads + q_head) * kHeadDim;
#pragma unroll
                for (int j = 0; j < 8; ++j) tv[j] = apply_sign(load_act(p.q_in, q_base + lane + 32 * j, p.io_bf16), lane + 32 * j);
                wht256_lanes(tv, lane);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) tv[j] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) q_stage[row8 * kHeadDim + lane + 32 * j] = __float2half_rn(tv[j] * p.q_scale);
        }
        team_barrier(team);
        // B fragments: k-step ks = 2 j + hk covers elements 4 hk .. 4 hk + 3 of virtual word
        // vw_j = 2 cset + j + 4 tig of this warp's half.
        uint32_t qb[4][NT][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int vw = 2 * cset + j + 4 * tig;
#pragma unroll
            for (int hk = 0; hk < 2; ++hk) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int e = 4 * hk + 2 * x;
                        const __half lo = q_stage[(8 * nt + gid) * kHeadDim + vword_col(half, vw, e)];
                        const __half hi = q_stage[(8 * nt + gid) * kHeadDim + vword_col(half, vw, e + 1)];
                        qb[2 * j + hk][nt][x] = (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
                    }
                }
            }
        }
        team_barrier(team);   // everyone has its fragments before copies overwrite the staging area

        float o[4][NT][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) { o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.0f; }
        }
        float m_run[2] = {-1e30f, -1e30f};
        float l_run[2] = {0.0f, 0.0f};

        const int32_t* blocks = p.batch.block_tables + (size_t)r * p.batch.max_blocks_per_req;
        const uint8_t* k_head_base = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
        const uint8_t* v_head_base = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
        // page ids are only needed by the issuing warp (t == 0)
        int32_t my_page = (t == 0 && lane < n_here) ? block_table_page(blocks, pg0 + lane, p.batch.max_blocks_per_req, kInTeam) : 0;
        int32_t next_page = (t == 0 && 32 + lane < n_here) ? block_table_page(blocks, pg0 + 32 + lane, p.batch.max_blocks_per_req, kInTeam) : 0;

        fence_proxy_async();
        auto issue = [&](int idx) {
            pending |= 1u << (idx % kTeamStages);
            if (t == 0) {
                const int32_t page = __shfl_sync(0xffffffffu, (idx & 32) ? next_page : my_page, idx & 31);
                if (lane == 0) {
                    const int s = idx % kTeamStages;
                    const uint32_t bar = bars + 8u * s;
                    const uint32_t dst = ring + (uint32_t)s * kStageStride;
                    const uint8_t* ksrc = k_head_base + (size_t)page * p.layout.k_page_stride_bytes;
                    const uint8_t* vsrc = v_head_base + (size_t)page * p.layout.v_page_stride_bytes;
                    mbar_expect_tx(bar, 4 * kHalfBytes);
                    bulk_g2s(dst, ksrc, kHalfBytes, bar);
                    bulk_g2s(dst + kHalfStride, ksrc + kHalfBytes, kHalfBytes, bar);
                    bulk_g2s(dst + kRunStride, vsrc, kHalfBytes, bar);
                    bulk_g2s(dst + kRunStride + kHalfStride, vsrc + kHalfBytes, kHalfBytes, bar);
                }
            }
        };
        // The page ids of units [32 c, 32 c + 32) alternate between my_page (c even) and next_page
        // (c odd); a window is replaced once every unit in it has been issued.
#pragma unroll 1
        for (int i = 0; i < kTeamStages && i < n_here; ++i) issue(i);

        // One meeting per page.  Iteration i: partial scores of page i -> meet -> (output product
        // of page i - 1, whose P fragments the owners published before arriving) -> owners'
        // softmax of page i -> V look-ups of page i.  The softmax of one page thus overlaps the
        // score product of the next in the other warps.
        uint32_t av[4][4];
        auto pv_product = [&](int buf) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 al = lds64f(ax + (uint32_t)(buf * (NT * 32) + (nt * 4 + tig) * 8));
                const uint32_t pb0 = lds32(px + (uint32_t)(buf * (NT * 512) + nt * 512 + half * 256 + lane * 4));
                const uint32_t pb1 = lds32(px + (uint32_t)(buf * (NT * 512) + nt * 512 + half * 256 + 128 + lane * 4));
                if (__any_sync(0xffffffffu, al.x != 1.0f || al.y != 1.0f)) {
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        o[mt][nt][0] *= al.x; o[mt][nt][1] *= al.y; o[mt][nt][2] *= al.x; o[mt][nt][3] *= al.y;
                    }
                }
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) mma16816(o[mt][nt], av[mt][0], av[mt][1], av[mt][2], av[mt][3], pb0, pb1);
            }
        };

#pragma unroll 1
        for (int i = 0; i < n_here; ++i) {
            const int s = i % kTeamStages;
            const int buf = i & 1;
            if (!failed && !mbar_wait(bars + 8u * s, (phase_bits >> s) & 1u)) {
                failed = true;                      // results are void; keep meeting the team's barriers
                if (lane == 0) atomicOr(&hdr->status, 1);
            }
            phase_bits ^= 1u << s;
            pending &= ~(1u << s);

            const uint32_t kst = ring + (uint32_t)s * kStageStride;
            const uint32_t vst = kst + kRunStride;
            const int kv_base = (pg0 + i) << 4;
            const bool full = (kv_base >= safe_lo) && (kv_base + 15 <= safe_hi);
#define W34_LUT(word, k) lds32(__byte_perm((word), lut_lane, 0x7604 + ((k) << 4)))

            // ---- partial scores over this warp's 64 channels -------------------------------
            {
                float sa[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) { sa[nt][0] = sa[nt][1] = sa[nt][2] = sa[nt][3] = 0.0f; }
                const uint32_t krow_a = kst + token_offset(key_a);
                const uint32_t krow_b = krow_a + 4u * kTq4RowBytes;
                const uint32_t sw_a = lds32(krow_a + (half ? 64u : 0u));   // word holding this half's scale
                const uint32_t sw_b = lds32(krow_b + (half ? 64u : 0u));
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t off = 4u * ((half ? 17u : 0u) + 2u * cset + j + 4u * tig);
                    uint32_t wa = lds32(krow_a + off);
                    uint32_t wb = lds32(krow_b + off);
                    if (j == 0 && t == 0 && tig == 0) {   // virtual word 0 of half 0: splice
                        wa = (wa >> 16) | (lds32(krow_a + 64) << 16);
                        wb = (wb >> 16) | (lds32(krow_b + 64) << 16);
                    }
#pragma unroll
                    for (int hk = 0; hk < 2; ++hk) {
                        const uint32_t a0 = W34_LUT(wa, 2 * hk);
                        const uint32_t a1 = W34_LUT(wb, 2 * hk);
                        const uint32_t a2 = W34_LUT(wa, 2 * hk + 1);
                        const uint32_t a3 = W34_LUT(wb, 2 * hk + 1);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            mma16816(sa[nt], a0, a1, a2, a3, qb[2 * j + hk][nt][0], qb[2 * j + hk][nt][1]);
                        }
                    }
                }
                const float dka = __half2float(__ushort_as_half((unsigned short)(half ? (sw_a >> 16) : (sw_a & 0xffffu))));
                const float dkb = __half2float(__ushort_as_half((unsigned short)(half ? (sw_b >> 16) : (sw_b & 0xffffu))));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    sts128f(sx + (uint32_t)(buf * (kTeamWarps * NT * 512) + (t * NT + nt) * 512 + lane * 16),
                            make_float4(dka * sa[nt][0], dka * sa[nt][1], dkb * sa[nt][2], dkb * sa[nt][3]));
                }
            }
            team_barrier(team);   // scores of page i are in shared memory; so is everything of page i - 1

            // page i - 1 is finished by every warp once it has passed this point's output product,
            // which the NEXT meeting certifies: refill the stage of page i - 1 now that all warps
            // have passed the meeting of page i (they read stage i - 1 before arriving).
            if (i >= 1 && i - 1 + kTeamStages < n_here) {
                if (t == 0 && ((i - 1 + kTeamStages) & 31) == 0) {
                    // entering a new id window: the window being replaced was fully issued long ago
                    const int base = i - 1 + kTeamStages + 32;
                    const int32_t fresh = (base + lane < n_here) ? block_table_page(blocks, pg0 + base + lane, p.batch.max_blocks_per_req, kInTeam) : 0;
                    if ((i - 1 + kTeamStages) & 32) my_page = fresh; else next_page = fresh;
                }
                issue(i - 1 + kTeamStages);
            }
            if (i >= 1) pv_product(buf ^ 1);

            // ---- the owner of query tile t sums the partials and runs the online softmax -------
            if (owner) {
                float sc[4];
                {
                    const uint32_t sb = sx + (uint32_t)(buf * (kTeamWarps * NT * 512) + tile * 512 + lane * 16);
                    const float4 p0 = lds128f(sb + 0 * NT * 512);
                    const float4 p1 = lds128f(sb + 1 * NT * 512);
                    const float4 p2 = lds128f(sb + 2 * NT * 512);
                    const float4 p3 = lds128f(sb + 3 * NT * 512);
                    sc[0] = ((p0.x + p1.x) + p2.x) + p3.x;
                    sc[1] = ((p0.y + p1.y) + p2.y) + p3.y;
                    sc[2] = ((p0.z + p1.z) + p2.z) + p3.z;
                    sc[3] = ((p0.w + p1.w) + p2.w) + p3.w;
                }
                const uint32_t vrow_a = vst + token_offset(key_a);
                const uint32_t va0 = lds32(vrow_a), va16 = lds32(vrow_a + 64);
                const uint32_t vb0 = lds32(vrow_a + 4u * kTq4RowBytes), vb16 = lds32(vrow_a + 4u * kTq4RowBytes + 64);
                float dva0 = __half2float(__ushort_as_half((unsigned short)(va0 & 0xffffu)));
                float dva1 = __half2float(__ushort_as_half((unsigned short)(va16 >> 16)));
                float dvb0 = __half2float(__ushort_as_half((unsigned short)(vb0 & 0xffffu)));
                float dvb1 = __half2float(__ushort_as_half((unsigned short)(vb16 >> 16)));
                bool msk[4] = {false, false, false, false};
                if (!full) {
                    const int pos_a = kv_base + key_a, pos_b = pos_a + 4;
                    msk[0] = !(pos_a >= rmin[0] && pos_a <= rmax[0]);
                    msk[1] = !(pos_a >= rmin[1] && pos_a <= rmax[1]);
                    msk[2] = !(pos_b >= rmin[0] && pos_b <= rmax[0]);
                    msk[3] = !(pos_b >= rmin[1] && pos_b <= rmax[1]);
#pragma unroll
                    for (int x = 0; x < 4; ++x) if (msk[x]) sc[x] = -1e30f;
                }
                float mx0 = fmaxf(sc[0], sc[2]), mx1 = fmaxf(sc[1], sc[3]);
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, d));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, d));
                }
                const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
                const float al0 = ex2(m_run[0] - mn0), al1 = ex2(m_run[1] - mn1);  // 1 when the max did not grow
                l_run[0] *= al0;
                l_run[1] *= al1;
                m_run[0] = mn0;
                m_run[1] = mn1;
                float pr[4];
                pr[0] = ex2(sc[0] - mn0);
                pr[1] = ex2(sc[1] - mn1);
                pr[2] = ex2(sc[2] - mn0);
                pr[3] = ex2(sc[3] - mn1);
                if (!full) {
#pragma unroll
                    for (int x = 0; x < 4; ++x) if (msk[x]) pr[x] = 0.0f;
                    if (msk[0] && msk[1]) { dva0 = 0.0f; dva1 = 0.0f; }
                    if (msk[2] && msk[3]) { dvb0 = 0.0f; dvb1 = 0.0f; }
                }
                l_run[0] += pr[0] + pr[2];
                l_run[1] += pr[1] + pr[3];
                const uint32_t pbase = px + (uint32_t)(buf * (NT * 512) + tile * 512 + lane * 4);
                sts32(pbase + 0, movmatrix_trans(pack_half2(pr[0] * dva0, pr[1] * dva0)));
                sts32(pbase + 128, movmatrix_trans(pack_half2(pr[2] * dvb0, pr[3] * dvb0)));
                sts32(pbase + 256, movmatrix_trans(pack_half2(pr[0] * dva1, pr[1] * dva1)));
                sts32(pbase + 384, movmatrix_trans(pack_half2(pr[2] * dvb1, pr[3] * dvb1)));
                if (gid == 0) sts64f(ax + (uint32_t)(buf * (NT * 32) + (tile * 4 + tig) * 8), make_float2(al0, al1));
            }

            // ---- V look-ups of page i (its product runs after the next meeting) ----------------
            {
                const uint32_t vr = vst + token_offset(kv0);
                const uint32_t vw = 4u * (uint32_t)(gid >> 1) + (uint32_t)(gid & 1) + 2u * cset;
                const uint32_t off = 4u * ((half ? 17u : 0u) + vw);
                uint32_t w[4];
                w[0] = lds32(vr + off);
                w[1] = lds32(vr + kTq4RowBytes + off);
                w[2] = lds32(vr + 4u * kTq4RowBytes + off);
                w[3] = lds32(vr + 5u * kTq4RowBytes + off);
                if (t == 0 && gid == 0) {
                    w[0] = (w[0] >> 16) | (lds32(vr + 64) << 16);
                    w[1] = (w[1] >> 16) | (lds32(vr + kTq4RowBytes + 64) << 16);
                    w[2] = (w[2] >> 16) | (lds32(vr + 4u * kTq4RowBytes + 64) << 16);
                    w[3] = (w[3] >> 16) | (lds32(vr + 5u * kTq4RowBytes + 64) << 16);
                }
                const uint32_t lo_ab = (w[0] & 0x0f0f0f0fu) | ((w[1] << 4) & 0xf0f0f0f0u);
                const uint32_t hi_ab = ((w[0] >> 4) & 0x0f0f0f0fu) | (w[1] & 0xf0f0f0f0u);
                const uint32_t lo_cd = (w[2] & 0x0f0f0f0fu) | ((w[3] << 4) & 0xf0f0f0f0u);
                const uint32_t hi_cd = ((w[2] >> 4) & 0x0f0f0f0fu) | (w[3] & 0xf0f0f0f0u);
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    av[mt][0] = W34_LUT(lo_ab, mt);
                    av[mt][1] = W34_LUT(hi_ab, mt);
                    av[mt][2] = W34_LUT(lo_cd, mt);
                    av[mt][3] = W34_LUT(hi_cd, mt);
                }
            }
#undef W34_LUT
        }
        team_barrier(team);   // the owners' last softmax is published
        if (n_here > 0) pv_product((n_here - 1) & 1);

        // ---- write the partial of this segment ------------------------------------------------
        if (slot < p.max_slots) {
            float* dst = partials + (size_t)slot * PARTIAL;
            const int vw = 4 * (gid >> 1) + (gid & 1) + 2 * cset;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const int ca = vword_col(half, vw, 2 * mt), cb = vword_col(half, vw, 2 * mt + 1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int r0 = 8 * nt + 2 * tig;
                    dst[r0 * kHeadDim + ca] = o[mt][nt][0];
                    dst[(r0 + 1) * kHeadDim + ca] = o[mt][nt][1];
                    dst[r0 * kHeadDim + cb] = o[mt][nt][2];
                    dst[(r0 + 1) * kHeadDim + cb] = o[mt][nt][3];
                }
            }
            if (owner) {
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
                    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
                }
                if (gid == 0) {
                    const int r0 = 8 * tile + 2 * tig;
                    dst[RG * kHeadDim + r0] = m_run[0];
                    dst[RG * kHeadDim + r0 + 1] = m_run[1];
                    dst[RG * kHeadDim + RG + r0] = l_run[0];
                    dst[RG * kHeadDim + RG + r0 + 1] = l_run[1];
                }
            }
        }
        team_barrier(team);   // the staging area is rewritten by the next segment
        u += n_here;
    }
    if (failed) {
        for (int s = 0; s < kTeamStages; ++s) {
            if (pending & (1u << s)) (void)mbar_wait(bars + 8u * s, (phase_bits >> s) & 1u);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Helpers shared by the tile-based kernels (tcgen05 prefill, uncompressed bf16 KV).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

W34_BOUNDS_HOST_HOOKS(attention)

}  // namespace w34
#include "tq4_prefill_tc.cuh"
#include "tq4_prefill_exact.cuh"
namespace w34 {

// Row triple written when the caller merges across page shards itself: 256 un-normalised
// accumulator values in the rotated domain (in lookup-table units), then m (log2 units of the
// pre-scaled scores) and l.
constexpr int kRowTripleFloats = kHeadDim + 2;

// One block of MW warps per (token, q head): warp w combines the partials w, w + MW, ... of the
// row with an online softmax merge, the MW results are combined through shared memory, then
// either normalise + inverse rotation + fp16 store, or (PARTIAL_OUT) store the merged
// (acc, m, l) triple for a cross-shard merge.  MW = 4 for batches; a long single sequence has
// hundreds of partials per row and only a few rows, for which MW = 32.
template <bool PARTIAL_OUT, int MW>
__global__ void __launch_bounds__(MW * 32) tq4_attention_merge_kernel(const StreamParams p) {
    __shared__ float s_acc[MW][kHeadDim];
    __shared__ float s_m[MW], s_l[MW];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long row_ll = blockIdx.x;
    int tok = (int)(row_ll / p.num_q_heads);
    const int q_head = (int)(row_ll % p.num_q_heads);
    if (p.rows_from_first_token) {   // a part of a larger batch: its tokens start at query_start_loc[0]
        tok += p.batch.query_start_loc[0];
        if (tok >= p.batch.query_start_loc[p.batch.num_reqs]) return;   // the grid is sized by max_q_len
    }
    // A row that takes no part (masked token or request, rows the plan dropped) leaves attn_out
    // untouched; as a triple it is written as "no keys" (l = 0), which the cross-shard merges skip.
    auto skip_row = [&]() {
        if (PARTIAL_OUT && wid == 0) {
            float* dst = p.triple_out + ((size_t)tok * p.num_q_heads + q_head) * (kHeadDim + 2);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[lane + 32 * j] = 0.0f;
            if (lane == 0) { dst[kHeadDim] = -1e30f; dst[kHeadDim + 1] = 0.0f; }
        }
        if (!PARTIAL_OUT && wid == 0 && p.sel_phys != nullptr) {   // query-sparse: masked rows are zeros
#pragma unroll
            for (int j = 0; j < 8; ++j) store_act(p.attn_out, ((size_t)tok * p.num_q_heads + q_head) * kHeadDim + lane + 32 * j, 0.0f, p.io_bf16);
        }
    };
    if (p.batch.valid_token_mask != nullptr && p.batch.valid_token_mask[tok] == 0) { skip_row(); return; }
    const int R = p.batch.num_reqs;
    const int r = p.sel_phys != nullptr ? tok : find_request(p.batch.query_start_loc, R, tok);
    if (r < 0) { skip_row(); return; }
    if (p.batch.valid_req_mask != nullptr && p.batch.valid_req_mask[r] == 0) { skip_row(); return; }

    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.scratch);
    const int32_t* unit_prefix = plan_array(p.scratch, 0, R);
    const int32_t* item_prefix = plan_array(p.scratch, 1, R);
    const int32_t* npages_a = plan_array(p.scratch, 3, R);
    const int32_t* ngroups_a = plan_array(p.scratch, 4, R);
    const float* partials = reinterpret_cast<const float*>(p.scratch + plan_bytes(R));

    const int kv_head = q_head / p.gqa;
    const int row_in_req = (tok - (p.sel_phys != nullptr ? r : p.batch.query_start_loc[r])) * p.gqa + (q_head - kv_head * p.gqa);
    const int rpg = p.rows_per_group;
    const int part_floats = rpg * kHeadDim + 2 * rpg;
    const int group = row_in_req / rpg, row8 = row_in_req - group * rpg;
    if (group >= ngroups_a[r]) { skip_row(); return; }  // rows the plan dropped (q_len above the declared max_q_len)
    const int item = kv_head * ngroups_a[r] + group;
    const int npages = npages_a[r];
    const int per = hdr->units_per_warp;

    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float l_tot = 0.0f;
    float m_tot = -1e30f;
    if (npages > 0 && per > 0) {
        const int us = unit_prefix[r] + item * npages;
        const int w_first = us / per, w_last = (us + npages - 1) / per;
        const float* base = partials + (size_t)(w_first + item_prefix[r] + item) * part_floats;
        const int nparts = w_last - w_first + 1;
        // this warp's partials: wid, wid + MW, ...; lanes fetch up to 32 (m, l) pairs at once so
        // that the accumulation runs over independent loads
        for (int c0 = wid; c0 < nparts; c0 += 32 * MW) {
            const int mine = c0 + MW * lane;
            float m_s = -1e30f, l_s = 0.0f;
            if (mine < nparts) {
                const float* ps = base + (size_t)mine * part_floats + rpg * kHeadDim;
                l_s = ps[rpg + row8];
                m_s = (l_s > 0.0f) ? ps[row8] : -1e30f;
            }
            float m_chunk = m_s;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) m_chunk = fmaxf(m_chunk, __shfl_xor_sync(0xffffffffu, m_chunk, d));
            const float m_new = fmaxf(m_tot, m_chunk);
            const float rescale = ex2(m_tot - m_new);
            l_tot *= rescale;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] *= rescale;
            m_tot = m_new;
            const float w_s = (l_s > 0.0f) ? ex2(m_s - m_tot) : 0.0f;
            float lw = l_s * w_s;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) lw += __shfl_xor_sync(0xffffffffu, lw, d);
            l_tot += lw;
            const int n_here = min(32, (nparts - c0 + MW - 1) / MW);
#pragma unroll 4
            for (int sidx = 0; sidx < n_here; ++sidx) {
                const float wgt = __shfl_sync(0xffffffffu, w_s, sidx);
                const float* pa = base + (size_t)(c0 + MW * sidx) * part_floats + row8 * kHeadDim;
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += pa[lane + 32 * j] * wgt;
            }
        }
    }
    // combine the warps
#pragma unroll
    for (int j = 0; j < 8; ++j) s_acc[wid][lane + 32 * j] = acc[j];
    if (lane == 0) { s_m[wid] = m_tot; s_l[wid] = l_tot; }
    __syncthreads();
    if (wid != 0) return;
    m_tot = s_m[0];
#pragma unroll
    for (int w = 1; w < MW; ++w) m_tot = fmaxf(m_tot, s_m[w]);
    l_tot = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 4
    for (int w = 0; w < MW; ++w) {
        const float wgt = (s_l[w] > 0.0f) ? ex2(s_m[w] - m_tot) : 0.0f;
        l_tot += s_l[w] * wgt;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += s_acc[w][lane + 32 * j] * wgt;
    }
    if (PARTIAL_OUT) {
        float* dst = p.triple_out + ((size_t)tok * p.num_q_heads + q_head) * kRowTripleFloats;
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[lane + 32 * j] = acc[j];
        if (lane == 0) { dst[kHeadDim] = m_tot; dst[kHeadDim + 1] = l_tot; }
        return;
    }
    const size_t out_base = ((size_t)tok * p.num_q_heads + q_head) * kHeadDim;
    if (p.natural) {
        const float inv = (l_tot > 0.0f) ? (1.0f / l_tot) : 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= inv;
        apply_output_gate(acc, p.og, out_base, lane, p.io_bf16);
#pragma unroll
        for (int j = 0; j < 8; ++j) store_act(p.attn_out, out_base + lane + 32 * j, acc[j], p.io_bf16);
        return;
    }
    const float inv_l = (l_tot > 0.0f) ? (1.0f / (l_tot * kLutScale)) : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv_l;
    wht256_lanes(acc, lane);
    store_output_row(p.attn_out, out_base, acc, lane, p.io_bf16, p.og);
}

// Cross-shard merge: parts is [num_parts][rows][258]; one warp per row.
__global__ void __launch_bounds__(128) tq4_attention_merge_shards_kernel(
    const float* __restrict__ parts, int num_parts, long long rows, void* __restrict__ attn_out, int io_bf16) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 4 + wid;
    if (row >= rows) return;
    float m_tot = -1e30f;
    for (int s = 0; s < num_parts; ++s) {
        const float* t = parts + ((size_t)s * rows + row) * kRowTripleFloats;
        if (t[kHeadDim + 1] > 0.0f) m_tot = fmaxf(m_tot, t[kHeadDim]);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float l_tot = 0.0f;
    for (int s = 0; s < num_parts; ++s) {
        const float* t = parts + ((size_t)s * rows + row) * kRowTripleFloats;
        const float ls = t[kHeadDim + 1];
        if (ls > 0.0f) {
            const float wgt = ex2(t[kHeadDim] - m_tot);
            l_tot += ls * wgt;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += t[lane + 32 * j] * wgt;
        }
    }
    if (!(l_tot > 0.0f)) return;   // no shard had a key for this row (a masked row): attn_out stays as it is
    const float inv_l = 1.0f / (l_tot * kLutScale);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv_l;
    wht256_lanes(acc, lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) store_act(attn_out, (size_t)row * kHeadDim + lane + 32 * j, apply_sign(acc[j], lane + 32 * j), io_bf16);
}

// ---- exchange + merge over peer-mapped mailboxes -------------------------------------------------
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One warp per row.  Stores the row's triple into every peer's inbox, publishes the step number,
// waits (bounded) for the peers' triples of the same step and merges all of them in rank order.
// Mailbox rows alternate between two buffers by step parity: a peer can run at most one step
// ahead of a rank that has not yet read its inbox (its own next wait needs that rank's next
// store), so the buffer being read is never the one being written.
__global__ void __launch_bounds__(128) tq4_attention_exchange_merge_kernel(
    const warp34_peer_mailboxes mb, const float* __restrict__ mine, long long rows, void* __restrict__ attn_out) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 4 + wid;
    if (row >= rows) return;
    uint32_t* steps = reinterpret_cast<uint32_t*>((uintptr_t)mb.steps);
    const uint32_t step = steps[row] + 1u;  // every lane reads the same word; lane 0 stores it last
    const size_t per_rank = (size_t)mb.max_rows * kRowTripleFloats;
    const size_t slot = ((size_t)(step & 1u) * mb.world + mb.rank) * per_rank + (size_t)row * kRowTripleFloats;
    const float* src = mine + (size_t)row * kRowTripleFloats;

    // own triple: 258 floats, kept in registers for the merge as well
    float t_own[9];
#pragma unroll
    for (int j = 0; j < 8; ++j) t_own[j] = src[lane + 32 * j];
    t_own[8] = (lane < 2) ? src[kHeadDim + lane] : 0.0f;
    for (int w = 0; w < mb.world; ++w) {
        if (w == mb.rank) continue;
        float* dst = reinterpret_cast<float*>((uintptr_t)mb.inbox[w]) + slot;
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[lane + 32 * j] = t_own[j];
        if (lane < 2) dst[kHeadDim + lane] = t_own[8];
    }
    __threadfence_system();  // every lane's stores are ordered before the flag of lane w below
    __syncwarp();
    if (lane < mb.world && lane != mb.rank) {
        uint32_t* f = reinterpret_cast<uint32_t*>((uintptr_t)mb.flags[lane]) + (size_t)mb.rank * mb.max_rows + row;
        st_release_sys_u32(f, step);
    }

    // wait for the peers: lane w watches rank w's flag in this rank's own mailbox
    bool ok = true;
    if (lane < mb.world && lane != mb.rank) {
        const uint32_t* f = reinterpret_cast<const uint32_t*>((uintptr_t)mb.flags[mb.rank]) + (size_t)lane * mb.max_rows + row;
        const uint32_t limit = mb.wait_limit ? mb.wait_limit : (1u << 22);
        uint32_t n = 0;
        // steps are compared as a signed distance so that the counter may wrap
        while ((int32_t)(ld_acquire_sys_u32(f) - step) < 0) {
            if (++n >= limit) { ok = false; break; }
            __nanosleep(200);
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) steps[row] = step;
    if (!ok) {
        if (lane == 0 && mb.status) atomicOr(reinterpret_cast<int*>((uintptr_t)mb.status), 1);
        return;
    }

    const float* inbox = reinterpret_cast<const float*>((uintptr_t)mb.inbox[mb.rank]) +
                         (size_t)(step & 1u) * mb.world * per_rank + (size_t)row * kRowTripleFloats;
    const float m_own = __shfl_sync(0xffffffffu, t_own[8], 0), l_own = __shfl_sync(0xffffffffu, t_own[8], 1);
    float m_tot = -1e30f;
    for (int w = 0; w < mb.world; ++w) {
        const float* t = inbox + (size_t)w * per_rank;
        const float ls = (w == mb.rank) ? l_own : __ldcg(t + kHeadDim + 1);
        const float ms = (w == mb.rank) ? m_own : __ldcg(t + kHeadDim);
        if (ls > 0.0f) m_tot = fmaxf(m_tot, ms);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float l_tot = 0.0f;
    for (int w = 0; w < mb.world; ++w) {
        const float* t = inbox + (size_t)w * per_rank;
        const bool own = (w == mb.rank);
        const float ls = own ? l_own : __ldcg(t + kHeadDim + 1);
        if (ls > 0.0f) {
            const float wgt = ex2((own ? m_own : __ldcg(t + kHeadDim)) - m_tot);
            l_tot += ls * wgt;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += (own ? t_own[j] : __ldcg(t + lane + 32 * j)) * wgt;
        }
    }
    if (!(l_tot > 0.0f)) return;   // a row without keys on any rank (a masked row): attn_out stays as it is
    const float inv_l = 1.0f / (l_tot * kLutScale);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= inv_l;
    wht256_lanes(acc, lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) store_act(attn_out, (size_t)row * kHeadDim + lane + 32 * j, apply_sign(acc[j], lane + 32 * j), 0);
}

// Copies the first `rows` token rows of every kv head of one page to another page of the same
// slabs (copy-on-write of a shared partial tail page).  One block per (kv head, K or V).
__global__ void __launch_bounds__(128) kv_page_copy_kernel(const warp34_kv_layer_layout layout, int src_page,
                                                           int dst_page, int rows) {
    const int head = blockIdx.x >> 1;
    const bool is_v = blockIdx.x & 1;
    const uint64_t base = is_v ? layout.v_base : layout.k_base;
    const uint64_t ps = is_v ? layout.v_page_stride_bytes : layout.k_page_stride_bytes;
    const uint64_t hs = is_v ? layout.v_head_stride_bytes : layout.k_head_stride_bytes;
    const uint64_t ts = is_v ? layout.v_token_stride_bytes : layout.k_token_stride_bytes;
    const uint16_t* src = (const uint16_t*)(uintptr_t)(base + (uint64_t)src_page * ps + (uint64_t)head * hs);
    uint16_t* dst = (uint16_t*)(uintptr_t)(base + (uint64_t)dst_page * ps + (uint64_t)head * hs);
    const int halves_per_row = kTq4RowBytes / 2;
    for (int i = threadIdx.x; i < rows * halves_per_row; i += blockDim.x) {
        const int row = i / halves_per_row, c = i - row * halves_per_row;
        const size_t off = ((size_t)row * ts) / 2 + c;
        dst[off] = src[off];
    }
}

// ---- host side ---------------------------------------------------------------------------
constexpr int kWarpsPerCta = kFastWarps > kExactWarps ? kFastWarps : kExactWarps;   // scratch is sized for the larger build

// LUT + rings + mbarriers, plus up to 64 KB - 1 of alignment slack in front of the table; the
// kernel is given the whole opt-in maximum and checks the carve-up itself.
static size_t stream_smem_min_bytes() {
    const size_t fast = (size_t)kFastWarps * kFastStages * (kStageStride + 8);
    const size_t exact = (size_t)kExactWarps * kExactStages * (kStageStride + 8);
    return kLutBytes + (fast > exact ? fast : exact);
}

// Exact prefill kernel: table, eight fragment areas, the page ring and its barriers.
static size_t prefill_exact_smem_min_bytes() {
    return kLutBytes + (size_t)kPxWarps * (kPxQHiBytes + kPxQLoBytes) + (size_t)kPxStages * kStageStride + 128 +
           2 * kPxStages * 8 + 16 * kPxWarps;
}

struct DeviceInfo {
    int sm_count;
    int smem_optin;
    bool configured;
};

static DeviceInfo* device_info(int* rc) {
    static DeviceInfo info[64];
    static std::mutex guard;   // the one-time set-up of a device may be reached from several host threads
    std::lock_guard<std::mutex> lock(guard);
    int dev = 0;
    *rc = (int)cudaGetDevice(&dev);
    if (*rc != 0) return nullptr;
    if (dev < 0 || dev >= 64) { *rc = (int)cudaErrorInvalidDevice; return nullptr; }
    DeviceInfo* d = &info[dev];
    if (!d->configured) {
        int sms = 0;
        *rc = (int)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (*rc != 0) return nullptr;
        int optin = 0;
        *rc = (int)cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (*rc != 0) return nullptr;
        if ((size_t)optin < stream_smem_min_bytes()) { *rc = (int)cudaErrorNotSupported; return nullptr; }
        *rc = (int)cudaFuncSetAttribute(tq4_attention_stream_kernel<kExactStages, kExactWarps, true>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_stream_kernel<kFastStages, kFastWarps, false>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_stream_kernel<kExactStages, kExactWarps, true, true>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_team_kernel<2>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_team_kernel<3>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        if ((size_t)optin < prefill_exact_smem_min_bytes()) { *rc = (int)cudaErrorNotSupported; return nullptr; }
        *rc = (int)cudaFuncSetAttribute(tq4_attention_prefill_exact_kernel<kPxWarps>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_prefill_exact_kernel<kPxWarps / 2>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_prefill_exact_kernel<kPxWarps / 4>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, optin);
        if (*rc != 0) return nullptr;
        *rc = (int)cudaFuncSetAttribute(tq4_attention_prefill_tc_kernel,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes);
        if (*rc != 0) return nullptr;
        d->smem_optin = optin;
        d->sm_count = sms;
        d->configured = true;
    }
    return d;
}

static bool tq4_layout_ok(const warp34_kv_layer_layout* l) {
    return l->head_dim == kHeadDim && l->block_size == kPageTokens && l->local_kv_heads > 0 &&
           l->k_format == WARP34_KV_FORMAT_TQ4 && l->v_format == WARP34_KV_FORMAT_TQ4 &&
           l->k_transform == WARP34_KV_TRANSFORM_RADEMACHER_WHT256 &&
           l->v_transform == WARP34_KV_TRANSFORM_RADEMACHER_WHT256 && l->k_base != 0 && l->v_base != 0;
}

// The streaming path needs the canonical packing: 132-byte rows, 16 rows contiguous per
// (page, head), every run 16-byte aligned (bulk-copy granularity).
static bool stream_layout_ok(const warp34_kv_layer_layout* l) {
    return l->k_token_stride_bytes == kTq4RowBytes && l->v_token_stride_bytes == kTq4RowBytes &&
           ((l->k_base | l->v_base | l->k_page_stride_bytes | l->v_page_stride_bytes |
             l->k_head_stride_bytes | l->v_head_stride_bytes) & 15u) == 0 &&
           l->k_head_stride_bytes >= (uint64_t)kTq4PageHeadBytes &&
           l->v_head_stride_bytes >= (uint64_t)kTq4PageHeadBytes;
}

static long long items_bound(const warp34_kv_layer_layout* l, const warp34_attention_batch* b, int hq,
                             int rows_per_group = kRowsPerGroup) {
    const long long gqa = hq / l->local_kv_heads;
    const long long rows = (long long)b->total_tokens * gqa;
    return (long long)l->local_kv_heads * ((rows + rows_per_group - 1) / rows_per_group + b->num_reqs);
}

// Entries of the query-fragment store of the one-warp path: requests x kv heads x row groups.
static long long qfrag_items(const warp34_kv_layer_layout* l, const warp34_attention_batch* b, int gqa) {
    const long long groups = ((long long)(b->max_q_len > 0 ? b->max_q_len : 1) * gqa + kRowsPerGroup - 1) / kRowsPerGroup;
    return (long long)b->num_reqs * l->local_kv_heads * groups;
}

// Query rows that share one KV pass.  Exact build: 8, one warp per work item; a request with more
// rows per kv head (several draft tokens) becomes several items that read the same pages, close
// enough in time for the second and third read to come from L2.  Fast build: 8 with one warp per
// item, 16 or 24 with four-warp teams.
static int pick_row_tiles(const warp34_attention_batch* b, int gqa, bool fast) {
    const long long rows = (long long)(b->max_q_len > 0 ? b->max_q_len : 1) * gqa;
    if (!fast || rows <= 8) return 1;
    return rows <= 16 ? 2 : 3;
}

// Workspace of the streaming path with `workers` worker warps (or teams): plan, one partial slot
// per worker and per work item, and the query fragments of one-warp items.
static size_t stream_scratch_bytes(const warp34_kv_layer_layout* l, const warp34_attention_batch* b, int hq,
                                   bool fast, long long workers) {
    const int gqa = hq / l->local_kv_heads;
    const int nt = pick_row_tiles(b, gqa, fast);
    const int rpg = 8 * nt;
    const long long slots = workers + items_bound(l, b, hq, rpg);
    const size_t qfrag = (nt == 1) ? (size_t)qfrag_items(l, b, gqa) * qfrag_item_bytes() : 0;
    return plan_bytes(b->num_reqs) + (size_t)slots * (size_t)(rpg * kHeadDim + 2 * rpg) * sizeof(float) + qfrag;
}

// ---- a batch in several passes ------------------------------------------------------------------
// A workspace that leaves fewer worker slots than half a grid for the whole batch is used for part of
// the requests at a time: plan, stream and merge per part, one after the other on the stream, every part
// reusing the workspace.  `workers_for(reqs, tokens)` says how many worker slots the workspace leaves for a
// batch of `reqs` requests with at most `tokens` query tokens (negative: its unit count does not fit 32
// bits).  Returns the requests per pass (num_reqs: one pass) and the worker slots of a full part.
static long long part_tokens(const warp34_attention_batch* b, int reqs) {
    const long long t = (long long)reqs * (b->max_q_len > 0 ? b->max_q_len : 1);
    return t < b->total_tokens ? t : (long long)b->total_tokens;
}

template <class F>
static int pick_reqs_per_pass(const warp34_attention_batch* batch, long long full_workers, int workers_per_cta,
                              bool parts_allowed, F workers_for, long long* workers_out) {
    int reqs_per_pass = batch->num_reqs;
    long long workers = workers_for(reqs_per_pass, (long long)batch->total_tokens);
    if (parts_allowed && workers < full_workers / 2 && batch->num_reqs > 1) {
        int best_r = batch->num_reqs, r_try = batch->num_reqs;
        long long best_w = workers;
        while (r_try > 1 && best_w < full_workers / 2) {   // halve the part until half a grid fits
            r_try = (r_try + 1) / 2;
            const long long w_try = workers_for(r_try, part_tokens(batch, r_try));
            if (best_w >= workers_per_cta && w_try < best_w + best_w / 4) break;   // twice the passes for little
            best_r = r_try;
            best_w = w_try;
        }
        if (best_w >= workers_per_cta && (workers < workers_per_cta || 2 * best_w >= 3 * workers)) {
            reqs_per_pass = best_r;
            workers = best_w;
        }
    }
    *workers_out = workers;
    return reqs_per_pass;
}

// The descriptor of requests [r0, r0 + reqs) of a batch: arrays by request start at r0, arrays by token stay.
static warp34_attention_batch batch_part(const warp34_attention_batch* batch, int r0, int reqs) {
    warp34_attention_batch b = *batch;
    b.query_start_loc += r0;
    if (b.context_lens_before != nullptr) b.context_lens_before += r0;
    b.seq_lens_after += r0;
    b.block_tables += (size_t)r0 * batch->max_blocks_per_req;
    if (b.valid_req_mask != nullptr) b.valid_req_mask += r0;
    b.num_reqs = reqs;
    b.total_tokens = (int)part_tokens(batch, reqs);
    return b;
}

}  // namespace w34

#include "kv8_attention.cuh"
#include "qsa_sparse.cuh"

namespace w34 {
static int launch_scalar(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                         const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                         int num_q_heads, int io_bf16, const OutputGate* og = nullptr);
static int launch_output_gate(const warp34_exec* ex, const void* attn, const void* gate, void* out,
                              const uint8_t* valid_token_mask, int num_tokens, int total_dim, int mode, int io_bf16);
}

extern "C" int warp34_paged_attention_scalar_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                 const warp34_attention_batch* batch, const void* q_in,
                                                 void* attn_out, int num_q_heads) {
    return w34::launch_scalar(ex, layout, batch, q_in, attn_out, num_q_heads, 0);
}

static int w34::launch_output_gate(const warp34_exec* ex, const void* attn, const void* gate, void* out,
                                   const uint8_t* valid_token_mask, int num_tokens, int total_dim, int mode,
                                   int io_bf16) {
    if (ex == nullptr || attn == nullptr || gate == nullptr || out == nullptr) return (int)cudaErrorInvalidValue;
    if (mode == 2 && (total_dim & 63) != 0) return (int)cudaErrorInvalidValue;
    if ((((uintptr_t)attn | (uintptr_t)gate | (uintptr_t)out) & 1u) != 0u) return (int)cudaErrorInvalidValue;
    if (num_tokens <= 0 || total_dim <= 0) return 0;
    const int chunk_blocks = ((total_dim + 255) / 256 + 3) / 4;
    if (chunk_blocks > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)num_tokens, (unsigned)chunk_blocks);
    cudaStream_t st = (cudaStream_t)ex->stream;
    if (mode != 1 && mode != 2) return (int)cudaErrorInvalidValue;
    const bool all_vec = (total_dim & 255) == 0 && ((((uintptr_t)attn | (uintptr_t)gate | (uintptr_t)out) & 15u) == 0u);
    if (all_vec) {   // every chunk full and aligned: the kernel without the element-wise path
        if (mode == 2) {
            if (io_bf16) w34::attn_output_gate_vec_kernel<2, true><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
            else w34::attn_output_gate_vec_kernel<2, false><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
        } else {
            if (io_bf16) w34::attn_output_gate_vec_kernel<1, true><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
            else w34::attn_output_gate_vec_kernel<1, false><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
        }
        return (int)cudaGetLastError();
    }
    if (mode == 2) {
        if (io_bf16) w34::attn_output_gate_kernel<2, true><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
        else w34::attn_output_gate_kernel<2, false><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
    } else {
        if (io_bf16) w34::attn_output_gate_kernel<1, true><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
        else w34::attn_output_gate_kernel<1, false><<<grid, 128, 0, st>>>(attn, gate, out, valid_token_mask, num_tokens, total_dim);
    }
    return (int)cudaGetLastError();
}

static int w34::launch_scalar(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                              const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                              int num_q_heads, int io_bf16, const OutputGate* og) {
    if (ex == nullptr || layout == nullptr || batch == nullptr || q_in == nullptr || attn_out == nullptr) {
        return (int)cudaErrorInvalidValue;
    }
    if (batch->total_tokens <= 0 || num_q_heads <= 0) return 0;
    w34::OutputGate none;
    none.gate = nullptr;
    none.mode = 0;
    if (w34::kv8_attention_layout_ok(layout)) {
        if (og != nullptr && og->mode != 0) return (int)cudaErrorNotSupported;   // callers gate these layers in a second step
        return w34::launch_kv8_attention(ex, layout, batch, q_in, attn_out, num_q_heads, io_bf16);
    }
    if (!w34::tq4_layout_ok(layout)) return (int)cudaErrorNotSupported;
    if (num_q_heads % layout->local_kv_heads != 0 || batch->num_reqs <= 0) return (int)cudaErrorInvalidValue;
    const long long rows = (long long)batch->total_tokens * num_q_heads;
    if (rows > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)rows;   // one block of four warps per row
    w34::tq4_attention_scalar_kernel<<<blocks, 128, 0, (cudaStream_t)ex->stream>>>(
        *layout, *batch, q_in, attn_out, num_q_heads, io_bf16, og != nullptr ? *og : none);
    return (int)cudaGetLastError();
}

extern "C" size_t warp34_paged_attention_scratch_bytes(const warp34_kv_layer_layout* layout,
                                                       const warp34_attention_batch* batch, int num_q_heads) {
    if (layout == nullptr || batch == nullptr || num_q_heads <= 0 || layout->local_kv_heads <= 0) return 0;
    int rc = 0;
    w34::DeviceInfo* d = w34::device_info(&rc);
    const int sms = d ? d->sm_count : 148;
    // enough for a full grid in either build
    const int gqa = num_q_heads / layout->local_kv_heads;
    const int nt_fast = w34::pick_row_tiles(batch, gqa, true);
    const size_t fast = w34::stream_scratch_bytes(layout, batch, num_q_heads, true,
                                                  (long long)sms * (nt_fast == 1 ? w34::kFastWarps : w34::kTeams));
    const size_t exact = w34::stream_scratch_bytes(layout, batch, num_q_heads, false, (long long)sms * w34::kExactWarps);
    return fast > exact ? fast : exact;
}

namespace w34 {

// Prefill chunks (more query rows per request and kv head than three row groups hold) go to a
// 128-row kernel, which needs no scratch beyond the status word.
static bool takes_prefill_path(uint64_t flags, const warp34_kv_layer_layout* l,
                               const warp34_attention_batch* b, int gqa) {
    const bool want_tc = (flags & WARP34_B200_EXEC_FLAG_TCGEN05_VERIFY) != 0 && (long long)b->max_q_len * gqa > 8;
    return (flags & WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION) == 0 && stream_layout_ok(l) &&
           b->max_blocks_per_req > 0 && gqa <= kPxRows && ((long long)b->max_q_len * gqa > 24 || want_tc);
}

// Shared body of the attention entry points.  triple_out != nullptr: stop after the split-KV
// merge and write per-row (acc, m, l) instead of attn_out (streaming path only).
// force: -1 = dispatch by batch geometry and flags; otherwise the kernel family the reference's
// test selector names: 0 = the row-group kernels (8 query rows per item), 1 = the register-MMA
// prefill kernel, 2 = the tcgen05 prefill kernel.
static int launch_attention(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                            const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                            float* triple_out, int num_q_heads, int io_bf16 = 0, int force = -1,
                            const OutputGate* gate = nullptr) {
    OutputGate og;
    og.gate = gate != nullptr ? gate->gate : nullptr;
    og.mode = gate != nullptr ? gate->mode : 0;
    if (og.mode != 0 && (triple_out != nullptr || og.gate == nullptr)) return (int)cudaErrorInvalidValue;
    if (ex == nullptr || layout == nullptr || batch == nullptr || q_in == nullptr ||
        (attn_out == nullptr && triple_out == nullptr)) {
        return (int)cudaErrorInvalidValue;
    }
    if (batch->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (kv8_attention_layout_ok(layout)) {   // unrotated 8-bit boundary layers: the epilogue is a second launch, in place
        if (triple_out != nullptr) return (int)cudaErrorNotSupported;
        const int rc8 = launch_kv8_attention(ex, layout, batch, q_in, attn_out, num_q_heads, io_bf16,
                                             (ex->flags & WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION) == 0 && force <= 0);
        if (rc8 != 0 || og.mode == 0) return rc8;
        return launch_output_gate(ex, attn_out, og.gate, attn_out, batch->valid_token_mask, batch->total_tokens,
                                  num_q_heads * kHeadDim, og.mode, io_bf16);
    }
    if (!tq4_layout_ok(layout)) return (int)cudaErrorNotSupported;
    if (num_q_heads % layout->local_kv_heads != 0 || batch->num_reqs <= 0) return (int)cudaErrorInvalidValue;

    int rc = 0;
    DeviceInfo* dev = device_info(&rc);
    if (dev == nullptr) return rc;

    const int gqa = num_q_heads / layout->local_kv_heads;
    // Prefill chunks: 128-row CTAs, no scratch.  Not for the partial-output mode, which is a
    // decode-time feature.  Default: register MMAs with value + residual operands; with the fast
    // flag (or the tcgen05-verify flag) tcgen05 + TMEM with single fp16 operands.
    const bool chunk_geometry_ok = stream_layout_ok(layout) && batch->max_blocks_per_req > 0 && gqa <= kPxRows;
    if (force >= 1 && (!chunk_geometry_ok || triple_out != nullptr)) return (int)cudaErrorNotSupported;
    if (force >= 1 || (force < 0 && triple_out == nullptr && takes_prefill_path(ex->flags, layout, batch, gqa))) {
        int32_t* status = nullptr;
        if (ex->scratch_ptr != 0 && (ex->scratch_ptr & 3u) == 0 && ex->scratch_size >= sizeof(PlanHeader)) {
            status = reinterpret_cast<int32_t*>((uintptr_t)ex->scratch_ptr);   // PlanHeader::status
            rc = (int)cudaMemsetAsync(status, 0, sizeof(int32_t), (cudaStream_t)ex->stream);
            if (rc != 0) return rc;
        }
        const bool tc = force == 2 || (force < 0 && (ex->flags & (WARP34_B200_EXEC_FLAG_FAST_ATTENTION |
                                                                  WARP34_B200_EXEC_FLAG_TCGEN05_VERIFY)) != 0);
        if (layout->local_kv_heads > 65535) return (int)cudaErrorInvalidValue;
        if (tc) {
            if ((size_t)dev->smem_optin < kTcSmemBytes) return (int)cudaErrorNotSupported;
            PrefillTcParams tp;
            tp.layout = *layout;
            tp.batch = *batch;
            tp.q_in = q_in;
            tp.attn_out = attn_out;
            tp.io_bf16 = io_bf16;
            tp.num_q_heads = num_q_heads;
            tp.gqa = gqa;
            tp.tok_per_tile = kTcRows / gqa;
            tp.q_scale = batch->sm_scale * 1.4426950408889634f;
            tp.status = status;
            tp.og = og;
            const long long tiles = (long long)batch->total_tokens / tp.tok_per_tile + batch->num_reqs;
            if (tiles > 0x7fffffffll) return (int)cudaErrorInvalidValue;
            const dim3 grid((unsigned)tiles, (unsigned)layout->local_kv_heads);
            tq4_attention_prefill_tc_kernel<<<grid, kTcThreads, kTcSmemBytes, (cudaStream_t)ex->stream>>>(tp);
            return (int)cudaGetLastError();
        }
        PrefillExactParams pp;
        pp.layout = *layout;
        pp.batch = *batch;
        pp.q_in = q_in;
        pp.attn_out = attn_out;
        pp.io_bf16 = io_bf16;
        pp.num_q_heads = num_q_heads;
        pp.gqa = gqa;
        pp.q_scale = batch->sm_scale * 1.4426950408889634f / kLutScale;
        pp.status = status;
        pp.smem_bytes = (uint32_t)dev->smem_optin;
        pp.og = og;
        // 128-row CTAs, or 64- / 32-row CTAs when that is faster for this call (a short chunk whose 128-row tiles
        // would leave SMs without a CTA).  One CTA fits an SM; a CTA of 4 (2) warps takes about 0.69 (0.55) of the
        // time of one of 8 warps over the same keys (measured: fewer warps share the SM's tensor pipe), so the
        // estimate is waves x that factor.
        int warps = kPxWarps;
        long long tiles = 0;
        {
            const float factor[3] = {1.0f, 0.69f, 0.55f};
            float best = 0.0f;
            for (int k = 0, w = kPxWarps; k < 3 && gqa <= 16 * w; ++k, w /= 2) {
                const int tpt = (16 * w) / gqa;
                const long long t = (long long)batch->total_tokens / tpt + batch->num_reqs;
                const long long waves = (t * layout->local_kv_heads + dev->sm_count - 1) / dev->sm_count;
                const float est = (float)waves * factor[k];
                if (k == 0 || est < best) { best = est; warps = w; tiles = t; pp.tok_per_tile = tpt; }
            }
        }
        if (tiles > 0x7fffffffll) return (int)cudaErrorInvalidValue;
        const dim3 grid((unsigned)tiles, (unsigned)layout->local_kv_heads);
        const size_t smem_px = (size_t)dev->smem_optin;
        cudaStream_t st_px = (cudaStream_t)ex->stream;
        if (warps == kPxWarps) tq4_attention_prefill_exact_kernel<kPxWarps><<<grid, kPxWarps * 32, smem_px, st_px>>>(pp);
        else if (warps == kPxWarps / 2) tq4_attention_prefill_exact_kernel<kPxWarps / 2><<<grid, (kPxWarps / 2) * 32, smem_px, st_px>>>(pp);
        else tq4_attention_prefill_exact_kernel<kPxWarps / 4><<<grid, (kPxWarps / 4) * 32, smem_px, st_px>>>(pp);
        return (int)cudaGetLastError();
    }

    // Streaming path: canonical layout, scratch that holds the plan plus at least one partial
    // per item and per worker, unit count within int32.  Workers are warps (8 query rows per
    // item) or four-warp teams (16 / 24 rows per item).
    const bool fast = (ex->flags & WARP34_B200_EXEC_FLAG_FAST_ATTENTION) != 0;
    const int nt = pick_row_tiles(batch, gqa, fast);
    const int rpg = 8 * nt;
    const int workers_per_cta = (nt == 1) ? (fast ? kFastWarps : kExactWarps) : kTeams;
    const size_t slot_bytes = (size_t)(rpg * kHeadDim + 2 * rpg) * sizeof(float);
    const long long full_workers = (long long)dev->sm_count * workers_per_cta;
    const bool stream_ok = (ex->flags & WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION) == 0 &&
                           stream_layout_ok(layout) && ex->scratch_ptr != 0 && (ex->scratch_ptr & 15u) == 0u &&
                           batch->max_blocks_per_req > 0;
    if (nt == 1 && qfrag_items(layout, batch, gqa) > 0x3fffffffll) return (int)cudaErrorInvalidValue;

    // Worker slots the workspace leaves for a batch of `reqs` requests with at most `tokens` query tokens
    // (-1: its unit count does not fit 32 bits).  Each of its items needs a slot and, one-warp items, a set
    // of query fragments.
    auto workers_for = [&](int reqs, long long tokens) -> long long {
        warp34_attention_batch b = *batch;
        b.num_reqs = reqs;
        b.total_tokens = (int)tokens;
        const long long items = items_bound(layout, &b, num_q_heads, rpg);
        if (items * (long long)batch->max_blocks_per_req >= 0x7fffffffll) return -1;
        const size_t fixed = plan_bytes(reqs) + ((nt == 1) ? (size_t)qfrag_items(layout, &b, gqa) * qfrag_item_bytes() : 0);
        const size_t avail = ex->scratch_size > fixed ? ex->scratch_size - fixed : 0;
        const long long w = (long long)(avail / slot_bytes) - items;
        return w < 0 ? 0 : w;
    };
    // Requests per pass: one pass unless the workspace is short (the cross-GPU partial mode keeps one pass:
    // its rows are addressed by the caller).
    long long workers = -1;
    int reqs_per_pass = batch->num_reqs;
    if (stream_ok) {
        reqs_per_pass = pick_reqs_per_pass(batch, full_workers, workers_per_cta, triple_out == nullptr, workers_for, &workers);
    }
    if (!stream_ok || workers < workers_per_cta) {
        if (triple_out != nullptr) return (int)cudaErrorNotSupported;
        return launch_scalar(ex, layout, batch, q_in, attn_out, num_q_heads, io_bf16, &og);
    }

    const bool in_parts = reqs_per_pass < batch->num_reqs;
    cudaStream_t st = (cudaStream_t)ex->stream;
    const size_t smem = (size_t)dev->smem_optin;
    for (int r0 = 0; r0 < batch->num_reqs; r0 += reqs_per_pass) {
        const int reqs = (batch->num_reqs - r0 < reqs_per_pass) ? batch->num_reqs - r0 : reqs_per_pass;
        StreamParams p;
        p.layout = *layout;
        p.batch = *batch;
        if (in_parts) p.batch = batch_part(batch, r0, reqs);
        const long long items = items_bound(layout, &p.batch, num_q_heads, rpg);
        const long long q_items = (nt == 1) ? qfrag_items(layout, &p.batch, gqa) : 0;
        long long part_workers = in_parts ? workers_for(reqs, p.batch.total_tokens) : workers;   // the last part is smaller
        if (part_workers > full_workers) part_workers = full_workers;
        const int grid = (int)(part_workers / workers_per_cta);
        if (grid < 1) return (int)cudaErrorInvalidValue;
        const size_t plan = plan_bytes(reqs);
        p.q_in = q_in;
        p.attn_out = attn_out;
        p.io_bf16 = io_bf16;
        p.triple_out = triple_out;
        p.scratch = reinterpret_cast<uint8_t*>((uintptr_t)ex->scratch_ptr);
        p.num_q_heads = num_q_heads;
        p.gqa = gqa;
        p.num_warps = grid * workers_per_cta;
        p.max_slots = (int)(p.num_warps + items);
        p.rows_per_group = rpg;
        p.q_scale = batch->sm_scale * 1.4426950408889634f / kLutScale;
        p.natural = 0;
        p.q_floor = fast ? 0 : 1;
        p.og = og;
        p.rows_from_first_token = in_parts ? 1 : 0;
        p.keep_status = r0 > 0 ? 1 : 0;
        p.qfrag = (nt == 1) ? reinterpret_cast<uint32_t*>(p.scratch + plan + (size_t)p.max_slots * slot_bytes) : nullptr;
        p.smem_bytes = (uint32_t)smem;
        p.q_groups_max = (nt == 1) ? (int)(q_items / ((long long)reqs * layout->local_kv_heads)) : 0;
        tq4_attention_plan_kernel<<<1 + (unsigned)q_items, q_items > 0 ? kPlanThreads : 32, 0, st>>>(p);
        if (nt == 1) {
            if (fast) tq4_attention_stream_kernel<kFastStages, kFastWarps, false><<<grid, kFastWarps * 32, smem, st>>>(p);
            else tq4_attention_stream_kernel<kExactStages, kExactWarps, true><<<grid, kExactWarps * 32, smem, st>>>(p);
        } else if (nt == 2) {
            tq4_attention_team_kernel<2><<<grid, kTeams * kTeamWarps * 32, smem, st>>>(p);
        } else {
            tq4_attention_team_kernel<3><<<grid, kTeams * kTeamWarps * 32, smem, st>>>(p);
        }
        // rows of the merge: every token of the batch, or (a part) as many as the part can hold, counted
        // from its first token
        const long long rows = (long long)p.batch.total_tokens * num_q_heads;
        // Few rows with hundreds of partials each (one long sequence): 32 warps per row instead of 4.
        const bool wide = rows * 4 < (long long)grid * workers_per_cta / 8;
        if (triple_out != nullptr) {
            if (wide) tq4_attention_merge_kernel<true, 32><<<(unsigned)rows, 1024, 0, st>>>(p);
            else tq4_attention_merge_kernel<true, 4><<<(unsigned)rows, 128, 0, st>>>(p);
        } else {
            if (wide) tq4_attention_merge_kernel<false, 32><<<(unsigned)rows, 1024, 0, st>>>(p);
            else tq4_attention_merge_kernel<false, 4><<<(unsigned)rows, 128, 0, st>>>(p);
        }
        rc = (int)cudaGetLastError();
        if (rc != 0) return rc;
    }
    return 0;
}

// Query-sparse lists on the exact stream kernel (TQ4 layers in the canonical packing, a workspace that
// holds the plan, the query fragments and at least one CTA's partial slots).  *taken = false: the caller
// runs its fp32 kernel instead.
// The same lists over 8-bit layers, on kv8_attention_stream_kernel<format, stages, sparse>.
static int launch_qsa_stream_kv8(const warp34_exec* ex, const QsaParams& q, bool* taken) {
    const warp34_kv_layer_layout* layout = &q.layout;
    warp34_attention_batch b = warp34_attention_batch{};
    b.block_tables = reinterpret_cast<const int32_t*>(q.sel_phys);   // only tested for presence by kv8_stream_ok
    b.max_blocks_per_req = 1;
    if (!kv8_stream_ok(ex, layout, &b, q.q, 0) || q.select_k <= 0) return 0;
    int rc = 0;
    DeviceInfo* dev = device_info(&rc);
    if (dev == nullptr) return rc;
    const int gqa = q.num_q_heads / layout->local_kv_heads;
    const long long groups = (gqa + kRowsPerGroup - 1) / kRowsPerGroup;
    const long long items = (long long)q.num_tokens * layout->local_kv_heads * groups;
    if (items * (((long long)q.select_k + 3) / 4) >= 0x7fffffffll) return 0;
    const size_t plan = plan_bytes(q.num_tokens);
    const size_t slot_bytes = (size_t)kPartialFloats * sizeof(float);
    const size_t avail = ex->scratch_size > plan ? ex->scratch_size - plan : 0;
    const long long workers = (long long)(avail / slot_bytes) - items;
    if (workers < kKv8StreamWarps) return 0;
    int grid = dev->sm_count;
    if (workers / kKv8StreamWarps < grid) grid = (int)(workers / kKv8StreamWarps);
    const bool fp8 = layout->k_format == WARP34_KV_FORMAT_FP8_E4M3;
    const uint32_t stage = 2u * (uint32_t)(fp8 ? Kv8Stage<WARP34_KV_FORMAT_FP8_E4M3>::kRunStride
                                               : Kv8Stage<WARP34_KV_FORMAT_Q8_0>::kRunStride) + 16u;
    const uint32_t smem = (uint32_t)(kKv8StreamWarps * kKv8StreamStages) * (stage + 8u);
    {
        static std::mutex mu;
        static bool done[64];
        int d = 0;
        rc = (int)cudaGetDevice(&d);
        if (rc != 0) return rc;
        if (d < 0 || d >= 64) return (int)cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu);
        if (!done[d]) {
            rc = (int)cudaFuncSetAttribute(kv8_attention_stream_kernel<WARP34_KV_FORMAT_FP8_E4M3, kKv8StreamStages, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)((uint32_t)(kKv8StreamWarps * kKv8StreamStages) *
                                                 (2u * Kv8Stage<WARP34_KV_FORMAT_FP8_E4M3>::kRunStride + 24u)));
            if (rc != 0) return rc;
            rc = (int)cudaFuncSetAttribute(kv8_attention_stream_kernel<WARP34_KV_FORMAT_Q8_0, kKv8StreamStages, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)((uint32_t)(kKv8StreamWarps * kKv8StreamStages) *
                                                 (2u * Kv8Stage<WARP34_KV_FORMAT_Q8_0>::kRunStride + 24u)));
            if (rc != 0) return rc;
            done[d] = true;
        }
    }
    StreamParams p;
    p.layout = *layout;
    p.batch = warp34_attention_batch{};
    p.batch.valid_token_mask = q.valid_token_mask;
    p.batch.num_reqs = q.num_tokens;
    p.batch.total_tokens = q.num_tokens;
    p.batch.max_q_len = 1;
    p.batch.mask_mode = WARP34_ATTN_MASK_CAUSAL;
    p.batch.sliding_window = 0;
    p.batch.sm_scale = q.sm_scale;
    p.q_in = q.q;
    p.attn_out = q.out;
    p.io_bf16 = 0;
    p.triple_out = nullptr;
    p.scratch = reinterpret_cast<uint8_t*>((uintptr_t)ex->scratch_ptr);
    p.num_q_heads = q.num_q_heads;
    p.gqa = gqa;
    p.num_warps = grid * kKv8StreamWarps;
    p.max_slots = (int)(p.num_warps + items);
    p.smem_bytes = smem;
    p.rows_per_group = kRowsPerGroup;
    p.q_scale = q.sm_scale * 1.4426950408889634f;
    p.natural = 1;
    p.og.gate = q.gate;
    p.og.mode = (q.gate != nullptr || q.hadamard) ? ((q.hadamard ? 2 : 1) | 4) : 0;
    p.qfrag = nullptr;
    p.q_groups_max = 0;
    p.sel_phys = q.sel_phys;
    p.sel_logical = q.sel_logical;
    p.num_selected = q.num_selected;
    p.seq_pos = q.seq_pos;
    p.select_k = q.select_k;
    cudaStream_t st = (cudaStream_t)ex->stream;
    tq4_attention_plan_kernel<<<1, 32, 0, st>>>(p);
    if (fp8) {
        kv8_attention_stream_kernel<WARP34_KV_FORMAT_FP8_E4M3, kKv8StreamStages, true><<<grid, kKv8StreamWarps * 32, smem, st>>>(p);
    } else {
        kv8_attention_stream_kernel<WARP34_KV_FORMAT_Q8_0, kKv8StreamStages, true><<<grid, kKv8StreamWarps * 32, smem, st>>>(p);
    }
    const long long rows = (long long)q.num_tokens * q.num_q_heads;
    if (rows * 4 < (long long)grid * kKv8StreamWarps / 8) {
        tq4_attention_merge_kernel<false, 32><<<(unsigned)rows, 1024, 0, st>>>(p);
    } else {
        tq4_attention_merge_kernel<false, 4><<<(unsigned)rows, 128, 0, st>>>(p);
    }
    *taken = true;
    return (int)cudaGetLastError();
}

static int launch_qsa_stream(const warp34_exec* ex, const QsaParams& q, bool* taken) {
    *taken = false;
    const warp34_kv_layer_layout* layout = &q.layout;
    if ((ex->flags & WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION) != 0 || ex->scratch_ptr == 0 || (ex->scratch_ptr & 15u) != 0u) {
        return 0;
    }
    if (kv8_attention_layout_ok(layout)) return launch_qsa_stream_kv8(ex, q, taken);
    if (!tq4_layout_ok(layout) || !stream_layout_ok(layout) || q.select_k <= 0) return 0;
    int rc = 0;
    DeviceInfo* dev = device_info(&rc);
    if (dev == nullptr) return rc;
    const int gqa = q.num_q_heads / layout->local_kv_heads;
    const long long groups = (gqa + kRowsPerGroup - 1) / kRowsPerGroup;
    const long long items = (long long)q.num_tokens * layout->local_kv_heads * groups;
    const long long units_bound = items * (((long long)q.select_k + 3) / 4);
    if (units_bound >= 0x7fffffffll || items > 0x3fffffffll) return 0;
    const size_t plan = plan_bytes(q.num_tokens);
    const size_t slot_bytes = (size_t)kPartialFloats * sizeof(float);
    const size_t qfrag_bytes = (size_t)items * qfrag_item_bytes();
    const size_t fixed = plan + qfrag_bytes;
    const size_t avail = ex->scratch_size > fixed ? ex->scratch_size - fixed : 0;
    const long long workers = (long long)(avail / slot_bytes) - items;
    if (workers < kExactWarps) return 0;
    int grid = dev->sm_count;
    if (workers / kExactWarps < grid) grid = (int)(workers / kExactWarps);

    StreamParams p;
    p.layout = *layout;
    p.batch = warp34_attention_batch{};
    p.batch.valid_token_mask = q.valid_token_mask;
    p.batch.num_reqs = q.num_tokens;
    p.batch.total_tokens = q.num_tokens;
    p.batch.max_q_len = 1;
    p.batch.mask_mode = WARP34_ATTN_MASK_CAUSAL;
    p.batch.sliding_window = 0;
    p.batch.sm_scale = q.sm_scale;
    p.q_in = q.q;
    p.attn_out = q.out;
    p.io_bf16 = 0;
    p.triple_out = nullptr;
    p.scratch = reinterpret_cast<uint8_t*>((uintptr_t)ex->scratch_ptr);
    p.num_q_heads = q.num_q_heads;
    p.gqa = gqa;
    p.num_warps = grid * kExactWarps;
    p.max_slots = (int)(p.num_warps + items);
    p.rows_per_group = kRowsPerGroup;
    p.q_scale = q.sm_scale * 1.4426950408889634f / kLutScale;
    p.natural = 0;
    p.q_floor = 1;
    p.og.gate = q.gate;
    p.og.mode = (q.gate != nullptr || q.hadamard) ? ((q.hadamard ? 2 : 1) | 4) : 0;
    p.qfrag = reinterpret_cast<uint32_t*>(p.scratch + plan + (size_t)p.max_slots * slot_bytes);
    p.q_groups_max = (int)groups;
    p.smem_bytes = (uint32_t)dev->smem_optin;
    p.sel_phys = q.sel_phys;
    p.sel_logical = q.sel_logical;
    p.num_selected = q.num_selected;
    p.seq_pos = q.seq_pos;
    p.select_k = q.select_k;
    cudaStream_t st = (cudaStream_t)ex->stream;
    tq4_attention_plan_kernel<<<1 + (unsigned)items, kPlanThreads, 0, st>>>(p);
    tq4_attention_stream_kernel<kExactStages, kExactWarps, true, true><<<grid, kExactWarps * 32, p.smem_bytes, st>>>(p);
    const long long rows = (long long)q.num_tokens * q.num_q_heads;
    if (rows * 4 < (long long)grid * kExactWarps / 8) {
        tq4_attention_merge_kernel<false, 32><<<(unsigned)rows, 1024, 0, st>>>(p);
    } else {
        tq4_attention_merge_kernel<false, 4><<<(unsigned)rows, 128, 0, st>>>(p);
    }
    *taken = true;
    return (int)cudaGetLastError();
}

}  // namespace w34

extern "C" int warp34_paged_attention_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                          const warp34_attention_batch* batch, const void* q_in,
                                          void* attn_out, int num_q_heads) {
    if (attn_out == nullptr) return (int)cudaErrorInvalidValue;
    return w34::launch_attention(ex, layout, batch, q_in, attn_out, nullptr, num_q_heads);
}

// Test-only selector of the reference (op_paged_attn.cu:1451-1458): 0 = its 16-row kernel, 1 = its
// 64-row, 2 = its 128-row prefill kernel.  Here: 0 = the row-group kernels, 1 = the register-MMA
// prefill kernel (value + residual operands), 2 = the tcgen05 prefill kernel.
extern "C" int warp34_paged_attention_f16_force_kernel_for_test(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                                const warp34_attention_batch* batch, const void* q_in,
                                                                void* attn_out, int num_q_heads, int use_64q) {
    if (ex == nullptr || layout == nullptr || batch == nullptr || q_in == nullptr || attn_out == nullptr) {
        return (int)cudaErrorInvalidValue;
    }
    if (batch->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (layout->head_dim != 256 || layout->block_size != 16 || layout->local_kv_heads <= 0 ||
        (num_q_heads % layout->local_kv_heads) != 0 || batch->num_reqs < 1) {
        return (int)cudaErrorInvalidValue;
    }
    return w34::launch_attention(ex, layout, batch, q_in, attn_out, nullptr, num_q_heads, 0,
                                 use_64q == 2 ? 2 : (use_64q != 0 ? 1 : 0));
}

// ---- attention without any caller-provided or allocated workspace ---------------------------
// Some hosts cannot hand this library a scratch buffer: an engine that has already given every
// byte of HBM it could reserve to the KV pool and the weights, a plugin that is only passed
// tensors and a stream, or a serving loop whose rules forbid allocator calls on the hot path.
// For them the split-KV workspace lives in this array, which every GPU that loads the library
// keeps for the life of the process.
constexpr size_t kStaticScratchBytes = (size_t)16 << 20;  // 16 MiB: 64 decode requests x 24 heads at full grid
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace w34 {
// Device address of g_static_scratch per device.  In host code the array's name is only a
// host-side handle; the address the kernels can use comes from cudaGetSymbolAddress, asked once
// per device while that device is current.
static int static_scratch_address(uint64_t* out) {
    static uint64_t addr[64];
    static bool known[64];
    static std::mutex guard;   // rank threads may make their first calls at the same time
    int dev = 0;
    int rc = (int)cudaGetDevice(&dev);
    if (rc != 0) return rc;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(guard);
    if (!known[dev]) {
        void* ptr = nullptr;
        rc = (int)cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (rc != 0) return rc;
        addr[dev] = (uint64_t)(uintptr_t)ptr;
        known[dev] = true;
    }
    *out = addr[dev];
    return 0;
}
}  // namespace w34

extern "C" int warp34_paged_attention_f16_static_scratch(uintptr_t stream, const warp34_kv_layer_layout* layout,
                                                         const warp34_attention_batch* batch, const void* q_in,
                                                         void* attn_out, int num_q_heads,
                                                         size_t* scratch_needed) {
    if (scratch_needed != nullptr) *scratch_needed = 0;
    if (layout == nullptr || batch == nullptr || q_in == nullptr || attn_out == nullptr) {
        return (int)cudaErrorInvalidValue;
    }
    if (batch->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (!w34::tq4_layout_ok(layout)) return (int)cudaErrorNotSupported;
    // Layouts the streaming and prefill kernels cannot take would fall to the fp32 kernel, which
    // uses no workspace at all; callers with such layouts have no use for this entry point.
    if (!w34::stream_layout_ok(layout) || batch->max_blocks_per_req <= 0) return (int)cudaErrorNotSupported;
    if (num_q_heads % layout->local_kv_heads != 0 || batch->num_reqs <= 0) return (int)cudaErrorInvalidValue;
    // What warp34_paged_attention_f16 needs at the least for the same batch with flags 0: a prefill
    // chunk only the status word, everything else the plan plus one partial per work item and per
    // warp of a single CTA plus the query fragments.
    const int gqa = num_q_heads / layout->local_kv_heads;
    const size_t needed = w34::takes_prefill_path(0, layout, batch, gqa)
                              ? sizeof(w34::PlanHeader)
                              : w34::stream_scratch_bytes(layout, batch, num_q_heads, false, w34::kExactWarps);
    if (scratch_needed != nullptr) *scratch_needed = needed;
    if (needed > kStaticScratchBytes) return (int)cudaErrorInvalidValue;  // batch too large for the built-in workspace
    warp34_exec ex;
    ex.stream = stream;
    ex.scratch_size = kStaticScratchBytes;
    ex.flags = 0;
    const int rc = w34::static_scratch_address(&ex.scratch_ptr);
    if (rc != 0) return rc;
    return w34::launch_attention(&ex, layout, batch, q_in, attn_out, nullptr, num_q_heads);
}

// ---- attention with the layer's output epilogue folded in ---------------------------------------
extern "C" int warp34_paged_attention_gated_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                const warp34_attention_batch* batch, const void* q_in,
                                                const void* gate, void* out, int num_q_heads, int hadamard64) {
    if (out == nullptr || gate == nullptr) return (int)cudaErrorInvalidValue;
    w34::OutputGate og;
    og.gate = gate;
    og.mode = hadamard64 ? 2 : 1;
    return w34::launch_attention(ex, layout, batch, q_in, out, nullptr, num_q_heads, 0, -1, &og);
}

// The two steps on their own, with the reference's names and signatures (warp34_cuda.h:297-300, :945-947).
extern "C" int warp34_apply_attn_output_gate_f16(const warp34_exec* ex, const void* attn_out, const void* gate,
                                                 void* out, const uint8_t* valid_token_mask, int num_tokens,
                                                 int total_dim) {
    return w34::launch_output_gate(ex, attn_out, gate, out, valid_token_mask, num_tokens, total_dim, 1, 0);
}

extern "C" int warp34_apply_attn_output_gate_hadamard_f16(const warp34_exec* ex, const void* attn_out, const void* gate,
                                                          void* out, const uint8_t* valid_token_mask, int num_tokens,
                                                          int total_dim) {
    return w34::launch_output_gate(ex, attn_out, gate, out, valid_token_mask, num_tokens, total_dim, 2, 0);
}

extern "C" int warp34_static_scratch_status(int32_t* status_out) {
    if (status_out == nullptr) return (int)cudaErrorInvalidValue;
    return (int)cudaMemcpyFromSymbol(status_out, g_static_scratch, sizeof(int32_t), 0, cudaMemcpyDeviceToHost);
}

extern "C" int warp34_tq4_paged_attention_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                               const warp34_attention_batch* batch, const void* q_in,
                                               void* attn_out, int num_q_heads) {
    if (attn_out == nullptr) return (int)cudaErrorInvalidValue;
    return w34::launch_attention(ex, layout, batch, q_in, attn_out, nullptr, num_q_heads, 1);
}

extern "C" int warp34_paged_attention_partial_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                  const warp34_attention_batch* batch, const void* q_in,
                                                  float* triples_out, int num_q_heads) {
    if (triples_out == nullptr) return (int)cudaErrorInvalidValue;
    return w34::launch_attention(ex, layout, batch, q_in, nullptr, triples_out, num_q_heads);
}

extern "C" int warp34_paged_attention_merge_shards_f16(const warp34_exec* ex, const float* triples,
                                                       int num_shards, int64_t num_rows, void* attn_out) {
    if (ex == nullptr || triples == nullptr || attn_out == nullptr || num_shards <= 0 || num_rows < 0) {
        return (int)cudaErrorInvalidValue;
    }
    if (num_rows == 0) return 0;
    w34::tq4_attention_merge_shards_kernel<<<(unsigned)((num_rows + 3) / 4), 128, 0, (cudaStream_t)ex->stream>>>(
        triples, num_shards, (long long)num_rows, attn_out, 0);
    return (int)cudaGetLastError();
}

extern "C" int warp34_paged_attention_exchange_merge_f16(const warp34_exec* ex, const warp34_peer_mailboxes* boxes,
                                                         const float* triples, int64_t num_rows, void* attn_out) {
    if (ex == nullptr || boxes == nullptr || triples == nullptr || attn_out == nullptr || num_rows < 0 ||
        boxes->world < 1 || boxes->world > WARP34_B200_MAX_PEERS || boxes->rank < 0 ||
        boxes->rank >= boxes->world || num_rows > boxes->max_rows || boxes->steps == 0) {
        return (int)cudaErrorInvalidValue;
    }
    for (int w = 0; w < boxes->world; ++w) {
        if (boxes->inbox[w] == 0 || boxes->flags[w] == 0) return (int)cudaErrorInvalidValue;
    }
    if (num_rows == 0) return 0;
    w34::tq4_attention_exchange_merge_kernel<<<(unsigned)((num_rows + 3) / 4), 128, 0, (cudaStream_t)ex->stream>>>(
        *boxes, triples, (long long)num_rows, attn_out);
    return (int)cudaGetLastError();
}

extern "C" int warp34_kv_page_copy(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                   int32_t src_page, int32_t dst_page, int32_t rows) {
    if (ex == nullptr || layout == nullptr || src_page < 0 || dst_page < 0 || rows < 0 ||
        rows > layout->block_size) {
        return (int)cudaErrorInvalidValue;
    }
    if (rows == 0 || src_page == dst_page || layout->local_kv_heads <= 0) return 0;
    if (layout->k_format != WARP34_KV_FORMAT_TQ4 || layout->v_format != WARP34_KV_FORMAT_TQ4 ||
        layout->head_dim != w34::kHeadDim) {
        return (int)cudaErrorNotSupported;
    }
    if ((layout->k_base | layout->v_base | layout->k_page_stride_bytes | layout->k_head_stride_bytes |
         layout->k_token_stride_bytes | layout->v_page_stride_bytes | layout->v_head_stride_bytes |
         layout->v_token_stride_bytes) & 1u) {
        return (int)cudaErrorInvalidValue;
    }
    w34::kv_page_copy_kernel<<<2 * layout->local_kv_heads, 128, 0, (cudaStream_t)ex->stream>>>(
        *layout, src_page, dst_page, rows);
    return (int)cudaGetLastError();
}

#include "bf16_kv.cuh"
