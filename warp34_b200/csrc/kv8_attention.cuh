// Paged attention over the unrotated 8-bit boundary-layer formats (Q8_0, FP8 E4M3), head_dim 256.
// Included by tq4_attention.cu.
//
// Replaces what the reference's dispatcher does for these layers: its row readers
// (crates/warp34-kernels/csrc/ops/op_paged_attn.cu:59-105) feed the same fp16 MMA kernels as TQ4
// rows; here it is a dequant-then-attend pass in fp32, one block per (token, kv head) that serves
// all the query heads of the group from one read of each K and V row (the rows are not rotated,
// so neither is the query nor the output).  Row layouts: see kv8_append.cuh.
#pragma once

#include <cuda_fp8.h>

namespace w34 {

constexpr int kKv8MaxGqa = 8;

// Lane L reads columns [8 L, 8 L + 8) of one row: two words of codes and the scale that covers them.
struct Kv8Raw {
    uint32_t w0, w1;
    float d;
};

__device__ __forceinline__ Kv8Raw kv8_load_raw(const uint8_t* row, int format, int lane) {
    Kv8Raw r;
    if (format == WARP34_KV_FORMAT_Q8_0) {
        const uint8_t* blk = row + (lane >> 3) * 68;            // block of 64 columns: float d, int8 qs[64]
        r.d = *reinterpret_cast<const float*>(blk);
        const uint32_t* q = reinterpret_cast<const uint32_t*>(blk + 4 + 8 * (lane & 7));
        r.w0 = q[0];
        r.w1 = q[1];
    } else {
        r.d = *reinterpret_cast<const float*>(row + kHeadDim + 4 * (lane >> 4));
        const uint32_t* q = reinterpret_cast<const uint32_t*>(row + 8 * lane);
        r.w0 = q[0];
        r.w1 = q[1];
    }
    return r;
}

__device__ __forceinline__ void kv8_decode(const Kv8Raw& r, int format, float (&x)[8]) {
    if (format == WARP34_KV_FORMAT_Q8_0) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            x[e] = r.d * (float)(int8_t)((r.w0 >> (8 * e)) & 0xffu);
            x[4 + e] = r.d * (float)(int8_t)((r.w1 >> (8 * e)) & 0xffu);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((r.w0 >> (16 * e)) & 0xffffu), __NV_E4M3);
            const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((r.w1 >> (16 * e)) & 0xffffu), __NV_E4M3);
            const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&a));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&b));
            x[2 * e] = r.d * fa.x;
            x[2 * e + 1] = r.d * fa.y;
            x[4 + 2 * e] = r.d * fb.x;
            x[4 + 2 * e + 1] = r.d * fb.y;
        }
    }
}

// One block of eight warps per (token, kv head); G = query heads per kv head (1..8), all served by
// one read of each row.  Warp w takes the pages with index = w (mod 8) of the row's key range and
// keeps a running (m, l, acc) per head; the eight partial states are merged through shared memory
// in two rounds (warps 4..7 into 0..3, then 1..3 into 0).
constexpr int kKv8Warps = 8;

template <int G>
__global__ void __launch_bounds__(kKv8Warps * 32) kv8_attention_kernel(
    const warp34_kv_layer_layout layout, const warp34_attention_batch batch,
    const void* __restrict__ q_in, void* __restrict__ attn_out, int num_q_heads, int io_bf16,
    int splits, float* __restrict__ partials) {
    __shared__ float s_acc[4][G][kHeadDim];
    __shared__ float s_ml[4][G][2];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int hkv = layout.local_kv_heads;
    const int tok = (int)(blockIdx.x / hkv), kv_head = (int)(blockIdx.x % hkv);
    // every exit below is taken by the whole block
    if (batch.valid_token_mask != nullptr && batch.valid_token_mask[tok] == 0) return;
    const int req = find_request(batch.query_start_loc, batch.num_reqs, tok);
    if (req < 0) return;
    const ReqGeom g = load_req(batch, req);
    if (!g.valid) return;
    const int q_off = tok - g.q_start;
    const int max_kv = row_max_kv(batch, g, q_off);
    const int min_kv = row_min_kv(batch, g, q_off);

    float qv[G][8], acc[G][8], m_i[G], l_i[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        const size_t base = ((size_t)tok * num_q_heads + (size_t)kv_head * G + h) * kHeadDim + 8 * lane;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            qv[h][e] = load_act(q_in, base + e, io_bf16) * batch.sm_scale;
            acc[h][e] = 0.0f;
        }
        m_i[h] = -1e30f;
        l_i[h] = 0.0f;
    }
    const int32_t* blocks = batch.block_tables + (size_t)req * batch.max_blocks_per_req;
    if (max_kv >= min_kv) {
        // blockIdx.y takes the y-th of `splits` equal page ranges of the row's keys
        const int p_lo = min_kv >> 4, p_hi = max_kv >> 4;
        const int chunk = (p_hi - p_lo + splits) / splits;
        const int my_lo = p_lo + (int)blockIdx.y * chunk;
        const int my_hi = min(p_hi, my_lo + chunk - 1);
        for (int pg = my_lo + wid; pg <= my_hi; pg += kKv8Warps) {
            const int page = block_table_page(blocks, pg, batch.max_blocks_per_req, kInKv8);
            const int lo = max(min_kv, pg << 4), hi = min(max_kv, (pg << 4) + 15);
            const uint8_t* kpage = (const uint8_t*)(uintptr_t)layout.k_base + (size_t)page * layout.k_page_stride_bytes +
                                   (size_t)kv_head * layout.k_head_stride_bytes;
            const uint8_t* vpage = (const uint8_t*)(uintptr_t)layout.v_base + (size_t)page * layout.v_page_stride_bytes +
                                   (size_t)kv_head * layout.v_head_stride_bytes;
            // four keys per step: their 24 loads are issued before the first is used, and the four
            // score reductions interleave
            for (int p0 = lo; p0 <= hi; p0 += 4) {
                Kv8Raw kr[4], vr[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int off = min(p0 + i, hi) & 15;   // past the end: re-read the last key, unused
                    kr[i] = kv8_load_raw(kpage + (size_t)off * layout.k_token_stride_bytes, layout.k_format, lane);
                    vr[i] = kv8_load_raw(vpage + (size_t)off * layout.v_token_stride_bytes, layout.v_format, lane);
                }
                float dot[4][G];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float kx[8];
                    kv8_decode(kr[i], layout.k_format, kx);
#pragma unroll
                    for (int h = 0; h < G; ++h) {
                        float s = 0.0f;
#pragma unroll
                        for (int e = 0; e < 8; ++e) s += qv[h][e] * kx[e];
                        dot[i][h] = s;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
#pragma unroll
                        for (int h = 0; h < G; ++h) dot[i][h] += __shfl_xor_sync(0xffffffffu, dot[i][h], o);
                    }
                }
                // one rescale per head for the four keys; keys past the end get weight 0
                float vx[4][8];
#pragma unroll
                for (int i = 0; i < 4; ++i) kv8_decode(vr[i], layout.v_format, vx[i]);
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    float m_new = m_i[h];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (p0 + i > hi) dot[i][h] = -1e30f;
                        m_new = fmaxf(m_new, dot[i][h]);
                    }
                    const float alpha = __expf(m_i[h] - m_new);
                    float pr[4], psum = 0.0f;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        pr[i] = (p0 + i <= hi) ? __expf(dot[i][h] - m_new) : 0.0f;
                        psum += pr[i];
                    }
                    l_i[h] = l_i[h] * alpha + psum;
                    m_i[h] = m_new;
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float t = acc[h][e] * alpha;
#pragma unroll
                        for (int i = 0; i < 4; ++i) t += pr[i] * vx[i][e];
                        acc[h][e] = t;
                    }
                }
            }
        }
    }
    // ---- merge the eight states: round 0 folds warps 4..7 into 0..3, round 1 folds 1..3 into 0 ----
#pragma unroll
    for (int round = 0; round < 2; ++round) {
        const bool writer = (round == 0) ? (wid >= 4) : (wid >= 1 && wid < 4);
        const int slot = (round == 0) ? wid - 4 : wid;
        if (writer) {
#pragma unroll
            for (int h = 0; h < G; ++h) {
#pragma unroll
                for (int e = 0; e < 8; ++e) s_acc[slot][h][8 * lane + e] = acc[h][e];
                if (lane == 0) { s_ml[slot][h][0] = m_i[h]; s_ml[slot][h][1] = l_i[h]; }
            }
        }
        __syncthreads();
        const int first = (round == 0) ? wid : 1, last = (round == 0) ? wid : 3;
        const bool reader = (round == 0) ? (wid < 4) : (wid == 0);
        if (reader) {
            for (int sidx = first; sidx <= last; ++sidx) {
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const float m_o = s_ml[sidx][h][0], l_o = s_ml[sidx][h][1];
                    const float m_new = fmaxf(m_i[h], m_o);
                    const float a = __expf(m_i[h] - m_new), b2 = __expf(m_o - m_new);
                    l_i[h] = l_i[h] * a + l_o * b2;
                    m_i[h] = m_new;
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[h][e] = acc[h][e] * a + s_acc[sidx][h][8 * lane + e] * b2;
                }
            }
        }
        __syncthreads();
    }
    if (wid != 0) return;
    if (splits > 1) {
        // un-normalised state of this page range: [item][split][head][256 acc | m | l]
        float* dst = partials + (((size_t)blockIdx.x * splits + blockIdx.y) * G) * kRowTripleFloats;
#pragma unroll
        for (int h = 0; h < G; ++h) {
#pragma unroll
            for (int e = 0; e < 8; ++e) dst[h * kRowTripleFloats + 8 * lane + e] = acc[h][e];
            if (lane == 0) {
                dst[h * kRowTripleFloats + kHeadDim] = m_i[h];
                dst[h * kRowTripleFloats + kHeadDim + 1] = l_i[h];
            }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < G; ++h) {
        const float inv_l = (l_i[h] > 0.0f) ? (1.0f / l_i[h]) : 0.0f;
        const size_t base = ((size_t)tok * num_q_heads + (size_t)kv_head * G + h) * kHeadDim + 8 * lane;
#pragma unroll
        for (int e = 0; e < 8; ++e) store_act(attn_out, base + e, acc[h][e] * inv_l, io_bf16);
    }
}

// Combines the `splits` states of every (token, q head): one warp per output row.
__global__ void __launch_bounds__(128) kv8_merge_kernel(
    const warp34_kv_layer_layout layout, const warp34_attention_batch batch, void* __restrict__ attn_out,
    int num_q_heads, int io_bf16, int splits, const float* __restrict__ partials) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 4 + wid;
    if (row >= (long long)batch.total_tokens * num_q_heads) return;
    const int tok = (int)(row / num_q_heads), q_head = (int)(row % num_q_heads);
    // the same exits as the attention blocks: rows they skipped have no states
    if (batch.valid_token_mask != nullptr && batch.valid_token_mask[tok] == 0) return;
    const int req = find_request(batch.query_start_loc, batch.num_reqs, tok);
    if (req < 0) return;
    const ReqGeom g = load_req(batch, req);
    if (!g.valid) return;
    const int gqa = num_q_heads / layout.local_kv_heads;
    const int kv_head = q_head / gqa, h = q_head - kv_head * gqa;
    const float* base = partials + ((((size_t)tok * layout.local_kv_heads + kv_head) * splits) * gqa + h) * kRowTripleFloats;
    const size_t stride = (size_t)gqa * kRowTripleFloats;
    float m_tot = -1e30f;
    for (int sidx = 0; sidx < splits; ++sidx) {
        const float* t = base + sidx * stride;
        if (t[kHeadDim + 1] > 0.0f) m_tot = fmaxf(m_tot, t[kHeadDim]);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float l_tot = 0.0f;
    for (int sidx = 0; sidx < splits; ++sidx) {
        const float* t = base + sidx * stride;
        const float ls = t[kHeadDim + 1];
        if (ls > 0.0f) {
            const float w = __expf(t[kHeadDim] - m_tot);
            l_tot += ls * w;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += t[8 * lane + e] * w;
        }
    }
    const float inv_l = (l_tot > 0.0f) ? (1.0f / l_tot) : 0.0f;
    const size_t out_base = ((size_t)tok * num_q_heads + q_head) * kHeadDim + 8 * lane;
#pragma unroll
    for (int e = 0; e < 8; ++e) store_act(attn_out, out_base + e, acc[e] * inv_l, io_bf16);
}

// ---------------------------------------------------------------------------------------------------
// Tensor-core path for 8-bit layers in the canonical packing (one (page, kv head) run of 16 rows for K
// and one for V).  Same persistent split-KV structure as the TQ4 stream kernel (plan launch, one share of
// (request, kv head, 8-row group, page) units per worker warp, per-warp mbarrier ring filled by bulk
// copies, partials merged by tq4_attention_merge_kernel in natural coordinates), but there is no table
// and nothing to round:
//   * the codes convert EXACTLY to fp16 straight into MMA A fragments: e4m3 with cvt.rn.f16x2.e4m3x2
//     (two codes per instruction); int8 through the byte trick 0x6400 | (q ^ 0x80) = 1152 + q, minus
//     1152.  The unrotated query is the fp16 B operand as it arrives; block scales and sm_scale stay
//     outside the operands in fp32, one score accumulator per scale block: S^T = K Q^T has no operand
//     rounding at all;
//   * P x d_v (d_v: the V scale of the key and block) is fed as fp16 value + fp16 residual, so
//     O^T += V^T (P d_v)^T carries P to about 2^-22.
// Shared-memory reads are conflict-free:
//   FP8 (264-byte rows = 66 words, consecutive tokens two banks apart, staged as they lie in memory),
//   64-bit loads.  K: lane (gid, tig) reads its key's words 32 h + 8 tig + 2 j + {0, 1} (h: 128-half,
//   j = 0..3); the 4 codes of a word are the k positions {2 tig, 2 tig + 1, 2 tig + 8, 2 tig + 9} of one
//   MMA step and the query fragments are loaded in the same order.  V: lane reads, for its four tokens,
//   words base(gid) + 16 jj + {0, 1}, base = 2 (gid & 1) + 8 ((gid >> 1) & 1) + 4 (gid >> 2); two PRMTs
//   pair the bytes of two tokens per channel (the k positions of an A register), a word gives two m-tiles.
//   Q8_0 (272-byte rows = 68 words: four blocks of {fp32 d; 64 int8}), staged as two 8-row halves 64
//   bytes apart so that tokens 8-15 sit 16 banks from tokens 0-7; 32-bit loads.  K: code word tig + 4 s
//   of block b (s = 0..3); V: code word gid + 8 x of block b (x = 0, 1).
// ---------------------------------------------------------------------------------------------------
template <int FMT> struct Kv8Stage;
template <> struct Kv8Stage<WARP34_KV_FORMAT_FP8_E4M3> {
    static constexpr int kRow = kHeadDim + 8;               // 264
    static constexpr int kHalf = 8 * kRow;                  // 2112
    static constexpr int kHalfStride = kHalf;               // the run is staged as it lies in memory
    static constexpr int kRunStride = 2 * kHalf;            // 4224
    static constexpr int kBlocks = 2;                       // scale blocks per row
};
template <> struct Kv8Stage<WARP34_KV_FORMAT_Q8_0> {
    static constexpr int kRow = 4 * 68;                     // 272
    static constexpr int kHalf = 8 * kRow;                  // 2176, a multiple of 16
    static constexpr int kHalfStride = kHalf + 64;          // tokens 8-15 sixteen banks from tokens 0-7
    static constexpr int kRunStride = 2 * kHalfStride;      // 4480
    static constexpr int kBlocks = 4;
};
constexpr int kKv8StreamWarps = 8;
constexpr int kKv8StreamStages = 3;

template <int FMT>
__host__ __device__ constexpr uint32_t kv8_token_offset(int t) {
    return (uint32_t)((t >> 3) * Kv8Stage<FMT>::kHalfStride + (t & 7) * Kv8Stage<FMT>::kRow);
}
__device__ __forceinline__ uint2 lds64_dep(uint32_t addr, uint32_t token) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0,%1}, [%2+0];  // dep %3" : "=r"(v.x), "=r"(v.y) : "r"(addr), "r"(token));
    return v;
}
// Four 8-bit codes -> two fp16 pairs (bytes 0,1 and bytes 2,3), exactly.
template <int FMT>
__device__ __forceinline__ void kv8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
    if (FMT == WARP34_KV_FORMAT_FP8_E4M3) {
        asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, l;\n\tcvt.rn.f16x2.e4m3x2 %1, h;\n\t}"
            : "=r"(lo), "=r"(hi) : "r"(w));
    } else {
        const uint32_t x = w ^ 0x80808080u;                               // q + 128 as an unsigned byte
        const uint32_t l = __byte_perm(x, 0x64646464u, 0x4140);           // halves 1024 + (q + 128)
        const uint32_t h = __byte_perm(x, 0x64646464u, 0x4342);
        const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));   // 1152
        const __half2 lh = __hsub2(*reinterpret_cast<const __half2*>(&l), bias);
        const __half2 hh = __hsub2(*reinterpret_cast<const __half2*>(&h), bias);
        lo = *reinterpret_cast<const uint32_t*>(&lh);
        hi = *reinterpret_cast<const uint32_t*>(&hh);
    }
}

// SPARSE: the query-sparse lists of warp34_qsa_sparse_paged_attn_f16 (see the TQ4 stream kernel): request r
// is token r, a unit is four entries of its selected list, lanes 0-3 copy their entry's four rows and leave
// its first position in 16 bytes behind the stage.
template <int FMT, int STAGES, bool SPARSE = false>
__global__ void __launch_bounds__(kKv8StreamWarps * 32, 1) kv8_attention_stream_kernel(const StreamParams p) {
    using G = Kv8Stage<FMT>;
    constexpr bool FP8 = FMT == WARP34_KV_FORMAT_FP8_E4M3;
    constexpr int NB = G::kBlocks;
    constexpr uint32_t kStage = 2u * G::kRunStride + (SPARSE ? 16u : 0u);
    extern __shared__ __align__(1024) uint8_t smem[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr uint32_t kRingBytes = STAGES * kStage;
    const uint32_t win_lo = smem_u32(smem);
    const uint32_t ring = win_lo + (uint32_t)wid * kRingBytes;
    const uint32_t bars = win_lo + (uint32_t)kKv8StreamWarps * kRingBytes + (uint32_t)wid * STAGES * 8u;
    uint8_t* ring_gen = smem + (size_t)wid * kRingBytes;
    PlanHeader* hdr = reinterpret_cast<PlanHeader*>(p.scratch);
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

    const int w_global = wid * (int)gridDim.x + (int)blockIdx.x;   // consecutive workers on different SMs
    const int per = hdr->units_per_warp;
    const int total_units = hdr->total_units;
    long long u_ll = (long long)w_global * per;
    if (per <= 0 || u_ll >= total_units) return;
    int u = (int)u_ll;
    const int u_end = min(u + per, total_units);

    const int gid = lane >> 2, tig = lane & 3;
    // MMA row m of S^T <-> token (m & 3) + 8 ((m >> 2) & 1) + 4 (m >> 3) of the page, which makes the
    // score accumulators of a lane, transposed by movmatrix, the P fragments of the tokens it owns in
    // the output product: kv0 + {0, 1, 4, 5} at k positions 2 tig, 2 tig + 1, 2 tig + 8, 2 tig + 9.
    const int key_a = (gid & 3) + 8 * (gid >> 2);
    const int kv0 = 2 * (tig & 1) + 8 * (tig >> 1);
    const uint32_t krow_off = kv8_token_offset<FMT>(key_a);          // token key_a + 4 is 4 rows further
    const uint32_t vrow_off = (uint32_t)G::kRunStride + kv8_token_offset<FMT>(kv0);
    // first code word (of 64, in column order) of this lane in the K and in the V loads
    const int kword0 = FP8 ? 8 * tig : tig;
    const int vword0 = FP8 ? 2 * (gid & 1) + 8 * ((gid >> 1) & 1) + 4 * (gid >> 2) : gid;
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

    while (u < u_end && !failed) {
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
        const int slot = w_global + item_prefix[r] + item;
        const ReqGeom g = stream_req(p, r);
        const int rows_in_req = g.q_len * p.gqa;

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
        int safe_hi = min(rvalid[0] ? rmax[0] : 0x7fffffff, rvalid[1] ? rmax[1] : 0x7fffffff);
        int safe_lo = max(rvalid[0] ? rmin[0] : 0, rvalid[1] ? rmin[1] : 0);
        int kv_hi = max(rmax[0], rmax[1]);   // last key any row of the group can see
#pragma unroll
        for (int d = 1; d < 4; d <<= 1) {
            safe_hi = min(safe_hi, __shfl_xor_sync(0xffffffffu, safe_hi, d));
            safe_lo = max(safe_lo, __shfl_xor_sync(0xffffffffu, safe_lo, d));
            kv_hi = max(kv_hi, __shfl_xor_sync(0xffffffffu, kv_hi, d));
        }

        // ---- query row gid of the group as B fragments, in the K loads' column order ----------------
        // k-step ks reads code word kw(ks) of the row: columns 4 kw .. 4 kw + 3.
        //   FP8: kw = 32 h + 8 tig + 2 j + x, ks = 2 (4 h + j) + x;  Q8_0: kw = 16 b + tig + 4 s, ks = 4 b + s
        uint32_t qb[16][2];
        {
            const int row = group * kRowsPerGroup + gid;
            const int q_off = row / p.gqa;
            const int q_head = kv_head * p.gqa + (row - q_off * p.gqa);
            const bool ok = row < rows_in_req &&
                            (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
            const size_t q_base = ((size_t)(g.q_start + q_off) * p.num_q_heads + q_head) * kHeadDim;
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                const int kw = FP8 ? 32 * (ks >> 3) + 2 * ((ks >> 1) & 3) + (ks & 1) + kword0
                                   : 16 * (ks >> 2) + 4 * (ks & 3) + kword0;
                uint2 v = make_uint2(0u, 0u);
                if (ok) {
                    if (p.io_bf16) {
                        v.x = pack_half2(load_act(p.q_in, q_base + 4 * kw, 1), load_act(p.q_in, q_base + 4 * kw + 1, 1));
                        v.y = pack_half2(load_act(p.q_in, q_base + 4 * kw + 2, 1), load_act(p.q_in, q_base + 4 * kw + 3, 1));
                    } else {
                        v = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p.q_in) + q_base + 4 * kw));
                    }
                }
                qb[ks][0] = v.x;
                qb[ks][1] = v.y;
            }
        }
        float o[16][4];
#pragma unroll
        for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
        float m_run[2] = {-1e30f, -1e30f};
        float l_run[2] = {0.0f, 0.0f};

        const int32_t* blocks = p.batch.block_tables + (size_t)r * p.batch.max_blocks_per_req;
        const uint8_t* k_head_base = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
        const uint8_t* v_head_base = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
        int32_t my_page = 0, next_page = 0;
        if (!SPARSE) {
            my_page = (lane < n_here) ? block_table_page(blocks, pg0 + lane, p.batch.max_blocks_per_req, kInKv8) : 0;
            next_page = (32 + lane < n_here) ? block_table_page(blocks, pg0 + 32 + lane, p.batch.max_blocks_per_req, kInKv8) : 0;
        }
        const int32_t* sel_phys = SPARSE ? p.sel_phys + (size_t)r * p.select_k : nullptr;
        const int32_t* sel_logical = SPARSE ? p.sel_logical + (size_t)r * p.select_k : nullptr;
        const int n_sel = SPARSE ? min(p.num_selected[r], p.select_k) : 0;

        fence_proxy_async();   // generic-proxy writes to the ring (partials, cleared rows) precede the copies
        auto issue = [&](int idx) {
            if (SPARSE) {
                const int s = idx % STAGES;
                const uint32_t bar = bars + 8u * s;
                const uint32_t dst = ring + (uint32_t)s * kStage;
                const int gi = 4 * (pg0 + idx) + lane;
                int ph = -1, first_pos = 0x3fffffff;
                if (lane < 4 && gi < n_sel) {
                    ph = sel_phys[gi];
                    const int lg = sel_logical[gi];
                    if (ph >= 0 && 4 * lg <= g.ctx_before) first_pos = 4 * lg; else ph = -1;
                }
                const int n_valid = __popc(__ballot_sync(0xffffffffu, ph >= 0));
                pending |= 1u << s;
                if (lane == 0) mbar_expect_tx(bar, (uint32_t)n_valid * 8u * G::kRow);
                __syncwarp();
                if (lane < 4) {
                    sts32(dst + 2u * G::kRunStride + 4u * lane, (uint32_t)first_pos);
                    if (ph >= 0) {
                        const int page = pool_page(ph >> 2, kInKv8);
                        const uint32_t row_off = (uint32_t)(ph & 3) * 4u * G::kRow;
                        bulk_g2s(dst + kv8_token_offset<FMT>(4 * lane),
                                 k_head_base + (size_t)page * p.layout.k_page_stride_bytes + row_off, 4u * G::kRow, bar);
                        bulk_g2s(dst + G::kRunStride + kv8_token_offset<FMT>(4 * lane),
                                 v_head_base + (size_t)page * p.layout.v_page_stride_bytes + row_off, 4u * G::kRow, bar);
                    }
                }
                return;
            }
            const int32_t page = __shfl_sync(0xffffffffu, (idx & 32) ? next_page : my_page, idx & 31);
            pending |= 1u << (idx % STAGES);
            if (lane == 0) {
                const int s = idx % STAGES;
                const uint32_t bar = bars + 8u * s;
                const uint32_t dst = ring + (uint32_t)s * kStage;
                const uint8_t* ksrc = k_head_base + (size_t)page * p.layout.k_page_stride_bytes;
                const uint8_t* vsrc = v_head_base + (size_t)page * p.layout.v_page_stride_bytes;
                mbar_expect_tx(bar, 4 * G::kHalf);
                if (G::kHalfStride == G::kHalf) {
                    bulk_g2s(dst, ksrc, 2 * G::kHalf, bar);
                    bulk_g2s(dst + G::kRunStride, vsrc, 2 * G::kHalf, bar);
                } else {
                    bulk_g2s(dst, ksrc, G::kHalf, bar);
                    bulk_g2s(dst + G::kHalfStride, ksrc + G::kHalf, G::kHalf, bar);
                    bulk_g2s(dst + G::kRunStride, vsrc, G::kHalf, bar);
                    bulk_g2s(dst + G::kRunStride + G::kHalfStride, vsrc + G::kHalf, G::kHalf, bar);
                }
            }
        };
#pragma unroll 1
        for (int i = 0; i < STAGES - 1 && i < n_here; ++i) issue(i);
        if (SPARSE) __syncwarp();   // the position words written by lanes 0-3 are read by all lanes

#pragma unroll 1
        for (int i = 0; i < n_here; ++i) {
            if (!SPARSE && (i & 31) == 0 && i > 0) {
                const int base = i + 32;
                const int32_t fresh = (base + lane < n_here) ? block_table_page(blocks, pg0 + base + lane, p.batch.max_blocks_per_req, kInKv8) : 0;
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

            const uint32_t st = ring + (uint32_t)s * kStage;
            const int kv_base = (pg0 + i) << 4;
            bool full = (kv_base >= safe_lo) && (kv_base + 15 <= safe_hi);
            // query-sparse: first position of the unit's four groups (0x3fffffff: nothing was copied)
            int fpos[4] = {0, 0, 0, 0};
            if (SPARSE) {
#pragma unroll
                for (int j = 0; j < 4; ++j) fpos[j] = (int)lds32(st + 2u * G::kRunStride + 4u * j);
                full = max(max(fpos[0], fpos[1]), max(fpos[2], fpos[3])) + 3 <= safe_hi;
            }
            // Tokens past the last visible key may never have been written (and the rows of a skipped
            // entry hold whatever the stage held before): as e4m3 codes their bytes can be NaN patterns,
            // and 0 x NaN is NaN inside the MMA.  Their V rows are cleared in the stage.
            const bool clear_tail = FP8 && (SPARSE ? !full : (kv_base + 15 > kv_hi));
            if (clear_tail) {
                if (SPARSE) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
#pragma unroll
                        for (int o4 = 0; o4 < 4; ++o4) {
                            if (fpos[j] + o4 <= kv_hi) continue;
                            for (int w = lane; w < G::kRow / 4; w += 32) {
                                sts32(st + (uint32_t)G::kRunStride + kv8_token_offset<FMT>(4 * j + o4) + 4u * (uint32_t)w, 0u);
                            }
                        }
                    }
                } else {
                    for (int t = max(kv_hi + 1 - kv_base, 0); t < kPageTokens; ++t) {
                        for (int w = lane; w < G::kRow / 4; w += 32) {
                            sts32(st + (uint32_t)G::kRunStride + kv8_token_offset<FMT>(t) + 4u * (uint32_t)w, 0u);
                        }
                    }
                }
                __syncwarp();
            }
            const uint32_t ptok = page_token(i);

            // ---- S^T = K Q^T: one accumulator per scale block, exact operands -------------------------
            float sa[NB][4];
            const uint32_t krow_a = st + krow_off, krow_b = krow_a + 4u * G::kRow;
            if (FP8) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t off = 4u * (uint32_t)(32 * h + 2 * j + kword0);
                        const uint2 wa = lds64_dep(krow_a + off, ptok);
                        const uint2 wb = lds64_dep(krow_b + off, ptok);
                        uint32_t a0, a1, a2, a3;
                        const int ks = 2 * (4 * h + j);
                        kv8x4_to_f16x4<FMT>(wa.x, a0, a2);
                        kv8x4_to_f16x4<FMT>(wb.x, a1, a3);
                        if (j == 0) mma16816_zero(sa[h], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
                        else mma16816(sa[h], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
                        kv8x4_to_f16x4<FMT>(wa.y, a0, a2);
                        kv8x4_to_f16x4<FMT>(wb.y, a1, a3);
                        mma16816(sa[h], a0, a1, a2, a3, qb[ks + 1][0], qb[ks + 1][1]);
                    }
                }
            } else {
#pragma unroll
                for (int b = 0; b < 4; ++b) {
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4) {
                        const uint32_t off = (uint32_t)(68 * b + 4 + 4 * (4 * s4 + kword0));
                        const uint32_t wa = lds32_dep(krow_a + off, ptok);
                        const uint32_t wb = lds32_dep(krow_b + off, ptok);
                        uint32_t a0, a1, a2, a3;
                        kv8x4_to_f16x4<FMT>(wa, a0, a2);
                        kv8x4_to_f16x4<FMT>(wb, a1, a3);
                        if (s4 == 0) mma16816_zero(sa[b], a0, a1, a2, a3, qb[4 * b][0], qb[4 * b][1]);
                        else mma16816(sa[b], a0, a1, a2, a3, qb[4 * b + s4][0], qb[4 * b + s4][1]);
                    }
                }
            }
            // block scales of this lane's two keys, K then V (fp32 words)
            float dka[NB], dkb[NB], dva[NB], dvb[NB];
            {
                const uint32_t vrow_a = st + (uint32_t)G::kRunStride + krow_off, vrow_b = vrow_a + 4u * G::kRow;
                if (FP8) {
                    const uint2 a = lds64_dep(krow_a + kHeadDim, ptok), b2 = lds64_dep(krow_b + kHeadDim, ptok);
                    const uint2 c = lds64_dep(vrow_a + kHeadDim, ptok), d = lds64_dep(vrow_b + kHeadDim, ptok);
                    dka[0] = __uint_as_float(a.x); dka[1] = __uint_as_float(a.y);
                    dkb[0] = __uint_as_float(b2.x); dkb[1] = __uint_as_float(b2.y);
                    dva[0] = __uint_as_float(c.x); dva[1] = __uint_as_float(c.y);
                    dvb[0] = __uint_as_float(d.x); dvb[1] = __uint_as_float(d.y);
                } else {
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        dka[b] = __uint_as_float(lds32_dep(krow_a + 68u * b, ptok));
                        dkb[b] = __uint_as_float(lds32_dep(krow_b + 68u * b, ptok));
                        dva[b] = __uint_as_float(lds32_dep(vrow_a + 68u * b, ptok));
                        dvb[b] = __uint_as_float(lds32_dep(vrow_b + 68u * b, ptok));
                    }
                }
            }
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                sc[0] += dka[b] * sa[b][0];
                sc[1] += dka[b] * sa[b][1];
                sc[2] += dkb[b] * sa[b][2];
                sc[3] += dkb[b] * sa[b][3];
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) sc[x] *= p.q_scale;

            bool msk[4] = {false, false, false, false};
            if (!full) {
                const int pos_a = SPARSE ? ((key_a >> 3) ? fpos[2] : fpos[0]) + (key_a & 3) : kv_base + key_a;
                const int pos_b = SPARSE ? ((key_a >> 3) ? fpos[3] : fpos[1]) + (key_a & 3) : pos_a + 4;
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
                // a key no row can see may hold never-written bytes: keep its scales finite
                if (msk[0] && msk[1]) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) dva[b] = 0.0f;
                }
                if (msk[2] && msk[3]) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) dvb[b] = 0.0f;
                }
            }
            l_run[0] += pr[0] + pr[2];
            l_run[1] += pr[1] + pr[3];
            // P x d_v per scale block as B fragments (k = key, n = query row): fp16 value + fp16 residual
            uint32_t pb[NB][2], pl[NB][2];
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const float pd[4] = {pr[0] * dva[b], pr[1] * dva[b], pr[2] * dvb[b], pr[3] * dvb[b]};
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const __half2 hi = __floats2half2_rn(pd[2 * x], pd[2 * x + 1]);
                    const float2 hf = __half22float2(hi);
                    const __half2 lo = __floats2half2_rn(pd[2 * x] - hf.x, pd[2 * x + 1] - hf.y);
                    pb[b][x] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hi));
                    pl[b][x] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&lo));
                }
            }

            // ---- O^T += V^T (P d_v)^T: m-tile mt covers the channels of code word vw(mt >> 1) -----------
            //   FP8: vw = vword0 + 16 jj + x, mt = 4 jj + 2 x + ps;  Q8_0: vw = 16 b + vword0 + 8 x, mt = 4 b + 2 x + ps
            const uint32_t vr = st + vrow_off;
            auto pv_word = [&](uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3, int mt, int blk) {
                // bytes (token a, token b) of channels 0, 1 | 2, 3 of the word
                const uint32_t ab01 = __byte_perm(t0, t1, 0x5140), ab23 = __byte_perm(t0, t1, 0x7362);
                const uint32_t cd01 = __byte_perm(t2, t3, 0x5140), cd23 = __byte_perm(t2, t3, 0x7362);
                uint32_t a0, a1, a2, a3;
                kv8x4_to_f16x4<FMT>(ab01, a0, a1);
                kv8x4_to_f16x4<FMT>(cd01, a2, a3);
                mma16816(o[mt], a0, a1, a2, a3, pb[blk][0], pb[blk][1]);
                mma16816(o[mt], a0, a1, a2, a3, pl[blk][0], pl[blk][1]);
                kv8x4_to_f16x4<FMT>(ab23, a0, a1);
                kv8x4_to_f16x4<FMT>(cd23, a2, a3);
                mma16816(o[mt + 1], a0, a1, a2, a3, pb[blk][0], pb[blk][1]);
                mma16816(o[mt + 1], a0, a1, a2, a3, pl[blk][0], pl[blk][1]);
            };
            if (FP8) {
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const uint32_t off = 4u * (uint32_t)(vword0 + 16 * jj);
                    const uint2 w0 = lds64_dep(vr + off, ptok);
                    const uint2 w1 = lds64_dep(vr + G::kRow + off, ptok);
                    const uint2 w2 = lds64_dep(vr + 4u * G::kRow + off, ptok);
                    const uint2 w3 = lds64_dep(vr + 5u * G::kRow + off, ptok);
                    pv_word(w0.x, w1.x, w2.x, w3.x, 4 * jj, jj >> 1);
                    pv_word(w0.y, w1.y, w2.y, w3.y, 4 * jj + 2, jj >> 1);
                }
            } else {
#pragma unroll
                for (int b = 0; b < 4; ++b) {
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const uint32_t off = (uint32_t)(68 * b + 4 + 4 * (vword0 + 8 * x));
                        const uint32_t t0 = lds32_dep(vr + off, ptok);
                        const uint32_t t1 = lds32_dep(vr + G::kRow + off, ptok);
                        const uint32_t t2 = lds32_dep(vr + 4u * G::kRow + off, ptok);
                        const uint32_t t3 = lds32_dep(vr + 5u * G::kRow + off, ptok);
                        pv_word(t0, t1, t2, t3, 4 * b + 2 * x, b);
                    }
                }
            }
            __syncwarp();   // every lane is done with stage s before it is refilled
            if (clear_tail) fence_proxy_async();   // the cleared rows precede the next copy into s
        }

        if (failed) {
            for (int s = 0; s < STAGES; ++s) {
                if (pending & (1u << s)) (void)mbar_wait(bars + 8u * s, (phase_bits >> s) & 1u);
            }
            if (lane == 0) atomicOr(&hdr->status, 1);
            break;
        }

        // ---- partial: natural column order, through the idle ring -----------------------------------
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
            l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
        }
        float* stage_o = reinterpret_cast<float*>(ring_gen);   // [8 rows][256]
#pragma unroll
        for (int mt = 0; mt < 16; ++mt) {
            // m-tile mt: row gid = channel c, row gid + 8 = channel c + 1
            const int vw = FP8 ? vword0 + 16 * (mt >> 2) + ((mt >> 1) & 1) : 16 * (mt >> 2) + vword0 + 8 * ((mt >> 1) & 1);
            const int c = 4 * vw + 2 * (mt & 1);
            *reinterpret_cast<float2*>(stage_o + (2 * tig) * kHeadDim + c) = make_float2(o[mt][0], o[mt][2]);
            *reinterpret_cast<float2*>(stage_o + (2 * tig + 1) * kHeadDim + c) = make_float2(o[mt][1], o[mt][3]);
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

static bool kv8_attention_layout_ok(const warp34_kv_layer_layout* l) {
    const bool k8 = l->k_format == WARP34_KV_FORMAT_Q8_0 || l->k_format == WARP34_KV_FORMAT_FP8_E4M3;
    const bool v8 = l->v_format == WARP34_KV_FORMAT_Q8_0 || l->v_format == WARP34_KV_FORMAT_FP8_E4M3;
    return k8 && v8 && l->head_dim == kHeadDim && l->block_size == kPageTokens &&
           l->k_transform == WARP34_KV_TRANSFORM_IDENTITY && l->v_transform == WARP34_KV_TRANSFORM_IDENTITY;
}

// The tensor-core path serves K and V of one 8-bit format in the canonical packing with 16-byte-aligned
// runs, an 8-byte-aligned query and a workspace that holds the plan and at least one CTA's partial slots.
static bool kv8_stream_ok(const warp34_exec* ex, const warp34_kv_layer_layout* l, const warp34_attention_batch* b,
                          const void* q_in, int io_bf16) {
    if (l->k_format != l->v_format) return false;
    const uint64_t row = l->k_format == WARP34_KV_FORMAT_FP8_E4M3 ? (uint64_t)Kv8Stage<WARP34_KV_FORMAT_FP8_E4M3>::kRow
                                                                  : (uint64_t)Kv8Stage<WARP34_KV_FORMAT_Q8_0>::kRow;
    if (l->k_token_stride_bytes != row || l->v_token_stride_bytes != row) return false;
    if ((l->k_base | l->v_base | l->k_page_stride_bytes | l->v_page_stride_bytes | l->k_head_stride_bytes |
         l->v_head_stride_bytes) & 15u) {
        return false;
    }
    if (!io_bf16 && ((uintptr_t)q_in & 7u) != 0) return false;
    if (b->block_tables == nullptr || b->max_blocks_per_req <= 0) return false;
    return ex->scratch_ptr != 0 && (ex->scratch_ptr & 15u) == 0;
}

static int launch_kv8_stream(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                             const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                             int num_q_heads, int io_bf16, bool* taken) {
    *taken = false;
    int rc = 0;
    DeviceInfo* dev = device_info(&rc);
    if (dev == nullptr) return rc;
    const size_t slot_bytes = (size_t)kPartialFloats * sizeof(float);
    const long long full_workers = (long long)dev->sm_count * kKv8StreamWarps;
    auto workers_for = [&](int reqs, long long tokens) -> long long {
        warp34_attention_batch b = *batch;
        b.num_reqs = reqs;
        b.total_tokens = (int)tokens;
        const long long items = items_bound(layout, &b, num_q_heads, kRowsPerGroup);
        if (items * (long long)batch->max_blocks_per_req >= 0x7fffffffll) return -1;
        const size_t plan = plan_bytes(reqs);
        const size_t avail = ex->scratch_size > plan ? ex->scratch_size - plan : 0;
        const long long w = (long long)(avail / slot_bytes) - items;
        return w < 0 ? 0 : w;
    };
    long long workers = 0;
    const int reqs_per_pass = pick_reqs_per_pass(batch, full_workers, kKv8StreamWarps, true, workers_for, &workers);
    if (workers < kKv8StreamWarps) return 0;      // the caller falls back to the fp32 kernel
    const bool in_parts = reqs_per_pass < batch->num_reqs;
    const bool fp8 = layout->k_format == WARP34_KV_FORMAT_FP8_E4M3;
    const uint32_t stage = 2u * (uint32_t)(fp8 ? Kv8Stage<WARP34_KV_FORMAT_FP8_E4M3>::kRunStride
                                               : Kv8Stage<WARP34_KV_FORMAT_Q8_0>::kRunStride);
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
            rc = (int)cudaFuncSetAttribute(kv8_attention_stream_kernel<WARP34_KV_FORMAT_FP8_E4M3, kKv8StreamStages>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)((uint32_t)(kKv8StreamWarps * kKv8StreamStages) *
                                                 (2u * Kv8Stage<WARP34_KV_FORMAT_FP8_E4M3>::kRunStride + 8u)));
            if (rc != 0) return rc;
            rc = (int)cudaFuncSetAttribute(kv8_attention_stream_kernel<WARP34_KV_FORMAT_Q8_0, kKv8StreamStages>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)((uint32_t)(kKv8StreamWarps * kKv8StreamStages) *
                                                 (2u * Kv8Stage<WARP34_KV_FORMAT_Q8_0>::kRunStride + 8u)));
            if (rc != 0) return rc;
            done[d] = true;
        }
    }
    cudaStream_t st = (cudaStream_t)ex->stream;
    for (int r0 = 0; r0 < batch->num_reqs; r0 += reqs_per_pass) {
        const int reqs = (batch->num_reqs - r0 < reqs_per_pass) ? batch->num_reqs - r0 : reqs_per_pass;
        StreamParams p;
        p.og.gate = nullptr;
        p.og.mode = 0;
        p.layout = *layout;
        p.batch = in_parts ? batch_part(batch, r0, reqs) : *batch;
        const long long items = items_bound(layout, &p.batch, num_q_heads, kRowsPerGroup);
        long long part_workers = in_parts ? workers_for(reqs, p.batch.total_tokens) : workers;   // the last part is smaller
        if (part_workers > full_workers) part_workers = full_workers;
        const int grid = (int)(part_workers / kKv8StreamWarps);
        if (grid < 1) return (int)cudaErrorInvalidValue;
        p.q_in = q_in;
        p.attn_out = attn_out;
        p.io_bf16 = io_bf16;
        p.triple_out = nullptr;
        p.scratch = reinterpret_cast<uint8_t*>((uintptr_t)ex->scratch_ptr);
        p.num_q_heads = num_q_heads;
        p.gqa = num_q_heads / layout->local_kv_heads;
        p.num_warps = grid * kKv8StreamWarps;
        p.max_slots = (int)(p.num_warps + items);
        p.smem_bytes = smem;
        p.rows_per_group = kRowsPerGroup;
        p.q_scale = batch->sm_scale * 1.4426950408889634f;
        p.natural = 1;
        p.qfrag = nullptr;
        p.q_groups_max = 0;
        p.rows_from_first_token = in_parts ? 1 : 0;
        p.keep_status = r0 > 0 ? 1 : 0;
        tq4_attention_plan_kernel<<<1, 32, 0, st>>>(p);
        if (fp8) {
            kv8_attention_stream_kernel<WARP34_KV_FORMAT_FP8_E4M3, kKv8StreamStages><<<grid, kKv8StreamWarps * 32, smem, st>>>(p);
        } else {
            kv8_attention_stream_kernel<WARP34_KV_FORMAT_Q8_0, kKv8StreamStages><<<grid, kKv8StreamWarps * 32, smem, st>>>(p);
        }
        const long long rows = (long long)p.batch.total_tokens * num_q_heads;
        if (rows * 4 < (long long)grid * kKv8StreamWarps / 8) {
            tq4_attention_merge_kernel<false, 32><<<(unsigned)rows, 1024, 0, st>>>(p);
        } else {
            tq4_attention_merge_kernel<false, 4><<<(unsigned)rows, 128, 0, st>>>(p);
        }
        rc = (int)cudaGetLastError();
        if (rc != 0) return rc;
    }
    *taken = true;
    return 0;
}

// allow_stream = false: the fp32 dequant-then-attend kernel whatever the layout (the scalar entry
// point and WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION).
static int launch_kv8_attention(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                                int num_q_heads, int io_bf16, bool allow_stream = false) {
    if (batch->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (layout->local_kv_heads <= 0 || num_q_heads % layout->local_kv_heads != 0 || batch->num_reqs <= 0) {
        return (int)cudaErrorInvalidValue;
    }
    if (layout->k_base == 0 || layout->v_base == 0) return (int)cudaErrorInvalidValue;
    if (allow_stream && kv8_stream_ok(ex, layout, batch, q_in, io_bf16)) {
        bool taken = false;
        const int rc = launch_kv8_stream(ex, layout, batch, q_in, attn_out, num_q_heads, io_bf16, &taken);
        if (rc != 0 || taken) return rc;
    }
    if ((layout->k_base | layout->v_base | layout->k_page_stride_bytes | layout->k_head_stride_bytes |
         layout->k_token_stride_bytes | layout->v_page_stride_bytes | layout->v_head_stride_bytes |
         layout->v_token_stride_bytes) & 3u) {
        return (int)cudaErrorInvalidValue;   // rows are read as 32-bit words
    }
    const int gqa = num_q_heads / layout->local_kv_heads;
    if (gqa > kKv8MaxGqa) return (int)cudaErrorNotSupported;
    const long long items = (long long)batch->total_tokens * layout->local_kv_heads;
    if (items > 0x7fffffffll) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)items;
    cudaStream_t st = (cudaStream_t)ex->stream;
    // One block fills an SM (registers): few (token, kv head) items leave SMs idle and long rows
    // finish last.  With a scratch buffer every row's pages are cut into `splits` ranges, about
    // four blocks per SM in all, and a second launch combines the states.
    int splits = 1;
    float* partials = nullptr;
    {
        int rc = 0;
        DeviceInfo* dev = device_info(&rc);
        const long long want = dev != nullptr ? (4ll * dev->sm_count + items - 1) / items : 1;
        const size_t per_split = (size_t)items * gqa * kRowTripleFloats * sizeof(float);
        if (want > 1 && ex->scratch_ptr != 0 && (ex->scratch_ptr & 15u) == 0 && per_split > 0) {
            long long fit = (long long)(ex->scratch_size / per_split);
            long long sp = want < 16 ? want : 16;
            if (sp > fit) sp = fit;
            if (sp > 1) {
                splits = (int)sp;
                partials = reinterpret_cast<float*>((uintptr_t)ex->scratch_ptr);
            }
        }
    }
    const dim3 grid(blocks, (unsigned)splits);
#define W34_KV8_CASE(Gv) case Gv: kv8_attention_kernel<Gv><<<grid, kKv8Warps * 32, 0, st>>>(*layout, *batch, q_in, attn_out, num_q_heads, io_bf16, splits, partials); break
    switch (gqa) {
        W34_KV8_CASE(1); W34_KV8_CASE(2); W34_KV8_CASE(3); W34_KV8_CASE(4);
        W34_KV8_CASE(5); W34_KV8_CASE(6); W34_KV8_CASE(7); W34_KV8_CASE(8);
        default: return (int)cudaErrorNotSupported;
    }
#undef W34_KV8_CASE
    if (splits > 1) {
        const long long rows = (long long)batch->total_tokens * num_q_heads;
        kv8_merge_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(*layout, *batch, attn_out, num_q_heads, io_bf16,
                                                                     splits, partials);
    }
    return (int)cudaGetLastError();
}

}  // namespace w34
