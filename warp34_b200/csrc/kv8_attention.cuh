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

static bool kv8_attention_layout_ok(const warp34_kv_layer_layout* l) {
    const bool k8 = l->k_format == WARP34_KV_FORMAT_Q8_0 || l->k_format == WARP34_KV_FORMAT_FP8_E4M3;
    const bool v8 = l->v_format == WARP34_KV_FORMAT_Q8_0 || l->v_format == WARP34_KV_FORMAT_FP8_E4M3;
    return k8 && v8 && l->head_dim == kHeadDim && l->block_size == kPageTokens &&
           l->k_transform == WARP34_KV_TRANSFORM_IDENTITY && l->v_transform == WARP34_KV_TRANSFORM_IDENTITY;
}

static int launch_kv8_attention(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                                int num_q_heads, int io_bf16) {
    if (batch->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (layout->local_kv_heads <= 0 || num_q_heads % layout->local_kv_heads != 0 || batch->num_reqs <= 0) {
        return (int)cudaErrorInvalidValue;
    }
    if (layout->k_base == 0 || layout->v_base == 0) return (int)cudaErrorInvalidValue;
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
