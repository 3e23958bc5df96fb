// Query-sparse paged attention over the KV pool: every token attends only to a list of selected
// 4-token groups.  Included by tq4_attention.cu.
//
// Replaces warp34_qsa_sparse_paged_attn_f16 / _hadamard_f16 of the reference
// (crates/warp34-kernels/csrc/ops/op_qsa.cu:716-1075 GQA kernel, :1076-1155 split merge, :1161-1448
// per-head fallback, :1450-1572 launcher, entry points :1711-1752) for head_dim 256, 16-token pages
// and the row formats this library stores: TQ4 with the Rademacher + WHT-256 rotation, Q8_0 and
// FP8 E4M3 unrotated.  Semantics kept from there:
//   * selected_phys_blocks[tok][i] is a physical group id = page * 4 + group in page (negative: skip),
//     selected_logical_blocks[tok][i] its logical group index; key (i, off) sits at logical position
//     4 * logical + off and takes part iff that is <= token_seq_pos[tok]; only the first
//     num_selected_blocks[tok] entries are read;
//   * a token masked out by valid_token_mask gets ZERO output rows (not untouched ones);
//   * the sigmoid gate multiplies the fp32 result (no rounding before it); the Hadamard-64 variant then
//     rounds to fp16 and rotates every 64 columns.
// Two paths.  With a workspace (ex->scratch_ptr) and the canonical packing the lists run on the
// tensor-core stream kernels (tq4_attention_stream_kernel<.., sparse> for TQ4 rows,
// kv8_attention_stream_kernel<.., sparse> for 8-bit rows: launch_qsa_stream in tq4_attention.cu).
// Otherwise (no workspace, other strides, WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION) the fp32
// dequant-then-attend kernel of this file: one block of four warps per (token, group of G query heads
// that share a kv head, split); a warp takes every fourth selected group and handles its four rows in
// one step: one read and one dequantisation of each K and V row serve all G heads, the loads of the
// four rows are issued before the first is used and their score reductions interleave.  The selected
// range is cut into `splits` parts when a workspace is there; without one the kernel runs unsplit.
#pragma once

namespace w34 {

constexpr int kQsaWarps = 4;
constexpr int kQsaMaxG = 8;
constexpr int kQsaMaxSplits = 16;

struct QsaParams {
    warp34_kv_layer_layout layout;
    const uint16_t* q;                 // fp16 [tokens, q heads, 256]
    const uint16_t* gate;              // fp16, same shape, or null
    const int32_t* sel_phys;           // [tokens, select_k]
    const int32_t* sel_logical;        // [tokens, select_k]
    const int32_t* num_selected;       // [tokens]
    const int32_t* seq_pos;            // [tokens]
    const uint8_t* valid_token_mask;   // [tokens] or null
    uint16_t* out;                     // fp16 [tokens, q heads, 256]
    float* partials;                   // [tokens, q groups, splits, G, 258] when splits > 1
    int num_tokens, num_q_heads, group_heads, select_k, splits, hadamard;
    float sm_scale;
};

struct QsaRaw {
    uint32_t w0, w1;
    float d;
};

// Lane L owns columns [8 L, 8 L + 8) of the stored row (rotated columns for TQ4).
__device__ __forceinline__ QsaRaw qsa_load_raw(const uint8_t* row, int format, int lane) {
    if (format == WARP34_KV_FORMAT_TQ4) {
        QsaRaw r;
        const uint8_t* blk = row + kTq4BlockBytes * (lane >> 4);
        r.d = __half2float(*reinterpret_cast<const __half*>(blk));
        const uint16_t* c = reinterpret_cast<const uint16_t*>(blk + 2 + 4 * (lane & 15));
        r.w0 = (uint32_t)c[0] | ((uint32_t)c[1] << 16);
        r.w1 = 0u;
        return r;
    }
    const Kv8Raw k = kv8_load_raw(row, format, lane);
    QsaRaw r;
    r.w0 = k.w0; r.w1 = k.w1; r.d = k.d;
    return r;
}

__device__ __forceinline__ void qsa_decode(const QsaRaw& r, int format, const float* centroids, float (&x)[8]) {
    if (format == WARP34_KV_FORMAT_TQ4) {
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = r.d * centroids[(r.w0 >> (4 * e)) & 15u];
    } else {
        Kv8Raw k;
        k.w0 = r.w0; k.w1 = r.w1; k.d = r.d;
        kv8_decode(k, format, x);
    }
}

// One finished row: acc_n[e] = normalised output at stored column 8 lane + e.  Through `row_smem` to
// the column-interleaved layout, inverse rotation and sign for rotated V, gate, Hadamard-64, store.
__device__ __forceinline__ void qsa_finish_row(const QsaParams& p, float* row_smem, const float (&acc_n)[8],
                                               size_t row_base, int lane) {
#pragma unroll
    for (int e = 0; e < 8; ++e) row_smem[8 * lane + e] = acc_n[e];
    __syncwarp();
    float t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = row_smem[lane + 32 * j];
    __syncwarp();
    if (p.layout.v_transform == WARP34_KV_TRANSFORM_RADEMACHER_WHT256) {
        wht256_lanes(t, lane);
#pragma unroll
        for (int j = 0; j < 8; ++j) t[j] = apply_sign(t[j], lane + 32 * j);
    }
    if (p.gate != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float g = __half2float(__ushort_as_half(p.gate[row_base + lane + 32 * j]));
            t[j] *= sigmoid_gate(g);
        }
    }
    if (p.hadamard) hadamard64_row(t, lane, 0);
#pragma unroll
    for (int j = 0; j < 8; ++j) p.out[row_base + lane + 32 * j] = __half_as_ushort(__float2half_rn(t[j]));
}

template <int G>
__global__ void __launch_bounds__(kQsaWarps * 32) qsa_sparse_attention_kernel(const QsaParams p) {
    __shared__ float s_acc[kQsaWarps][G][kHeadDim];     // query staging first, then the warps' states
    __shared__ float s_ml[kQsaWarps][G][2];
    __shared__ float s_centroid[16];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int tok = (int)blockIdx.x, qgroup = (int)blockIdx.y, split = (int)blockIdx.z;
    const int head0 = qgroup * G;
    const int gqa = p.num_q_heads / p.layout.local_kv_heads;
    const int kv_head = head0 / gqa;
    // every exit below is taken by the whole block
    if (p.valid_token_mask != nullptr && p.valid_token_mask[tok] == 0) {
        if (p.splits == 1) {
            for (int i = threadIdx.x; i < G * kHeadDim; i += blockDim.x) {
                p.out[((size_t)tok * p.num_q_heads + head0) * kHeadDim + i] = 0;
            }
        }
        return;   // with splits the merge kernel writes the zeros
    }
    if (threadIdx.x < 16) s_centroid[threadIdx.x] = tq4_centroid(threadIdx.x);
    const bool rotated_k = p.layout.k_transform == WARP34_KV_TRANSFORM_RADEMACHER_WHT256;

    // ---- queries: warp w prepares heads w, w + 4; afterwards lane L holds columns [8 L, 8 L + 8) ----
    for (int h = wid; h < G; h += kQsaWarps) {
        const size_t base = ((size_t)tok * p.num_q_heads + head0 + h) * kHeadDim;
        float t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            t[j] = __half2float(__ushort_as_half(p.q[base + lane + 32 * j])) * p.sm_scale;
            if (rotated_k) t[j] = apply_sign(t[j], lane + 32 * j);
        }
        if (rotated_k) wht256_lanes(t, lane);
#pragma unroll
        for (int j = 0; j < 8; ++j) s_acc[0][h][lane + 32 * j] = t[j];
    }
    __syncthreads();
    float qv[G][8], acc[G][8], m_i[G], l_i[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { qv[h][e] = s_acc[0][h][8 * lane + e]; acc[h][e] = 0.0f; }
        m_i[h] = -1e30f;
        l_i[h] = 0.0f;
    }
    __syncthreads();

    // ---- this block's part of the selected list ---------------------------------------------------
    int n_sel = p.num_selected[tok];
    if (n_sel > p.select_k) n_sel = p.select_k;
    const int seq_pos = p.seq_pos[tok];
    const int per_split = (n_sel + p.splits - 1) / p.splits;
    const int g_lo = split * per_split, g_hi = min(n_sel, g_lo + per_split);
    const int32_t* phys = p.sel_phys + (size_t)tok * p.select_k;
    const int32_t* logical = p.sel_logical + (size_t)tok * p.select_k;
    const uint8_t* k_head = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
    const uint8_t* v_head = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
    for (int gi = g_lo + wid; gi < g_hi; gi += kQsaWarps) {
        const int pg = phys[gi];
        const int visible = seq_pos - 4 * logical[gi] + 1;      // rows 0 .. visible - 1 of the group take part
        if (pg < 0 || visible <= 0) continue;                   // warp-uniform
        const int page = pool_page(pg >> 2, kInSparse);
        const int row0 = 4 * (pg & 3);
        const int n_rows = visible < 4 ? visible : 4;
        const uint8_t* kp = k_head + (size_t)page * p.layout.k_page_stride_bytes + (size_t)row0 * p.layout.k_token_stride_bytes;
        const uint8_t* vp = v_head + (size_t)page * p.layout.v_page_stride_bytes + (size_t)row0 * p.layout.v_token_stride_bytes;
        QsaRaw kr[4], vr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int off = min(i, n_rows - 1);                 // past the end: re-read the last row, unused
            kr[i] = qsa_load_raw(kp + (size_t)off * p.layout.k_token_stride_bytes, p.layout.k_format, lane);
            vr[i] = qsa_load_raw(vp + (size_t)off * p.layout.v_token_stride_bytes, p.layout.v_format, lane);
        }
        float dot[4][G];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float kx[8];
            qsa_decode(kr[i], p.layout.k_format, s_centroid, kx);
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
        float vx[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) qsa_decode(vr[i], p.layout.v_format, s_centroid, vx[i]);
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float m_new = m_i[h];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i >= n_rows) dot[i][h] = -1e30f;
                m_new = fmaxf(m_new, dot[i][h]);
            }
            const float alpha = __expf(m_i[h] - m_new);
            float pr[4], psum = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pr[i] = (i < n_rows) ? __expf(dot[i][h] - m_new) : 0.0f;
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

    // ---- fold warps 1..3 into warp 0 ----------------------------------------------------------------
    if (wid != 0) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s_acc[wid][h][8 * lane + e] = acc[h][e];
            if (lane == 0) { s_ml[wid][h][0] = m_i[h]; s_ml[wid][h][1] = l_i[h]; }
        }
    }
    __syncthreads();
    if (wid != 0) return;
    for (int w = 1; w < kQsaWarps; ++w) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            const float m_o = s_ml[w][h][0], l_o = s_ml[w][h][1];
            const float m_new = fmaxf(m_i[h], m_o);
            const float a = __expf(m_i[h] - m_new), b = (l_o > 0.0f) ? __expf(m_o - m_new) : 0.0f;
            l_i[h] = l_i[h] * a + l_o * b;
            m_i[h] = m_new;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[h][e] = acc[h][e] * a + s_acc[w][h][8 * lane + e] * b;
        }
    }
    if (p.splits > 1) {
        float* dst = p.partials + ((((size_t)tok * gridDim.y + qgroup) * p.splits + split) * G) * kRowTripleFloats;
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
        float acc_n[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc_n[e] = acc[h][e] * inv_l;
        qsa_finish_row(p, &s_acc[0][0][0], acc_n, ((size_t)tok * p.num_q_heads + head0 + h) * kHeadDim, lane);
    }
}

// Combines the `splits` states of every (token, q head): one warp per output row.
__global__ void __launch_bounds__(128) qsa_sparse_merge_kernel(const QsaParams p) {
    __shared__ float s_row[4][kHeadDim];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 4 + wid;
    if (row >= (long long)p.num_tokens * p.num_q_heads) return;
    const int tok = (int)(row / p.num_q_heads), q_head = (int)(row % p.num_q_heads);
    const size_t row_base = (size_t)row * kHeadDim;
    if (p.valid_token_mask != nullptr && p.valid_token_mask[tok] == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) p.out[row_base + lane + 32 * j] = 0;
        return;
    }
    const int G = p.group_heads;
    const int qgroup = q_head / G, h = q_head - qgroup * G;
    const int qgroups = p.num_q_heads / G;
    const float* base = p.partials + ((((size_t)tok * qgroups + qgroup) * p.splits) * G + h) * kRowTripleFloats;
    const size_t stride = (size_t)G * kRowTripleFloats;
    float m_tot = -1e30f;
    for (int s = 0; s < p.splits; ++s) {
        const float* t = base + s * stride;
        if (t[kHeadDim + 1] > 0.0f) m_tot = fmaxf(m_tot, t[kHeadDim]);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float l_tot = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
        const float* t = base + s * stride;
        const float ls = t[kHeadDim + 1];
        if (ls > 0.0f) {
            const float w = __expf(t[kHeadDim] - m_tot);
            l_tot += ls * w;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += t[8 * lane + e] * w;
        }
    }
    const float inv_l = (l_tot > 0.0f) ? (1.0f / l_tot) : 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv_l;
    qsa_finish_row(p, s_row[wid], acc, row_base, lane);
}

static int launch_qsa_stream(const warp34_exec* ex, const QsaParams& q, bool* taken);   // tq4_attention.cu

static bool qsa_layout_ok(const warp34_kv_layer_layout* l) {
    if (l->head_dim != kHeadDim || l->block_size != kPageTokens || l->local_kv_heads <= 0 || l->k_base == 0 || l->v_base == 0) {
        return false;
    }
    auto side_ok = [](int fmt, int tr, uint64_t base, uint64_t ps, uint64_t hs, uint64_t ts) {
        if (fmt == WARP34_KV_FORMAT_TQ4) {
            return tr == WARP34_KV_TRANSFORM_RADEMACHER_WHT256 && ((base | ps | hs | ts) & 1u) == 0;   // 16-bit reads
        }
        if (fmt == WARP34_KV_FORMAT_Q8_0 || fmt == WARP34_KV_FORMAT_FP8_E4M3) {
            return tr == WARP34_KV_TRANSFORM_IDENTITY && ((base | ps | hs | ts) & 3u) == 0;           // 32-bit reads
        }
        return false;
    };
    return side_ok(l->k_format, l->k_transform, l->k_base, l->k_page_stride_bytes, l->k_head_stride_bytes, l->k_token_stride_bytes) &&
           side_ok(l->v_format, l->v_transform, l->v_base, l->v_page_stride_bytes, l->v_head_stride_bytes, l->v_token_stride_bytes);
}

static int launch_qsa_sparse(const warp34_exec* ex, const void* q, const void* gate, const warp34_kv_layer_layout* layout,
                             const int32_t* sel_phys, const int32_t* sel_logical, const int32_t* num_selected,
                             const int32_t* seq_pos, const uint8_t* valid_token_mask, void* out, int num_tokens,
                             int num_q_heads, int select_k, float sm_scale, int hadamard) {
    // the reference's argument checks (op_qsa.cu:1464-1470)
    if (ex == nullptr || q == nullptr || layout == nullptr || sel_phys == nullptr || sel_logical == nullptr ||
        num_selected == nullptr || seq_pos == nullptr || out == nullptr || num_tokens < 0 || num_q_heads <= 0 ||
        layout->local_kv_heads <= 0 || num_q_heads % layout->local_kv_heads != 0 || layout->head_dim != kHeadDim ||
        select_k < 0) {
        return (int)cudaErrorInvalidValue;
    }
    if (!qsa_layout_ok(layout)) return (int)cudaErrorNotSupported;
    if (num_tokens == 0) return 0;
    const int gqa = num_q_heads / layout->local_kv_heads;
    int G = 1;
    for (int cand = kQsaMaxG; cand >= 1; --cand) {
        if (gqa % cand == 0) { G = cand; break; }
    }
    const int qgroups = num_q_heads / G;
    int rc = 0;
    DeviceInfo* dev = device_info(&rc);
    if (dev == nullptr) return rc;
    // about four blocks per SM, at least two selected groups per warp of a split, and only with scratch
    int splits = 1;
    {
        const long long blocks = (long long)num_tokens * qgroups;
        long long want = (4ll * dev->sm_count + blocks - 1) / blocks;
        const long long by_work = select_k / (2 * kQsaWarps);
        if (want > by_work) want = by_work;
        if (want > kQsaMaxSplits) want = kQsaMaxSplits;
        const size_t per_split = (size_t)num_tokens * num_q_heads * kRowTripleFloats * sizeof(float);
        if (want > 1 && ex->scratch_ptr != 0 && (ex->scratch_ptr & 15u) == 0) {
            const long long fit = (long long)(ex->scratch_size / per_split);
            if (want > fit) want = fit;
            if (want > 1) splits = (int)want;
        }
    }
    QsaParams p;
    p.layout = *layout;
    p.q = static_cast<const uint16_t*>(q);
    p.gate = static_cast<const uint16_t*>(gate);
    p.sel_phys = sel_phys;
    p.sel_logical = sel_logical;
    p.num_selected = num_selected;
    p.seq_pos = seq_pos;
    p.valid_token_mask = valid_token_mask;
    p.out = static_cast<uint16_t*>(out);
    p.partials = splits > 1 ? reinterpret_cast<float*>((uintptr_t)ex->scratch_ptr) : nullptr;
    p.num_tokens = num_tokens;
    p.num_q_heads = num_q_heads;
    p.group_heads = G;
    p.select_k = select_k;
    p.splits = splits;
    p.hadamard = hadamard;
    p.sm_scale = sm_scale;
    {
        // canonical packing with enough workspace: the tensor-core stream kernels (TQ4 or 8-bit rows)
        bool taken = false;
        const int rcs = launch_qsa_stream(ex, p, &taken);
        if (rcs != 0 || taken) return rcs;
    }
    cudaStream_t st = (cudaStream_t)ex->stream;
    if (qgroups > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)num_tokens, (unsigned)qgroups, (unsigned)splits);
#define W34_QSA_CASE(Gv) case Gv: qsa_sparse_attention_kernel<Gv><<<grid, kQsaWarps * 32, 0, st>>>(p); break
    switch (G) {
        W34_QSA_CASE(1); W34_QSA_CASE(2); W34_QSA_CASE(3); W34_QSA_CASE(4);
        W34_QSA_CASE(5); W34_QSA_CASE(6); W34_QSA_CASE(7); W34_QSA_CASE(8);
        default: return (int)cudaErrorNotSupported;
    }
#undef W34_QSA_CASE
    if (splits > 1) {
        const long long rows = (long long)num_tokens * num_q_heads;
        qsa_sparse_merge_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(p);
    }
    return (int)cudaGetLastError();
}

}  // namespace w34

extern "C" int warp34_qsa_sparse_paged_attn_f16(const warp34_exec* ex, const void* q, const void* gate,
                                                const warp34_kv_layer_layout* kv_layout,
                                                const int32_t* selected_phys_blocks,
                                                const int32_t* selected_logical_blocks,
                                                const int32_t* num_selected_blocks, const int32_t* token_seq_pos,
                                                const uint8_t* valid_token_mask, void* out, int num_tokens,
                                                int local_q_heads, int select_k_blocks, float sm_scale) {
    return w34::launch_qsa_sparse(ex, q, gate, kv_layout, selected_phys_blocks, selected_logical_blocks,
                                  num_selected_blocks, token_seq_pos, valid_token_mask, out, num_tokens, local_q_heads,
                                  select_k_blocks, sm_scale, 0);
}

extern "C" int warp34_qsa_sparse_paged_attn_hadamard_f16(const warp34_exec* ex, const void* q, const void* gate,
                                                         const warp34_kv_layer_layout* kv_layout,
                                                         const int32_t* selected_phys_blocks,
                                                         const int32_t* selected_logical_blocks,
                                                         const int32_t* num_selected_blocks,
                                                         const int32_t* token_seq_pos, const uint8_t* valid_token_mask,
                                                         void* out, int num_tokens, int local_q_heads,
                                                         int select_k_blocks, float sm_scale) {
    return w34::launch_qsa_sparse(ex, q, gate, kv_layout, selected_phys_blocks, selected_logical_blocks,
                                  num_selected_blocks, token_seq_pos, valid_token_mask, out, num_tokens, local_q_heads,
                                  select_k_blocks, sm_scale, 1);
}
