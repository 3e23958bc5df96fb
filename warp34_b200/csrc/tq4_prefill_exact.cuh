// Chunked-prefill attention over TQ4 pages that meets 2e-3 + 1e-2 |b| against dequant-then-attend on
// every element: register-fragment MMAs (mma.sync m16n8k16, fp32 accumulators) whose fp16 operands
// are fed as value + rounding residual.  Included by tq4_attention.cu (shares the PTX wrappers, the
// lookup-table layout and the geometry helpers of the streaming kernel).
//
// Replaces paged_attention_prefill_mma_f16_kernel<64 / 128> (crates/warp34-kernels/csrc/ops/
// op_paged_attn.cu:594-1128) for head_dim 256, 16-token pages, canonical TQ4 packing.  It is the
// default for chunks; the tcgen05 kernel (tq4_prefill_tc.cuh) is several times faster and is taken
// with WARP34_B200_EXEC_FLAG_FAST_ATTENTION, at single-fp16-operand accuracy.
//
// One CTA = 128 query rows (128 / gqa tokens x gqa heads of one kv head) = 8 warps of 16 rows.
// All warps walk the same pages: lane 0 of warp 0 bulk-copies the raw (page, head) runs into a
// ring of shared-memory stages (full barrier: transaction bytes; empty barrier: one arrival per
// warp), and every warp dequantises straight into MMA fragments through the byte-pair tables, as the
// streaming kernel does, so no dequantised tile ever exists in shared memory:
//   S[16 rows x 16 keys]  = Q' K^T      A = Q' fragments (shared memory, prepared once per CTA),
//                                        B = K centroids from the table (value and residual)
//                                        three products per k-step: Q' K, Q'_res K, Q' K_res
//   O[16 rows x 256]     += (P d_v) V   A = P d_v straight from the score accumulators' layout
//                                        (value and residual), B = V centroids from the table;
//                                        on pages with a large weight also (P d_v) V_res
// Scales stay outside the operands: scores are d0 S[0:128] + d1 S[128:256], P is multiplied by the
// V scale of its key and 128-half.  No scratch, no split: a CTA walks every page its rows can see.
#pragma once

namespace w34 {

constexpr int kPxWarps = 8;
constexpr int kPxRows = 16 * kPxWarps;
constexpr int kPxStages = 4;
constexpr uint32_t kPxQHiBytes = 16u * 32u * 16u;   // per warp [k-step][lane][a0 a1 a2 a3]
constexpr uint32_t kPxQLoBytes = 16u * 32u * 8u;    // per warp [k-step][lane][two residual bytes per register]

struct PrefillExactParams {
    warp34_kv_layer_layout layout;
    warp34_attention_batch batch;
    const void* q_in;
    void* attn_out;
    int io_bf16;
    int num_q_heads;
    int gqa;
    int tok_per_tile;      // rows of a CTA (128 or 64) / gqa
    float q_scale;         // sm_scale * log2(e) / kLutScale
    int32_t* status;       // may be null; bit 0: a wait gave up, bit 1: shared-memory window too small
    uint32_t smem_bytes;
    OutputGate og;
};

__device__ __forceinline__ uint4 lds128_v(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64_v(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts16(uint32_t addr, unsigned short v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ void sts8(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void mma16816_a4(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    mma16816(c, a[0], a[1], a[2], a[3], b0, b1);
}

// WARPS = 8: 128 query rows per CTA.  WARPS = 4: 64 rows, for launches whose 128-row tiles would leave SMs empty (a short
// chunk): twice the CTAs, and half as many warps share an SM's tensor pipe.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) tq4_attention_prefill_exact_kernel(const PrefillExactParams p) {
    constexpr int kRows = 16 * WARPS;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    const uint32_t win_lo = smem_u32(smem);
    const uint32_t win_hi = win_lo + p.smem_bytes;
    const uint32_t lut_addr = (win_lo + 0xffffu) & ~0xffffu;

    SmemCarver carve(win_lo, lut_addr, win_hi);
    uint32_t qhi = 0, ring = 0, bars = 0;
    for (int w = 0; w < WARPS; ++w) {
        const uint32_t a = carve.take(kPxQHiBytes + kPxQLoBytes, 16);
        if (w == wid) qhi = a;
    }
    ring = carve.take(kPxStages * kStageStride, 128);
    bars = carve.take(2 * kPxStages * 8, 8);        // full[stage], then empty[stage]
    const uint32_t red = carve.take((4 * WARPS + 1) * 4 + kRows * 4, 4);   // per-warp key ranges, abort flag, row steps
    if (!carve.ok) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, 2);
        return;
    }
    const uint32_t qlo = qhi + kPxQHiBytes;
    uint8_t* qhi_gen = smem + (qhi - win_lo);
    int* s_lo = reinterpret_cast<int*>(smem + (red - win_lo));
    int* s_hi = s_lo + WARPS;
    int* s_slo = s_hi + WARPS;
    int* s_shi = s_slo + WARPS;
    int* s_failed = s_shi + WARPS;
    float* s_qstep = reinterpret_cast<float*>(s_failed + 1);   // [128 rows]: step of the row's Q' residual bytes

    // Tables as in the exact streaming kernel: (value pair, residual pair) in 16
    // copies of 8 bytes for K, value pair in 32 copies of 4 bytes in the upper half of the entry for V.
    for (int i = tid; i < 256 * 32; i += blockDim.x) {
        const int byte = i >> 5, ln = i & 31;
        const float c0 = kLutScale * tq4_centroid(byte & 15), c1 = kLutScale * tq4_centroid(byte >> 4);
        const uint32_t hi = pack_half2(c0, c1);
        const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
        if (ln < 16) {
            sts32(lut_addr + (uint32_t)(byte * 256 + ln * 8), hi);
            sts32(lut_addr + (uint32_t)(byte * 256 + ln * 8 + 4),
                  pack_half2(c0 - hf.x, c1 - hf.y));
        }
        sts32(lut_addr + (uint32_t)(byte * 256 + 128 + ln * 4), hi);
    }
    if (tid == 0) {
        for (int s = 0; s < kPxStages; ++s) {
            mbar_init(bars + 8u * s, 1u);
            mbar_init(bars + 8u * (kPxStages + s), (uint32_t)WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *s_failed = 0;
    }

    // ---- which (request, token tile) is this CTA? ---------------------------------------------
    const int tpt = p.tok_per_tile;
    const int kv_head = blockIdx.y;
    int req = -1, tile_in_req = 0;
    {
        int t = blockIdx.x;
        for (int r = 0; r < p.batch.num_reqs; ++r) {
            const int ql = p.batch.query_start_loc[r + 1] - p.batch.query_start_loc[r];
            const int nt = (ql + tpt - 1) / tpt;
            if (t < nt) { req = r; tile_in_req = t; break; }
            t -= nt;
        }
    }
    if (req < 0) return;   // block-uniform
    const ReqGeom g = load_req(p.batch, req);
    if (!g.valid) return;
    const int tok0 = tile_in_req * tpt;
    const int ntok = min(tpt, g.q_len - tok0);
    const int rows_used = ntok * p.gqa;

    // this lane's two rows: 16 wid + gid and + 8
    int rmax[2], rmin[2];
    bool rvalid[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int row = 16 * wid + gid + 8 * x;
        const int q_off = tok0 + row / p.gqa;
        rvalid[x] = row < rows_used &&
                    (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
        rmax[x] = rvalid[x] ? row_max_kv(p.batch, g, q_off) : -1;
        rmin[x] = rvalid[x] ? row_min_kv(p.batch, g, q_off) : 0x7fffffff;
    }
    {
        int lo = min(rmin[0], rmin[1]), hi = max(rmax[0], rmax[1]);
        int slo = max(rvalid[0] ? rmin[0] : 0, rvalid[1] ? rmin[1] : 0);
        int shi = min(rvalid[0] ? rmax[0] : 0x7fffffff, rvalid[1] ? rmax[1] : 0x7fffffff);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, d));
            hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, d));
            slo = max(slo, __shfl_xor_sync(0xffffffffu, slo, d));
            shi = min(shi, __shfl_xor_sync(0xffffffffu, shi, d));
        }
        if (lane == 0) { s_lo[wid] = lo; s_hi[wid] = hi; s_slo[wid] = slo; s_shi[wid] = shi; }
    }

    // ---- Q' rows of this warp -> A fragments in shared memory ---------------------------------
    // Element (row rr, rotated column c) belongs to k-step ks = 2 (4 half + (vw & 3)) + (e >> 2) of
    // lane (rr & 7, tig = vw >> 2), register 2 ((e >> 1) & 1) + (rr >> 3), half-word e & 1, where
    // (half, vw, e) is the position of c in the row's code words (vword_col is the inverse map).
    for (int rr = 0; rr < 16; ++rr) {
        const int row = 16 * wid + rr;
        const int q_off = tok0 + row / p.gqa;
        const int q_head = kv_head * p.gqa + row % p.gqa;
        const bool ok = row < rows_used &&
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
        // Q' = hi + lo, hi the fp16 value just below Q': 0 <= lo < 1 ulp, stored as a byte in units of the
        // row's step (largest lo / 255); as the low byte of an fp16 word that byte is the subnormal
        // number byte x 2^-24, exact and free to widen.
        float lo_max = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float f = tv[j] * p.q_scale;
            lo_max = fmaxf(lo_max, f - __half2float(__float2half_rd(f)));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) lo_max = fmaxf(lo_max, __shfl_xor_sync(0xffffffffu, lo_max, d));
        const float step = lo_max * (1.0f / 255.0f);
        const float inv_step = step > 0.0f ? 1.0f / step : 0.0f;
        if (lane == 0) s_qstep[16 * wid + rr] = step * 16777216.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = lane + 32 * j;
            int half, vw, e;
            if (c >= 128) { half = 1; vw = (c - 128) >> 3; e = (c - 128) & 7; }
            else if (c < 4) { half = 0; vw = 0; e = c; }
            else if (c >= 124) { half = 0; vw = 0; e = c - 120; }
            else { half = 0; vw = (c + 4) >> 3; e = (c + 4) & 7; }
            const int ks = 2 * (4 * half + (vw & 3)) + (e >> 2);
            const int dst_lane = (rr & 7) * 4 + (vw >> 2);
            const int reg = 2 * ((e >> 1) & 1) + (rr >> 3);
            const float f = tv[j] * p.q_scale;
            const __half h = __float2half_rd(f);
            const uint32_t r8 = (uint32_t)max(min(__float2int_rn((f - __half2float(h)) * inv_step), 255), 0);
            sts16(qhi + (uint32_t)(ks * 512 + dst_lane * 16 + reg * 4 + (e & 1) * 2), __half_as_ushort(h));
            sts8(qlo + (uint32_t)(ks * 256 + dst_lane * 8 + reg * 2 + (e & 1)), r8 & 0xffu);
        }
    }
    __syncthreads();   // tables, barriers, fragments and the per-warp key ranges are in place

    int kv_lo = 0x7fffffff, kv_hi = -1, safe_lo = 0, safe_hi = 0x7fffffff;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
        kv_lo = min(kv_lo, s_lo[w]); kv_hi = max(kv_hi, s_hi[w]);
        safe_lo = max(safe_lo, s_slo[w]); safe_hi = min(safe_hi, s_shi[w]);
    }
    const int pg_lo = (kv_hi >= kv_lo) ? (kv_lo >> 4) : 0;
    const int npages = (kv_hi >= kv_lo) ? ((kv_hi >> 4) - pg_lo + 1) : 0;
    // steps (x 2^24) of the Q' residual bytes of the two rows whose scores this lane holds
    const float qstep_a = s_qstep[16 * wid + gid], qstep_b = s_qstep[16 * wid + gid + 8];

    float o[32][4];
#pragma unroll
    for (int n = 0; n < 32; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};

    const int32_t* blocks = p.batch.block_tables + (size_t)req * p.batch.max_blocks_per_req;
    const uint8_t* k_head_base = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
    const uint8_t* v_head_base = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
    // MMA column n of S <-> token key(n) = (n & 3) + 8 ((n >> 2) & 1) + 4 (n >> 3) of the page: this lane
    // supplies the K codes of tokens key_a (n = gid) and key_a + 4 (n = gid + 8) ...
    const int key_a = (gid & 3) + 8 * (gid >> 2);
    // ... and holds the scores, and supplies the V codes, of tokens kv0 + {0, 1, 4, 5}.
    const int kv0 = 2 * (tig & 1) + 8 * (tig >> 1);
    const uint32_t lut_lane = lut_addr + 128u + 4u * lane;        // V values
    const uint32_t lutk_lane = lut_addr + 8u * (lane & 15);       // K (and V) value + residual
    int issued = 0;       // thread 0: pages whose copies have been issued
    bool failed = false;

    auto issue = [&](int idx) {   // thread 0 only
        const int s = idx % kPxStages;
        const int32_t page = block_table_page(blocks, pg_lo + idx, p.batch.max_blocks_per_req, kInPrefillExact);
        const uint32_t bar = bars + 8u * s;
        const uint32_t dst = ring + (uint32_t)s * kStageStride;
        const uint8_t* ksrc = k_head_base + (size_t)page * p.layout.k_page_stride_bytes;
        const uint8_t* vsrc = v_head_base + (size_t)page * p.layout.v_page_stride_bytes;
        mbar_expect_tx(bar, 4 * kHalfBytes);
        bulk_g2s(dst, ksrc, kHalfBytes, bar);
        bulk_g2s(dst + kHalfStride, ksrc + kHalfBytes, kHalfBytes, bar);
        bulk_g2s(dst + kRunStride, vsrc, kHalfBytes, bar);
        bulk_g2s(dst + kRunStride + kHalfStride, vsrc + kHalfBytes, kHalfBytes, bar);
        issued = idx + 1;
    };
    fence_proxy_async();
    if (tid == 0) {
        for (int i = 0; i < kPxStages - 1 && i < npages; ++i) issue(i);
    }

#pragma unroll 1
    for (int i = 0; i < npages; ++i) {
        const int s = i % kPxStages;
        if (tid == 0) {
            // page i + kPxStages - 1 goes into the stage page i - 1 used: every warp must have left it
            const int ahead = i + kPxStages - 1;
            if (ahead < npages) {
                bool ok = true;
                if (i >= 1) ok = mbar_wait(bars + 8u * (kPxStages + (ahead % kPxStages)), (uint32_t)(((i - 1) / kPxStages) & 1));
                if (ok) issue(ahead); else *s_failed = 1;
            }
        }
        {   // warp-uniform: a lane whose wait ran out takes the whole warp with it
            const bool ok = mbar_wait(bars + 8u * s, (uint32_t)((i / kPxStages) & 1)) &&
                            *reinterpret_cast<volatile int*>(s_failed) == 0;
            if (!__all_sync(0xffffffffu, ok)) { failed = true; break; }
        }

        const uint32_t kst = ring + (uint32_t)s * kStageStride;
        const uint32_t vst = kst + kRunStride;
        const int kv_base = (pg_lo + i) << 4;
        const bool full = (kv_base >= safe_lo) && (kv_base + 15 <= safe_hi);
        const uint32_t ptok = page_token(i);
#define W34_LDS(addr) lds32_dep(addr, ptok)
#define W34_LUT(word, k) lds32_lut(__byte_perm((word), lut_lane, 0x7604 + ((k) << 4)))
#define W34_LUTK(word, k) lds64_lut(__byte_perm((word), lutk_lane, 0x7604 + ((k) << 4)))

        // ---- S = Q' K^T: n-tile 0 = tokens key(0..7), n-tile 1 = tokens key(8..15); per 128-half;
        //      sa also takes the product with the K residuals; sr the one with the Q' residual bytes,
        //      which carries the steps of the rows (gid for c = 0, 1; gid + 8 for c = 2, 3) ----------
        float sa[2][2][4], sr[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                sa[h][n][0] = sa[h][n][1] = sa[h][n][2] = sa[h][n][3] = 0.0f;
                sr[h][n][0] = sr[h][n][1] = sr[h][n][2] = sr[h][n][3] = 0.0f;
            }
        }
        const uint32_t krow_a = kst + token_offset(key_a);
        const uint32_t krow_b = krow_a + 4u * kTq4RowBytes;
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) {
            const int half = s8 >> 2;
            uint32_t wa, wb;
            if (half == 0) {
                const uint32_t off = 4u * (4u * tig + (s8 & 3));
                wa = W34_LDS(krow_a + off);
                wb = W34_LDS(krow_b + off);
                if ((s8 & 3) == 0 && tig == 0) {   // virtual word 0 of half 0: splice (W0 >> 16) | (W16 << 16)
                    wa = (wa >> 16) | (W34_LDS(krow_a + 64) << 16);
                    wb = (wb >> 16) | (W34_LDS(krow_b + 64) << 16);
                }
            } else {
                const uint32_t off = 4u * (17u + 4u * tig + (s8 & 3));
                wa = W34_LDS(krow_a + off);
                wb = W34_LDS(krow_b + off);
            }
#pragma unroll
            for (int hk = 0; hk < 2; ++hk) {
                const int ks = 2 * s8 + hk;
                const uint4 qh4 = lds128_v(qhi + (uint32_t)(ks * 512 + lane * 16));
                const uint2 ql2 = lds64_v(qlo + (uint32_t)(ks * 256 + lane * 8));
                const uint32_t qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
                const uint32_t qr[4] = {__byte_perm(ql2.x, 0, 0x4140), __byte_perm(ql2.x, 0, 0x4342),
                                        __byte_perm(ql2.y, 0, 0x4140), __byte_perm(ql2.y, 0, 0x4342)};
                const uint2 e0 = W34_LUTK(wa, 2 * hk), e1 = W34_LUTK(wb, 2 * hk);
                const uint2 e2 = W34_LUTK(wa, 2 * hk + 1), e3 = W34_LUTK(wb, 2 * hk + 1);
                mma16816_a4(sa[half][0], qh, e0.x, e2.x);
                mma16816_a4(sa[half][1], qh, e1.x, e3.x);
                mma16816_a4(sr[half][0], qr, e0.x, e2.x);
                mma16816_a4(sr[half][1], qr, e1.x, e3.x);
                mma16816_a4(sa[half][0], qh, e0.y, e2.y);
                mma16816_a4(sa[half][1], qh, e1.y, e3.y);
            }
        }
        // ---- scales of this lane's four tokens kv0 + {0, 1, 4, 5} (index 2 n + e) -------------------
        float dk0[4], dk1[4], dv0[4], dv1[4];
        {
            const uint32_t kq = kst + token_offset(kv0), vq = vst + token_offset(kv0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t off = (uint32_t)((j & 1) + 4 * (j >> 1)) * kTq4RowBytes;
                dk0[j] = __half2float(__ushort_as_half((unsigned short)(W34_LDS(kq + off) & 0xffffu)));
                dk1[j] = __half2float(__ushort_as_half((unsigned short)(W34_LDS(kq + off + 64) >> 16)));
                dv0[j] = __half2float(__ushort_as_half((unsigned short)(W34_LDS(vq + off) & 0xffffu)));
                dv1[j] = __half2float(__ushort_as_half((unsigned short)(W34_LDS(vq + off + 64) >> 16)));
            }
        }
        // sc[n][c]: c = 0, 1: row gid, tokens 2 n + {0, 1} of the four; c = 2, 3: row gid + 8
        float sc[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = 2 * n + (c & 1);
                const float qs = (c < 2) ? qstep_a : qstep_b;
                sc[n][c] = dk0[j] * (sa[0][n][c] + sr[0][n][c] * qs) + dk1[j] * (sa[1][n][c] + sr[1][n][c] * qs);
            }
        }
        bool msk[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) msk[n][c] = false;
        }
        if (!full) {
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int pos = kv_base + kv0 + e + 4 * n;
                    msk[n][e] = !(pos >= rmin[0] && pos <= rmax[0]);
                    msk[n][2 + e] = !(pos >= rmin[1] && pos <= rmax[1]);
                    if (msk[n][e]) sc[n][e] = -1e30f;
                    if (msk[n][2 + e]) sc[n][2 + e] = -1e30f;
                    // a key no row of the CTA can see may hold never-written bytes: keep its V scale finite
                    if (pos > kv_hi || pos < kv_lo) { dv0[2 * n + e] = 0.0f; dv1[2 * n + e] = 0.0f; }
                }
            }
        }
        // ---- online softmax: rows gid (x = 0) and gid + 8 (x = 1); the four lanes of a quad share a row
        float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
        float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
#pragma unroll
        for (int d = 1; d < 4; d <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, d));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, d));
        }
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        if (__any_sync(0xffffffffu, mn0 > m_run[0] || mn1 > m_run[1])) {
            const float al0 = ex2(m_run[0] - mn0), al1 = ex2(m_run[1] - mn1);
            l_run[0] *= al0;
            l_run[1] *= al1;
#pragma unroll
            for (int n = 0; n < 32; ++n) { o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1; }
            m_run[0] = mn0;
            m_run[1] = mn1;
        }
        float pr[2][4];
        float pk0 = 0.0f, pk1 = 0.0f, ps0 = 0.0f, ps1 = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            pr[n][0] = msk[n][0] ? 0.0f : ex2(sc[n][0] - mn0);
            pr[n][1] = msk[n][1] ? 0.0f : ex2(sc[n][1] - mn0);
            pr[n][2] = msk[n][2] ? 0.0f : ex2(sc[n][2] - mn1);
            pr[n][3] = msk[n][3] ? 0.0f : ex2(sc[n][3] - mn1);
            ps0 += pr[n][0] + pr[n][1];
            ps1 += pr[n][2] + pr[n][3];
            pk0 = fmaxf(pk0, fmaxf(pr[n][0], pr[n][1]));
            pk1 = fmaxf(pk1, fmaxf(pr[n][2], pr[n][3]));
        }
        // row totals (every lane of a quad holds the same l): a page is peaked when one key holds more
        // than kPeakedWeight of a row's softmax mass so far
#pragma unroll
        for (int d = 1; d < 4; d <<= 1) {
            ps0 += __shfl_xor_sync(0xffffffffu, ps0, d);
            ps1 += __shfl_xor_sync(0xffffffffu, ps1, d);
        }
        l_run[0] += ps0;
        l_run[1] += ps1;
        // rows that do not exist score 0 against their zero query; they must not count as peaks
        const bool peaked = __any_sync(0xffffffffu, (rvalid[0] && pk0 > kPxPeakedWeight * l_run[0]) ||
                                                    (rvalid[1] && pk1 > kPxPeakedWeight * l_run[1]));
        // The fp16 rounding residual of P d_v (2^-12 relative, independent from key to key) goes through
        // its own product only on pages where some key holds more than kPResidualWeight of a row's mass
        // so far: keys below it move an output by less than 1.4e-4 sqrt(kPResidualWeight) max|v| in all.
        const bool p_residual = __any_sync(0xffffffffu, (rvalid[0] && pk0 > kPResidualWeight * l_run[0]) ||
                                                        (rvalid[1] && pk1 > kPResidualWeight * l_run[1]));
        // P d_v as A fragments (k = the page's 16 tokens), value and residual, one set per 128-half of V
        float pd[2][2][4];   // [half][n][c]
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                pd[0][n][c] = pr[n][c] * dv0[2 * n + (c & 1)];
                pd[1][n][c] = pr[n][c] * dv1[2 * n + (c & 1)];
            }
        }
        uint32_t pa[2][4], pl[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int r4 = 0; r4 < 4; ++r4) {   // a0: n 0 row gid, a1: n 0 row gid + 8, a2: n 1 row gid, a3: n 1 row gid + 8
                const int n = r4 >> 1, c = 2 * (r4 & 1);
                const __half2 hi = __floats2half2_rn(pd[h][n][c], pd[h][n][c + 1]);
                const float2 hf = __half22float2(hi);
                const __half2 lo = __floats2half2_rn(pd[h][n][c] - hf.x, pd[h][n][c + 1] - hf.y);
                pa[h][r4] = *reinterpret_cast<const uint32_t*>(&hi);
                pl[h][r4] = *reinterpret_cast<const uint32_t*>(&lo);
            }
        }

        // ---- O += (P d_v) V.  Step (i4, t): the streaming kernel's 16-channel tile, here two n-tiles:
        //      channels of table rows gid (2 (4 i4 + t)) and gid + 8 (2 (4 i4 + t) + 1) ---------------
        const uint32_t vr = vst + token_offset(kv0);
        const uint32_t vwb = 4u * (uint32_t)(gid >> 1) + (uint32_t)(gid & 1);
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
                const uint32_t a0 = W34_LUT(lo_ab, t);
                const uint32_t a1 = W34_LUT(hi_ab, t);
                const uint32_t a2 = W34_LUT(lo_cd, t);
                const uint32_t a3 = W34_LUT(hi_cd, t);
                const int n = 2 * (4 * i4 + t);
                mma16816_a4(o[n], pa[half], a0, a2);
                mma16816_a4(o[n + 1], pa[half], a1, a3);
            }
        }
        if (p_residual) {   // (P d_v)_residual V, a second pass over the page's V codes
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
                    const uint32_t a0 = W34_LUT(lo_ab, t);
                    const uint32_t a1 = W34_LUT(hi_ab, t);
                    const uint32_t a2 = W34_LUT(lo_cd, t);
                    const uint32_t a3 = W34_LUT(hi_cd, t);
                    const int n = 2 * (4 * i4 + t);
                    mma16816_a4(o[n], pl[half], a0, a2);
                    mma16816_a4(o[n + 1], pl[half], a1, a3);
                }
            }
        }
        if (peaked) {   // (P d_v) V_residual, a second pass over the page's V codes
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
                    const int n = 2 * (4 * i4 + t);
                    mma16816_a4(o[n], pa[half], e0.y, e2.y);
                    mma16816_a4(o[n + 1], pa[half], e1.y, e3.y);
                }
            }
        }
#undef W34_LUT
#undef W34_LUTK
#undef W34_LDS
        __syncwarp();                                       // every lane is done with stage s
        if (lane == 0) mbar_arrive(bars + 8u * (kPxStages + s));
    }

    if (failed) {
        if (lane == 0) {
            *s_failed = 1;
            if (p.status != nullptr) atomicOr(p.status, 1);
        }
        // The CTA must not end under copies in flight; shared memory lives until its last thread
        // leaves, so thread 0 alone waits (bounded) for the last use of every stage it filled.
        if (tid == 0) {
            for (int j = max(0, issued - kPxStages); j < issued; ++j) {
                (void)mbar_wait(bars + 8u * (j % kPxStages), (uint32_t)((j / kPxStages) & 1));
            }
        }
        return;
    }

    // ---- epilogue: normalise, inverse rotation, store; 8 rows at a time through this warp's
    //      fragment area (8 KB of fp32) -------------------------------------------------------------
    const float inv0 = (l_run[0] > 0.0f) ? (1.0f / (l_run[0] * kLutScale)) : 0.0f;
    const float inv1 = (l_run[1] > 0.0f) ? (1.0f / (l_run[1] * kLutScale)) : 0.0f;
    float* ostage = reinterpret_cast<float*>(qhi_gen);   // [8 rows][256]
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        __syncwarp();
        // accumulator (n-tile, column 2 tig + e) holds the channel the table lane with gid' = 2 tig + e supplied
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const int half = i4 >> 1;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int g2 = 2 * tig + e;
                    const int vw = 4 * (g2 >> 1) + (g2 & 1) + 2 * (i4 & 1);
                    const int n = 2 * (4 * i4 + t);
                    ostage[gid * kHeadDim + vword_col(half, vw, 2 * t)] = o[n][2 * x + e] * (x ? inv1 : inv0);
                    ostage[gid * kHeadDim + vword_col(half, vw, 2 * t + 1)] = o[n + 1][2 * x + e] * (x ? inv1 : inv0);
                }
            }
        }
        __syncwarp();
        for (int rr = 0; rr < 8; ++rr) {
            const int row = 16 * wid + rr + 8 * x;
            const int q_off = tok0 + row / p.gqa;
            const int q_head = kv_head * p.gqa + row % p.gqa;
            const bool ok = row < rows_used &&
                            (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
            if (!ok) continue;   // warp-uniform
            float tv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) tv[j] = ostage[rr * kHeadDim + lane + 32 * j];
            wht256_lanes(tv, lane);
            const size_t out_base = ((size_t)(g.q_start + q_off) * p.num_q_heads + q_head) * kHeadDim;
            store_output_row(p.attn_out, out_base, tv, lane, p.io_bf16, p.og);
        }
    }
}

}  // namespace w34
