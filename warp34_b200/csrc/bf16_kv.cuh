// Uncompressed BF16 KV path (the comparison arm of the long-context configuration).
//
// Replaces, for BF16 storage with identity transforms, head_dim 256 and 16-token pages:
//   kv_cache_write_bf16_kernel + warp34_kv_cache_write[_strided]_bf16
//       (crates/warp34-kernels/csrc/ops/op_kv_cache.cu:798-824, :1170-1205)
//   paged_attention_gqa_bf16_kernel + warp34_paged_attention_bf16
//       (op_kv_cache.cu:873-1168, :1207-1241)
//
// Rows are 512 B, a (page, head) run is 8 KB for K and 8 KB for V: this path is HBM-bound at
// four times the bytes of TQ4 and has no dequantisation, so the kernel is the plain split-KV
// stream: one warp per share of the flattened (request, kv head, 16-row group, page) list,
// pages staged by cp.async (16-byte chunks into rows padded to 528 B, which makes ldmatrix
// bank-conflict-free; a bulk copy cannot pad), bf16 m16n8k16 MMAs with fp32 accumulation.
// Q and K are exact bf16 operands, so scores are fp32-exact; P is split into bf16 hi + lo
// (two MMAs) so the output keeps fp32-like weights.  The (m, l, acc) partials go through the
// same plan / merge kernels as the TQ4 path, without the rotation.
// Included at the end of tq4_attention.cu: shares the plan / merge kernels and the PTX wrappers.
#include <cuda_bf16.h>

namespace w34 {

constexpr int kBfWarps = 6;
constexpr int kBfStages = 2;
constexpr int kBfRowStride = 528;                       // bytes per staged row (512 + 16 pad)
constexpr int kBfTileBytes = 16 * kBfRowStride;         // one K or V tile
constexpr int kBfStageBytes = 2 * kBfTileBytes;         // K then V
constexpr int kBfRows = 16;                             // query rows per work item

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(128) kv_cache_write_bf16_kernel(const warp34_kv_layer_layout layout,
                                                                 const warp34_attention_batch batch,
                                                                 const void* __restrict__ k_in,
                                                                 const void* __restrict__ v_in, int row_stride_elems,
                                                                 int vec16) {
    // one warp per (token, head): 32 lanes x 16 B = one 512-byte row of K and one of V
    const int lane = threadIdx.x & 31;
    const long long idx = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int heads = layout.local_kv_heads;
    if (idx >= (long long)batch.total_tokens * heads) return;
    const int tok = (int)(idx / heads), head = (int)(idx % heads);
    if (batch.valid_token_mask != nullptr && batch.valid_token_mask[tok] == 0) return;
    const int req = find_request(batch.query_start_loc, batch.num_reqs, tok);
    if (req < 0 || (batch.valid_req_mask != nullptr && batch.valid_req_mask[req] == 0)) return;
    const int slot = batch.write_slot_mapping[tok];
    if (slot < 0 || !write_slot_ok(slot, kInBf16)) return;
    const int page = slot >> 4, off = slot & 15;
    const uint64_t kd = layout.k_base + (uint64_t)page * layout.k_page_stride_bytes +
                        (uint64_t)head * layout.k_head_stride_bytes + (uint64_t)off * layout.k_token_stride_bytes;
    const uint64_t vd = layout.v_base + (uint64_t)page * layout.v_page_stride_bytes +
                        (uint64_t)head * layout.v_head_stride_bytes + (uint64_t)off * layout.v_token_stride_bytes;
    const size_t src = (size_t)tok * row_stride_elems + (size_t)head * kHeadDim;   // in elements
    if (vec16) {
        reinterpret_cast<uint4*>((uintptr_t)kd)[lane] = reinterpret_cast<const uint4*>(k_in)[src / 8 + lane];
        reinterpret_cast<uint4*>((uintptr_t)vd)[lane] = reinterpret_cast<const uint4*>(v_in)[src / 8 + lane];
    } else {
        const uint16_t* ks = reinterpret_cast<const uint16_t*>(k_in) + src;
        const uint16_t* vs = reinterpret_cast<const uint16_t*>(v_in) + src;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            reinterpret_cast<uint16_t*>((uintptr_t)kd)[lane + 32 * j] = ks[lane + 32 * j];
            reinterpret_cast<uint16_t*>((uintptr_t)vd)[lane + 32 * j] = vs[lane + 32 * j];
        }
    }
}

__global__ void __launch_bounds__(kBfWarps * 32, 1) bf16kv_attention_stream_kernel(const StreamParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int PARTIAL = kBfRows * kHeadDim + 2 * kBfRows;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int gid = lane >> 2, tig = lane & 3;
    uint8_t* ring_gen = smem + (size_t)wid * kBfStages * kBfStageBytes;
    const uint32_t ring = smem_u32(ring_gen);

    const int R = p.batch.num_reqs;
    const PlanHeader* hdr = reinterpret_cast<const PlanHeader*>(p.scratch);
    const int32_t* unit_prefix = plan_array(p.scratch, 0, R);
    const int32_t* item_prefix = plan_array(p.scratch, 1, R);
    const int32_t* page_lo_a = plan_array(p.scratch, 2, R);
    const int32_t* npages_a = plan_array(p.scratch, 3, R);
    const int32_t* ngroups_a = plan_array(p.scratch, 4, R);
    float* partials = reinterpret_cast<float*>(p.scratch + plan_bytes(R));

    const int worker = blockIdx.x * kBfWarps + wid;
    const int per = hdr->units_per_warp;
    const int total_units = hdr->total_units;
    const long long u_ll = (long long)worker * per;
    if (per <= 0 || u_ll >= total_units) return;
    int u = (int)u_ll;
    const int u_end = min(u + per, total_units);
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

        int rmax[2], rmin[2];
        bool rvalid[2];
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            const int row = group * kBfRows + gid + 8 * x;
            const int q_off = row / p.gqa;
            rvalid[x] = row < rows_in_req &&
                        (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
            rmax[x] = rvalid[x] ? row_max_kv(p.batch, g, q_off) : -1;
            rmin[x] = rvalid[x] ? row_min_kv(p.batch, g, q_off) : 0x7fffffff;
        }
        int safe_hi = min(rvalid[0] ? rmax[0] : 0x7fffffff, rvalid[1] ? rmax[1] : 0x7fffffff);
        int safe_lo = max(rvalid[0] ? rmin[0] : 0, rvalid[1] ? rmin[1] : 0);
        int kv_hi = max(rmax[0], rmax[1]);
#pragma unroll
        for (int d = 4; d < 32; d <<= 1) {
            safe_hi = min(safe_hi, __shfl_xor_sync(0xffffffffu, safe_hi, d));
            safe_lo = max(safe_lo, __shfl_xor_sync(0xffffffffu, safe_lo, d));
            kv_hi = max(kv_hi, __shfl_xor_sync(0xffffffffu, kv_hi, d));
        }

        // ---- Q rows (pre-scaled, bf16) -> A fragments, staged through the idle ring -----------------
        uint32_t qa[16][4];
        {
            __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(ring_gen);   // [16][264]
            for (int rr = 0; rr < kBfRows; ++rr) {
                const int row = group * kBfRows + rr;
                const int q_off = row / p.gqa;
                const int q_head = kv_head * p.gqa + row % p.gqa;
                const bool ok = row < rows_in_req &&
                                (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + q_off] != 0);
                const size_t q_base = ((size_t)(g.q_start + q_off) * p.num_q_heads + q_head) * kHeadDim;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float x = ok ? load_act(p.q_in, q_base + lane + 32 * j, p.io_bf16) : 0.0f;
                    stage[rr * 264 + lane + 32 * j] = __float2bfloat16_rn(x);
                }
            }
            __syncwarp();
            const uint32_t* st32 = reinterpret_cast<const uint32_t*>(stage);
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                qa[ks][0] = st32[(gid * 264 + 16 * ks + 2 * tig) >> 1];
                qa[ks][1] = st32[((gid + 8) * 264 + 16 * ks + 2 * tig) >> 1];
                qa[ks][2] = st32[(gid * 264 + 16 * ks + 8 + 2 * tig) >> 1];
                qa[ks][3] = st32[((gid + 8) * 264 + 16 * ks + 8 + 2 * tig) >> 1];
            }
            __syncwarp();
        }

        float o[32][4];
#pragma unroll
        for (int n = 0; n < 32; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }
        float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.0f, 0.0f};

        const int32_t* blocks = p.batch.block_tables + (size_t)r * p.batch.max_blocks_per_req;
        const uint8_t* k_head_base = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
        const uint8_t* v_head_base = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
        auto issue = [&](int idx) {
            const int32_t page = block_table_page(blocks, pg0 + idx, p.batch.max_blocks_per_req, kInBf16);
            const uint8_t* ks = k_head_base + (size_t)page * p.layout.k_page_stride_bytes + lane * 16;
            const uint8_t* vs = v_head_base + (size_t)page * p.layout.v_page_stride_bytes + lane * 16;
            const uint32_t dst = ring + (uint32_t)(idx % kBfStages) * kBfStageBytes + lane * 16;
#pragma unroll
            for (int row = 0; row < 16; ++row) {
                cp_async16(dst + row * kBfRowStride, ks + (size_t)row * p.layout.k_token_stride_bytes);
                cp_async16(dst + kBfTileBytes + row * kBfRowStride, vs + (size_t)row * p.layout.v_token_stride_bytes);
            }
            cp_async_commit();
        };
        issue(0);
#pragma unroll 1
        for (int i = 0; i < n_here; ++i) {
            if (i + 1 < n_here) issue(i + 1); else cp_async_commit();   // keep one group per iteration
            cp_async_wait<1>();
            __syncwarp();
            const uint32_t kt = ring + (uint32_t)(i % kBfStages) * kBfStageBytes, vt = kt + kBfTileBytes;
            const int kv_base = (pg0 + i) << 4;
            const bool full = (kv_base >= safe_lo) && (kv_base + 15 <= safe_hi);

            float sacc[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) { sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.0f; }
            const uint32_t kaddr = kt + (uint32_t)(((lane & 7) + 8 * (lane >> 4)) * kBfRowStride + 16 * ((lane >> 3) & 1));
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, kaddr + 32u * ks);
                mma16816_bf16(sacc[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
                mma16816_bf16(sacc[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
            }
            float sc[2][4];
            bool msk[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) { sc[n][e] = sacc[n][e] * p.q_scale; msk[n][e] = false; }
            }
            if (!full) {
#pragma unroll
                for (int n = 0; n < 2; ++n) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int pos = kv_base + 8 * n + 2 * tig + e;
                        msk[n][e] = !(pos >= rmin[0] && pos <= rmax[0]);
                        msk[n][2 + e] = !(pos >= rmin[1] && pos <= rmax[1]);
                        if (msk[n][e]) sc[n][e] = -1e30f;
                        if (msk[n][2 + e]) sc[n][2 + e] = -1e30f;
                    }
                }
            }
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
                l_run[0] *= al0; l_run[1] *= al1;
#pragma unroll
                for (int n = 0; n < 32; ++n) { o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1; }
                m_run[0] = mn0; m_run[1] = mn1;
            }
            float pr[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                pr[n][0] = msk[n][0] ? 0.0f : ex2(sc[n][0] - mn0);
                pr[n][1] = msk[n][1] ? 0.0f : ex2(sc[n][1] - mn0);
                pr[n][2] = msk[n][2] ? 0.0f : ex2(sc[n][2] - mn1);
                pr[n][3] = msk[n][3] ? 0.0f : ex2(sc[n][3] - mn1);
                l_run[0] += pr[n][0] + pr[n][1];
                l_run[1] += pr[n][2] + pr[n][3];
            }
            // P = hi + lo in bf16.  Keys past the sequence may hold never-written bytes (NaN
            // patterns); their P is exactly zero, but 0 x NaN is NaN inside the MMA, so such pages
            // zero those V rows' contribution by clearing the tile rows first.
            if (!full && kv_base + 15 > kv_hi) {
                for (int row = max(kv_hi + 1 - kv_base, 0); row < 16; ++row) {
                    *reinterpret_cast<uint4*>(ring_gen + (size_t)(i % kBfStages) * kBfStageBytes + kBfTileBytes +
                                              row * kBfRowStride + lane * 16) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const float a = pr[n][2 * x], b = pr[n][2 * x + 1];
                    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                    const float2 hf = __bfloat1622float2(h);
                    ph[2 * n + x] = *reinterpret_cast<const uint32_t*>(&h);
                    pl[2 * n + x] = pack_bf162(a - hf.x, b - hf.y);
                }
            }
            const uint32_t vaddr = vt + (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * kBfRowStride + 16 * (lane >> 4));
#pragma unroll
            for (int np = 0; np < 16; ++np) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vaddr + 32u * np);
                mma16816_bf16(o[2 * np], ph[0], ph[1], ph[2], ph[3], b[0], b[1]);
                mma16816_bf16(o[2 * np], pl[0], pl[1], pl[2], pl[3], b[0], b[1]);
                mma16816_bf16(o[2 * np + 1], ph[0], ph[1], ph[2], ph[3], b[2], b[3]);
                mma16816_bf16(o[2 * np + 1], pl[0], pl[1], pl[2], pl[3], b[2], b[3]);
            }
            __syncwarp();   // stage may be overwritten by the copy issued in the next iteration
        }
        cp_async_wait<0>();
        __syncwarp();

        // ---- partial: rows gid and gid + 8, natural column order --------------------------------------
#pragma unroll
        for (int d = 1; d < 4; d <<= 1) {
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], d);
            l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], d);
        }
        if (slot < p.max_slots) {
            float* dst = partials + (size_t)slot * PARTIAL;
#pragma unroll
            for (int n = 0; n < 32; ++n) {
                *reinterpret_cast<float2*>(dst + gid * kHeadDim + 8 * n + 2 * tig) = make_float2(o[n][0], o[n][1]);
                *reinterpret_cast<float2*>(dst + (gid + 8) * kHeadDim + 8 * n + 2 * tig) = make_float2(o[n][2], o[n][3]);
            }
            if (tig == 0) {
                dst[kBfRows * kHeadDim + gid] = m_run[0];
                dst[kBfRows * kHeadDim + gid + 8] = m_run[1];
                dst[kBfRows * kHeadDim + kBfRows + gid] = l_run[0];
                dst[kBfRows * kHeadDim + kBfRows + gid + 8] = l_run[1];
            }
        }
        __syncwarp();
        u += n_here;
    }
}

// ---- host side ---------------------------------------------------------------------------------
static bool bf16_layout_ok(const warp34_kv_layer_layout* l) {
    return l != nullptr && l->local_kv_heads > 0 && l->k_base != 0 && l->v_base != 0 &&
           l->k_format == WARP34_KV_FORMAT_BF16 && l->v_format == WARP34_KV_FORMAT_BF16 &&
           l->k_transform == WARP34_KV_TRANSFORM_IDENTITY && l->v_transform == WARP34_KV_TRANSFORM_IDENTITY;
}

static bool bf16_strides_aligned16(const warp34_kv_layer_layout* l) {
    return ((l->k_base | l->v_base | l->k_page_stride_bytes | l->v_page_stride_bytes | l->k_head_stride_bytes |
             l->v_head_stride_bytes | l->k_token_stride_bytes | l->v_token_stride_bytes) & 15u) == 0;
}

static int bf16kv_configure() {
    static bool done[64];
    int dev = 0;
    int rc = (int)cudaGetDevice(&dev);
    if (rc != 0) return rc;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!done[dev]) {
        rc = (int)cudaFuncSetAttribute(bf16kv_attention_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kBfWarps * kBfStages * kBfStageBytes);
        if (rc != 0) return rc;
        done[dev] = true;
    }
    return 0;
}

}  // namespace w34

extern "C" int warp34_kv_cache_write_strided_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                  const warp34_attention_batch* batch, const void* k_in,
                                                  const void* v_in, int row_stride_elems) {
    if (ex == nullptr || !w34::bf16_layout_ok(layout) || batch == nullptr || k_in == nullptr || v_in == nullptr ||
        row_stride_elems < layout->local_kv_heads * layout->head_dim || batch->total_tokens < 0 ||
        batch->num_reqs <= 0 || batch->query_start_loc == nullptr || batch->write_slot_mapping == nullptr) {
        return (int)cudaErrorInvalidValue;
    }
    if (batch->total_tokens == 0) return 0;
    if (layout->head_dim != w34::kHeadDim || layout->block_size != w34::kPageTokens) return (int)cudaErrorNotSupported;
    const int vec16 = w34::bf16_strides_aligned16(layout) && (row_stride_elems % 8) == 0 &&
                      ((((uintptr_t)k_in) | ((uintptr_t)v_in)) & 15u) == 0;
    const long long rows = (long long)batch->total_tokens * layout->local_kv_heads;
    w34::kv_cache_write_bf16_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, (cudaStream_t)ex->stream>>>(
        *layout, *batch, k_in, v_in, row_stride_elems, vec16);
    return (int)cudaGetLastError();
}

extern "C" int warp34_kv_cache_write_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                          const warp34_attention_batch* batch, const void* k_in, const void* v_in) {
    if (!w34::bf16_layout_ok(layout)) return (int)cudaErrorInvalidValue;
    return warp34_kv_cache_write_strided_bf16(ex, layout, batch, k_in, v_in,
                                              layout->local_kv_heads * layout->head_dim);
}

extern "C" size_t warp34_paged_attention_bf16_scratch_bytes(const warp34_kv_layer_layout* layout,
                                                            const warp34_attention_batch* batch, int num_q_heads) {
    if (layout == nullptr || batch == nullptr || num_q_heads <= 0 || layout->local_kv_heads <= 0) return 0;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long slots = (long long)sms * w34::kBfWarps + w34::items_bound(layout, batch, num_q_heads, w34::kBfRows);
    return w34::plan_bytes(batch->num_reqs) +
           (size_t)slots * (size_t)(w34::kBfRows * w34::kHeadDim + 2 * w34::kBfRows) * sizeof(float);
}

extern "C" int warp34_paged_attention_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                           const warp34_attention_batch* batch, const void* q_in, void* attn_out,
                                           int num_q_heads) {
    if (ex == nullptr || !w34::bf16_layout_ok(layout) || batch == nullptr || q_in == nullptr || attn_out == nullptr ||
        num_q_heads <= 0 || num_q_heads % layout->local_kv_heads != 0 || batch->total_tokens < 0 ||
        batch->num_reqs <= 0 || batch->query_start_loc == nullptr || batch->seq_lens_after == nullptr ||
        batch->block_tables == nullptr || batch->max_blocks_per_req <= 0 || batch->sliding_window < 0 ||
        (batch->mask_mode != WARP34_ATTN_MASK_CAUSAL && batch->mask_mode != WARP34_ATTN_MASK_SYMMETRIC_WINDOW)) {
        return (int)cudaErrorInvalidValue;
    }
    if (batch->total_tokens == 0) return 0;
    // Unlike the TQ4 entry point this one has no scratch-free fallback: the caller must pass the
    // split-KV workspace (warp34_paged_attention_bf16_scratch_bytes for the full grid; the
    // persistent grid shrinks to what a smaller workspace holds).
    if (layout->head_dim != w34::kHeadDim || layout->block_size != w34::kPageTokens ||
        !w34::bf16_strides_aligned16(layout) || ex->scratch_ptr == 0 || (ex->scratch_ptr & 15u) != 0) {
        return (int)cudaErrorNotSupported;
    }
    int rc = w34::bf16kv_configure();
    if (rc != 0) return rc;
    int dev = 0, sms = 0;
    rc = (int)cudaGetDevice(&dev);
    if (rc != 0) return rc;
    rc = (int)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (rc != 0) return rc;

    const int gqa = num_q_heads / layout->local_kv_heads;
    const long long items = w34::items_bound(layout, batch, num_q_heads, w34::kBfRows);
    if (items * (long long)batch->max_blocks_per_req >= 0x7fffffffll) return (int)cudaErrorNotSupported;
    const size_t plan = w34::plan_bytes(batch->num_reqs);
    const size_t slot_bytes = (size_t)(w34::kBfRows * w34::kHeadDim + 2 * w34::kBfRows) * sizeof(float);
    const size_t avail = ex->scratch_size > plan ? ex->scratch_size - plan : 0;
    const long long workers = (long long)(avail / slot_bytes) - items;
    if (workers < w34::kBfWarps) return (int)cudaErrorNotSupported;
    int grid = sms;
    if (workers / w34::kBfWarps < grid) grid = (int)(workers / w34::kBfWarps);

    w34::StreamParams p;
    p.og.gate = nullptr;
    p.og.mode = 0;
    p.layout = *layout;
    p.batch = *batch;
    p.q_in = q_in;
    p.attn_out = attn_out;
    p.io_bf16 = 1;
    p.triple_out = nullptr;
    p.scratch = reinterpret_cast<uint8_t*>((uintptr_t)ex->scratch_ptr);
    p.num_q_heads = num_q_heads;
    p.gqa = gqa;
    p.num_warps = grid * w34::kBfWarps;
    p.max_slots = (int)(p.num_warps + items);
    p.rows_per_group = w34::kBfRows;
    p.q_scale = batch->sm_scale * 1.4426950408889634f;
    p.natural = 1;
    p.qfrag = nullptr;
    p.q_groups_max = 0;
    p.smem_bytes = (uint32_t)(w34::kBfWarps * w34::kBfStages * w34::kBfStageBytes);
    cudaStream_t st = (cudaStream_t)ex->stream;
    w34::tq4_attention_plan_kernel<<<1, 32, 0, st>>>(p);
    w34::bf16kv_attention_stream_kernel<<<grid, w34::kBfWarps * 32, p.smem_bytes, st>>>(p);
    const long long rows = (long long)batch->total_tokens * num_q_heads;
    if (rows * 4 < (long long)grid * w34::kBfWarps / 8) {
        w34::tq4_attention_merge_kernel<false, 32><<<(unsigned)rows, 1024, 0, st>>>(p);
    } else {
        w34::tq4_attention_merge_kernel<false, 4><<<(unsigned)rows, 128, 0, st>>>(p);
    }
    return (int)cudaGetLastError();
}
