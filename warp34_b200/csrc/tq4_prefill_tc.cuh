// Chunked-prefill attention over TQ4 pages on the 5th-generation tensor cores (tcgen05 + TMEM).
// Included by tq4_attention.cu (shares the PTX wrappers, geometry helpers and the codebook).
//
// Replaces paged_attention_prefill_mma_f16_kernel<128> (crates/warp34-kernels/csrc/ops/
// op_paged_attn.cu:594-1128) for head_dim 256, 16-token pages, canonical TQ4 packing.
//
// One CTA = 128 query rows (128 / gqa tokens x gqa heads of one KV head) and 14 warps:
//   warps 0-3 (consumers): thread r owns query row r = TMEM lane r.  Per block of 64 keys they
//     read the scores S from TMEM (tcgen05.ld), run the online softmax with a lazily updated
//     reference maximum, write P as fp16 pairs over the scores they came from (tcgen05.st) and,
//     rarely, rescale the output accumulator in TMEM.
//   warps 4-11 (producers): take the code words of a block from the staging buffer into
//     registers (releasing it at once), then dequantise them once per CTA into fp16 tiles in the
//     128-byte-swizzled layout the MMA descriptors expect: lookup of a code byte -> half2 of
//     table centroids, times the row scale, 16-byte stores.  K and V tiles are double-buffered.
//   warp 12: lane 0 issues every tcgen05.mma, the scores of block j + 1 ahead of the output
//     product of block j so that they are computed during the softmax of block j:
//       S[128 x 64]   = Q'[128 x 256] K^T   16 instructions (K = 16), A = Q' in TMEM, B = K tile
//       O[128 x 256] += P[128 x 64] V        4 instructions, A = P in TMEM, B = V tile (MN-major)
//   warp 13: lane 0 bulk-copies the raw (page, head) runs of the next block's four pages
//     (2112 B each for K and for V) into the staging buffer.
// Completion of MMAs is tracked with tcgen05.commit on mbarriers; every wait is bounded and
// warp-uniform, and a wait that gives up raises a flag that ends all loops (no thread is ever
// left at a barrier, and the tensor memory is always freed).
//
// Shared-memory tiles (1024-byte aligned, rows of 128 B = 64 fp16, 16-byte chunk index XOR
// (row & 7)):
//   K  [2][4 dim blocks][64 keys][64]  K-major B operand      2 x 32 KB
//   V  [2][4 dim blocks][64 keys][64]  MN-major B operand     2 x 32 KB  (same physical layout)
// TMEM (512 columns): O in [0, 256), two score buffers in [256, 320) and [320, 384) (fp32, lane =
// query row; the first 32 columns of a buffer are reused for the P of the same block), Q' in
// [384, 512) (two fp16 per column).  Both A operands of the MMAs come from TMEM: with P in shared
// memory the output product competed with the producers for shared-memory bandwidth and ran at
// half rate.
// Scales: every K and V element is table centroid x row scale, the product rounded once
// (scale = hi + lo in fp16, v = fma(e, hi, e * lo)).  (A scale, or P times a scale, rounded to
// fp16 per 128-half puts a different relative error on the two halves of a row; through the
// inverse rotation that difference moves a fraction of channel c ^ 128 into channel c, which is
// visible next to a x20 outlier channel.)  The V scale is dithered per coordinate, see
// kVScaleDither; K needs none (its rounding errors meet a different query value at every coordinate).
#pragma once

namespace w34 {

constexpr int kTcRows = 128;
constexpr int kTcKeys = 64;                      // keys per block = 4 pages
constexpr int kTcProducerWarps = 8;
constexpr int kTcProducers = kTcProducerWarps * 32;
constexpr int kTcWarps = 4 + kTcProducerWarps + 2;   // 4 consumer, 8 producer, 1 MMA-issue, 1 copy-issue warp
constexpr int kTcThreads = kTcWarps * 32;
constexpr uint32_t kTcKvBytes = 4u * kTcKeys * 128u;         // 32768
constexpr uint32_t kTcRawStage = 2u * 4u * kTq4PageHeadBytes;  // K runs then V runs of four pages: 16896
constexpr uint32_t kTcLutBytes = 256u * 128u;                // lane-replicated, 128-byte entry stride
constexpr uint32_t kTcOffK = 0;                               // K is double-buffered
constexpr uint32_t kTcOffQStage = 0;                          // Q' staging (before the first block), 64 KB
constexpr uint32_t kTcOffV = kTcOffK + 2u * kTcKvBytes;
constexpr uint32_t kTcOffRaw = kTcOffV + 2u * kTcKvBytes;    // V is double-buffered
constexpr int kTcRawStages = 1;                  // producers take the code words into registers and release it at once
constexpr uint32_t kTcOffLut = kTcOffRaw + (uint32_t)kTcRawStages * kTcRawStage;
constexpr uint32_t kTcOffBars = kTcOffLut + kTcLutBytes;
// barriers, then (at +128 / +132) the TMEM address and the abort flag
constexpr uint32_t kTcOffRed = kTcOffBars + 144u;                 // 16 ints: per-warp key-range reduction
constexpr uint32_t kTcSmemBytes = kTcOffRed + 64u;
constexpr int kTcStageStride = 257;              // floats per row of the epilogue staging
static_assert(kTcRows * kTcStageStride * 4 <= (int)kTcOffLut, "epilogue staging (over the tiles and the idle staging buffer) must not reach the table");
constexpr uint32_t kTcTmemCols = 512;
constexpr uint32_t kTcColO = 0, kTcColS = 256;   // S: two buffers of 64 columns
constexpr uint32_t kTcColQ = 384;                // Q' as the A operand: 256 fp16 per row = 128 columns
constexpr float kTcRescaleThreshold = 8.0f;      // log2 units: P stays below 2^8

// Dither of the V scale, one half2 per pair of rotated coordinates (128 per row): uniform in
// +-0.5 x 2^-11, fixed.  Rounding centroid x scale to fp16 gives the same error to every
// coordinate that holds the same code; for a row dominated by a few outlier channels the codes
// follow the sign patterns of those channels' Hadamard rows, and the inverse rotation then
// collects that error on the channels whose index is an XOR of outlier channel indices (up to
// 1e-2 there).  Perturbing the scale per coordinate by less than the rounding step makes the
// rounding errors independent of the codes; they then add up incoherently (about 1e-3).
__constant__ uint32_t kVScaleDither[128] = {
    0x86800500u, 0x878f83ccu, 0x8b0a0b6cu, 0x06c7086eu, 0x0b5c881bu, 0x0b0e8945u, 0x071f89b6u, 0x8a800892u,
    0x8731012fu, 0x89e80215u, 0x87d388d6u, 0x093806e6u, 0x09300aebu, 0x06268b99u, 0x01020a1du, 0x046a84aeu,
    0x09988a15u, 0x059c0753u, 0x096f04adu, 0x84978851u, 0x034c04a2u, 0x095f88cbu, 0x00bb80cbu, 0x8473042bu,
    0x80d20039u, 0x0a6505fbu, 0x0aad8b40u, 0x816b0496u, 0x058701b2u, 0x0b340bbfu, 0x0a6c8a79u, 0x005c0b72u,
    0x017b89deu, 0x08928a7du, 0x83930734u, 0x06c384beu, 0x060a81feu, 0x0b200ad2u, 0x0b85830cu, 0x8a4d0a8bu,
    0x83660225u, 0x07660206u, 0x8ba20a9cu, 0x04c583e9u, 0x0af880c0u, 0x05f78642u, 0x887c88d8u, 0x8ad18b86u,
    0x09120910u, 0x8a758b9fu, 0x822f882bu, 0x86250b71u, 0x898288c8u, 0x02618ae5u, 0x03168192u, 0x05de8487u,
    0x8b5a880fu, 0x83a80835u, 0x8b708447u, 0x0a3489a3u, 0x00db0090u, 0x88da0134u, 0x86e48a86u, 0x09c608e6u,
    0x095a8866u, 0x06360ae6u, 0x841081eeu, 0x89868941u, 0x0b148258u, 0x861f0986u, 0x876f0280u, 0x0b6a0506u,
    0x02b08a38u, 0x8ab900b6u, 0x81ea0a2bu, 0x898882b5u, 0x0b30831du, 0x887982d9u, 0x0ae98851u, 0x884009c4u,
    0x8b4304cdu, 0x06390147u, 0x09e38298u, 0x8366888cu, 0x078f8488u, 0x8b4c091du, 0x07248965u, 0x089d814bu,
    0x865c059au, 0x034700d9u, 0x842301aeu, 0x0b27039bu, 0x88fc0a8bu, 0x882901f8u, 0x090f04b7u, 0x03640932u,
    0x0a870a23u, 0x80558889u, 0x83c08862u, 0x81d38a8cu, 0x89b709efu, 0x023089cdu, 0x05378b6au, 0x82df00a9u,
    0x88bd80d4u, 0x02af8a46u, 0x856c89f9u, 0x83af08b8u, 0x08718b8fu, 0x082088bbu, 0x87bd88cbu, 0x870a8001u,
    0x0a478713u, 0x021a817bu, 0x01230300u, 0x84a583beu, 0x87880a9cu, 0x09148713u, 0x073b0786u, 0x82cb0424u,
    0x8a858588u, 0x07d00867u, 0x0bc80b32u, 0x0aba8410u, 0x89d20991u, 0x060f8608u, 0x805e0a3au, 0x8a9f8b2au};

// barrier slots (8 bytes each)
enum { kBarFullK0 = 0, kBarFullK1, kBarFullV0, kBarFullV1, kBarEmptyK0, kBarEmptyK1, kBarEmptyV0, kBarEmptyV1,
       kBarS0, kBarS1, kBarSFree0, kBarSFree1,
       kBarPv, kBarPReady,
       kBarRawFull0, kBarRawFree0 = kBarRawFull0 + kTcRawStages, kBarCount = kBarRawFree0 + kTcRawStages };
static_assert(kBarCount * 8 <= 128, "barrier slots end before the TMEM address slot");

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by one thread.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// Same with the A operand in tensor memory (lane = row, two fp16 per 32-bit column).
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte
// offsets in 16-byte units, descriptor version 1 (bits 46-47), layout type 2 (bits 61-63).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp32 accumulate (bits 4-5 = 1), fp16 A and B (formats 0),
// A K-major, B K-major or MN-major (bit 16), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t tc_idesc(int m, int n, int b_mn_major) {
    return (1u << 4) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct PrefillTcParams {
    warp34_kv_layer_layout layout;
    warp34_attention_batch batch;
    const void* q_in;
    void* attn_out;
    int io_bf16;
    int num_q_heads;
    int gqa;
    int tok_per_tile;      // 128 / gqa
    float q_scale;         // sm_scale * log2(e)
    int32_t* status;       // may be null; bit 2 is set when a wait gave up
    OutputGate og;
};

__global__ void __launch_bounds__(kTcThreads, 1) tq4_attention_prefill_tc_kernel(const PrefillTcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    // The swizzled tiles need a 1024-byte-aligned window; the kernel has no static shared memory,
    // so the dynamic window starts aligned.  If it ever does not, every thread leaves here.
    const uint32_t base = smem_u32(smem_raw);
    if ((base & 1023u) != 0u) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, 8);
        return;
    }
    uint8_t* gen = smem_raw;
    const uint32_t k_t = base + kTcOffK, v_t = base + kTcOffV;
    const uint32_t q_stage = base + kTcOffQStage;
    const uint32_t raw = base + kTcOffRaw, lut = base + kTcOffLut, bars = base + kTcOffBars;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + kTcOffBars + 128);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(gen + kTcOffBars + 132);
    auto bar = [&](int which) { return bars + 8u * (uint32_t)which; };
    // Waits and abort checks are made warp-uniform, so that no lane leaves a loop alone and the
    // warp-collective instructions below always see all 32 lanes.
    auto wait_all = [&](uint32_t b, uint32_t parity) {
        const bool ok = mbar_wait(b, parity);
        return __all_sync(0xffffffffu, ok) != 0;
    };
    auto aborted_any = [&]() { return __any_sync(0xffffffffu, *abort_flag != 0u) != 0; };

    // ---- one-time setup -------------------------------------------------------------------------
    for (int i = tid; i < 256 * 32; i += kTcThreads) {
        const int byte = i >> 5, ln = i & 31;
        // kLutScale x centroid lands close to the fp16 grid for all eight magnitudes; the factor is
        // divided out of the row scale before the fp16 multiply
        sts32(lut + (uint32_t)(byte * 128 + ln * 4),
              pack_half2(kLutScale * tq4_centroid(byte & 15), kLutScale * tq4_centroid(byte >> 4)));
    }
    if (tid == 0) {
        mbar_init(bar(kBarFullK0), (uint32_t)kTcProducers);
        mbar_init(bar(kBarFullK1), (uint32_t)kTcProducers);
        mbar_init(bar(kBarFullV0), (uint32_t)kTcProducers);
        mbar_init(bar(kBarFullV1), (uint32_t)kTcProducers);
        mbar_init(bar(kBarEmptyK0), 1u);
        mbar_init(bar(kBarEmptyK1), 1u);
        mbar_init(bar(kBarEmptyV0), 1u);
        mbar_init(bar(kBarEmptyV1), 1u);
        mbar_init(bar(kBarS0), 1u);
        mbar_init(bar(kBarS1), 1u);
        mbar_init(bar(kBarSFree0), 128u);
        mbar_init(bar(kBarSFree1), 128u);
        mbar_init(bar(kBarPv), 1u);
        mbar_init(bar(kBarPReady), 128u);
        for (int st = 0; st < kTcRawStages; ++st) {
            mbar_init(bar(kBarRawFull0 + st), 1u);
            mbar_init(bar(kBarRawFree0 + st), (uint32_t)kTcProducers);
        }
        *abort_flag = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (wid == 0) {
        tc_alloc(base + kTcOffBars + 128, kTcTmemCols);
        tc_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

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
    ReqGeom g;
    g.q_start = g.q_len = g.ctx_before = g.seq_after = 0;
    g.valid = false;
    if (req >= 0) g = load_req(p.batch, req);
    const bool active = req >= 0 && g.valid;     // uniform over the CTA
    const int tok0 = tile_in_req * tpt;
    const int ntok = active ? min(tpt, g.q_len - tok0) : 0;
    const int rows_used = ntok * p.gqa;

    // every thread evaluates the limits of row (tid & 127); consumers keep them
    const int my_row = tid & 127;
    const int my_qoff = tok0 + my_row / p.gqa;
    const bool row_ok = my_row < rows_used &&
                        (p.batch.valid_token_mask == nullptr || p.batch.valid_token_mask[g.q_start + my_qoff] != 0);
    const int rmax = row_ok ? row_max_kv(p.batch, g, my_qoff) : -1;
    const int rmin = row_ok ? row_min_kv(p.batch, g, my_qoff) : 0x7fffffff;
    int* s_lo = reinterpret_cast<int*>(gen + kTcOffRed);
    int* s_hi = s_lo + 8;
    {
        int lo = rmin, hi = rmax;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, d));
            hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, d));
        }
        if (lane == 0 && wid < 4) { s_lo[wid] = lo; s_hi[wid] = hi; }
    }
    __syncthreads();
    int kv_lo = 0x7fffffff, kv_hi = -1;
#pragma unroll
    for (int w = 0; w < 4; ++w) { kv_lo = min(kv_lo, s_lo[w]); kv_hi = max(kv_hi, s_hi[w]); }
    const bool any_keys = active && kv_hi >= kv_lo;
    const int kb_lo = any_keys ? (kv_lo >> 6) : 0;
    const int nblocks = any_keys ? ((kv_hi >> 6) - kb_lo + 1) : 0;
    const int pg_hi = any_keys ? (kv_hi >> 4) : -1;

    // ---- Q' -> swizzled A tile: one warp per row, natural rotated-column order -------------------
    for (int row = wid; row < kTcRows; row += kTcWarps) {
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
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = lane + 32 * j;                 // rotated column
            // staging row = 512 B; its 16-byte chunks are XOR-swizzled by the row so that the
            // thread-per-row reads below spread over the banks
            const uint32_t addr = q_stage + (uint32_t)row * 512u + (uint32_t)((((c >> 3) ^ (row & 31)) << 4) + ((c & 7) << 1));
            sts16(addr, (uint32_t)__half_as_ushort(__float2half_rn(tv[j] * p.q_scale)));
        }
    }
    __syncthreads();
    // Q' is the A operand of the score product and lives in TMEM: lane = row, 256 fp16 = 128 columns
    if (wid < 4) {
        const uint32_t t_q = tmem + ((uint32_t)(32 * wid) << 16) + kTcColQ;
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {     // 32 columns = 64 fp16 = 8 chunks per step
            uint32_t r[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t chunk = (uint32_t)(8 * c4 + c);
                const uint32_t addr = q_stage + (uint32_t)tid * 512u + ((chunk ^ (uint32_t)(tid & 31)) << 4);
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(r[4 * c]), "=r"(r[4 * c + 1]), "=r"(r[4 * c + 2]), "=r"(r[4 * c + 3]) : "r"(addr));
            }
            tc_st32(t_q + 32u * c4, r);
        }
        tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();      // the staging area becomes the K tiles

    const int32_t* blocks = p.batch.block_tables + (size_t)(req >= 0 ? req : 0) * p.batch.max_blocks_per_req;
    float l_run = 0.0f;

    if (wid == 4 + kTcProducerWarps) {
        // ======================= MMA issue: lane 0 feeds the tensor core ================================
        // Order in the tensor pipe: QK(0), QK(1), PV(0), QK(2), PV(1), ...: the scores of block j + 1
        // are computed while the consumers run the softmax of block j.
        constexpr uint32_t kIdescQk = tc_idesc(kTcRows, kTcKeys, 0);
        constexpr uint32_t kIdescPv = tc_idesc(kTcRows, kHeadDim, 1);
        const uint64_t desc_k = tc_smem_desc(k_t, 16u, 1024u);
        const uint64_t desc_v = tc_smem_desc(v_t, kTcKeys * 128u, 1024u);
#pragma unroll 1
        for (int j = 0; j <= nblocks; ++j) {
            if (aborted_any()) break;
            if (j < nblocks) {
                bool ok = wait_all(bar(kBarFullK0 + (j & 1)), (uint32_t)((j >> 1) & 1));
                // S buffer j & 1 was last read by the softmax of block j - 2
                if (ok && j > 1) ok = wait_all(bar(kBarSFree0 + (j & 1)), (uint32_t)(((j - 2) >> 1) & 1));
                if (!ok) { *abort_flag = 1u; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t d = tmem + kTcColS + 64u * (uint32_t)(j & 1);
#pragma unroll
                    for (int ks = 0; ks < 16; ++ks) {
                        // start-address field is in 16-byte units: dim block ks >> 2, 32 bytes per k-step
                        const uint64_t b = desc_k + (uint64_t)((j & 1) * (kTcKvBytes / 16) + (ks >> 2) * (kTcKeys * 128 / 16) + 2 * (ks & 3));
                        tc_mma_f16_ts(d, tmem + kTcColQ + 8u * (uint32_t)ks, b, kIdescQk, ks ? 1u : 0u);
                    }
                    tc_commit(bar(kBarS0 + (j & 1)));
                    tc_commit(bar(kBarEmptyK0 + (j & 1)));
                }
                __syncwarp();
            }
            if (j > 0) {
                const int i = j - 1;
                bool ok = wait_all(bar(kBarPReady), (uint32_t)(i & 1));
                ok = ok && wait_all(bar(kBarFullV0 + (i & 1)), (uint32_t)((i >> 1) & 1));
                if (!ok) { *abort_flag = 1u; break; }
                tc_fence_after();
                if (lane == 0) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // A = P(i): fp16 pairs the consumers wrote over the first 32 columns of score buffer i & 1
                        const uint64_t b = desc_v + (uint64_t)((i & 1) * (kTcKvBytes / 16) + (2048 / 16) * ks);
                        tc_mma_f16_ts(tmem + kTcColO, tmem + kTcColS + 64u * (uint32_t)(i & 1) + 8u * (uint32_t)ks, b, kIdescPv,
                                      (i > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit(bar(kBarPv));
                    tc_commit(bar(kBarEmptyV0 + (i & 1)));
                }
                __syncwarp();
            }
        }
    } else if (wid == 4 + kTcProducerWarps + 1) {
        // ======================= copy issue: raw (page, head) runs of four pages per block ==============
        const uint8_t* k_head_base = (const uint8_t*)(uintptr_t)p.layout.k_base + (size_t)kv_head * p.layout.k_head_stride_bytes;
        const uint8_t* v_head_base = (const uint8_t*)(uintptr_t)p.layout.v_base + (size_t)kv_head * p.layout.v_head_stride_bytes;
        // page ids of block j, read one block ahead of their use (a global load)
        auto page_ids = [&](int j, int32_t (&ids)[4]) {
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
                const int pg = 4 * (kb_lo + j) + pp;
                ids[pp] = (j < nblocks && pg <= pg_hi) ? block_table_page(blocks, pg, p.batch.max_blocks_per_req, kInPrefillTc) : -1;
            }
        };
        int32_t ids[4];
        page_ids(0, ids);
#pragma unroll 1
        for (int j = 0; j < nblocks; ++j) {
            if (aborted_any()) break;
            // the staging buffer is free once every producer has taken block j - 1 into registers
            if (j > 0 && !wait_all(bar(kBarRawFree0), (uint32_t)((j - 1) & 1))) { *abort_flag = 1u; break; }
            if (lane == 0) {
                const uint32_t fb = bar(kBarRawFull0);
                int npg = 0;
#pragma unroll
                for (int pp = 0; pp < 4; ++pp) npg += (ids[pp] >= 0) ? 1 : 0;
                mbar_expect_tx(fb, (uint32_t)npg * 2u * kTq4PageHeadBytes);
                for (int pp = 0; pp < npg; ++pp) {
                    const int32_t page = ids[pp];
                    bulk_g2s(raw + (uint32_t)pp * kTq4PageHeadBytes,
                             k_head_base + (size_t)page * p.layout.k_page_stride_bytes, kTq4PageHeadBytes, fb);
                    bulk_g2s(raw + (uint32_t)(4 + pp) * kTq4PageHeadBytes,
                             v_head_base + (size_t)page * p.layout.v_page_stride_bytes, kTq4PageHeadBytes, fb);
                }
            }
            __syncwarp();
            page_ids(j + 1, ids);
        }
    } else if (wid >= 4) {
        // ======================= producers: dequantisation ==========================================
        const int tp = tid - 128;                       // 0 .. kTcProducers - 1
        const int key = tp & 63, qd = tp >> 6;       // qd: 64-dim block of the row
        const int half = qd >> 1, sub = qd & 1;
        // one (key, 64-dim block) of K or V: 8 code words -> 8 swizzled 16-byte chunks
        auto load_words = [&](uint32_t rowp, uint32_t (&w)[8], uint32_t& dbits) {
            if (half == 0) {      // codes of half 0 start at byte 2: read 9 words and shift by 16 bits
                uint32_t x[9];
#pragma unroll
                for (int j = 0; j < 9; ++j) x[j] = lds32(rowp + 32u * sub + 4u * j);
                dbits = lds_u16(rowp);
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = __funnelshift_r(x[j], x[j + 1], 16);
            } else {
                dbits = lds_u16(rowp + 66u);
#pragma unroll
                for (int j = 0; j < 8; ++j) w[j] = lds32(rowp + 68u + 32u * sub + 4u * j);
            }
        };
        uint32_t dith[32];          // this thread's 64 coordinates = 32 pairs
#pragma unroll
        for (int i = 0; i < 32; ++i) dith[i] = kVScaleDither[32 * qd + i];
        auto convert = [&](const uint32_t (&w)[8], uint32_t dbits, uint32_t tile, bool key_ok, bool is_v) {
            if (!key_ok) dbits = 0u;      // a key no row can see may hold never-written bytes
            // scale (table factor divided out) = hi + lo in fp16; v = fma(e, hi, e * lo) is the
            // product rounded once (to within 2^-22)
            const float dscaled = __half2float(__ushort_as_half((unsigned short)dbits)) * (1.0f / kLutScale);
            const __half d_hi = __float2half_rn(dscaled);
            const __half2 hi2 = __half2half2(d_hi);
            const __half2 lo2 = __float2half2_rn(dscaled - __half2float(d_hi));
            const uint32_t lut_lane = lut + 4u * (uint32_t)lane;
            const uint32_t dst = tile + (uint32_t)qd * (kTcKeys * 128u) + (uint32_t)key * 128u;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t h[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t e = lds32(lut_lane + (__byte_perm(w[c], 0, 0x4440 + k) << 7));
                    const __half2 e2 = *reinterpret_cast<const __half2*>(&e);
                    // V: the low part of the scale carries the per-coordinate dither
                    const __half2 lo_j = is_v ? __hfma2(hi2, *reinterpret_cast<const __half2*>(&dith[4 * c + k]), lo2) : lo2;
                    const __half2 v = __hfma2(e2, hi2, __hmul2(e2, lo_j));
                    h[k] = *reinterpret_cast<const uint32_t*>(&v);
                }
                sts128(dst + (uint32_t)((c ^ (key & 7)) << 4), h[0], h[1], h[2], h[3]);
            }
        };

#pragma unroll 1
        for (int j = 0; j < nblocks; ++j) {
            if (aborted_any()) break;
            const uint32_t par = (uint32_t)(j & 1);
            if (!wait_all(bar(kBarRawFull0), par)) { *abort_flag = 1u; break; }
            const int pos = ((kb_lo + j) << 6) + key;
            const bool key_ok = pos >= kv_lo && pos <= kv_hi;
            const uint32_t rowp = raw + (uint32_t)key * kTq4RowBytes;
            uint32_t wk[8], wv[8], dk, dv;
            load_words(rowp, wk, dk);
            load_words(rowp + 4u * kTq4PageHeadBytes, wv, dv);
            mbar_arrive(bar(kBarRawFree0));     // the next block's runs can be copied in
            // K buffer j & 1 was last read by the score product of block j - 2
            if (j > 1 && !wait_all(bar(kBarEmptyK0 + (j & 1)), (uint32_t)(((j - 2) >> 1) & 1))) { *abort_flag = 1u; break; }
            convert(wk, dk, k_t + (uint32_t)(j & 1) * kTcKvBytes, key_ok, false);
            fence_proxy_async();
            mbar_arrive(bar(kBarFullK0 + (j & 1)));
            // V buffer j & 1 was last read by the output product of block j - 2
            if (j > 1 && !wait_all(bar(kBarEmptyV0 + (j & 1)), (uint32_t)(((j - 2) >> 1) & 1))) { *abort_flag = 1u; break; }
            convert(wv, dv, v_t + (uint32_t)(j & 1) * kTcKvBytes, key_ok, true);
            fence_proxy_async();
            mbar_arrive(bar(kBarFullV0 + (j & 1)));
        }
    } else {
        // ======================= consumers: MMA issue, softmax, P, rescale =========================
        const uint32_t lane_base = (uint32_t)(32 * wid) << 16;
        const uint32_t t_o = tmem + lane_base + kTcColO, t_s = tmem + lane_base + kTcColS;
        float m_ref = -1e30f;
#pragma unroll 1
        for (int j = 0; j < nblocks; ++j) {
            if (aborted_any()) break;
            const uint32_t par = (uint32_t)(j & 1);
            if (!wait_all(bar(kBarS0 + (j & 1)), (uint32_t)((j >> 1) & 1))) { *abort_flag = 1u; break; }
            tc_fence_after();
            const uint32_t t_sj = t_s + 64u * (uint32_t)(j & 1);
            float sv[64];
            {
                uint32_t r0[32], r1[32];
                tc_ld32(r0, t_sj);
                tc_ld32(r1, t_sj + 32u);
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) { sv[i] = __uint_as_float(r0[i]); sv[32 + i] = __uint_as_float(r1[i]); }
            }
            tc_fence_before();
            mbar_arrive(bar(kBarSFree0 + (j & 1)));      // the scores are in registers
            const int kbase = (kb_lo + j) << 6;
            if (!(kbase >= rmin && kbase + 63 <= rmax)) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int pos = kbase + i;
                    if (!(pos >= rmin && pos <= rmax)) sv[i] = -1e30f;
                }
            }
            float mx4[4] = {sv[0], sv[1], sv[2], sv[3]};     // four independent chains
#pragma unroll
            for (int i = 4; i < 64; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the reference maximum moves only when the true maximum ran ahead by more than the threshold
            const bool need = mx > m_ref + kTcRescaleThreshold;
            float alpha = 1.0f;
            if (need) {
                alpha = ex2(m_ref - mx);      // 0 when nothing was visible before
                m_ref = mx;
            }
            // P(j - 1) and O are in use until the previous output product has completed
            if (j > 0 && !wait_all(bar(kBarPv), par ^ 1u)) { *abort_flag = 1u; break; }
            tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                for (int c = 0; c < 8; ++c) {
                    uint32_t o[32];
                    tc_ld32(o, t_o + 32u * c);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tc_st32(t_o + 32u * c, o);
                }
                tc_wait_st();
            }
            float ls4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const float m_use = (m_ref < -1e29f) ? 0.0f : m_ref;     // nothing visible yet: every P is 0
            // P as fp16 pairs goes where its own scores were: the first 32 columns of this score buffer
            // (A operand of the output product, lane = row, key 2 i in the low half of column i)
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                // masked scores are -1e30: ex2 gives exactly 0 against any finite reference
                const float pa = ex2(sv[2 * i] - m_use), pb = ex2(sv[2 * i + 1] - m_use);
                ls4[i & 3] += pa + pb;
                pk[i] = pack_half2(pa, pb);
            }
            tc_st32(t_sj, pk);
            tc_wait_st();
            l_run = l_run * alpha + ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3]));
            tc_fence_before();
            mbar_arrive(bar(kBarPReady));
        }
        // the last output product
        if (nblocks > 0 && !aborted_any()) {
            if (!wait_all(bar(kBarPv), (uint32_t)((nblocks - 1) & 1))) *abort_flag = 1u;
        }
        tc_fence_after();
    }

    // ---- epilogue: O / l -> staging -> inverse rotation -> global ---------------------------------
    // (staging aliases the Q / K / V tiles: every MMA that read them has completed)
    __syncthreads();
    const bool aborted = *abort_flag != 0u;
    float* stage = reinterpret_cast<float*>(gen);
    if (wid < 4 && nblocks > 0 && !aborted) {
        const uint32_t t_o = tmem + ((uint32_t)(32 * wid) << 16) + kTcColO;
        const float inv = (l_run > 0.0f) ? (1.0f / l_run) : 0.0f;
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
            uint32_t o[32];
            tc_ld32(o, t_o + 32u * c);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) stage[tid * kTcStageStride + 32 * c + i] = __uint_as_float(o[i]) * inv;
        }
        stage[tid * kTcStageStride + 256] = l_run;
    }
    tc_fence_before();
    __syncthreads();
    if (wid == 0) {
        tc_fence_after();
        tc_dealloc(tmem, kTcTmemCols);
    }
    if (aborted) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, 4);
        return;
    }
    if (!active) return;
    for (int row = wid; row < rows_used; row += kTcWarps) {
        const int q_off = tok0 + row / p.gqa;
        const int q_head = kv_head * p.gqa + row % p.gqa;
        if (p.batch.valid_token_mask != nullptr && p.batch.valid_token_mask[g.q_start + q_off] == 0) continue;
        float tv[8];
        const bool has = nblocks > 0 && stage[row * kTcStageStride + 256] > 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) tv[j] = has ? stage[row * kTcStageStride + lane + 32 * j] : 0.0f;
        wht256_lanes(tv, lane);
        const size_t out_base = ((size_t)(g.q_start + q_off) * p.num_q_heads + q_head) * kHeadDim;
        store_output_row(p.attn_out, out_base, tv, lane, p.io_bf16, p.og);
    }
}

}  // namespace w34
