/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's TQ4 KV path.
 *
 * Nothing in the product links, loads or calls this file.  It exists so that
 * tests, the smoke check and the benchmark's cpu_baseline leg have a
 * hardware-independent statement of what the reference computes:
 *
 *   - w34o_kv_cache_write      follows kv_cache_write_kernel / write_kv_row
 *                              (crates/warp34-kernels/csrc/ops/op_kv_cache.cu:152-218, :325-368)
 *   - w34o_wht256              follows wht256_warp
 *                              (crates/warp34-kernels/csrc/tq/tq4_kv_common.cuh:75-107)
 *   - butterfly_sum            follows warp_reduce_sum (tq4_kv_common.cuh:54-60)
 *   - w34o_paged_attention_f16 follows the scalar dequant-then-attend kernel
 *                              paged_attention_kernel<__half>
 *                              (op_kv_cache.cu:373-461, :619-792)
 *   - tables                   tq4_codebook.cuh:46-101 (via ../warp34_b200/csrc/tq4_tables.h)
 *   - w34o_kv8_encode_row / _decode_row and the 8-bit branches of the two entry points follow the
 *                              Q8_0 / FP8 E4M3 rows of the unrotated boundary layers
 *                              (op_kv_cache.cu:32-151, op_paged_attn.cu:59-105); pinned on the GPU against the
 *                              bytes the reference's kernels write, and here against a second, independent
 *                              restatement (oracle/kv8.py)
 *
 * Parity status: the reference has no byte-level golden vectors for TQ4 and no
 * CPU implementation; this restatement is pinned against outputs of the
 * reference's own kernels (built unmodified by oracle/build_ref.sh and run on
 * a B200), stored under tests/golden/.  The GPU build of the reference uses
 * rsqrt.approx and an approximate division (-use_fast_math); this file uses
 * IEEE arithmetic and reports, per element, whether an approximation error of
 * a few ulp could change the 4-bit code ("ambiguous"), so comparisons can be
 * exact everywhere else.
 *
 * All pointers are HOST pointers, including layout->k_base / v_base.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/warp34_b200.h"
#include "../warp34_b200/csrc/tq4_tables.h"

static const uint32_t kCentroidBits[16] = W34_TQ4_CENTROID_BITS;
static const uint32_t kBoundaryBits[15] = W34_TQ4_BOUNDARY_BITS;
static const uint32_t kSignMask[8] = W34_TQ4_SIGN_MASK;

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }
static inline float centroid(int i) { return bits_f32(kCentroidBits[i]); }
static inline float boundary(int i) { return bits_f32(kBoundaryBits[i]); }
static inline float sign_of(int col) { return ((kSignMask[col >> 5] >> (col & 31)) & 1u) ? -1.0f : 1.0f; }

/* ---- fp16 <-> fp32, round to nearest even ---------------------------------- */
float w34o_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        out = sign | 0x7f800000u | (man << 13);
    } else {
        out = sign | ((exp + 112u) << 23) | (man << 13);
    }
    return bits_f32(out);
}

uint16_t w34o_float_to_half(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t abs = x & 0x7fffffffu;
    if (abs >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((abs > 0x7f800000u) ? 0x200u : 0));
    if (abs >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);            /* rounds to inf */
    if (abs < 0x33000001u) return (uint16_t)sign;                        /* rounds to zero */
    int e = (int)(abs >> 23) - 127;
    uint32_t man = (abs & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }                    /* subnormal half */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x7fffffu; }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));
}

/* ---- warp emulation --------------------------------------------------------- */
/* xor-butterfly all-reduce over 32 lanes, offsets 16,8,4,2,1; every lane ends
 * with the same bits because fp32 addition is commutative.                    */
static float butterfly_sum(const float in[32]) {
    float a[32], b[32];
    memcpy(a, in, sizeof(a));
    for (int off = 16; off > 0; off >>= 1) {
        for (int l = 0; l < 32; ++l) b[l] = a[l] + a[l ^ off];
        memcpy(a, b, sizeof(a));
    }
    return a[0];
}

/* 256-point normalised Walsh-Hadamard transform, stage order h = 1,2,...,128,
 * each stage (lower + upper, lower - upper), final scale 1/16.               */
void w34o_wht256(float v[256]) {
    for (int h = 1; h < 256; h <<= 1) {
        for (int c = 0; c < 256; ++c) {
            if (c & h) continue;
            float a = v[c], b = v[c | h];
            v[c] = a + b;
            v[c | h] = a - b;
        }
    }
    for (int c = 0; c < 256; ++c) v[c] *= 0.0625f;
}

static inline int bucketise(float rv) {
    int q = 0;
    for (int i = 0; i < 15; ++i) q += (rv > boundary(i)) ? 1 : 0;
    return q;
}

/*
 * Encodes one 256-value fp16 row into a 132-byte TQ4 row
 * ({fp16 d0; u8 qs0[64]; fp16 d1; u8 qs1[64]}).  If `ambiguous` is non-NULL
 * it receives, per rotated coordinate, 1 when a relative error of 2^-21 in the
 * normalisation factor would change the code.  Returns the rotated fp32 row in
 * `rot` when non-NULL.
 */
void w34o_tq4_encode_row(const uint16_t* x, uint8_t* out, uint8_t* ambiguous, float* rot) {
    float v[256];
    for (int c = 0; c < 256; ++c) v[c] = w34o_half_to_float(x[c]) * sign_of(c);
    w34o_wht256(v);
    if (rot) memcpy(rot, v, sizeof(v));

    float s_sq[2] = {0.0f, 0.0f};
    for (int j = 0; j < 8; ++j) {
        float p[32];
        for (int l = 0; l < 32; ++l) p[l] = v[32 * j + l] * v[32 * j + l];
        s_sq[j >> 2] += butterfly_sum(p);
    }
    float inv[2];
    for (int b = 0; b < 2; ++b) {
        inv[b] = (s_sq[b] > 1e-20f) ? (0.7071067811865475f * (float)(1.0 / sqrt((double)s_sq[b]))) : 0.0f;
    }
    float vc_dot[2] = {0.0f, 0.0f}, c_sq[2] = {0.0f, 0.0f};
    uint8_t code[256];
    for (int j = 0; j < 8; ++j) {
        float pv[32], pc[32];
        const float in = inv[j >> 2];
        for (int l = 0; l < 32; ++l) {
            const int col = 32 * j + l;
            const float raw = v[col];
            const float rv = raw * in;
            const int q = bucketise(rv);
            code[col] = (uint8_t)q;
            if (ambiguous) {
                const float lo = raw * (in * (1.0f - 4.8e-7f));
                const float hi = raw * (in * (1.0f + 4.8e-7f));
                ambiguous[col] = (bucketise(lo) != q || bucketise(hi) != q) ? 1 : 0;
            }
            const float c = centroid(q);
            pv[l] = raw * c;
            pc[l] = c * c;
        }
        vc_dot[j >> 2] += butterfly_sum(pv);
        c_sq[j >> 2] += butterfly_sum(pc);
    }
    for (int b = 0; b < 2; ++b) {
        const float d = (c_sq[b] > 1e-10f) ? (vc_dot[b] / c_sq[b]) : 0.0f;
        const uint16_t dh = w34o_float_to_half(d);
        uint8_t* blk = out + 66 * b;
        memcpy(blk, &dh, 2);
        for (int i = 0; i < 64; ++i) {
            blk[2 + i] = (uint8_t)(code[128 * b + 2 * i] | (code[128 * b + 2 * i + 1] << 4));
        }
    }
}

/* Dequantises a 132-byte TQ4 row into 256 fp32 values in the rotated domain
 * (op_kv_cache.cu:298-306).                                                    */
void w34o_tq4_decode_row(const uint8_t* row, float* out) {
    for (int b = 0; b < 2; ++b) {
        uint16_t dh;
        memcpy(&dh, row + 66 * b, 2);
        const float d = w34o_half_to_float(dh);
        for (int i = 0; i < 64; ++i) {
            const uint8_t p = row[66 * b + 2 + i];
            out[128 * b + 2 * i] = d * centroid(p & 15);
            out[128 * b + 2 * i + 1] = d * centroid(p >> 4);
        }
    }
}

/* ---- request lookup shared by both entry points ------------------------------ */
/* ---- unrotated 8-bit rows (Q8_0, FP8 E4M3) ----------------------------------------
 * Row definitions: crates/warp34-kernels/csrc/tq/tq4_kv_common.cuh:29-46; encode:
 * ops/op_kv_cache.cu:32-151 (identity transform); decode to fp16: ops/op_paged_attn.cu:59-105. */
static float e4m3_to_float(uint8_t v) {
    const int e = (v >> 3) & 15, m = v & 7;
    float a;
    if (e == 0) a = ldexpf((float)m, -9);
    else if (e == 15 && m == 7) a = NAN;
    else a = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (v & 0x80) ? -a : a;
}

/* round to nearest even, saturating at +-448, NaN -> 0x7F (the satfinite conversion) */
static uint8_t float_to_e4m3(float x) {
    if (x != x) return 0x7F;
    const uint8_t sign = signbit(x) ? 0x80 : 0;
    float a = fabsf(x);
    if (a > 448.0f) a = 448.0f;
    if (a == 0.0f) return sign;
    int e;
    (void)frexpf(a, &e);      /* a = f * 2^e, f in [0.5, 1) */
    e -= 1;                   /* floor(log2 a) */
    if (e < -6) e = -6;       /* subnormal range shares the smallest normal's step */
    float q = nearbyintf(ldexpf(a, 3 - e));   /* in units of 2^(e-3): 8..16 normal, 0..8 subnormal */
    if (q >= 16.0f) { q = 8.0f; e += 1; }
    const int r = (int)q;
    if (r < 8) return (uint8_t)(sign | r);                       /* exponent field 0 */
    return (uint8_t)(sign | ((e + 7) << 3) | (r - 8));
}

void w34o_kv8_encode_row(const uint16_t* x, int format, uint8_t* out) {
    float v[256];
    for (int i = 0; i < 256; ++i) v[i] = w34o_half_to_float(x[i]);
    if (format == WARP34_KV_FORMAT_Q8_0) {
        for (int sb = 0; sb < 4; ++sb) {
            float amax = 0.0f;
            for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(v[64 * sb + i]));
            const float d = amax / 127.0f;
            const float inv = (d > 1e-12f) ? (1.0f / d) : 0.0f;
            memcpy(out + 68 * sb, &d, 4);
            for (int i = 0; i < 64; ++i) {
                float q = roundf(v[64 * sb + i] * inv);
                q = fminf(127.0f, fmaxf(-127.0f, q));
                out[68 * sb + 4 + i] = (uint8_t)(int8_t)q;
            }
        }
        return;
    }
    for (int h = 0; h < 2; ++h) {
        float amax = 0.0f;
        for (int i = 0; i < 128; ++i) amax = fmaxf(amax, fabsf(v[128 * h + i]));
        const float d = amax * (1.0f / 448.0f);
        const float inv = (d > 1e-30f) ? (1.0f / d) : 0.0f;
        memcpy(out + 256 + 4 * h, &d, 4);
        for (int i = 0; i < 128; ++i) out[128 * h + i] = float_to_e4m3(v[128 * h + i] * inv);
    }
}

/* Values as the reference's readers hand them to the tensor cores: d * code, rounded to fp16. */
void w34o_kv8_decode_row(const uint8_t* row, int format, float* out) {
    if (format == WARP34_KV_FORMAT_Q8_0) {
        for (int sb = 0; sb < 4; ++sb) {
            float d;
            memcpy(&d, row + 68 * sb, 4);
            for (int i = 0; i < 64; ++i) {
                out[64 * sb + i] = w34o_half_to_float(w34o_float_to_half(d * (float)(int8_t)row[68 * sb + 4 + i]));
            }
        }
        return;
    }
    float d[2];
    memcpy(d, row + 256, 8);
    for (int i = 0; i < 256; ++i) {
        out[i] = w34o_half_to_float(w34o_float_to_half(e4m3_to_float(row[i]) * d[i >> 7]));
    }
}

static int is_kv8(const warp34_kv_layer_layout* l) {
    const int k8 = l->k_format == WARP34_KV_FORMAT_Q8_0 || l->k_format == WARP34_KV_FORMAT_FP8_E4M3;
    const int v8 = l->v_format == WARP34_KV_FORMAT_Q8_0 || l->v_format == WARP34_KV_FORMAT_FP8_E4M3;
    return k8 && v8 && l->head_dim == 256 && l->k_transform == WARP34_KV_TRANSFORM_IDENTITY &&
           l->v_transform == WARP34_KV_TRANSFORM_IDENTITY;
}

static int find_req(const warp34_attention_batch* b, int tok, int* q_start, int* q_end) {
    for (int r = 0; r < b->num_reqs; ++r) {
        const int lo = b->query_start_loc[r], hi = b->query_start_loc[r + 1];
        if (tok >= lo && tok < hi) { *q_start = lo; *q_end = hi; return r; }
    }
    return -1;
}

/* ---- threading helper -------------------------------------------------------- */
typedef struct {
    void (*fn)(void*, long);
    void* ctx;
    long begin, end;
} w34o_span;

static void* span_main(void* p) {
    w34o_span* s = (w34o_span*)p;
    for (long i = s->begin; i < s->end; ++i) s->fn(s->ctx, i);
    return NULL;
}

static void parallel_for(long n, int nthreads, void (*fn)(void*, long), void* ctx) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 256) nthreads = 256;
    if (n < nthreads) nthreads = (int)(n > 0 ? n : 1);
    if (nthreads == 1) {
        for (long i = 0; i < n; ++i) fn(ctx, i);
        return;
    }
    pthread_t th[256];
    w34o_span sp[256];
    for (int t = 0; t < nthreads; ++t) {
        sp[t].fn = fn; sp[t].ctx = ctx;
        sp[t].begin = n * t / nthreads; sp[t].end = n * (t + 1) / nthreads;
        pthread_create(&th[t], NULL, span_main, &sp[t]);
    }
    for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
}

/* ---- append ------------------------------------------------------------------- */
typedef struct {
    const warp34_kv_layer_layout* l;
    const warp34_attention_batch* b;
    const uint16_t* k; const uint16_t* v;
    int ks, vs;
} write_ctx;

static void write_one(void* p, long idx) {
    write_ctx* c = (write_ctx*)p;
    const warp34_kv_layer_layout* l = c->l;
    const warp34_attention_batch* b = c->b;
    const int heads = l->local_kv_heads;
    const int tok = (int)(idx / heads), head = (int)(idx % heads);
    if (b->valid_token_mask && b->valid_token_mask[tok] == 0) return;
    if (b->valid_req_mask && b->query_start_loc && b->num_reqs > 0) {
        int qs, qe;
        const int r = find_req(b, tok, &qs, &qe);
        if (r < 0 || b->valid_req_mask[r] == 0) return;
    }
    const int32_t slot = b->write_slot_mapping[tok];
    if (slot < 0) return;
    const int page = slot / l->block_size, off = slot % l->block_size;
    uint8_t* kd = (uint8_t*)(uintptr_t)l->k_base + (size_t)page * l->k_page_stride_bytes +
                  (size_t)head * l->k_head_stride_bytes + (size_t)off * l->k_token_stride_bytes;
    uint8_t* vd = (uint8_t*)(uintptr_t)l->v_base + (size_t)page * l->v_page_stride_bytes +
                  (size_t)head * l->v_head_stride_bytes + (size_t)off * l->v_token_stride_bytes;
    if (is_kv8(l)) {
        w34o_kv8_encode_row(c->k + (size_t)tok * c->ks + (size_t)head * 256, l->k_format, kd);
        w34o_kv8_encode_row(c->v + (size_t)tok * c->vs + (size_t)head * 256, l->v_format, vd);
        return;
    }
    w34o_tq4_encode_row(c->k + (size_t)tok * c->ks + (size_t)head * 256, kd, NULL, NULL);
    w34o_tq4_encode_row(c->v + (size_t)tok * c->vs + (size_t)head * 256, vd, NULL, NULL);
}

/* Returns 0, or 1 (cudaErrorInvalidValue) / 801 (not supported) like the GPU entry point. */
int w34o_kv_cache_write_strided(const warp34_kv_layer_layout* l, const warp34_attention_batch* b,
                                const uint16_t* k_in, const uint16_t* v_in,
                                int k_row_stride, int v_row_stride, int nthreads) {
    if (!l || !b || !k_in || !v_in) return 1;
    if (b->total_tokens <= 0 || l->local_kv_heads <= 0) return 0;
    if (!is_kv8(l) &&
        (l->head_dim != 256 || l->k_format != WARP34_KV_FORMAT_TQ4 || l->v_format != WARP34_KV_FORMAT_TQ4 ||
         l->k_transform != WARP34_KV_TRANSFORM_RADEMACHER_WHT256 ||
         l->v_transform != WARP34_KV_TRANSFORM_RADEMACHER_WHT256)) return 801;
    const int min_stride = l->local_kv_heads * l->head_dim;
    if (k_row_stride < min_stride || v_row_stride < min_stride) return 1;
    write_ctx c = {l, b, k_in, v_in, k_row_stride, v_row_stride};
    parallel_for((long)b->total_tokens * l->local_kv_heads, nthreads, write_one, &c);
    return 0;
}

/* ---- dequant-then-attend -------------------------------------------------------- */
typedef struct {
    const warp34_kv_layer_layout* l;
    const warp34_attention_batch* b;
    const uint16_t* q; uint16_t* out;
    int hq;
    float* triples;  /* when non-NULL: write (acc[256], m, l) per row instead of the output */
} attn_ctx;

static void attn_one(void* p, long idx) {
    attn_ctx* c = (attn_ctx*)p;
    const warp34_kv_layer_layout* l = c->l;
    const warp34_attention_batch* b = c->b;
    const int hq = c->hq;
    const int tok = (int)(idx / hq), q_head = (int)(idx % hq);
    if (b->valid_token_mask && b->valid_token_mask[tok] == 0) return;
    int q_start = 0, q_end = 0;
    const int req = find_req(b, tok, &q_start, &q_end);
    if (req < 0) return;
    if (b->valid_req_mask && b->valid_req_mask[req] == 0) return;
    const int gqa = hq / l->local_kv_heads;
    const int kv_head = q_head / gqa;
    const int q_off = tok - q_start;
    const int ctx_before = b->context_lens_before ? b->context_lens_before[req]
                                                  : (b->seq_lens_after[req] - (q_end - q_start));
    const int seq_after = b->seq_lens_after[req];
    int max_kv = (b->mask_mode == WARP34_ATTN_MASK_SYMMETRIC_WINDOW) ? (seq_after - 1) : (ctx_before + q_off);
    if (max_kv >= seq_after) max_kv = seq_after - 1;
    int min_kv = 0;
    if (b->sliding_window > 0) {
        const int win_start = ctx_before + q_off - b->sliding_window + 1;
        if (win_start > min_kv) min_kv = win_start;
    }
    const uint16_t* q_row = c->q + ((size_t)tok * hq + q_head) * 256;
    uint16_t* out_row = c->out + ((size_t)tok * hq + q_head) * 256;

    if (is_kv8(l)) {
        /* unrotated rows: plain dequant-then-attend, one stream, fp32 with an online softmax */
        if (c->triples) return;
        float q[256], kx[256], vx[256], o[256];
        for (int i = 0; i < 256; ++i) { q[i] = w34o_half_to_float(q_row[i]); o[i] = 0.0f; }
        const int32_t* bl = b->block_tables + (size_t)req * b->max_blocks_per_req;
        float m_i = -3.402823466e+38f, l_i = 0.0f;
        for (int pos = min_kv; pos <= max_kv; ++pos) {
            const int page = bl[pos / l->block_size], off = pos % l->block_size;
            const uint8_t* kp = (const uint8_t*)(uintptr_t)l->k_base + (size_t)page * l->k_page_stride_bytes +
                                (size_t)kv_head * l->k_head_stride_bytes + (size_t)off * l->k_token_stride_bytes;
            const uint8_t* vp = (const uint8_t*)(uintptr_t)l->v_base + (size_t)page * l->v_page_stride_bytes +
                                (size_t)kv_head * l->v_head_stride_bytes + (size_t)off * l->v_token_stride_bytes;
            w34o_kv8_decode_row(kp, l->k_format, kx);
            w34o_kv8_decode_row(vp, l->v_format, vx);
            double dot = 0.0;
            for (int i = 0; i < 256; ++i) dot += (double)q[i] * kx[i];
            const float score = (float)dot * b->sm_scale;
            const float m_new = fmaxf(m_i, score);
            const float alpha = expf(m_i - m_new), pr = expf(score - m_new);
            l_i = l_i * alpha + pr;
            m_i = m_new;
            for (int i = 0; i < 256; ++i) o[i] = o[i] * alpha + pr * vx[i];
        }
        const float inv = (l_i > 0.0f) ? (1.0f / l_i) : 0.0f;
        for (int i = 0; i < 256; ++i) out_row[i] = w34o_float_to_half(o[i] * inv);
        return;
    }
    float qr[256];
    for (int i = 0; i < 256; ++i) qr[i] = w34o_half_to_float(q_row[i]) * sign_of(i);
    w34o_wht256(qr);

    /* Four interleaved streams (the reference's four warps take key positions
     * min_kv + w, +4, +8, ...), each with its own online softmax, merged at the end. */
    float m_w[4], l_w[4];
    static _Thread_local float acc[4][256];
    const int32_t* blocks = b->block_tables + (size_t)req * b->max_blocks_per_req;
    for (int w = 0; w < 4; ++w) {
        float m_i = -3.402823466e+38f, l_i = 0.0f;
        float* a = acc[w];
        for (int i = 0; i < 256; ++i) a[i] = 0.0f;
        for (int pos = min_kv + w; pos <= max_kv; pos += 4) {
            const int page = blocks[pos / l->block_size], off = pos % l->block_size;
            const uint8_t* kp = (const uint8_t*)(uintptr_t)l->k_base + (size_t)page * l->k_page_stride_bytes +
                                (size_t)kv_head * l->k_head_stride_bytes + (size_t)off * l->k_token_stride_bytes;
            const uint8_t* vp = (const uint8_t*)(uintptr_t)l->v_base + (size_t)page * l->v_page_stride_bytes +
                                (size_t)kv_head * l->v_head_stride_bytes + (size_t)off * l->v_token_stride_bytes;
            uint16_t dh0, dh1;
            memcpy(&dh0, kp, 2); memcpy(&dh1, kp + 66, 2);
            const float d0 = w34o_half_to_float(dh0), d1 = w34o_half_to_float(dh1);
            /* per-lane partial dots over col = lane + 32 j, then butterfly over lanes */
            float part[32];
            for (int lane = 0; lane < 32; ++lane) {
                float dot0 = 0.0f, dot1 = 0.0f;
                for (int j = 0; j < 4; ++j) {
                    const int col = lane + 32 * j;
                    const uint8_t p0 = kp[2 + (col >> 1)], p1 = kp[68 + (col >> 1)];
                    const int n0 = (col & 1) ? (p0 >> 4) : (p0 & 15);
                    const int n1 = (col & 1) ? (p1 >> 4) : (p1 & 15);
                    dot0 += qr[col] * centroid(n0);
                    dot1 += qr[col + 128] * centroid(n1);
                }
                part[lane] = d0 * dot0 + d1 * dot1;
            }
            const float score = butterfly_sum(part) * b->sm_scale;
            const float m_new = fmaxf(m_i, score);
            const float alpha = expf(m_i - m_new);
            const float pr = expf(score - m_new);
            l_i = l_i * alpha + pr;
            m_i = m_new;
            memcpy(&dh0, vp, 2); memcpy(&dh1, vp + 66, 2);
            const float pd0 = pr * w34o_half_to_float(dh0), pd1 = pr * w34o_half_to_float(dh1);
            for (int i = 0; i < 64; ++i) {
                const uint8_t p0 = vp[2 + i], p1 = vp[68 + i];
                a[2 * i] = a[2 * i] * alpha + pd0 * centroid(p0 & 15);
                a[2 * i + 1] = a[2 * i + 1] * alpha + pd0 * centroid(p0 >> 4);
                a[128 + 2 * i] = a[128 + 2 * i] * alpha + pd1 * centroid(p1 & 15);
                a[128 + 2 * i + 1] = a[128 + 2 * i + 1] * alpha + pd1 * centroid(p1 >> 4);
            }
        }
        m_w[w] = m_i; l_w[w] = l_i;
    }
    float m_tot = -3.402823466e+38f;
    for (int w = 0; w < 4; ++w) if (l_w[w] > 0.0f) m_tot = fmaxf(m_tot, m_w[w]);
    float l_tot = 0.0f, ws[4];
    for (int w = 0; w < 4; ++w) {
        if (l_w[w] > 0.0f) { ws[w] = expf(m_w[w] - m_tot); l_tot += l_w[w] * ws[w]; }
        else ws[w] = 0.0f;
    }
    if (c->triples) {
        /* un-normalised, still rotated: what a page shard hands to the cross-shard merge
         * (the partial layout of op_paged_attn.cu:1329-1338, m in natural-log units here) */
        float* t = c->triples + ((size_t)tok * hq + q_head) * 258;
        for (int i = 0; i < 256; ++i) {
            t[i] = acc[0][i] * ws[0] + acc[1][i] * ws[1] + acc[2][i] * ws[2] + acc[3][i] * ws[3];
        }
        t[256] = m_tot;
        t[257] = l_tot;
        return;
    }
    const float inv_l = (l_tot > 0.0f) ? (1.0f / l_tot) : 0.0f;
    float o[256];
    for (int i = 0; i < 256; ++i) {
        const float s = acc[0][i] * ws[0] + acc[1][i] * ws[1] + acc[2][i] * ws[2] + acc[3][i] * ws[3];
        o[i] = s * inv_l;
    }
    w34o_wht256(o);
    for (int i = 0; i < 256; ++i) out_row[i] = w34o_float_to_half(o[i] * sign_of(i));
}

int w34o_paged_attention_f16(const warp34_kv_layer_layout* l, const warp34_attention_batch* b,
                             const uint16_t* q_in, uint16_t* attn_out, int num_q_heads, int nthreads) {
    if (!l || !b || !q_in || !attn_out) return 1;
    if (b->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (!is_kv8(l) &&
        (l->head_dim != 256 || l->k_format != WARP34_KV_FORMAT_TQ4 || l->v_format != WARP34_KV_FORMAT_TQ4 ||
         l->k_transform != WARP34_KV_TRANSFORM_RADEMACHER_WHT256 ||
         l->v_transform != WARP34_KV_TRANSFORM_RADEMACHER_WHT256)) return 801;
    if (l->local_kv_heads <= 0 || num_q_heads % l->local_kv_heads) return 1;
    attn_ctx c = {l, b, q_in, attn_out, num_q_heads, NULL};
    parallel_for((long)b->total_tokens * num_q_heads, nthreads, attn_one, &c);
    return 0;
}

/* Attention over a page shard, stopped before normalisation: triples is fp32
 * [total_tokens, num_q_heads, 258] = 256 rotated accumulator values, m, l. */
int w34o_paged_attention_partial(const warp34_kv_layer_layout* l, const warp34_attention_batch* b,
                                 const uint16_t* q_in, float* triples, int num_q_heads, int nthreads) {
    if (!l || !b || !q_in || !triples) return 1;
    if (b->total_tokens <= 0 || num_q_heads <= 0) return 0;
    if (l->local_kv_heads <= 0 || num_q_heads % l->local_kv_heads) return 1;
    if (is_kv8(l)) return 801;   /* page-sharded partials exist for TQ4 layers only */
    attn_ctx c = {l, b, q_in, NULL, num_q_heads, triples};
    parallel_for((long)b->total_tokens * num_q_heads, nthreads, attn_one, &c);
    return 0;
}

/* Cross-shard merge (algebra of op_paged_attn.cu:1168-1202): triples is
 * [num_shards, rows, 258]; out is fp16 [rows, 256]. */
int w34o_merge_shards(const float* triples, int num_shards, long rows, uint16_t* out) {
    if (!triples || !out || num_shards <= 0 || rows < 0) return 1;
    for (long r = 0; r < rows; ++r) {
        float m_tot = -3.402823466e+38f;
        for (int s = 0; s < num_shards; ++s) {
            const float* t = triples + ((size_t)s * rows + r) * 258;
            if (t[257] > 0.0f) m_tot = fmaxf(m_tot, t[256]);
        }
        float o[256], l_tot = 0.0f;
        for (int i = 0; i < 256; ++i) o[i] = 0.0f;
        for (int s = 0; s < num_shards; ++s) {
            const float* t = triples + ((size_t)s * rows + r) * 258;
            if (t[257] > 0.0f) {
                const float w = expf(t[256] - m_tot);
                l_tot += t[257] * w;
                for (int i = 0; i < 256; ++i) o[i] += t[i] * w;
            }
        }
        const float inv_l = (l_tot > 0.0f) ? (1.0f / l_tot) : 0.0f;
        for (int i = 0; i < 256; ++i) o[i] *= inv_l;
        w34o_wht256(o);
        for (int i = 0; i < 256; ++i) out[r * 256 + i] = w34o_float_to_half(o[i] * sign_of(i));
    }
    return 0;
}

/* Table accessors for tests. */
float w34o_centroid(int i) { return centroid(i); }
float w34o_boundary(int i) { return boundary(i); }
float w34o_sign(int i) { return sign_of(i); }
