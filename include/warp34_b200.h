/*
 * warp34_b200 -- C ABI of the B200 (sm_100a) TQ4 paged-KV hot path.
 *
 * The three descriptor structs, the enums and the first group of entry points
 * are binary-compatible with the reference project's FFI seam
 * (crates/warp34-kernels/csrc/warp34_cuda.h:11-101 and :353-373, mirrored in
 * crates/warp34-kernels/src/ffi.rs), so a host built against that seam can
 * load this library in place of the reference kernels for the KV-cache write
 * and paged-attention calls.  Every pointer is borrowed; no call allocates,
 * frees or synchronises with the host unless its comment says otherwise; all
 * work is enqueued on `ex->stream`; the caller has already made the target
 * device current.  Return value: 0 on success, otherwise a cudaError_t value
 * (cudaErrorInvalidValue = 1 for ill-formed arguments,
 * cudaErrorNotSupported = 801 for a combination this library does not
 * implement).
 */
#ifndef WARP34_B200_H
#define WARP34_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums (reference: warp34_cuda.h:20-48) -------------------------------- */
enum {
    WARP34_KV_NAMESPACE_TARGET_FULL_ATTN = 0,
    WARP34_KV_NAMESPACE_MTP_FULL_ATTN    = 1,
    WARP34_KV_NAMESPACE_DFLASH_DRAFT_CTX = 2,
};
enum {
    WARP34_KV_FORMAT_FP16     = 0,
    WARP34_KV_FORMAT_BF16     = 1,
    WARP34_KV_FORMAT_TQ4      = 2,
    WARP34_KV_FORMAT_Q8_0     = 3,
    WARP34_KV_FORMAT_FP8_E4M3 = 4,
};
enum {
    WARP34_KV_TRANSFORM_IDENTITY          = 0,
    WARP34_KV_TRANSFORM_RADEMACHER_WHT256 = 1,
};
enum {
    WARP34_ATTN_MASK_CAUSAL           = 0,
    WARP34_ATTN_MASK_SYMMETRIC_WINDOW = 1,
    WARP34_ATTN_MASK_NONCAUSAL_WINDOW = 1,
};

/* warp34_exec.flags.  Bit 0 is the reference's WARP34_EXEC_FLAG_ALLOW_W4A8_PREFILL
 * (warp34_cuda.h:46-48), ignored here.  The high bit below is additive: it makes
 * warp34_paged_attention_f16 take the fp32 dequant-then-attend kernel (no fp16 tensor-core
 * operands, no scratch) for callers that want scores at fp32 accuracy. */
#define WARP34_EXEC_FLAG_ALLOW_W4A8_PREFILL (1ull << 0)
#define WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION (1ull << 40)
/* Additive: multi-token verify batches (more than 8 query rows per request and KV head) take the
 * tcgen05 kernel, one 128-row CTA per request and KV head, instead of the split-KV team kernel. */
#define WARP34_B200_EXEC_FLAG_TCGEN05_VERIFY (1ull << 42)
/* Additive: the tensor-core kernels feed every operand as one fp16 value, as the reference's own
 * tensor-core kernel does (op_paged_attn.cu:357, :47-50, :470).  Faster; a softmax weight is then
 * off by a few 1e-4 relative, so an output channel in which large values of V cancel can miss
 * 2e-3 + 1e-2 |b| against dequant-then-attend.  Without the flag the kernels carry the rounding
 * residuals of Q', of the K centroids and of P through extra products and meet that bound. */
#define WARP34_B200_EXEC_FLAG_FAST_ATTENTION (1ull << 43)

/* ---- descriptors (reference: warp34_cuda.h:50-101) -------------------------- */
typedef struct {
    uintptr_t stream;       /* cudaStream_t */
    uint64_t  scratch_ptr;  /* device workspace, 16-byte aligned */
    size_t    scratch_size; /* bytes */
    uint64_t  flags;
} warp34_exec;

typedef struct {
    uint64_t k_base;
    uint64_t v_base;
    uint64_t k_page_stride_bytes;
    uint64_t k_head_stride_bytes;
    uint64_t k_token_stride_bytes;
    uint64_t v_page_stride_bytes;
    uint64_t v_head_stride_bytes;
    uint64_t v_token_stride_bytes;
    int32_t  namespace_id;
    int32_t  layer_id;
    int32_t  local_kv_heads;
    int32_t  head_dim;
    int32_t  block_size;
    int32_t  k_format;
    int32_t  v_format;
    int32_t  k_transform;
    int32_t  v_transform;
    int32_t  reserved;
} warp34_kv_layer_layout;

typedef struct {
    const int32_t* query_start_loc;     /* [num_reqs + 1]  device */
    const int32_t* context_lens_before; /* [num_reqs]      device, may be NULL */
    const int32_t* seq_lens_after;      /* [num_reqs]      device */
    const int32_t* block_tables;        /* [num_reqs, max_blocks_per_req] device */
    const int32_t* write_slot_mapping;  /* [total_tokens]  device: page*16 + offset, < 0 = skip */
    const uint8_t* valid_token_mask;    /* [total_tokens]  device, may be NULL */
    const uint8_t* valid_req_mask;      /* [num_reqs]      device, may be NULL */
    int32_t        num_reqs;
    int32_t        total_tokens;
    int32_t        max_blocks_per_req;
    int32_t        max_q_len;
    int32_t        max_seq_len;
    int32_t        mask_mode;
    int32_t        sliding_window;
    float          sm_scale;
    int32_t        reserved;
} warp34_attention_batch;

#if defined(__cplusplus)
static_assert(sizeof(warp34_exec) == 32, "warp34_exec ABI size");
static_assert(sizeof(warp34_kv_layer_layout) == 104, "warp34_kv_layer_layout ABI size");
static_assert(sizeof(warp34_attention_batch) == 96, "warp34_attention_batch ABI size");
#else
_Static_assert(sizeof(warp34_exec) == 32, "warp34_exec ABI size");
_Static_assert(sizeof(warp34_kv_layer_layout) == 104, "warp34_kv_layer_layout ABI size");
_Static_assert(sizeof(warp34_attention_batch) == 96, "warp34_attention_batch ABI size");
#endif

/* ======================================================================== *
 * 1. Drop-in entry points (same names, argument meaning and error behaviour
 *    as the reference).
 * ======================================================================== */

/*
 * Quantize-and-append: encodes one fp16 K row and one fp16 V row of 256
 * values per (token, kv head) into the paged pool at
 * write_slot_mapping[token].  Replaces warp34_kv_cache_write
 * (warp34_cuda.h:354-356, op_kv_cache.cu:852-858); k_in / v_in are
 * [total_tokens, local_kv_heads * head_dim] contiguous.
 *
 * Layer formats covered at head_dim 256, 16-token pages: TQ4 rows with the sign-diagonal +
 * WHT-256 rotation (132 B), and the unrotated 8-bit rows of the boundary layers,
 * WARP34_KV_FORMAT_Q8_0 (272 B: 4 x { float d; int8 qs[64] }) and WARP34_KV_FORMAT_FP8_E4M3
 * (264 B: uint8 qs[256], float d0, d1), K and V each in either 8-bit format
 * (op_kv_cache.cu:32-151; cache.rs:62-108 pairs them with the identity transform only).  Rows of
 * the 8-bit formats must be 4-byte aligned.  Anything else returns cudaErrorNotSupported (801).
 * warp34_paged_attention_f16 and warp34_paged_attention_scalar_f16 read the same layers.
 */
int warp34_kv_cache_write(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                          const warp34_attention_batch* batch,
                          const void* k_in, const void* v_in);

/*
 * Same with an explicit row stride (in elements) for K and V, so K and V can
 * be slices of a packed QKV activation.  Replaces
 * warp34_kv_cache_write_strided (warp34_cuda.h:357-360,
 * op_kv_cache.cu:828-850).  Strides below local_kv_heads * head_dim are
 * rejected with cudaErrorInvalidValue; an empty batch returns 0 without a
 * launch.  Tokens with valid_token_mask == 0, requests with
 * valid_req_mask == 0 and slots < 0 have no side effects.
 */
int warp34_kv_cache_write_strided(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                  const warp34_attention_batch* batch,
                                  const void* k_in, const void* v_in,
                                  int k_row_stride, int v_row_stride);

/*
 * The layer's K producer fused in front of the append (additive): per-head Gemma RMS norm
 * (weight 1 + w) and partial interleaved 3-D mRoPE of the K rows, then the TQ4 rotate /
 * quantise / pack / scale-write, in one kernel; V rows are appended as they are.  Replaces,
 * for the K and V half of the layer, the pair
 *   warp34_fused_qk_rmsnorm_rope_gate_strided_f16   (warp34_cuda.h:264-287, op_norms_rope_act.cu:524-680)
 *   warp34_kv_cache_write_strided                   (warp34_cuda.h:357-360)
 * at the reference's call site crates/warp34-host/src/model/forward.rs:1109-1149, and saves the
 * round trip of the fp16 K rows through HBM (the reference has such a fused kernel for another
 * KV family only: warp34_dflash_qk_norm_rope_kv_write_bf16_f32_table, warp34_cuda.h:625-628).
 * The Q half of the producer stays the caller's (the reference kernel with num_kv_heads = 0).
 * k_in / v_in are row slices of the packed QKV activation (strides in elements), k_norm_w is
 * fp16 [256], positions is int32 [3 planes][pos_plane_stride]; the remaining arguments are
 * those of the reference's producer.  The packed bytes equal those of the two-kernel sequence.
 * TQ4 layers, fp16 activations, rotary_dim a multiple of 16 (cudaErrorNotSupported otherwise).
 */
int warp34_fused_k_rmsnorm_rope_kv_cache_write_f16(
    const warp34_exec* ex, const warp34_kv_layer_layout* layout, const warp34_attention_batch* batch,
    const void* k_in, const void* v_in, const void* k_norm_w, const int32_t* positions, int pos_plane_stride,
    int rotary_dim, int mrope_s0, int mrope_s1, int mrope_s2, int k_row_stride, int v_row_stride,
    float rope_theta, float rms_eps);

/*
 * Paged attention over the pool: q_in and attn_out are fp16
 * [total_tokens, num_q_heads, head_dim].  Replaces warp34_paged_attention_f16
 * (warp34_cuda.h:370-373, op_paged_attn.cu:1266-1448).  Split-KV partials
 * live in ex->scratch_ptr; warp34_paged_attention_scratch_bytes() says how
 * much a batch geometry can use.  Any 16-byte-aligned scratch is accepted.  Less
 * than that bound means fewer, longer KV partitions.  A batch needs the plan, one
 * partial slot (8.1 KiB) and one set of query fragments (6.25 KiB) per (request,
 * kv head, 8-row group) and one slot per worker warp; when the scratch leaves
 * fewer worker slots than half a grid, the requests are served in several passes
 * over the same scratch (8 MiB, the reference engine's minimum: two passes for a
 * decode batch of 64 sequences x 4 kv heads, 0.88 ms instead of 0.51 ms with
 * 17.5 MB; eight passes for 256 sequences).  Only a scratch too small for one
 * request and one thread block's workers (about 100 KiB) leaves the fp32 kernel,
 * which needs none.
 * Masked rows of attn_out are left untouched.
 *
 * Accuracy: every output is within 2e-3 + 1e-2 |b| of fp32 dequant-then-attend (b).  The
 * tensor-core kernels get there by feeding each fp16 operand as value + rounding residual;
 * measured against float64 this holds with margin from K, V ~ N(0, 1) with x20 outlier channels
 * and Q ~ N(0, 1) up to twice as many outlier channels, x30 (K) and x60 (V) outliers and a query
 * scale of 2 (V outlier channels that alternate in sign from key to key: up to magnitude 60).  For
 * activations far beyond that (x60 outliers in 32 channels and a query scale of
 * 3: a few outputs per million miss the bound by up to 3.6x) WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION
 * selects the fp32 kernel, which stays below a seventh of the bound on all of these.
 * WARP34_B200_EXEC_FLAG_FAST_ATTENTION trades the residual operands for speed.  Kernels: decode and verify batches
 * (up to 24 query rows per request and kv head) stream split-KV work items of 8 rows; larger
 * chunks take a 128-row prefill kernel (register MMAs; tcgen05 + TMEM with the fast flag).
 * 8-bit boundary layers (Q8_0, FP8 E4M3) in the canonical packing stream the same way on a
 * tensor-core kernel whose operands are exact (codes convert exactly to fp16); other packings of
 * them, callers without scratch and WARP34_B200_EXEC_FLAG_PRECISE_ATTENTION take an fp32 kernel.
 */
int warp34_paged_attention_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                               const warp34_attention_batch* batch,
                               const void* q_in, void* attn_out,
                               int num_q_heads);

/*
 * The literal dequant-then-attend kernel (four warps per query row, fp32
 * throughout, no scratch).  Replaces warp34_paged_attention_scalar_f16
 * (op_kv_cache.cu:1244), which the reference keeps as its fallback and test
 * selector; accepts any strides in the layout.
 */
int warp34_paged_attention_scalar_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                      const warp34_attention_batch* batch,
                                      const void* q_in, void* attn_out,
                                      int num_q_heads);

/*
 * Test-only kernel selector.  Replaces warp34_paged_attention_f16_force_kernel_for_test
 * (op_paged_attn.cu:1451-1458), against which the reference's variant-equality tests link
 * (crates/warp34-host/src/cuda/tests.rs:111-576).  use_64q: 0 = the reference's 16-row kernel,
 * here the 8-row split-KV items; 1 = its 64-row prefill kernel, here the 128-row register-MMA
 * prefill kernel; 2 = its 128-row prefill kernel, here the 128-row tcgen05 kernel.  The
 * reference's three variants share their arithmetic and are compared at 0 ULP; these do not:
 * selectors 0 and 1 meet 2e-3 + 1e-2 |b| against dequant-then-attend on every element,
 * selector 2 computes with single fp16 operands (see WARP34_B200_EXEC_FLAG_FAST_ATTENTION).
 * TQ4 layers in the canonical packing only (cudaErrorNotSupported otherwise).
 */
int warp34_paged_attention_f16_force_kernel_for_test(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                                     const warp34_attention_batch* batch,
                                                     const void* q_in, void* attn_out,
                                                     int num_q_heads, int use_64q);

/*
 * Paged attention with the layer's output epilogue folded into the kernels' final store: the
 * sigmoid output gate and, with hadamard64 != 0, the 64-point Hadamard (x 1/8) over every 64
 * columns that pre-rotates the input of an offline-rotated o_proj.  Additive: replaces the pair
 * warp34_paged_attention_f16 + warp34_apply_attn_output_gate(_hadamard)_f16 of the reference's
 * layer (crates/warp34-host/src/model/forward.rs:1181-1211) and saves the round trip of the
 * attention output through HBM.  gate and out are fp16 [total_tokens, num_q_heads, 256]; out may
 * not alias q_in.  Rounding follows the two-kernel sequence (attention output to fp16, gated value
 * to fp16 before the Hadamard); masked rows of out are left untouched.  TQ4 layers apply the
 * epilogue inside the merge / prefill kernels, 8-bit layers in a second launch in place.
 */
int warp34_paged_attention_gated_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                     const warp34_attention_batch* batch,
                                     const void* q_in, const void* gate, void* out,
                                     int num_q_heads, int hadamard64);

/*
 * The epilogue's two steps on their own.  Replace warp34_apply_attn_output_gate_f16
 * (warp34_cuda.h:297-300, op_norms_rope_act.cu:742-764, :1329-1345) and
 * warp34_apply_attn_output_gate_hadamard_f16 (warp34_cuda.h:945-947,
 * op_norms_rope_act.cu:805-851, :2032-2056): out = fp16(attn_out * sigmoid(gate)), the second
 * followed by the Hadamard-64; rows with valid_token_mask == 0 are skipped; out may alias
 * attn_out.  total_dim must be a multiple of 64 for the Hadamard variant.  The sigmoid is
 * ex2.approx and rcp.approx, as the reference's -use_fast_math build lowers it: the results are
 * the reference kernels' bit for bit.
 */
int warp34_apply_attn_output_gate_f16(const warp34_exec* ex, const void* attn_out, const void* gate, void* out,
                                      const uint8_t* valid_token_mask, int num_tokens, int total_dim);
int warp34_apply_attn_output_gate_hadamard_f16(const warp34_exec* ex, const void* attn_out, const void* gate,
                                               void* out, const uint8_t* valid_token_mask, int num_tokens,
                                               int total_dim);

/*
 * Uncompressed BF16 KV storage with identity transforms (the comparison arm of the TQ4 path).
 * Replace warp34_kv_cache_write_bf16 / warp34_kv_cache_write_strided_bf16 /
 * warp34_paged_attention_bf16 (warp34_cuda.h:363-368; op_kv_cache.cu:1170-1241) for
 * {BF16, BF16, IDENTITY, IDENTITY} descriptors with head_dim 256 and 16-token pages; other
 * head sizes return cudaErrorNotSupported, descriptors of another format cudaErrorInvalidValue
 * as in the reference (op_kv_cache.cu:860-865).  K / V / Q / output are bf16.  The append copies
 * rows bit for bit (row_stride_elems >= heads * 256 lets packed [K, V] or [Q, K, V]
 * activations be written without a column copy).  The attention call streams pages through
 * the split-KV path and, unlike the reference's, needs ex->scratch_ptr
 * (warp34_paged_attention_bf16_scratch_bytes for the full grid, less shrinks the grid) and
 * 16-byte-aligned strides; without them it returns cudaErrorNotSupported.
 */
int warp34_kv_cache_write_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                               const warp34_attention_batch* batch,
                               const void* k_in, const void* v_in);
int warp34_kv_cache_write_strided_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                       const warp34_attention_batch* batch,
                                       const void* k_in, const void* v_in, int row_stride_elems);
int warp34_paged_attention_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                const warp34_attention_batch* batch,
                                const void* q_in, void* attn_out, int num_q_heads);

/* ======================================================================== *
 * 2. Additive entry points (no reference symbol changes meaning).
 * ======================================================================== */

/*
 * Upper bound of the scratch the split-KV path can use for a batch geometry
 * (only host-known fields of `batch` are read).  The reference sizes the same
 * buffer inline (op_paged_attn.cu:1301-1338).
 */
size_t warp34_paged_attention_scratch_bytes(const warp34_kv_layer_layout* layout,
                                            const warp34_attention_batch* batch,
                                            int num_q_heads);

/* The same bound for warp34_paged_attention_bf16 (16 query rows per work item). */
size_t warp34_paged_attention_bf16_scratch_bytes(const warp34_kv_layer_layout* layout,
                                                 const warp34_attention_batch* batch,
                                                 int num_q_heads);

/*
 * bf16 activations over TQ4 pages.  The reference's TQ4 path takes fp16 activations only (its
 * bf16 entry points, warp34_cuda.h:363-368, require BF16 *storage*: op_kv_cache.cu:860-865);
 * these two take bf16 K / V (append) and bf16 Q / output (attention) with the same descriptors.
 * Values representable in both types produce the same packed bytes as the fp16 entry points.
 */
int warp34_tq4_kv_cache_write_strided_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                           const warp34_attention_batch* batch,
                                           const void* k_in, const void* v_in,
                                           int k_row_stride, int v_row_stride);
int warp34_tq4_paged_attention_bf16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                    const warp34_attention_batch* batch,
                                    const void* q_in, void* attn_out, int num_q_heads);

/*
 * Attention over a page shard of longer sequences: same arguments as
 * warp34_paged_attention_f16, but the result is left un-normalised so that shards held by
 * different GPUs can be merged.  triples_out is fp32 [total_tokens, num_q_heads, 258]: 256
 * accumulator values in the rotated domain, then the running maximum m (base-2 logarithm
 * units of the scaled scores) and the sum l.  Needs the streaming path (canonical layout and
 * scratch); returns cudaErrorNotSupported otherwise.  The reference has no multi-GPU
 * attention; the triple is the (acc, m, l) of its split-KV scratch (op_paged_attn.cu:1329-1338).
 */
int warp34_paged_attention_partial_f16(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                                       const warp34_attention_batch* batch,
                                       const void* q_in, float* triples_out, int num_q_heads);

/*
 * Merges num_shards sets of triples ([num_shards, num_rows, 258], e.g. the all-gather of every
 * GPU's warp34_paged_attention_partial_f16 output) into fp16 attention output
 * [num_rows, 256]: w_s = 2^(m_s - max m), out = sum acc_s w_s / sum l_s w_s, inverse rotation
 * (the algebra of op_paged_attn.cu:1168-1202).  Shards with l <= 0 are skipped.
 */
int warp34_paged_attention_merge_shards_f16(const warp34_exec* ex, const float* triples,
                                            int num_shards, int64_t num_rows, void* attn_out);

/*
 * Page-sharded attention without a library collective: the exchange of the (acc, m, l) triples and
 * their merge in ONE kernel over peer-mapped memory (NVLink).  Every rank owns a mailbox that all
 * ranks have mapped (CUDA IPC / symmetric memory; the caller does the mapping):
 *
 *   inbox  float    [2][world][max_rows][258]   parity of the step, source rank, row
 *   flags  uint32_t [world][max_rows]           step number of the last triple that arrived
 *
 * and, private to the rank, steps uint32_t [max_rows] (the number of steps this rank has run).  All
 * three start as zeros.  A call makes one warp per row: it stores its own triple row into every
 * peer's inbox[step & 1][rank][row], publishes the step number in the peer's flags[rank][row] with
 * a system-scope release, waits (acquire, bounded) for every peer's flag of this row to reach the
 * step, merges the world triples exactly as warp34_paged_attention_merge_shards_f16 does (shards in
 * rank order, so every rank computes bit-identical output) and writes fp16 [num_rows, 256].
 * Every rank must make the same sequence of calls with the same num_rows.  The step number lives
 * in device memory, so a captured CUDA graph can be replayed.  A wait that runs out (wait_limit
 * polls of about 0.25 us; 0 = about one second) ORs 1 into *status (device memory, may be null),
 * leaves the row's output untouched and still counts the step, so later steps stay aligned.
 * No counterpart in the reference, which has no multi-GPU attention.
 */
#define WARP34_B200_MAX_PEERS 8
typedef struct warp34_peer_mailboxes {
    int32_t world;                             /* 1..8 */
    int32_t rank;
    int64_t max_rows;
    uint64_t inbox[WARP34_B200_MAX_PEERS];     /* rank w's inbox as mapped in THIS process */
    uint64_t flags[WARP34_B200_MAX_PEERS];     /* rank w's flags as mapped in THIS process */
    uint64_t steps;                            /* this rank's private step counters */
    uint64_t status;                           /* int32_t in device memory, or 0 */
    uint32_t wait_limit;
    uint32_t reserved;
} warp34_peer_mailboxes;

int warp34_paged_attention_exchange_merge_f16(const warp34_exec* ex, const warp34_peer_mailboxes* boxes,
                                              const float* triples, int64_t num_rows, void* attn_out);

/*
 * Copies the first `rows` token rows (all kv heads, K and V) of page src_page to page dst_page
 * of one layer: the device half of copy-on-write for a shared partial tail page
 * (docs/contracts/cache-layout.md:106-110 specifies the copy; the reference never implemented
 * it).  Pair with w34_seq_prepare_append() of warp34_host.h.
 */
int warp34_kv_page_copy(const warp34_exec* ex, const warp34_kv_layer_layout* layout,
                        int32_t src_page, int32_t dst_page, int32_t rows);

/*
 * warp34_paged_attention_f16 for callers that have no workspace to offer and may not allocate
 * one.  This entry point has no counterpart in the reference, whose engine always passes an
 * 8 MiB scratch arena in warp34_exec.  It exists for hosts where that is not possible: the
 * process has already committed all the device memory it was allowed (KV pool, weights) before
 * this library is reached, the caller is a plugin that receives only tensors and a stream, or
 * allocator calls are banned on the serving path.  The split-KV workspace is a 16 MiB array
 * built into the library image (each GPU that loads the library holds it until the process
 * exits); nothing is allocated or freed by this call, by the CUDA runtime on its behalf, or by
 * any other library.
 *
 *  - Same inputs, outputs, masks and result as warp34_paged_attention_f16; `stream` replaces
 *    the warp34_exec.
 *  - Limit: the batch must fit the built-in workspace: the plan, 8256-byte partials (one per
 *    group of 8 query rows and one more per request, for every kv head, plus 8) and 6.25 KiB of
 *    query fragments per group; about 730 (request, kv head) pairs of a decode batch, e.g. 182
 *    requests at 4 kv heads, is the ceiling.  A
 *    prefill chunk (more than 24 query rows per request and kv head) uses only the status word,
 *    whatever its size.  Larger batches are refused with cudaErrorInvalidValue and nothing is
 *    launched; when `scratch_needed` is not NULL it receives the bytes the batch would have
 *    needed, so the caller can tell "too large" from a malformed argument.
 *  - TQ4 layers in the canonical 132-byte-row packing only: other packings and the 8-bit
 *    boundary layers (Q8_0, FP8 E4M3), which warp34_paged_attention_f16 serves, are refused
 *    here with cudaErrorNotSupported (801).
 *  - The status word that warp34_paged_attention_f16 leaves at the start of the caller's
 *    scratch sits in the built-in array; warp34_static_scratch_status() reads it.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and configures the kernel's shared
 *    memory; make that first call outside any stream capture.
 *  - All calls on a device share the one array, and it keeps whatever the previous call left.
 *    Every call rewrites the plan and each partial before reading it, so no clearing is needed,
 *    but two calls whose kernels overlap on the GPU (different streams without an event
 *    between them) race on it.  Serialise them.
 */
int warp34_paged_attention_f16_static_scratch(uintptr_t stream, const warp34_kv_layer_layout* layout,
                                              const warp34_attention_batch* batch,
                                              const void* q_in, void* attn_out, int num_q_heads,
                                              size_t* scratch_needed);

/*
 * Status word of the last warp34_paged_attention_f16_static_scratch call on the current device
 * (no counterpart in the reference): 0 = ok; bit 0 = a bounded wait inside a kernel gave up (the
 * output is void); bit 1 = the shared-memory window could not hold the kernel's layout; bit 2 =
 * a request had more query tokens than batch->max_q_len declared and its extra rows were
 * dropped.  A blocking 4-byte copy from the built-in array: it waits for the work queued before
 * it, so call it where a synchronisation is acceptable, never inside a stream capture.
 * Allocates nothing.
 */
int warp34_static_scratch_status(int32_t* status_out);

/*
 * Query-sparse paged attention: every token attends only to its list of selected 4-token groups.
 * Replaces warp34_qsa_sparse_paged_attn_f16 / _hadamard_f16 (warp34_cuda.h, QSA section;
 * crates/warp34-kernels/csrc/ops/op_qsa.cu:716-1572, entry points :1711-1752) with the same
 * signatures and semantics:
 *   q, gate, out            fp16 [num_tokens, local_q_heads, 256]; gate may be NULL
 *   selected_phys_blocks    [num_tokens, select_k_blocks] physical group ids (page * 4 + group in page;
 *                           negative = skip), selected_logical_blocks their logical group indices: key
 *                           (entry, off) sits at position 4 * logical + off and takes part iff that is
 *                           <= token_seq_pos[token]; only the first num_selected_blocks[token] entries are read
 *   valid_token_mask        may be NULL; a masked token's output rows are written as zeros
 * The sigmoid gate multiplies the fp32 result; the _hadamard variant then rounds to fp16 and applies the
 * normalised 64-point Hadamard to every 64 columns.  Layers: head_dim 256, 16-token pages, K and V each
 * TQ4 with the Rademacher + WHT-256 rotation or Q8_0 / FP8 E4M3 unrotated, any strides; FP16 rows, which
 * the reference's kernel also reads, are refused with cudaErrorNotSupported like everywhere else here.
 * An fp32 dequant-then-attend kernel; ex->scratch_ptr, when set, lets it split a token's list over several
 * blocks (num_tokens * local_q_heads * 1032 bytes per split).
 */
int warp34_qsa_sparse_paged_attn_f16(const warp34_exec* ex, const void* q, const void* gate,
                                     const warp34_kv_layer_layout* kv_layout, const int32_t* selected_phys_blocks,
                                     const int32_t* selected_logical_blocks, const int32_t* num_selected_blocks,
                                     const int32_t* token_seq_pos, const uint8_t* valid_token_mask, void* out,
                                     int num_tokens, int local_q_heads, int select_k_blocks, float sm_scale);
int warp34_qsa_sparse_paged_attn_hadamard_f16(const warp34_exec* ex, const void* q, const void* gate,
                                              const warp34_kv_layer_layout* kv_layout,
                                              const int32_t* selected_phys_blocks,
                                              const int32_t* selected_logical_blocks,
                                              const int32_t* num_selected_blocks, const int32_t* token_seq_pos,
                                              const uint8_t* valid_token_mask, void* out, int num_tokens,
                                              int local_q_heads, int select_k_blocks, float sm_scale);

/*
 * Bounds-checked build (stand-in for the reference's sanitizer runs of this path,
 * tools/check_cuda_sanitizer.py:77-102).  A library compiled with -DW34_BOUNDS
 * (`python -m warp34_b200.build --bounds` -> libwarp34_b200_bounds.so) range-checks, in every kernel,
 * each index into a block table against batch->max_blocks_per_req, each page id read from one and each
 * write slot against the pool's page count, before an address is formed.  The layer descriptor does
 * not carry that count, so the host states it once per device with warp34_bounds_set_pool_pages()
 * (0 = unknown: only block-table indices are checked).  A violating access goes to entry 0 / page 0
 * (reads) or is skipped (writes); nothing traps.  warp34_bounds_report() fills
 *   out4[0] = what | where << 8   what: 1 block-table index, 2 page id, 3 write slot; 0 = no violation
 *                                 where: 1 append, 2 fp32 attention, 3 decode stream, 4 verify team,
 *                                        5 / 6 prefill kernels, 7 bf16 KV, 8 8-bit KV
 *   out4[1] = the offending value, out4[2] = its limit     (of the first violation seen)
 *   out4[3] = number of violations since the last reset
 * and clears the record when `reset` is non-zero.  Both calls are blocking copies.  In the regular
 * build both return cudaErrorNotSupported (801) and the checks cost nothing.
 */
int warp34_bounds_set_pool_pages(int32_t num_pages);
int warp34_bounds_report(int32_t* out4, int32_t reset);

/* Library identification: returns a static string "warp34_b200 <version> sm_100a". */
const char* warp34_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* WARP34_B200_H */
