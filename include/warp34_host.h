/*
 * warp34_host -- C ABI of the host-side KV page manager that feeds the kernels of
 * warp34_b200.h: page allocator and free list, reference-counted prefix-shared pages with
 * copy-on-write of a shared partial tail page, block-table / slot-map builders and rollback
 * of rejected speculative tokens.
 *
 * The reference keeps this state in Rust (crates/warp34-host/src/cache.rs, radix.rs,
 * model/graph_io.rs, model/execution.rs).  No Rust toolchain exists in this build
 * environment, so the same semantics are implemented in C++ behind a C ABI that a Rust
 * `extern "C"` block (or any other FFI) can bind.  No function here touches the GPU; page ids
 * are logical and are never multiplied by a byte size outside the layout helper
 * (docs/contracts/cache-layout.md:5-10).
 *
 * Error convention: functions returning int32_t return >= 0 on success and a negative
 * W34_ERR_* code on failure; nothing aborts.
 */
#ifndef WARP34_HOST_H
#define WARP34_HOST_H

#include <stddef.h>
#include <stdint.h>

#include "warp34_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

enum {
    W34_OK = 0,
    W34_ERR_INVALID = -1,      /* bad argument */
    W34_ERR_EXHAUSTED = -2,    /* pool has too few free pages; state unchanged */
    W34_ERR_PROTECTED = -3,    /* would free or overwrite a shared / protected page */
    W34_ERR_CAPACITY = -4,     /* output buffer too small */
};

/* KvFormatPolicy (cache.rs:27-45) */
enum {
    W34_KV_POLICY_FP16 = 0,
    W34_KV_POLICY_BF16 = 1,
    W34_KV_POLICY_Q8_0 = 2,
    W34_KV_POLICY_FP8 = 3,
    W34_KV_POLICY_TQ4 = 4,      /* last 4 full-attention layers 8-bit, the rest TQ4 */
    W34_KV_POLICY_TQ4_ALL = 5,
};

/* Row bytes of one head in a format; kv_format_row_bytes (cache.rs:156-165). */
int32_t w34_kv_format_row_bytes(int32_t format, int32_t head_dim);

/* (k_format, v_format, k_transform, v_transform) of one layer;
 * KvFormatPolicy::resolve_layer_with_fp8 (cache.rs:56-113). */
int32_t w34_kv_policy_resolve_layer(int32_t policy, int32_t layer_ordinal, int32_t num_layers,
                                    int32_t supports_fp8, int32_t out_formats[4]);

/* KvFormatPolicy::bytes_per_token_with_fp8 (cache.rs:126-143). */
int64_t w34_kv_policy_bytes_per_token(int32_t policy, int32_t num_layers, int32_t kv_heads,
                                      int32_t head_dim, int32_t supports_fp8);

/* Fills a layer descriptor with the pool's canonical strides (token = row bytes,
 * head = block_size * token, page = heads * head); KvPool::new (cache.rs:296-334).
 * Returns the bytes one slab (K or V) needs for num_pages via out_k_bytes / out_v_bytes. */
int32_t w34_kv_layout_init(warp34_kv_layer_layout* layout, uint64_t k_base, uint64_t v_base,
                           int32_t namespace_id, int32_t layer_id, int32_t local_kv_heads,
                           int32_t head_dim, int32_t block_size, const int32_t formats[4],
                           int64_t num_pages, uint64_t* out_k_bytes, uint64_t* out_v_bytes);

/* ---- page pool: PageBitmap + KvPool page API (cache.rs:185-265, :385-416) ------------------ */
typedef struct w34_page_pool w34_page_pool;

w34_page_pool* w34_pool_create(int32_t num_pages, int32_t block_size);
void w34_pool_destroy(w34_page_pool* pool);
int32_t w34_pool_num_pages(const w34_page_pool* pool);
int32_t w34_pool_block_size(const w34_page_pool* pool);
int32_t w34_pool_free_count(const w34_page_pool* pool);
/* Lowest free page id (ascending order), or W34_ERR_EXHAUSTED.  The page gets refcount 1. */
int32_t w34_pool_alloc_page(w34_page_pool* pool);
/* Drops one reference; the page returns to the free list at zero.  Negative, out-of-range
 * and already-free ids are ignored (idempotent free, cache.rs:247-265).  Returns the
 * remaining reference count. */
int32_t w34_pool_free_page(w34_page_pool* pool, int32_t page_id);
/* Adds a reference to an allocated page (prefix sharing).  Returns the new count. */
int32_t w34_pool_ref_page(w34_page_pool* pool, int32_t page_id);
int32_t w34_pool_refcount(const w34_page_pool* pool, int32_t page_id);
void w34_pool_reset(w34_page_pool* pool);
/* KvPool::truncate_pages (cache.rs:405-410): shrink and reset. */
void w34_pool_truncate(w34_page_pool* pool, int32_t max_pages);
/* Benchmark mode: allocation order becomes a seeded Fisher-Yates shuffle of the currently
 * free pages (page 0 is withheld as the trash sink when reserve_page0 != 0) instead of
 * lowest-first; freed pages go to the back of the list. */
int32_t w34_pool_shuffle_free_list(w34_page_pool* pool, uint64_t seed, int32_t reserve_page0);

typedef struct {
    int32_t capacity;
    int32_t free_pages;
    int32_t shared_pages;   /* refcount > 1 */
    int32_t active_pages;   /* refcount == 1 */
} w34_pool_stats;
void w34_pool_get_stats(const w34_page_pool* pool, w34_pool_stats* out);

/* ---- per-sequence page state: ReqRadixState KV half (radix.rs:1070-1245) ------------------- */
typedef struct w34_seq w34_seq;

w34_seq* w34_seq_create(w34_page_pool* pool);
/* Releases every page reference the sequence holds, then frees it. */
void w34_seq_destroy(w34_seq* seq);

/* Prefix hit (restore_prefix_hit, radix.rs:1129-1157): the sequence starts with `num_tokens`
 * committed tokens stored in `pages` (ceil(num_tokens / block) entries), which it shares:
 * each gets one more reference and is protected from rollback.  num_tokens need not be a
 * multiple of the block size; a shared partial tail page is copied on the first write
 * (docs/contracts/cache-layout.md:106-110). */
int32_t w34_seq_attach_prefix(w34_seq* seq, const int32_t* pages, int32_t num_pages, int32_t num_tokens);

/* ensure_kv_pages_for_len (model/generation.rs:83-96, batch.rs:59-93): make the block table
 * cover `total_tokens` positions, allocating fresh private pages.  All-or-nothing: returns
 * the number of pages added, or W34_ERR_EXHAUSTED with nothing changed. */
int32_t w34_seq_reserve(w34_seq* seq, int32_t total_tokens);

/* Copy-on-write check before appending at position committed_len: when that position falls
 * into a page with refcount > 1, a private page is allocated, swapped into the block table
 * and the shared one released.  Returns 1 and fills (src_page, dst_page, rows) when the
 * caller must copy `rows` token rows of every layer from src to dst before the append,
 * 0 when no copy is needed, negative on error. */
int32_t w34_seq_prepare_append(w34_seq* seq, int32_t* src_page, int32_t* dst_page, int32_t* rows);

/* commit_tokens (radix.rs:1197-1216): `n` more tokens are now committed. */
int32_t w34_seq_commit(w34_seq* seq, int32_t n);
/* Sets the committed length directly (tests / resume). */
int32_t w34_seq_set_committed(w34_seq* seq, int32_t committed_len);

/* rollback_uncommitted_kv_pages (radix.rs:1234-1245): drop block-table entries beyond
 * ceil(committed / block), never below the protected prefix; the dropped page ids are
 * written to `freed` (in block-table order) and released to the pool.  Returns their count
 * or W34_ERR_CAPACITY. */
int32_t w34_seq_rollback(w34_seq* seq, int32_t* freed, int32_t freed_capacity);

/* One speculative step for a batch (mtp/propose.rs + radix.rs:1197-1245 per sequence): before the
 * step every sequence gets pages for committed + extra_tokens positions (all-or-nothing over the
 * batch when the sequences share one pool; returns pages added).  After the verify pass
 * accepted[i] of the extra tokens are committed and the pages that only held rejected tokens are
 * released; their ids go to `freed` (may be NULL with capacity 0 only if nothing is freed).
 * Returns the number of pages freed. */
int32_t w34_seqs_reserve_ahead(w34_seq* const* seqs, int32_t num_seqs, int32_t extra_tokens);
int32_t w34_seqs_commit_and_rollback(w34_seq* const* seqs, const int32_t* accepted, int32_t num_seqs,
                                     int32_t* freed, int32_t freed_capacity);

int32_t w34_seq_committed_len(const w34_seq* seq);
int32_t w34_seq_num_pages(const w34_seq* seq);
int32_t w34_seq_protected_pages(const w34_seq* seq);
const int32_t* w34_seq_pages(const w34_seq* seq);
/* Tests only: replace the block table without touching reference counts. */
int32_t w34_seq_set_pages_unchecked(w34_seq* seq, const int32_t* pages, int32_t n, int32_t protected_pages);

/* ---- page-aligned radix prefix cache: MambaRadixCache, KV half (radix.rs:383-692, :950-980) -- */
typedef struct w34_radix w34_radix;

typedef struct {
    int32_t nodes;            /* live nodes, root excluded */
    int32_t cached_pages;     /* pages the tree holds a reference on */
    int32_t protected_pages;  /* of those, on locked paths */
    int32_t evictable_pages;
} w34_radix_stats;

w34_radix* w34_radix_create(w34_page_pool* pool);
/* Releases the tree's page references. */
void w34_radix_destroy(w34_radix* radix);

/* Longest cached prefix of `tokens`, in whole pages (match_prefix, radix.rs:383-490).  Writes
 * the matched page ids, the matched token count (a multiple of the block size) and the deepest
 * matched node (0 = root = no match); refreshes recency along the path.  A node that matches
 * only partly is split at the page boundary.  Returns the number of pages or a negative error. */
int32_t w34_radix_match_prefix(w34_radix* radix, const int32_t* tokens, int32_t num_tokens,
                               int32_t* out_pages, int32_t page_capacity, int32_t* matched_tokens,
                               int32_t* last_node);

/* inc_lock_ref / dec_lock_ref (radix.rs:494-550): pin / unpin the path from `node` to the
 * root against eviction.  Unbalanced unlocks return W34_ERR_PROTECTED and change nothing. */
int32_t w34_radix_lock(w34_radix* radix, int32_t node);
int32_t w34_radix_unlock(w34_radix* radix, int32_t node);

/* insert (radix.rs:552-692): caches a page-aligned token sequence with its pages.  The tree
 * takes one pool reference on every page it newly stores.  Returns the number of leading
 * tokens that were already cached (the caller may free its duplicate pages for that prefix);
 * `last_node` receives the node that now ends the sequence. */
int32_t w34_radix_insert(w34_radix* radix, const int32_t* tokens, int32_t num_tokens,
                         const int32_t* pages, int32_t num_pages, int32_t* last_node);

/* evict_full_pages (radix.rs:950-980): drops least-recently-used unlocked leaves until at least
 * num_pages pages were released (or nothing evictable is left); their ids are written to
 * `freed` and their references returned to the pool.  Returns the count. */
int32_t w34_radix_evict(w34_radix* radix, int32_t num_pages, int32_t* freed, int32_t capacity);

void w34_radix_get_stats(const w34_radix* radix, w34_radix_stats* out);
/* 0 when the structural invariants hold (sanity_check, radix.rs:983-1041). */
int32_t w34_radix_sanity_check(const w34_radix* radix);

/* ---- step metadata (model/graph_io.rs:368-420, :505-576; execution.rs:386, :618) ----------- */
/*
 * Packs the device-side arrays of one attention step for `num_seqs` sequences, sequence i
 * contributing q_lens[i] new tokens after its committed length:
 *   query_start_loc[num_seqs + 1], context_lens_before[num_seqs], seq_lens_after[num_seqs],
 *   block_tables[num_seqs * max_blocks_per_req] (unused entries 0 = trash page),
 *   write_slot_mapping[sum q_lens]:  slot = block_table[pos / B] * B + pos % B.
 * Every sequence must already cover committed + q_len positions (w34_seq_reserve).
 * Returns total tokens, or a negative error (W34_ERR_CAPACITY if a block table does not fit
 * in max_blocks_per_req).  Also reports max q_len / seq_len for the descriptor.
 */
int32_t w34_build_step_metadata(w34_seq* const* seqs, const int32_t* q_lens, int32_t num_seqs,
                                int32_t max_blocks_per_req, int32_t* query_start_loc,
                                int32_t* context_lens_before, int32_t* seq_lens_after,
                                int32_t* block_tables, int32_t* write_slot_mapping,
                                int32_t* out_max_q_len, int32_t* out_max_seq_len);

/* The same packer for a persistent arena: block_tables must still hold what the previous call
 * left there.  For every row i it reports the column range [changed_lo[i], changed_hi[i]) whose
 * entries differ from before (changed_lo >= changed_hi: nothing), so that the caller uploads only
 * those suffixes (graph_io.rs:109-195). */
int32_t w34_build_step_metadata_delta(w34_seq* const* seqs, const int32_t* q_lens, int32_t num_seqs,
                                      int32_t max_blocks_per_req, int32_t* query_start_loc,
                                      int32_t* context_lens_before, int32_t* seq_lens_after,
                                      int32_t* block_tables, int32_t* write_slot_mapping,
                                      int32_t* out_max_q_len, int32_t* out_max_seq_len,
                                      int32_t* changed_lo, int32_t* changed_hi);

#ifdef __cplusplus
}
#endif
#endif /* WARP34_HOST_H */
