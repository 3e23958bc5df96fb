// Host-side KV page manager behind the C ABI of include/warp34_host.h.
//
// Follows the semantics of the reference's Rust host state:
//   PageBitmap / KvPool page API      crates/warp34-host/src/cache.rs:185-265, :385-416
//   KvFormatPolicy, row bytes, strides crates/warp34-host/src/cache.rs:27-165, :296-334
//   ReqRadixState (KV half), rollback  crates/warp34-host/src/radix.rs:1070-1245
//   slot / block-table packing         crates/warp34-host/src/model/graph_io.rs:393-398, :554-557
// and adds what the contract specifies but the reference never built: per-page reference
// counts and copy-on-write of a shared partial tail page (docs/contracts/cache-layout.md:106-110).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <new>
#include <vector>

#include "../../../include/warp34_host.h"

namespace {

inline int ctz64(uint64_t x) { return __builtin_ctzll(x); }

// splitmix64: seeds the shuffled free list reproducibly on every platform.
inline uint64_t splitmix64(uint64_t& s) {
    uint64_t z = (s += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

}  // namespace

struct w34_page_pool {
    int32_t num_pages = 0;
    int32_t block_size = 16;
    std::vector<uint64_t> words;      // bit set = page free
    std::vector<int32_t> refcount;    // 0 = free
    int32_t free_count = 0;
    size_t next_word = 0;
    bool shuffled = false;
    std::deque<int32_t> order;        // allocation order in shuffled mode
    int32_t withheld = -1;            // page kept out of circulation in shuffled mode

    void reset() {
        const size_t full = (size_t)num_pages / 64, rem = (size_t)num_pages % 64;
        std::fill(words.begin(), words.end(), 0ull);
        for (size_t w = 0; w < full; ++w) words[w] = ~0ull;
        if (rem) words[full] = (1ull << rem) - 1ull;
        std::fill(refcount.begin(), refcount.end(), 0);
        free_count = num_pages;
        next_word = 0;
        shuffled = false;
        order.clear();
        withheld = -1;
    }

    void resize(int32_t n) {
        num_pages = n;
        words.assign(((size_t)n + 63) / 64, 0ull);
        refcount.assign((size_t)n, 0);
        reset();
    }

    bool is_free(int32_t p) const { return (words[(size_t)p / 64] >> (p % 64)) & 1ull; }

    int32_t alloc() {
        if (shuffled) {
            while (!order.empty()) {
                const int32_t p = order.front();
                order.pop_front();
                if (p >= 0 && p < num_pages && is_free(p)) {
                    words[(size_t)p / 64] &= ~(1ull << (p % 64));
                    --free_count;
                    refcount[(size_t)p] = 1;
                    return p;
                }
            }
            return W34_ERR_EXHAUSTED;
        }
        if (free_count == 0) return W34_ERR_EXHAUSTED;
        const size_t n = words.size();
        for (int pass = 0; pass < 2; ++pass) {
            const size_t lo = pass == 0 ? next_word : 0, hi = pass == 0 ? n : next_word;
            for (size_t w = lo; w < hi; ++w) {
                if (words[w] != 0) {
                    const int bit = ctz64(words[w]);
                    words[w] &= ~(1ull << bit);
                    --free_count;
                    next_word = w;
                    const int32_t p = (int32_t)(w * 64 + (size_t)bit);
                    refcount[(size_t)p] = 1;
                    return p;
                }
            }
        }
        return W34_ERR_EXHAUSTED;
    }

    int32_t available() const { return shuffled && withheld >= 0 && is_free(withheld) ? free_count - 1 : free_count; }

    int32_t unref(int32_t p) {
        if (p < 0 || p >= num_pages) return 0;
        if (is_free(p)) return 0;
        int32_t& rc = refcount[(size_t)p];
        if (rc > 1) return --rc;
        rc = 0;
        const size_t w = (size_t)p / 64;
        words[w] |= 1ull << (p % 64);
        ++free_count;
        if (w < next_word) next_word = w;
        if (shuffled) order.push_back(p);
        return 0;
    }
};

struct w34_seq {
    w34_page_pool* pool = nullptr;
    std::vector<int32_t> pages;       // block table: logical page ids
    int32_t committed = 0;            // committed tokens
    int32_t protected_pages = 0;      // shared prefix entries that rollback never drops
};

extern "C" {

int32_t w34_kv_format_row_bytes(int32_t format, int32_t head_dim) {
    switch (format) {
        case WARP34_KV_FORMAT_FP16:
        case WARP34_KV_FORMAT_BF16: return head_dim * 2;
        case WARP34_KV_FORMAT_TQ4: return 66 * (head_dim / 128);
        case WARP34_KV_FORMAT_Q8_0: return 68 * (head_dim / 64);
        case WARP34_KV_FORMAT_FP8_E4M3: return head_dim + 4 * (head_dim / 128);
        default: return head_dim * 2;
    }
}

int32_t w34_kv_policy_resolve_layer(int32_t policy, int32_t ord, int32_t num_layers,
                                    int32_t supports_fp8, int32_t out[4]) {
    if (!out || ord < 0 || num_layers < 0) return W34_ERR_INVALID;
    int32_t fmt, tf = WARP34_KV_TRANSFORM_IDENTITY;
    switch (policy) {
        case W34_KV_POLICY_FP16: fmt = WARP34_KV_FORMAT_FP16; break;
        case W34_KV_POLICY_BF16: fmt = WARP34_KV_FORMAT_BF16; break;
        case W34_KV_POLICY_Q8_0: fmt = WARP34_KV_FORMAT_Q8_0; break;
        case W34_KV_POLICY_FP8: fmt = WARP34_KV_FORMAT_FP8_E4M3; break;
        case W34_KV_POLICY_TQ4: {
            const int32_t first_boundary = num_layers > 4 ? num_layers - 4 : 0;
            if (ord >= first_boundary) {
                fmt = supports_fp8 ? WARP34_KV_FORMAT_FP8_E4M3 : WARP34_KV_FORMAT_Q8_0;
            } else {
                fmt = WARP34_KV_FORMAT_TQ4;
                tf = WARP34_KV_TRANSFORM_RADEMACHER_WHT256;
            }
            break;
        }
        case W34_KV_POLICY_TQ4_ALL:
            fmt = WARP34_KV_FORMAT_TQ4;
            tf = WARP34_KV_TRANSFORM_RADEMACHER_WHT256;
            break;
        default: return W34_ERR_INVALID;
    }
    out[0] = fmt; out[1] = fmt; out[2] = tf; out[3] = tf;
    return W34_OK;
}

int64_t w34_kv_policy_bytes_per_token(int32_t policy, int32_t num_layers, int32_t kv_heads,
                                      int32_t head_dim, int32_t supports_fp8) {
    int64_t total = 0;
    for (int32_t ord = 0; ord < num_layers; ++ord) {
        int32_t f[4];
        if (w34_kv_policy_resolve_layer(policy, ord, num_layers, supports_fp8, f) != W34_OK) return W34_ERR_INVALID;
        total += (int64_t)kv_heads * (w34_kv_format_row_bytes(f[0], head_dim) + w34_kv_format_row_bytes(f[1], head_dim));
    }
    return total;
}

int32_t w34_kv_layout_init(warp34_kv_layer_layout* l, uint64_t k_base, uint64_t v_base, int32_t ns,
                           int32_t layer_id, int32_t heads, int32_t head_dim, int32_t block_size,
                           const int32_t f[4], int64_t num_pages, uint64_t* out_k, uint64_t* out_v) {
    if (!l || !f || heads <= 0 || head_dim <= 0 || block_size <= 0 || num_pages < 0) return W34_ERR_INVALID;
    const uint64_t kt = (uint64_t)w34_kv_format_row_bytes(f[0], head_dim);
    const uint64_t vt = (uint64_t)w34_kv_format_row_bytes(f[1], head_dim);
    std::memset(l, 0, sizeof(*l));
    l->k_base = k_base; l->v_base = v_base;
    l->k_token_stride_bytes = kt; l->v_token_stride_bytes = vt;
    l->k_head_stride_bytes = (uint64_t)block_size * kt; l->v_head_stride_bytes = (uint64_t)block_size * vt;
    l->k_page_stride_bytes = (uint64_t)heads * l->k_head_stride_bytes;
    l->v_page_stride_bytes = (uint64_t)heads * l->v_head_stride_bytes;
    l->namespace_id = ns; l->layer_id = layer_id; l->local_kv_heads = heads; l->head_dim = head_dim;
    l->block_size = block_size;
    l->k_format = f[0]; l->v_format = f[1]; l->k_transform = f[2]; l->v_transform = f[3];
    if (out_k) *out_k = (uint64_t)num_pages * l->k_page_stride_bytes;
    if (out_v) *out_v = (uint64_t)num_pages * l->v_page_stride_bytes;
    return W34_OK;
}

// ---- pool ---------------------------------------------------------------------------------
w34_page_pool* w34_pool_create(int32_t num_pages, int32_t block_size) {
    if (num_pages < 0 || block_size <= 0) return nullptr;
    w34_page_pool* p = new (std::nothrow) w34_page_pool();
    if (!p) return nullptr;
    p->block_size = block_size;
    p->resize(num_pages);
    return p;
}
void w34_pool_destroy(w34_page_pool* p) { delete p; }
int32_t w34_pool_num_pages(const w34_page_pool* p) { return p ? p->num_pages : 0; }
int32_t w34_pool_block_size(const w34_page_pool* p) { return p ? p->block_size : 0; }
int32_t w34_pool_free_count(const w34_page_pool* p) { return p ? p->free_count : 0; }
int32_t w34_pool_alloc_page(w34_page_pool* p) { return p ? p->alloc() : W34_ERR_INVALID; }
int32_t w34_pool_free_page(w34_page_pool* p, int32_t page) { return p ? p->unref(page) : 0; }
int32_t w34_pool_ref_page(w34_page_pool* p, int32_t page) {
    if (!p || page < 0 || page >= p->num_pages || p->is_free(page)) return W34_ERR_INVALID;
    return ++p->refcount[(size_t)page];
}
int32_t w34_pool_refcount(const w34_page_pool* p, int32_t page) {
    if (!p || page < 0 || page >= p->num_pages) return 0;
    return p->refcount[(size_t)page];
}
void w34_pool_reset(w34_page_pool* p) { if (p) p->reset(); }
void w34_pool_truncate(w34_page_pool* p, int32_t max_pages) {
    if (p && max_pages >= 0 && max_pages < p->num_pages) p->resize(max_pages);
}
int32_t w34_pool_shuffle_free_list(w34_page_pool* p, uint64_t seed, int32_t reserve_page0) {
    if (!p) return W34_ERR_INVALID;
    std::vector<int32_t> ids;
    ids.reserve((size_t)p->free_count);
    for (int32_t i = 0; i < p->num_pages; ++i) {
        if (p->is_free(i) && !(reserve_page0 && i == 0)) ids.push_back(i);
    }
    uint64_t s = seed;
    for (size_t i = ids.size(); i > 1; --i) {
        const size_t j = (size_t)(splitmix64(s) % (uint64_t)i);
        std::swap(ids[i - 1], ids[j]);
    }
    p->order.assign(ids.begin(), ids.end());
    p->shuffled = true;
    p->withheld = reserve_page0 ? 0 : -1;
    return (int32_t)ids.size();
}
void w34_pool_get_stats(const w34_page_pool* p, w34_pool_stats* out) {
    if (!p || !out) return;
    out->capacity = p->num_pages;
    out->free_pages = p->free_count;
    int32_t shared = 0, active = 0;
    for (int32_t rc : p->refcount) { if (rc > 1) ++shared; else if (rc == 1) ++active; }
    out->shared_pages = shared;
    out->active_pages = active;
}

// ---- sequences -------------------------------------------------------------------------------
w34_seq* w34_seq_create(w34_page_pool* pool) {
    if (!pool) return nullptr;
    w34_seq* s = new (std::nothrow) w34_seq();
    if (s) s->pool = pool;
    return s;
}
void w34_seq_destroy(w34_seq* s) {
    if (!s) return;
    for (int32_t p : s->pages) s->pool->unref(p);
    delete s;
}

int32_t w34_seq_attach_prefix(w34_seq* s, const int32_t* pages, int32_t n_pages, int32_t n_tokens) {
    if (!s || !pages || n_pages < 0 || n_tokens < 0 || !s->pages.empty()) return W34_ERR_INVALID;
    const int32_t B = s->pool->block_size;
    if ((n_tokens + B - 1) / B != n_pages) return W34_ERR_INVALID;
    for (int32_t i = 0; i < n_pages; ++i) {
        const int32_t p = pages[i];
        if (p < 0 || p >= s->pool->num_pages || s->pool->is_free(p)) return W34_ERR_INVALID;
    }
    for (int32_t i = 0; i < n_pages; ++i) ++s->pool->refcount[(size_t)pages[i]];
    s->pages.assign(pages, pages + n_pages);
    s->committed = n_tokens;
    s->protected_pages = n_pages;
    return W34_OK;
}

int32_t w34_seq_reserve(w34_seq* s, int32_t total_tokens) {
    if (!s || total_tokens < 0) return W34_ERR_INVALID;
    const int32_t B = s->pool->block_size;
    const int32_t need = (total_tokens + B - 1) / B;
    const int32_t have = (int32_t)s->pages.size();
    if (need <= have) return 0;
    if (need - have > s->pool->available()) return W34_ERR_EXHAUSTED;
    for (int32_t i = have; i < need; ++i) {
        const int32_t p = s->pool->alloc();
        if (p < 0) {  // cannot happen after the check above; undo to stay all-or-nothing
            while ((int32_t)s->pages.size() > have) { s->pool->unref(s->pages.back()); s->pages.pop_back(); }
            return W34_ERR_EXHAUSTED;
        }
        s->pages.push_back(p);
    }
    return need - have;
}

int32_t w34_seq_prepare_append(w34_seq* s, int32_t* src_page, int32_t* dst_page, int32_t* rows) {
    if (!s) return W34_ERR_INVALID;
    const int32_t B = s->pool->block_size;
    const int32_t idx = s->committed / B, off = s->committed % B;
    if (off == 0 || idx >= (int32_t)s->pages.size()) return 0;   // next write starts a fresh page
    const int32_t shared = s->pages[(size_t)idx];
    if (s->pool->refcount[(size_t)shared] <= 1) {
        if (idx < s->protected_pages) s->protected_pages = idx;   // sole owner: now private
        return 0;
    }
    if (s->pool->available() < 1) return W34_ERR_EXHAUSTED;
    const int32_t fresh = s->pool->alloc();
    if (fresh < 0) return W34_ERR_EXHAUSTED;
    s->pages[(size_t)idx] = fresh;
    s->pool->unref(shared);
    if (idx < s->protected_pages) s->protected_pages = idx;
    if (src_page) *src_page = shared;
    if (dst_page) *dst_page = fresh;
    if (rows) *rows = off;
    return 1;
}

int32_t w34_seq_commit(w34_seq* s, int32_t n) {
    if (!s || n < 0) return W34_ERR_INVALID;
    const int64_t cap = (int64_t)s->pages.size() * s->pool->block_size;
    if ((int64_t)s->committed + n > cap) return W34_ERR_INVALID;
    s->committed += n;
    return s->committed;
}
int32_t w34_seq_set_committed(w34_seq* s, int32_t committed_len) {
    if (!s || committed_len < 0) return W34_ERR_INVALID;
    s->committed = committed_len;
    return W34_OK;
}

int32_t w34_seq_rollback(w34_seq* s, int32_t* freed, int32_t cap) {
    if (!s) return W34_ERR_INVALID;
    const int32_t B = s->pool->block_size;
    const int32_t needed = std::max((s->committed + B - 1) / B, s->protected_pages);
    const int32_t have = (int32_t)s->pages.size();
    if (have <= needed) return 0;
    const int32_t n = have - needed;
    if (n > cap || (!freed && n > 0)) return W34_ERR_CAPACITY;
    for (int32_t i = 0; i < n; ++i) {
        freed[i] = s->pages[(size_t)(needed + i)];
        s->pool->unref(freed[i]);
    }
    s->pages.resize((size_t)needed);
    return n;
}

int32_t w34_seqs_reserve_ahead(w34_seq* const* seqs, int32_t num_seqs, int32_t extra_tokens) {
    if (!seqs || num_seqs < 0 || extra_tokens < 0) return W34_ERR_INVALID;
    // all-or-nothing over the batch: count first, then allocate
    int64_t need_total = 0;
    for (int32_t i = 0; i < num_seqs; ++i) {
        const w34_seq* s = seqs[i];
        if (!s) return W34_ERR_INVALID;
        const int32_t B = s->pool->block_size;
        const int32_t need = (s->committed + extra_tokens + B - 1) / B - (int32_t)s->pages.size();
        if (need > 0) need_total += need;
    }
    if (num_seqs > 0 && need_total > seqs[0]->pool->available()) return W34_ERR_EXHAUSTED;
    int32_t added = 0;
    for (int32_t i = 0; i < num_seqs; ++i) {
        const int32_t rc = w34_seq_reserve(seqs[i], seqs[i]->committed + extra_tokens);
        if (rc < 0) return rc;      // sequences of different pools: the earlier ones keep their pages
        added += rc;
    }
    return added;
}

int32_t w34_seqs_commit_and_rollback(w34_seq* const* seqs, const int32_t* accepted, int32_t num_seqs,
                                     int32_t* freed, int32_t freed_capacity) {
    if (!seqs || !accepted || num_seqs < 0 || freed_capacity < 0) return W34_ERR_INVALID;
    int32_t total = 0;
    for (int32_t i = 0; i < num_seqs; ++i) {
        if (!seqs[i] || accepted[i] < 0) return W34_ERR_INVALID;
        const int32_t rc = w34_seq_commit(seqs[i], accepted[i]);
        if (rc < 0) return rc;
        const int32_t n = w34_seq_rollback(seqs[i], freed ? freed + total : nullptr, freed_capacity - total);
        if (n < 0) return n;
        total += n;
    }
    return total;
}

int32_t w34_seq_committed_len(const w34_seq* s) { return s ? s->committed : 0; }
int32_t w34_seq_num_pages(const w34_seq* s) { return s ? (int32_t)s->pages.size() : 0; }
int32_t w34_seq_protected_pages(const w34_seq* s) { return s ? s->protected_pages : 0; }
const int32_t* w34_seq_pages(const w34_seq* s) { return s ? s->pages.data() : nullptr; }
int32_t w34_seq_set_pages_unchecked(w34_seq* s, const int32_t* pages, int32_t n, int32_t protected_pages) {
    if (!s || n < 0 || (n > 0 && !pages) || protected_pages < 0) return W34_ERR_INVALID;
    s->pages.assign(pages, pages + n);
    s->protected_pages = protected_pages;
    return W34_OK;
}

int32_t w34_build_step_metadata_delta(w34_seq* const* seqs, const int32_t* q_lens, int32_t num_seqs,
                                      int32_t max_blocks, int32_t* qsl, int32_t* ctx_before,
                                      int32_t* seq_after, int32_t* block_tables, int32_t* slots,
                                      int32_t* out_max_q, int32_t* out_max_seq,
                                      int32_t* changed_lo, int32_t* changed_hi) {
    if (!seqs || !q_lens || num_seqs < 0 || max_blocks <= 0 || !qsl || !ctx_before || !seq_after ||
        !block_tables || !slots) return W34_ERR_INVALID;
    int32_t total = 0, max_q = 0, max_seq = 0;
    qsl[0] = 0;
    for (int32_t i = 0; i < num_seqs; ++i) {
        const w34_seq* s = seqs[i];
        if (!s || q_lens[i] < 0) return W34_ERR_INVALID;
        const int32_t B = s->pool->block_size;
        const int32_t after = s->committed + q_lens[i];
        const int32_t need = (after + B - 1) / B;
        if (need > (int32_t)s->pages.size()) return W34_ERR_INVALID;   // reserve first
        if (need > max_blocks) return W34_ERR_CAPACITY;
        int32_t* row = block_tables + (size_t)i * (size_t)max_blocks;
        int32_t lo = max_blocks, hi = 0;          // columns [lo, hi) of this row differ from what was there
        const int32_t* pages = s->pages.data();
        if (std::memcmp(row, pages, (size_t)need * sizeof(int32_t)) != 0) {   // rare: find the range
            for (int32_t b = 0; b < need; ++b) {
                if (row[b] != pages[b]) {
                    row[b] = pages[b];
                    if (b < lo) lo = b;
                    hi = b + 1;
                }
            }
        }
        // Entries past the sequence are never read by the kernels and are kept at 0, the trash page.
        // Plain call (no change report): the whole tail is cleared.  Persistent arena: the row held a
        // valid table before, so clearing stops at the first zero (if page 0 was a real entry of a
        // longer old table, ids behind it stay: harmless, and host and device copies still agree).
        for (int32_t b = need; b < max_blocks && (changed_lo == nullptr || row[b] != 0); ++b) {
            if (row[b] != 0) {
                row[b] = 0;
                if (b < lo) lo = b;
                hi = b + 1;
            }
        }
        if (changed_lo) changed_lo[i] = lo;
        if (changed_hi) changed_hi[i] = hi;
        for (int32_t t = 0; t < q_lens[i]; ++t) {
            const int32_t pos = s->committed + t;
            slots[total + t] = s->pages[(size_t)(pos / B)] * B + pos % B;
        }
        ctx_before[i] = s->committed;
        seq_after[i] = after;
        total += q_lens[i];
        qsl[i + 1] = total;
        max_q = std::max(max_q, q_lens[i]);
        max_seq = std::max(max_seq, after);
    }
    if (out_max_q) *out_max_q = max_q;
    if (out_max_seq) *out_max_seq = max_seq;
    return total;
}

int32_t w34_build_step_metadata(w34_seq* const* seqs, const int32_t* q_lens, int32_t num_seqs,
                                int32_t max_blocks, int32_t* qsl, int32_t* ctx_before,
                                int32_t* seq_after, int32_t* block_tables, int32_t* slots,
                                int32_t* out_max_q, int32_t* out_max_seq) {
    return w34_build_step_metadata_delta(seqs, q_lens, num_seqs, max_blocks, qsl, ctx_before, seq_after,
                                         block_tables, slots, out_max_q, out_max_seq, nullptr, nullptr);
}

}  // extern "C"
