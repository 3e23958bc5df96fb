// Page-aligned radix prefix cache over token ids: the KV half of the reference's
// MambaRadixCache (crates/warp34-host/src/radix.rs:383-692 match / insert / split,
// :494-550 path lock references, :950-980 LRU leaf eviction, :983-1041 sanity check).
// The GDN-checkpoint ("mamba") half of that structure is out of scope here.
//
// Keys are compared a page (block_size tokens) at a time, so matches, splits and inserts
// always fall on page boundaries; children are keyed by their first page of tokens.  A node
// owns one pool reference on each of its pages (w34_pool_ref_page at insert, released at
// eviction); requests that reuse a prefix take their own references through
// w34_seq_attach_prefix and pin the path with w34_radix_lock.
#include <algorithm>
#include <cstdint>
#include <list>
#include <map>
#include <new>
#include <vector>

#include "../../../include/warp34_host.h"

namespace {

struct Node {
    int32_t parent = -1;
    std::vector<int32_t> key;      // tokens of this edge, a multiple of the page size
    std::vector<int32_t> pages;    // key.size() / page pages
    std::map<std::vector<int32_t>, int32_t> children;  // first page of child's key -> child id
    int32_t lock_ref = 0;
    uint64_t last_access = 0;
    bool alive = false;
};

}  // namespace

struct w34_radix {
    w34_page_pool* pool = nullptr;
    int32_t page = 16;
    std::vector<Node> nodes;        // node 0 is the root
    std::vector<int32_t> free_ids;
    uint64_t clock = 0;
    int64_t cached_pages = 0, protected_pages = 0;

    int32_t alloc_node() {
        int32_t id;
        if (!free_ids.empty()) { id = free_ids.back(); free_ids.pop_back(); nodes[(size_t)id] = Node(); }
        else { id = (int32_t)nodes.size(); nodes.emplace_back(); }
        nodes[(size_t)id].alive = true;
        return id;
    }

    size_t common_pages(const std::vector<int32_t>& key, const int32_t* tok, size_t n_tok) const {
        const size_t max_pages = std::min(key.size(), n_tok) / (size_t)page;
        size_t m = 0;
        while (m < max_pages && std::equal(key.begin() + (long)(m * page), key.begin() + (long)((m + 1) * page),
                                           tok + m * page)) ++m;
        return m;
    }

    // Splits `child` after `keep_pages` pages; returns the new intermediate node, which inherits
    // the child's lock count (every lock on the child also pins its new parent).
    int32_t split(int32_t child, size_t keep_pages) {
        const int32_t mid = alloc_node();
        Node& c = nodes[(size_t)child];
        Node& m = nodes[(size_t)mid];
        const size_t keep_tok = keep_pages * (size_t)page;
        m.parent = c.parent;
        m.key.assign(c.key.begin(), c.key.begin() + (long)keep_tok);
        m.pages.assign(c.pages.begin(), c.pages.begin() + (long)keep_pages);
        m.lock_ref = c.lock_ref;
        m.last_access = c.last_access;
        std::vector<int32_t> first(m.key.begin(), m.key.begin() + page);
        nodes[(size_t)c.parent].children[first] = mid;
        c.key.erase(c.key.begin(), c.key.begin() + (long)keep_tok);
        c.pages.erase(c.pages.begin(), c.pages.begin() + (long)keep_pages);
        c.parent = mid;
        std::vector<int32_t> cfirst(c.key.begin(), c.key.begin() + page);
        m.children[cfirst] = child;
        return mid;
    }
};

extern "C" {

w34_radix* w34_radix_create(w34_page_pool* pool) {
    if (!pool) return nullptr;
    w34_radix* r = new (std::nothrow) w34_radix();
    if (!r) return nullptr;
    r->pool = pool;
    r->page = w34_pool_block_size(pool);
    r->nodes.emplace_back();
    r->nodes[0].alive = true;
    return r;
}

void w34_radix_destroy(w34_radix* r) {
    if (!r) return;
    for (const Node& n : r->nodes) {
        if (n.alive) for (int32_t p : n.pages) w34_pool_free_page(r->pool, p);
    }
    delete r;
}

int32_t w34_radix_match_prefix(w34_radix* r, const int32_t* tokens, int32_t num_tokens, int32_t* out_pages,
                               int32_t page_capacity, int32_t* matched_tokens, int32_t* last_node) {
    if (!r || (!tokens && num_tokens > 0) || num_tokens < 0) return W34_ERR_INVALID;
    const size_t aligned = (size_t)num_tokens / (size_t)r->page * (size_t)r->page;
    int32_t cur = 0, n_out = 0;
    size_t off = 0;
    ++r->clock;
    while (off < aligned) {
        std::vector<int32_t> first(tokens + off, tokens + off + r->page);
        auto it = r->nodes[(size_t)cur].children.find(first);
        if (it == r->nodes[(size_t)cur].children.end()) break;
        int32_t child = it->second;
        const size_t m = r->common_pages(r->nodes[(size_t)child].key, tokens + off, aligned - off);
        if (m * (size_t)r->page < r->nodes[(size_t)child].key.size()) child = r->split(child, m);
        Node& c = r->nodes[(size_t)child];
        if (n_out + (int32_t)c.pages.size() > page_capacity) return W34_ERR_CAPACITY;
        for (int32_t p : c.pages) out_pages[n_out++] = p;
        c.last_access = r->clock;
        off += c.key.size();
        cur = child;
        if (m * (size_t)r->page < c.key.size()) break;  // cannot happen after the split; kept for clarity
    }
    // refresh recency from the root down so the deepest node is the most recent
    for (int32_t n = cur; n > 0; n = r->nodes[(size_t)n].parent) r->nodes[(size_t)n].last_access = r->clock;
    if (matched_tokens) *matched_tokens = (int32_t)off;
    if (last_node) *last_node = cur;
    return n_out;
}

int32_t w34_radix_lock(w34_radix* r, int32_t node) {
    if (!r || node < 0 || node >= (int32_t)r->nodes.size() || !r->nodes[(size_t)node].alive) return W34_ERR_INVALID;
    for (int32_t n = node; n > 0; n = r->nodes[(size_t)n].parent) {
        Node& x = r->nodes[(size_t)n];
        if (x.lock_ref == 0) r->protected_pages += (int64_t)x.pages.size();
        ++x.lock_ref;
    }
    return W34_OK;
}

int32_t w34_radix_unlock(w34_radix* r, int32_t node) {
    if (!r || node < 0 || node >= (int32_t)r->nodes.size() || !r->nodes[(size_t)node].alive) return W34_ERR_INVALID;
    for (int32_t n = node; n > 0; n = r->nodes[(size_t)n].parent) {
        if (r->nodes[(size_t)n].lock_ref <= 0) return W34_ERR_PROTECTED;  // unbalanced unlock: nothing changed below
    }
    for (int32_t n = node; n > 0; n = r->nodes[(size_t)n].parent) {
        Node& x = r->nodes[(size_t)n];
        --x.lock_ref;
        if (x.lock_ref == 0) r->protected_pages -= (int64_t)x.pages.size();
    }
    return W34_OK;
}

int32_t w34_radix_insert(w34_radix* r, const int32_t* tokens, int32_t num_tokens, const int32_t* pages,
                         int32_t num_pages, int32_t* last_node) {
    if (!r || !tokens || !pages || num_tokens < 0 || num_tokens % r->page != 0 ||
        num_pages != num_tokens / r->page) return W34_ERR_INVALID;
    int32_t cur = 0;
    size_t off = 0;
    ++r->clock;
    const size_t total = (size_t)num_tokens;
    while (off < total) {
        std::vector<int32_t> first(tokens + off, tokens + off + r->page);
        auto it = r->nodes[(size_t)cur].children.find(first);
        if (it == r->nodes[(size_t)cur].children.end()) {
            // new leaf with everything that is left; the tree takes one reference per page
            for (size_t p = off / (size_t)r->page; p < (size_t)num_pages; ++p) {
                if (w34_pool_ref_page(r->pool, pages[p]) < 0) {
                    for (size_t q = off / (size_t)r->page; q < p; ++q) w34_pool_free_page(r->pool, pages[q]);
                    return W34_ERR_INVALID;
                }
            }
            const int32_t leaf = r->alloc_node();
            Node& l = r->nodes[(size_t)leaf];
            l.parent = cur;
            l.key.assign(tokens + off, tokens + total);
            l.pages.assign(pages + off / (size_t)r->page, pages + num_pages);
            l.last_access = r->clock;
            r->nodes[(size_t)cur].children[first] = leaf;
            r->cached_pages += (int64_t)l.pages.size();
            cur = leaf;
            const int32_t already = (int32_t)off;
            if (last_node) *last_node = cur;
            return already;
        }
        int32_t child = it->second;
        const size_t m = r->common_pages(r->nodes[(size_t)child].key, tokens + off, total - off);
        if (m * (size_t)r->page < r->nodes[(size_t)child].key.size()) child = r->split(child, m);
        r->nodes[(size_t)child].last_access = r->clock;
        off += r->nodes[(size_t)child].key.size();
        cur = child;
    }
    if (last_node) *last_node = cur;
    return (int32_t)off;  // whole sequence was already cached
}

int32_t w34_radix_evict(w34_radix* r, int32_t num_pages, int32_t* freed, int32_t capacity) {
    if (!r || num_pages < 0 || (num_pages > 0 && !freed)) return W34_ERR_INVALID;
    int32_t n_freed = 0;
    while (n_freed < num_pages) {
        int32_t best = -1;
        for (int32_t i = 1; i < (int32_t)r->nodes.size(); ++i) {
            const Node& n = r->nodes[(size_t)i];
            if (!n.alive || !n.children.empty() || n.lock_ref != 0) continue;
            if (best < 0 || n.last_access < r->nodes[(size_t)best].last_access) best = i;
        }
        if (best < 0) break;
        Node& b = r->nodes[(size_t)best];
        if (n_freed + (int32_t)b.pages.size() > capacity) return W34_ERR_CAPACITY;
        for (int32_t p : b.pages) { freed[n_freed++] = p; w34_pool_free_page(r->pool, p); }
        r->cached_pages -= (int64_t)b.pages.size();
        std::vector<int32_t> first(b.key.begin(), b.key.begin() + r->page);
        r->nodes[(size_t)b.parent].children.erase(first);
        b.alive = false;
        b.children.clear();
        r->free_ids.push_back(best);
    }
    return n_freed;
}

void w34_radix_get_stats(const w34_radix* r, w34_radix_stats* out) {
    if (!r || !out) return;
    int32_t nodes = 0;
    for (const Node& n : r->nodes) if (n.alive) ++nodes;
    out->nodes = nodes - 1;
    out->cached_pages = (int32_t)r->cached_pages;
    out->protected_pages = (int32_t)r->protected_pages;
    out->evictable_pages = (int32_t)(r->cached_pages - r->protected_pages);
}

// Structural invariants (radix.rs:983-1041): page-aligned keys, one page per block of key,
// children keyed by their first page, parents at least as locked as their children, counters
// consistent.  Returns 0 when everything holds, else the number of the first failed check.
int32_t w34_radix_sanity_check(const w34_radix* r) {
    if (!r) return 1;
    int64_t cached = 0, prot = 0;
    for (int32_t i = 1; i < (int32_t)r->nodes.size(); ++i) {
        const Node& n = r->nodes[(size_t)i];
        if (!n.alive) continue;
        if (n.key.empty() || n.key.size() % (size_t)r->page != 0) return 2;
        if (n.pages.size() * (size_t)r->page != n.key.size()) return 3;
        if (n.parent < 0 || !r->nodes[(size_t)n.parent].alive) return 4;
        std::vector<int32_t> first(n.key.begin(), n.key.begin() + r->page);
        auto it = r->nodes[(size_t)n.parent].children.find(first);
        if (it == r->nodes[(size_t)n.parent].children.end() || it->second != i) return 5;
        if (n.lock_ref < 0) return 6;
        int32_t child_locks = 0;
        for (const auto& kv : n.children) child_locks = std::max(child_locks, r->nodes[(size_t)kv.second].lock_ref);
        if (n.lock_ref < child_locks) return 7;
        for (int32_t p : n.pages) if (w34_pool_refcount(r->pool, p) < 1) return 8;
        cached += (int64_t)n.pages.size();
        if (n.lock_ref > 0) prot += (int64_t)n.pages.size();
    }
    if (cached != r->cached_pages) return 9;
    if (prot != r->protected_pages) return 10;
    return 0;
}

}  // extern "C"
