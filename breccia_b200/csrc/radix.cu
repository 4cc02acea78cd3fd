// Radix prefix tree over token ids at page granularity (host side, no device work).
//
// The reference has no prefix sharing ("Radix/prompt prefix sharing | open", docs/BRIEF.md:287); its
// design note fixes the granule: a block is 16 tokens, identified by the hash of its tokens and of
// everything before them, with a refcount and a free queue
// (docs/reference-engines/02-kv-and-context.md:543-581).  This tree is that note made concrete:
//   * an edge is one full page of 16 token ids; a node owns one reference to the page that caches
//     the K/V of that page of the prefix (in every layer);
//   * match walks full pages from the root, takes a reference for the caller on every page it
//     returns and stamps the nodes for LRU;
//   * insert adds the missing nodes along a path (the tree takes its own reference on their pages);
//   * evict drops least-recently-used leaves whose page nobody but the tree holds.
// A partially filled last page is never shared through the tree; a caller that wants to continue a
// sequence ending mid-page forks it copy-on-write (brc_seq_fork).
#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <new>
#include <vector>

#include "brc_internal.h"

struct brc_radix_node {
    std::vector<uint32_t> key;  // page_tokens token ids
    uint32_t page = 0;
    uint64_t tick = 0;
    brc_radix_node *parent = nullptr;
    std::map<std::vector<uint32_t>, std::unique_ptr<brc_radix_node>> children;
};

struct brc_radix {
    brc_pool *pool = nullptr;
    std::mutex mu;
    brc_radix_node root;
    uint64_t clock = 0;
    uint64_t n_nodes = 0, hits = 0, misses = 0, evictions = 0;
};

namespace {

// The pool counts, per page, how many of its references radix trees hold, so that the tier can tell a
// page "held by exactly one caller" from a page only a tree holds.
void tree_mark(brc_pool *pool, uint32_t page, int delta) {
    std::lock_guard<std::mutex> lock(pool->mu);
    if (page < pool->tree_refs.size()) pool->tree_refs[page] = (uint32_t)((int)pool->tree_refs[page] + delta);
}

void release_subtree(brc_radix *r, brc_radix_node *n) {
    for (auto &kv : n->children) {
        release_subtree(r, kv.second.get());
        tree_mark(r->pool, kv.second->page, -1);
        brc_pages_release(r->pool, &kv.second->page, 1);
    }
    n->children.clear();
}

void collect_leaves(brc_radix_node *n, std::vector<brc_radix_node *> &out) {
    for (auto &kv : n->children) {
        if (kv.second->children.empty())
            out.push_back(kv.second.get());
        else
            collect_leaves(kv.second.get(), out);
    }
}

}  // namespace

extern "C" {

brc_status brc_radix_create(brc_pool *pool, brc_radix **out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_radix_create: NULL argument");
    brc_radix *r = new (std::nothrow) brc_radix();
    if (!r) return brc_fail(BRC_ERR_INVALID, "brc_radix_create: out of host memory");
    r->pool = pool;
    *out = r;
    return BRC_OK;
}

brc_status brc_radix_destroy(brc_radix *radix) {
    if (!radix) return BRC_OK;
    {
        std::lock_guard<std::mutex> lock(radix->mu);
        release_subtree(radix, &radix->root);
    }
    delete radix;
    return BRC_OK;
}

brc_status brc_radix_match(brc_radix *radix, const uint32_t *tokens, uint32_t n_tokens, uint32_t *out_pages,
                           uint32_t max_pages, uint32_t *out_n_pages) {
    if (!radix || !out_n_pages || (!tokens && n_tokens) || (!out_pages && max_pages))
        return brc_fail(BRC_ERR_INVALID, "brc_radix_match: NULL argument");
    *out_n_pages = 0;
    const uint32_t pt = radix->pool->page_tokens;
    std::lock_guard<std::mutex> lock(radix->mu);
    brc_radix_node *n = &radix->root;
    uint32_t got = 0;
    std::vector<uint32_t> key(pt);
    const uint64_t now = ++radix->clock;
    while (got < max_pages && (uint64_t)(got + 1) * pt <= n_tokens) {
        std::memcpy(key.data(), tokens + (size_t)got * pt, pt * sizeof(uint32_t));
        auto it = n->children.find(key);
        if (it == n->children.end()) break;
        n = it->second.get();
        n->tick = now;
        out_pages[got++] = n->page;
    }
    if (got) {
        if (brc_status rc = brc_pages_retain(radix->pool, out_pages, got)) return rc;
        radix->hits += got;
    }
    radix->misses += n_tokens / pt > got ? n_tokens / pt - got : 0;
    *out_n_pages = got;
    return BRC_OK;
}

brc_status brc_radix_insert(brc_radix *radix, const uint32_t *tokens, uint32_t n_tokens, const uint32_t *pages,
                            uint32_t n_pages, uint32_t *out_n_new) {
    if (!radix || (!tokens && n_tokens) || (!pages && n_pages))
        return brc_fail(BRC_ERR_INVALID, "brc_radix_insert: NULL argument");
    if (out_n_new) *out_n_new = 0;
    const uint32_t pt = radix->pool->page_tokens;
    const uint32_t full = std::min<uint32_t>(n_tokens / pt, n_pages);
    std::lock_guard<std::mutex> lock(radix->mu);
    brc_radix_node *n = &radix->root;
    std::vector<uint32_t> key(pt);
    const uint64_t now = ++radix->clock;
    uint32_t added = 0;
    for (uint32_t i = 0; i < full; ++i) {
        std::memcpy(key.data(), tokens + (size_t)i * pt, pt * sizeof(uint32_t));
        auto it = n->children.find(key);
        if (it == n->children.end()) {
            // the tree takes its own reference; refused if the caller does not hold the page
            if (brc_status rc = brc_pages_retain(radix->pool, pages + i, 1)) return rc;
            tree_mark(radix->pool, pages[i], +1);
            std::unique_ptr<brc_radix_node> child(new brc_radix_node());
            child->key = key;
            child->page = pages[i];
            child->parent = n;
            it = n->children.emplace(key, std::move(child)).first;
            ++radix->n_nodes;
            ++added;
        }
        n = it->second.get();
        n->tick = now;
    }
    if (out_n_new) *out_n_new = added;
    return BRC_OK;
}

brc_status brc_radix_evict(brc_radix *radix, uint32_t n_pages, uint32_t *out_n_evicted) {
    if (!radix) return brc_fail(BRC_ERR_INVALID, "brc_radix_evict: radix is NULL");
    if (out_n_evicted) *out_n_evicted = 0;
    std::lock_guard<std::mutex> lock(radix->mu);
    uint32_t done = 0;
    while (done < n_pages) {
        // least recently used leaf whose page only the tree still holds
        std::vector<brc_radix_node *> leaves;
        collect_leaves(&radix->root, leaves);
        brc_radix_node *victim = nullptr;
        for (brc_radix_node *leaf : leaves) {
            uint32_t rc = 0;
            if (brc_page_refcount(radix->pool, leaf->page, &rc) != BRC_OK || rc != 1) continue;
            if (!victim || leaf->tick < victim->tick) victim = leaf;
        }
        if (!victim) break;
        tree_mark(radix->pool, victim->page, -1);
        brc_pages_release(radix->pool, &victim->page, 1);
        brc_radix_node *parent = victim->parent;
        const std::vector<uint32_t> key = victim->key;  // the node dies inside erase
        parent->children.erase(key);
        --radix->n_nodes;
        ++radix->evictions;
        ++done;
    }
    if (out_n_evicted) *out_n_evicted = done;
    return BRC_OK;
}

brc_status brc_radix_release(brc_radix *radix, const uint32_t *pages, uint32_t n_pages) {
    if (!radix) return brc_fail(BRC_ERR_INVALID, "brc_radix_release: radix is NULL");
    return brc_pages_release(radix->pool, pages, n_pages);
}

brc_status brc_radix_prefix_tags(const uint32_t *tokens, uint32_t n_tokens, uint32_t page_tokens, uint64_t *out_tags,
                                 uint32_t capacity, uint32_t *out_n) {
    if (!out_n || (!tokens && n_tokens) || page_tokens == 0) return brc_fail(BRC_ERR_INVALID, "brc_radix_prefix_tags: NULL argument or zero page size");
    const uint32_t pages = n_tokens / page_tokens;
    if (pages > capacity || (pages && !out_tags))
        return brc_fail(BRC_ERR_CAPACITY, "brc_radix_prefix_tags: %u full pages but room for %u tags", pages, capacity);
    // splitmix64 finaliser over a running state: the tag of page i depends on every token of pages 0 .. i
    uint64_t h = 0x9E3779B97F4A7C15ull;
    for (uint32_t pg = 0; pg < pages; ++pg) {
        for (uint32_t t = 0; t < page_tokens; ++t) {
            uint64_t z = h ^ ((uint64_t)tokens[(size_t)pg * page_tokens + t] + 0x9E3779B97F4A7C15ull);
            z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
            z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
            h = z ^ (z >> 31);
        }
        out_tags[pg] = h | 1ull;   // never zero: zero is the cold store's "untagged"
    }
    *out_n = pages;
    return BRC_OK;
}

brc_status brc_radix_stats(brc_radix *radix, uint64_t *out_nodes, uint64_t *out_hit_pages, uint64_t *out_miss_pages,
                           uint64_t *out_evictions) {
    if (!radix) return brc_fail(BRC_ERR_INVALID, "brc_radix_stats: radix is NULL");
    std::lock_guard<std::mutex> lock(radix->mu);
    if (out_nodes) *out_nodes = radix->n_nodes;
    if (out_hit_pages) *out_hit_pages = radix->hits;
    if (out_miss_pages) *out_miss_pages = radix->misses;
    if (out_evictions) *out_evictions = radix->evictions;
    return BRC_OK;
}

}  // extern "C"
