// Tiered paging of KV pages between HBM and pinned host memory on a side stream.
//
// The reference has no KV tiering (docs/plan/BRECCIA-PLAN.md:52-56: Phase 6 / M5, not started); its
// only analogue is the H2D transfer ring (crates/breccia-vk/src/transfer.rs:120-138, 247-369) and the
// rules of its design note: only complete pages move, a page is in exactly one tier, promotion is
// asynchronous and off the decode critical path, all layers of a page move together
// (docs/reference-engines/02-kv-and-context.md:543-581, 617-626).  Here:
//   * the host tier is one pinned allocation of `host_pages` slots; a slot holds a page of every
//     layer, K then V ([K: layer][half page] [V: layer][half page] = 2 * n_layers * half_page_bytes);
//   * demote packs the pages of a batch (24 separate 16 KiB pieces each at 12 layers) into a staging
//     buffer in HBM with one kernel, then copies staging -> slots with one cudaMemcpyAsync per run of
//     neighbouring slots (free slots are handed out lowest first, so a batch is mostly one run), on the
//     tier's own stream; it releases the HBM pages and hands back the slots;
//   * promote allocates fresh HBM pages, copies slots -> staging (one copy per run of neighbouring
//     slots) and scatters staging -> pages with one kernel; the caller patches its block tables;
//   * brc_tier_fence makes another stream wait for every copy issued so far.  A freed HBM page may be
//     handed out again at once by the allocator: whoever writes it must fence first;
//   * an LRU helper ranks resident pages by the last brc_tier_touch.
// Copies of whole 384 KiB slots keep the copy engine near the link's rate; a strided copy per
// (page, K|V) measured 26 GB/s on the same box.
#include <algorithm>
#include <new>
#include <set>
#include <vector>

#include "brc_internal.h"

struct brc_tier {
    brc_pool *pool = nullptr;
    uint8_t *host = nullptr;        // pinned
    uint32_t host_pages = 0;
    uint64_t slot_bytes = 0;
    cudaStream_t stream = nullptr;  // side stream of the tier
    cudaEvent_t event = nullptr;    // recorded after every batch
    std::mutex mu;
    std::set<uint32_t> free_slots;  // handed out lowest first: batches land on neighbouring slots
    uint8_t *staging = nullptr;     // HBM, STAGE_PAGES slots
    std::vector<uint8_t> slot_used;
    std::vector<uint64_t> last_use;  // per HBM page, 0 = never touched
    uint64_t clock = 0;
    uint64_t demoted_pages = 0, promoted_pages = 0, d2h_bytes = 0, h2d_bytes = 0;
};

namespace {

constexpr uint32_t STAGE_PAGES = 256;   // pages per staging pass (96 MiB at 12 layers, 2 kv heads, head_dim 256)

struct PageList {
    uint32_t ids[STAGE_PAGES];
};

// One CTA per (page of the batch, layer, K|V): a 16-byte-vector copy of one half page between the pool
// and staging slot `i` ([K: layer][half page] [V: layer][half page]).
template <bool TO_STAGING>
__global__ void __launch_bounds__(256) tier_pack_kernel(uint8_t *k_base, uint8_t *v_base, uint8_t *staging, const PageList pages,
                                                        uint32_t n_layers, uint64_t half_page_bytes, uint64_t layer_bytes) {
    const uint32_t i = blockIdx.x / (2u * n_layers), piece = blockIdx.x % (2u * n_layers);
    const bool is_v = piece >= n_layers;
    const uint32_t layer = is_v ? piece - n_layers : piece;
    uint4 *pool = reinterpret_cast<uint4 *>((is_v ? v_base : k_base) + (uint64_t)layer * layer_bytes +
                                            (uint64_t)pages.ids[i] * half_page_bytes);
    uint4 *stage = reinterpret_cast<uint4 *>(staging + ((uint64_t)i * 2u * n_layers + piece) * half_page_bytes);
    const uint32_t n_vec = (uint32_t)(half_page_bytes / 16);
    for (uint32_t v = threadIdx.x; v < n_vec; v += 256) {
        if (TO_STAGING)
            stage[v] = pool[v];
        else
            pool[v] = stage[v];
    }
}

}  // namespace

extern "C" {

brc_status brc_tier_create(brc_pool *pool, uint32_t host_pages, brc_tier **out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_tier_create: NULL argument");
    *out = nullptr;
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "brc_tier_create: this pool holds bookkeeping only (no device memory)");
    if (host_pages == 0) return brc_fail(BRC_ERR_INVALID, "brc_tier_create: host_pages is 0");
    brc_device_guard guard(pool->device);
    brc_tier *t = new (std::nothrow) brc_tier();
    if (!t) return brc_fail(BRC_ERR_INVALID, "brc_tier_create: out of host memory");
    t->pool = pool;
    t->host_pages = host_pages;
    t->slot_bytes = 2ull * pool->n_layers * pool->half_page_bytes;
    cudaError_t e;
    if ((e = cudaMallocHost(&t->host, (size_t)t->slot_bytes * host_pages)) != cudaSuccess ||
        (e = cudaMalloc(&t->staging, (size_t)t->slot_bytes * STAGE_PAGES)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&t->stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&t->event, cudaEventDisableTiming)) != cudaSuccess) {
        brc_status rc = brc_fail(BRC_ERR_CUDA, "brc_tier_create: %u pinned slots of %llu bytes: %s", host_pages,
                                 (unsigned long long)t->slot_bytes, cudaGetErrorString(e));
        brc_tier_destroy(t);
        return rc;
    }
    cudaEventRecord(t->event, t->stream);
    for (uint32_t i = 0; i < host_pages; ++i) t->free_slots.insert(t->free_slots.end(), i);
    t->slot_used.assign(host_pages, 0);
    t->last_use.assign(pool->n_pages, 0);
    *out = t;
    return BRC_OK;
}

brc_status brc_tier_destroy(brc_tier *tier) {
    if (!tier) return BRC_OK;
    brc_device_guard guard(tier->pool->device);
    if (tier->stream) {
        cudaStreamSynchronize(tier->stream);
        cudaStreamDestroy(tier->stream);
    }
    if (tier->event) cudaEventDestroy(tier->event);
    if (tier->host) cudaFreeHost(tier->host);
    if (tier->staging) cudaFree(tier->staging);
    delete tier;
    return BRC_OK;
}

// Copies between staging positions [0, n) and the host slots `slots[0..n)` (ascending): one copy per
// run of neighbouring slots.
static cudaError_t copy_runs(brc_tier *t, const uint32_t *slots, uint32_t n, bool to_host) {
    for (uint32_t i = 0; i < n;) {
        uint32_t j = i + 1;
        while (j < n && slots[j] == slots[j - 1] + 1) ++j;
        uint8_t *h = t->host + (uint64_t)slots[i] * t->slot_bytes;
        uint8_t *d = t->staging + (uint64_t)i * t->slot_bytes;
        const size_t bytes = (size_t)(j - i) * t->slot_bytes;
        cudaError_t e = to_host ? cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, t->stream)
                                : cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, t->stream);
        if (e != cudaSuccess) return e;
        i = j;
    }
    return cudaSuccess;
}

static void launch_pack(brc_tier *t, const PageList &pl, uint32_t n, bool to_staging) {
    brc_pool *p = t->pool;
    const uint32_t grid = n * 2u * p->n_layers;
    if (to_staging)
        tier_pack_kernel<true><<<grid, 256, 0, t->stream>>>(p->k_base, p->v_base, t->staging, pl, p->n_layers, p->half_page_bytes,
                                                            p->layer_bytes);
    else
        tier_pack_kernel<false><<<grid, 256, 0, t->stream>>>(p->k_base, p->v_base, t->staging, pl, p->n_layers, p->half_page_bytes,
                                                             p->layer_bytes);
}

brc_status brc_tier_demote(brc_tier *tier, const uint32_t *page_ids, uint32_t n, uint32_t *out_slots, void *after_stream) {
    if (!tier || (!page_ids && n) || (!out_slots && n)) return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: NULL argument");
    if (n == 0) return BRC_OK;
    brc_pool *p = tier->pool;
    brc_device_guard guard(p->device);
    std::lock_guard<std::mutex> lock(tier->mu);
    if (tier->free_slots.size() < n)
        return brc_fail(BRC_ERR_CAPACITY, "brc_tier_demote: %u pages but %zu of %u host slots are free", n,
                        tier->free_slots.size(), tier->host_pages);
    for (uint32_t i = 0; i < n; ++i) {
        uint32_t rc = 0;
        if (brc_status st = brc_page_refcount(p, page_ids[i], &rc)) return st;
        if (rc != 1)
            return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: page %u has %u holders; only a page with exactly one holder "
                                             "(the caller) can leave HBM", page_ids[i], rc);
    }
    // the copies must see everything `after_stream` has written to these pages so far
    if (after_stream) {
        cudaEvent_t ev;
        BRC_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        BRC_CUDA(cudaEventRecord(ev, brc_stream(after_stream)));
        BRC_CUDA(cudaStreamWaitEvent(tier->stream, ev, 0));
        BRC_CUDA(cudaEventDestroy(ev));
    }
    for (uint32_t i0 = 0; i0 < n; i0 += STAGE_PAGES) {
        const uint32_t m = std::min(STAGE_PAGES, n - i0);
        PageList pl;
        uint32_t slots[STAGE_PAGES];
        auto it = tier->free_slots.begin();
        for (uint32_t i = 0; i < m; ++i, ++it) {
            pl.ids[i] = page_ids[i0 + i];
            slots[i] = *it;   // ascending
        }
        launch_pack(tier, pl, m, true);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = copy_runs(tier, slots, m, true);
        if (e != cudaSuccess) return brc_fail(BRC_ERR_CUDA, "brc_tier_demote: copy of %u pages failed: %s", m, cudaGetErrorString(e));
        for (uint32_t i = 0; i < m; ++i) {
            tier->free_slots.erase(slots[i]);
            tier->slot_used[slots[i]] = 1;
            out_slots[i0 + i] = slots[i];
            tier->last_use[page_ids[i0 + i]] = 0;
        }
    }
    BRC_CUDA(cudaEventRecord(tier->event, tier->stream));
    tier->demoted_pages += n;
    tier->d2h_bytes += (uint64_t)n * tier->slot_bytes;
    // the HBM pages go back to the allocator; their next writer must brc_tier_fence first
    return brc_pages_release(p, page_ids, n);
}

brc_status brc_tier_promote(brc_tier *tier, const uint32_t *slots, uint32_t n, uint32_t *out_page_ids) {
    if (!tier || (!slots && n) || (!out_page_ids && n)) return brc_fail(BRC_ERR_INVALID, "brc_tier_promote: NULL argument");
    if (n == 0) return BRC_OK;
    brc_pool *p = tier->pool;
    brc_device_guard guard(p->device);
    std::lock_guard<std::mutex> lock(tier->mu);
    for (uint32_t i = 0; i < n; ++i) {
        if (slots[i] >= tier->host_pages || tier->slot_used[slots[i]] != 1) {
            for (uint32_t j = 0; j < i; ++j) tier->slot_used[slots[j]] = 1;
            return brc_fail(BRC_ERR_NOT_RESIDENT, "brc_tier_promote: host slot %u holds no page (or is listed twice)", slots[i]);
        }
        tier->slot_used[slots[i]] = 2;   // claimed by this call
    }
    if (brc_status rc = brc_pages_alloc(p, n, out_page_ids)) {
        for (uint32_t i = 0; i < n; ++i) tier->slot_used[slots[i]] = 1;
        return rc;
    }
    for (uint32_t i0 = 0; i0 < n; i0 += STAGE_PAGES) {
        const uint32_t m = std::min(STAGE_PAGES, n - i0);
        // staging order = ascending slot order, so that neighbouring slots arrive with one copy
        uint32_t order[STAGE_PAGES], sorted[STAGE_PAGES];
        for (uint32_t i = 0; i < m; ++i) order[i] = i0 + i;
        std::sort(order, order + m, [&](uint32_t a, uint32_t b) { return slots[a] < slots[b]; });
        PageList pl;
        for (uint32_t i = 0; i < m; ++i) {
            sorted[i] = slots[order[i]];
            pl.ids[i] = out_page_ids[order[i]];
        }
        cudaError_t e = copy_runs(tier, sorted, m, false);
        if (e == cudaSuccess) {
            launch_pack(tier, pl, m, false);
            e = cudaGetLastError();
        }
        if (e != cudaSuccess) return brc_fail(BRC_ERR_CUDA, "brc_tier_promote: copy of %u slots failed: %s", m, cudaGetErrorString(e));
        for (uint32_t i = 0; i < m; ++i) {
            tier->slot_used[sorted[i]] = 0;
            tier->free_slots.insert(sorted[i]);
            tier->last_use[pl.ids[i]] = ++tier->clock;
        }
    }
    BRC_CUDA(cudaEventRecord(tier->event, tier->stream));
    tier->promoted_pages += n;
    tier->h2d_bytes += (uint64_t)n * tier->slot_bytes;
    return BRC_OK;
}

brc_status brc_tier_fence(brc_tier *tier, void *stream) {
    if (!tier) return brc_fail(BRC_ERR_INVALID, "brc_tier_fence: tier is NULL");
    brc_device_guard guard(tier->pool->device);
    std::lock_guard<std::mutex> lock(tier->mu);
    BRC_CUDA(cudaStreamWaitEvent(brc_stream(stream), tier->event, 0));
    return BRC_OK;
}

brc_status brc_tier_sync(brc_tier *tier) {
    if (!tier) return brc_fail(BRC_ERR_INVALID, "brc_tier_sync: tier is NULL");
    brc_device_guard guard(tier->pool->device);
    BRC_CUDA(cudaStreamSynchronize(tier->stream));
    return BRC_OK;
}

brc_status brc_tier_touch(brc_tier *tier, const uint32_t *page_ids, uint32_t n) {
    if (!tier || (!page_ids && n)) return brc_fail(BRC_ERR_INVALID, "brc_tier_touch: NULL argument");
    std::lock_guard<std::mutex> lock(tier->mu);
    const uint64_t now = ++tier->clock;
    for (uint32_t i = 0; i < n; ++i) {
        if (page_ids[i] >= tier->pool->n_pages)
            return brc_fail(BRC_ERR_INVALID, "brc_tier_touch: page %u of %u", page_ids[i], tier->pool->n_pages);
        tier->last_use[page_ids[i]] = now;
    }
    return BRC_OK;
}

brc_status brc_tier_lru(brc_tier *tier, uint32_t n, uint32_t *out_page_ids, uint32_t *out_n) {
    if (!tier || !out_n || (!out_page_ids && n)) return brc_fail(BRC_ERR_INVALID, "brc_tier_lru: NULL argument");
    std::lock_guard<std::mutex> lock(tier->mu);
    // touched pages with exactly one holder, least recently touched first
    std::vector<std::pair<uint64_t, uint32_t>> cand;
    for (uint32_t pg = 0; pg < tier->pool->n_pages; ++pg) {
        if (!tier->last_use[pg]) continue;
        uint32_t rc = 0;
        if (brc_page_refcount(tier->pool, pg, &rc) != BRC_OK || rc != 1) continue;
        cand.emplace_back(tier->last_use[pg], pg);
    }
    const uint32_t k = std::min<uint32_t>(n, (uint32_t)cand.size());
    std::partial_sort(cand.begin(), cand.begin() + k, cand.end());
    for (uint32_t i = 0; i < k; ++i) out_page_ids[i] = cand[i].second;
    *out_n = k;
    return BRC_OK;
}

brc_status brc_tier_stats(brc_tier *tier, uint64_t *out_demoted_pages, uint64_t *out_promoted_pages, uint64_t *out_d2h_bytes,
                          uint64_t *out_h2d_bytes, uint32_t *out_free_slots) {
    if (!tier) return brc_fail(BRC_ERR_INVALID, "brc_tier_stats: tier is NULL");
    std::lock_guard<std::mutex> lock(tier->mu);
    if (out_demoted_pages) *out_demoted_pages = tier->demoted_pages;
    if (out_promoted_pages) *out_promoted_pages = tier->promoted_pages;
    if (out_d2h_bytes) *out_d2h_bytes = tier->d2h_bytes;
    if (out_h2d_bytes) *out_h2d_bytes = tier->h2d_bytes;
    if (out_free_slots) *out_free_slots = (uint32_t)tier->free_slots.size();
    return BRC_OK;
}

}  // extern "C"
