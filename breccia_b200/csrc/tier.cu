// Tiered paging of KV pages between HBM and pinned host memory on a side stream.
//
// The reference has no KV tiering (docs/plan/BRECCIA-PLAN.md:52-56: Phase 6 / M5, not started); its
// only analogue is the H2D transfer ring (crates/breccia-vk/src/transfer.rs:120-138, 247-369) and the
// rules of its design note: only complete pages move, a page is in exactly one tier, promotion is
// asynchronous and off the decode critical path, all layers of a page move together
// (docs/reference-engines/02-kv-and-context.md:543-581, 617-626).  Here:
//   * the host tier is one pinned allocation of `host_pages` slots; a slot holds a page of every
//     layer, K then V ([K: layer][half page] [V: layer][half page] = 2 * n_layers * half_page_bytes; on a
//     q8_0 V pool the V half pages are 9/16 of the K ones);
//   * demote packs the pages of a batch (24 separate 16 KiB pieces each at 12 layers) into a staging
//     buffer in HBM with one kernel, then copies staging -> slots with one cudaMemcpyAsync per run of
//     neighbouring slots (free slots are handed out lowest first, so a batch is mostly one run), on the
//     tier's outbound stream; it releases the HBM pages and hands back the slots;
//   * promote allocates fresh HBM pages, copies slots -> staging (one copy per run of neighbouring
//     slots) and scatters staging -> pages with one kernel; the caller patches its block tables;
//   * promotions run on a second stream with a staging buffer of their own, so the link carries both
//     directions at once; what orders the two streams is tracked per slot and per page (which batch
//     last wrote or read it) and enforced with the events of those batches, so a promotion only ever
//     waits for the demotion that filled its slots and for the pack kernel that emptied its pages;
//   * free slots are handed out in address order from a moving cursor: a batch lands on neighbouring
//     slots, and a slot that was just freed is not reused until the cursor comes round again;
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

constexpr uint32_t EVENT_RING = 64;     // batches per direction whose completion can still be waited for

struct brc_tier {
    brc_pool *pool = nullptr;
    uint8_t *host = nullptr;        // pinned
    uint32_t host_pages = 0;
    uint64_t slot_bytes = 0;
    cudaStream_t out_stream = nullptr, in_stream = nullptr;   // demotions / promotions
    uint8_t *out_staging = nullptr, *in_staging = nullptr;    // HBM, STAGE_PAGES slots each
    cudaEvent_t packed = nullptr;                             // after the newest pack kernel (pages read out)
    cudaEvent_t out_done[EVENT_RING] = {}, in_done[EVENT_RING] = {};
    uint64_t out_batch = 0, in_batch = 0;                     // batches issued so far (batch b uses ring entry b % EVENT_RING)
    std::mutex mu;
    std::vector<uint8_t> slot_used;
    std::vector<uint64_t> slot_written_by;   // demotion batch that last filled the slot
    std::vector<uint64_t> slot_read_by;      // promotion batch that last emptied it
    std::vector<uint64_t> page_written_by;   // promotion batch that last filled the HBM page
    uint32_t free_slot_count = 0, cursor = 0;
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
// and staging slot `i` ([K: layer][K half page] [V: layer][V half page]; on a q8_0 V pool the V half of a
// page is 9/16 of the K half, crates/breccia-kernels/src/qsa/mod.rs:339-349).
template <bool TO_STAGING>
__global__ void __launch_bounds__(256) tier_pack_kernel(uint8_t *k_base, uint8_t *v_base, uint8_t *staging, const PageList pages,
                                                        uint32_t n_layers, uint64_t k_half_bytes, uint64_t k_layer_bytes,
                                                        uint64_t v_half_bytes, uint64_t v_layer_bytes) {
    const uint32_t i = blockIdx.x / (2u * n_layers), piece = blockIdx.x % (2u * n_layers);
    const bool is_v = piece >= n_layers;
    const uint32_t layer = is_v ? piece - n_layers : piece;
    const uint64_t half = is_v ? v_half_bytes : k_half_bytes;
    uint4 *pool = reinterpret_cast<uint4 *>((is_v ? v_base + (uint64_t)layer * v_layer_bytes : k_base + (uint64_t)layer * k_layer_bytes) +
                                            (uint64_t)pages.ids[i] * half);
    const uint64_t slot_bytes = n_layers * (k_half_bytes + v_half_bytes);
    uint4 *stage = reinterpret_cast<uint4 *>(staging + (uint64_t)i * slot_bytes +
                                             (is_v ? n_layers * k_half_bytes + (uint64_t)layer * v_half_bytes : (uint64_t)layer * k_half_bytes));
    const uint32_t n_vec = (uint32_t)(half / 16);
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
    t->slot_bytes = (uint64_t)pool->n_layers * (pool->half_page_bytes + pool->v_layer_bytes / pool->n_pages);   // K half + V half (9/16 of it on q8_0 V)
    cudaError_t e;
    if ((e = cudaMallocHost(&t->host, (size_t)t->slot_bytes * host_pages)) != cudaSuccess ||
        (e = cudaMalloc(&t->out_staging, (size_t)t->slot_bytes * STAGE_PAGES)) != cudaSuccess ||
        (e = cudaMalloc(&t->in_staging, (size_t)t->slot_bytes * STAGE_PAGES)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&t->out_stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&t->in_stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&t->packed, cudaEventDisableTiming)) != cudaSuccess) {
        brc_status rc = brc_fail(BRC_ERR_CUDA, "brc_tier_create: %u pinned slots of %llu bytes: %s", host_pages,
                                 (unsigned long long)t->slot_bytes, cudaGetErrorString(e));
        brc_tier_destroy(t);
        return rc;
    }
    for (uint32_t i = 0; i < EVENT_RING; ++i) {
        if ((e = cudaEventCreateWithFlags(&t->out_done[i], cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&t->in_done[i], cudaEventDisableTiming)) != cudaSuccess) {
            brc_status rc = brc_fail(BRC_ERR_CUDA, "brc_tier_create: cudaEventCreate: %s", cudaGetErrorString(e));
            brc_tier_destroy(t);
            return rc;
        }
    }
    cudaEventRecord(t->packed, t->out_stream);
    cudaEventRecord(t->out_done[0], t->out_stream);   // batch 0 = nothing, complete
    cudaEventRecord(t->in_done[0], t->in_stream);
    t->slot_used.assign(host_pages, 0);
    t->slot_written_by.assign(host_pages, 0);
    t->slot_read_by.assign(host_pages, 0);
    t->page_written_by.assign(pool->n_pages, 0);
    t->free_slot_count = host_pages;
    t->last_use.assign(pool->n_pages, 0);
    *out = t;
    return BRC_OK;
}

brc_status brc_tier_destroy(brc_tier *tier) {
    if (!tier) return BRC_OK;
    brc_device_guard guard(tier->pool->device);
    for (cudaStream_t st : {tier->out_stream, tier->in_stream})
        if (st) {
            cudaStreamSynchronize(st);
            cudaStreamDestroy(st);
        }
    if (tier->packed) cudaEventDestroy(tier->packed);
    for (uint32_t i = 0; i < EVENT_RING; ++i) {
        if (tier->out_done[i]) cudaEventDestroy(tier->out_done[i]);
        if (tier->in_done[i]) cudaEventDestroy(tier->in_done[i]);
    }
    if (tier->host) cudaFreeHost(tier->host);
    if (tier->out_staging) cudaFree(tier->out_staging);
    if (tier->in_staging) cudaFree(tier->in_staging);
    delete tier;
    return BRC_OK;
}

// Copies between staging positions [0, n) and the host slots `slots[0..n)` (ascending): one copy per
// run of neighbouring slots.
static cudaError_t copy_runs(brc_tier *t, const uint32_t *slots, uint32_t n, bool to_host) {
    uint8_t *staging = to_host ? t->out_staging : t->in_staging;
    cudaStream_t st = to_host ? t->out_stream : t->in_stream;
    for (uint32_t i = 0; i < n;) {
        uint32_t j = i + 1;
        while (j < n && slots[j] == slots[j - 1] + 1) ++j;
        uint8_t *h = t->host + (uint64_t)slots[i] * t->slot_bytes;
        uint8_t *d = staging + (uint64_t)i * t->slot_bytes;
        const size_t bytes = (size_t)(j - i) * t->slot_bytes;
        cudaError_t e = to_host ? cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, st)
                                : cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return e;
        i = j;
    }
    return cudaSuccess;
}

static void launch_pack(brc_tier *t, const PageList &pl, uint32_t n, bool to_staging) {
    brc_pool *p = t->pool;
    const uint32_t grid = n * 2u * p->n_layers;
    if (to_staging)
        tier_pack_kernel<true><<<grid, 256, 0, t->out_stream>>>(p->k_base, p->v_base, t->out_staging, pl, p->n_layers,
                                                                p->half_page_bytes, p->layer_bytes, p->v_layer_bytes / p->n_pages,
                                                                p->v_layer_bytes);
    else
        tier_pack_kernel<false><<<grid, 256, 0, t->in_stream>>>(p->k_base, p->v_base, t->in_staging, pl, p->n_layers,
                                                                p->half_page_bytes, p->layer_bytes, p->v_layer_bytes / p->n_pages,
                                                                p->v_layer_bytes);
}

// Make `waiter` wait for batch `dep` of the other direction unless that batch is known to be complete:
// before ring entry b % EVENT_RING is recorded again for batch b, the host waits for batch b - EVENT_RING.
static cudaError_t wait_for_batch(cudaStream_t waiter, const cudaEvent_t *ring, uint64_t newest, uint64_t dep) {
    if (dep == 0 || dep + EVENT_RING <= newest) return cudaSuccess;
    return cudaStreamWaitEvent(waiter, ring[dep % EVENT_RING], 0);
}

static cudaError_t record_batch(cudaStream_t st, cudaEvent_t *ring, uint64_t batch) {
    cudaEvent_t ev = ring[batch % EVENT_RING];
    if (batch >= EVENT_RING) {
        cudaError_t e = cudaEventSynchronize(ev);   // batch - EVENT_RING: long done unless the host runs far ahead
        if (e != cudaSuccess) return e;
    }
    return cudaEventRecord(ev, st);
}

brc_status brc_tier_demote(brc_tier *tier, const uint32_t *page_ids, uint32_t n, uint32_t *out_slots, void *after_stream) {
    if (!tier || (!page_ids && n) || (!out_slots && n)) return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: NULL argument");
    if (n == 0) return BRC_OK;
    brc_pool *p = tier->pool;
    brc_device_guard guard(p->device);
    std::lock_guard<std::mutex> lock(tier->mu);
    if (tier->free_slot_count < n)
        return brc_fail(BRC_ERR_CAPACITY, "brc_tier_demote: %u pages but %u of %u host slots are free", n, tier->free_slot_count,
                        tier->host_pages);
    {
        // everything is validated before the first copy is queued: ids in range, no id twice, exactly one
        // holder, and that holder not a radix tree (its node would go on naming a freed page)
        std::lock_guard<std::mutex> pool_lock(p->mu);
        std::vector<uint8_t> seen(p->n_pages, 0);
        for (uint32_t i = 0; i < n; ++i) {
            const uint32_t pg = page_ids[i];
            if (pg >= p->n_pages) return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: page %u of %u", pg, p->n_pages);
            if (seen[pg]) return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: page %u is named twice", pg);
            seen[pg] = 1;
            if (p->refcount[pg] != 1)
                return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: page %u has %u holders; only a page with exactly one holder "
                                                 "(the caller) can leave HBM", pg, p->refcount[pg]);
            if (p->tree_refs[pg])
                return brc_fail(BRC_ERR_INVALID, "brc_tier_demote: page %u is held by a radix tree; evict it from the tree "
                                                 "(brc_radix_evict) before it leaves HBM", pg);
        }
    }
    // the copies must see everything `after_stream` has written to these pages so far
    if (after_stream) {
        cudaEvent_t ev;
        BRC_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        BRC_CUDA(cudaEventRecord(ev, brc_stream(after_stream)));
        BRC_CUDA(cudaStreamWaitEvent(tier->out_stream, ev, 0));
        BRC_CUDA(cudaEventDestroy(ev));
    }
    for (uint32_t i0 = 0; i0 < n; i0 += STAGE_PAGES) {
        const uint32_t m = std::min(STAGE_PAGES, n - i0);
        const uint64_t batch = tier->out_batch + 1;
        PageList pl;
        uint32_t slots[STAGE_PAGES];
        // the next m free slots from the cursor on, in address order (wrapping once at most)
        uint32_t c = tier->cursor, found = 0, wrapped_at = m;
        for (uint32_t scanned = 0; found < m && scanned < tier->host_pages; ++scanned) {
            if (!tier->slot_used[c]) slots[found++] = c;
            if (++c == tier->host_pages) {
                c = 0;
                if (found < m && wrapped_at == m) wrapped_at = found;
            }
        }
        tier->cursor = c;
        if (wrapped_at < m) std::rotate(slots, slots + wrapped_at, slots + m);   // ascending again
        uint64_t dep_read = 0, dep_write = 0;
        for (uint32_t i = 0; i < m; ++i) {
            pl.ids[i] = page_ids[i0 + i];
            dep_read = std::max(dep_read, tier->slot_read_by[slots[i]]);           // a promotion still reading the slot
            dep_write = std::max(dep_write, tier->page_written_by[pl.ids[i]]);     // a promotion still filling the page
        }
        cudaError_t e = wait_for_batch(tier->out_stream, tier->in_done, tier->in_batch, std::max(dep_read, dep_write));
        if (e == cudaSuccess) {
            launch_pack(tier, pl, m, true);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaEventRecord(tier->packed, tier->out_stream);
        if (e == cudaSuccess) e = copy_runs(tier, slots, m, true);
        if (e == cudaSuccess) e = record_batch(tier->out_stream, tier->out_done, batch);
        if (e != cudaSuccess) return brc_fail(BRC_ERR_CUDA, "brc_tier_demote: copy of %u pages failed: %s", m, cudaGetErrorString(e));
        tier->out_batch = batch;
        for (uint32_t i = 0; i < m; ++i) {
            tier->slot_used[slots[i]] = 1;
            tier->slot_written_by[slots[i]] = batch;
            out_slots[i0 + i] = slots[i];
            tier->last_use[page_ids[i0 + i]] = 0;
        }
        tier->free_slot_count -= m;
    }
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
        const uint64_t batch = tier->in_batch + 1;
        // staging order = ascending slot order, so that neighbouring slots arrive with one copy
        uint32_t order[STAGE_PAGES], sorted[STAGE_PAGES];
        for (uint32_t i = 0; i < m; ++i) order[i] = i0 + i;
        std::sort(order, order + m, [&](uint32_t a, uint32_t b) { return slots[a] < slots[b]; });
        PageList pl;
        uint64_t dep = 0;
        for (uint32_t i = 0; i < m; ++i) {
            sorted[i] = slots[order[i]];
            pl.ids[i] = out_page_ids[order[i]];
            dep = std::max(dep, tier->slot_written_by[sorted[i]]);   // the demotion that filled the slot
        }
        cudaError_t e = wait_for_batch(tier->in_stream, tier->out_done, tier->out_batch, dep);
        // the pages may have been freed by a demotion whose pack kernel has yet to read them
        if (e == cudaSuccess) e = cudaStreamWaitEvent(tier->in_stream, tier->packed, 0);
        if (e == cudaSuccess) e = copy_runs(tier, sorted, m, false);
        if (e == cudaSuccess) {
            launch_pack(tier, pl, m, false);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = record_batch(tier->in_stream, tier->in_done, batch);
        if (e != cudaSuccess) return brc_fail(BRC_ERR_CUDA, "brc_tier_promote: copy of %u slots failed: %s", m, cudaGetErrorString(e));
        tier->in_batch = batch;
        for (uint32_t i = 0; i < m; ++i) {
            tier->slot_used[sorted[i]] = 0;
            tier->slot_read_by[sorted[i]] = batch;
            tier->page_written_by[pl.ids[i]] = batch;
            tier->last_use[pl.ids[i]] = ++tier->clock;
        }
        tier->free_slot_count += m;
    }
    tier->promoted_pages += n;
    tier->h2d_bytes += (uint64_t)n * tier->slot_bytes;
    return BRC_OK;
}

brc_status brc_tier_fence(brc_tier *tier, void *stream) {
    if (!tier) return brc_fail(BRC_ERR_INVALID, "brc_tier_fence: tier is NULL");
    brc_device_guard guard(tier->pool->device);
    std::lock_guard<std::mutex> lock(tier->mu);
    BRC_CUDA(cudaStreamWaitEvent(brc_stream(stream), tier->out_done[tier->out_batch % EVENT_RING], 0));
    BRC_CUDA(cudaStreamWaitEvent(brc_stream(stream), tier->in_done[tier->in_batch % EVENT_RING], 0));
    return BRC_OK;
}

brc_status brc_tier_sync(brc_tier *tier) {
    if (!tier) return brc_fail(BRC_ERR_INVALID, "brc_tier_sync: tier is NULL");
    brc_device_guard guard(tier->pool->device);
    BRC_CUDA(cudaStreamSynchronize(tier->out_stream));
    BRC_CUDA(cudaStreamSynchronize(tier->in_stream));
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
    {
        std::lock_guard<std::mutex> pool_lock(tier->pool->mu);   // one look at all refcounts, not a lock per page
        for (uint32_t pg = 0; pg < tier->pool->n_pages; ++pg)
            if (tier->last_use[pg] && tier->pool->refcount[pg] == 1 && !tier->pool->tree_refs[pg]) cand.emplace_back(tier->last_use[pg], pg);
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
    if (out_free_slots) *out_free_slots = tier->free_slot_count;
    return BRC_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Cold store: a file of page records behind the host tier (the design note's third tier: NVMe, read
// and written in whole-page records of 2 * n_layers * half_page_bytes, 384 KiB at 12 layers;
// docs/reference-engines/02-kv-and-context.md:536-548, milestone item 5 of :617-626).  The reference has
// no code for it.  A record is byte for byte what a host slot holds, so a page goes
//     HBM --demote--> host slot --spill--> file record --fetch--> host slot --promote--> HBM
// and nothing on the way reinterprets it.  Every record carries a caller-chosen 64-bit tag (for a cached
// prefix: a hash of the tokens up to and including the page); the tag table lives in the file, so a
// later process can open the file and find a prefix's pages again (a disk-persisted prefix cache).
// File: a 4 KiB header (magic, geometry, slot count), the tag table, then the records, all on 4 KiB
// boundaries.  Plain pread / pwrite on the calling thread; both calls are synchronous.
// ---------------------------------------------------------------------------------------------
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <string>

namespace {

constexpr char COLD_MAGIC[8] = {'B', 'R', 'C', 'C', 'O', 'L', 'D', '1'};
constexpr uint64_t COLD_ALIGN = 4096;

struct ColdHeader {
    char magic[8];
    uint32_t n_layers, n_kv_head, head_dim, page_tokens;
    uint64_t slot_bytes;
    uint32_t n_slots, reserved;
};

struct ColdEntry {
    uint64_t tag;
    uint32_t used, reserved;
};

uint64_t round_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

bool write_all(int fd, const void *buf, size_t n, uint64_t off) {
    const uint8_t *p = static_cast<const uint8_t *>(buf);
    while (n) {
        const ssize_t w = pwrite(fd, p, n, (off_t)off);
        if (w < 0 && errno == EINTR) continue;
        if (w <= 0) return false;
        p += w, n -= (size_t)w, off += (uint64_t)w;
    }
    return true;
}

bool read_all(int fd, void *buf, size_t n, uint64_t off) {
    uint8_t *p = static_cast<uint8_t *>(buf);
    while (n) {
        const ssize_t r = pread(fd, p, n, (off_t)off);
        if (r < 0 && errno == EINTR) continue;
        if (r <= 0) return false;
        p += r, n -= (size_t)r, off += (uint64_t)r;
    }
    return true;
}

}  // namespace

struct brc_cold {
    brc_tier *tier = nullptr;
    int fd = -1;
    std::string path;
    uint32_t n_slots = 0;
    uint64_t table_off = 0, data_off = 0;
    std::vector<ColdEntry> table;
    uint32_t used = 0;
    uint64_t bytes_written = 0, bytes_read = 0;
    std::mutex mu;
};

static brc_status cold_flush_table(brc_cold *c) {
    if (!write_all(c->fd, c->table.data(), c->table.size() * sizeof(ColdEntry), c->table_off))
        return brc_fail(BRC_ERR_INVALID, "cold store %s: writing the tag table failed: %s", c->path.c_str(), std::strerror(errno));
    return BRC_OK;
}

extern "C" {

brc_status brc_cold_open(brc_tier *tier, const char *path, uint32_t n_slots, int32_t create, brc_cold **out) {
    if (!tier || !path || !out) return brc_fail(BRC_ERR_INVALID, "brc_cold_open: NULL argument");
    *out = nullptr;
    const brc_pool *p = tier->pool;
    ColdHeader want = {};
    std::memcpy(want.magic, COLD_MAGIC, 8);
    want.n_layers = p->n_layers;
    want.n_kv_head = p->n_kv_head;
    want.head_dim = p->head_dim;
    want.page_tokens = p->page_tokens;
    want.slot_bytes = tier->slot_bytes;
    brc_cold *c = new (std::nothrow) brc_cold();
    if (!c) return brc_fail(BRC_ERR_INVALID, "brc_cold_open: out of host memory");
    c->tier = tier;
    c->path = path;
    if (create) {
        if (n_slots == 0) {
            delete c;
            return brc_fail(BRC_ERR_INVALID, "brc_cold_open: a new store needs n_slots > 0");
        }
        c->fd = open(path, O_RDWR | O_CREAT | O_TRUNC, 0644);
        want.n_slots = n_slots;
    } else {
        c->fd = open(path, O_RDWR);
    }
    if (c->fd < 0) {
        brc_status rc = brc_fail(BRC_ERR_INVALID, "brc_cold_open: cannot open %s: %s", path, std::strerror(errno));
        delete c;
        return rc;
    }
    ColdHeader h = want;
    if (!create) {
        if (!read_all(c->fd, &h, sizeof h, 0) || std::memcmp(h.magic, COLD_MAGIC, 8) != 0) {
            close(c->fd);
            delete c;
            return brc_fail(BRC_ERR_INVALID, "brc_cold_open: %s is not a page store of this library", path);
        }
        if (h.n_layers != want.n_layers || h.n_kv_head != want.n_kv_head || h.head_dim != want.head_dim ||
            h.page_tokens != want.page_tokens || h.slot_bytes != want.slot_bytes || h.n_slots == 0) {
            close(c->fd);
            delete c;
            return brc_fail(BRC_ERR_INVALID,
                            "brc_cold_open: %s holds pages of %u layers x %u kv heads x %u x %u cells (%llu bytes each); the pool's are "
                            "%u x %u x %u x %u (%llu bytes)",
                            path, h.n_layers, h.n_kv_head, h.head_dim, h.page_tokens, (unsigned long long)h.slot_bytes, want.n_layers,
                            want.n_kv_head, want.head_dim, want.page_tokens, (unsigned long long)want.slot_bytes);
        }
    }
    c->n_slots = h.n_slots;
    c->table_off = COLD_ALIGN;
    c->data_off = c->table_off + round_up((uint64_t)c->n_slots * sizeof(ColdEntry), COLD_ALIGN);
    c->table.assign(c->n_slots, ColdEntry{0, 0, 0});
    bool ok = true;
    if (create) {
        ok = write_all(c->fd, &h, sizeof h, 0) && cold_flush_table(c) == BRC_OK &&
             ftruncate(c->fd, (off_t)(c->data_off + (uint64_t)c->n_slots * tier->slot_bytes)) == 0;
    } else {
        ok = read_all(c->fd, c->table.data(), c->table.size() * sizeof(ColdEntry), c->table_off);
        for (const ColdEntry &e : c->table) c->used += e.used ? 1u : 0u;
    }
    if (!ok) {
        brc_status rc = brc_fail(BRC_ERR_INVALID, "brc_cold_open: %s: %s", path, std::strerror(errno));
        close(c->fd);
        delete c;
        return rc;
    }
    *out = c;
    return BRC_OK;
}

brc_status brc_cold_close(brc_cold *c) {
    if (!c) return BRC_OK;
    brc_status rc = BRC_OK;
    {
        std::lock_guard<std::mutex> lock(c->mu);
        rc = cold_flush_table(c);
        if (fsync(c->fd) != 0 && rc == BRC_OK) rc = brc_fail(BRC_ERR_INVALID, "brc_cold_close: fsync of %s: %s", c->path.c_str(), std::strerror(errno));
        close(c->fd);
    }
    delete c;
    return rc;
}

brc_status brc_cold_spill(brc_cold *c, const uint32_t *host_slots, const uint64_t *tags, uint32_t n, uint32_t *out_cold_slots) {
    if (!c || (!host_slots && n) || (!out_cold_slots && n)) return brc_fail(BRC_ERR_INVALID, "brc_cold_spill: NULL argument");
    if (n == 0) return BRC_OK;
    brc_tier *t = c->tier;
    brc_device_guard guard(t->pool->device);
    std::lock_guard<std::mutex> lock(c->mu);
    std::lock_guard<std::mutex> tier_lock(t->mu);
    if (c->n_slots - c->used < n)
        return brc_fail(BRC_ERR_CAPACITY, "brc_cold_spill: %u pages but %u of %u records are free", n, c->n_slots - c->used, c->n_slots);
    uint64_t dep = 0;
    for (uint32_t i = 0; i < n; ++i) {
        if (host_slots[i] >= t->host_pages || t->slot_used[host_slots[i]] != 1)
            return brc_fail(BRC_ERR_NOT_RESIDENT, "brc_cold_spill: host slot %u holds no page", host_slots[i]);
        for (uint32_t j = 0; j < i; ++j)
            if (host_slots[j] == host_slots[i]) return brc_fail(BRC_ERR_INVALID, "brc_cold_spill: host slot %u is named twice", host_slots[i]);
        dep = std::max(dep, t->slot_written_by[host_slots[i]]);
    }
    // the demotion that filled these slots must have landed in host memory before the file reads it
    if (dep && dep + EVENT_RING > t->out_batch) BRC_CUDA(cudaEventSynchronize(t->out_done[dep % EVENT_RING]));
    uint32_t at = 0;
    for (uint32_t i = 0; i < n; ++i) {
        while (c->table[at].used) ++at;
        if (!write_all(c->fd, t->host + (uint64_t)host_slots[i] * t->slot_bytes, t->slot_bytes, c->data_off + (uint64_t)at * t->slot_bytes))
            return brc_fail(BRC_ERR_INVALID, "brc_cold_spill: write to %s failed: %s", c->path.c_str(), std::strerror(errno));
        c->table[at].tag = tags ? tags[i] : 0;
        c->table[at].used = 1;
        ++c->used;
        c->bytes_written += t->slot_bytes;
        out_cold_slots[i] = at;
        t->slot_used[host_slots[i]] = 0;
        t->slot_written_by[host_slots[i]] = 0;
        ++t->free_slot_count;
    }
    return cold_flush_table(c);
}

brc_status brc_cold_fetch(brc_cold *c, const uint32_t *cold_slots, uint32_t n, int32_t keep, uint32_t *out_host_slots) {
    if (!c || (!cold_slots && n) || (!out_host_slots && n)) return brc_fail(BRC_ERR_INVALID, "brc_cold_fetch: NULL argument");
    if (n == 0) return BRC_OK;
    brc_tier *t = c->tier;
    brc_device_guard guard(t->pool->device);
    std::lock_guard<std::mutex> lock(c->mu);
    std::lock_guard<std::mutex> tier_lock(t->mu);
    if (t->free_slot_count < n)
        return brc_fail(BRC_ERR_CAPACITY, "brc_cold_fetch: %u pages but %u of %u host slots are free", n, t->free_slot_count, t->host_pages);
    for (uint32_t i = 0; i < n; ++i)
        if (cold_slots[i] >= c->n_slots || !c->table[cold_slots[i]].used)
            return brc_fail(BRC_ERR_NOT_RESIDENT, "brc_cold_fetch: record %u of %s holds no page", cold_slots[i], c->path.c_str());
    uint32_t hs = 0;
    for (uint32_t i = 0; i < n; ++i) {
        while (t->slot_used[hs]) ++hs;
        // a promotion that emptied this slot may still be reading it
        const uint64_t dep = t->slot_read_by[hs];
        if (dep && dep + EVENT_RING > t->in_batch) BRC_CUDA(cudaEventSynchronize(t->in_done[dep % EVENT_RING]));
        if (!read_all(c->fd, t->host + (uint64_t)hs * t->slot_bytes, t->slot_bytes, c->data_off + (uint64_t)cold_slots[i] * t->slot_bytes))
            return brc_fail(BRC_ERR_INVALID, "brc_cold_fetch: read of %s failed: %s", c->path.c_str(), std::strerror(errno));
        c->bytes_read += t->slot_bytes;
        t->slot_used[hs] = 1;
        t->slot_written_by[hs] = 0;   // filled by the host, nothing on the device to wait for
        --t->free_slot_count;
        out_host_slots[i] = hs;
        if (!keep) {
            c->table[cold_slots[i]].used = 0;
            --c->used;
        }
    }
    return keep ? BRC_OK : cold_flush_table(c);
}

brc_status brc_cold_find(brc_cold *c, uint64_t tag, uint32_t *out_cold_slot) {
    if (!c || !out_cold_slot) return brc_fail(BRC_ERR_INVALID, "brc_cold_find: NULL argument");
    std::lock_guard<std::mutex> lock(c->mu);
    for (uint32_t i = 0; i < c->n_slots; ++i)
        if (c->table[i].used && c->table[i].tag == tag) {
            *out_cold_slot = i;
            return BRC_OK;
        }
    return brc_fail(BRC_ERR_NOT_RESIDENT, "brc_cold_find: no record tagged %016llx in %s", (unsigned long long)tag, c->path.c_str());
}

brc_status brc_cold_stats(brc_cold *c, uint32_t *out_used, uint32_t *out_total, uint64_t *out_bytes_written, uint64_t *out_bytes_read) {
    if (!c) return brc_fail(BRC_ERR_INVALID, "brc_cold_stats: NULL handle");
    std::lock_guard<std::mutex> lock(c->mu);
    if (out_used) *out_used = c->used;
    if (out_total) *out_total = c->n_slots;
    if (out_bytes_written) *out_bytes_written = c->bytes_written;
    if (out_bytes_read) *out_bytes_read = c->bytes_read;
    return BRC_OK;
}

}  // extern "C"
