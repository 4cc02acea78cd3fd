// Page files: the live K/V pages of one sequence and layer as raw bytes, in the reference's dump format.
//
// The reference's `dump_state` (crates/breccia-engine/src/graph.rs:2179-2231, BRECCIA_DUMP_STATE) writes,
// per attention block b after decode position pos, the first ceil((pos + 1) / 16) pages of the K pool
// and of the V pool as they sit in device memory:
//     <dir>/p<pos:06>-b<block:02>-qsa_k.bin      pages * n_kv * 16 * head_dim * 2 bytes
//     <dir>/p<pos:06>-b<block:02>-qsa_v.bin      the same for V (f16 layout), or
//     <dir>/p<pos:06>-b<block:02>-qsa_vq8.bin    pages * n_kv * 16 * head_dim / 32 * 36 bytes (q8_0 V layout, :2183-2186)
// Its page table is the identity, so "the first pages of the pool" are the sequence's logical pages in
// order.  Here the pages are scattered in a shared pool; `brc_state_dump` walks the block table, so the
// file holds the same bytes the reference would have written for the same cache contents, and
// `brc_state_load` is the way back (a persisted prefix: fill freshly allocated pages from a file pair).
// Bench / lab facility like the reference's: both calls synchronise.
#include <cstdio>
#include <string>
#include <vector>

#include "brc_internal.h"

namespace {

std::string page_file(const char *dir, uint32_t pos, uint32_t block, const char *part) {
    char name[64];
    std::snprintf(name, sizeof name, "/p%06u-b%02u-%s.bin", pos, block, part);
    return std::string(dir) + name;
}

// Bytes of the K (or V) half of a page of one layer; the V half of a q8_0 pool is 9/16 of the K half.
uint64_t half_bytes(const brc_pool *pool, bool is_v) { return is_v ? pool->v_layer_bytes / pool->n_pages : pool->half_page_bytes; }

const char *part_name(const brc_pool *pool, bool is_v) { return !is_v ? "qsa_k" : pool->v_q8 ? "qsa_vq8" : "qsa_v"; }

// Moves `n_pages` half pages between the pool (pages named by `table`, layer `layer`) and `host`.
brc_status move_pages(brc_pool *pool, bool is_v, uint32_t layer, const uint32_t *table, uint32_t n_pages, uint8_t *host,
                      bool to_host, cudaStream_t st) {
    const uint64_t half = half_bytes(pool, is_v);
    uint8_t *base = is_v ? pool->v_base + (uint64_t)layer * pool->v_layer_bytes : pool->k_base + (uint64_t)layer * pool->layer_bytes;
    for (uint32_t i = 0; i < n_pages; ++i) {
        uint8_t *dev = base + (uint64_t)table[i] * half;
        uint8_t *h = host + (uint64_t)i * half;
        if (to_host)
            BRC_CUDA(cudaMemcpyAsync(h, dev, half, cudaMemcpyDeviceToHost, st));
        else
            BRC_CUDA(cudaMemcpyAsync(dev, h, half, cudaMemcpyHostToDevice, st));
    }
    BRC_CUDA(cudaStreamSynchronize(st));
    return BRC_OK;
}

brc_status check_args(const brc_pool *pool, const char *who, uint32_t layer, const uint32_t *table, uint32_t table_len,
                      uint32_t pos, const char *dir, uint32_t *out_pages) {
    if (!pool || !dir) return brc_fail(BRC_ERR_INVALID, "%s: NULL pool or directory", who);
    if (pool->device < 0 || !pool->k_base) return brc_fail(BRC_ERR_CUDA, "%s: this pool holds bookkeeping only (no device memory)", who);
    if (layer >= pool->n_layers) return brc_fail(BRC_ERR_INVALID, "%s: layer %u but the pool has %u", who, layer, pool->n_layers);
    const uint32_t pages = pos / pool->page_tokens + 1;   // ceil((pos + 1) / page_tokens)
    if (!table || pages > table_len)
        return brc_fail(BRC_ERR_CAPACITY, "%s: position %u needs %u pages but the block table holds %u", who, pos, pages, table_len);
    for (uint32_t i = 0; i < pages; ++i)
        if (table[i] >= pool->n_pages)
            return brc_fail(BRC_ERR_INVALID, "%s: block table entry %u is page %u of %u", who, i, table[i], pool->n_pages);
    *out_pages = pages;
    return BRC_OK;
}

}  // namespace

extern "C" {

brc_status brc_state_dump(brc_pool *pool, uint32_t layer, const uint32_t *block_table_host, uint32_t table_len, uint32_t pos,
                          uint32_t block, const char *dir, void *stream) {
    uint32_t pages = 0;
    if (brc_status rc = check_args(pool, "brc_state_dump", layer, block_table_host, table_len, pos, dir, &pages)) return rc;
    brc_device_guard guard(pool->device);
    std::vector<uint8_t> host((size_t)pages * pool->half_page_bytes);
    for (int is_v = 0; is_v < 2; ++is_v) {
        host.resize((size_t)pages * half_bytes(pool, is_v != 0));
        if (brc_status rc = move_pages(pool, is_v != 0, layer, block_table_host, pages, host.data(), true, brc_stream(stream))) return rc;
        const std::string path = page_file(dir, pos, block, part_name(pool, is_v != 0));
        std::FILE *f = std::fopen(path.c_str(), "wb");
        if (!f) return brc_fail(BRC_ERR_INVALID, "brc_state_dump: cannot create %s", path.c_str());
        const size_t n = std::fwrite(host.data(), 1, host.size(), f);
        const int rc = std::fclose(f);
        if (n != host.size() || rc != 0) return brc_fail(BRC_ERR_INVALID, "brc_state_dump: short write to %s", path.c_str());
    }
    return BRC_OK;
}

brc_status brc_state_load(brc_pool *pool, uint32_t layer, const uint32_t *block_table_host, uint32_t table_len, uint32_t pos,
                          uint32_t block, const char *dir, void *stream) {
    uint32_t pages = 0;
    if (brc_status rc = check_args(pool, "brc_state_load", layer, block_table_host, table_len, pos, dir, &pages)) return rc;
    brc_device_guard guard(pool->device);
    std::vector<uint8_t> host((size_t)pages * pool->half_page_bytes);
    for (int is_v = 0; is_v < 2; ++is_v) {
        host.resize((size_t)pages * half_bytes(pool, is_v != 0));
        const std::string path = page_file(dir, pos, block, part_name(pool, is_v != 0));
        std::FILE *f = std::fopen(path.c_str(), "rb");
        if (!f) return brc_fail(BRC_ERR_INVALID, "brc_state_load: cannot open %s", path.c_str());
        const size_t n = std::fread(host.data(), 1, host.size(), f);
        const bool at_end = std::fgetc(f) == EOF;
        std::fclose(f);
        if (n != host.size() || !at_end)
            return brc_fail(BRC_ERR_INVALID, "brc_state_load: %s does not hold exactly %zu bytes (%u pages of this geometry)",
                            path.c_str(), host.size(), pages);
        if (brc_status rc = move_pages(pool, is_v != 0, layer, block_table_host, pages, host.data(), false, brc_stream(stream))) return rc;
    }
    return BRC_OK;
}

}  // extern "C"
