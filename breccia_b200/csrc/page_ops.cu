// KV append (scatter through block tables), page gather, page copy and copy-on-write fork.
// All of these are HBM-bound byte movers: 16-byte accesses, fully coalesced within a cache row
// (one row = head_dim binary16 = 512 B at head_dim 256), grids sized from the work.
#include <algorithm>
#include <vector>

#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

struct AppendParams {
    uint8_t *k_layer;  // this layer's K pool
    uint8_t *v_layer;
    const uint32_t *block_tables;
    const uint32_t *pos0;
    const uint32_t *cu_tokens;  // nullable
    const void *k_src;
    const void *v_src;
    uint32_t *status;
    uint32_t table_stride, n_seqs, tokens_per_seq, total_tokens, max_pos_end;
    uint32_t n_kv_head, head_dim, page_tokens, n_pages;
};

// Largest s with cu[s] <= t  (cu has n+1 ascending entries, cu[0] = 0, cu[n] = total).
__device__ __forceinline__ uint32_t seq_of_token(const uint32_t *cu, uint32_t n, uint32_t t) {
    uint32_t lo = 0, hi = n;  // answer in [lo, hi)
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// One thread moves 8 consecutive elements (16 B of cache) of K and of V for one (token, kv head).
// The address rule is the reference's (shaders/qsa_kv_append.comp:137-161):
//   cell = pos0 + t, page = table[cell / page_tokens],
//   element = ((page * n_kv + kvh) * page_tokens + cell % page_tokens) * head_dim + d.
// V_Q8: the V row is stored as q8_0 instead (store rule of shaders/qsa_kv_append.comp:117-133): per block of
// 32 values scale = amax / 127 (1 for an all-zero block), q = round-half-away(clamp(x / scale, +-127)), taken
// from the f32 value; a block is one f32 scale then 32 signed bytes.  The four threads that share a block each
// read all of it for the maximum (the repeats hit L1) and quantise their own eight values.
template <bool SRC_F32, bool V_Q8>
__global__ void __launch_bounds__(256) kv_append_kernel(const AppendParams p) {
    const uint32_t vec_per_row = p.head_dim / 8u;
    const uint32_t vec_per_token = p.n_kv_head * vec_per_row;
    const uint64_t total = (uint64_t)p.total_tokens * vec_per_token;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t tok = (uint32_t)(i / vec_per_token);
        const uint32_t r = (uint32_t)(i % vec_per_token);
        const uint32_t kvh = r / vec_per_row;
        const uint32_t v8 = r % vec_per_row;
        uint32_t s, t;
        if (p.cu_tokens) {
            s = seq_of_token(p.cu_tokens, p.n_seqs, tok);
            t = tok - p.cu_tokens[s];
        } else {
            s = tok / p.tokens_per_seq;
            t = tok % p.tokens_per_seq;
        }
        const uint32_t cell = p.pos0[s] + t;
        if (cell >= p.max_pos_end) {
            if (r == 0) { atomicOr(p.status, BRC_DEV_BAD_POS); p.status[1] = cell; }
            continue;
        }
        const uint32_t page = p.block_tables[(uint64_t)s * p.table_stride + cell / p.page_tokens];
        if (page >= p.n_pages) {
            if (r == 0) { atomicOr(p.status, BRC_DEV_BAD_PAGE); p.status[1] = page; }
            continue;
        }
        const uint64_t row = ((uint64_t)page * p.n_kv_head + kvh) * p.page_tokens + cell % p.page_tokens;
        const uint64_t dst = (row * p.head_dim + (uint64_t)v8 * 8u) * 2u;  // bytes
        const uint64_t src = ((uint64_t)tok * p.n_kv_head + kvh) * p.head_dim + (uint64_t)v8 * 8u;  // elements
        uint4 ko, vo;
        if (V_Q8) {
            const float *vrow = static_cast<const float *>(p.v_src) + src - (uint64_t)(v8 & 3u) * 8u;   // the block's 32 values
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 x = __ldg(reinterpret_cast<const float4 *>(vrow) + j);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
            }
            const float scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
            const float4 a = __ldg(reinterpret_cast<const float4 *>(vrow) + 2u * (v8 & 3u));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(vrow) + 2u * (v8 & 3u) + 1);
            auto quant = [scale](float x) {
                return (uint32_t)(int32_t)roundf(fminf(fmaxf(__fdiv_rn(x, scale), -127.f), 127.f)) & 0xffu;
            };
            const uint32_t w0 = quant(a.x) | (quant(a.y) << 8) | (quant(a.z) << 16) | (quant(a.w) << 24);
            const uint32_t w1 = quant(b.x) | (quant(b.y) << 8) | (quant(b.z) << 16) | (quant(b.w) << 24);
            uint32_t *blk = reinterpret_cast<uint32_t *>(p.v_layer) + (row * (p.head_dim / 32u) + (v8 >> 2)) * 9u;
            if ((v8 & 3u) == 0u) blk[0] = __float_as_uint(scale);
            blk[1u + 2u * (v8 & 3u)] = w0;
            blk[2u + 2u * (v8 & 3u)] = w1;
        }
        if (SRC_F32) {
            const float4 *ks = reinterpret_cast<const float4 *>(static_cast<const float *>(p.k_src) + src);
            const float4 *vs = reinterpret_cast<const float4 *>(static_cast<const float *>(p.v_src) + src);
            const float4 k0 = __ldg(ks), k1 = __ldg(ks + 1), v0 = __ldg(vs), v1 = __ldg(vs + 1);
            ko = make_uint4(brc::pack_f16x2(k0.x, k0.y), brc::pack_f16x2(k0.z, k0.w), brc::pack_f16x2(k1.x, k1.y),
                            brc::pack_f16x2(k1.z, k1.w));
            vo = make_uint4(brc::pack_f16x2(v0.x, v0.y), brc::pack_f16x2(v0.z, v0.w), brc::pack_f16x2(v1.x, v1.y),
                            brc::pack_f16x2(v1.z, v1.w));
        } else {
            // binary16 sources: stored as they are except that an exponent field of zero becomes a
            // signed zero, which is what the reference's loader would read anyway
            // (shaders/f16_storage.glsl:62-64) and keeps the pool free of subnormals.
            ko = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.k_src) + src));
            vo = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.v_src) + src));
            auto flush = [](uint32_t w) {
                if ((w & 0x7c00u) == 0u) w &= 0xffff8000u;
                if ((w & 0x7c000000u) == 0u) w &= 0x8000ffffu;
                return w;
            };
            ko = make_uint4(flush(ko.x), flush(ko.y), flush(ko.z), flush(ko.w));
            vo = make_uint4(flush(vo.x), flush(vo.y), flush(vo.z), flush(vo.w));
        }
        *reinterpret_cast<uint4 *>(p.k_layer + dst) = ko;
        if (!V_Q8) *reinterpret_cast<uint4 *>(p.v_layer + dst) = vo;
    }
}

// Gather one sequence's cells into logical [cell][kv_head][d] arrays; one thread per 16 bytes.
__global__ void __launch_bounds__(256)
    page_gather_kernel(const uint8_t *k_layer, const uint8_t *v_layer, const uint32_t *block_table, uint32_t n_tokens,
                       uint32_t n_kv_head, uint32_t head_dim, uint32_t page_tokens, uint32_t n_pages, uint4 *k_out,
                       uint4 *v_out, uint32_t *status) {
    const uint32_t vec_per_row = head_dim / 8u;
    const uint32_t vec_per_token = n_kv_head * vec_per_row;
    const uint64_t total = (uint64_t)n_tokens * vec_per_token;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t cell = (uint32_t)(i / vec_per_token);
        const uint32_t r = (uint32_t)(i % vec_per_token);
        const uint32_t kvh = r / vec_per_row;
        const uint32_t v8 = r % vec_per_row;
        const uint32_t page = block_table[cell / page_tokens];
        if (page >= n_pages) {
            if (r == 0) { atomicOr(status, BRC_DEV_BAD_PAGE); status[1] = page; }
            continue;
        }
        const uint64_t row = ((uint64_t)page * n_kv_head + kvh) * page_tokens + cell % page_tokens;
        const uint64_t src = (row * head_dim + (uint64_t)v8 * 8u) * 2u;
        k_out[i] = *reinterpret_cast<const uint4 *>(k_layer + src);
        v_out[i] = *reinterpret_cast<const uint4 *>(v_layer + src);
    }
}

// The same for ONE of K / V with rows of `row_bytes` (a multiple of 16): the V rows of a q8_0 pool are
// head_dim / 32 blocks of 36 bytes and come out as they are stored.
__global__ void __launch_bounds__(256)
    row_gather_kernel(const uint8_t *layer_base, uint32_t row_bytes, const uint32_t *block_table, uint32_t n_tokens, uint32_t n_kv_head,
                      uint32_t page_tokens, uint32_t n_pages, uint4 *out, uint32_t *status) {
    const uint32_t vec_per_row = row_bytes / 16u;
    const uint32_t vec_per_token = n_kv_head * vec_per_row;
    const uint64_t total = (uint64_t)n_tokens * vec_per_token;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t cell = (uint32_t)(i / vec_per_token);
        const uint32_t r = (uint32_t)(i % vec_per_token);
        const uint32_t kvh = r / vec_per_row, vec = r % vec_per_row;
        const uint32_t page = block_table[cell / page_tokens];
        if (page >= n_pages) {
            if (r == 0) { atomicOr(status, BRC_DEV_BAD_PAGE); status[1] = page; }
            continue;
        }
        const uint64_t row = ((uint64_t)page * n_kv_head + kvh) * page_tokens + cell % page_tokens;
        out[i] = *reinterpret_cast<const uint4 *>(layer_base + row * row_bytes + (uint64_t)vec * 16u);
    }
}

// Whole-page copies in every layer, K and V.  blockIdx.y = pair; the x dimension strides over the
// (layer, K|V, 16-byte vector) space of one page.  The V half of a page may be smaller than the K half
// (q8_0 bodies: 9/16 of it); both are whole numbers of 16-byte vectors.
__global__ void __launch_bounds__(256)
    page_copy_kernel(uint8_t *k_base, uint8_t *v_base, const uint32_t *src_ids, const uint32_t *dst_ids, uint32_t n_layers,
                     uint32_t n_pages, uint64_t half_page_bytes, uint64_t layer_bytes, uint64_t v_half_page_bytes,
                     uint64_t v_layer_bytes, uint32_t *status) {
    const uint32_t pair = blockIdx.y;
    const uint32_t s = src_ids[pair], d = dst_ids[pair];
    if (s >= n_pages || d >= n_pages) {
        if (threadIdx.x == 0 && blockIdx.x == 0) { atomicOr(status, BRC_DEV_BAD_PAGE); status[1] = s >= n_pages ? s : d; }
        return;
    }
    if (s == d) return;
    const uint32_t vec_k = (uint32_t)(half_page_bytes / 16u), vec_v = (uint32_t)(v_half_page_bytes / 16u);
    const uint64_t total = (uint64_t)n_layers * (vec_k + vec_v);
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t layer = (uint32_t)(i / (vec_k + vec_v));
        const uint32_t r = (uint32_t)(i % (vec_k + vec_v));
        const bool is_v = r >= vec_k;
        const uint32_t v = is_v ? r - vec_k : r;
        uint8_t *lay = is_v ? v_base + (uint64_t)layer * v_layer_bytes : k_base + (uint64_t)layer * layer_bytes;
        const uint64_t page_bytes = is_v ? v_half_page_bytes : half_page_bytes;
        const uint4 *sp = reinterpret_cast<const uint4 *>(lay + (uint64_t)s * page_bytes);
        uint4 *dp = reinterpret_cast<uint4 *>(lay + (uint64_t)d * page_bytes);
        dp[v] = sp[v];
    }
}

uint32_t grid_for(uint64_t work_items, uint32_t block, int sm_count, uint32_t per_sm) {
    const uint64_t need = (work_items + block - 1) / block;
    const uint64_t cap = (uint64_t)(sm_count > 0 ? sm_count : 148) * per_sm;
    return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(need, cap));
}

brc_status need_device_pool(const brc_pool *pool, const char *who) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "%s: pool is NULL", who);
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "%s: this pool holds bookkeeping only (no device memory); compute calls need a GPU pool",
                        who);
    return BRC_OK;
}

}  // namespace

extern "C" {

brc_status brc_kv_append(brc_pool *pool, uint32_t layer, const uint32_t *block_tables_dev, uint32_t table_stride,
                         const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t tokens_per_seq,
                         const uint32_t *cu_tokens_dev, uint32_t total_tokens, uint32_t max_pos_end,
                         const void *k_src_dev, const void *v_src_dev, int32_t src_dtype, void *stream) {
    if (brc_status rc = need_device_pool(pool, "brc_kv_append")) return rc;
    if (pool->v_q8 && src_dtype != BRC_DTYPE_F32)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_kv_append: a q8_0 V pool quantises from f32 sources only (src_dtype %d)", src_dtype);
    if (layer >= pool->n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_kv_append: layer %u but the pool has %u", layer, pool->n_layers);
    if (!block_tables_dev || !pos0_dev || !k_src_dev || !v_src_dev)
        return brc_fail(BRC_ERR_INVALID, "brc_kv_append: NULL block table, position or source pointer");
    if (src_dtype != BRC_DTYPE_F32 && src_dtype != BRC_DTYPE_F16)
        return brc_fail(BRC_ERR_INVALID, "brc_kv_append: src_dtype %d is neither f32 (0) nor f16 (1)", src_dtype);
    if (!cu_tokens_dev && (uint64_t)n_seqs * tokens_per_seq != total_tokens)
        return brc_fail(BRC_ERR_INVALID, "brc_kv_append: %u sequences x %u tokens != total_tokens %u", n_seqs,
                        tokens_per_seq, total_tokens);
    const uint64_t capacity = (uint64_t)table_stride * pool->page_tokens;
    if (max_pos_end > capacity)
        return brc_fail(BRC_ERR_CAPACITY,
                        "kv_append would write cells up to %u but each block table holds %llu (%u pages of %u cells): "
                        "a write past the table would read an unmapped page id",
                        max_pos_end, (unsigned long long)capacity, table_stride, pool->page_tokens);
    if (total_tokens == 0 || n_seqs == 0) return BRC_OK;
    brc_device_guard guard(pool->device);
    AppendParams p;
    p.k_layer = pool->k_base + (uint64_t)layer * pool->layer_bytes;
    p.v_layer = pool->v_base + (uint64_t)layer * pool->v_layer_bytes;
    p.block_tables = block_tables_dev;
    p.pos0 = pos0_dev;
    p.cu_tokens = cu_tokens_dev;
    p.k_src = k_src_dev;
    p.v_src = v_src_dev;
    p.status = pool->status_dev;
    p.table_stride = table_stride;
    p.n_seqs = n_seqs;
    p.tokens_per_seq = tokens_per_seq ? tokens_per_seq : 1;
    p.total_tokens = total_tokens;
    p.max_pos_end = max_pos_end;
    p.n_kv_head = pool->n_kv_head;
    p.head_dim = pool->head_dim;
    p.page_tokens = pool->page_tokens;
    p.n_pages = pool->n_pages;
    const uint64_t work = (uint64_t)total_tokens * pool->n_kv_head * (pool->head_dim / 8u);
    const uint32_t grid = grid_for(work, 256, pool->sm_count, 8);
    brc_stage_begin(pool, BRC_STAGE_KV_APPEND, brc_stream(stream));
    if (pool->v_q8)
        kv_append_kernel<true, true><<<grid, 256, 0, brc_stream(stream)>>>(p);
    else if (src_dtype == BRC_DTYPE_F32)
        kv_append_kernel<true, false><<<grid, 256, 0, brc_stream(stream)>>>(p);
    else
        kv_append_kernel<false, false><<<grid, 256, 0, brc_stream(stream)>>>(p);
    brc_stage_end(pool, BRC_STAGE_KV_APPEND, brc_stream(stream));
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

brc_status brc_page_gather(brc_pool *pool, uint32_t layer, const uint32_t *block_table_dev, uint32_t table_len,
                           uint32_t n_tokens, void *k_out_dev, void *v_out_dev, void *stream) {
    if (brc_status rc = need_device_pool(pool, "brc_page_gather")) return rc;
    if (layer >= pool->n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_page_gather: layer %u but the pool has %u", layer, pool->n_layers);
    if ((uint64_t)n_tokens > (uint64_t)table_len * pool->page_tokens)
        return brc_fail(BRC_ERR_CAPACITY, "page_gather of %u cells but the block table holds %llu (%u pages)", n_tokens,
                        (unsigned long long)table_len * pool->page_tokens, table_len);
    if (n_tokens == 0) return BRC_OK;
    if (!block_table_dev || !k_out_dev || !v_out_dev)
        return brc_fail(BRC_ERR_INVALID, "brc_page_gather: NULL pointer");
    brc_device_guard guard(pool->device);
    const uint64_t work = (uint64_t)n_tokens * pool->n_kv_head * (pool->head_dim / 8u);
    const uint32_t grid = grid_for(work, 256, pool->sm_count, 8);
    if (pool->v_q8) {   // K as binary16 rows, V as the stored q8_0 rows
        const uint32_t v_row = pool->head_dim / 32u * 36u;
        row_gather_kernel<<<grid, 256, 0, brc_stream(stream)>>>(pool->k_base + (uint64_t)layer * pool->layer_bytes, pool->head_dim * 2u,
                                                              block_table_dev, n_tokens, pool->n_kv_head, pool->page_tokens,
                                                              pool->n_pages, static_cast<uint4 *>(k_out_dev), pool->status_dev);
        row_gather_kernel<<<grid, 256, 0, brc_stream(stream)>>>(pool->v_base + (uint64_t)layer * pool->v_layer_bytes, v_row,
                                                              block_table_dev, n_tokens, pool->n_kv_head, pool->page_tokens,
                                                              pool->n_pages, static_cast<uint4 *>(v_out_dev), pool->status_dev);
        BRC_CUDA(cudaGetLastError());
        return BRC_OK;
    }
    page_gather_kernel<<<grid, 256, 0, brc_stream(stream)>>>(
        pool->k_base + (uint64_t)layer * pool->layer_bytes, pool->v_base + (uint64_t)layer * pool->layer_bytes,
        block_table_dev, n_tokens, pool->n_kv_head, pool->head_dim, pool->page_tokens, pool->n_pages,
        static_cast<uint4 *>(k_out_dev), static_cast<uint4 *>(v_out_dev), pool->status_dev);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

brc_status brc_page_copy(brc_pool *pool, const uint32_t *src_ids_dev, const uint32_t *dst_ids_dev, uint32_t n,
                         void *stream) {
    if (brc_status rc = need_device_pool(pool, "brc_page_copy")) return rc;
    if (n == 0) return BRC_OK;
    if (!src_ids_dev || !dst_ids_dev) return brc_fail(BRC_ERR_INVALID, "brc_page_copy: NULL id list");
    if (n > 65535u) return brc_fail(BRC_ERR_INVALID, "brc_page_copy: %u pairs in one call (limit 65535)", n);
    brc_device_guard guard(pool->device);
    const uint64_t work = (uint64_t)pool->n_layers * 2u * (pool->half_page_bytes / 16u);
    // Enough CTAs per pair to spread a single fork over the machine, fewer when many pairs run.
    uint32_t gx = (uint32_t)std::min<uint64_t>((work + 255) / 256, n >= 64 ? 4 : 48);
    dim3 grid(gx, n);
    page_copy_kernel<<<grid, 256, 0, brc_stream(stream)>>>(pool->k_base, pool->v_base, src_ids_dev, dst_ids_dev,
                                                         pool->n_layers, pool->n_pages, pool->half_page_bytes,
                                                         pool->layer_bytes, pool->v_layer_bytes / pool->n_pages,
                                                         pool->v_layer_bytes, pool->status_dev);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

brc_status brc_seq_fork(brc_pool *pool, const uint32_t *parent_table, uint32_t n_tokens, uint32_t *child_table,
                        uint32_t *out_new_page, void *stream) {
    if (!pool || (!parent_table && n_tokens) || (!child_table && n_tokens))
        return brc_fail(BRC_ERR_INVALID, "brc_seq_fork: NULL argument");
    if (out_new_page) *out_new_page = UINT32_MAX;
    const uint32_t pt = pool->page_tokens;
    const uint32_t full = n_tokens / pt;
    const bool partial = (n_tokens % pt) != 0;
    if (partial)
        if (brc_status rc = need_device_pool(pool, "brc_seq_fork (partial last page needs a device copy)")) return rc;
    for (uint32_t i = 0; i < full + (partial ? 1u : 0u); ++i)
        if (parent_table[i] >= pool->n_pages)
            return brc_fail(BRC_ERR_INVALID, "brc_seq_fork: parent table entry %u is page %u of %u", i, parent_table[i],
                            pool->n_pages);
    uint32_t fresh = UINT32_MAX;
    if (partial)
        if (brc_status rc = brc_pages_alloc(pool, 1, &fresh)) return rc;
    if (brc_status rc = brc_pages_retain(pool, parent_table, full)) {
        if (partial) brc_pages_release(pool, &fresh, 1);
        return rc;
    }
    for (uint32_t i = 0; i < full; ++i) child_table[i] = parent_table[i];
    if (partial) {
        child_table[full] = fresh;
        brc_device_guard guard(pool->device);
        cudaStream_t s = brc_stream(stream);
        // Stage the one (src, dst) pair through the pool's id buffer, ordered on the stream.
        const uint32_t pair[2] = {parent_table[full], fresh};
        cudaError_t e = cudaMemcpyAsync(pool->ids_dev, pair, sizeof pair, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);  // `pair` lives on this stack frame
        if (e != cudaSuccess) {
            brc_pages_release(pool, parent_table, full);
            brc_pages_release(pool, &fresh, 1);
            return brc_fail(BRC_ERR_CUDA, "brc_seq_fork: staging the page pair failed: %s", cudaGetErrorString(e));
        }
        if (brc_status rc = brc_page_copy(pool, pool->ids_dev, pool->ids_dev + 1, 1, stream)) return rc;
        if (out_new_page) *out_new_page = fresh;
    }
    return BRC_OK;
}

}  // extern "C"
