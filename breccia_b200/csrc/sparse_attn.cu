// Decode attention over a SELECTED set of cells: the reference's block-list contract.
//
// The reference's QSA layers do not attend densely: an indexer picks, per query row, up to 513 blocks of 4
// cells (`ids [T, max_ids]` ascending, `counts [T]`; slot r * 4 + k names cell ids[r] * 4 + k; cells past
// the row's own position are masked), and scores / softmax / weighted V run over those cells only
// (crates/breccia-kernels/src/qsa/mod.rs:620-625, 1382-1580; qsa_attn_scores.comp:8-19, 62-118;
// qsa_attn_apply.comp:85-140; the CPU statement is cpu::attend over cpu::cells_of, qsa/cpu.rs:197-257).
// This entry point takes those lists as they are.  At most ~2052 cells per row are read, so the work is
// small and latency-sized; the kernel is plain CUDA-core code:
//   one CTA per (row, query head), 8 or 16 warps; warp w takes the selected blocks w, w + warps, ...; a lane holds
//   head_dim / 32 elements of q, of the running O and of each K / V row (one 16- or 8-byte load per row);
//   the dot product is reduced by shuffles; every warp keeps an online softmax (base 2); the warps'
//   (m, l, O) are merged through shared memory; sigmoid(gate) last.
// Any number of query heads per kv head is accepted (the reference's 24q / 2kv included).
// On a pool whose V pages are q8_0 (blocks of one f32 scale + 32 signed bytes) a lane reads the scale word of its
// block and the one or two words that hold its own quanta and multiplies in registers (qsa_attn_apply.comp:69-77):
// 36 bytes cross the memory system per 32 values instead of 64.
#include "brc_device.cuh"
#include "brc_internal.h"

namespace {


struct SparseParams {
    const void *q;                 // [rows][n_head][HD], f32 or binary16
    const uint8_t *k_layer;
    const uint8_t *v_layer;
    const uint32_t *block_tables;  // [n_seqs][table_stride]
    const uint32_t *pos0;          // [n_seqs]: position of each sequence's first row
    const uint32_t *ids;           // [rows][max_ids] selected 4-cell blocks
    const uint32_t *counts;        // [rows]
    const float *gate;
    float *out;                    // [rows][n_head][HD]
    uint32_t *status;
    uint32_t rows_per_seq, table_stride, max_ids, max_pos_end;
    uint32_t n_head, n_kv_head, n_pages, q_f32, gate_head_stride;
    float scale_log2;
};

__device__ __forceinline__ float sp_sigmoid(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

// SP_WARPS: 16 when the launch has few CTAs (one decode row: every head's list is cut sixteen ways), 8 when rows x
// heads already fill the GPU (more CTAs per SM, a cheaper merge).
template <int HD, int SP_WARPS, bool V_Q8>
__global__ void __launch_bounds__(SP_WARPS * 32) sparse_attn_kernel(const SparseParams p) {
    constexpr int EPL = HD / 32;   // elements per lane: 8 (one 16-byte load of binary16) or 4
    __shared__ float part_o[SP_WARPS][HD];
    __shared__ float part_ml[SP_WARPS][2];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t head = blockIdx.x, row = blockIdx.y;
    const uint32_t s = row / p.rows_per_seq, t = row % p.rows_per_seq;
    const uint32_t pos = p.pos0[s] + t;                     // this row's own position: cells beyond it are masked
    const uint32_t kvh = (uint32_t)(((uint64_t)head * p.n_kv_head) / p.n_head);   // qsa_attn_scores.comp:79
    const bool bad_pos = pos >= p.max_pos_end;
    if (bad_pos && threadIdx.x == 0) { atomicOr(p.status, BRC_DEV_BAD_POS); p.status[1] = pos; }

    float qv[EPL];
    {
        const size_t qo = ((size_t)row * p.n_head + head) * HD + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; ++e)
            qv[e] = (p.q_f32 ? static_cast<const float *>(p.q)[qo + e] : __half2float(static_cast<const __half *>(p.q)[qo + e])) * p.scale_log2;
    }
    float m = -INFINITY, l = 0.f, o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[e] = 0.f;

    const uint32_t count = bad_pos ? 0u : min(p.counts[row], p.max_ids);
    const uint32_t *ids = p.ids + (size_t)row * p.max_ids;
    const uint32_t *table = p.block_tables + (size_t)s * p.table_stride;
    for (uint32_t r = warp; r < count; r += SP_WARPS) {
        const uint32_t cell0 = ids[r] * 4u;
        if (cell0 > pos) continue;                          // the whole block lies in the future
        const uint32_t lp = cell0 >> 4;                     // logical page of the block (4 | 16: it never straddles pages)
        uint32_t page = lp < p.table_stride ? table[lp] : 0xffffffffu;
        if (page >= p.n_pages) {
            if (lane == 0) { atomicOr(p.status, BRC_DEV_BAD_PAGE); p.status[1] = page; }
            continue;
        }
        const size_t base = (((size_t)page * p.n_kv_head + kvh) * 16u + (cell0 & 15u)) * HD + lane * EPL;
        const uint32_t n_live = min(4u, pos - cell0 + 1u);
        // the block's four K rows and four V rows are requested before anything is consumed
        float kf[4][EPL], vf[4][EPL];
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c) {
            const size_t at = (base + (size_t)min(c, n_live - 1u) * HD) * 2u;   // masked cells re-read a live one (weight 0)
            uint32_t kw[EPL / 2], vw[EPL / 2];
            if (EPL == 8) {
                const uint4 kb = *reinterpret_cast<const uint4 *>(p.k_layer + at);
                kw[0] = kb.x, kw[1] = kb.y, kw[EPL / 2 - 2] = kb.z, kw[EPL / 2 - 1] = kb.w;
            } else {
                const uint2 kb = *reinterpret_cast<const uint2 *>(p.k_layer + at);
                kw[0] = kb.x, kw[1] = kb.y;
            }
#pragma unroll
            for (int e = 0; e < EPL / 2; ++e) {
                const float2 x = __half22float2(*reinterpret_cast<const __half2 *>(&kw[e]));
                kf[c][2 * e] = x.x, kf[c][2 * e + 1] = x.y;
            }
            if (V_Q8) {
                // row of the cell in the pool, then the lane's block: EPL * lane / 32
                const size_t vrow = ((size_t)page * p.n_kv_head + kvh) * 16u + (cell0 & 15u) + min(c, n_live - 1u);
                const uint32_t *blk = reinterpret_cast<const uint32_t *>(p.v_layer) + (vrow * (HD / 32) + (lane * EPL) / 32u) * 9u;
                const float vs = __uint_as_float(blk[0]);
                const uint32_t first = 1u + ((lane * EPL) % 32u) / 4u;
#pragma unroll
                for (int w = 0; w < EPL / 4; ++w) {
                    const uint32_t packed = blk[first + w];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        vf[c][4 * w + j] = (float)(int8_t)(packed >> (8 * j)) * vs;
                }
            } else {
                if (EPL == 8) {
                    const uint4 vb = *reinterpret_cast<const uint4 *>(p.v_layer + at);
                    vw[0] = vb.x, vw[1] = vb.y, vw[EPL / 2 - 2] = vb.z, vw[EPL / 2 - 1] = vb.w;
                } else {
                    const uint2 vb = *reinterpret_cast<const uint2 *>(p.v_layer + at);
                    vw[0] = vb.x, vw[1] = vb.y;
                }
#pragma unroll
                for (int e = 0; e < EPL / 2; ++e) {
                    const float2 y = __half22float2(*reinterpret_cast<const __half2 *>(&vw[e]));
                    vf[c][2 * e] = y.x, vf[c][2 * e + 1] = y.y;
                }
            }
        }
        float sc[4];
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c) {
            sc[c] = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) sc[c] = fmaf(qv[e], kf[c][e], sc[c]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) sc[c] += __shfl_xor_sync(0xffffffffu, sc[c], off);
        }
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c)
            if (c >= n_live) sc[c] = -INFINITY;
        // online softmax, base 2 (the scale carries log2 e); cell 0 of the block is always live
        const float m_new = fmaxf(fmaxf(m, sc[0]), fmaxf(fmaxf(sc[1], sc[2]), sc[3]));
        const float f = m == -INFINITY ? 0.f : exp2f(m - m_new);
        float pr[4];
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c) pr[c] = exp2f(sc[c] - m_new);
        l = l * f + (pr[0] + pr[1]) + (pr[2] + pr[3]);
#pragma unroll
        for (int e = 0; e < EPL; ++e)
            o[e] = fmaf(pr[0], vf[0][e], fmaf(pr[1], vf[1][e], fmaf(pr[2], vf[2][e], fmaf(pr[3], vf[3][e], o[e] * f))));
        m = m_new;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) part_o[warp][lane * EPL + e] = o[e];
    if (lane == 0) { part_ml[warp][0] = m; part_ml[warp][1] = l; }
    __syncthreads();
    // merge the warps' partials: thread = output element
    for (uint32_t d = threadIdx.x; d < HD; d += SP_WARPS * 32) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < SP_WARPS; ++w)
            if (part_ml[w][1] > 0.f) M = fmaxf(M, part_ml[w][0]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < SP_WARPS; ++w) {
            if (!(part_ml[w][1] > 0.f)) continue;
            const float wt = exp2f(part_ml[w][0] - M);
            L += wt * part_ml[w][1];
            acc += wt * part_o[w][d];
        }
        float v = L > 0.f ? acc / L : 0.f;    // a row with no selected live cell yields zeros
        if (p.gate) v *= sp_sigmoid(p.gate[((size_t)row * p.n_head + head) * p.gate_head_stride + d]);
        p.out[((size_t)row * p.n_head + head) * HD + d] = v;
    }
}

}  // namespace

extern "C" {

brc_status brc_paged_sparse_attn(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype, uint32_t n_head,
                                 const float *gate_dev, uint32_t gate_head_stride, const uint32_t *block_tables_dev,
                                 uint32_t table_stride, const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t rows_per_seq,
                                 const uint32_t *ids_dev, uint32_t max_ids, const uint32_t *counts_dev, uint32_t max_pos_end,
                                 float scale, float *out_dev, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: pool is NULL");
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "brc_paged_sparse_attn: this pool holds bookkeeping only (no device memory)");
    if (layer >= pool->n_layers) return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: layer %u but the pool has %u", layer, pool->n_layers);
    const uint32_t hd = pool->head_dim;
    if (hd != 128 && hd != 256) return brc_fail(BRC_ERR_UNSUPPORTED, "brc_paged_sparse_attn: head_dim %u (128 or 256)", hd);
    if (pool->page_tokens != 16) return brc_fail(BRC_ERR_UNSUPPORTED, "brc_paged_sparse_attn: %u-cell pages (16)", pool->page_tokens);
    if (q_dtype != BRC_DTYPE_F32 && q_dtype != BRC_DTYPE_F16)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: q_dtype %d is neither f32 (0) nor f16 (1)", q_dtype);
    if (n_head == 0 || n_head % pool->n_kv_head)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: %u query heads do not divide over %u kv heads", n_head, pool->n_kv_head);
    if (gate_dev && gate_head_stride < hd)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: gate_head_stride %u < head_dim %u", gate_head_stride, hd);
    const uint64_t capacity = (uint64_t)table_stride * pool->page_tokens;
    if (max_pos_end > capacity)
        return brc_fail(BRC_ERR_CAPACITY, "brc_paged_sparse_attn would read cells up to %u but each block table holds %llu (%u pages of %u cells)",
                        max_pos_end, (unsigned long long)capacity, table_stride, pool->page_tokens);
    if (n_seqs == 0 || rows_per_seq == 0) return BRC_OK;
    if (!q_dev || !block_tables_dev || !pos0_dev || !ids_dev || !counts_dev || !out_dev || max_ids == 0)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: NULL query, block table, position, id list, count or output pointer");
    const uint64_t rows = (uint64_t)n_seqs * rows_per_seq;
    if (rows > 65535u) return brc_fail(BRC_ERR_INVALID, "brc_paged_sparse_attn: %llu rows in one call (limit 65535)", (unsigned long long)rows);
    brc_device_guard guard(pool->device);
    SparseParams p;
    p.q = q_dev;
    p.k_layer = pool->k_base + (uint64_t)layer * pool->layer_bytes;
    p.v_layer = pool->v_base + (uint64_t)layer * pool->v_layer_bytes;
    p.block_tables = block_tables_dev;
    p.pos0 = pos0_dev;
    p.ids = ids_dev;
    p.counts = counts_dev;
    p.gate = gate_dev;
    p.out = out_dev;
    p.status = pool->status_dev;
    p.rows_per_seq = rows_per_seq;
    p.table_stride = table_stride;
    p.max_ids = max_ids;
    p.max_pos_end = max_pos_end;
    p.n_head = n_head;
    p.n_kv_head = pool->n_kv_head;
    p.n_pages = pool->n_pages;
    p.q_f32 = q_dtype == BRC_DTYPE_F32;
    p.gate_head_stride = gate_head_stride;
    p.scale_log2 = scale * 1.4426950408889634f;
    const dim3 grid(n_head, (uint32_t)rows);
    cudaStream_t st = brc_stream(stream);
    brc_stage_begin(pool, BRC_STAGE_ATTN_PARTIAL, st);
    const uint64_t sms = (uint64_t)(pool->sm_count > 0 ? pool->sm_count : 148);
    const bool few = rows * n_head < 2u * sms;
    if (pool->v_q8) {
        if (hd == 256) {
            if (few) sparse_attn_kernel<256, 16, true><<<grid, 512, 0, st>>>(p);
            else sparse_attn_kernel<256, 8, true><<<grid, 256, 0, st>>>(p);
        } else {
            if (few) sparse_attn_kernel<128, 16, true><<<grid, 512, 0, st>>>(p);
            else sparse_attn_kernel<128, 8, true><<<grid, 256, 0, st>>>(p);
        }
    } else if (hd == 256) {
        if (few) sparse_attn_kernel<256, 16, false><<<grid, 512, 0, st>>>(p);
        else sparse_attn_kernel<256, 8, false><<<grid, 256, 0, st>>>(p);
    } else {
        if (few) sparse_attn_kernel<128, 16, false><<<grid, 512, 0, st>>>(p);
        else sparse_attn_kernel<128, 8, false><<<grid, 256, 0, st>>>(p);
    }
    brc_stage_end(pool, BRC_STAGE_ATTN_PARTIAL, st);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"
