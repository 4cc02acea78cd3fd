// The steps in front of the cache in Qsa::forward, fused into one launch per layer:
//   q_norm   (qsa_q_norm.comp:37-71: per-head RMSNorm of the query half of each head's `q | gate` block)
//   k_norm   (Qsa::k_norm, qsa/mod.rs:1051-1058: per-kv-head RMSNorm of k_cur, in place)
//   rope_q / rope_k  (ops_rope.comp:62-95: partial NEOX-paired rotary, pairs (j, j + n_rot/2), cos/sin from
//             a host-built table, dims [n_rot, head_dim) pass through)
//   kv_append        (qsa_kv_append.comp:137-161: f32 -> binary16 by the integer rule, scatter by block table)
// in the order the reference runs them (crates/breccia-kernels/src/qsa/mod.rs:1607-1617): five dispatches
// that each move a few hundred KiB become one kernel whose rows never leave the SM between the steps.
// Arithmetic is fp32 like the shaders': y = x * (1 / sqrt(mean(x^2) + eps)) * gamma, sum of squares by the
// same pairwise tree (element i adds element i + off, off = head_dim/2 .. 1); the rotation reads the
// normalised partner element from shared memory.  The stored K/V bits follow the pool's f16 rule.
#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

struct PrepareParams {
    const float *q_full;      // [tokens][n_head][q_head_stride]; the query is the first head_dim of each head's block
    const float *k_cur;       // [tokens][n_kv_head * head_dim]
    const float *v_cur;
    const float *q_gamma;     // [head_dim]
    const float *k_gamma;     // [head_dim]
    const float2 *rope;       // [max_pos][n_rot / 2] (cos, sin)
    const uint32_t *block_tables;
    const uint32_t *pos0;     // [n_seqs]
    void *q_out;              // [tokens][n_head][head_dim], f32 or binary16
    uint8_t *k_layer;         // this layer's K pool
    uint8_t *v_layer;
    uint32_t *status;
    uint32_t n_seqs, tokens_per_seq, table_stride, max_pos_end;
    uint32_t n_head, n_kv_head, q_head_stride, n_rot, max_pos, n_pages, q_out_f16;
    float eps;
};

// One CTA per row: (token, query head) | (token, kv head, K) | (token, kv head, V); thread = element.
template <int HD>
__global__ void __launch_bounds__(HD) qk_prepare_kernel(const PrepareParams p) {
    __shared__ float red[HD];
    __shared__ float y_sm[HD];
    const uint32_t tid = threadIdx.x;
    const uint32_t rows_per_token = p.n_head + 2u * p.n_kv_head;
    const uint32_t tok = blockIdx.x / rows_per_token, r = blockIdx.x % rows_per_token;
    const uint32_t s = tok / p.tokens_per_seq, t = tok % p.tokens_per_seq;
    const uint32_t pos = p.pos0[s] + t;
    if (pos >= p.max_pos_end) {   // the caller's bound: skip the row, report
        if (tid == 0) { atomicOr(p.status, BRC_DEV_BAD_POS); p.status[1] = pos; }
        return;
    }
    const bool is_q = r < p.n_head;
    const bool is_v = !is_q && r >= p.n_head + p.n_kv_head;
    const uint32_t kvh = is_q ? 0u : (r - p.n_head) % p.n_kv_head;

    float x;
    if (is_q)
        x = p.q_full[((size_t)tok * p.n_head + r) * p.q_head_stride + tid];
    else
        x = (is_v ? p.v_cur : p.k_cur)[((size_t)tok * p.n_kv_head + kvh) * HD + tid];

    float out = x;
    if (!is_v) {
        // ---- RMSNorm: the shader's tree (qsa_q_norm.comp:54-66)
        red[tid] = x * x;
        __syncthreads();
#pragma unroll
        for (uint32_t off = HD / 2; off > 0; off >>= 1) {
            if (tid < off) red[tid] += red[tid + off];
            __syncthreads();
        }
        const float inv = 1.0f / sqrtf(red[0] / (float)HD + p.eps);
        const float y = x * inv * (is_q ? p.q_gamma : p.k_gamma)[tid];
        // ---- partial NEOX rotary (ops_rope.comp:72-94); the position is clamped into the table
        y_sm[tid] = y;
        __syncthreads();
        const uint32_t hrot = p.n_rot / 2u;
        const uint32_t pi = pos < p.max_pos ? pos : p.max_pos - 1u;
        out = y;
        if (tid < hrot) {
            const float2 cs = p.rope[(size_t)pi * hrot + tid];
            out = y * cs.x - y_sm[tid + hrot] * cs.y;
        } else if (tid < p.n_rot) {
            const float2 cs = p.rope[(size_t)pi * hrot + (tid - hrot)];
            out = y_sm[tid - hrot] * cs.y + y * cs.x;
        }
    }
    if (is_q) {
        const size_t o = ((size_t)tok * p.n_head + r) * HD + tid;
        if (p.q_out_f16)
            static_cast<__half *>(p.q_out)[o] = __float2half_rn(out);
        else
            static_cast<float *>(p.q_out)[o] = out;
        return;
    }
    // ---- append: cell `pos` of sequence s through its block table
    uint32_t page = p.block_tables[(size_t)s * p.table_stride + (pos >> 4)];
    if (page >= p.n_pages) {
        if (tid == 0) { atomicOr(p.status, BRC_DEV_BAD_PAGE); p.status[1] = page; }
        return;
    }
    uint16_t *dst = reinterpret_cast<uint16_t *>(is_v ? p.v_layer : p.k_layer) +
                    (((size_t)page * p.n_kv_head + kvh) * 16u + (pos & 15u)) * HD + tid;
    *dst = (uint16_t)brc::f32_to_f16_bits(out);
}

}  // namespace

extern "C" {

brc_status brc_qk_prepare_append(brc_pool *pool, uint32_t layer, const float *q_full_dev, uint32_t q_head_stride, uint32_t n_head,
                                 const float *k_cur_dev, const float *v_cur_dev, const float *q_gamma_dev,
                                 const float *k_gamma_dev, float eps, const float *rope_table_dev, uint32_t n_rot,
                                 uint32_t max_pos, const uint32_t *block_tables_dev, uint32_t table_stride,
                                 const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t tokens_per_seq, uint32_t max_pos_end,
                                 void *q_out_dev, int32_t q_out_dtype, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: pool is NULL");
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "brc_qk_prepare_append: this pool holds bookkeeping only (no device memory)");
    if (layer >= pool->n_layers) return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: layer %u but the pool has %u", layer, pool->n_layers);
    const uint32_t hd = pool->head_dim;
    if (hd != 128 && hd != 256) return brc_fail(BRC_ERR_UNSUPPORTED, "brc_qk_prepare_append: head_dim %u (128 or 256)", hd);
    if (pool->page_tokens != 16) return brc_fail(BRC_ERR_UNSUPPORTED, "brc_qk_prepare_append: %u-cell pages (16)", pool->page_tokens);
    if (q_out_dtype != BRC_DTYPE_F32 && q_out_dtype != BRC_DTYPE_F16)
        return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: q_out_dtype %d is neither f32 (0) nor f16 (1)", q_out_dtype);
    if (n_head == 0 || n_head % pool->n_kv_head) return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: %u query heads over %u kv heads", n_head, pool->n_kv_head);
    if (q_head_stride < hd) return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: q_head_stride %u < head_dim %u", q_head_stride, hd);
    if (n_rot > hd || (n_rot & 1u) || max_pos == 0)
        return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: n_rot %u (even, <= head_dim %u), rotary table of %u positions", n_rot, hd, max_pos);
    // the reference's refusal, made on the host before any launch (qsa/mod.rs:1108-1116)
    const uint64_t capacity = (uint64_t)table_stride * pool->page_tokens;
    if (max_pos_end > capacity)
        return brc_fail(BRC_ERR_CAPACITY, "kv_append would write cells up to %u but each block table holds %llu (%u pages of %u cells)",
                        max_pos_end, (unsigned long long)capacity, table_stride, pool->page_tokens);
    if (n_seqs == 0 || tokens_per_seq == 0) return BRC_OK;
    if (!q_full_dev || !k_cur_dev || !v_cur_dev || !q_gamma_dev || !k_gamma_dev || !rope_table_dev || !block_tables_dev || !pos0_dev ||
        !q_out_dev)
        return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: NULL pointer argument");
    const uint64_t rows = (uint64_t)n_seqs * tokens_per_seq * (n_head + 2ull * pool->n_kv_head);
    if (rows > 0x7fffffffull) return brc_fail(BRC_ERR_INVALID, "brc_qk_prepare_append: %llu rows in one call", (unsigned long long)rows);
    brc_device_guard guard(pool->device);
    PrepareParams p;
    p.q_full = q_full_dev;
    p.k_cur = k_cur_dev;
    p.v_cur = v_cur_dev;
    p.q_gamma = q_gamma_dev;
    p.k_gamma = k_gamma_dev;
    p.rope = reinterpret_cast<const float2 *>(rope_table_dev);
    p.block_tables = block_tables_dev;
    p.pos0 = pos0_dev;
    p.q_out = q_out_dev;
    p.k_layer = pool->k_base + (uint64_t)layer * pool->layer_bytes;
    p.v_layer = pool->v_base + (uint64_t)layer * pool->layer_bytes;
    p.status = pool->status_dev;
    p.n_seqs = n_seqs;
    p.tokens_per_seq = tokens_per_seq;
    p.table_stride = table_stride;
    p.max_pos_end = max_pos_end;
    p.n_head = n_head;
    p.n_kv_head = pool->n_kv_head;
    p.q_head_stride = q_head_stride;
    p.n_rot = n_rot;
    p.max_pos = max_pos;
    p.n_pages = pool->n_pages;
    p.q_out_f16 = q_out_dtype == BRC_DTYPE_F16;
    p.eps = eps;
    cudaStream_t st = brc_stream(stream);
    brc_stage_begin(pool, BRC_STAGE_KV_APPEND, st);
    if (hd == 256)
        qk_prepare_kernel<256><<<(uint32_t)rows, 256, 0, st>>>(p);
    else
        qk_prepare_kernel<128><<<(uint32_t)rows, 128, 0, st>>>(p);
    brc_stage_end(pool, BRC_STAGE_KV_APPEND, st);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"
