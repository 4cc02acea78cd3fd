// The steps in front of the cache in Qsa::forward, fused into one launch per layer:
//   q_norm   (qsa_q_norm.comp:37-71: per-head RMSNorm of the query half of each head's `q | gate` block)
//   k_norm   (Qsa::k_norm, qsa/mod.rs:1051-1058: per-kv-head RMSNorm of k_cur, in place)
//   rope_q / rope_k  (ops_rope.comp:62-95: partial NEOX-paired rotary, pairs (j, j + n_rot/2), cos/sin from
//             a host-built table, dims [n_rot, head_dim) pass through)
//   kv_append        (qsa_kv_append.comp:137-161: f32 -> binary16 by the integer rule, scatter by block table)
// in the order the reference runs them (crates/breccia-kernels/src/qsa/mod.rs:1607-1617): five dispatches
// that each move a few hundred KiB become one kernel whose rows never leave the SM between the steps.
// Arithmetic is fp32 like the shaders': y = x * (1 / sqrt(mean(x^2) + eps)) * gamma; the rotation reads the
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
    uint32_t v_q8;            // the pool stores V as q8_0 blocks
    float eps;
};

// One warp per row: (token, query head) | (token, kv head, K) | (token, kv head, V); a lane holds HD / 32
// elements as float4 chunks [128 c + 4 lane, + 4), so every load and store of the warp is one contiguous run.
constexpr int PREP_WARPS = 8;

template <int HD>
__global__ void __launch_bounds__(PREP_WARPS * 32) qk_prepare_kernel(const PrepareParams p, uint32_t total_rows) {
    constexpr int CH = HD / 128;   // float4 chunks per lane
    __shared__ float y_sm[PREP_WARPS][HD];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_id = blockIdx.x * PREP_WARPS + warp;
    if (row_id >= total_rows) return;
    const uint32_t rows_per_token = p.n_head + 2u * p.n_kv_head;
    const uint32_t tok = row_id / rows_per_token, r = row_id % rows_per_token;
    const uint32_t s = tok / p.tokens_per_seq, t = tok % p.tokens_per_seq;
    const uint32_t pos = p.pos0[s] + t;
    if (pos >= p.max_pos_end) {   // the caller's bound: skip the row, report
        if (lane == 0) { atomicOr(p.status, BRC_DEV_BAD_POS); p.status[1] = pos; }
        return;
    }
    const bool is_q = r < p.n_head;
    const bool is_v = !is_q && r >= p.n_head + p.n_kv_head;
    const uint32_t kvh = is_q ? 0u : (r - p.n_head) % p.n_kv_head;
    const float *src = is_q ? p.q_full + ((size_t)tok * p.n_head + r) * p.q_head_stride
                            : (is_v ? p.v_cur : p.k_cur) + ((size_t)tok * p.n_kv_head + kvh) * HD;
    float4 x[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) x[c] = __ldg(reinterpret_cast<const float4 *>(src + c * 128 + lane * 4));

    if (!is_v) {
        // ---- RMSNorm (qsa_q_norm.comp:54-70; the sum of squares by a shuffle tree instead of the shader's
        //      shared-memory tree: fp32 either way, the order differs)
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) ss += x[c].x * x[c].x + x[c].y * x[c].y + x[c].z * x[c].z + x[c].w * x[c].w;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float inv = 1.0f / sqrtf(ss / (float)HD + p.eps);
        const float *gamma = is_q ? p.q_gamma : p.k_gamma;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const float4 g = __ldg(reinterpret_cast<const float4 *>(gamma + c * 128 + lane * 4));
            x[c] = make_float4(x[c].x * inv * g.x, x[c].y * inv * g.y, x[c].z * inv * g.z, x[c].w * inv * g.w);
            *reinterpret_cast<float4 *>(&y_sm[warp][c * 128 + lane * 4]) = x[c];
        }
        __syncwarp();
        // ---- partial NEOX rotary (ops_rope.comp:72-94); the position is clamped into the table
        const uint32_t hrot = p.n_rot / 2u;
        const uint32_t pi = pos < p.max_pos ? pos : p.max_pos - 1u;
        const float2 *cs_row = p.rope + (size_t)pi * hrot;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float v[4] = {x[c].x, x[c].y, x[c].z, x[c].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t i = c * 128 + lane * 4 + e;
                if (i < hrot) {
                    const float2 cs = __ldg(cs_row + i);
                    v[e] = v[e] * cs.x - y_sm[warp][i + hrot] * cs.y;
                } else if (i < p.n_rot) {
                    const float2 cs = __ldg(cs_row + (i - hrot));
                    v[e] = y_sm[warp][i - hrot] * cs.y + v[e] * cs.x;
                }
            }
            x[c] = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
    if (is_q) {
        const size_t o = ((size_t)tok * p.n_head + r) * HD;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            if (p.q_out_f16) {
                const __half2 lo = __floats2half2_rn(x[c].x, x[c].y), hi = __floats2half2_rn(x[c].z, x[c].w);
                uint2 w;
                w.x = *reinterpret_cast<const uint32_t *>(&lo);
                w.y = *reinterpret_cast<const uint32_t *>(&hi);
                *reinterpret_cast<uint2 *>(static_cast<__half *>(p.q_out) + o + c * 128 + lane * 4) = w;
            } else {
                *reinterpret_cast<float4 *>(static_cast<float *>(p.q_out) + o + c * 128 + lane * 4) = x[c];
            }
        }
        return;
    }
    // ---- append: cell `pos` of sequence s through its block table
    const uint32_t page = p.block_tables[(size_t)s * p.table_stride + (pos >> 4)];
    if (page >= p.n_pages) {
        if (lane == 0) { atomicOr(p.status, BRC_DEV_BAD_PAGE); p.status[1] = page; }
        return;
    }
    if (is_v && p.v_q8) {
        // q8_0 V row (store rule of shaders/qsa_kv_append.comp:117-133, as in the append kernel): the eight lanes
        // that hold a block's 32 values share its maximum; scale = amax / 127 (1 for an all-zero block), quanta
        // = round-half-away(clamp(x / scale, +-127)); a block is one f32 scale then 32 signed bytes.
        const size_t row = ((size_t)page * p.n_kv_head + kvh) * 16u + (pos & 15u);
        uint32_t *vrow = reinterpret_cast<uint32_t *>(p.v_layer) + row * (HD / 32) * 9u;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            float amax = fmaxf(fmaxf(fabsf(x[c].x), fabsf(x[c].y)), fmaxf(fabsf(x[c].z), fabsf(x[c].w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
            auto quant = [scale](float v) { return (uint32_t)(int32_t)roundf(fminf(fmaxf(__fdiv_rn(v, scale), -127.f), 127.f)) & 0xffu; };
            uint32_t *blk = vrow + (c * 4 + (lane >> 3)) * 9u;
            if ((lane & 7u) == 0u) blk[0] = __float_as_uint(scale);
            blk[1u + (lane & 7u)] = quant(x[c].x) | (quant(x[c].y) << 8) | (quant(x[c].z) << 16) | (quant(x[c].w) << 24);
        }
        return;
    }
    uint16_t *dst = reinterpret_cast<uint16_t *>(is_v ? p.v_layer : p.k_layer) + (((size_t)page * p.n_kv_head + kvh) * 16u + (pos & 15u)) * HD;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        uint2 w;
        w.x = brc::pack_f16x2(x[c].x, x[c].y);
        w.y = brc::pack_f16x2(x[c].z, x[c].w);
        *reinterpret_cast<uint2 *>(dst + c * 128 + lane * 4) = w;
    }
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
    p.v_layer = pool->v_base + (uint64_t)layer * pool->v_layer_bytes;
    p.v_q8 = pool->v_q8 ? 1u : 0u;
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
    const uint32_t grid = (uint32_t)((rows + PREP_WARPS - 1) / PREP_WARPS);
    if (hd == 256)
        qk_prepare_kernel<256><<<grid, PREP_WARPS * 32, 0, st>>>(p, (uint32_t)rows);
    else
        qk_prepare_kernel<128><<<grid, PREP_WARPS * 32, 0, st>>>(p, (uint32_t)rows);
    brc_stage_end(pool, BRC_STAGE_KV_APPEND, st);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"
