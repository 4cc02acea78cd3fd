// One decode step of a batch over a range of layers: advance positions, then per layer append the
// new token's K/V and run paged decode attention.  This is the composition the reference performs in
// `Qsa::forward` (crates/breccia-kernels/src/qsa/mod.rs:1587-1645: kv_append -> attend -> apply) and
// the engine repeats for every attention layer (crates/breccia-engine/src/graph.rs:5899-5966); it adds
// no arithmetic of its own.  Also holds the optional per-stage GPU timers (the counterpart of the
// reference's BRECCIA_GPU_TIME probe, crates/breccia-kernels/src/dispatch_batch.rs:453-512).
#include "brc_internal.h"

namespace {

__global__ void advance_positions_kernel(uint32_t *seq_lens, uint32_t *pos0, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const uint32_t len = seq_lens[i];
        pos0[i] = len;
        seq_lens[i] = len + 1u;
    }
}

}  // namespace

extern "C" {

brc_status brc_decode_step(brc_pool *pool, uint32_t layer0, uint32_t n_layers, const uint32_t *block_tables_dev,
                           uint32_t table_stride, uint32_t *seq_lens_dev, uint32_t *pos0_dev, uint32_t n_seqs,
                           uint32_t max_seq_len_after, const void *q_dev, int32_t q_dtype, uint64_t q_layer_stride_bytes,
                           uint32_t n_head, const void *k_new_dev, const void *v_new_dev, int32_t kv_dtype,
                           uint64_t kv_layer_stride_bytes, const float *gate_dev, uint32_t gate_head_stride,
                           uint64_t gate_layer_stride_bytes, float scale, float *out_dev, uint64_t out_layer_stride_bytes,
                           void *workspace_dev, uint64_t workspace_bytes, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_decode_step: pool is NULL");
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "brc_decode_step: this pool holds bookkeeping only (no device memory)");
    if ((uint64_t)layer0 + n_layers > pool->n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step: layers %u..%u but the pool has %u", layer0, layer0 + n_layers,
                        pool->n_layers);
    if (!seq_lens_dev || !pos0_dev || !block_tables_dev || !q_dev || !k_new_dev || !v_new_dev || !out_dev)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step: NULL pointer");
    const uint64_t capacity = (uint64_t)table_stride * pool->page_tokens;
    if (max_seq_len_after > capacity)
        return brc_fail(BRC_ERR_CAPACITY,
                        "decode step would write cell %u but each block table holds %llu (%u pages of %u cells)",
                        max_seq_len_after ? max_seq_len_after - 1 : 0, (unsigned long long)capacity, table_stride,
                        pool->page_tokens);
    if (n_seqs == 0 || n_layers == 0) return BRC_OK;
    {
        brc_device_guard guard(pool->device);
        advance_positions_kernel<<<(n_seqs + 255) / 256, 256, 0, brc_stream(stream)>>>(seq_lens_dev, pos0_dev, n_seqs);
        BRC_CUDA(cudaGetLastError());
    }
    for (uint32_t i = 0; i < n_layers; ++i) {
        const uint8_t *k = static_cast<const uint8_t *>(k_new_dev) + i * kv_layer_stride_bytes;
        const uint8_t *v = static_cast<const uint8_t *>(v_new_dev) + i * kv_layer_stride_bytes;
        const uint8_t *q = static_cast<const uint8_t *>(q_dev) + i * q_layer_stride_bytes;
        const float *g = gate_dev ? reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(gate_dev) + i * gate_layer_stride_bytes) : nullptr;
        float *o = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(out_dev) + i * out_layer_stride_bytes);
        // one kernel per layer: it writes the new cell (fused append) and attends over the whole cache
        if (brc_status rc = brc_decode_attn_append_fused(pool, layer0 + i, q, q_dtype, n_head, g, gate_head_stride,
                                                         block_tables_dev, table_stride, seq_lens_dev, n_seqs,
                                                         max_seq_len_after, scale, o, workspace_dev, workspace_bytes, k, v,
                                                         kv_dtype, i, n_layers, stream))
            return rc;
    }
    return BRC_OK;
}

}  // extern "C"
