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

// Layers [first, first + count) of a step of n_layers layers; the part that holds the step's first
// layer advances the positions.  Every pointer and stride is the whole step's.
static brc_status decode_step_range(brc_pool *pool, uint32_t layer0, uint32_t n_layers, uint32_t first, uint32_t count,
                                    const uint32_t *block_tables_dev, uint32_t table_stride, uint32_t *seq_lens_dev,
                                    uint32_t *pos0_dev, uint32_t n_seqs, uint32_t max_seq_len_after, const void *q_dev,
                                    int32_t q_dtype, uint64_t q_layer_stride_bytes, uint32_t n_head, const void *k_new_dev,
                                    const void *v_new_dev, int32_t kv_dtype, uint64_t kv_layer_stride_bytes,
                                    const float *gate_dev, uint32_t gate_head_stride, uint64_t gate_layer_stride_bytes,
                                    float scale, float *out_dev, uint64_t out_layer_stride_bytes, void *workspace_dev,
                                    uint64_t workspace_bytes, void *stream) {
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
    if ((uint64_t)first + count > n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step_part: layers %u..%u of a step of %u", first, first + count, n_layers);
    if (n_seqs == 0 || count == 0) return BRC_OK;
    if (first == 0) {
        brc_device_guard guard(pool->device);
        advance_positions_kernel<<<(n_seqs + 255) / 256, 256, 0, brc_stream(stream)>>>(seq_lens_dev, pos0_dev, n_seqs);
        BRC_CUDA(cudaGetLastError());
    }
    // one launch for all the layers of the part (when the workspace holds their partial slots): the kernel
    // writes every sequence's new cell (fused append) and attends over the whole cache, layer after layer
    brc_layers_args a;
    a.layer0 = layer0 + first;
    a.n_layers = count;
    a.q = static_cast<const uint8_t *>(q_dev) + first * q_layer_stride_bytes;
    a.q_dtype = q_dtype;
    a.q_layer_stride_bytes = q_layer_stride_bytes;
    a.n_head = n_head;
    a.gate = gate_dev ? reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(gate_dev) + first * gate_layer_stride_bytes) : nullptr;
    a.gate_head_stride = gate_head_stride;
    a.gate_layer_stride_bytes = gate_layer_stride_bytes;
    a.block_tables = block_tables_dev;
    a.table_stride = table_stride;
    a.seq_lens = seq_lens_dev;
    a.n_seqs = n_seqs;
    a.max_seq_len = max_seq_len_after;
    a.scale = scale;
    a.out = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(out_dev) + first * out_layer_stride_bytes);
    a.out_layer_stride_bytes = out_layer_stride_bytes;
    a.workspace = workspace_dev;
    a.workspace_bytes = workspace_bytes;
    a.k_new = static_cast<const uint8_t *>(k_new_dev) + first * kv_layer_stride_bytes;
    a.v_new = static_cast<const uint8_t *>(v_new_dev) + first * kv_layer_stride_bytes;
    a.kv_dtype = kv_dtype;
    a.kv_layer_stride_bytes = kv_layer_stride_bytes;
    return brc_decode_layers(pool, "brc_decode_step", a, stream);
}

extern "C" {

brc_status brc_decode_step(brc_pool *pool, uint32_t layer0, uint32_t n_layers, const uint32_t *block_tables_dev,
                           uint32_t table_stride, uint32_t *seq_lens_dev, uint32_t *pos0_dev, uint32_t n_seqs,
                           uint32_t max_seq_len_after, const void *q_dev, int32_t q_dtype, uint64_t q_layer_stride_bytes,
                           uint32_t n_head, const void *k_new_dev, const void *v_new_dev, int32_t kv_dtype,
                           uint64_t kv_layer_stride_bytes, const float *gate_dev, uint32_t gate_head_stride,
                           uint64_t gate_layer_stride_bytes, float scale, float *out_dev, uint64_t out_layer_stride_bytes,
                           void *workspace_dev, uint64_t workspace_bytes, void *stream) {
    return decode_step_range(pool, layer0, n_layers, 0, n_layers, block_tables_dev, table_stride, seq_lens_dev, pos0_dev,
                             n_seqs, max_seq_len_after, q_dev, q_dtype, q_layer_stride_bytes, n_head, k_new_dev, v_new_dev,
                             kv_dtype, kv_layer_stride_bytes, gate_dev, gate_head_stride, gate_layer_stride_bytes, scale,
                             out_dev, out_layer_stride_bytes, workspace_dev, workspace_bytes, stream);
}

brc_status brc_decode_step_part(brc_pool *pool, uint32_t layer0, uint32_t n_layers, uint32_t first, uint32_t count,
                                const uint32_t *block_tables_dev, uint32_t table_stride, uint32_t *seq_lens_dev,
                                uint32_t *pos0_dev, uint32_t n_seqs, uint32_t max_seq_len_after, const void *q_dev,
                                int32_t q_dtype, uint64_t q_layer_stride_bytes, uint32_t n_head, const void *k_new_dev,
                                const void *v_new_dev, int32_t kv_dtype, uint64_t kv_layer_stride_bytes,
                                const float *gate_dev, uint32_t gate_head_stride, uint64_t gate_layer_stride_bytes,
                                float scale, float *out_dev, uint64_t out_layer_stride_bytes, void *workspace_dev,
                                uint64_t workspace_bytes, void *stream) {
    return decode_step_range(pool, layer0, n_layers, first, count, block_tables_dev, table_stride, seq_lens_dev, pos0_dev,
                             n_seqs, max_seq_len_after, q_dev, q_dtype, q_layer_stride_bytes, n_head, k_new_dev, v_new_dev,
                             kv_dtype, kv_layer_stride_bytes, gate_dev, gate_head_stride, gate_layer_stride_bytes, scale,
                             out_dev, out_layer_stride_bytes, workspace_dev, workspace_bytes, stream);
}

static uint64_t align256(uint64_t x) { return (x + 255u) & ~(uint64_t)255u; }

struct host_step_layout {
    uint64_t q_layer, kv_layer, out_layer;   // bytes per layer
    uint64_t q_off, k_off, v_off, out_off, total;
};

static host_step_layout host_step_sizes(const brc_pool *pool, uint32_t n_layers, uint32_t n_seqs, uint32_t n_head,
                                        int32_t q_dtype, int32_t kv_dtype) {
    host_step_layout l;
    l.q_layer = (uint64_t)n_seqs * n_head * pool->head_dim * (q_dtype == BRC_DTYPE_F32 ? 4u : 2u);
    l.kv_layer = (uint64_t)n_seqs * pool->n_kv_head * pool->head_dim * (kv_dtype == BRC_DTYPE_F32 ? 4u : 2u);
    l.out_layer = (uint64_t)n_seqs * n_head * pool->head_dim * 4u;
    l.q_off = 0;
    l.k_off = align256(l.q_off + n_layers * l.q_layer);
    l.v_off = align256(l.k_off + n_layers * l.kv_layer);
    l.out_off = align256(l.v_off + n_layers * l.kv_layer);
    l.total = align256(l.out_off + n_layers * l.out_layer);
    return l;
}

brc_status brc_decode_step_host_staging_bytes(const brc_pool *pool, uint32_t n_layers, uint32_t n_seqs, uint32_t n_head,
                                              int32_t q_dtype, int32_t kv_dtype, uint64_t *out_bytes) {
    if (!pool || !out_bytes) return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host_staging_bytes: NULL argument");
    *out_bytes = host_step_sizes(pool, n_layers, n_seqs, n_head, q_dtype, kv_dtype).total;
    return BRC_OK;
}

brc_status brc_decode_step_host(brc_pool *pool, uint32_t layer0, uint32_t n_layers, uint32_t parts, uint32_t flags,
                                const uint32_t *block_tables_dev, uint32_t table_stride, uint32_t *seq_lens_dev,
                                uint32_t *pos0_dev, uint32_t n_seqs, uint32_t max_seq_len_after, const void *q_host,
                                int32_t q_dtype, uint32_t n_head, const void *k_new_host, const void *v_new_host,
                                int32_t kv_dtype, float scale, float *out_host, void *staging_dev, uint64_t staging_bytes,
                                void *workspace_dev, uint64_t workspace_bytes, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host: pool is NULL");
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "brc_decode_step_host: this pool holds bookkeeping only (no device memory)");
    if (!q_host || !k_new_host || !v_new_host || !out_host)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host: NULL pointer");
    if ((q_dtype != BRC_DTYPE_F32 && q_dtype != BRC_DTYPE_F16) || (kv_dtype != BRC_DTYPE_F32 && kv_dtype != BRC_DTYPE_F16))
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host: dtypes %d / %d are not f32 (0) or f16 (1)", q_dtype, kv_dtype);
    if (n_seqs == 0 || n_layers == 0) return BRC_OK;
    const host_step_layout l = host_step_sizes(pool, n_layers, n_seqs, n_head, q_dtype, kv_dtype);

    brc_device_guard guard(pool->device);
    // Pinned host memory is addressable from the device.  The kernels then read q / k / v where they lie
    // and store the output straight into out_host: the step's bytes cross PCIe while the attention runs
    // instead of in front of and behind it (measured on the 32-sequence batch: 0.57 against 0.64 ms per
    // step), and nothing is staged.  What is pageable is copied through `staging_dev`.
    auto device_view = [](const void *host) -> void * {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
            return attr.devicePointer;
        cudaGetLastError();   // pageable memory is not an error here
        return nullptr;
    };
    const void *q_direct = nullptr, *k_direct = nullptr, *v_direct = nullptr;
    if (!(flags & BRC_STEP_HOST_UPLOAD)) {
        q_direct = device_view(q_host), k_direct = device_view(k_new_host), v_direct = device_view(v_new_host);
        if (!q_direct || !k_direct || !v_direct) q_direct = k_direct = v_direct = nullptr;   // all three or none
    }
    float *out_direct = (flags & BRC_STEP_HOST_DOWNLOAD) ? nullptr : static_cast<float *>(device_view(out_host));
    if (q_direct && out_direct) {
        // Nothing to stage: one call of the device-resident step on the caller's own buffers.
        brc_status rc = decode_step_range(pool, layer0, n_layers, 0, n_layers, block_tables_dev, table_stride, seq_lens_dev,
                                          pos0_dev, n_seqs, max_seq_len_after, q_direct, q_dtype, l.q_layer, n_head, k_direct,
                                          v_direct, kv_dtype, l.kv_layer, nullptr, 0, 0, scale, out_direct, l.out_layer,
                                          workspace_dev, workspace_bytes, stream);
        cudaError_t e = cudaStreamSynchronize(brc_stream(stream));   // the caller's buffers are in use until here
        if (rc != BRC_OK) return rc;
        BRC_CUDA(e);
        return BRC_OK;
    }
    if (!staging_dev) return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host: NULL staging buffer for a step that has to be staged");
    if (reinterpret_cast<uintptr_t>(staging_dev) & 255u)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host: the staging buffer must be 256-byte aligned");
    if (staging_bytes < l.total)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_step_host: staging of %llu bytes, %llu needed",
                        (unsigned long long)staging_bytes, (unsigned long long)l.total);
    if (q_direct) parts = 1;   // nothing is uploaded, so there is nothing to run ahead
    parts = parts == 0 ? 1u : parts;
    if (parts > n_layers) parts = n_layers;
    if (parts > brc_pool::HOST_PARTS_MAX) parts = brc_pool::HOST_PARTS_MAX;

    if (!pool->host_up) {
        BRC_CUDA(cudaStreamCreateWithFlags(&pool->host_up, cudaStreamNonBlocking));
        BRC_CUDA(cudaStreamCreateWithFlags(&pool->host_down, cudaStreamNonBlocking));
        for (uint32_t i = 0; i < brc_pool::HOST_PARTS_MAX; ++i) {
            BRC_CUDA(cudaEventCreateWithFlags(&pool->host_uploaded[i], cudaEventDisableTiming));
            BRC_CUDA(cudaEventCreateWithFlags(&pool->host_computed[i], cudaEventDisableTiming));
        }
        BRC_CUDA(cudaEventCreateWithFlags(&pool->host_all_down, cudaEventDisableTiming));
    }
    uint8_t *st = static_cast<uint8_t *>(staging_dev);
    const uint8_t *qh = static_cast<const uint8_t *>(q_host), *kh = static_cast<const uint8_t *>(k_new_host),
                  *vh = static_cast<const uint8_t *>(v_new_host);
    uint8_t *oh = reinterpret_cast<uint8_t *>(out_host);
    cudaStream_t s = brc_stream(stream);
    auto lo = [&](uint32_t i) { return (uint32_t)((uint64_t)n_layers * i / parts); };
    // The first part's upload goes to `stream` itself (nothing to overlap it with, and no event between
    // the copy and the first kernel); the later ones run ahead on the upload stream.
    auto upload = [&](uint32_t i) -> cudaError_t {
        const uint64_t a = lo(i), n = lo(i + 1) - a;
        cudaStream_t us = i == 0 ? s : pool->host_up;
        cudaError_t e = cudaMemcpyAsync(st + l.q_off + a * l.q_layer, qh + a * l.q_layer, n * l.q_layer, cudaMemcpyHostToDevice, us);
        if (e == cudaSuccess) e = cudaMemcpyAsync(st + l.k_off + a * l.kv_layer, kh + a * l.kv_layer, n * l.kv_layer, cudaMemcpyHostToDevice, us);
        if (e == cudaSuccess) e = cudaMemcpyAsync(st + l.v_off + a * l.kv_layer, vh + a * l.kv_layer, n * l.kv_layer, cudaMemcpyHostToDevice, us);
        if (e == cudaSuccess && i > 0) e = cudaEventRecord(pool->host_uploaded[i], us);
        return e;
    };
    // Order of issue: every upload before the first kernel, so the copy engine never waits for this
    // thread; each part's output leaves as soon as it is computed.
    if (!q_direct)
        for (uint32_t i = 0; i < parts; ++i) BRC_CUDA(upload(i));
    brc_status rc = BRC_OK;
    for (uint32_t i = 0; i < parts && rc == BRC_OK; ++i) {
        const uint32_t a = lo(i), n = lo(i + 1) - a;
        if (i > 0 && !q_direct) BRC_CUDA(cudaStreamWaitEvent(s, pool->host_uploaded[i], 0));
        rc = decode_step_range(pool, layer0, n_layers, a, n, block_tables_dev, table_stride, seq_lens_dev, pos0_dev, n_seqs,
                               max_seq_len_after, q_direct ? q_direct : st + l.q_off, q_dtype, l.q_layer, n_head,
                               k_direct ? k_direct : st + l.k_off, v_direct ? v_direct : st + l.v_off, kv_dtype,
                               l.kv_layer, nullptr, 0, 0, scale,
                               out_direct ? out_direct : reinterpret_cast<float *>(st + l.out_off), l.out_layer, workspace_dev,
                               workspace_bytes, stream);
        if (rc != BRC_OK) break;
        if (out_direct) continue;
        BRC_CUDA(cudaEventRecord(pool->host_computed[i], s));
        BRC_CUDA(cudaStreamWaitEvent(pool->host_down, pool->host_computed[i], 0));
        BRC_CUDA(cudaMemcpyAsync(oh + a * l.out_layer, st + l.out_off + a * l.out_layer, n * l.out_layer, cudaMemcpyDeviceToHost,
                                 pool->host_down));
    }
    // Whatever was issued has to drain before the caller may touch its buffers again, error or not.
    cudaError_t e = cudaEventRecord(pool->host_all_down, pool->host_down);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, pool->host_all_down, 0);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && rc != BRC_OK) e = cudaStreamSynchronize(pool->host_up);   // kernels that waited for it never went out
    if (rc != BRC_OK) return rc;
    BRC_CUDA(e);
    return BRC_OK;
}

}  // extern "C"
