// Top-k block selection: the stage of the reference that turns indexer scores into the `ids` / `counts` lists the
// selected-block attention walks (crates/breccia-kernels/shaders/qsa_topk.comp; CPU statement
// cpu::topk_blocks, crates/breccia-kernels/src/qsa/cpu.rs:129-151).
//
// Contract, the shader's: per row, the min(n_blocks, topk_blocks) highest scores in DESCENDING score order, equal
// scores resolved towards the LOWER block index; a score <= -1e29 (or NaN) is a dead block and is never selected
// (the score stage writes that value for blocks the row must not see); then the row's own block
// (pos / 4) is appended unless the selection already holds it.  `dense` (n_blocks <= topk_blocks): every block up to the
// row's own, ascending, unscored.  The scores are left untouched (the shader destroys them).
//
// The reference runs k argmax passes over the row (O(k * n_blocks), 512 passes).  Here one CTA per row selects with a
// bitonic network over 64-bit keys (orderable score bits, then inverted block index) in shared memory: runs of k keys
// are sorted, then pairs of runs are reduced to their k largest until one run is left.  Rows of up to 8192 blocks
// take one pass; longer rows go in chunks of 8192 whose best k are merged with the best so far, so any row length
// works with the same 81 KiB of shared memory.
#include <algorithm>

#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

constexpr uint32_t TK_THREADS = 1024;
constexpr uint32_t TK_SORT_MAX = 8192;      // keys per sort: 64 KiB of shared memory
constexpr uint32_t TK_K_MAX = 1024;         // survivors carried between chunks (the reference's k is 512)
constexpr uint32_t BLOCK_CELLS = 4;         // qsa::IDX_BLOCK

struct TopkParams {
    const float *scores;        // [rows][n_blocks]
    const uint32_t *pos0;       // [n_seqs]
    uint32_t *ids;              // [rows][max_ids]
    uint32_t *counts;           // [rows]
    uint32_t rows_per_seq, n_blocks, topk_blocks, max_ids, dense;
};

// Larger key = selected earlier: score ascending in the high word, lower block index larger in the low word.
// Dead blocks (score <= -1e29, NaN) get key 0, below every live key.
__device__ __forceinline__ uint64_t make_key(float s, uint32_t b) {
    if (!(s > -1.0e29f)) return 0ull;
    uint32_t u = s == 0.f ? 0u : __float_as_uint(s);          // -0 and +0 tie, as they compare equal
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((uint64_t)u << 32) | (uint64_t)(0xffffffffu - b);
}

// Where key i lives in shared memory: one unused slot after every 8 keys, so that threads which each read 8
// neighbouring keys (lanes 72 bytes apart instead of 64) spread over all banks.
__device__ __forceinline__ uint32_t pad(uint32_t i) { return i + (i >> 3); }

// One compare-exchange stage of the bitonic network over keys[0 .. n): partners `stride` apart, runs of `size`
// alternately descending and ascending (the first descends).
__device__ __forceinline__ void stage(uint64_t *keys, uint32_t n, uint32_t size, uint32_t stride) {
    __syncthreads();
    for (uint32_t t = threadIdx.x; t < (n >> 1); t += TK_THREADS) {
        const uint32_t lo = 2u * t - (t & (stride - 1u));   // insert a zero bit at the stride position
        const uint32_t hi = lo + stride;
        const bool down = (lo & size) == 0u;
        const uint64_t a = keys[pad(lo)], b = keys[pad(hi)];
        if ((a < b) == down) { keys[pad(lo)] = b; keys[pad(hi)] = a; }
    }
}

// Compare-exchanges `stride` apart inside a group of 8 keys held in registers (indices are compile-time constants
// after unrolling).  `base` is the index of the group's first key in the array, for the direction of each pair.
template <uint32_t STRIDE>
__device__ __forceinline__ void reg_stage(uint64_t (&k)[8], uint32_t base, uint32_t size) {
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        if ((i & STRIDE) == 0u) {
            const bool down = ((base + i) & size) == 0u;
            const uint64_t a = k[i], b = k[i + STRIDE];
            if ((a < b) == down) { k[i] = b; k[i + STRIDE] = a; }
        }
    }
}

// The last three stages (strides 4, 2, 1) of the `size` network, or with FIRST the whole network up to size 8:
// every thread takes groups of 8 neighbouring keys through registers, one barrier instead of three (or six).
template <bool FIRST>
__device__ __forceinline__ void stages_in_registers(uint64_t *keys, uint32_t n, uint32_t size) {
    __syncthreads();
    for (uint32_t g = threadIdx.x; g < (n >> 3); g += TK_THREADS) {
        uint64_t k[8];
        const uint32_t base = g << 3;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) k[i] = keys[base + g + i];   // pad(base + i) = base + g + i
        if (FIRST) {
            reg_stage<1>(k, base, 2);
            reg_stage<2>(k, base, 4);
            reg_stage<1>(k, base, 4);
        }
        reg_stage<4>(k, base, size);
        reg_stage<2>(k, base, size);
        reg_stage<1>(k, base, size);
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) keys[base + g + i] = k[i];
    }
}

// The stages of the `size` network from stride `from` down to 1.
__device__ __forceinline__ void stages_down(uint64_t *keys, uint32_t n, uint32_t size, uint32_t from) {
    if (n >= 8u && size >= 8u) {
        for (uint32_t stride = from; stride >= 8u; stride >>= 1) stage(keys, n, size, stride);
        stages_in_registers<false>(keys, n, size);
    } else {
        for (uint32_t stride = from; stride > 0; stride >>= 1) stage(keys, n, size, stride);
    }
}

// The `run` largest of keys[0 .. n) (n and run powers of two, run <= n <= TK_SORT_MAX), left in keys[0 .. run) in
// descending order.  Runs of `run` keys are sorted in alternating directions; then, while more than one run is left,
// each descending / ascending pair of runs is replaced by its element-wise maximum (a bitonic sequence that holds the
// pair's `run` largest keys) and the halved array is merged back into sorted runs.  Against a full sort this does the
// later, widest stages on ever fewer keys.
__device__ void top_run(uint64_t *keys, uint32_t n, uint32_t run) {
    uint32_t size = 2;
    if (n >= 8u && run >= 8u) {
        stages_in_registers<true>(keys, n, 8);    // sizes 2, 4 and 8 in one go
        size = 16;
    }
    for (; size <= run; size <<= 1) stages_down(keys, n, size, size >> 1);
    while (n > run) {
        const uint32_t half = n >> 1;
        uint64_t m[TK_SORT_MAX / 2 / TK_THREADS];
        __syncthreads();
#pragma unroll
        for (uint32_t r = 0; r < TK_SORT_MAX / 2 / TK_THREADS; ++r) {
            const uint32_t t = threadIdx.x + r * TK_THREADS;
            if (t < half) {
                const uint32_t j = t / run, i = t % run;
                const uint64_t a = keys[pad(2u * j * run + i)], b = keys[pad((2u * j + 1u) * run + i)];
                m[r] = a > b ? a : b;
            }
        }
        __syncthreads();
#pragma unroll
        for (uint32_t r = 0; r < TK_SORT_MAX / 2 / TK_THREADS; ++r) {
            const uint32_t t = threadIdx.x + r * TK_THREADS;
            if (t < half) keys[pad(t)] = m[r];
        }
        n = half;
        stages_down(keys, n, run, run >> 1);
    }
    __syncthreads();
}

__global__ void __launch_bounds__(TK_THREADS) topk_blocks_kernel(const TopkParams p) {
    extern __shared__ uint64_t keys[];
    __shared__ uint32_t s_count, s_present;
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    const uint32_t own = (p.pos0[row / p.rows_per_seq] + row % p.rows_per_seq) / BLOCK_CELLS;
    uint32_t *ids = p.ids + (size_t)row * p.max_ids;

    if (p.dense) {
        uint32_t n = min(min(p.n_blocks, own + 1u), p.max_ids);
        for (uint32_t i = tid; i < n; i += TK_THREADS) ids[i] = i;
        if (tid == 0) {
            if (own >= p.n_blocks && n < p.max_ids) ids[n++] = own;
            p.counts[row] = n;
        }
        return;
    }

    const float *sc = p.scores + (size_t)row * p.n_blocks;
    const uint32_t want = min(min(p.n_blocks, p.topk_blocks), p.max_ids);
    uint32_t run = 2;
    while (run < want) run <<= 1;
    if (p.n_blocks <= TK_SORT_MAX) {
        uint32_t n_sort = 2;
        while (n_sort < p.n_blocks) n_sort <<= 1;
        for (uint32_t i = tid; i < n_sort; i += TK_THREADS) keys[pad(i)] = i < p.n_blocks ? make_key(sc[i], i) : 0ull;
        top_run(keys, n_sort, min(run, n_sort));
    } else {
        // chunks of TK_SORT_MAX scores: the chunk's best `run`, merged with the best so far (kept behind the chunk)
        uint64_t *best = keys + TK_SORT_MAX + TK_SORT_MAX / 8u;
        for (uint32_t i = tid; i < run; i += TK_THREADS) best[pad(i)] = 0ull;
        for (uint32_t at = 0; at < p.n_blocks; at += TK_SORT_MAX) {
            __syncthreads();
            for (uint32_t i = tid; i < TK_SORT_MAX; i += TK_THREADS)
                keys[pad(i)] = at + i < p.n_blocks ? make_key(sc[at + i], at + i) : 0ull;
            top_run(keys, TK_SORT_MAX, run);
            // both descending: the maximum of best[i] and the chunk's run read backwards is bitonic
            for (uint32_t i = tid; i < run; i += TK_THREADS) {
                const uint64_t a = best[pad(i)], b = keys[pad(run - 1u - i)];
                best[pad(i)] = a > b ? a : b;
            }
            stages_down(best, run, run, run >> 1);
        }
        __syncthreads();
        for (uint32_t i = tid; i < run; i += TK_THREADS) keys[pad(i)] = best[pad(i)];
        __syncthreads();
    }
    // keys[0 .. want) are the selection, best first; dead keys (0) sort last
    if (tid == 0) { s_count = 0; s_present = 0; }
    __syncthreads();
    for (uint32_t i = tid; i < want; i += TK_THREADS) {
        const uint64_t k = keys[pad(i)];
        if (k != 0ull) {
            const uint32_t b = 0xffffffffu - (uint32_t)k;
            ids[i] = b;
            if (b == own) s_present = 1u;
            if (i + 1u == want || keys[pad(i + 1u)] == 0ull) s_count = i + 1u;
        }
    }
    __syncthreads();
    if (tid == 0) {
        uint32_t count = s_count;
        if (!s_present && count < p.max_ids) ids[count++] = own;
        p.counts[row] = count;
    }
}

}  // namespace

extern "C" {

brc_status brc_topk_blocks(brc_pool *pool, const float *scores_dev, uint32_t n_seqs, uint32_t rows_per_seq, uint32_t n_blocks,
                           uint32_t topk_blocks, uint32_t max_ids, const uint32_t *pos0_dev, int32_t dense,
                           uint32_t *ids_out_dev, uint32_t *counts_out_dev, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_topk_blocks: pool is NULL");
    if (pool->device < 0) return brc_fail(BRC_ERR_CUDA, "brc_topk_blocks: this pool holds bookkeeping only (no device memory)");
    if (n_seqs == 0 || rows_per_seq == 0) return BRC_OK;
    if (!pos0_dev || !ids_out_dev || !counts_out_dev || (!dense && !scores_dev))
        return brc_fail(BRC_ERR_INVALID, "brc_topk_blocks: NULL score, position, id or count pointer");
    if (n_blocks == 0 || topk_blocks == 0) return brc_fail(BRC_ERR_INVALID, "brc_topk_blocks: n_blocks %u, topk_blocks %u", n_blocks, topk_blocks);
    if (topk_blocks > TK_K_MAX)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_topk_blocks: topk_blocks %u (at most %u; the reference selects 512)", topk_blocks, TK_K_MAX);
    if (max_ids < std::min(n_blocks, topk_blocks) + 1u)
        return brc_fail(BRC_ERR_INVALID, "brc_topk_blocks: max_ids %u but a row can hold %u selected blocks and its own",
                        max_ids, std::min(n_blocks, topk_blocks));
    if (dense && n_blocks > topk_blocks)
        return brc_fail(BRC_ERR_INVALID, "brc_topk_blocks: dense selection needs n_blocks %u <= topk_blocks %u", n_blocks, topk_blocks);
    const uint64_t rows = (uint64_t)n_seqs * rows_per_seq;
    if (rows > 0x7fffffffull) return brc_fail(BRC_ERR_INVALID, "brc_topk_blocks: %llu rows in one call", (unsigned long long)rows);
    brc_device_guard guard(pool->device);
    TopkParams p;
    p.scores = scores_dev;
    p.pos0 = pos0_dev;
    p.ids = ids_out_dev;
    p.counts = counts_out_dev;
    p.rows_per_seq = rows_per_seq;
    p.n_blocks = n_blocks;
    p.topk_blocks = topk_blocks;
    p.max_ids = max_ids;
    p.dense = dense ? 1u : 0u;
    uint32_t n_keys = TK_SORT_MAX + TK_K_MAX;           // a chunk and the best so far
    if (n_blocks <= TK_SORT_MAX) {
        n_keys = 2;
        while (n_keys < n_blocks) n_keys <<= 1;
    }
    const size_t smem = dense ? 0 : (size_t)(n_keys + n_keys / 8u + 1u) * sizeof(uint64_t);   // one slot of padding per 8 keys
    BRC_CUDA(cudaFuncSetAttribute(topk_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(((TK_SORT_MAX + TK_K_MAX) / 8u * 9u + 1u) * sizeof(uint64_t))));
    topk_blocks_kernel<<<(uint32_t)rows, TK_THREADS, smem, brc_stream(stream)>>>(p);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"
