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
// works with the same 81 KiB of shared memory.  For k above 256 (the reference's 512) the network runs with the keys
// in REGISTERS, 256 per warp: shuffles instead of barrier stages, shared memory only between warps; and rows of 4096
// keys or more first drop what lies below a sampled, then verified, threshold, so the network sorts 1024 or 2048 keys.
#include <algorithm>

#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

constexpr uint32_t TK_THREADS = 1024;
constexpr uint32_t TK_SORT_MAX = 8192;      // keys per sort: 64 KiB of shared memory
constexpr uint32_t TK_K_MAX = 1024;         // survivors carried between chunks (the reference's k is 512)
constexpr uint32_t BLOCK_CELLS = 4;         // qsa::IDX_BLOCK
constexpr uint32_t TK_SAMPLE = 256;         // keys sampled for the threshold of the filtered selection
constexpr uint32_t TK_SEL_MAX = 2048;       // survivors of the threshold that are sorted instead of the whole row

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

// ---- the same network with the keys in registers -------------------------------------------------------------
// A barrier per stage is what the shared-memory form above spends its time on.  Here a warp holds 256 neighbouring
// keys, 8 per lane (key i of the warp in lane i / 8, register i % 8): partners 1, 2 and 4 apart are registers of
// one lane, partners 8 .. 128 apart sit in the same register of lane ^ (stride / 8) and come by shuffle, and only
// partners 256 or more apart (another warp) go through shared memory.  Sorting runs of 512 out of 8192 keys takes 1
// exchange through shared memory instead of 28 barrier stages, each halving round 2 instead of 9.

// Compare-exchange with the lane `m` lanes away (partners 8 m apart), all 8 registers; `down`: the lower index keeps
// the larger key.
__device__ __forceinline__ void warp_cx(uint64_t (&k)[8], uint32_t m, bool down, uint32_t lane) {
    const bool keep_max = ((lane & m) == 0u) == down;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const uint64_t o = __shfl_xor_sync(0xffffffffu, k[r], m);
        k[r] = (o > k[r]) == keep_max ? o : k[r];
    }
}

// Strides min(size / 2, 128) .. 1 of the `size` network on this warp's keys; g = array index of the lane's first key.
__device__ __forceinline__ void warp_merge(uint64_t (&k)[8], uint32_t g, uint32_t size, uint32_t lane) {
    const bool down = (g & size) == 0u;
    for (uint32_t m = min(size >> 4, 16u); m >= 1u; m >>= 1) warp_cx(k, m, down, lane);
    reg_stage<4>(k, g, size);
    reg_stage<2>(k, g, size);
    reg_stage<1>(k, g, size);
}

// One stage with partners in another warp (stride >= 256): through shared memory, two barriers.  Every thread of the
// CTA calls it; `active` threads hold keys.
__device__ __forceinline__ void cross_stage(uint64_t *keys, uint64_t (&k)[8], uint32_t g, uint32_t stride, uint32_t size, bool active) {
    if (active) {
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) keys[g + (g >> 3) + r] = k[r];     // pad(g + r)
    }
    __syncthreads();
    if (active) {
        const uint32_t pg = g ^ stride;
        const bool keep_max = ((g & stride) == 0u) == ((g & size) == 0u);
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) {
            const uint64_t o = keys[pg + (pg >> 3) + r];
            k[r] = (o > k[r]) == keep_max ? o : k[r];
        }
    }
    __syncthreads();
}

// top_run for run = 512 or 1024 and 512 <= n <= TK_SORT_MAX (powers of two, run <= n): same result, same place.
__device__ void top_run_regs(uint64_t *keys, uint32_t n, uint32_t run) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t g = (threadIdx.x >> 5) * 256u + lane * 8u;
    uint64_t k[8];
    bool active = g < n;
    __syncthreads();
    if (active) {
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) k[r] = keys[g + (g >> 3) + r];
        reg_stage<1>(k, g, 2);
        reg_stage<2>(k, g, 4);
        reg_stage<1>(k, g, 4);
        reg_stage<4>(k, g, 8);
        reg_stage<2>(k, g, 8);
        reg_stage<1>(k, g, 8);
        for (uint32_t size = 16; size <= 256u; size <<= 1) warp_merge(k, g, size, lane);
    }
    for (uint32_t size = 512; size <= run; size <<= 1) {
        for (uint32_t stride = size >> 1; stride >= 256u; stride >>= 1) cross_stage(keys, k, g, stride, size, active);
        if (active) warp_merge(k, g, size, lane);
    }
    while (n > run) {
        // runs 2j (descending) and 2j + 1 (ascending) -> their element-wise maximum, a bitonic run that holds the
        // pair's `run` largest keys; then the `run` network's merge puts it in order
        if (active) {
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) keys[g + (g >> 3) + r] = k[r];
        }
        __syncthreads();
        n >>= 1;
        active = g < n;
        if (active) {
            const uint32_t a = 2u * (g / run) * run + g % run, b = a + run;
#pragma unroll
            for (uint32_t r = 0; r < 8; ++r) {
                const uint64_t x = keys[a + (a >> 3) + r], y = keys[b + (b >> 3) + r];
                k[r] = x > y ? x : y;
            }
        }
        __syncthreads();
        for (uint32_t stride = run >> 1; stride >= 256u; stride >>= 1) cross_stage(keys, k, g, stride, run, active);
        if (active) warp_merge(k, g, run, lane);
    }
    if (active) {
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) keys[g + (g >> 3) + r] = k[r];
    }
    __syncthreads();
}

// ---- selection behind a threshold ---------------------------------------------------------------------------
// Sorting 8192 keys to keep 512 does sixteen times the work the answer needs.  For run = 512 out of n >= 4096 keys:
// the CTA ranks 256 sampled keys among themselves (all pairs, 64 per thread), takes the sample of rank 2 * 256 * run / n
// as a threshold - about 2 * run keys of the row lie above it - counts the keys >= threshold, and when there are at
// least `run` and at most TK_SEL_MAX of them compacts those into `sel` and runs the network on 1024 or 2048 keys.
// The count makes it exact: every key of the best `run` is >= a threshold that at least `run` keys reach, and live keys
// are distinct, so the result is the full network's.  Any other outcome (a row of mostly dead keys, an unlucky sample)
// returns nullptr with `keys` untouched and the caller sorts the whole row.
__device__ uint64_t *top_run_filtered(uint64_t *keys, uint64_t *sel, uint32_t n, uint32_t run) {
    __shared__ uint64_t s_sample[TK_SAMPLE];
    __shared__ uint32_t s_rank[TK_SAMPLE];
    __shared__ uint32_t s_warp[TK_THREADS / 32 + 1];
    __shared__ uint64_t s_thr;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t step = n / TK_SAMPLE;
    __syncthreads();   // the keys are in place
    if (tid < TK_SAMPLE) {
        s_sample[tid] = keys[pad(tid * step + (tid * 7u) % step)];
        s_rank[tid] = 0u;
    }
    if (tid == 0) s_thr = 0ull;
    __syncthreads();
    {
        const uint32_t j = tid % TK_SAMPLE, part = tid / TK_SAMPLE;
        constexpr uint32_t PER = TK_SAMPLE / (TK_THREADS / TK_SAMPLE);
        const uint64_t mine = s_sample[j];
        uint32_t c = 0;
        for (uint32_t i = part * PER; i < (part + 1u) * PER; ++i) c += s_sample[i] > mine ? 1u : 0u;
        atomicAdd(&s_rank[j], c);
    }
    __syncthreads();
    const uint32_t r = 2u * run * TK_SAMPLE / n;
    if (tid < TK_SAMPLE && s_rank[tid] == r - 1u) s_thr = s_sample[tid];
    __syncthreads();
    const uint64_t thr = s_thr;
    if (thr == 0ull) return nullptr;   // the sample reached into the dead keys

    uint64_t k[8];
    const uint32_t per = n / TK_THREADS, base = tid * per;   // 4 or 8 neighbouring keys per thread
    uint32_t c = 0;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        k[i] = i < per ? keys[pad(base + i)] : 0ull;
        c += k[i] >= thr ? 1u : 0u;
    }
    uint32_t inc = c;
#pragma unroll
    for (uint32_t off = 1; off < 32; off <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += t;
    }
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        const uint32_t w = s_warp[lane];
        uint32_t wi = w;
#pragma unroll
        for (uint32_t off = 1; off < 32; off <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= off) wi += t;
        }
        s_warp[lane] = wi - w;
        if (lane == 31) s_warp[TK_THREADS / 32] = wi;
    }
    __syncthreads();
    const uint32_t total = s_warp[TK_THREADS / 32];
    if (total < run || total > TK_SEL_MAX) return nullptr;
    uint32_t at = s_warp[warp] + inc - c;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i)
        if (k[i] >= thr) sel[pad(at++)] = k[i];
    const uint32_t n2 = total <= 1024u ? 1024u : 2048u;
    for (uint32_t i = total + tid; i < n2; i += TK_THREADS) sel[pad(i)] = 0ull;
    top_run_regs(sel, n2, run);
    return sel;
}

// The `run` largest of keys[0 .. n), best first, by whichever form applies.
__device__ __forceinline__ void select_run(uint64_t *keys, uint32_t n, uint32_t run) {
    if (run >= 512u && n >= run) top_run_regs(keys, n, run);
    else top_run(keys, n, run);
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
    const uint64_t *res = keys;                 // where the selection ends up, best first
    const uint32_t want = min(min(p.n_blocks, p.topk_blocks), p.max_ids);
    uint32_t run = 2;
    while (run < want) run <<= 1;
    if (p.n_blocks <= TK_SORT_MAX) {
        uint32_t n_sort = 2;
        while (n_sort < p.n_blocks) n_sort <<= 1;
        for (uint32_t i = tid; i < n_sort; i += TK_THREADS) keys[pad(i)] = i < p.n_blocks ? make_key(sc[i], i) : 0ull;
        uint64_t *filtered = nullptr;
        if (run == 512u && n_sort >= 4096u) filtered = top_run_filtered(keys, keys + n_sort + n_sort / 8u + 1u, n_sort, run);
        if (filtered) res = filtered;
        else select_run(keys, n_sort, min(run, n_sort));
    } else {
        // chunks of TK_SORT_MAX scores: the chunk's best `run`, merged with the best so far (kept behind the chunk)
        uint64_t *best = keys + TK_SORT_MAX + TK_SORT_MAX / 8u;
        for (uint32_t i = tid; i < run; i += TK_THREADS) best[pad(i)] = 0ull;
        for (uint32_t at = 0; at < p.n_blocks; at += TK_SORT_MAX) {
            __syncthreads();
            for (uint32_t i = tid; i < TK_SORT_MAX; i += TK_THREADS)
                keys[pad(i)] = at + i < p.n_blocks ? make_key(sc[at + i], at + i) : 0ull;
            const uint64_t *top = run == 512u ? top_run_filtered(keys, best + TK_K_MAX + TK_K_MAX / 8u + 1u, TK_SORT_MAX, run) : nullptr;
            if (!top) {
                select_run(keys, TK_SORT_MAX, run);
                top = keys;
            }
            // both descending: the maximum of best[i] and the chunk's run read backwards is bitonic
            for (uint32_t i = tid; i < run; i += TK_THREADS) {
                const uint64_t a = best[pad(i)], b = top[pad(run - 1u - i)];
                best[pad(i)] = a > b ? a : b;
            }
            stages_down(best, run, run, run >> 1);
        }
        __syncthreads();
        for (uint32_t i = tid; i < run; i += TK_THREADS) keys[pad(i)] = best[pad(i)];
        __syncthreads();
    }
    // res[0 .. want) are the selection, best first; dead keys (0) sort last
    if (tid == 0) { s_count = 0; s_present = 0; }
    __syncthreads();
    for (uint32_t i = tid; i < want; i += TK_THREADS) {
        const uint64_t k = res[pad(i)];
        if (k != 0ull) {
            const uint32_t b = 0xffffffffu - (uint32_t)k;
            ids[i] = b;
            if (b == own) s_present = 1u;
            if (i + 1u == want || res[pad(i + 1u)] == 0ull) s_count = i + 1u;
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
    size_t smem = dense ? 0 : (size_t)(n_keys + n_keys / 8u + 2u) * sizeof(uint64_t);   // one slot of padding per 8 keys
    if (!dense && n_keys >= 4096u) smem += (size_t)(TK_SEL_MAX + TK_SEL_MAX / 8u + 1u) * sizeof(uint64_t);   // the filtered selection's keys
    static bool configured[64] = {};   // per device, once: the attribute call costs the host several microseconds
    if (pool->device >= 64 || !configured[pool->device]) {
        BRC_CUDA(cudaFuncSetAttribute(topk_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(((TK_SORT_MAX + TK_K_MAX + TK_SEL_MAX) / 8u * 9u + 3u) * sizeof(uint64_t))));
        if (pool->device < 64) configured[pool->device] = true;
    }
    topk_blocks_kernel<<<(uint32_t)rows, TK_THREADS, smem, brc_stream(stream)>>>(p);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"
