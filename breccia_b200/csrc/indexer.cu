// Indexer stages in front of the top-k block selection: the pooled-key cache of every sequence and the
// block scores of every query row.  Replaces shaders/qsa_idx_pool.comp, qsa_idx_tail.comp and
// qsa_idx_score.comp of the reference (driven from Qsa::idx_pool / idx_tail / idx_score,
// crates/breccia-kernels/src/qsa/mod.rs:1168-1262, in the order Qsa::forward runs them, :1618-1630; CPU
// statements cpu::pool_keys and cpu::indexer_score, crates/breccia-kernels/src/qsa/cpu.rs:97-121, 159-195).
//
//   pooled[s][b] = rope( rmsnorm( mean(raw key of cells 4b .. 4b+3), gamma ), position 4b )
//   tail[s][slot] = raw key of cell (cell % 4 == slot < 3) of the sequence's last, incomplete block
//   score[row][b] = (1/sqrt(idx_dim)) * sum_h relu( q[row][h] . pooled[s][b] ),  -1e30 for a block whose last
//                   cell lies beyond the row's position
//
// The reference keeps one such state per sequence and layer and is called once per sequence; here the
// state arrays carry a leading sequence dimension and one launch serves a batch.  The scores are exactly the
// [rows][n_blocks] f32 array brc_topk_blocks consumes.
//
// The score stage is the one that scales with context: it streams 512 B per block of every sequence
// (HBM-bound at decode, L2-resident re-reads for the further rows of a chunk).  Eight lanes share a block:
// each holds 16 of the 128 key dims as four 16-byte loads (lane-interleaved, so the eight read 128 contiguous bytes at a time), the query heads sit in shared memory, and the
// per-head dots are reduced with three shuffles, so a warp scores four blocks per step with fully
// coalesced 2 KiB reads.  Pooling and the tail move a few KiB per call and are launch-latency sized.
#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

constexpr uint32_t IDX_DIM = 128;        // qsa::IDX_DIM
constexpr uint32_t IDX_BLOCK = 4;        // qsa::IDX_BLOCK
constexpr uint32_t IDX_HEAD_MAX = 8;     // the shader's MAX_IDX_HEAD
constexpr float MASK_DEAD = -1.0e30f;    // the shader's MASK_DEAD; brc_topk_blocks never selects it

struct PoolParams {
    const float *raw;          // [n_seqs][tokens][IDX_DIM]
    const float *tail;         // [n_seqs][IDX_BLOCK - 1][IDX_DIM]
    const float *gamma;        // [IDX_DIM]
    const float *rope;         // [max_pos][n_rot / 2][2]
    float *pooled;             // [n_seqs][max_blocks][IDX_DIM]
    const uint32_t *pos0;      // [n_seqs]
    uint32_t *status;
    uint32_t n_seqs, tokens, max_blocks, n_rot, max_pos, max_pos_end;
    float eps;
};

// One CTA of IDX_DIM threads per (sequence, block completed by this call); blocks_completed() of the
// reference (qsa/mod.rs:1673-1687) is evaluated per sequence on the device.
__global__ void __launch_bounds__(IDX_DIM) idx_pool_kernel(const PoolParams p) {
    __shared__ float s_val[IDX_DIM];
    __shared__ float s_sum[IDX_DIM / 32];
    const uint32_t s = blockIdx.y, tid = threadIdx.x;
    const uint32_t pos0 = p.pos0[s];
    if (pos0 + p.tokens > p.max_pos_end) {
        if (tid == 0 && blockIdx.x == 0) {
            atomicOr(p.status, BRC_DEV_BAD_POS);
            p.status[1] = pos0 + p.tokens;
        }
        return;
    }
    const uint32_t last = pos0 + p.tokens - 1u;
    if (last < IDX_BLOCK - 1u) return;
    const uint32_t b0 = pos0 / IDX_BLOCK, b_last = (last - (IDX_BLOCK - 1u)) / IDX_BLOCK;
    const uint32_t block = b0 + blockIdx.x;
    if (block > b_last || block >= p.max_blocks) return;
    // mean of the RAW keys: a cell of this call comes from `raw`, an earlier one from the tail (slot 3
    // never holds a key: the cell that completes a block always arrives with the call)
    float mean = 0.f;
#pragma unroll
    for (uint32_t k = 0; k < IDX_BLOCK; ++k) {
        const uint32_t cell = block * IDX_BLOCK + k;
        float v = 0.f;
        if (cell >= pos0)
            v = p.raw[((size_t)s * p.tokens + (cell - pos0)) * IDX_DIM + tid];
        else if (k + 1u < IDX_BLOCK)
            v = p.tail[((size_t)s * (IDX_BLOCK - 1u) + k) * IDX_DIM + tid];
        mean += v;
    }
    mean /= (float)IDX_BLOCK;
    float ss = mean * mean;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31u) == 0u) s_sum[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (uint32_t w = 0; w < IDX_DIM / 32; ++w) tot += s_sum[w];
    const float inv = rsqrtf(tot / (float)IDX_DIM + p.eps);
    s_val[tid] = mean * inv * p.gamma[tid];
    __syncthreads();
    // NEOX pairs (j, j + n_rot / 2), rotated at the block's FIRST cell; dims beyond n_rot pass through
    const uint32_t pairs = p.n_rot / 2u;
    float *out = p.pooled + ((size_t)s * p.max_blocks + block) * IDX_DIM;
    if (tid < pairs) {
        const uint32_t tpos = min(IDX_BLOCK * block, p.max_pos - 1u);
        const float2 cs = *reinterpret_cast<const float2 *>(p.rope + ((size_t)tpos * pairs + tid) * 2u);
        const float a = s_val[tid], bb = s_val[tid + pairs];
        out[tid] = a * cs.x - bb * cs.y;
        out[tid + pairs] = a * cs.y + bb * cs.x;
    } else if (tid >= p.n_rot) {
        out[tid] = s_val[tid];
    }
}

// One thread per (sequence, token, dim): only the cells of the call's last, incomplete block are stored.
__global__ void idx_tail_kernel(const float *raw, float *tail, const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t tokens) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_seqs * tokens * IDX_DIM) return;
    const uint32_t d = (uint32_t)(i % IDX_DIM);
    const uint32_t t = (uint32_t)((i / IDX_DIM) % tokens);
    const uint32_t s = (uint32_t)(i / ((size_t)IDX_DIM * tokens));
    const uint32_t pos0 = pos0_dev[s];
    const uint32_t cell = pos0 + t, last_cell = pos0 + tokens - 1u;
    const uint32_t slot = cell % IDX_BLOCK;
    if (cell / IDX_BLOCK == last_cell / IDX_BLOCK && slot + 1u < IDX_BLOCK)
        tail[((size_t)s * (IDX_BLOCK - 1u) + slot) * IDX_DIM + d] = raw[i];
}

struct ScoreParams {
    const float *q;            // [rows][n_head][IDX_DIM]
    const float *pooled;       // [n_seqs][max_blocks][IDX_DIM]
    float *scores;             // [rows][n_blocks]
    const uint32_t *pos0;      // [n_seqs]
    uint32_t rows_per_seq, n_blocks, max_blocks, n_head;
    float scale;
};

constexpr uint32_t SC_THREADS = 256;
constexpr uint32_t SC_BLOCKS_PER_CTA = 128;   // blocks one CTA scores: 4 steps of its 8 warps x 4 blocks (small CTAs: a short tail)

// grid = (ceil(n_blocks / SC_BLOCKS_PER_CTA), rows).
__global__ void __launch_bounds__(SC_THREADS, 4) idx_score_kernel(const ScoreParams p) {
    __shared__ float4 s_q[IDX_HEAD_MAX * IDX_DIM / 4];
    const uint32_t row = blockIdx.y, tid = threadIdx.x;
    const uint32_t s = row / p.rows_per_seq, t = row % p.rows_per_seq;
    const uint32_t pos = p.pos0[s] + t;
    for (uint32_t i = tid; i < p.n_head * IDX_DIM / 4; i += SC_THREADS)
        s_q[i] = reinterpret_cast<const float4 *>(p.q + (size_t)row * p.n_head * IDX_DIM)[i];
    __syncthreads();
    const uint32_t sub = tid & 7u;              // this lane holds dims 4 sub + 32 j + {0..3}, j = 0..3 (neighbouring lanes, neighbouring 16 bytes)
    const uint32_t slot = tid >> 3;             // block slot within a step of the CTA: 0 .. 31
    const uint32_t b_begin = blockIdx.x * SC_BLOCKS_PER_CTA;
    const float *pooled = p.pooled + (size_t)s * p.max_blocks * IDX_DIM;
    constexpr uint32_t STEPS = SC_BLOCKS_PER_CTA / (SC_THREADS / 8);
    // The pooled key averages ALL cells of its block, so a row may use it only when it sees the whole
    // block: masked on the block's last cell (qsa_idx_score.comp:74-81).
    auto load_key = [&](uint32_t step, float4 (&k)[4]) {
        const uint32_t b = b_begin + step * (SC_THREADS / 8) + slot;
        k[0] = k[1] = k[2] = k[3] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < p.n_blocks && b * IDX_BLOCK + IDX_BLOCK - 1u <= pos) {
            const float4 *kp = reinterpret_cast<const float4 *>(pooled + (size_t)b * IDX_DIM) + sub;
            k[0] = __ldg(kp), k[1] = __ldg(kp + 8), k[2] = __ldg(kp + 16), k[3] = __ldg(kp + 24);
        }
    };
    float4 k[4], kn[4];
    load_key(0, k);
#pragma unroll
    for (uint32_t step = 0; step < STEPS; ++step) {   // the same trip count for every lane
        if (step + 1u < STEPS) load_key(step + 1u, kn);   // the next step's key is on its way while this one is scored
        const uint32_t b = b_begin + step * (SC_THREADS / 8) + slot;
        const bool valid = b < p.n_blocks;
        const bool dead = b * IDX_BLOCK + IDX_BLOCK - 1u > pos;
        float sum = 0.f;
        for (uint32_t h = 0; h < p.n_head; ++h) {
            const float4 *qp = s_q + h * (IDX_DIM / 4) + sub;
            const float4 q0 = qp[0], q1 = qp[8], q2 = qp[16], q3 = qp[24];
            float dot = k[0].x * q0.x + k[0].y * q0.y + k[0].z * q0.z + k[0].w * q0.w + k[1].x * q1.x + k[1].y * q1.y + k[1].z * q1.z + k[1].w * q1.w +
                        k[2].x * q2.x + k[2].y * q2.y + k[2].z * q2.z + k[2].w * q2.w + k[3].x * q3.x + k[3].y * q3.y + k[3].z * q3.z + k[3].w * q3.w;
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            sum += fmaxf(dot, 0.f);
        }
        if (valid && sub == 0u) p.scores[(size_t)row * p.n_blocks + b] = dead ? MASK_DEAD : sum * p.scale;
#pragma unroll
        for (int j = 0; j < 4; ++j) k[j] = kn[j];
    }
}

// Several rows of one sequence per CTA (prefill chunks, speculative rows): the rows share the sequence's pooled
// keys, so a key is loaded once and held in registers while SC_ROWS rows are scored against it - one row per
// CTA re-read every key from L2 for every row (8.6 GB of L2 reads for a 2048-row chunk over 8192 blocks).
// A lane holds its 16 dims of TWO blocks (slots `slot` and `slot + 32` of a step of 64 blocks); per row the
// eight partial dots (2 blocks x 4 heads) of the eight lanes that share the blocks are reduced TRANSPOSED
// (7 shuffles for 8 dots: each step halves the values a lane holds), so that lane `sub` ends with the whole dot
// of (block sub / 4, head sub % 4); relu, and two more shuffles sum the heads.  Built for 4 index heads (the
// reference's IDX_N_HEAD); other head counts take the one-row kernel.
constexpr uint32_t SC_ROWS = 8;
constexpr uint32_t SC_TILE_BLOCKS = 512;   // blocks one CTA scores: 8 steps of 64

// grid = (ceil(n_blocks / SC_TILE_BLOCKS), n_seqs * ceil(rows_per_seq / SC_ROWS)).
__global__ void __launch_bounds__(SC_THREADS) idx_score_rows_kernel(const ScoreParams p) {
    __shared__ float4 s_q[SC_ROWS * 4 * IDX_DIM / 4];
    const uint32_t tid = threadIdx.x;
    const uint32_t tiles_per_seq = (p.rows_per_seq + SC_ROWS - 1u) / SC_ROWS;
    const uint32_t s = blockIdx.y / tiles_per_seq, t0 = (blockIdx.y % tiles_per_seq) * SC_ROWS;
    const uint32_t n_rows = min(SC_ROWS, p.rows_per_seq - t0);
    const size_t row0 = (size_t)s * p.rows_per_seq + t0;
    const uint32_t pos_first = p.pos0[s] + t0;
    for (uint32_t i = tid; i < n_rows * 4u * IDX_DIM / 4u; i += SC_THREADS)
        s_q[i] = reinterpret_cast<const float4 *>(p.q + row0 * 4u * IDX_DIM)[i];
    __syncthreads();
    const uint32_t sub = tid & 7u, slot = tid >> 3;
    const bool hi4 = (sub & 4u) != 0u, hi2 = (sub & 2u) != 0u, hi1 = (sub & 1u) != 0u;
    const float *pooled = p.pooled + (size_t)s * p.max_blocks * IDX_DIM;
    for (uint32_t step = 0; step < SC_TILE_BLOCKS / 64u; ++step) {   // the same trip count for every lane
        const uint32_t bA = blockIdx.x * SC_TILE_BLOCKS + step * 64u + slot, bB = bA + 32u;
        // a block that even the tile's last row cannot see whole is dead for all of them: no need to load it
        const uint32_t pos_last = pos_first + n_rows - 1u;
        const bool liveA = bA < p.n_blocks && bA * IDX_BLOCK + IDX_BLOCK - 1u <= pos_last;
        const bool liveB = bB < p.n_blocks && bB * IDX_BLOCK + IDX_BLOCK - 1u <= pos_last;
        float4 ka[4], kb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) ka[j] = kb[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (liveA) {
            const float4 *kp = reinterpret_cast<const float4 *>(pooled + (size_t)bA * IDX_DIM) + sub;
#pragma unroll
            for (int j = 0; j < 4; ++j) ka[j] = __ldg(kp + 8 * j);
        }
        if (liveB) {
            const float4 *kp = reinterpret_cast<const float4 *>(pooled + (size_t)bB * IDX_DIM) + sub;
#pragma unroll
            for (int j = 0; j < 4; ++j) kb[j] = __ldg(kp + 8 * j);
        }
        for (uint32_t r = 0; r < n_rows; ++r) {
            float v[8];   // partial dots: v[4 blk + h]
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const float4 *qp = s_q + (r * 4u + h) * (IDX_DIM / 4) + sub;
                float da = 0.f, db = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 q4 = qp[8 * j];
                    da += ka[j].x * q4.x + ka[j].y * q4.y + ka[j].z * q4.z + ka[j].w * q4.w;
                    db += kb[j].x * q4.x + kb[j].y * q4.y + kb[j].z * q4.z + kb[j].w * q4.w;
                }
                v[h] = da;
                v[4 + h] = db;
            }
            float w[4], x[2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float got = __shfl_xor_sync(0xffffffffu, hi4 ? v[i] : v[i + 4], 4);
                w[i] = (hi4 ? v[i + 4] : v[i]) + got;
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float got = __shfl_xor_sync(0xffffffffu, hi2 ? w[i] : w[i + 2], 2);
                x[i] = (hi2 ? w[i + 2] : w[i]) + got;
            }
            const float got = __shfl_xor_sync(0xffffffffu, hi1 ? x[0] : x[1], 1);
            float sum = fmaxf((hi1 ? x[1] : x[0]) + got, 0.f);   // relu of the dot of (block sub / 4, head sub % 4)
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((sub & 3u) == 0u) {
                const uint32_t b = hi4 ? bB : bA;
                // the pooled key averages ALL cells of its block: usable only by a row that sees the whole block
                if (b < p.n_blocks)
                    p.scores[(row0 + r) * p.n_blocks + b] = b * IDX_BLOCK + IDX_BLOCK - 1u > pos_first + r ? MASK_DEAD : sum * p.scale;
            }
        }
    }
}

brc_status check_pool(const brc_pool *pool, const char *who) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "%s: pool is NULL", who);
    if (pool->device < 0 || !pool->status_dev)
        return brc_fail(BRC_ERR_CUDA, "%s: this pool holds bookkeeping only (no device memory)", who);
    return BRC_OK;
}

brc_status check_geometry(const char *who, uint32_t idx_dim, uint32_t idx_block) {
    if (idx_dim != IDX_DIM || idx_block != IDX_BLOCK)
        return brc_fail(BRC_ERR_UNSUPPORTED, "%s: built for %u-dim indexer keys pooled over %u cells (given %u, %u)", who, IDX_DIM,
                        IDX_BLOCK, idx_dim, idx_block);
    return BRC_OK;
}

}  // namespace

extern "C" {

brc_status brc_idx_pool(brc_pool *pool, const float *raw_dev, const float *tail_dev, const float *gamma_dev,
                        const float *rope_table_dev, uint32_t n_rot, uint32_t max_pos, float eps, const uint32_t *pos0_dev,
                        uint32_t n_seqs, uint32_t tokens_per_seq, uint32_t max_pos_end, uint32_t idx_dim, uint32_t idx_block,
                        float *pooled_dev, uint32_t max_blocks, void *stream) {
    if (brc_status rc = check_pool(pool, "brc_idx_pool")) return rc;
    if (brc_status rc = check_geometry("brc_idx_pool", idx_dim, idx_block)) return rc;
    if (n_rot > idx_dim || (n_rot & 1u) || (n_rot && (!rope_table_dev || max_pos == 0)))
        return brc_fail(BRC_ERR_INVALID, "brc_idx_pool: n_rot %u (even, at most %u, with a table of max_pos > 0 rows)", n_rot, idx_dim);
    // the reference's refusal (qsa/mod.rs:1178-1184): the blocks this call can complete must fit the state
    const uint64_t blocks_end = max_pos_end / IDX_BLOCK;
    if (blocks_end > max_blocks)
        return brc_fail(BRC_ERR_CAPACITY, "idx_pool would write pooled rows up to %llu but the state holds %u",
                        (unsigned long long)blocks_end, max_blocks);
    if (n_seqs == 0 || tokens_per_seq == 0) return BRC_OK;
    if (!raw_dev || !tail_dev || !gamma_dev || !pos0_dev || !pooled_dev) return brc_fail(BRC_ERR_INVALID, "brc_idx_pool: NULL pointer");
    brc_device_guard guard(pool->device);
    PoolParams p;
    p.raw = raw_dev;
    p.tail = tail_dev;
    p.gamma = gamma_dev;
    p.rope = rope_table_dev;
    p.pooled = pooled_dev;
    p.pos0 = pos0_dev;
    p.status = pool->status_dev;
    p.n_seqs = n_seqs;
    p.tokens = tokens_per_seq;
    p.max_blocks = max_blocks;
    p.n_rot = n_rot;
    p.max_pos = max_pos;
    p.max_pos_end = max_pos_end;
    p.eps = eps;
    const uint32_t max_new = (tokens_per_seq + IDX_BLOCK - 1u) / IDX_BLOCK + 1u;   // blocks one call can complete, at most
    if (n_seqs > 65535u) return brc_fail(BRC_ERR_UNSUPPORTED, "brc_idx_pool: %u sequences in one call (at most 65535)", n_seqs);
    idx_pool_kernel<<<dim3(max_new, n_seqs), IDX_DIM, 0, brc_stream(stream)>>>(p);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

brc_status brc_idx_tail(brc_pool *pool, const float *raw_dev, const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t tokens_per_seq,
                        uint32_t idx_dim, uint32_t idx_block, float *tail_dev, void *stream) {
    if (brc_status rc = check_pool(pool, "brc_idx_tail")) return rc;
    if (brc_status rc = check_geometry("brc_idx_tail", idx_dim, idx_block)) return rc;
    if (n_seqs == 0 || tokens_per_seq == 0) return BRC_OK;
    if (!raw_dev || !pos0_dev || !tail_dev) return brc_fail(BRC_ERR_INVALID, "brc_idx_tail: NULL pointer");
    brc_device_guard guard(pool->device);
    const size_t n = (size_t)n_seqs * tokens_per_seq * IDX_DIM;
    idx_tail_kernel<<<(uint32_t)((n + 255) / 256), 256, 0, brc_stream(stream)>>>(raw_dev, tail_dev, pos0_dev, n_seqs, tokens_per_seq);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

brc_status brc_idx_score(brc_pool *pool, const float *q_dev, uint32_t idx_n_head, const float *pooled_dev, uint32_t max_blocks,
                         const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t rows_per_seq, uint32_t n_blocks, uint32_t idx_dim,
                         uint32_t idx_block, float scale, float *scores_out_dev, void *stream) {
    if (brc_status rc = check_pool(pool, "brc_idx_score")) return rc;
    if (brc_status rc = check_geometry("brc_idx_score", idx_dim, idx_block)) return rc;
    if (idx_n_head == 0 || idx_n_head > IDX_HEAD_MAX)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_idx_score: %u indexer heads (1 to %u)", idx_n_head, IDX_HEAD_MAX);
    // the reference's refusal (qsa/mod.rs:1237-1243)
    if (n_blocks > max_blocks)
        return brc_fail(BRC_ERR_CAPACITY, "idx_score covers %u blocks but the state holds %u pooled rows", n_blocks, max_blocks);
    const uint64_t rows = (uint64_t)n_seqs * rows_per_seq;
    if (rows == 0 || n_blocks == 0) return BRC_OK;
    if (!q_dev || !pooled_dev || !pos0_dev || !scores_out_dev) return brc_fail(BRC_ERR_INVALID, "brc_idx_score: NULL pointer");
    if ((reinterpret_cast<uintptr_t>(q_dev) & 15u) || (reinterpret_cast<uintptr_t>(pooled_dev) & 15u))
        return brc_fail(BRC_ERR_INVALID, "brc_idx_score: query and pooled-key pointers must be 16-byte aligned");
    if (rows > 65535u) return brc_fail(BRC_ERR_UNSUPPORTED, "brc_idx_score: %llu rows in one call (at most 65535)", (unsigned long long)rows);
    brc_device_guard guard(pool->device);
    ScoreParams p;
    p.q = q_dev;
    p.pooled = pooled_dev;
    p.scores = scores_out_dev;
    p.pos0 = pos0_dev;
    p.rows_per_seq = rows_per_seq;
    p.n_blocks = n_blocks;
    p.max_blocks = max_blocks;
    p.n_head = idx_n_head;
    p.scale = scale;
    if (rows_per_seq >= 2u && idx_n_head == 4u) {
        const uint32_t tiles = n_seqs * ((rows_per_seq + SC_ROWS - 1u) / SC_ROWS);
        idx_score_rows_kernel<<<dim3((n_blocks + SC_TILE_BLOCKS - 1) / SC_TILE_BLOCKS, tiles), SC_THREADS, 0, brc_stream(stream)>>>(p);
    } else {
        idx_score_kernel<<<dim3((n_blocks + SC_BLOCKS_PER_CTA - 1) / SC_BLOCKS_PER_CTA, (uint32_t)rows), SC_THREADS, 0, brc_stream(stream)>>>(p);
    }
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"
