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
// Up to 16 query heads per kv head go to the clustered tensor-core kernel further down instead (both V layouts);
// this one serves wider head groups.
#include <cooperative_groups.h>

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


// ---------------------------------------------------------------------------------------------
// The same contract with the query heads of a kv head sharing every K / V byte (binary16 or q8_0 V, up to 16 query
// heads per kv head): the reference's apply shader for chunks loads each V row once for its 12 heads
// (shaders/qsa_attn_apply_gqa.comp:71-136); the kernel above re-reads every selected row once per QUERY head.
//
//   one thread-block CLUSTER per (row, kv head); its CTAs (four tile streams each) deal the row's selected blocks out in
//   tiles of 16 cells (4 blocks); the warps that own a stream (one per group of 8 query heads) gather a tile's K and V rows
//   with 16-byte cp.async (zero fill for cells beyond the row's position) into a 128-byte-swizzled tile, in three
//   buffers (the copies of two tiles in flight while a third is computed), and compute on the tensor cores as the dense decode kernel does: S^T[16 cells x 8 heads] = K . Q^T
//   (mma.sync m16n8k16, Q^T fragments from shared memory), online softmax in base 2 by shuffles, P transposed in
//   registers (movmatrix) and split into a binary16 head and tail, O^T += V^T . P^T with V^T fragments from ldmatrix.trans
//   (q8_0 V: the rows are gathered as they lie in the pool and the quanta reach the tensor cores as exact binary16
//   integers, the block scales folded into the probabilities);
//   the streams of a CTA merge their (m, l, O) in shared memory, and the CTAs of the cluster merge through DISTRIBUTED
//   shared memory: CTA r reads the partials of all its peers for the heads r, r + cluster size, ... and writes those
//   output rows.  No scratch in global memory, no second kernel.
// ---------------------------------------------------------------------------------------------
namespace gqa {

constexpr int GROUPS_PER_CTA = 4;   // tile streams per CTA: each owned by NT warps (one per group of 8 heads)
constexpr int NBUF = 3;             // tile buffers per stream: two tiles' copies in flight while a third is computed
constexpr int MAX_CLUSTER = 8;

constexpr float Q8_P_SCALE = 128.f;                     // see the q8_0 V product below

template <int HD, bool V_Q8>
struct Tile {
    static constexpr int GROUPS = HD / 64;               // 64-column groups
    static constexpr int SLAB = 16 * 128;                // [16 cells][64 columns] binary16
    // binary16 V: per column group a K slab then a V slab.  q8_0 V: the K slabs, then the 16 V rows as they lie in
    // the pool (HD / 32 blocks of 36 bytes each, unswizzled).
    static constexpr int GROUP_BYTES = V_Q8 ? SLAB : 2 * SLAB;
    static constexpr int VROW_BYTES = HD / 32 * 36;
    static constexpr int V_OFF = GROUPS * SLAB;
    static constexpr int BYTES = V_Q8 ? (GROUPS * SLAB + 16 * VROW_BYTES + 1023) / 1024 * 1024 : GROUPS * GROUP_BYTES;   // 16 KiB / 13 KiB at head_dim 256
    static constexpr int Q_STRIDE = HD * 2 + 16;         // bytes between heads of the query in shared memory (bank spread)
    static constexpr int CHUNKS = HD / 8;                // 16-byte chunks per K (or binary16 V) row
    static constexpr int VCHUNKS = VROW_BYTES / 16;      // 16-byte chunks per q8_0 V row
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, bool live) {
    const uint32_t n = live ? 16u : 0u;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// NT = groups of 8 query heads per kv head (1 or 2) = warps that share a tile: warp nt of a tile's owners computes heads
// 8 nt .. 8 nt + 7 over the same K / V rows, so 12 heads per kv head keep 8 warps busy on 4 tiles.
template <int HD, int NT, bool V_Q8>
__global__ void __launch_bounds__(GROUPS_PER_CTA * NT * 32, 1) sparse_gqa_kernel(const SparseParams p) {
    using T = Tile<HD, V_Q8>;
    constexpr int KSTEPS = HD / 16, MT = HD / 16;
    constexpr int THREADS = GROUPS_PER_CTA * NT * 32;
    constexpr uint32_t OWNERS = NT * 32;                 // threads that share a tile
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t cs = cluster.num_blocks(), rank = cluster.block_rank();
    extern __shared__ uint8_t sg_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(sg_raw) + 1023u) & ~uintptr_t(1023));
    uint8_t *tiles = smem;                                                   // [GROUPS_PER_CTA][NBUF][T::BYTES]
    uint8_t *q_hi = tiles + GROUPS_PER_CTA * NBUF * T::BYTES;                   // [NT * 8][Q_STRIDE] binary16 heads of the query
    uint8_t *q_lo = q_hi + NT * 8 * T::Q_STRIDE;                             // tails (f32 queries only)
    float *cta_o = reinterpret_cast<float *>(q_lo + NT * 8 * T::Q_STRIDE);   // [NT * 8][HD] this CTA's merged O
    float *cta_ml = cta_o + NT * 8 * HD;                                     // [NT * 8][2]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t grp = warp / NT, nt = warp % NT;                          // which tile stream, which 8 heads
    const uint32_t row = blockIdx.y, kvh = blockIdx.x / cs;
    const uint32_t s = row / p.rows_per_seq, t = row % p.rows_per_seq;
    const uint32_t count_listed = p.counts[row];        // asked for together with the position: neither waits for the other
    const uint32_t pos = p.pos0[s] + t;
    const uint32_t group = p.n_head / p.n_kv_head;
    const uint32_t head_base = kvh * group;
    const bool bad_pos = pos >= p.max_pos_end;
    if (bad_pos && tid == 0 && rank == 0) { atomicOr(p.status, BRC_DEV_BAD_POS); p.status[1] = pos; }

    const uint32_t count = bad_pos ? 0u : min(count_listed, p.max_ids);
    const uint32_t *ids = p.ids + (size_t)row * p.max_ids;
    const uint32_t *table = p.block_tables + (size_t)s * p.table_stride;
    const uint32_t n_tiles = (count + 3u) / 4u;
    const uint32_t stride = cs * GROUPS_PER_CTA;
    // Lane r < 16 (and its twin r + 16) resolves cell r of a tile: block r / 4 of the tile's four, cell r % 4 of the
    // block.  The way from a tile number to its rows is a chain of dependent loads (id list -> block table -> K / V
    // rows), so it is walked in three steps, one tile further ahead each: the id of tile j + 4 strides, the page of tile
    // j + 3 strides and the row copies of tile j + 2 strides are all issued while tile j is computed.
    auto fetch_id = [&](uint32_t j) -> uint32_t {
        const uint32_t li = j * 4u + ((lane & 15u) >> 2);
        return (j < n_tiles && li < count) ? ids[li] : 0xffffffffu;
    };
    auto fetch_page = [&](uint32_t id, uint32_t &cell) -> uint32_t {   // cell = 0xffffffff: nothing to read
        cell = 0xffffffffu;
        if (id == 0xffffffffu) return 0u;
        const uint32_t c = id * 4u + (lane & 3u), lp = c >> 4;
        if (c > pos || lp >= p.table_stride) return 0u;
        cell = c;
        return table[lp];
    };
    const uint32_t j_first = rank * GROUPS_PER_CTA + warp / NT;
    // The first four tiles' ids are asked for before the row's count has arrived (one load less in the chain in front of
    // the first tile); what lies beyond the count is dropped below, once both are here.
    auto id_at = [&](uint32_t j) -> uint32_t {
        const uint32_t li = j * 4u + ((lane & 15u) >> 2);
        return li < p.max_ids ? ids[li] : 0xffffffffu;
    };
    auto within = [&](uint32_t id, uint32_t j) -> uint32_t {
        return (j < n_tiles && j * 4u + ((lane & 15u) >> 2) < count) ? id : 0xffffffffu;
    };
    uint32_t id_a = id_at(j_first), id_b = id_at(j_first + stride), id_c = id_at(j_first + 2u * stride);
    uint32_t id_d = id_at(j_first + 3u * stride);

    // ---- the query heads of this kv head into shared memory: binary16 head (and tail of an f32 query)
    for (uint32_t i = tid; i < NT * 8 * (HD / 2); i += THREADS) {
        const uint32_t h = i / (HD / 2), d2 = (i % (HD / 2)) * 2;
        float2 x = make_float2(0.f, 0.f);
        if (h < group) {
            const size_t qo = ((size_t)row * p.n_head + head_base + h) * HD + d2;
            if (p.q_f32) x = *reinterpret_cast<const float2 *>(static_cast<const float *>(p.q) + qo);
            else x = __half22float2(*reinterpret_cast<const __half2 *>(static_cast<const __half *>(p.q) + qo));
        }
        const __half2 hi = __floats2half2_rn(x.x, x.y);
        const float2 hf = __half22float2(hi);
        *reinterpret_cast<__half2 *>(q_hi + h * T::Q_STRIDE + d2 * 2) = hi;
        *reinterpret_cast<__half2 *>(q_lo + h * T::Q_STRIDE + d2 * 2) = __floats2half2_rn(x.x - hf.x, x.y - hf.y);
    }
    __syncthreads();

    uint8_t *my_tiles = tiles + (size_t)grp * NBUF * T::BYTES;
    auto owners_sync = [&]() {
        if (NT == 1) __syncwarp();
        else brc::named_bar_sync(1 + grp, OWNERS);
    };

    // Copies this warp's part of a tile, whose cells were resolved to (page, cell), into buffer b; returns the mask of live cells.
    auto gather = [&](uint32_t page, uint32_t cell, uint32_t b) -> uint32_t {
        bool live = false;
        size_t src_row = 0;
        if (cell != 0xffffffffu) {
            if (page < p.n_pages) {
                live = true;
                src_row = ((size_t)page * p.n_kv_head + kvh) * 16u + (cell & 15u);   // row of the layer's K (and V) pool
            } else if (lane < 16 && nt == 0) {
                atomicOr(p.status, BRC_DEV_BAD_PAGE);
                p.status[1] = page;
            }
        }
        const uint32_t mask = __ballot_sync(0xffffffffu, live) & 0xffffu;
        const uint32_t base = brc::smem_u32(my_tiles + (size_t)b * T::BYTES);
        if (!V_Q8) {
#pragma unroll
            for (uint32_t i = 0; i < 2u * 16u * T::CHUNKS / OWNERS; ++i) {
                const uint32_t idx = i * OWNERS + nt * 32u + lane;
                const uint32_t which = idx / (16u * T::CHUNKS);                 // 0: K, 1: V
                const uint32_t rr = (idx / T::CHUNKS) % 16u, ch = idx % T::CHUNKS;
                const size_t off = __shfl_sync(0xffffffffu, src_row, rr) * (HD * 2u);
                const bool lv = (mask >> rr) & 1u;
                const uint32_t dst = base + (ch >> 3) * T::GROUP_BYTES + which * T::SLAB + rr * 128u + (((ch & 7u) ^ (rr & 7u)) << 4);
                cp_async_16(dst, (which ? p.v_layer : p.k_layer) + off + ch * 16u, lv);
            }
        } else {
            // K rows into the swizzled slabs, then the V rows whole.  A dead cell's destination is zero-filled: quanta
            // of zero under a scale of zero.
            constexpr uint32_t K_CH = 16u * T::CHUNKS, ALL_CH = K_CH + 16u * T::VCHUNKS;
#pragma unroll
            for (uint32_t i = 0; i < (ALL_CH + OWNERS - 1u) / OWNERS; ++i) {
                const uint32_t idx = i * OWNERS + nt * 32u + lane;
                const bool in = idx < ALL_CH, is_k = idx < K_CH;
                const uint32_t v_idx = in && !is_k ? idx - K_CH : 0u;
                const uint32_t rr = is_k ? idx / T::CHUNKS : v_idx / T::VCHUNKS;
                const uint32_t ch = is_k ? idx % T::CHUNKS : v_idx % T::VCHUNKS;
                const size_t r = __shfl_sync(0xffffffffu, src_row, rr);
                const bool lv = (mask >> rr) & 1u;
                if (is_k)
                    cp_async_16(base + (ch >> 3) * T::GROUP_BYTES + rr * 128u + (((ch & 7u) ^ (rr & 7u)) << 4),
                                p.k_layer + r * (HD * 2u) + ch * 16u, lv);
                else if (in)
                    cp_async_16(base + T::V_OFF + rr * T::VROW_BYTES + ch * 16u, p.v_layer + r * T::VROW_BYTES + ch * 16u, lv);
            }
        }
        return mask;
    };

    // fragment lane constants (as in the dense decode kernel)
    const uint32_t t0 = lane >> 2, h0 = (lane & 3u) * 2u;
    const uint32_t k_r = (lane & 7u) + ((lane >> 3) & 1u) * 8u, k_x = (lane >> 4) ^ (k_r & 7u), k_lane = k_r * 128u;
    const uint32_t v_r = (lane & 7u) + (lane >> 4) * 8u, v_x = ((lane >> 3) & 1u) ^ (v_r & 7u), v_lane = T::SLAB + v_r * 128u;
    // B operand of S^T = K . Q^T: head 8 nt + t0, elements 16 ks + 2 (lane & 3) + {0, 1} and + 8
    const uint32_t q_lane = brc::smem_u32(q_hi) + (nt * 8u + t0) * T::Q_STRIDE + (lane & 3u) * 4u;
    const uint32_t q_lo_off = (uint32_t)(q_lo - q_hi);

    float o[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    uint32_t j = j_first, buf = 0;
    uint32_t mask = 0, mask_1 = 0, mask_2 = 0;     // live cells of tile j, j + stride, j + 2 strides
    uint32_t cell_a, cell_b, cell_c;
    id_a = within(id_a, j_first), id_b = within(id_b, j_first + stride);
    id_c = within(id_c, j_first + 2u * stride), id_d = within(id_d, j_first + 3u * stride);
    uint32_t page_a = fetch_page(id_a, cell_a), page_b = fetch_page(id_b, cell_b), page_c = fetch_page(id_c, cell_c);
    if (j < n_tiles) mask = gather(page_a, cell_a, 0);
    cp_async_commit();
    if (j + stride < n_tiles) mask_1 = gather(page_b, cell_b, 1);
    cp_async_commit();
    for (; j < n_tiles; j += stride, buf = buf + 1u == NBUF ? 0u : buf + 1u) {
        if (j + 2u * stride < n_tiles) mask_2 = gather(page_c, cell_c, buf >= 1u ? buf - 1u : buf + 2u);   // (buf + 2) % 3
        cp_async_commit();
        page_c = fetch_page(id_d, cell_c);          // tile j + 3 strides: used in the next iteration
        id_d = fetch_id(j + 4u * stride);           // tile j + 4 strides: used in the next iteration
        cp_async_wait<NBUF - 1>();
        owners_sync();        // every owner's copies of this tile have landed
        const uint32_t sbase = brc::smem_u32(my_tiles + (size_t)buf * T::BYTES);
        // ---- S^T = K . Q^T
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t af[4];
            brc::ldmatrix_x4(af, sbase + (ks >> 2) * T::GROUP_BYTES + k_lane + ((k_x ^ ((ks & 3) * 2u)) << 4));
            const uint32_t qa = q_lane + ks * 32u;
            uint32_t b0, b1;
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(b0) : "r"(qa));
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(b1) : "r"(qa + 16u));
            if (ks & 1) brc::mma_16816(sb, af, b0, b1); else brc::mma_16816(sa, af, b0, b1);
            if (p.q_f32) {
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(b0) : "r"(qa + q_lo_off));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(b1) : "r"(qa + q_lo_off + 16u));
                if (ks & 1) brc::mma_16816(sb, af, b0, b1); else brc::mma_16816(sa, af, b0, b1);
            }
        }
        float sc[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[i] = (sa[i] + sb[i]) * p.scale_log2;
        if (!((mask >> t0) & 1u)) sc[0] = sc[1] = -INFINITY;
        if (!((mask >> (t0 + 8u)) & 1u)) sc[2] = sc[3] = -INFINITY;
        float x0 = fmaxf(sc[0], sc[2]), x1 = fmaxf(sc[1], sc[3]);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, off));
            x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, off));
        }
        const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
        const float z0 = n0 == -INFINITY ? 0.f : n0, z1 = n1 == -INFINITY ? 0.f : n1;   // no live cell so far
        const float al0 = brc::fast_exp2(m0 - z0), al1 = brc::fast_exp2(m1 - z1);
        m0 = n0;
        m1 = n1;
        const float p0 = brc::fast_exp2(sc[0] - z0), p1 = brc::fast_exp2(sc[1] - z1);
        const float p2 = brc::fast_exp2(sc[2] - z0), p3 = brc::fast_exp2(sc[3] - z1);
        l0 = l0 * al0 + (p0 + p2);
        l1 = l1 * al1 + (p1 + p3);
        if (__any_sync(0xffffffffu, (al0 != 1.f) | (al1 != 1.f))) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                o[mt][0] *= al0;
                o[mt][1] *= al1;
                o[mt][2] *= al0;
                o[mt][3] *= al1;
            }
        }
        const __half2 ph01 = __floats2half2_rn(p0, p1), ph23 = __floats2half2_rn(p2, p3);
        const float2 f01 = __half22float2(ph01), f23 = __half22float2(ph23);
        const uint32_t bh0 = brc::movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph01));
        const uint32_t bh1 = brc::movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph23));
        const uint32_t bl0 = brc::movmatrix_trans(brc::pack_half2(p0 - f01.x, p1 - f01.y));
        const uint32_t bl1 = brc::movmatrix_trans(brc::pack_half2(p2 - f23.x, p3 - f23.y));
        if (!V_Q8) {
            // ---- O^T += V^T . P^T
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t af[4];
                brc::ldmatrix_x4_trans(af, sbase + (mt >> 2) * T::GROUP_BYTES + v_lane + ((v_x ^ ((mt & 3) * 2u)) << 4));
                brc::mma_16816(o[mt], af, bh0, bh1);
                brc::mma_16816(o[mt], af, bl0, bl1);
            }
        } else {
            // ---- q8_0 V (VLayout::Q8_0, shaders/qsa_attn_apply.comp with BRECCIA_KV_Q8V): as in the dense decode
            //      kernel.  The probabilities in the B-operand layout back in f32 (this lane: cells 2t, 2t + 1, 2t + 8,
            //      2t + 9 of head g), times 2^7 so that the binary16 tail of probability x scale stays normal; each
            //      block's scale is folded into them (head + tail again), and the quanta go to the tensor cores as EXACT
            //      binary16 integers (bits 0x6400 | (q ^ 0x80) are 1024 + q + 128; 1152 is subtracted).  Rows of the
            //      product are permuted: tile 2 blk holds values 32 blk + 4 g + {0, 1}, tile 2 blk + 1 values + {2, 3}.
            const float2 h0f = __half22float2(*reinterpret_cast<const __half2 *>(&bh0)), t0f = __half22float2(*reinterpret_cast<const __half2 *>(&bl0));
            const float2 h1f = __half22float2(*reinterpret_cast<const __half2 *>(&bh1)), t1f = __half22float2(*reinterpret_cast<const __half2 *>(&bl1));
            const float pb0 = (h0f.x + t0f.x) * Q8_P_SCALE, pb1 = (h0f.y + t0f.y) * Q8_P_SCALE;
            const float pb2 = (h1f.x + t1f.x) * Q8_P_SCALE, pb3 = (h1f.y + t1f.y) * Q8_P_SCALE;
            const uint32_t vrow = sbase + T::V_OFF + (lane & 3u) * 2u * T::VROW_BYTES;
#pragma unroll
            for (int blk = 0; blk < HD / 32; ++blk) {
                const uint32_t at = vrow + blk * 36u;
                float s0, s1, s2, s3;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s0) : "r"(at));
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s1) : "r"(at + T::VROW_BYTES));
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s2) : "r"(at + 8u * T::VROW_BYTES));
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s3) : "r"(at + 9u * T::VROW_BYTES));
                const float w0 = pb0 * s0, w1 = pb1 * s1, w2 = pb2 * s2, w3 = pb3 * s3;
                const __half2 wh01 = __floats2half2_rn(w0, w1), wh23 = __floats2half2_rn(w2, w3);
                const float2 g01 = __half22float2(wh01), g23 = __half22float2(wh23);
                const uint32_t ph0 = *reinterpret_cast<const uint32_t *>(&wh01), ph1 = *reinterpret_cast<const uint32_t *>(&wh23);
                const uint32_t pl0 = brc::pack_half2(w0 - g01.x, w1 - g01.y), pl1 = brc::pack_half2(w2 - g23.x, w3 - g23.y);
                uint32_t x0, x1, x2, x3;
                const uint32_t qa = at + 4u + (lane >> 2) * 4u;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x0) : "r"(qa));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x1) : "r"(qa + T::VROW_BYTES));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x2) : "r"(qa + 8u * T::VROW_BYTES));
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x3) : "r"(qa + 9u * T::VROW_BYTES));
                x0 ^= 0x80808080u, x1 ^= 0x80808080u, x2 ^= 0x80808080u, x3 ^= 0x80808080u;
                const uint32_t ya = __byte_perm(x0, x1, 0x5410), yb = __byte_perm(x0, x1, 0x7632);   // bytes (0, 1) and (2, 3) of cells 2t, 2t + 1
                const uint32_t za = __byte_perm(x2, x3, 0x5410), zb = __byte_perm(x2, x3, 0x7632);   // of cells 2t + 8, 2t + 9
                const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));        // 1152
                auto ints = [bias](uint32_t y, uint32_t sel) {
                    const uint32_t r = __byte_perm(y, 0x64646464u, sel);
                    const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&r), bias);
                    return *reinterpret_cast<const uint32_t *>(&v);
                };
                const uint32_t a_lo[4] = {ints(ya, 0x4240), ints(ya, 0x4341), ints(za, 0x4240), ints(za, 0x4341)};
                const uint32_t a_hi[4] = {ints(yb, 0x4240), ints(yb, 0x4341), ints(zb, 0x4240), ints(zb, 0x4341)};
                brc::mma_16816(o[2 * blk], a_lo, ph0, ph1);
                brc::mma_16816(o[2 * blk], a_lo, pl0, pl1);
                brc::mma_16816(o[2 * blk + 1], a_hi, ph0, ph1);
                brc::mma_16816(o[2 * blk + 1], a_hi, pl0, pl1);
            }
        }
        owners_sync();   // the buffer is refilled in the next iteration, by all owners
        mask = mask_1;
        mask_1 = mask_2;
    }
    cp_async_wait<0>();
    __syncthreads();    // every warp is done with its tiles: their memory now carries the warps' partials

    // ---- warps -> CTA: (m, l) and O of every tile stream through shared memory, merged per head
    float *w_o = reinterpret_cast<float *>(tiles);                          // [GROUPS_PER_CTA][NT * 8][HD]
    float *w_ml = w_o + GROUPS_PER_CTA * NT * 8 * HD;                       // [GROUPS_PER_CTA][NT * 8][2]
    {
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
        }
        float *wo = w_o + ((size_t)grp * NT * 8 + nt * 8) * HD;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            // binary16 V: rows t0 and t0 + 8 of tile mt; q8_0 V: the permuted rows of the product above
            const uint32_t d0 = V_Q8 ? (mt >> 1) * 32 + t0 * 4 + (mt & 1) * 2 : mt * 16 + t0;
            const uint32_t d1 = V_Q8 ? d0 + 1 : d0 + 8;
            constexpr float back = V_Q8 ? 1.f / Q8_P_SCALE : 1.f;   // undoes the factor on the q8_0 probabilities (exact)
            wo[h0 * HD + d0] = o[mt][0] * back;
            wo[(h0 + 1) * HD + d0] = o[mt][1] * back;
            wo[h0 * HD + d1] = o[mt][2] * back;
            wo[(h0 + 1) * HD + d1] = o[mt][3] * back;
        }
        if (lane < 4) {
            float *ml = w_ml + ((size_t)grp * NT * 8 + nt * 8 + h0) * 2;
            ml[0] = m0, ml[1] = l0, ml[2] = m1, ml[3] = l1;
        }
    }
    __syncthreads();
    for (uint32_t h = warp; h < group; h += THREADS / 32) {     // a warp per head
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < GROUPS_PER_CTA; ++w)
            if (w_ml[(w * NT * 8 + h) * 2 + 1] > 0.f) M = fmaxf(M, w_ml[(w * NT * 8 + h) * 2]);
        float L = 0.f, wt[GROUPS_PER_CTA];
#pragma unroll
        for (int w = 0; w < GROUPS_PER_CTA; ++w) {
            const float lw = w_ml[(w * NT * 8 + h) * 2 + 1];
            wt[w] = lw > 0.f ? exp2f(w_ml[(w * NT * 8 + h) * 2] - M) : 0.f;
            L += wt[w] * lw;
        }
        for (uint32_t d = lane; d < HD; d += 32) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < GROUPS_PER_CTA; ++w) acc += wt[w] * w_o[((size_t)w * NT * 8 + h) * HD + d];
            cta_o[h * HD + d] = acc;
        }
        if (lane == 0) { cta_ml[h * 2] = M; cta_ml[h * 2 + 1] = L; }
    }
    cluster.sync();

    // ---- CTAs -> output: CTA `rank` finishes heads rank, rank + cs, ... from the partials of all its peers
    for (uint32_t h = rank; h < group; h += cs) {
        float M = -INFINITY, Ms[MAX_CLUSTER], Ls[MAX_CLUSTER];
#pragma unroll
        for (uint32_t r = 0; r < MAX_CLUSTER; ++r) {
            if (r < cs) {
                const float *ml = cluster.map_shared_rank(cta_ml, r);
                Ms[r] = ml[h * 2];
                Ls[r] = ml[h * 2 + 1];
                if (Ls[r] > 0.f) M = fmaxf(M, Ms[r]);
            }
        }
        float L = 0.f, wt[MAX_CLUSTER];
#pragma unroll
        for (uint32_t r = 0; r < MAX_CLUSTER; ++r) {
            wt[r] = (r < cs && Ls[r] > 0.f) ? exp2f(Ms[r] - M) : 0.f;
            if (r < cs) L += wt[r] * Ls[r];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;    // a row with no selected live cell yields zeros
        for (uint32_t d = tid; d < HD; d += THREADS) {
            float acc = 0.f;
#pragma unroll
            for (uint32_t r = 0; r < MAX_CLUSTER; ++r)
                if (r < cs) acc += wt[r] * cluster.map_shared_rank(cta_o, r)[h * HD + d];
            float v = acc * inv;
            const size_t orow = (size_t)row * p.n_head + head_base + h;
            if (p.gate) v *= sp_sigmoid(p.gate[orow * p.gate_head_stride + d]);
            p.out[orow * HD + d] = v;
        }
    }
    cluster.sync();   // nobody leaves while a peer may still read its shared memory
}

template <int HD, bool V_Q8>
constexpr uint32_t smem_bytes(int nt) {
    return 1024u + GROUPS_PER_CTA * NBUF * Tile<HD, V_Q8>::BYTES + 2u * nt * 8 * Tile<HD, V_Q8>::Q_STRIDE + nt * 8 * HD * 4u + nt * 8 * 2 * 4u + 64u;
}

template <int HD, int NT, bool V_Q8>
cudaError_t launch(const SparseParams &p, uint32_t rows, uint32_t n_kv_head, uint32_t cs, cudaStream_t st) {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(sparse_gqa_kernel<HD, NT, V_Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<HD, V_Q8>(NT));
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_kv_head * cs, rows);
    cfg.blockDim = dim3(GROUPS_PER_CTA * NT * 32);
    cfg.dynamicSmemBytes = smem_bytes<HD, V_Q8>(NT);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sparse_gqa_kernel<HD, NT, V_Q8>, p);
}

}  // namespace gqa

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
    const uint32_t group = n_head / pool->n_kv_head;
    if (group <= 16u) {
        // one cluster per (row, kv head): as many CTAs per cluster (a power of two, at most 8) as keep every SM busy
        const uint64_t units = rows * pool->n_kv_head;
        uint32_t cs = 1;
        while (cs < (uint32_t)gqa::MAX_CLUSTER && units * cs * 2u <= sms) cs *= 2u;
        cudaError_t e;
        const uint32_t r32 = (uint32_t)rows, nkv = pool->n_kv_head;
        if (pool->v_q8) {
            if (hd == 256) e = group <= 8u ? gqa::launch<256, 1, true>(p, r32, nkv, cs, st) : gqa::launch<256, 2, true>(p, r32, nkv, cs, st);
            else e = group <= 8u ? gqa::launch<128, 1, true>(p, r32, nkv, cs, st) : gqa::launch<128, 2, true>(p, r32, nkv, cs, st);
        } else {
            if (hd == 256) e = group <= 8u ? gqa::launch<256, 1, false>(p, r32, nkv, cs, st) : gqa::launch<256, 2, false>(p, r32, nkv, cs, st);
            else e = group <= 8u ? gqa::launch<128, 1, false>(p, r32, nkv, cs, st) : gqa::launch<128, 2, false>(p, r32, nkv, cs, st);
        }
        brc_stage_end(pool, BRC_STAGE_ATTN_PARTIAL, st);
        if (e != cudaSuccess) return brc_fail(BRC_ERR_CUDA, "brc_paged_sparse_attn: launch failed: %s", cudaGetErrorString(e));
        BRC_CUDA(cudaGetLastError());
        return BRC_OK;
    }
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
