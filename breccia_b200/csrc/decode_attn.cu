// Paged GQA decode attention for sm_100a: one split-KV kernel with an in-kernel log-sum-exp combine.
//
// Replaces, for a batch of sequences at T = 1, the reference's four dispatches
// scores -> softmax -> split-K apply -> reduce (crates/breccia-kernels/src/qsa/mod.rs:1439-1461,
// 1491-1521; shaders qsa_attn_scores_small.comp, ops_softmax.comp, qsa_attn_apply_split.comp,
// qsa_attn_apply_reduce.comp).  The reference materialises the score matrix in memory and re-reads V
// once per query head; here every cached byte is read from HBM exactly once per step:
//
//   * work unit = (sequence, group of KVB kv heads); KVB = 2 when the number of kv heads is even, so a
//     page's rows of two neighbouring kv heads (contiguous in the pool) travel together.  The pages of
//     all units form one flat list of "page-units", cut into contiguous shares of equal cost, one per CTA
//     (one CTA per SM; cost = pages plus a surcharge per unit touched), so every SM is busy for the same
//     time whatever the length distribution;
//   * a producer warp walks the block table and issues, per page-unit, one TMA tiled load per
//     64-column group: a 3-D box [64 columns][16 KVB rows][K|V] over a view that spans the K and the
//     V pool (128-byte swizzle), 8 KiB per operation at KVB = 2.  Measured on B200, a TMA operation
//     costs >= ~215 SM cycles whatever its size, so 4 KiB operations cap a SM at ~19 B/cycle while
//     8 KiB operations reach the HBM limit (~26 B/cycle/SM); this is why two kv heads share a box.
//     (Opt-in, see stage_in_one_operation(): one 4-D box [64][16 KVB][K|V][column groups] per page-unit.)
//     Stages of a shared-memory ring are guarded by full/empty mbarriers;
//   * four consumer warps: warp w serves kv head (w % KVB) of every (w / KVB)-th page-unit.  Per page:
//     S^T[16 cells x 8 heads] = K . Q^T with mma.sync m16n8k16 (K fragments by ldmatrix from the
//     swizzled tile, Q^T fragments resident in registers), online softmax in base 2 with warp shuffles
//     across the cell dimension, the probabilities transposed in registers by movmatrix into the B
//     operand, and O^T[head_dim x 8 heads] += V^T . P^T with V^T fragments from ldmatrix.trans.  P is
//     split into a binary16 head and tail so the product carries ~22 significant bits;
//   * at the end of a unit's share the warps merge (m, l, O) per kv head through shared memory, write
//     one partial per kv head and add one to the unit's ticket.  When a CTA has streamed all of its share
//     it merges the units it holds pieces of TOGETHER with the other CTAs that hold pieces of them: each
//     waits (bounded) until the ticket shows every piece written and takes an equal run of the unit's
//     (row, column) items - log-sum-exp weights, normalisation, gate, output rows.  The pieces of a unit
//     complete at the same moment (the end of their CTAs' streaming), so the merge costs a few trips to
//     L2 however many CTAs a unit spans.  The launch is cooperative (all CTAs resident), and there is no
//     second kernel;
//   * a decode step's KV append can ride along: the CTA that is about to stream the page holding a
//     sequence's newest cell first writes that cell (same encoding and address rule as the append
//     kernel), fenced against its own TMA read;
//   * one launch can cover several layers: the flat list then runs over (layer, unit, page) and is cut
//     into the same equal shares, so the launch ramp, the schedule scan and the tail are paid once per
//     decode token instead of once per layer, and most units lie inside one CTA's share;
//   * split-KV across GPUs rides in the same launch: the CTAs that merge a unit store its merged
//     (acc, m, l) into this rank's slot of every peer's receive buffer with plain global stores over
//     NVLink - no flags, no fences: an empty slot holds 0xFFFFFFFF words, and the same CTAs then poll
//     (bounded), segment by segment, all ranks' slots of their own buffer, merge the ranks' rows, write
//     the output and empty the slots again: the exchange of all layers of a token is one round of stores
//     at the end of one launch.  No load targets peer memory.
//
// HBM-bound by design: 8 FLOP per cached byte, all of it on the tensor pipe.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

// Consumer warps: 4 keep up with HBM on binary16 V at head_dim 256 (one per scheduler); the q8_0 V path issues about
// three times the instructions per page (the quanta are converted in registers), and at head_dim 128 a page brings half
// the bytes for the same softmax round and ring hand-over, so those run 6 to hide the latency of what they issue
// (head_dim 128: +1 % measured; 5.0 - 5.3 TB/s is what its page-sized stages allow).
__host__ __device__ constexpr int consumer_warps(bool v_q8, int head_dim) { return v_q8 || head_dim == 128 ? 6 : 4; }
constexpr int MAX_UNITS = 2048;            // (sequence, kv-head group) units per launch
constexpr int MAX_CTAS = 256;              // CTAs of a launch (one per SM)
constexpr int GROUP_TILE = 8;              // query heads per kv head held by one n-tile
constexpr uint32_t SMEM_LIMIT = 232448;    // 227 KiB opt-in maximum per CTA
constexpr uint64_t WAIT_NS = 1000000000ull;  // one second: far beyond any legitimate wait here
constexpr float Q8_P_SCALE = 128.f;          // see the q8_0 V path of the kernel

template <int HD, int KVB, bool VQ8 = false>
struct Cfg {
    static constexpr int NW = consumer_warps(VQ8, HD);
    static constexpr int NTHREADS = (NW + 1) * 32;         // + one producer warp
    static constexpr int KSTEPS = HD / 16;
    static constexpr int MT = HD / 16;
    static constexpr int BOXES = HD / 64;                  // 64-column groups = TMA operations per stage (per K, or per K|V pair)
    static constexpr int ROWS = 16 * KVB;                  // pool rows per box: 16 cells of KVB kv heads
    static constexpr int SLAB_BYTES = ROWS * 128;          // one [rows][64 columns] slab
    // binary16 V: [group][K slab | V slab].  q8_0 V: the K slabs, then the V rows as they lie in the pool
    // ([rows][HD / 32 blocks of 36 bytes], unswizzled).
    static constexpr int GROUP_BYTES = VQ8 ? SLAB_BYTES : 2 * SLAB_BYTES;   // from one column group of K to the next
    static constexpr int VROW_BYTES = HD / 32 * 36;
    static constexpr int VROW_WORDS = VROW_BYTES / 4;
    static constexpr int V_OFF = BOXES * SLAB_BYTES;       // q8_0: where the V rows start in a stage
    static constexpr int TX_BYTES = VQ8 ? BOXES * SLAB_BYTES + ROWS * VROW_BYTES : BOXES * 2 * SLAB_BYTES;   // bytes a stage receives
    static constexpr int STAGE_BYTES = (TX_BYTES + 1023) / 1024 * 1024;     // stages start on the swizzle pattern's period
    static constexpr int NWP = NW / KVB;                   // warps that share one kv head (page interleave)
    static constexpr int OPAD = HD / 2 + 4;                // padded row of the merge scratch (half of head_dim)
    static constexpr int SCRATCH_WARP = GROUP_TILE * OPAD + 16;  // floats per warp
    static constexpr int SCRATCH_BYTES = NW * SCRATCH_WARP * 4;
    static constexpr int PREFIX_BYTES = (MAX_UNITS + 4) * 4;
    static constexpr int NZ_BYTES = (MAX_UNITS + 8) * 2;   // units with pages before unit u (16-bit)
    static constexpr int CUT_BYTES = (MAX_CTAS + 4) * 4;   // where every CTA's share begins
    static constexpr int BAR_BYTES = 1024;
    static constexpr int FIXED_BYTES = SCRATCH_BYTES + PREFIX_BYTES + NZ_BYTES + CUT_BYTES + BAR_BYTES + 1024 /*alignment slack*/;
};

struct DecodeParams {
    const void *q;                 // [n_seqs][n_head][HD]
    const uint32_t *block_tables;  // [n_seqs][table_stride]
    const uint32_t *seq_lens;      // [n_seqs]
    float *part_acc;               // [slots][KVB][GROUP_TILE][HD]
    float *part_ml;                // [slots][KVB][GROUP_TILE][2]
    uint32_t *done;                // [layer bank][2048] ticket words of the units (see TICKET_ALL)
    float *out;                    // final [n_seqs][n_head][HD]; partial mode: merged acc, same shape
    float *out_ml;                 // partial mode: [n_seqs][n_head][2] (m, l); nullptr = final output
    const float *gate;             // nullable
    uint32_t gate_head_stride;
    // fused append (nullable): this step's K/V of the cell seq_len - 1 of every sequence,
    // [n_seqs][n_kv_head * HD], written into the pool by the CTA that streams that cell's page
    const void *k_new;
    const void *v_new;
    uint32_t kv_new_f32;           // 1: f32 sources, 0: binary16
    uint8_t *k_base;               // base of the K pool (row 0 of the TMA view)
    uint64_t v_offset;             // bytes from the K pool to the V pool
    uint32_t *status;
    uint32_t n_seqs, table_stride, max_seq_len;
    uint32_t n_kv_head, group, n_head;   // group = query heads per kv head handled by THIS launch (<= GROUP_TILE)
    uint32_t group_all, head0;           // query heads per kv head in q / out, and the first of them this launch takes
    uint32_t n_pages;    // pages per layer
    uint32_t layer_row0; // first row of the launch's first layer in the TMA view
    uint32_t n_stages;
    float scale_log2;    // scale * log2(e)
    // layers of this launch: per-layer arrays lie these many ELEMENTS of their own type apart
    uint32_t n_layers;
    uint32_t layer_rows;           // rows of one layer in the TMA view
    uint64_t q_layer_stride;       // elements of q's type
    uint64_t out_layer_stride;     // floats
    uint64_t out_ml_layer_stride;  // floats
    uint64_t gate_layer_stride;    // floats
    uint64_t kv_new_layer_stride;  // elements of k_new's type
    // split-KV across GPUs (world > 1): merged partials go to the receive buffers, the output is written by
    // the cross-rank merge at the end of the launch
    uint32_t world, rank;
    uint32_t unit_items;           // units the receive buffers were sized for
    uint32_t rows_total;           // n_layers * n_seqs * n_head: rows of the partial as laid out in a slot
    uint8_t *peer_recv[BRC_MAX_WORLD];
    uint64_t slot_stride, bank_stride, push_offset;   // push_offset: where the banks of this exchange begin in a receive buffer
    uint32_t *calls;               // exchanges completed so far on this rank (device-resident epoch)
    uint32_t *fin_ticket;          // CTAs of this launch that have finished
    uint64_t wait_ns;
    uint32_t unit_cost;            // page-units charged per unit with pages when the list is cut into shares
    const uint32_t *cut_prefix;    // nullable: [CTAs] where CTA i's share begins, as a fraction of the launch's cost x 2^32
    uint32_t one_op;               // binary16 V: the second tensor map is the 4-D view that brings a whole stage in one operation;
                                   // q8_0 V: the first one is the 3-D view of K that brings all K slabs in one
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait on an mbarrier phase: gives up after WAIT_NS of wall time (or 2^30 polls).
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity) {
    if (brc::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        if (brc::mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && globaltimer_ns() - t0 > WAIT_NS) return false;
    }
    return false;
}

__device__ __forceinline__ uint32_t pages_of(uint32_t len) { return (len + 15u) >> 4; }

// Largest u in [0, n_units) with S[u] <= g  (S ascending, S[0] = 0).
__device__ __forceinline__ uint32_t unit_of(const uint32_t *S, uint32_t n_units, uint32_t g) {
    uint32_t lo = 0, hi = n_units;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (S[mid] <= g) lo = mid; else hi = mid;
    }
    return lo;
}

// Shares: CTA i streams the page-units [B[i], B[i + 1]) of the flat list; the table is built at the start of the
// kernel (see there).  The share that holds page-unit g: the one with B[i] <= g < B[i + 1].
__device__ __forceinline__ uint32_t share_of(const uint32_t *B, uint32_t n_cta, uint32_t g) {
    uint32_t lo = 0, hi = n_cta;            // B[lo] <= g, B[hi] > g
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (B[mid] <= g) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ float sigmoid_f32(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

// CTAs whose share meets the page-unit range [first_g, last_g].
__device__ __forceinline__ void share_range(const uint32_t *B, uint32_t n_cta, uint32_t first_g, uint32_t last_g, uint32_t &i_lo, uint32_t &i_hi) {
    i_lo = share_of(B, n_cta, first_g);
    i_hi = share_of(B, n_cta, last_g);
}

// A unit of a launch that covers several layers: flat index over (layer, unit) and its parts.
struct UnitRef {
    uint32_t U, layer, u;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *ptr) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

__device__ __forceinline__ void st_release_sys(uint32_t *ptr, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ptr), "r"(v) : "memory");
}

// The exchange carries no flags: a slot of a receive buffer that nothing has been stored to yet holds the word
// PUSH_EMPTY everywhere (a NaN pattern that no arithmetic produces; a pusher that would send it sends the canonical
// NaN instead), every 16-byte segment and every (m, l) pair is polled by the very thread that consumes it, and the
// consumer puts PUSH_EMPTY back when it has read it.  So no store has to be ordered after another one and the
// senders need neither a fence nor a count of who has stored: what is there is there.  A bank is reused four
// exchanges later, which a peer cannot begin before this rank has finished the launch that emptied it.
constexpr uint32_t PUSH_EMPTY = 0xffffffffu;

__device__ __forceinline__ float keep_off_empty(float v) { return __float_as_uint(v) == PUSH_EMPTY ? __uint_as_float(0x7fffffffu) : v; }

__device__ __forceinline__ float4 ld_volatile_f4(const void *ptr) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ float2 ld_volatile_f2(const void *ptr) {
    float2 v;
    asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(ptr) : "memory");
    return v;
}
__device__ __forceinline__ bool landed(float4 v) {
    return __float_as_uint(v.x) != PUSH_EMPTY && __float_as_uint(v.y) != PUSH_EMPTY && __float_as_uint(v.z) != PUSH_EMPTY &&
           __float_as_uint(v.w) != PUSH_EMPTY;
}
__device__ __forceinline__ bool landed(float2 v) { return __float_as_uint(v.x) != PUSH_EMPTY && __float_as_uint(v.y) != PUSH_EMPTY; }

// Byte offset, inside any rank's receive buffer, of row R of THIS rank's partial in bank `bank`:
// acc [rows_total][HD] f32, then (m, l) [rows_total][2] f32.
__device__ __forceinline__ uint64_t push_acc_off(const DecodeParams &p, uint32_t bank, uint32_t src, size_t R, uint32_t hd, uint32_t d) {
    return p.push_offset + (uint64_t)bank * p.bank_stride + (uint64_t)src * p.slot_stride + (R * hd + d) * 4u;
}
__device__ __forceinline__ uint64_t push_ml_off(const DecodeParams &p, uint32_t bank, uint32_t src, size_t R, uint32_t hd) {
    return p.push_offset + (uint64_t)bank * p.bank_stride + (uint64_t)src * p.slot_stride + ((size_t)p.rows_total * hd + R * 2u) * 4u;
}

// Ticket word of a unit: the CTA that has written piece j of the unit's k pieces adds piece_weight(j, k); the
// weights of a unit's pieces add up to exactly 2^16 and no smaller group of them does, so the low 16 bits are zero
// exactly when no piece or every piece is written - and a CTA that has added its own weight can only see the
// second.  Nothing is ever cleared: every launch adds 2^16 per unit it streams, whatever k is this time (the
// high bits count launches and wrap harmlessly).
constexpr uint32_t TICKET_ALL = 1u << 16, TICKET_LOW = TICKET_ALL - 1u;

__device__ __forceinline__ uint32_t piece_weight(uint32_t j, uint32_t k) { return ((j + 1u) << 16) / k - (j << 16) / k; }

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *ptr) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

// Which of the shares i_lo .. i_hi hold pages (a unit's pieces): k of them, this CTA's is the j-th.  With `dense`
// no share is empty and the answer is arithmetic.  One thread's view; no shared memory.
__device__ __forceinline__ void piece_of(const uint32_t *B, bool dense, uint32_t i_lo, uint32_t i_hi, uint32_t &j, uint32_t &k) {
    if (dense) {
        k = i_hi - i_lo + 1;
        j = blockIdx.x - i_lo;
        return;
    }
    uint32_t n = 0, mine = 0;
    for (uint32_t i = i_lo; i <= i_hi; ++i)
        if (B[i] != B[i + 1]) {
            if (i == blockIdx.x) mine = n;
            ++n;
        }
    j = mine;
    k = n;
}

// The same for a whole CTA, plus list[0 .. k) in shared memory: the CTAs that hold the pieces.
__device__ __forceinline__ void unit_pieces(const uint32_t *B, bool dense, uint32_t i_lo, uint32_t i_hi, uint32_t tid, uint32_t n_threads,
                                            uint16_t *list, volatile uint32_t *jk, uint32_t &j, uint32_t &k) {
    if (dense) {
        k = i_hi - i_lo + 1;
        j = blockIdx.x - i_lo;
        for (uint32_t t = tid; t < k; t += n_threads) list[t] = (uint16_t)(i_lo + t);
        return;   // the caller's next barrier publishes the list
    }
    if (tid == 0) {
        uint32_t n = 0, mine = 0;
        for (uint32_t i = i_lo; i <= i_hi; ++i)
            if (B[i] != B[i + 1]) {
                if (i == blockIdx.x) mine = n;
                list[n++] = (uint16_t)i;
            }
        jk[0] = mine;
        jk[1] = n;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(n_threads) : "memory");
    j = jk[0];
    k = jk[1];
}

// One merged row segment (row `row` of the unit, columns d .. d + 3) goes out: normalised and gated, or in partial
// mode as the merged (acc, m, l), or with p.world > 1 into this rank's slot of every rank's receive buffer.
template <int HD, int KVB, bool CAN_PUSH>
__device__ __forceinline__ void merge_emit(const DecodeParams &p, const UnitRef ur, uint32_t s, uint32_t kv0, uint32_t row, uint32_t d,
                                           float2 ml, float4 acc, uint32_t bank) {
    const uint32_t k2 = row / p.group, h = row - k2 * p.group;
    const uint32_t head = (kv0 + k2) * p.group_all + p.head0 + h;
    const size_t o = ur.layer * p.out_layer_stride + ((size_t)s * p.n_head + head) * HD + d;
    if (CAN_PUSH && p.world > 1) {
        const size_t R = ((size_t)ur.layer * p.n_seqs + s) * p.n_head + head;
        const uint64_t oa = push_acc_off(p, bank, p.rank, R, HD, d), om = push_ml_off(p, bank, p.rank, R, HD);
        const float4 a4 = make_float4(keep_off_empty(acc.x), keep_off_empty(acc.y), keep_off_empty(acc.z), keep_off_empty(acc.w));
        const float2 ml2 = make_float2(keep_off_empty(ml.x), keep_off_empty(ml.y));
        for (uint32_t r = 0; r < p.world; ++r) {
            *reinterpret_cast<float4 *>(p.peer_recv[r] + oa) = a4;
            if (d == 0) *reinterpret_cast<float2 *>(p.peer_recv[r] + om) = ml2;
        }
    } else if (p.out_ml) {
        *reinterpret_cast<float4 *>(p.out + o) = acc;
        if (d == 0) {
            float *om = p.out_ml + ur.layer * p.out_ml_layer_stride + ((size_t)s * p.n_head + head) * 2;
            om[0] = ml.x;
            om[1] = ml.y;
        }
    } else {
        const float inv = ml.y > 0.f ? 1.f / ml.y : 0.f;
        float4 r = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        if (p.gate) {
            const float *gt = p.gate + ur.layer * p.gate_layer_stride + ((size_t)s * p.n_head + head) * p.gate_head_stride + d;
            r.x *= sigmoid_f32(gt[0]);
            r.y *= sigmoid_f32(gt[1]);
            r.z *= sigmoid_f32(gt[2]);
            r.w *= sigmoid_f32(gt[3]);
        }
        *reinterpret_cast<float4 *>(p.out + o) = r;
    }
}

// What one CTA does of a unit's merge once every piece is written: items it0 .. it0 + items_c - 1, k pieces.
// The code runs once per CTA, from a cold instruction cache (unrolled over registers it took 13 us where this
// takes 2): small rolled loops.  All of the CTA's accumulator segments - items_c x k, 32 KiB at most - are
// copied into `stage` (the ring's shared memory, idle once the CTA has streamed its share) with 16-byte
// asynchronous copies, [piece][item], together with the (m, l) sweep: one trip to L2 for everything.  Then the
// weights (one warp per row) and the sums: 2^lg threads per item (within a warp), each taking every 2^lg-th
// piece, a shuffle reduction, and the segment goes out.
template <int HD, int KVB, bool CAN_PUSH, int NT>
__device__ __forceinline__ void merge_items(const DecodeParams &p, const UnitRef ur, const uint16_t *list, float2 *mls, float2 *rowml,
                                            float4 *stage, uint32_t it0, uint32_t items_c, uint32_t k, uint32_t tid, uint32_t s,
                                            uint32_t kv0, uint32_t bank) {
    constexpr uint32_t TPR = HD / 4;
    constexpr int NW = NT / 32;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t r0 = it0 / TPR, nr = (it0 + items_c - 1) / TPR - r0 + 1;
    // ---- accumulator segments, stage[pc * items_c + il], and the (m, l) of this CTA's rows from every piece: every
    //      thread an equal number of copies, all in flight together
    for (uint32_t idx = tid; idx < k * items_c; idx += NT) {
        const uint32_t pc = idx / items_c, il = idx - pc * items_c;
        const uint32_t item = it0 + il, row = item / TPR, d = (item - row * TPR) * 4u;
        const uint32_t k2 = row / p.group, h = row - k2 * p.group;
        const float *src = p.part_acc + (((size_t)(ur.U + list[pc]) * KVB + k2) * GROUP_TILE + h) * HD + d;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(brc::smem_u32(stage + idx)), "l"(src) : "memory");
    }
    for (uint32_t idx = tid; idx < nr * k; idx += NT) {
        const uint32_t rl = idx / k, pc = idx - rl * k, row = r0 + rl;
        const uint32_t k2 = row / p.group, h = row - k2 * p.group;
        const float *src = p.part_ml + (((size_t)(ur.U + list[pc]) * KVB + k2) * GROUP_TILE + h) * 2;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(brc::smem_u32(mls + idx)), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    brc::named_bar_sync(1, NT);
    // ---- weights 2^(m - M): one warp per row
    for (uint32_t rl = warp; rl < nr; rl += NW) {
        float M = -INFINITY;
        for (uint32_t pc = lane; pc < k; pc += 32) {
            const float2 ml = mls[rl * k + pc];
            if (ml.y > 0.f) M = fmaxf(M, ml.x);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        float L = 0.f;
        for (uint32_t pc = lane; pc < k; pc += 32) {
            const float2 ml = mls[rl * k + pc];
            const float w = ml.y > 0.f ? exp2f(ml.x - M) : 0.f;
            mls[rl * k + pc].x = w;
            L += w * ml.y;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
        if (lane == 0) rowml[rl] = make_float2(M, L);
    }
    brc::named_bar_sync(1, NT);
    // ---- weighted sums and the segments (the same trip counts for every thread: the shuffles are warp-wide)
    uint32_t lg = 0;                                     // 2^lg threads per item: as many as leave every item a thread
    while (lg < 5u && (items_c << (lg + 1)) <= NT) ++lg;
    const uint32_t g = 1u << lg, per_round = NT >> lg, grp = tid & (g - 1u), slot = tid >> lg;
    for (uint32_t base = 0; base < items_c; base += per_round) {
        const uint32_t il = base + slot;
        const bool act = il < items_c;
        const uint32_t ilc = min(il, items_c - 1u);
        const uint32_t item = it0 + ilc, row = item / TPR, d = (item - row * TPR) * 4u;
        const float2 *wrow = mls + (row - r0) * k;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t pc = grp; pc < k; pc += g) {
            const float4 v = stage[pc * items_c + ilc];
            const float wt = wrow[pc].x;
            acc.x += wt * v.x;
            acc.y += wt * v.y;
            acc.z += wt * v.z;
            acc.w += wt * v.w;
        }
        for (uint32_t off = g >> 1; off > 0; off >>= 1) {
            acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
            acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
            acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
            acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
        }
        if (act && grp == 0u) merge_emit<HD, KVB, CAN_PUSH>(p, ur, s, kv0, row, d, rowml[row - r0], acc, bank);
    }
}

// Log-sum-exp merge of the pieces of unit `ur`, done by the CTAs that streamed one of them (all but the holder of
// the last piece), each with its NW * 32 consumer threads once its own streaming is over: the unit's (row,
// 16-byte column) items are dealt over those CTAs in equal runs, so whatever the number of pieces k, a CTA reads
// one or two pieces' worth of partials and the merge takes two trips to L2 instead of one per four pieces
// through a single SM.  (All pieces of a unit but its last complete at the end of their CTAs' streaming, i.e. at
// the same time, and those CTAs have nothing else left to do; a trip to L2 costs 1.5-3 us while other CTAs
// still stream, and the last arriver merging alone took 7-11 us with 5-10 pieces and 40 us with 148.)  The CTA
// first waits, with a time limit, until the unit's ticket shows every piece written (unless its own ticket
// was the last: `all_written`, thread 0's knowledge); the launch is
// cooperative, so all CTAs are resident and the pieces it waits for are being produced.  Then merge_items.
// With p.world > 1 the CTA that stores last releases one flag per rank.  Partials come from other SMs: they
// are read from L2 (.cg).  `sm` is the CTA's merge scratch and `stage` the ring, both free at this point.
template <int HD, int KVB, bool CAN_PUSH, bool VQ8>
__device__ __forceinline__ void merge_unit(const DecodeParams &p, const UnitRef ur, uint32_t i_lo, uint32_t i_hi, const uint32_t *B,
                                           bool dense, uint32_t tid, float *sm, float4 *stage, uint32_t epoch, uint32_t bank,
                                           volatile uint32_t *gave_up, bool all_written) {
    constexpr int NW = consumer_warps(VQ8, HD);
    constexpr uint32_t NT = NW * 32;
    constexpr uint32_t TPR = HD / 4;                    // 16-byte columns of a row
    const uint32_t n_rows = KVB * p.group;              // (kv head of the unit, query head)
    const uint32_t n_items = n_rows * TPR;
    const uint32_t n_groups = p.n_kv_head / KVB;
    const uint32_t s = ur.u / n_groups, kv0 = (ur.u % n_groups) * KVB;

    uint16_t *list = reinterpret_cast<uint16_t *>(sm);                           // [MAX_CTAS] CTAs that hold a piece
    volatile uint32_t *jk = reinterpret_cast<volatile uint32_t *>(list + MAX_CTAS);   // [4]
    float2 *rowml = reinterpret_cast<float2 *>(const_cast<uint32_t *>(jk) + 4);   // [<= n_rows] merged (m, l) of this CTA's rows
    float2 *mls = rowml + KVB * GROUP_TILE;                                      // [rows of this CTA][k]: (m, l), then (weight, l)

    brc::named_bar_sync(1, NT);                          // the scratch is free (previous unit's merge, or the epilogue)
    uint32_t j, k;
    unit_pieces(B, dense, i_lo, i_hi, tid, NT, list, jk, j, k);
    uint32_t *const ticket = p.done + ur.layer * BRC_DONE_BANK_WORDS + ur.u;
    // The CTA that holds a unit's LAST piece streamed it first thing and has another unit's merge to attend to at
    // its own end: the unit's other CTAs (all of them at the end of their streaming) share the merge among them.
    const bool pushing = CAN_PUSH && p.world > 1;
    uint32_t n_part = k > 1u ? k - 1u : 1u;              // CTAs that take part
    if (j >= n_part) return;                             // CTA-uniform
    // ---- every piece written?  (this CTA's own weight is in: zero low bits mean all of them)
    if (tid == 0 && !gave_up[0]) {
        bool ok = all_written;                           // thread 0 took the unit's last ticket itself: nothing to wait for
        if (ok) __threadfence();                         // the add that told it so was relaxed: order the reads below after it
        if (!ok) ok = (ld_acquire_gpu(ticket) & TICKET_LOW) == 0u;
        if (!ok) {
            const uint64_t t0 = globaltimer_ns();
            for (uint32_t i = 0; i < (1u << 30); ++i) {
                if ((ld_acquire_gpu(ticket) & TICKET_LOW) == 0u) { ok = true; break; }
                if ((i & 63u) == 63u && globaltimer_ns() - t0 > WAIT_NS) break;
            }
        }
        if (!ok) {
            gave_up[0] = 1u;
            atomicOr(p.status, BRC_DEV_WAIT_LIMIT);
            p.status[1] = 4000000u + blockIdx.x;   // a piece of the unit was never written
            p.status[2] = ur.U;
        }
    }
    brc::named_bar_sync(1, NT);
    if (gave_up[0]) return;                              // nobody clears the flag: every later wait of this CTA is skipped too

    const uint32_t it0 = (uint32_t)((uint64_t)j * n_items / n_part), it1 = (uint32_t)((uint64_t)(j + 1) * n_items / n_part);
    const uint32_t items_c = it1 - it0;
    if (items_c != 0) {
        merge_items<HD, KVB, CAN_PUSH, NT>(p, ur, list, mls, rowml, stage, it0, items_c, k, tid, s, kv0, bank);
    }
}

// Cross-rank merge of rows row_first, row_first + row_step, ... of unit `ur` (split-KV across GPUs).  The rows of a
// unit are dealt over the CTAs that streamed a share of it, each running this with its NW * 32 consumer threads
// after it has finished streaming.  A thread owns one 16-byte segment of a row: it polls, with a time limit,
// that segment and the row's (m, l) in every rank's slot of this rank's receive buffer until none of them holds
// PUSH_EMPTY any more (all loads of a sweep are issued together), merges, normalises, applies the gate, writes
// its segment of the output and puts PUSH_EMPTY back.  On expiry the segment is left as it was, the check word
// reports it, and the CTA's later waits give up at once.
template <int HD, int KVB, bool VQ8>
__device__ __forceinline__ void finalize_unit(const DecodeParams &p, const UnitRef ur, uint32_t row_first, uint32_t row_step,
                                              uint32_t bank, uint32_t tid, volatile uint32_t *gave_up) {
    constexpr int NW = consumer_warps(VQ8, HD);
    constexpr uint32_t TPR = HD / 4;
    constexpr uint32_t ROWS_PER_PASS = (NW * 32) / TPR;
    const uint32_t n_rows = KVB * p.group;
    if (row_first >= n_rows) return;   // CTA-uniform: more CTAs than rows
    const uint32_t n_groups = p.n_kv_head / KVB;
    const uint32_t s = ur.u / n_groups, kv0 = (ur.u % n_groups) * KVB;
    const uint32_t d = (tid % TPR) * 4;
    uint8_t *own = p.peer_recv[p.rank];
    const float4 empty4 = make_float4(__uint_as_float(PUSH_EMPTY), __uint_as_float(PUSH_EMPTY), __uint_as_float(PUSH_EMPTY),
                                      __uint_as_float(PUSH_EMPTY));
    for (uint32_t row = row_first + (tid / TPR) * row_step; row < n_rows; row += ROWS_PER_PASS * row_step) {
        const uint32_t k2 = row / p.group, h = row % p.group;
        const uint32_t head = (kv0 + k2) * p.group_all + p.head0 + h;
        const size_t R = ((size_t)ur.layer * p.n_seqs + s) * p.n_head + head;
        float2 ml[BRC_MAX_WORLD];
        float4 a[BRC_MAX_WORLD];
        bool ok = false;
        const uint64_t t0 = globaltimer_ns();
        for (uint32_t i = 0; i < (1u << 30) && !gave_up[0]; ++i) {
            bool all = true;
#pragma unroll
            for (uint32_t r = 0; r < BRC_MAX_WORLD; ++r) {
                if (r < p.world) {
                    ml[r] = ld_volatile_f2(own + push_ml_off(p, bank, r, R, HD));
                    a[r] = ld_volatile_f4(own + push_acc_off(p, bank, r, R, HD, d));
                }
            }
#pragma unroll
            for (uint32_t r = 0; r < BRC_MAX_WORLD; ++r)
                if (r < p.world) all = all && landed(ml[r]) && landed(a[r]);
            if (all) {
                ok = true;
                break;
            }
            if ((i & 15u) == 15u && globaltimer_ns() - t0 > p.wait_ns) break;
        }
        if (!ok) {
            if (!gave_up[0]) {
                gave_up[0] = 1u;   // benign race: every writer stores 1
                atomicOr(p.status, BRC_DEV_WAIT_LIMIT);
                p.status[1] = 3000000u + p.rank;   // a rank's partial never arrived here
                p.status[2] = ur.U;
            }
            continue;
        }
        float M = -INFINITY;
#pragma unroll
        for (uint32_t r = 0; r < BRC_MAX_WORLD; ++r)
            if (r < p.world && ml[r].y > 0.f) M = fmaxf(M, ml[r].x);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll
        for (uint32_t r = 0; r < BRC_MAX_WORLD; ++r) {
            if (r < p.world && ml[r].y > 0.f) {
                const float w = exp2f(ml[r].x - M);
                L += w * ml[r].y;
                acc.x += w * a[r].x;
                acc.y += w * a[r].y;
                acc.z += w * a[r].z;
                acc.w += w * a[r].w;
            }
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        float4 o = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        if (p.gate) {
            const float *g = p.gate + ur.layer * p.gate_layer_stride + ((size_t)s * p.n_head + head) * p.gate_head_stride + d;
            o.x *= sigmoid_f32(g[0]);
            o.y *= sigmoid_f32(g[1]);
            o.z *= sigmoid_f32(g[2]);
            o.w *= sigmoid_f32(g[3]);
        }
        *reinterpret_cast<float4 *>(p.out + ur.layer * p.out_layer_stride + ((size_t)s * p.n_head + head) * HD + d) = o;
        for (uint32_t r = 0; r < p.world; ++r) *reinterpret_cast<float4 *>(own + push_acc_off(p, bank, r, R, HD, d)) = empty4;
    }
    // ---- the (m, l) of a row is read by every thread of the row: it is emptied when all of them are through
    brc::named_bar_sync(1, NW * 32);
    if (d == 0 && !gave_up[0]) {
        for (uint32_t row = row_first + (tid / TPR) * row_step; row < n_rows; row += ROWS_PER_PASS * row_step) {
            const uint32_t k2 = row / p.group, h = row % p.group;
            const uint32_t head = (kv0 + k2) * p.group_all + p.head0 + h;
            const size_t R = ((size_t)ur.layer * p.n_seqs + s) * p.n_head + head;
            for (uint32_t r = 0; r < p.world; ++r)
                *reinterpret_cast<float2 *>(own + push_ml_off(p, bank, r, R, HD)) = make_float2(empty4.x, empty4.y);
        }
    }
}

// WHOLE_FAST: compile the direct-output path for units that lie wholly inside one CTA's share.  It pays when
// there are at least as many units as CTAs (many short sequences); with few long sequences no unit can
// be of that kind, and leaving the path out keeps the streaming loop's code as lean as it was.
//
// VQ8: the pool stores V as q8_0 blocks (one f32 scale + 32 signed bytes per 32 values, 0.5625x the bytes;
// crates/breccia-kernels/src/qsa/mod.rs:325-349, read rule shaders/qsa_attn_apply.comp:60-77).  tm_kv is then
// the 2-D view of K alone and tm_v8 the view of the V rows in 32-bit words; a stage holds the K slabs and the
// page's V rows as they lie in the pool.  The quanta enter the tensor cores as EXACT binary16 integers
// (built in registers: no dequantised tile is ever written), and the per-(cell, block) scale is folded
// into the probabilities of that block, split into a binary16 head and tail as before - so the result
// carries the same ~22 significant bits as the binary16 path.
template <int HD, bool Q_F32, int KVB, bool WHOLE_FAST, bool VQ8>
__global__ void __launch_bounds__((consumer_warps(VQ8, HD) + 1) * 32, 1)
    decode_partial_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_v8, const DecodeParams p) {
    using C = Cfg<HD, KVB, VQ8>;
    constexpr int NW = C::NW;
    constexpr int NTHREADS = C::NTHREADS;
    extern __shared__ uint8_t smem_raw[];
    // The 128-byte swizzle pattern repeats every 1024 bytes: tiles must start on that boundary.
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    uint8_t *ring = smem;
    float *scratch = reinterpret_cast<float *>(ring + (size_t)p.n_stages * C::STAGE_BYTES);
    uint32_t *S = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(scratch) + C::SCRATCH_BYTES);
    uint16_t *nz = reinterpret_cast<uint16_t *>(reinterpret_cast<uint8_t *>(S) + C::PREFIX_BYTES);   // [n_units + 1] units with pages before u
    uint32_t *B = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(nz) + C::NZ_BYTES);          // [CTAs + 1] where every share begins
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(B) + C::CUT_BYTES);
    const uint32_t full0 = brc::smem_u32(bars);
    const uint32_t empty0 = full0 + 8u * p.n_stages;
    // small words after the barriers (2 x 24 barriers at most = 384 bytes): flags, merge weights
    volatile uint32_t *flags = reinterpret_cast<volatile uint32_t *>(bars + 64);
    volatile uint32_t *dead_cta = flags + 1;
    volatile uint32_t *gave_up = flags + 2;
    float *wts = reinterpret_cast<float *>(const_cast<uint32_t *>(flags) + 8);  // [NWP][KVB * GROUP_TILE]
    float *inv_l = wts + NW * GROUP_TILE;                                       // [KVB * GROUP_TILE] 1 / l of the merged rows

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n_groups = p.n_kv_head / KVB;   // kv-head groups per sequence
    const uint32_t n_units = p.n_seqs * n_groups;  // units of one layer
    const bool push = !WHOLE_FAST && p.world > 1;   // the host launches the cross-GPU form without the direct-output path
    // Split-KV across GPUs: this launch's epoch is the number of exchanges completed so far plus one
    // (read by every CTA before any of them can take the launch's last ticket, which advances it).
    const uint32_t epoch = push ? *reinterpret_cast<volatile uint32_t *>(p.calls) + 1u : 0u;
    const uint32_t bank = epoch % BRC_COMM_BANKS;

    if (tid == 0) {
        for (uint32_t i = 0; i < p.n_stages; ++i) {
            brc::mbar_init(full0 + 8u * i, 1);
            brc::mbar_init(empty0 + 8u * i, KVB);   // every kv head's warp hands the stage back
        }
        brc::mbar_fence_init();
        brc::tma_prefetch_desc(&tm_kv);
        if (VQ8 || p.one_op) brc::tma_prefetch_desc(&tm_v8);
        dead_cta[0] = 0u;
        gave_up[0] = 0u;
    }
    // Exclusive prefix of pages per unit of ONE layer, S[0..n_units] (the layers of a launch share the
    // sequence lengths), and nz[0..n_units], how many of the units before u have pages; every CTA computes
    // both (n_units <= 2048).
    if (warp == 0) {
        uint32_t run = 0, nz_run = 0;
        for (uint32_t base = 0; base < n_units; base += 32) {
            const uint32_t u = base + lane;
            uint32_t pg = 0;
            if (u < n_units) {
                uint32_t len = p.seq_lens[u / n_groups];
                if (len > p.max_seq_len) {
                    atomicOr(p.status, BRC_DEV_BAD_POS);
                    p.status[1] = len;
                    len = p.max_seq_len;
                }
                pg = pages_of(len);
            }
            uint32_t inc = pg;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, inc, o);
                if ((int)lane >= o) inc += v;
            }
            const uint32_t live = __ballot_sync(0xffffffffu, pg != 0);
            if (u < n_units) {
                S[u] = run + inc - pg;
                nz[u] = (uint16_t)(nz_run + __popc(live & ((1u << lane) - 1u)));
            }
            run += __shfl_sync(0xffffffffu, inc, 31);
            nz_run += __popc(live);
        }
        if (lane == 0) {
            S[n_units] = run;
            nz[n_units] = (uint16_t)nz_run;
        }
    }
    __syncthreads();

    const uint32_t total_l = S[n_units];            // page-units of one layer
    const uint32_t total = total_l * p.n_layers;    // of the launch (the host keeps this below 2^32)
    const uint32_t n_units_all = n_units * p.n_layers;

    // ---- the cut: where every CTA's share begins.  The flat list is cut into equal shares not of page-units
    // but of COST: every unit with pages costs p.unit_cost page-units on top of its pages, charged where the
    // unit begins (a CTA pays one epilogue per unit it touches: one in any case, one more for every unit that
    // begins inside its share).  Cost position of page g of unit u in layer l:
    //   l * cost_l + S[u] + unit_cost * (nz[u] + 1) + (g - S[u]),   cost_l = total_l + unit_cost * nz[n_units].
    // A threshold that falls into a unit's surcharge cuts at the unit's first page.  Every CTA builds the same
    // table; B is ascending, B[0] = 0, B[gridDim.x] = total.
    {
        const uint32_t E = p.unit_cost;
        const uint64_t cost_l = (uint64_t)total_l + (uint64_t)E * nz[n_units];
        const uint64_t cost = cost_l * p.n_layers;
        for (uint32_t i = tid; i <= gridDim.x; i += NTHREADS) {
            uint32_t at = total;
            if (i < gridDim.x && total != 0) {
                // equal shares of the cost, or shares in proportion to the measured streaming rate of the CTAs' SMs
                const uint64_t f = p.cut_prefix ? p.cut_prefix[i] : 0;
                const uint64_t t = p.cut_prefix ? (cost >> 32) * f + (((cost & 0xffffffffull) * f) >> 32) : cost * i / gridDim.x;
                const uint32_t l = (uint32_t)(t / cost_l);
                const uint32_t tl = (uint32_t)(t - (uint64_t)l * cost_l);
                uint32_t lo = 0, hi = n_units;          // largest u with S[u] + E * nz[u] <= tl: a unit with pages
                while (hi - lo > 1) {
                    const uint32_t mid = (lo + hi) >> 1;
                    if (S[mid] + E * nz[mid] <= tl) lo = mid; else hi = mid;
                }
                const uint32_t off = tl - (S[lo] + E * nz[lo]);
                at = l * total_l + S[lo] + (off > E ? off - E : 0u);
            }
            B[i] = at;
        }
        __syncthreads();
        int live = 1;
        for (uint32_t i = tid; i < gridDim.x; i += NTHREADS) live &= B[i] != B[i + 1];
        live = __syncthreads_and(live);
        if (tid == 0) B[MAX_CTAS + 2] = live != 0;      // read back where needed instead of held in a register
        __syncthreads();
    }
#define all_shares_live (B[MAX_CTAS + 2] != 0u)         /* no CTA has an empty share */

    // A sequence without cells has no pages, hence no share and no ticket: its rows are written here.
    for (uint32_t U = blockIdx.x; U < n_units_all; U += gridDim.x) {
        const uint32_t layer = U / n_units, u = U - layer * n_units;
        if (S[u + 1] != S[u]) continue;
        const uint32_t s = u / n_groups, kv0 = (u % n_groups) * KVB;
        for (uint32_t i = tid; i < KVB * p.group * HD; i += NTHREADS) {
            const uint32_t head = (kv0 + (i / HD) / p.group) * p.group_all + p.head0 + (i / HD) % p.group;
            if (push) {
                const size_t R = ((size_t)layer * p.n_seqs + s) * p.n_head + head;
                const uint64_t oa = push_acc_off(p, bank, p.rank, R, HD, i % HD), om = push_ml_off(p, bank, p.rank, R, HD);
                for (uint32_t r = 0; r < p.world; ++r) {
                    *reinterpret_cast<float *>(p.peer_recv[r] + oa) = 0.f;
                    if (i % HD == 0) *reinterpret_cast<float2 *>(p.peer_recv[r] + om) = make_float2(-INFINITY, 0.f);
                }
                continue;
            }
            p.out[layer * p.out_layer_stride + ((size_t)s * p.n_head + head) * HD + i % HD] = 0.f;
            if (p.out_ml && i % HD == 0) {
                float *om = p.out_ml + layer * p.out_ml_layer_stride + ((size_t)s * p.n_head + head) * 2;
                om[0] = -INFINITY;
                om[1] = 0.f;
            }
        }
    }

    const uint32_t a = B[blockIdx.x];
    const uint32_t b = B[blockIdx.x + 1];
    const uint32_t count = b - a;

    if (warp == NW) {
        // ------------------------------------------------------------------ producer warp
        const uint64_t policy = brc::l2_policy_evict_first();
        uint32_t dead = 0;
        uint32_t issued = 0;
        for (uint32_t k0 = 0; k0 < count && !dead; k0 += 32) {
            const uint32_t k = k0 + lane;
            uint32_t row = 0;
            uint32_t app = 0;  // fused append: bit 31 = this page holds the sequence's newest cell, then cell (4 bits), layer (6), unit (11)
            uint32_t q_of = 0xffffffffu;   // (layer << 16 | unit) when this page opens a unit the consumers have not reached yet
            if (k < count) {
                const uint32_t g = a + k;
                const uint32_t layer = g / total_l, gl = g - layer * total_l;
                const uint32_t u = unit_of(S, n_units, gl);
                const uint32_t s = u / n_groups, kv0 = (u % n_groups) * KVB;
                if (k > 0 && gl == S[u]) q_of = (layer << 16) | u;
                uint32_t page = __ldg(p.block_tables + (uint64_t)s * p.table_stride + (gl - S[u]));
                if (page >= p.n_pages) {
                    atomicOr(p.status, BRC_DEV_BAD_PAGE);
                    p.status[1] = page;
                    page = 0;  // stay inside the pool; the result of this unit is void and the call reports it
                } else if (p.k_new) {
                    // a sequence beyond the caller's bound is reported and attended up to the bound; nothing
                    // is appended for it (the append kernel skips such tokens too)
                    const uint32_t len = p.seq_lens[s];
                    if (len <= p.max_seq_len && gl - S[u] == (len - 1u) >> 4)
                        app = 0x80000000u | (((len - 1u) & 15u) << 24) | (layer << 16) | u;
                }
                row = p.layer_row0 + layer * p.layer_rows + (page * p.n_kv_head + kv0) * 16u;
            }
            // The consumers load a unit's query rows when they reach its first page, a ring's depth from now:
            // bring the rows into L2 meanwhile (they may lie in host memory, a PCIe round trip away).
            for (uint32_t opens = __ballot_sync(0xffffffffu, q_of != 0xffffffffu); opens; opens &= opens - 1u) {
                const uint32_t qo = __shfl_sync(0xffffffffu, q_of, __ffs(opens) - 1);
                const uint32_t ql = qo >> 16, qu = qo & 0xffffu;
                const uint32_t q_elem = Q_F32 ? 4u : 2u, head_bytes = p.group * HD * q_elem;
#pragma unroll
                for (int k2 = 0; k2 < KVB; ++k2) {
                    const uint64_t first = ql * p.q_layer_stride + ((uint64_t)(qu / n_groups) * p.n_head + ((qu % n_groups) * KVB + k2) * p.group_all + p.head0) * HD;
                    const uint8_t *rows = static_cast<const uint8_t *>(p.q) + first * q_elem;
                    for (uint32_t off = lane * 128u; off < head_bytes; off += 32u * 128u)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(rows + off));
                }
            }
            const uint32_t n_here = min(32u, count - k0);
            for (uint32_t i = 0; i < n_here; ++i) {
                const uint32_t r = __shfl_sync(0xffffffffu, row, i);
                const uint32_t kk = k0 + i;
                const uint32_t stage = kk % p.n_stages;
                const uint32_t fb = full0 + 8u * stage;
                if (lane == 0) {
                    if (!wait_bounded(empty0 + 8u * stage, ((kk / p.n_stages) & 1u) ^ 1u))
                        dead = 1;
                    else
                        brc::mbar_arrive_expect_tx(fb, C::TX_BYTES);
                }
                dead = __shfl_sync(0xffffffffu, dead, 0);
                if (dead) break;
                if (p.k_new) {
                    // Fused KV append (the reference's qsa_kv_append.comp rule, one cell): the page about to
                    // be streamed holds the sequence's newest cell, whose K/V this step brings.  Exactly one
                    // CTA streams that page, so it writes the cell first; the proxy fence orders these
                    // generic-proxy stores before the TMA (async-proxy) read of the same rows.
                    const uint32_t ap = __shfl_sync(0xffffffffu, app, i);
                    if (ap & 0x80000000u) {
                        const uint32_t au = ap & 0xffffu, cell = (ap >> 24) & 15u, al = (ap >> 16) & 63u;
                        const uint32_t as = au / n_groups, akv0 = (au % n_groups) * KVB;
                        if (lane < HD / 8) {
#pragma unroll
                            for (int k2 = 0; k2 < KVB; ++k2) {
                                const uint64_t src = al * p.kv_new_layer_stride + ((uint64_t)as * p.n_kv_head + akv0 + k2) * HD + lane * 8u;
                                const uint64_t dst = ((uint64_t)(r + k2 * 16u + cell) * HD + lane * 8u) * 2u;
                                uint4 ko, vo;
                                if (p.kv_new_f32) {
                                    const float4 *ks = reinterpret_cast<const float4 *>(static_cast<const float *>(p.k_new) + src);
                                    const float4 *vs = reinterpret_cast<const float4 *>(static_cast<const float *>(p.v_new) + src);
                                    const float4 x0 = __ldg(ks), x1 = __ldg(ks + 1), y0 = __ldg(vs), y1 = __ldg(vs + 1);
                                    ko = make_uint4(brc::pack_f16x2(x0.x, x0.y), brc::pack_f16x2(x0.z, x0.w),
                                                    brc::pack_f16x2(x1.x, x1.y), brc::pack_f16x2(x1.z, x1.w));
                                    vo = make_uint4(brc::pack_f16x2(y0.x, y0.y), brc::pack_f16x2(y0.z, y0.w),
                                                    brc::pack_f16x2(y1.x, y1.y), brc::pack_f16x2(y1.z, y1.w));
                                } else {
                                    ko = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.k_new) + src));
                                    vo = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.v_new) + src));
                                    ko = make_uint4(brc::flush_f16x2(ko.x), brc::flush_f16x2(ko.y), brc::flush_f16x2(ko.z), brc::flush_f16x2(ko.w));
                                    vo = make_uint4(brc::flush_f16x2(vo.x), brc::flush_f16x2(vo.y), brc::flush_f16x2(vo.z), brc::flush_f16x2(vo.w));
                                }
                                *reinterpret_cast<uint4 *>(p.k_base + dst) = ko;
                                if (!VQ8) {
                                    *reinterpret_cast<uint4 *>(p.k_base + p.v_offset + dst) = vo;
                                } else {
                                    // q8_0 store rule (shaders/qsa_kv_append.comp:117-133), from the f32 value: the four
                                    // lanes of a 32-value block share its maximum; scale = amax / 127 (1 for an all-zero
                                    // block), q = round-half-away(clamp(x / scale, +-127)); IEEE division and roundf, so the
                                    // bytes equal the append kernel's
                                    const float4 *vs = reinterpret_cast<const float4 *>(static_cast<const float *>(p.v_new) + src);
                                    const float4 y0 = __ldg(vs), y1 = __ldg(vs + 1);
                                    float amax = fmaxf(fmaxf(fmaxf(fabsf(y0.x), fabsf(y0.y)), fmaxf(fabsf(y0.z), fabsf(y0.w))),
                                                       fmaxf(fmaxf(fabsf(y1.x), fabsf(y1.y)), fmaxf(fabsf(y1.z), fabsf(y1.w))));
                                    constexpr uint32_t row_lanes = HD / 8 >= 32 ? 0xffffffffu : ((1u << (HD / 8 % 32)) - 1u);
                                    amax = fmaxf(amax, __shfl_xor_sync(row_lanes, amax, 1));
                                    amax = fmaxf(amax, __shfl_xor_sync(row_lanes, amax, 2));
                                    const float scale = amax > 0.f ? __fdiv_rn(amax, 127.f) : 1.f;
                                    auto quant = [scale](float x) {
                                        return (uint32_t)(int32_t)roundf(fminf(fmaxf(__fdiv_rn(x, scale), -127.f), 127.f)) & 0xffu;
                                    };
                                    const uint32_t w0 = quant(y0.x) | (quant(y0.y) << 8) | (quant(y0.z) << 16) | (quant(y0.w) << 24);
                                    const uint32_t w1 = quant(y1.x) | (quant(y1.y) << 8) | (quant(y1.z) << 16) | (quant(y1.w) << 24);
                                    uint32_t *blk = reinterpret_cast<uint32_t *>(p.k_base + p.v_offset) +
                                                    ((uint64_t)(r + k2 * 16u + cell) * (HD / 32) + (lane >> 2)) * 9u;
                                    if ((lane & 3u) == 0u) blk[0] = __float_as_uint(scale);
                                    blk[1u + 2u * (lane & 3u)] = w0;
                                    blk[2u + 2u * (lane & 3u)] = w1;
                                }
                            }
                            brc::fence_proxy_async_global();
                        }
                        __syncwarp();
                    }
                }
                // One operation per 64-column group (issued by neighbouring lanes of one instruction).
                // Shared memory: [group][K|V][row = kv head * 16 + cell][64 columns], 128-byte swizzled; with q8_0 V the
                // K slabs of all groups, then one more operation for the page's V rows (whole rows, unswizzled).
                if (!VQ8) {
                    if (p.one_op) {
                        if (lane == 0)
                            brc::tma_load_4d(brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES), &tm_v8, 0, (int32_t)r, 0, 0, fb, policy);
                    } else if (lane < C::BOXES)
                        brc::tma_load_3d(brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES) + lane * C::GROUP_BYTES, &tm_kv,
                                         (int32_t)(lane * 64u), (int32_t)r, 0, fb, policy);
                } else if (p.one_op) {   // the K slabs of all column groups in one box (3-D view of K), then the V rows
                    if (lane == 0)
                        brc::tma_load_3d(brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES), &tm_kv, 0, (int32_t)r, 0, fb, policy);
                    else if (lane == 1)
                        brc::tma_load_2d(brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES) + C::V_OFF, &tm_v8, 0, (int32_t)r, fb, policy);
                } else {
                    if (lane < C::BOXES)
                        brc::tma_load_2d(brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES) + lane * C::GROUP_BYTES, &tm_kv,
                                         (int32_t)(lane * 64u), (int32_t)r, fb, policy);
                    else if (lane == C::BOXES)
                        brc::tma_load_2d(brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES) + C::V_OFF, &tm_v8, 0, (int32_t)r, fb, policy);
                }
                issued = kk + 1;
            }
        }
        if (dead && lane == 0) {
            atomicOr(p.status, BRC_DEV_WAIT_LIMIT);
            p.status[1] = 1000000u + blockIdx.x;
        }
        // Nothing may still be landing in this CTA's shared memory when it is released: wait (bounded)
        // for the copies of the last ring's worth of pages, whatever the consumers did with them.
        // Only those: an earlier page's barrier has since moved on to a later page's phase.
        if (lane == 0) {
            const uint32_t first = count > p.n_stages ? count - p.n_stages : 0;
            for (uint32_t kk = first; kk < issued; ++kk)
                wait_bounded(full0 + 8u * (kk % p.n_stages), (kk / p.n_stages) & 1u);
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    const uint32_t kl = warp % KVB;           // kv head of the group this warp serves
    const uint32_t cw = warp / KVB;           // its place among the NWP warps that interleave pages
    const uint32_t t0 = lane >> 2;            // cell row of c0/c1 (c2/c3: +8); also the head of the B operand
    const uint32_t h0 = (lane & 3u) * 2u;     // head column of c0/c2 (c1/c3: +1)
    // ldmatrix lane constants.  A slab row is 128 bytes; 16-byte chunk j of row r sits at chunk
    // j ^ (r & 7) (the TMA 128-byte swizzle); this kv head's rows start at kl * 16, a multiple of 8.
    const uint32_t k_r = (lane & 7u) + ((lane >> 3) & 1u) * 8u;
    const uint32_t k_x = (lane >> 4) ^ (k_r & 7u);
    const uint32_t k_lane = (kl * 16u + k_r) * 128u;
    const uint32_t v_r = (lane & 7u) + (lane >> 4) * 8u;
    const uint32_t v_x = ((lane >> 3) & 1u) ^ (v_r & 7u);
    const uint32_t v_lane = C::SLAB_BYTES + (kl * 16u + v_r) * 128u;
    // q8_0 V: this lane's four cells in the B-operand layout (k = 2t, 2t + 1, 2t + 8, 2t + 9 with t = lane & 3) and its
    // word of every 32-value block (bytes 4g .. 4g + 3 with g = lane >> 2); byte offsets from the stage's V rows
    const uint32_t q8_c0 = C::V_OFF + (kl * 16u + (lane & 3u) * 2u) * C::VROW_BYTES;

    uint32_t kw = cw;                          // next local page-unit of this warp
    uint32_t stage = cw % p.n_stages, parity = 0;
    uint32_t dead = 0;

    // the first unit of the share: (layer, u) with flat index U = layer * n_units + u
    uint32_t layer = 0, u = 0;
    if (a < b) {
        layer = a / total_l;
        u = unit_of(S, n_units, a - layer * total_l);
    }
    const uint32_t first_layer = layer, first_u = u;
    uint32_t tk_unit = 0xffffffffu, tk_sum = 1u;   // thread 0: the unit it last took a ticket of, and the ticket's value then
    uint32_t g0 = a;
    while (g0 < b) {
        const uint32_t lbase = layer * total_l;     // first page-unit of this layer in the flat list
        const uint32_t ge = min(b, lbase + S[u + 1]);
        const uint32_t s = u / n_groups, kvh = (u % n_groups) * KVB + kl;
        const uint32_t len = min(p.seq_lens[s], p.max_seq_len);
        const uint32_t unit_first = lbase + S[u];
        const UnitRef ur = {layer * n_units + u, layer, u};

        // Q^T fragments (B operand, k = d, n = head): b0 = Q[head t0][16 ks + 2 (lane & 3) + {0,1}],
        // b1 = same + 8.  Heads past the group read as zero.
        uint32_t qh[C::KSTEPS][2];
        uint32_t ql[Q_F32 ? C::KSTEPS : 1][2];
        {
            const bool live = t0 < p.group;
            const uint64_t qoff = layer * p.q_layer_stride + ((uint64_t)s * p.n_head + kvh * p.group_all + p.head0 + t0) * HD + (lane & 3u) * 2u;
#pragma unroll
            for (int ks = 0; ks < C::KSTEPS; ++ks) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (Q_F32) {
                        float2 x = make_float2(0.f, 0.f);
                        if (live) x = __ldg(reinterpret_cast<const float2 *>(static_cast<const float *>(p.q) + qoff + ks * 16 + half * 8));
                        const __half2 hi = __floats2half2_rn(x.x, x.y);
                        const float2 hf = __half22float2(hi);
                        qh[ks][half] = *reinterpret_cast<const uint32_t *>(&hi);
                        ql[Q_F32 ? ks : 0][half] = brc::pack_half2(x.x - hf.x, x.y - hf.y);
                    } else {
                        qh[ks][half] = live ? __ldg(reinterpret_cast<const uint32_t *>(static_cast<const uint16_t *>(p.q) + qoff + ks * 16 + half * 8)) : 0u;
                    }
                }
            }
        }

        float o[C::MT][4];
#pragma unroll
        for (int mt = 0; mt < C::MT; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

        const uint32_t local_end = ge - a;
        for (; kw < local_end; kw += C::NWP) {
            if (!dead) {
                if (!wait_bounded(full0 + 8u * stage, parity)) {
                    dead = 1;
                    if (lane == 0) {
                        atomicOr(p.status, BRC_DEV_WAIT_LIMIT);
                        p.status[1] = 2000000u + blockIdx.x;
                        p.status[2] = kw;      // local page-unit the wait was for
                        p.status[3] = count;   // page-units of this CTA's share
                    }
                }
            }
            if (!dead) {
                const uint32_t page_in_unit = a + kw - unit_first;
                const uint32_t nv = min(16u, len - page_in_unit * 16u);  // live cells in this page (>= 1)
                const uint32_t sbase = brc::smem_u32(ring + (size_t)stage * C::STAGE_BYTES);

                if (nv < 16u) {
                    // Cells past the sequence end may hold anything (NaN included); their scores are
                    // masked below, and their V rows are cleared so 0 * NaN never reaches the sum.
                    if (!VQ8) {
                        for (uint32_t i = lane; i < (16u - nv) * 8u * C::BOXES; i += 32) {
                            const uint32_t row = kl * 16u + nv + i / (8u * C::BOXES);
                            const uint32_t within = i % (8u * C::BOXES);
                            const uint32_t addr = sbase + (within >> 3) * C::GROUP_BYTES + C::SLAB_BYTES + row * 128u + (within & 7u) * 16u;
                            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
                        }
                    } else {   // scales and quanta alike: a zero scale times a zero probability is zero
                        for (uint32_t i = lane; i < (16u - nv) * (C::VROW_BYTES / 16u); i += 32) {
                            const uint32_t addr = sbase + C::V_OFF + (kl * 16u + nv) * C::VROW_BYTES + i * 16u;
                            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
                        }
                    }
                    __syncwarp();
                }

                // ---- S^T = K . Q^T   (two accumulators to halve the dependent mma chain)
                float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < C::KSTEPS; ++ks) {
                    uint32_t af[4];
                    brc::ldmatrix_x4(af, sbase + (ks >> 2) * C::GROUP_BYTES + k_lane + ((k_x ^ ((ks & 3) * 2u)) << 4));
                    if (ks & 1) {
                        brc::mma_16816(sb, af, qh[ks][0], qh[ks][1]);
                        if (Q_F32) brc::mma_16816(sb, af, ql[Q_F32 ? ks : 0][0], ql[Q_F32 ? ks : 0][1]);
                    } else {
                        brc::mma_16816(sa, af, qh[ks][0], qh[ks][1]);
                        if (Q_F32) brc::mma_16816(sa, af, ql[Q_F32 ? ks : 0][0], ql[Q_F32 ? ks : 0][1]);
                    }
                }
                float sc[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) sc[i] = (sa[i] + sb[i]) * p.scale_log2;
                if (nv < 16u) {
                    if (t0 >= nv) sc[0] = sc[1] = -INFINITY;
                    if (t0 + 8u >= nv) sc[2] = sc[3] = -INFINITY;
                }
                // ---- online softmax over the 16 cells (rows: lanes with equal lane & 3 share heads)
                float x0 = fmaxf(sc[0], sc[2]), x1 = fmaxf(sc[1], sc[3]);
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) {
                    x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, off));
                    x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, off));
                }
                const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);
                const float al0 = brc::fast_exp2(m0 - n0), al1 = brc::fast_exp2(m1 - n1);
                m0 = n0;
                m1 = n1;
                const float p0 = brc::fast_exp2(sc[0] - n0), p1 = brc::fast_exp2(sc[1] - n1);
                const float p2 = brc::fast_exp2(sc[2] - n0), p3 = brc::fast_exp2(sc[3] - n1);
                l0 = l0 * al0 + (p0 + p2);
                l1 = l1 * al1 + (p1 + p3);
                if (__any_sync(0xffffffffu, (al0 != 1.f) | (al1 != 1.f))) {
#pragma unroll
                    for (int mt = 0; mt < C::MT; ++mt) {
                        o[mt][0] *= al0;
                        o[mt][1] *= al1;
                        o[mt][2] *= al0;
                        o[mt][3] *= al1;
                    }
                }
                // ---- P^T as the B operand: binary16 head + tail, transposed in registers
                const __half2 ph01 = __floats2half2_rn(p0, p1), ph23 = __floats2half2_rn(p2, p3);
                const float2 f01 = __half22float2(ph01), f23 = __half22float2(ph23);
                const uint32_t bh0 = brc::movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph01));
                const uint32_t bh1 = brc::movmatrix_trans(*reinterpret_cast<const uint32_t *>(&ph23));
                const uint32_t bl0 = brc::movmatrix_trans(brc::pack_half2(p0 - f01.x, p1 - f01.y));
                const uint32_t bl1 = brc::movmatrix_trans(brc::pack_half2(p2 - f23.x, p3 - f23.y));
                if (!VQ8) {
                    // ---- O^T += V^T . P^T
#pragma unroll
                    for (int mt = 0; mt < C::MT; ++mt) {
                        uint32_t af[4];
                        brc::ldmatrix_x4_trans(af, sbase + (mt >> 2) * C::GROUP_BYTES + v_lane + ((v_x ^ ((mt & 3) * 2u)) << 4));
                        brc::mma_16816(o[mt], af, bh0, bh1);
                        brc::mma_16816(o[mt], af, bl0, bl1);
                    }
                } else {
                    // ---- q8_0 V.  The probabilities in the B-operand layout, back in f32 (head + tail): this lane holds
                    //      cells 2t, 2t + 1, 2t + 8, 2t + 9 of head g.
                    const float2 h0f = __half22float2(*reinterpret_cast<const __half2 *>(&bh0)), t0f = __half22float2(*reinterpret_cast<const __half2 *>(&bl0));
                    const float2 h1f = __half22float2(*reinterpret_cast<const __half2 *>(&bh1)), t1f = __half22float2(*reinterpret_cast<const __half2 *>(&bl1));
                    // Scaled by 2^7 here and back at the end of the unit: a block's scale is ~amax / 127, so p * scale is
                    // small and the binary16 tail of the product would fall among the subnormals, whose fixed step
                    // (2^-24) is then multiplied by quanta of up to 127.  The factor keeps the tails normal for any V
                    // inside binary16's range and costs nothing (a power of two).
                    const float pb0 = (h0f.x + t0f.x) * Q8_P_SCALE, pb1 = (h0f.y + t0f.y) * Q8_P_SCALE;
                    const float pb2 = (h1f.x + t1f.x) * Q8_P_SCALE, pb3 = (h1f.y + t1f.y) * Q8_P_SCALE;
                    const uint32_t vrow = sbase + q8_c0;
#pragma unroll
                    for (int blk = 0; blk < HD / 32; ++blk) {
                        // the block's scale of each of the four cells folded into their probabilities, head + tail again
                        const uint32_t at = vrow + blk * 36u;
                        float s0, s1, s2, s3;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s0) : "r"(at));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s1) : "r"(at + C::VROW_BYTES));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s2) : "r"(at + 8u * C::VROW_BYTES));
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s3) : "r"(at + 9u * C::VROW_BYTES));
                        const float w0 = pb0 * s0, w1 = pb1 * s1, w2 = pb2 * s2, w3 = pb3 * s3;
                        const __half2 wh01 = __floats2half2_rn(w0, w1), wh23 = __floats2half2_rn(w2, w3);
                        const float2 g01 = __half22float2(wh01), g23 = __half22float2(wh23);
                        const uint32_t ph0 = *reinterpret_cast<const uint32_t *>(&wh01), ph1 = *reinterpret_cast<const uint32_t *>(&wh23);
                        const uint32_t pl0 = brc::pack_half2(w0 - g01.x, w1 - g01.y), pl1 = brc::pack_half2(w2 - g23.x, w3 - g23.y);
                        // the quanta: this lane's word of the block in each of its four cells = values d = 32 blk + 4 g + j;
                        // byte j of two neighbouring cells becomes one binary16 pair, EXACT: bits 0x6400 | (q ^ 0x80) are
                        // 1024 + (q + 128), and 1152 is subtracted
                        uint32_t x0, x1, x2, x3;
                        const uint32_t qa = at + 4u + (lane >> 2) * 4u;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x0) : "r"(qa));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x1) : "r"(qa + C::VROW_BYTES));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x2) : "r"(qa + 8u * C::VROW_BYTES));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(x3) : "r"(qa + 9u * C::VROW_BYTES));
                        x0 ^= 0x80808080u, x1 ^= 0x80808080u, x2 ^= 0x80808080u, x3 ^= 0x80808080u;
                        const uint32_t ya = __byte_perm(x0, x1, 0x5410), yb = __byte_perm(x0, x1, 0x7632);   // bytes (0, 1) and (2, 3) of cells 2t, 2t + 1
                        const uint32_t za = __byte_perm(x2, x3, 0x5410), zb = __byte_perm(x2, x3, 0x7632);   // of cells 2t + 8, 2t + 9
                        const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));        // 1152
                        auto ints = [bias](uint32_t y, uint32_t sel) {
                            const uint32_t r = __byte_perm(y, 0x64646464u, sel);
                            const __half2 v = __hsub2(*reinterpret_cast<const __half2 *>(&r), bias);
                            return *reinterpret_cast<const uint32_t *>(&v);
                        };
                        // tile 2 blk: rows g, g + 8 = bytes 0, 1; tile 2 blk + 1: bytes 2, 3
                        const uint32_t a_lo[4] = {ints(ya, 0x4240), ints(ya, 0x4341), ints(za, 0x4240), ints(za, 0x4341)};
                        const uint32_t a_hi[4] = {ints(yb, 0x4240), ints(yb, 0x4341), ints(zb, 0x4240), ints(zb, 0x4341)};
                        brc::mma_16816(o[2 * blk], a_lo, ph0, ph1);
                        brc::mma_16816(o[2 * blk], a_lo, pl0, pl1);
                        brc::mma_16816(o[2 * blk + 1], a_hi, ph0, ph1);
                        brc::mma_16816(o[2 * blk + 1], a_hi, pl0, pl1);
                    }
                }
                // ---- hand the stage back to the producer
                if (nv < 16u) brc::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) brc::mbar_arrive(empty0 + 8u * stage);
            }
            stage += C::NWP;
            if (stage >= p.n_stages) {
                stage -= p.n_stages;
                parity ^= 1u;
            }
        }

        if (dead && lane == 0) dead_cta[0] = 1u;
        // ---- merge, per kv head, the (m, l, O) of its warps and write this share's partial
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            l0 += __shfl_xor_sync(0xffffffffu, l0, off);
            l1 += __shfl_xor_sync(0xffffffffu, l1, off);
        }
        // The exchange goes through shared memory in two halves of head_dim (half the scratch, which
        // buys the ring more stages).  Weights of the warps are computed once, by one thread per head.
        float *sw = scratch + warp * C::SCRATCH_WARP;
        if (lane < 4) {
            float *ml = sw + GROUP_TILE * C::OPAD;
            ml[h0 * 2] = m0;
            ml[h0 * 2 + 1] = l0;
            ml[h0 * 2 + 2] = m1;
            ml[h0 * 2 + 3] = l1;
        }
        const size_t slot0 = (size_t)(ur.U + blockIdx.x) * KVB;
        // A unit that lies wholly inside this CTA's share has no other share to meet: its rows go
        // straight to the output (normalised and gated, or as the merged partial), with no partial slot,
        // no fence, no ticket and no read-back.  With many short sequences, or with several layers in one
        // launch, most units are of this kind.
        const bool whole = WHOLE_FAST && unit_first >= a && lbase + S[u + 1] <= b;
        const uint32_t seq_of_u = u / n_groups, kv0_of_u = (u % n_groups) * KVB;
        float *const out_l = p.out + layer * p.out_layer_stride;
        float *const out_ml_l = p.out_ml ? p.out_ml + layer * p.out_ml_layer_stride : nullptr;
        const float *const gate_l = p.gate ? p.gate + layer * p.gate_layer_stride : nullptr;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
            for (int mh = 0; mh < C::MT / 2; ++mh) {
                const int mt = hf * (C::MT / 2) + mh;
                // rows t0 and t0 + 8 of accumulator tile mt hold value d0 and d1 of this half of head_dim: with
                // binary16 V the tile's rows are consecutive values; with q8_0 V a lane's four bytes of a block
                // sit in rows t0, t0 + 8 of two neighbouring tiles
                const uint32_t d0 = VQ8 ? (mh >> 1) * 32 + t0 * 4 + (mh & 1) * 2 : mh * 16 + t0;
                const uint32_t d1 = VQ8 ? d0 + 1 : d0 + 8;
                constexpr float back = VQ8 ? 1.f / Q8_P_SCALE : 1.f;   // undoes the factor on the q8_0 probabilities (exact)
                sw[h0 * C::OPAD + d0] = o[mt][0] * back;
                sw[(h0 + 1) * C::OPAD + d0] = o[mt][1] * back;
                sw[h0 * C::OPAD + d1] = o[mt][2] * back;
                sw[(h0 + 1) * C::OPAD + d1] = o[mt][3] * back;
            }
            brc::named_bar_sync(1, NW * 32);
            if (hf == 0 && tid < KVB * GROUP_TILE) {
                // thread = (kv head of the group, query head): weights 2^(m_w - M) of its NWP warps
                const uint32_t k2 = tid / GROUP_TILE, h = tid % GROUP_TILE;
                float mw[C::NWP], lw[C::NWP], M = -INFINITY, L = 0.f;
#pragma unroll
                for (int w = 0; w < C::NWP; ++w) {
                    const float *ml = scratch + (w * KVB + k2) * C::SCRATCH_WARP + GROUP_TILE * C::OPAD;
                    mw[w] = ml[h * 2];
                    lw[w] = ml[h * 2 + 1];
                    if (lw[w] > 0.f) M = fmaxf(M, mw[w]);
                }
#pragma unroll
                for (int w = 0; w < C::NWP; ++w) {
                    const float wt = (lw[w] > 0.f && !dead_cta[0]) ? brc::fast_exp2(mw[w] - M) : 0.f;
                    wts[w * KVB * GROUP_TILE + tid] = wt;
                    L += wt * lw[w];
                }
                inv_l[tid] = L > 0.f ? 1.f / L : 0.f;
                if (h < p.group) {
                    if (!whole) {
                        float *ml_out = p.part_ml + ((slot0 + k2) * GROUP_TILE + h) * 2;
                        ml_out[0] = M;
                        ml_out[1] = L;
                    } else if (out_ml_l) {
                        float *ml_out = out_ml_l + ((size_t)seq_of_u * p.n_head + (kv0_of_u + k2) * p.group_all + p.head0 + h) * 2;
                        ml_out[0] = M;
                        ml_out[1] = L;
                    }
                }
            }
            if (hf == 0) brc::named_bar_sync(1, NW * 32);
            // flat, independent iterations: (kv head, query head) = j, d = tid (+ 128)
#pragma unroll 4
            for (uint32_t idx = tid; idx < KVB * GROUP_TILE * (HD / 2); idx += NW * 32) {
                const uint32_t kh = idx / (HD / 2), d = idx % (HD / 2);
                const uint32_t k2 = kh / GROUP_TILE, h = kh % GROUP_TILE;
                if (h < p.group) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < C::NWP; ++w)
                        v += wts[w * KVB * GROUP_TILE + kh] * scratch[(w * KVB + k2) * C::SCRATCH_WARP + h * C::OPAD + d];
                    if (!whole) {
                        p.part_acc[((slot0 + k2) * GROUP_TILE + h) * HD + hf * (HD / 2) + d] = v;
                    } else {
                        const size_t row = (size_t)seq_of_u * p.n_head + (kv0_of_u + k2) * p.group_all + p.head0 + h;
                        const uint32_t col = hf * (HD / 2) + d;
                        if (!out_ml_l) {
                            v *= inv_l[kh];
                            if (gate_l) v *= sigmoid_f32(gate_l[row * p.gate_head_stride + col]);
                        }
                        out_l[row * HD + col] = v;
                    }
                }
            }
            brc::named_bar_sync(1, NW * 32);
        }
        if (!whole && tid == 0) {
            // ---- ticket: this piece of the unit is written.  The barrier above ordered every thread's stores before
            //      this thread's fence (the pattern of a grid-wide barrier).  What the add returns says whether this
            //      was the unit's last piece to arrive: remembered for the merge of the share's last unit.
            uint32_t i_lo, i_hi, j, k;
            share_range(B, gridDim.x, unit_first, lbase + S[u + 1] - 1, i_lo, i_hi);
            piece_of(B, all_shares_live, i_lo, i_hi, j, k);
            __threadfence();
            const uint32_t w = piece_weight(j, k);
            tk_sum = atomicAdd(p.done + layer * BRC_DONE_BANK_WORDS + u, w) + w;   // not waited for until the merges
            tk_unit = ur.U;
        }

        // ---- next unit of the flat (layer, unit) list that has pages
        g0 = ge;
        ++u;
        for (;;) {
            if (u == n_units) {
                u = 0;
                if (++layer == p.n_layers) break;
            }
            if (S[u + 1] != S[u]) break;
            ++u;
        }
    }

    // ---------------------------------------------------------------------- merges
    // Every unit of which this CTA streamed a share that is not the whole unit (at most the first and the last unit
    // of its share, when no share is empty) is merged now, together with the other CTAs that hold shares of it.
    // All of this CTA's streaming is done and all of its shares are written, so waiting here holds nothing up
    // and no CTA waits for one that waits for it.
    if (a < b) {
        uint32_t fl = first_layer, fu = first_u;
        while (fl < p.n_layers) {
            const uint32_t ubeg = fl * total_l + S[fu], uend = fl * total_l + S[fu + 1];   // [ubeg, uend): the unit's page-units
            if (ubeg >= b) break;
            if (uend != ubeg && !(WHOLE_FAST && ubeg >= a && uend <= b)) {
                const UnitRef ur = {fl * n_units + fu, fl, fu};
                uint32_t i_lo, i_hi;
                share_range(B, gridDim.x, ubeg, uend - 1, i_lo, i_hi);
                merge_unit<HD, KVB, !WHOLE_FAST, VQ8>(p, ur, i_lo, i_hi, B, all_shares_live, tid, scratch, reinterpret_cast<float4 *>(ring), epoch, bank,
                                                      gave_up, tk_unit == ur.U && (tk_sum & TICKET_LOW) == 0u);
            }
            if (++fu == n_units) {
                fu = 0;
                ++fl;
            }
        }
    }
    if (!push) return;
    // ---------------------------------------------------------------------- cross-rank merge
    // The rows of a unit are dealt over the CTAs that streamed a share of it; units without pages go round the
    // grid.  The ranks that still stream never wait for this one.
    if (a < b) {
        uint32_t fl = first_layer, fu = first_u;
        while (fl < p.n_layers) {
            const uint32_t ubeg = fl * total_l + S[fu], uend = fl * total_l + S[fu + 1];
            if (ubeg >= b) break;
            if (uend != ubeg) {
                const UnitRef ur = {fl * n_units + fu, fl, fu};
                uint32_t i_lo, i_hi, j, k;
                share_range(B, gridDim.x, ubeg, uend - 1, i_lo, i_hi);
                brc::named_bar_sync(1, NW * 32);
                unit_pieces(B, all_shares_live, i_lo, i_hi, tid, NW * 32, reinterpret_cast<uint16_t *>(scratch),
                            reinterpret_cast<volatile uint32_t *>(reinterpret_cast<uint16_t *>(scratch) + MAX_CTAS), j, k);
                finalize_unit<HD, KVB, VQ8>(p, ur, j, k, bank, tid, gave_up);
            }
            if (++fu == n_units) {
                fu = 0;
                ++fl;
            }
        }
    }
    for (uint32_t U = blockIdx.x; U < n_units_all; U += gridDim.x) {
        const uint32_t fl = U / n_units, fu = U - fl * n_units;
        if (S[fu + 1] != S[fu]) continue;
        const UnitRef ur = {U, fl, fu};
        finalize_unit<HD, KVB, VQ8>(p, ur, 0, 1, bank, tid, gave_up);
    }
    // ---- the launch's last CTA advances the epoch (every CTA has read it by now)
    brc::named_bar_sync(1, NW * 32);
    if (tid == 0) {
        const uint32_t t = atomicAdd(p.fin_ticket, 1u);
        if (t + 1u == gridDim.x) {
            *p.fin_ticket = 0u;
            *p.calls = epoch;
        }
    }
}

// Merge n_parts exchanged partial buffers (acc block followed by (m, l) block each).
template <int HD>
__global__ void __launch_bounds__(HD)
    parts_combine_kernel(const uint8_t *parts, uint32_t n_parts, uint64_t part_stride, uint32_t n_rows /* n_seqs*n_head */,
                         const float *gate, uint32_t gate_head_stride, float *out) {
    const uint32_t row = blockIdx.x, tid = threadIdx.x;
    float M = -INFINITY;
    for (uint32_t r = 0; r < n_parts; ++r) {
        const float *ml = reinterpret_cast<const float *>(parts + r * part_stride + (size_t)n_rows * HD * 4) + (size_t)row * 2;
        if (ml[1] > 0.f) M = fmaxf(M, ml[0]);
    }
    float acc = 0.f, L = 0.f;
    for (uint32_t r = 0; r < n_parts; ++r) {
        const float *base = reinterpret_cast<const float *>(parts + r * part_stride);
        const float *ml = base + (size_t)n_rows * HD + (size_t)row * 2;
        const float l = ml[1];
        if (!(l > 0.f)) continue;
        const float w = exp2f(ml[0] - M);
        L += w * l;
        acc += w * base[(size_t)row * HD + tid];
    }
    float v = L > 0.f ? acc / L : 0.f;
    if (gate) v *= sigmoid_f32(gate[(size_t)row * gate_head_stride + tid]);
    out[(size_t)row * HD + tid] = v;
}

#undef all_shares_live

// How fast does each CTA's SM stream from HBM while all the others do too?  The SMs of a B200 do not get equal
// shares of the memory system (always the same ones are slow, whatever is read), and with equal shares of a
// 12-layer launch the last CTAs stream for 35 us of 520 after the median one has finished.  One thread per CTA keeps a ring of
// CAL_STAGES bulk copies of CAL_CHUNK bytes in flight from pseudo-random places in `base` for `window_ns` and
// counts what has landed; same grid, block size and shared memory as the decode kernel, launched the same
// way, so that block i lands on the SM that the decode kernel's block i gets on an otherwise idle GPU.
constexpr uint32_t CAL_CHUNK = 32768, CAL_STAGES = 6;

__global__ void __launch_bounds__(160, 1) stream_rate_kernel(const uint8_t *base, uint32_t n_chunks, uint64_t window_ns, uint32_t *landed,
                                                             uint32_t *status) {
    extern __shared__ uint8_t cal_smem_raw[];
    uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(cal_smem_raw) + 1023u) & ~uintptr_t(1023));
    __shared__ uint64_t bars[CAL_STAGES];
    if (threadIdx.x != 0) return;
    const uint32_t bar0 = brc::smem_u32(bars), ring0 = brc::smem_u32(ring);
    for (uint32_t i = 0; i < CAL_STAGES; ++i) brc::mbar_init(bar0 + 8u * i, 1);
    brc::mbar_fence_init();
    uint32_t next = 0, done = 0;
    auto issue = [&](uint32_t stage) {
        const uint32_t chunk = (uint32_t)(((uint64_t)blockIdx.x * 7919u + (uint64_t)next * 104729u) % n_chunks);
        ++next;
        brc::mbar_arrive_expect_tx(bar0 + 8u * stage, CAL_CHUNK);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ring0 + stage * CAL_CHUNK),
                     "l"(base + (size_t)chunk * CAL_CHUNK), "r"(CAL_CHUNK), "r"(bar0 + 8u * stage)
                     : "memory");
    };
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t i = 0; i < CAL_STAGES; ++i) issue(i);
    uint32_t in_flight = CAL_STAGES, stage = 0, parity = 0;
    bool counting = true;
    while (in_flight) {
        if (!brc::mbar_wait(bar0 + 8u * stage, parity)) {   // bounded: gives up after seconds
            atomicOr(status, BRC_DEV_WAIT_LIMIT);
            status[1] = 5000000u + blockIdx.x;
            break;
        }
        --in_flight;
        counting = counting && globaltimer_ns() - t0 < window_ns;
        if (counting) {
            ++done;
            issue(stage);
            ++in_flight;
        }
        if (++stage == CAL_STAGES) {
            stage = 0;
            parity ^= 1u;
        }
    }
    landed[blockIdx.x] = done;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
uint32_t kvb_of(const brc_pool *pool) { return pool->n_kv_head % 2u == 0u ? 2u : 1u; }

// Bytes from one ring stage to the next (Cfg::STAGE_BYTES): K and V tiles of 16 cells of `kvb` kv heads; with q8_0 V
// the V part is 36 bytes per 32 values, and the sum is rounded up to the swizzle pattern's 1024-byte period.
uint32_t stage_bytes_of(uint32_t head_dim, uint32_t kvb, bool v_q8) {
    const uint32_t k = kvb * 16u * head_dim * 2u;
    const uint32_t v = v_q8 ? kvb * 16u * (head_dim / 32u * 36u) : k;
    return (k + v + 1023u) / 1024u * 1024u;
}

uint32_t fixed_bytes_of(uint32_t head_dim, bool v_q8) {   // independent of KVB
    if (v_q8) return head_dim == 256 ? Cfg<256, 1, true>::FIXED_BYTES : Cfg<128, 1, true>::FIXED_BYTES;
    return head_dim == 256 ? Cfg<256, 1>::FIXED_BYTES : Cfg<128, 1>::FIXED_BYTES;
}

// Ring depth: what fits, rounded down to a multiple of the NW / KVB warps that interleave page-units.
// Page-unit kk uses stage kk % n_stages and consumer slot kk % (NW / KVB); with the multiple, a stage
// is always consumed by the same warps.  This matters: a parity wait on an mbarrier is only valid if
// the waiter knows the previous phase of that barrier has completed.  A warp that has itself consumed
// round r - 1 of a stage knows; a different warp asking for round r while round r - 1 is still
// landing would see "parity r done" (it is round r - 2 that is), read a half-written stage and hand
// it back a second time.
uint32_t stages_for(uint32_t head_dim, uint32_t kvb, bool v_q8) {
    const uint32_t fit = std::min<uint32_t>((SMEM_LIMIT - fixed_bytes_of(head_dim, v_q8)) / stage_bytes_of(head_dim, kvb, v_q8), 24u);
    const uint32_t nwp = (uint32_t)consumer_warps(v_q8, (int)head_dim) / kvb;
    return fit / nwp * nwp;
}

}  // namespace

// Shares of a launch's cost per CTA, in proportion to the streaming rates measured by stream_rate_kernel.  OFF unless
// BRC_DECODE_CALIBRATE=1 is in the environment.  Measured on B200: the rates differ by -19 .. +16 % between SMs in
// pure streaming and by about -8 .. +9 % inside the decode kernel; a launch as a whole is bound by HBM rather than
// by its slowest SM (while the slow CTAs finish alone they stream faster), so only a part of the measured
// deviation is applied (BRC_DECODE_RATE_DAMP, default 0.4).  With that, a 12-layer launch over ONE long sequence
// gets 3-4 % faster (485 -> 468 us for 131 072 cells, 135.6 -> 130 us for 32 768); the batched workloads move
// between +1 % and -2 % from box to box, and the q8_0 V path, which is bound by instruction issue and not by the
// memory system, loses 9 % - hence off by default, and results never depend on a measurement unless asked to.
// When on: measured once per device and process (every pool of the device cuts alike), on the first pool of at
// least 1 GiB (smaller ones would be read from L2); deviations are rounded to 1/64 and kept within 0.75 .. 1.25.
// Never fails the caller: without a measurement the shares stay equal.
void brc_decode_calibrate(brc_pool *pool) {
    static std::mutex mu;
    static uint32_t *prefix_of_device[64] = {};
    static std::vector<float> rates_of_device[64];
    static bool tried[64] = {};
    if (pool->device < 0 || pool->device >= 64 || !pool->k_base) return;
    std::lock_guard<std::mutex> lock(mu);
    if (prefix_of_device[pool->device]) {
        pool->cut_prefix = prefix_of_device[pool->device];
        pool->cut_rates = rates_of_device[pool->device];
        return;
    }
    const char *env = std::getenv("BRC_DECODE_CALIBRATE");
    const uint64_t bytes = (uint64_t)(pool->v_base - pool->k_base);   // the K pool
    if (tried[pool->device] || !(env && *env == '1') || bytes < (1ull << 30)) return;
    tried[pool->device] = true;
    const uint32_t grid = std::min<uint32_t>((uint32_t)(pool->sm_count > 0 ? pool->sm_count : 148), MAX_CTAS);
    uint32_t *landed = nullptr, *prefix = nullptr;
    if (cudaMalloc(&landed, (MAX_CTAS + 4) * 4) != cudaSuccess || cudaMalloc(&prefix, (MAX_CTAS + 4) * 4) != cudaSuccess) {
        cudaGetLastError();
        if (landed) cudaFree(landed);
        return;
    }
    const uint32_t smem = CAL_STAGES * CAL_CHUNK + 2048;   // the ring, and room to start it on a 1024-byte boundary
    cudaFuncSetAttribute(stream_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    std::vector<double> rate(grid, 0.0);
    bool ok = true;
    for (int rep = 0; rep < 4 && ok; ++rep) {            // the first run warms up; three are averaged
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(160);
        cfg.dynamicSmemBytes = smem;                      // more than half an SM's shared memory: one CTA per SM, as the decode kernel
        cfg.stream = nullptr;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        std::vector<uint32_t> host(grid);
        ok = cudaLaunchKernelEx(&cfg, stream_rate_kernel, (const uint8_t *)pool->k_base, (uint32_t)(bytes / CAL_CHUNK), (uint64_t)300000,
                                landed, pool->status_dev) == cudaSuccess &&
             cudaMemcpy(host.data(), landed, grid * 4, cudaMemcpyDeviceToHost) == cudaSuccess;
        if (ok && rep > 0)
            for (uint32_t i = 0; i < grid; ++i) rate[i] += host[i];
    }
    cudaFree(landed);
    double mean = 0.0;
    for (double r : rate) mean += r / grid;
    if (!ok || mean < 16.0) {   // nothing measured (or a failed launch): equal shares
        cudaGetLastError();
        cudaFree(prefix);
        return;
    }
    const char *damp_env = std::getenv("BRC_DECODE_RATE_DAMP");
    const double damp = damp_env && *damp_env ? std::atof(damp_env) : 0.4;
    std::vector<uint32_t> host_prefix(grid + 1);
    double total = 0.0;
    for (uint32_t i = 0; i < grid; ++i) {
        rate[i] = std::min(1.25, std::max(0.75, std::round((1.0 + damp * (rate[i] / mean - 1.0)) * 64.0) / 64.0));
        total += rate[i];
    }
    double run = 0.0;
    for (uint32_t i = 0; i < grid; ++i) {
        host_prefix[i] = (uint32_t)std::min(4294967295.0, run / total * 4294967296.0);
        run += rate[i];
    }
    host_prefix[grid] = 0xffffffffu;
    if (cudaMemcpy(prefix, host_prefix.data(), (grid + 1) * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(prefix);
        return;
    }
    prefix_of_device[pool->device] = prefix;             // kept for the life of the process
    pool->cut_prefix = prefix;
    rates_of_device[pool->device].assign(rate.begin(), rate.end());
    pool->cut_rates = rates_of_device[pool->device];
}

namespace {

uint32_t seqs_per_launch(const brc_pool *pool) { return MAX_UNITS / (pool->n_kv_head / kvb_of(pool)); }

uint32_t grid_ctas(const brc_pool *pool) { return std::min<uint32_t>((uint32_t)(pool->sm_count > 0 ? pool->sm_count : 148), MAX_CTAS); }

// One TMA operation per page-unit (the pool's views whose last dimension is the 64-column group) instead of one per
// column group.  OFF unless BRC_DECODE_STAGE_OP=1 is in the environment: in those views the group's stride (128 bytes)
// follows a larger one, which the driver's encoder accepts but its documentation does not allow (every stride a
// multiple of the one before).  Measured here over some tens of thousands of launches without a fault and with
// identical results - 0.5 % on the 32-sequence batch, 9 % over q8_0 V pages (67.4 k -> 73.6 k tok/s), 15 % with one kv
// head per unit - but an earlier build with such a view saw bounded waits give up now and then, so the default
// stays inside the documented rules.
bool stage_in_one_operation() {
    static const bool on = [] {
        const char *e = std::getenv("BRC_DECODE_STAGE_OP");
        return e && *e == '1';
    }();
    return on;
}

// What every unit it touches costs a CTA on top of the unit's pages (merge of the warps, partial or output
// written, ticket, perhaps the unit's merge), in page-units of this pool.  Measured on the 32-sequence batches
// of skewed and of equal lengths: an isolated launch gets faster up to about 16 page-units of 32 KiB (64 -> 60 us
// and 101 -> 98 us), a 12-layer launch by 1.5 %, and nothing changes beyond; hence 512 KiB worth of page-units.
// BRC_DECODE_UNIT_COST in the environment overrides it (0 = cut into equal numbers of page-units).
uint32_t unit_cost_of(uint32_t head_dim, uint32_t kvb, bool v_q8) {
    static const long env = [] {
        const char *e = std::getenv("BRC_DECODE_UNIT_COST");
        return e && *e ? std::strtol(e, nullptr, 10) : -1L;
    }();
    if (env >= 0) return (uint32_t)std::min(env, 64L);
    return std::max<uint32_t>(1u, (512u * 1024u + stage_bytes_of(head_dim, kvb, v_q8) / 2u) / stage_bytes_of(head_dim, kvb, v_q8));
}

// Partial slots of one launch over `n_layers` layers of `n_seqs` sequences: one per (layer, unit) plus one
// per CTA (a share boundary inside a unit makes one more partial), x KVB kv heads; acc then (m, l).
uint64_t slots_for(const brc_pool *pool, uint32_t n_seqs, uint32_t n_layers = 1) {
    const uint32_t per = std::min<uint32_t>(n_seqs, seqs_per_launch(pool));
    const uint32_t kvb = kvb_of(pool);
    return ((uint64_t)n_layers * per * (pool->n_kv_head / kvb) + grid_ctas(pool)) * kvb;
}

uint64_t slot_floats(const brc_pool *pool) { return (uint64_t)GROUP_TILE * (pool->head_dim + 2u); }

template <int HD, bool Q_F32, int KVB, bool VQ8>
brc_status launch_partial(brc_pool *pool, const DecodeParams &p, uint32_t grid, uint32_t smem, cudaStream_t st) {
    static bool configured[64] = {};
    if (pool->device < 64 && !configured[pool->device]) {
        BRC_CUDA(cudaFuncSetAttribute(decode_partial_kernel<HD, Q_F32, KVB, false, VQ8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)SMEM_LIMIT));
        BRC_CUDA(cudaFuncSetAttribute(decode_partial_kernel<HD, Q_F32, KVB, true, VQ8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)SMEM_LIMIT));
        configured[pool->device] = true;
    }
    // With at least as many units as CTAs most units lie inside one share: compile their direct-output
    // path in.  The cross-GPU form always goes through the partial slots (one place pushes to the peers).
    const bool many_units = p.world <= 1 && (uint64_t)p.n_layers * p.n_seqs * (p.n_kv_head / KVB) >= grid;
    auto kern = many_units ? decode_partial_kernel<HD, Q_F32, KVB, true, VQ8> : decode_partial_kernel<HD, Q_F32, KVB, false, VQ8>;
    // binary16 V: one 3-D view over K and V.  q8_0 V: K alone, and the V rows in 32-bit words.
    const CUtensorMap &tm_a = VQ8 ? (p.one_op ? (KVB == 2 ? pool->tm_k2_stage : pool->tm_k_stage) : (KVB == 2 ? pool->tm_k2 : pool->tm_k))
                                  : (KVB == 2 ? pool->tm_kv2 : pool->tm_kv);
    const CUtensorMap &tm_b = VQ8 ? (KVB == 2 ? pool->tm_v8_2 : pool->tm_v8) : p.one_op ? (KVB == 2 ? pool->tm_kv2_stage : pool->tm_kv_stage) : tm_a;
    brc_stage_begin(pool, BRC_STAGE_ATTN_PARTIAL, st);
    // Cooperative: the CTAs of a unit wait for one another's shares at the end of the launch, so all of them must be
    // resident at once (one per SM; the launch fails instead of starting when the device cannot hold the grid).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(Cfg<HD, KVB, VQ8>::NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, p);
    brc_stage_end(pool, BRC_STAGE_ATTN_PARTIAL, st);
    BRC_CUDA(e);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

template <int HD, bool Q_F32>
brc_status launch_partial_kvb(brc_pool *pool, const DecodeParams &p, uint32_t grid, uint32_t smem, cudaStream_t st) {
    if (pool->v_q8)
        return kvb_of(pool) == 2 ? launch_partial<HD, Q_F32, 2, true>(pool, p, grid, smem, st)
                                 : launch_partial<HD, Q_F32, 1, true>(pool, p, grid, smem, st);
    return kvb_of(pool) == 2 ? launch_partial<HD, Q_F32, 2, false>(pool, p, grid, smem, st)
                             : launch_partial<HD, Q_F32, 1, false>(pool, p, grid, smem, st);
}

brc_status validate_decode(const brc_pool *pool, const char *who, uint32_t layer0, uint32_t n_layers, const void *q,
                           int32_t q_dtype, uint32_t n_head, const uint32_t *bt, uint32_t table_stride, const uint32_t *lens,
                           uint32_t n_seqs, uint32_t max_seq_len, const void *out, const void *ws, uint64_t ws_bytes) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "%s: pool is NULL", who);
    if (pool->device < 0 || !pool->has_tma)
        return brc_fail(BRC_ERR_CUDA, "%s: this pool holds bookkeeping only (no device memory); compute calls need a GPU pool", who);
    if ((uint64_t)layer0 + n_layers > pool->n_layers)
        return n_layers == 1 ? brc_fail(BRC_ERR_INVALID, "%s: layer %u but the pool has %u", who, layer0, pool->n_layers)
                             : brc_fail(BRC_ERR_INVALID, "%s: layers %u..%u but the pool has %u", who, layer0, layer0 + n_layers,
                                        pool->n_layers);
    if (q_dtype != BRC_DTYPE_F32 && q_dtype != BRC_DTYPE_F16)
        return brc_fail(BRC_ERR_INVALID, "%s: q_dtype %d is neither f32 (0) nor f16 (1)", who, q_dtype);
    if (n_head == 0 || n_head % pool->n_kv_head != 0)
        return brc_fail(BRC_ERR_INVALID, "%s: %u query heads do not divide over %u kv heads", who, n_head, pool->n_kv_head);
    if (n_head / pool->n_kv_head > 4 * GROUP_TILE)
        return brc_fail(BRC_ERR_UNSUPPORTED, "%s: %u query heads per kv head (up to %d, in passes of %d)", who,
                        n_head / pool->n_kv_head, 4 * GROUP_TILE, GROUP_TILE);
    const uint64_t capacity = (uint64_t)table_stride * pool->page_tokens;
    if (max_seq_len > capacity)
        return brc_fail(BRC_ERR_CAPACITY, "%s would read cells up to %u but each block table holds %llu (%u pages of %u cells)",
                        who, max_seq_len, (unsigned long long)capacity, table_stride, pool->page_tokens);
    if (n_seqs == 0 || n_layers == 0) return BRC_OK;
    if (!q || !bt || !lens || !out) return brc_fail(BRC_ERR_INVALID, "%s: NULL query, block table, length or output pointer", who);
    if ((reinterpret_cast<uintptr_t>(q) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
        return brc_fail(BRC_ERR_INVALID, "%s: query and output pointers must be 16-byte aligned", who);
    uint64_t need = 0;
    brc_decode_workspace_bytes(pool, n_seqs, n_head, &need);
    if (!ws || ws_bytes < need)
        return brc_fail(BRC_ERR_INVALID, "%s: workspace of %llu bytes, %llu needed", who, (unsigned long long)ws_bytes,
                        (unsigned long long)need);
    return BRC_OK;
}

// Decode calls on one pool share its arrival counters.  Calls on one stream are ordered anyway; a call
// on another stream than the previous one is made to wait for it (an event recorded after every decode
// launch), so two streams can never have decode kernels of one pool in flight together.  While a stream
// is being captured nothing is recorded or awaited: a captured graph must be replayed on its own.
brc_status order_after_previous_decode(brc_pool *pool, cudaStream_t st, bool *capturing) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) cudaGetLastError();
    *capturing = cs != cudaStreamCaptureStatusNone;
    if (*capturing) return BRC_OK;
    if (pool->decode_event && pool->decode_stream_set && pool->decode_stream != st)
        BRC_CUDA(cudaStreamWaitEvent(st, pool->decode_event, 0));
    return BRC_OK;
}

brc_status note_decode_issued(brc_pool *pool, cudaStream_t st, bool capturing) {
    if (capturing) return BRC_OK;
    if (!pool->decode_event) BRC_CUDA(cudaEventCreateWithFlags(&pool->decode_event, cudaEventDisableTiming));
    BRC_CUDA(cudaEventRecord(pool->decode_event, st));
    pool->decode_stream = st;
    pool->decode_stream_set = true;
    return BRC_OK;
}

}  // namespace

// The one implementation behind every decode entry point.  out_ml != nullptr: partial mode (out = merged
// acc, out_ml = (m, l)); push != nullptr with world > 1: split-KV across GPUs; else the final output.
// Launches: one per (chunk of <= 2048 units per layer) x (group of layers whose partial slots fit the
// workspace, at most BRC_DONE_BANKS) x (pass of GROUP_TILE query heads per kv head).
brc_status brc_decode_layers(brc_pool *pool, const char *who, const brc_layers_args &a, void *stream) {
    if (brc_status rc = validate_decode(pool, who, a.layer0, a.n_layers, a.q, a.q_dtype, a.n_head, a.block_tables, a.table_stride,
                                        a.seq_lens, a.n_seqs, a.max_seq_len, a.out, a.workspace, a.workspace_bytes))
        return rc;
    if (a.gate && a.gate_head_stride < pool->head_dim)
        return brc_fail(BRC_ERR_INVALID, "%s: gate_head_stride %u < head_dim %u", who, a.gate_head_stride, pool->head_dim);
    if (a.k_new || a.v_new) {
        if (a.kv_dtype != BRC_DTYPE_F32 && a.kv_dtype != BRC_DTYPE_F16)
            return brc_fail(BRC_ERR_INVALID, "%s: kv_dtype %d is neither f32 (0) nor f16 (1)", who, a.kv_dtype);
        if (!a.k_new || !a.v_new || (reinterpret_cast<uintptr_t>(a.k_new) & 15u) || (reinterpret_cast<uintptr_t>(a.v_new) & 15u))
            return brc_fail(BRC_ERR_INVALID, "%s: new K/V pointers must be non-NULL and 16-byte aligned", who);
        if (pool->v_q8 && a.kv_dtype != BRC_DTYPE_F32)
            return brc_fail(BRC_ERR_UNSUPPORTED, "%s: a q8_0 V pool quantises from f32 sources (as the reference's store rule does), "
                                                 "never through binary16", who);
    }
    if (a.n_seqs == 0 || a.n_layers == 0) return BRC_OK;

    brc_device_guard guard(pool->device);
    cudaStream_t st = brc_stream(stream);
    const uint32_t hd = pool->head_dim;
    const uint32_t kvb = kvb_of(pool);
    const uint32_t n_groups = pool->n_kv_head / kvb;
    const uint32_t n_stages = stages_for(hd, kvb, pool->v_q8);
    const uint32_t smem = n_stages * stage_bytes_of(hd, kvb, pool->v_q8) + fixed_bytes_of(hd, pool->v_q8);
    const uint32_t grid = grid_ctas(pool);
    const uint32_t per = seqs_per_launch(pool);
    const size_t q_elem = a.q_dtype == BRC_DTYPE_F32 ? 4 : 2;
    const size_t kv_elem = a.kv_dtype == BRC_DTYPE_F32 ? 4 : 2;
    const bool push = a.push && a.push->world > 1;
    const uint32_t ns_max = std::min(per, a.n_seqs);

    // layers per launch: bounded by the counter banks, by the partial slots the workspace holds, and by
    // 32-bit page-unit indices
    const uint64_t ws_slots = a.workspace_bytes / (slot_floats(pool) * sizeof(float));
    uint64_t lpl = std::min<uint64_t>(a.n_layers, BRC_DONE_BANKS);
    {
        const uint64_t unit_slots = (uint64_t)ns_max * n_groups * kvb;          // per layer
        const uint64_t fit = (ws_slots - (uint64_t)grid * kvb) / unit_slots;    // >= 1: validated above
        lpl = std::min(lpl, std::max<uint64_t>(fit, 1));
        const uint64_t pu_layer = (uint64_t)ns_max * n_groups * ((a.max_seq_len + 15u) / 16u);
        if (pu_layer >= (1ull << 32))
            return brc_fail(BRC_ERR_UNSUPPORTED, "%s: %llu page-units in one layer of one launch (32-bit indices)", who,
                            (unsigned long long)pu_layer);
        if (pu_layer) lpl = std::min(lpl, std::max<uint64_t>(((1ull << 32) - 1) / pu_layer, 1));
    }
    if (push && (lpl < a.n_layers || a.n_seqs > per))
        return brc_fail(BRC_ERR_CAPACITY,
                        "%s: the exchange across GPUs takes one launch per call: %u layers x %u sequences need a workspace of "
                        "%llu bytes (given %llu), at most %u layers and %u sequences",
                        who, a.n_layers, a.n_seqs,
                        (unsigned long long)(slots_for(pool, a.n_seqs, a.n_layers) * slot_floats(pool) * sizeof(float)),
                        (unsigned long long)a.workspace_bytes, BRC_DONE_BANKS, per);

    bool capturing = false;
    if (brc_status rc = order_after_previous_decode(pool, st, &capturing)) return rc;

    const uint64_t layer_rows = (uint64_t)pool->n_pages * pool->n_kv_head * pool->page_tokens;
    for (uint32_t s0 = 0; s0 < a.n_seqs; s0 += per) {
        const uint32_t ns = std::min(per, a.n_seqs - s0);
        for (uint32_t l0 = 0; l0 < a.n_layers; l0 += (uint32_t)lpl) {
            const uint32_t nl = std::min<uint32_t>((uint32_t)lpl, a.n_layers - l0);
            const uint64_t slots = ((uint64_t)nl * ns * n_groups + grid) * kvb;
            DecodeParams p = {};
            p.q = static_cast<const uint8_t *>(a.q) + l0 * a.q_layer_stride_bytes + (size_t)s0 * a.n_head * hd * q_elem;
            p.block_tables = a.block_tables + (size_t)s0 * a.table_stride;
            p.seq_lens = a.seq_lens + s0;
            p.part_acc = static_cast<float *>(a.workspace);
            p.part_ml = p.part_acc + slots * GROUP_TILE * hd;
            p.done = pool->status_dev + BRC_STATUS_WORDS;
            p.out = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(a.out) + l0 * a.out_layer_stride_bytes) + (size_t)s0 * a.n_head * hd;
            p.out_ml = a.out_ml ? a.out_ml + l0 * (a.out_ml_layer_stride_bytes / 4) + (size_t)s0 * a.n_head * 2 : nullptr;
            p.gate = a.gate ? reinterpret_cast<const float *>(reinterpret_cast<const uint8_t *>(a.gate) + l0 * a.gate_layer_stride_bytes) +
                                  (size_t)s0 * a.n_head * a.gate_head_stride
                            : nullptr;
            p.gate_head_stride = a.gate_head_stride;
            p.k_new = a.k_new ? static_cast<const uint8_t *>(a.k_new) + l0 * a.kv_layer_stride_bytes + (size_t)s0 * pool->n_kv_head * hd * kv_elem : nullptr;
            p.v_new = a.v_new ? static_cast<const uint8_t *>(a.v_new) + l0 * a.kv_layer_stride_bytes + (size_t)s0 * pool->n_kv_head * hd * kv_elem : nullptr;
            p.kv_new_f32 = a.kv_dtype == BRC_DTYPE_F32;
            p.k_base = pool->k_base;
            p.v_offset = (uint64_t)(pool->v_base - pool->k_base);
            p.status = pool->status_dev;
            p.n_seqs = ns;
            p.table_stride = a.table_stride;
            p.max_seq_len = a.max_seq_len;
            p.n_kv_head = pool->n_kv_head;
            p.group_all = a.n_head / pool->n_kv_head;
            p.n_head = a.n_head;
            p.n_pages = pool->n_pages;
            p.layer_rows = (uint32_t)layer_rows;
            p.layer_row0 = (uint32_t)((a.layer0 + l0) * layer_rows);
            p.n_stages = n_stages;
            p.scale_log2 = a.scale * 1.4426950408889634f;
            p.n_layers = nl;
            p.unit_cost = unit_cost_of(hd, kvb, pool->v_q8);
            p.one_op = (pool->stage_maps && stage_in_one_operation()) ? 1u : 0u;
            p.cut_prefix = grid == grid_ctas(pool) ? pool->cut_prefix : nullptr;
            p.q_layer_stride = a.q_layer_stride_bytes / q_elem;
            p.out_layer_stride = a.out_layer_stride_bytes / 4;
            p.out_ml_layer_stride = a.out_ml_layer_stride_bytes / 4;
            p.gate_layer_stride = a.gate_layer_stride_bytes / 4;
            p.kv_new_layer_stride = a.kv_layer_stride_bytes / kv_elem;
            p.world = 1;
            if (push) {
                const brc_push_args &x = *a.push;
                p.world = x.world;
                p.rank = x.rank;
                p.unit_items = x.unit_items;
                p.rows_total = nl * ns * a.n_head;
                for (uint32_t r = 0; r < x.world; ++r) p.peer_recv[r] = x.peer_recv[r];
                p.slot_stride = x.slot_stride;
                p.bank_stride = x.bank_stride;
                p.push_offset = x.push_offset;
                p.calls = x.calls;
                p.fin_ticket = x.fin_ticket;
                p.wait_ns = x.wait_ns;
                if ((uint64_t)nl * ns * n_groups > x.unit_items || (uint64_t)p.rows_total * (hd + 2u) * 4u > x.slot_stride)
                    return brc_fail(BRC_ERR_CAPACITY, "%s: %u layers x %u sequences exceed the exchange buffers", who, nl, ns);
            }
            // A tile holds GROUP_TILE query heads per kv head.  More than that (the reference model has 12) are
            // taken in passes of GROUP_TILE heads, each streaming the cache again: correct, at that price.  The
            // passes share the partials and counters, so they run strictly one after the other (stream
            // order), and only the first one appends.
            const uint32_t passes = (p.group_all + GROUP_TILE - 1) / GROUP_TILE;
            for (uint32_t pass = 0; pass < passes; ++pass) {
                p.head0 = pass * GROUP_TILE;
                p.group = std::min<uint32_t>(GROUP_TILE, p.group_all - p.head0);
                if (pass > 0) p.k_new = p.v_new = nullptr;
                brc_status rc;
                if (hd == 256)
                    rc = a.q_dtype == BRC_DTYPE_F32 ? launch_partial_kvb<256, true>(pool, p, grid, smem, st)
                                                    : launch_partial_kvb<256, false>(pool, p, grid, smem, st);
                else
                    rc = a.q_dtype == BRC_DTYPE_F32 ? launch_partial_kvb<128, true>(pool, p, grid, smem, st)
                                                    : launch_partial_kvb<128, false>(pool, p, grid, smem, st);
                if (rc != BRC_OK) return rc;
            }
        }
    }
    return note_decode_issued(pool, st, capturing);
}

uint32_t brc_decode_kvb(const brc_pool *pool) { return kvb_of(pool); }

namespace {

brc_layers_args one_layer(uint32_t layer, const void *q, int32_t q_dtype, uint32_t n_head, const float *gate, uint32_t gate_head_stride,
                          const uint32_t *bt, uint32_t table_stride, const uint32_t *lens, uint32_t n_seqs, uint32_t max_seq_len,
                          float scale, float *out, void *ws, uint64_t ws_bytes) {
    brc_layers_args a;
    a.layer0 = layer;
    a.n_layers = 1;
    a.q = q;
    a.q_dtype = q_dtype;
    a.n_head = n_head;
    a.gate = gate;
    a.gate_head_stride = gate_head_stride;
    a.block_tables = bt;
    a.table_stride = table_stride;
    a.seq_lens = lens;
    a.n_seqs = n_seqs;
    a.max_seq_len = max_seq_len;
    a.scale = scale;
    a.out = out;
    a.workspace = ws;
    a.workspace_bytes = ws_bytes;
    return a;
}

}  // namespace

extern "C" {

brc_status brc_decode_share_rates(const brc_pool *pool, float *rates, uint32_t capacity, uint32_t *out_n) {
    if (!pool || !out_n || (!rates && capacity)) return brc_fail(BRC_ERR_INVALID, "brc_decode_share_rates: NULL argument");
    const uint32_t n = pool->cut_prefix ? (uint32_t)pool->cut_rates.size() : 0u;
    if (n > capacity) return brc_fail(BRC_ERR_CAPACITY, "brc_decode_share_rates: %u rates, room for %u", n, capacity);
    for (uint32_t i = 0; i < n; ++i) rates[i] = pool->cut_rates[i];
    *out_n = n;
    return BRC_OK;
}

brc_status brc_decode_workspace_bytes(const brc_pool *pool, uint32_t n_seqs, uint32_t n_head, uint64_t *out_bytes) {
    if (!pool || !out_bytes) return brc_fail(BRC_ERR_INVALID, "brc_decode_workspace_bytes: NULL argument");
    (void)n_head;
    *out_bytes = slots_for(pool, n_seqs) * slot_floats(pool) * sizeof(float);
    return BRC_OK;
}

brc_status brc_paged_decode_attn(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype, uint32_t n_head,
                                 const float *gate_dev, uint32_t gate_head_stride, const uint32_t *block_tables_dev,
                                 uint32_t table_stride, const uint32_t *seq_lens_dev, uint32_t n_seqs,
                                 uint32_t max_seq_len, float scale, float *out_dev, void *workspace_dev,
                                 uint64_t workspace_bytes, void *stream) {
    return brc_decode_layers(pool, "brc_paged_decode_attn",
                             one_layer(layer, q_dev, q_dtype, n_head, gate_dev, gate_head_stride, block_tables_dev, table_stride,
                                       seq_lens_dev, n_seqs, max_seq_len, scale, out_dev, workspace_dev, workspace_bytes),
                             stream);
}

brc_status brc_decode_partial_bytes(uint32_t n_seqs, uint32_t n_head, uint32_t head_dim, uint64_t *out_bytes) {
    if (!out_bytes) return brc_fail(BRC_ERR_INVALID, "brc_decode_partial_bytes: NULL argument");
    *out_bytes = (uint64_t)n_seqs * n_head * ((uint64_t)head_dim + 2u) * sizeof(float);
    return BRC_OK;
}

brc_status brc_decode_partial(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype, uint32_t n_head,
                              const uint32_t *block_tables_dev, uint32_t table_stride, const uint32_t *seq_lens_dev,
                              uint32_t n_seqs, uint32_t max_seq_len, float scale, void *partial_dev, void *workspace_dev,
                              uint64_t workspace_bytes, void *stream) {
    brc_layers_args a = one_layer(layer, q_dev, q_dtype, n_head, nullptr, 0, block_tables_dev, table_stride, seq_lens_dev, n_seqs,
                                  max_seq_len, scale, static_cast<float *>(partial_dev), workspace_dev, workspace_bytes);
    if (pool && partial_dev) a.out_ml = static_cast<float *>(partial_dev) + (size_t)n_seqs * n_head * pool->head_dim;
    return brc_decode_layers(pool, "brc_decode_partial", a, stream);
}

brc_status brc_decode_combine(int32_t device, const void *parts_dev, uint32_t n_parts, uint64_t part_stride_bytes,
                              uint32_t n_seqs, uint32_t n_head, uint32_t head_dim, const float *gate_dev,
                              uint32_t gate_head_stride, float *out_dev, void *stream) {
    if (!parts_dev || !out_dev) return brc_fail(BRC_ERR_INVALID, "brc_decode_combine: NULL pointer");
    if (head_dim != 256 && head_dim != 128)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_decode_combine: head_dim %u (kernels are built for 128 and 256)", head_dim);
    uint64_t need = 0;
    brc_decode_partial_bytes(n_seqs, n_head, head_dim, &need);
    if (n_parts == 0 || (n_parts > 1 && part_stride_bytes < need) || (part_stride_bytes & 15u))
        return brc_fail(BRC_ERR_INVALID, "brc_decode_combine: %u parts laid %llu bytes apart, each needs %llu (16-byte multiple)",
                        n_parts, (unsigned long long)part_stride_bytes, (unsigned long long)need);
    if (gate_dev && gate_head_stride < head_dim)
        return brc_fail(BRC_ERR_INVALID, "brc_decode_combine: gate_head_stride %u < head_dim %u", gate_head_stride, head_dim);
    if (n_seqs == 0 || n_head == 0) return BRC_OK;
    brc_device_guard guard(device);
    if (!guard.ok) return brc_fail(BRC_ERR_CUDA, "brc_decode_combine: cannot make device %d current", device);
    const uint32_t rows = n_seqs * n_head;
    if (head_dim == 256)
        parts_combine_kernel<256><<<rows, 256, 0, brc_stream(stream)>>>(static_cast<const uint8_t *>(parts_dev), n_parts,
                                                                       part_stride_bytes, rows, gate_dev, gate_head_stride, out_dev);
    else
        parts_combine_kernel<128><<<rows, 128, 0, brc_stream(stream)>>>(static_cast<const uint8_t *>(parts_dev), n_parts,
                                                                       part_stride_bytes, rows, gate_dev, gate_head_stride, out_dev);
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Two kinds of caller are meant.  An engine that handed its whole HBM budget to its own arena at
// start-up has nothing left for a later cudaMalloc, and must not fragment what it planned.  And a
// latency-critical decode loop cannot afford cudaMalloc at all: the call synchronises the device, so
// every stream would stall behind it.  For them the split-KV partials live in the array below, which
// is part of the library image: every GPU that loads the library holds BRC_STATIC_WS_BYTES of it
// until the process exits, whether or not this entry point is ever called.  Nothing in the array has
// to start at any value: every partial is written before it is read.
// ---------------------------------------------------------------------------------------------
#define BRC_STATIC_WS_BYTES (4u << 20)

static __device__ __align__(256) unsigned char g_static_decode_ws[BRC_STATIC_WS_BYTES];

namespace {

// In host code the array's name is only a handle for the runtime, not a device address; the address
// is asked for once per device, with that device current, and kept.
std::mutex g_static_ws_mu;
void *g_static_ws_ptr[64] = {};

brc_status static_ws_for(int device, void **out) {
    if (device < 0 || device >= 64) return brc_fail(BRC_ERR_INVALID, "static decode scratch: device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_static_ws_mu);
    if (!g_static_ws_ptr[device]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_decode_ws);
        if (e != cudaSuccess || !ptr)
            return brc_fail(BRC_ERR_CUDA, "static decode scratch: cudaGetSymbolAddress on device %d failed: %s", device,
                            cudaGetErrorString(e));
        g_static_ws_ptr[device] = ptr;
    }
    *out = g_static_ws_ptr[device];
    return BRC_OK;
}

}  // namespace

extern "C" {

brc_status brc_paged_decode_attn_static(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype, uint32_t n_head,
                                        const float *gate_dev, uint32_t gate_head_stride,
                                        const uint32_t *block_tables_dev, uint32_t table_stride,
                                        const uint32_t *seq_lens_dev, uint32_t n_seqs, uint32_t max_seq_len, float scale,
                                        float *out_dev, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_paged_decode_attn_static: pool is NULL");
    if (pool->device < 0 || !pool->has_tma)
        return brc_fail(BRC_ERR_CUDA, "brc_paged_decode_attn_static: this pool holds bookkeeping only (no device memory)");
    uint64_t need = 0;
    brc_decode_workspace_bytes(pool, n_seqs, n_head, &need);
    if (need > BRC_STATIC_WS_BYTES) {
        const uint64_t per_slot = (uint64_t)GROUP_TILE * (pool->head_dim + 2u) * sizeof(float);
        const uint64_t slots = BRC_STATIC_WS_BYTES / per_slot;
        const uint64_t fixed = (uint64_t)grid_ctas(pool) * kvb_of(pool);
        return brc_fail(BRC_ERR_CAPACITY,
                        "brc_paged_decode_attn_static: %u sequences need %llu bytes of scratch but the built-in array holds %u "
                        "(room for about %llu sequences with this pool); use brc_paged_decode_attn with a caller-owned workspace",
                        n_seqs, (unsigned long long)need, BRC_STATIC_WS_BYTES,
                        (unsigned long long)(slots > fixed ? (slots - fixed) / pool->n_kv_head : 0));
    }
    void *ws = nullptr;
    {
        brc_device_guard guard(pool->device);
        if (!guard.ok) return brc_fail(BRC_ERR_CUDA, "brc_paged_decode_attn_static: cannot make device %d current", pool->device);
        if (brc_status rc = static_ws_for(pool->device, &ws)) return rc;
    }
    return brc_decode_layers(pool, "brc_paged_decode_attn_static",
                             one_layer(layer, q_dev, q_dtype, n_head, gate_dev, gate_head_stride, block_tables_dev, table_stride,
                                       seq_lens_dev, n_seqs, max_seq_len, scale, out_dev, ws, BRC_STATIC_WS_BYTES),
                             stream);
}

}  // extern "C"
