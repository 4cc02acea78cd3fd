// Chunked-prefill attention over a paged prefix on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Replaces the reference's T >= 16 path: qsa_attn_scores_gqa.comp + ops_softmax.comp +
// qsa_attn_apply_gqa.comp driven tile by tile from Qsa::forward
// (crates/breccia-kernels/src/qsa/mod.rs:1631-1641), i.e. one workgroup per (token, kv head) doing
// CUDA-core style dot products.  Semantics kept: all cells of the chunk are in the cache before any
// row attends; row t (position pos0 + t) sees cells <= pos0 + t; kv head = h * n_kv / n_head; f16 K/V,
// fp32 accumulation; gate optional (sigmoid, applied last).
//
// One CTA = one (sequence, kv head, 16 query tokens): a 128-row tile, row = token * 8 + query head of
// the group (GQA: the 8 query heads of a kv head share every K/V byte the CTA stages).  More than 8 query
// heads per kv head (the reference model has 12, shaders/qsa_attn_scores_gqa.comp:51-133 hard-codes GROUP 12)
// take `group` rows per token and floor(128 / group) tokens per tile: 10 tokens x 12 heads = 120 of the 128 rows.
// Per block of
// 64 cells (4 pages):
//   S[128 x 64]  = Q[128 x 256] . K^T      tcgen05.mma kind::f16, M=128 N=64, 16 steps of K=16, fp32 in TMEM
//   P            = 2^(scale' S - m)        4 softmax warps, one thread per row, tcgen05.ld; causal mask
//   O[128 x 256] += P[128 x 64] . V        tcgen05.mma M=128 N=256, 4 steps of K=16, V read MN-major
// Q and P are A operands read from tensor memory (Q is stored there once; P overwrites the S buffer it
// was computed from), so shared memory holds only K and V tiles, in the canonical 128-byte-swizzled
// layouts the matrix descriptors name: with A in shared memory every S MMA re-read 4 KiB of Q for 2 KiB
// of K, and the kernel ran at the shared-memory bandwidth, not at the tensor pipe's.  K/V pages are gathered through the block table by four loader warps with 16-byte cp.async
// (a 16-cell page is too small a TMA box: ~215 cycles per operation whatever its size), K and V in
// separate three-deep rings; cells at or past the end of the cache are zero-filled.  S and P are double
// buffered: the MMA thread issues S of block j + 1 before P.V of block j, so the tensor pipe computes
// the next scores while the softmax warps work on the current ones.  O stays in TMEM across blocks and is
// rescaled only when a row's maximum grew by more than 2^8 since the scale in use (rare after the
// first blocks), so P may exceed 1 by at most that factor — harmless in binary16 with fp32 sums.
// Every wait is bounded; TMEM is released on every path.
#include <algorithm>

#include "brc_device.cuh"
#include "brc_internal.h"

namespace {

constexpr int PF_HD = 256;
constexpr int PF_ROWS = 128;              // 16 tokens x 8 head slots
constexpr int PF_BLK = 64;                // cells per block
constexpr int PF_STAGES = 3;               // depth of the K ring and of the V ring
constexpr int PF_SOFTMAX_WARPS = 4;       // warps 0-3: TMEM lane quarter = warp id
constexpr int PF_MMA_WARP = 4;
constexpr int PF_LOAD_WARP0 = 5;          // warps 5-8
constexpr int PF_LOAD_WARPS = 4;
constexpr int PF_THREADS = (PF_SOFTMAX_WARPS + 1 + PF_LOAD_WARPS) * 32;
constexpr uint32_t PF_Q_BYTES = PF_ROWS * PF_HD * 2;      // 64 KiB: 4 slabs [128 rows][128 B]
constexpr uint32_t PF_Q_SLAB = PF_ROWS * 128;
constexpr uint32_t PF_KV_SLAB = PF_BLK * 128;             // [64 cells][128 B]
constexpr uint32_t PF_K_BYTES = 4 * PF_KV_SLAB;           // 32 KiB
constexpr uint32_t PF_STAGE_BYTES = 2 * PF_K_BYTES;       // K then V
constexpr uint32_t PF_P_BYTES = PF_ROWS * 128;            // [128 rows][64 cells] f16
constexpr uint32_t PF_SMEM = 1024 + PF_STAGES * PF_STAGE_BYTES + 1024;
constexpr uint32_t PF_TMEM_COLS = 512;
// Tensor memory: Q (128 rows x 256 binary16 = 128 columns), O (256 columns, fp32), two S buffers of 64 columns
// (fp32) whose first 32 columns are overwritten by P (binary16 pairs).
constexpr uint32_t PF_Q_COL = 0, PF_O_COL = 128, PF_S0_COL = 384, PF_S1_COL = 448;
constexpr uint64_t PF_WAIT_NS = 1000000000ull;
constexpr float PF_RESCALE_THRESHOLD = 8.0f;              // log2 units

struct PrefillParams {
    const void *q;                 // [n_seqs][chunk][n_head][256], f16 or f32
    const uint8_t *k_layer;        // this layer's K pool
    const uint8_t *v_layer;
    const uint32_t *block_tables;  // [n_seqs][table_stride]
    const uint32_t *pos0;          // [n_seqs]
    const float *gate;             // nullable, [n_seqs][chunk][n_head][..] with gate_head_stride
    float *out;                    // [n_seqs][chunk][n_head][256] f32
    uint32_t *status;
    uint32_t n_seqs, chunk, table_stride, max_pos_end;
    uint32_t n_kv_head, group, n_head, n_pages, q_f32, gate_head_stride;
    uint32_t head_slots;           // rows per token in a tile: 8, or the group when it is larger
    uint32_t tile_tokens;          // tokens per tile: 128 / head_slots
    uint32_t v_q8;                 // the pool stores V as q8_0 blocks (one f32 scale + 32 signed bytes per 32 values)
    float scale_log2;
};

__device__ __forceinline__ uint64_t pf_globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity) {
    if (brc::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = pf_globaltimer();
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        if (brc::mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && pf_globaltimer() - t0 > PF_WAIT_NS) return false;
    }
    return false;
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// K-major operands: rows 128 B apart inside an 8-row group, groups `sbo` bytes apart (lbo unused = 1).
// MN-major operands: 64 contiguous elements per 128-byte row, 64-element groups `lbo` bytes apart,
// 8-row (K) groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;   // version
    d |= (uint64_t)2 << 61;   // SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16: D = f32, A = B = f16, M = 128.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t n, bool b_mn_major) {
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same with the A operand in tensor memory (row = lane, two binary16 per 32-bit column cell).
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One lane of the (converged) warp, the same one every time.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
          "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
          "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
          "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
    float a[32], b[32];
    tmem_ld32(taddr, a);
    tmem_ld32(taddr + 32, b);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = a[i];
        v[32 + i] = b[i];
    }
}

// 16-byte async copy; src_bytes = 0 writes zeros.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float pf_sigmoid(float x) {
    if (x >= 0.f) return 1.f / (1.f + expf(-x));
    const float e = expf(x);
    return e / (1.f + e);
}

__global__ void __launch_bounds__(PF_THREADS, 1) prefill_attn_kernel(const PrefillParams p) {
    extern __shared__ uint8_t pf_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023u) & ~uintptr_t(1023));
    uint8_t *k_sm0 = smem;                                   // [PF_STAGES][32 KiB]
    uint8_t *v_sm0 = k_sm0 + PF_STAGES * PF_K_BYTES;         // [PF_STAGES][32 KiB]
    uint64_t *bars = reinterpret_cast<uint64_t *>(v_sm0 + PF_STAGES * PF_K_BYTES);
    const uint32_t bar_kfull = brc::smem_u32(bars);          // [PF_STAGES] loaders -> MMA
    const uint32_t bar_vfull = bar_kfull + 8u * PF_STAGES;   // [PF_STAGES]
    const uint32_t bar_kempty = bar_vfull + 8u * PF_STAGES;  // [PF_STAGES] S MMAs of the stage retired
    const uint32_t bar_vempty = bar_kempty + 8u * PF_STAGES; // [PF_STAGES] P.V MMAs of the stage retired
    const uint32_t bar_s = bar_vempty + 8u * PF_STAGES;      // [2] S buffer written
    const uint32_t bar_p = bar_s + 16u;                      // [2] P written over the S buffer
    const uint32_t bar_o = bar_p + 16u;                      // [2] P.V of the block retired
    const uint32_t bar_q = bar_o + 16u;                      // Q is in tensor memory
    volatile uint32_t *misc = reinterpret_cast<volatile uint32_t *>(bars + 32);   // [0] tmem base, [1] dead

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t kvh = blockIdx.x % p.n_kv_head;
    const uint32_t tile = blockIdx.x / p.n_kv_head;
    const uint32_t s = blockIdx.y;
    const uint32_t t0 = tile * p.tile_tokens;
    const uint32_t pos0 = p.pos0[s];
    const uint32_t kv_len = pos0 + p.chunk;                    // cells in the cache (all of the chunk is appended)
    if (kv_len > p.max_pos_end) {
        if (tid == 0) { atomicOr(p.status, BRC_DEV_BAD_POS); p.status[1] = kv_len; }
        return;
    }
    const uint32_t n_tok = min(p.tile_tokens, p.chunk - t0);
    const uint32_t cells_needed = pos0 + t0 + n_tok;           // the tile's last row sees cells < this
    const uint32_t n_blk = (cells_needed + PF_BLK - 1) / PF_BLK;

    if (tid == 0) {
        for (uint32_t i = 0; i < PF_STAGES; ++i) {
            brc::mbar_init(bar_kfull + 8u * i, PF_LOAD_WARPS * 32);
            brc::mbar_init(bar_vfull + 8u * i, PF_LOAD_WARPS * 32);
            brc::mbar_init(bar_kempty + 8u * i, 1);
            brc::mbar_init(bar_vempty + 8u * i, 1);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            brc::mbar_init(bar_s + 8u * i, 1);
            brc::mbar_init(bar_p + 8u * i, PF_SOFTMAX_WARPS * 32);
            brc::mbar_init(bar_o + 8u * i, 1);
        }
        brc::mbar_init(bar_q, PF_SOFTMAX_WARPS * 32);
        brc::mbar_fence_init();
        misc[1] = 0u;
    }
    if (warp == PF_MMA_WARP) {   // one warp owns the TMEM allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(brc::smem_u32(const_cast<uint32_t *>(misc))),
                     "r"(PF_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];

    if (warp >= PF_LOAD_WARP0) {
        // ------------------------------------------------------------------ loader warps
        // K and V of a block go into rings of their own (PF_STAGES deep): the K stage is free again when
        // the S MMAs of block j retire, long before the block's V stage is.  The copies write shared
        // memory through the generic proxy; the MMA thread orders them before its (async-proxy) operand
        // reads with a proxy fence after it has seen the stage's barrier complete.
        // Thread -> (row r0 + 4 i, 16-byte chunk ch) of the [64 cells][512 B] tile, i < 16; the rows of a
        // thread walk through the block's 4 pages, 4 rows per page.
        const uint32_t lt = tid - PF_LOAD_WARP0 * 32;   // 0..127
        const uint32_t *table = p.block_tables + (uint64_t)s * p.table_stride;
        const uint32_t ch = lt & 31u, r0 = lt >> 5;
        bool dead = false;
        uint32_t stg = 0, par = 1;                      // stage j % PF_STAGES, parity of its "empty" phase
        for (uint32_t j = 0; j < n_blk && !dead; ++j) {
            uint32_t page[4];
#pragma unroll
            for (uint32_t g = 0; g < 4; ++g) {
                const uint32_t cell = j * PF_BLK + g * 16u;
                page[g] = 0;
                if (cell < kv_len) {
                    page[g] = __ldg(table + (cell >> 4));
                    if (page[g] >= p.n_pages) {
                        atomicOr(p.status, BRC_DEV_BAD_PAGE);
                        p.status[1] = page[g];
                        page[g] = 0;
                    }
                }
            }
#pragma unroll
            for (uint32_t kv = 0; kv < 2; ++kv) {
                if (!pf_wait((kv ? bar_vempty : bar_kempty) + 8u * stg, par) || misc[1]) {
                    dead = true;
                    break;
                }
                const uint32_t dst0 = brc::smem_u32(kv ? v_sm0 : k_sm0) + stg * PF_K_BYTES;
                const uint8_t *base = kv ? p.v_layer : p.k_layer;
                if (kv && p.v_q8) {
                    // q8_0 V (crates/breccia-kernels/src/qsa/mod.rs:325-349; read rule shaders/qsa_attn_apply.comp:60-77):
                    // the thread's eight values of a row are a quarter of one 36-byte block; scale x quantum in fp32,
                    // rounded to the binary16 the tile holds (the tensor cores take binary16 V: the rounding, 2^-11
                    // relative, is inside this path's tolerance).  Loads first, all sixteen rows in flight, then the
                    // conversions and plain shared-memory stores, then an ordinary arrival on the stage's barrier.
                    uint32_t sc[16], qa[16], qb[16];
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const uint32_t r = r0 + 4u * i;
                        const uint32_t cell = j * PF_BLK + r;
                        sc[i] = qa[i] = qb[i] = 0u;
                        if (cell < kv_len) {
                            const uint32_t *blk = reinterpret_cast<const uint32_t *>(base) +
                                                  ((((uint64_t)page[i >> 2] * p.n_kv_head + kvh) * 16u + (r & 15u)) * (PF_HD / 32u) + (ch >> 2)) * 9u;
                            sc[i] = __ldg(blk);
                            qa[i] = __ldg(blk + 1u + 2u * (ch & 3u));
                            qb[i] = __ldg(blk + 2u + 2u * (ch & 3u));
                        }
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const uint32_t r = r0 + 4u * i;
                        const uint32_t off = (ch >> 3) * PF_KV_SLAB + r * 128u + (((ch & 7u) ^ (r & 7u)) << 4);
                        const float d = __uint_as_float(sc[i]);
                        auto v = [d](uint32_t w, int b) { return d * (float)(int)(int8_t)(w >> (8 * b)); };
                        const uint32_t w0 = brc::pack_half2(v(qa[i], 0), v(qa[i], 1)), w1 = brc::pack_half2(v(qa[i], 2), v(qa[i], 3));
                        const uint32_t w2 = brc::pack_half2(v(qb[i], 0), v(qb[i], 1)), w3 = brc::pack_half2(v(qb[i], 2), v(qb[i], 3));
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst0 + off), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                    }
                    brc::mbar_arrive(bar_vfull + 8u * stg);
                    continue;
                }
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) {
                    const uint32_t r = r0 + 4u * i;
                    const uint32_t cell = j * PF_BLK + r;
                    const bool live = cell < kv_len;   // past the end of the cache: zeros
                    const uint64_t src = (((uint64_t)page[i >> 2] * p.n_kv_head + kvh) * 16u + (r & 15u)) * (PF_HD * 2u) + ch * 16u;
                    const uint32_t off = (ch >> 3) * PF_KV_SLAB + r * 128u + (((ch & 7u) ^ (r & 7u)) << 4);
                    cp_async16(dst0 + off, base + src, live ? 16u : 0u);
                }
                // The arrival is carried by the copies themselves: it fires when all of this thread's copies
                // issued so far have landed, so the loader never waits for data, only for a free stage.
                cp_async_arrive_noinc((kv ? bar_vfull : bar_kfull) + 8u * stg);
            }
            if (++stg == PF_STAGES) { stg = 0; par ^= 1u; }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        if (dead) {
            if (!misc[1] && lt == 0) { atomicOr(p.status, BRC_DEV_WAIT_LIMIT); p.status[1] = 3000000u + blockIdx.x; }
            misc[1] = 1u;
        }
    } else if (warp == PF_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        // Both A operands come from tensor memory (Q, written once by the softmax warps; P, written over
        // the S buffer it was computed from), so shared memory only serves the K and V tiles.
        // S of block j + 1 is issued before P.V of block j: the tensor pipe works on the next scores while
        // the softmax warps turn the current ones into P, and on P.V while they read the next scores.
        // The whole warp runs the loop (waits, descriptor arithmetic: warp-uniform, so it stays on the
        // uniform datapath); one elected lane issues the MMAs and commits.
        const bool leader = elect_one();
        const uint32_t idesc_s = umma_idesc(PF_BLK, false);
        const uint32_t idesc_o = umma_idesc(PF_HD, true);
        const uint32_t k_base = brc::smem_u32(k_sm0), v_base = brc::smem_u32(v_sm0);
        bool ok = __all_sync(0xffffffffu, pf_wait(bar_q, 0));
        tc_fence_after();
        auto issue_s = [&](uint32_t j) -> bool {
            const uint32_t stg = j % PF_STAGES, buf = j & 1u;
            if (!__all_sync(0xffffffffu, pf_wait(bar_kfull + 8u * stg, (j / PF_STAGES) & 1u))) return false;
            brc::fence_proxy_async_smem();
            tc_fence_after();
            const uint32_t k_sm = k_base + stg * PF_K_BYTES;
            const uint32_t s_tm = tmem + (buf ? PF_S1_COL : PF_S0_COL);
            if (leader) {
                // S = Q . K^T: 16 steps of K = 16: 8 columns of Q in tensor memory (two binary16 per
                // 32-bit cell), 32 bytes inside a 128-byte swizzled row of K (4 steps per slab)
#pragma unroll
                for (uint32_t ks = 0; ks < PF_HD / 16; ++ks) {
                    const uint64_t b = umma_desc(k_sm + (ks >> 2) * PF_KV_SLAB + (ks & 3u) * 32u, 16, 1024);
                    umma_f16_ts(s_tm, tmem + PF_Q_COL + ks * 8u, b, idesc_s, ks > 0);
                }
                umma_commit(bar_s + 8u * buf);
                umma_commit(bar_kempty + 8u * stg);
            }
            __syncwarp();
            return true;
        };
        if (ok && n_blk > 0) ok = issue_s(0);
        for (uint32_t j = 0; j < n_blk && ok; ++j) {
            if (__any_sync(0xffffffffu, misc[1] != 0u)) break;
            const uint32_t stg = j % PF_STAGES, buf = j & 1u;
            // The S buffer of block j + 1 held P of block j - 1, whose P.V was issued before this
            // point: the tensor pipe runs in issue order.
            if (j + 1 < n_blk) {
                ok = issue_s(j + 1);
                if (!ok) break;
            }
            ok = __all_sync(0xffffffffu, pf_wait(bar_p + 8u * buf, (j >> 1) & 1u) && pf_wait(bar_vfull + 8u * stg, (j / PF_STAGES) & 1u));
            if (!ok) break;
            brc::fence_proxy_async_smem();
            tc_fence_after();
            const uint32_t v_sm = v_base + stg * PF_K_BYTES;
            const uint32_t p_tm = tmem + (buf ? PF_S1_COL : PF_S0_COL);
            if (leader) {
                // O += P . V: 4 steps of K = 16 cells: 8 columns of P in tensor memory; V is MN-major:
                // 16 cells = 2048 bytes down a slab, the four 64-column slabs are 8 KiB apart (leading
                // offset), 8-cell groups 1 KiB apart
#pragma unroll
                for (uint32_t ks = 0; ks < PF_BLK / 16; ++ks) {
                    const uint64_t b = umma_desc(v_sm + ks * 2048u, PF_KV_SLAB, 1024);
                    umma_f16_ts(tmem + PF_O_COL, p_tm + ks * 8u, b, idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(bar_o + 8u * buf);
                umma_commit(bar_vempty + 8u * stg);
            }
            __syncwarp();
        }
        if (!ok) {
            if (!misc[1] && lane == 0) { atomicOr(p.status, BRC_DEV_WAIT_LIMIT); p.status[1] = 4000000u + blockIdx.x; }
            misc[1] = 1u;
        }
    } else {
        // ------------------------------------------------------------------ softmax warps: thread = row
        const uint32_t row = tid;                       // TMEM lane
        const uint32_t tl = row / p.head_slots, h = row - tl * p.head_slots;
        const uint32_t limit = pos0 + t0 + tl;          // last cell this row sees
        const uint32_t lane_base = (warp * 32u) << 16;  // this warp's TMEM lane quarter
        const bool live_row = tl < n_tok && h < p.group;
        // Q row (token t0 + tl, query head h of the group) into tensor memory: two binary16 per 32-bit
        // cell, 128 cells; rows outside the tile are zero.
        {
            const uint64_t qrow = ((uint64_t)(s * p.chunk + t0 + (live_row ? tl : 0)) * p.n_head + kvh * p.group + (live_row ? h : 0)) * PF_HD;
#pragma unroll 1
            for (uint32_t c = 0; c < 4; ++c) {          // 64 elements = 32 cells per pass
                uint32_t w[32];
                if (!p.q_f32) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(p.q) + qrow + c * 64u);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint4 x = live_row ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
                        w[i * 4] = x.x, w[i * 4 + 1] = x.y, w[i * 4 + 2] = x.z, w[i * 4 + 3] = x.w;
                    }
                } else {
                    const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(p.q) + qrow + c * 64u);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float4 x = live_row ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                        w[i * 2] = brc::pack_half2(x.x, x.y), w[i * 2 + 1] = brc::pack_half2(x.z, x.w);
                    }
                }
                tmem_st32u(tmem + lane_base + PF_Q_COL + c * 32u, w);
            }
            tc_fence_before();
            brc::mbar_arrive(bar_q);
        }
        float m_used = -INFINITY, l = 0.f;              // m_used in units of scale_log2 * score
        bool ok = true;
        for (uint32_t j = 0; j < n_blk; ++j) {
            const uint32_t buf = j & 1u, par = (j >> 1) & 1u;
            const uint32_t s_col = buf ? PF_S1_COL : PF_S0_COL;
            // warp-uniform control flow: the TMEM accesses below are warp-wide
            if (__any_sync(0xffffffffu, misc[1] != 0u)) { ok = true; break; }
            ok = __all_sync(0xffffffffu, pf_wait(bar_s + 8u * buf, par));
            if (!ok) break;
            tc_fence_after();
            float sc[PF_BLK];
            tmem_ld64(tmem + lane_base + s_col, sc);
            const uint32_t c0 = j * PF_BLK;
            if (c0 + PF_BLK - 1 > limit) {
#pragma unroll
                for (int i = 0; i < PF_BLK; ++i)
                    if (c0 + i > limit) sc[i] = -INFINITY;
            }
            // eight independent chains: a single chain of 64 dependent maxima costs more than the exponentials
            float mx8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = sc[i];
#pragma unroll
            for (int i = 8; i < PF_BLK; ++i) mx8[i & 7] = fmaxf(mx8[i & 7], sc[i]);
            float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            mx *= p.scale_log2;   // the scale is positive: max commutes with it
            // Raise the scale in use when this row's maximum grew a lot (or at its first live block):
            // O *= 2^(old - new).  TMEM loads and stores are warp-wide, so the warp goes through the
            // rescale together and rows that need none multiply by one.
            const bool raise = mx > m_used + PF_RESCALE_THRESHOLD;
            float f = 1.f;
            if (raise) {
                if (m_used != -INFINITY) f = brc::fast_exp2(m_used - mx);
                l *= f;
                m_used = mx;
            }
            if (j > 0 && __any_sync(0xffffffffu, f != 1.f)) {
                // O is about to change: P.V of the block before this one must have retired
                ok = __all_sync(0xffffffffu, pf_wait(bar_o + 8u * ((j - 1) & 1u), ((j - 1) >> 1) & 1u));
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int cg = 0; cg < PF_HD / 32; ++cg) {
                    float v[32];
                    tmem_ld32(tmem + lane_base + PF_O_COL + cg * 32, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= f;
                    tmem_st32(tmem + lane_base + PF_O_COL + cg * 32, v);
                }
            }
            // P row (binary16, two cells per 32-bit cell) over the first 32 columns of the S buffer it came
            // from: S of block j is in registers, and the buffer's previous P (block j - 2) was consumed
            // before the MMAs that wrote this S (the tensor pipe runs in issue order).
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;   // a row with no live cell yet has only -inf scores
            uint32_t w[32];
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float a = brc::fast_exp2(fmaf(sc[2 * i], p.scale_log2, neg_m));
                const float b = brc::fast_exp2(fmaf(sc[2 * i + 1], p.scale_log2, neg_m));
                l4[i & 3] += a + b;
                w[i] = brc::pack_half2(a, b);
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tmem_st32u(tmem + lane_base + s_col, w);
            tc_fence_before();
            brc::mbar_arrive(bar_p + 8u * buf);
        }
        if (ok && n_blk > 0 && !__any_sync(0xffffffffu, misc[1] != 0u)) {
            ok = __all_sync(0xffffffffu, pf_wait(bar_o + 8u * ((n_blk - 1) & 1u), ((n_blk - 1) >> 1) & 1u));
            if (ok) {
                tc_fence_after();
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const uint64_t orow = ((uint64_t)(s * p.chunk + t0 + tl) * p.n_head + kvh * p.group + h);
#pragma unroll 1
                for (int cg = 0; cg < PF_HD / 32; ++cg) {
                    float v[32];
                    tmem_ld32(tmem + lane_base + PF_O_COL + cg * 32, v);
                    if (live_row) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float4 r = make_float4(v[i] * inv, v[i + 1] * inv, v[i + 2] * inv, v[i + 3] * inv);
                            if (p.gate) {
                                const float *g = p.gate + orow * p.gate_head_stride + cg * 32 + i;
                                r.x *= pf_sigmoid(g[0]);
                                r.y *= pf_sigmoid(g[1]);
                                r.z *= pf_sigmoid(g[2]);
                                r.w *= pf_sigmoid(g[3]);
                            }
                            *reinterpret_cast<float4 *>(p.out + orow * PF_HD + cg * 32 + i) = r;
                        }
                    }
                }
            }
        }
        if (!ok) {
            if (!misc[1] && lane == 0) { atomicOr(p.status, BRC_DEV_WAIT_LIMIT); p.status[1] = 5000000u + blockIdx.x; }
            misc[1] = 1u;
        }
    }
    // everyone is done with TMEM (or has given up): release it
    tc_fence_before();
    __syncthreads();
    if (warp == PF_MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(PF_TMEM_COLS) : "memory");
    }
}


}  // namespace

extern "C" {

brc_status brc_paged_prefill_attn(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype, uint32_t n_head,
                                  const float *gate_dev, uint32_t gate_head_stride, const uint32_t *block_tables_dev,
                                  uint32_t table_stride, const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t chunk_len,
                                  uint32_t max_pos_end, float scale, float *out_dev, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: pool is NULL");
    if (pool->device < 0 || !pool->k_base)
        return brc_fail(BRC_ERR_CUDA, "brc_paged_prefill_attn: this pool holds bookkeeping only (no device memory)");
    if (layer >= pool->n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: layer %u but the pool has %u", layer, pool->n_layers);
    if (pool->head_dim != PF_HD)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_paged_prefill_attn: head_dim %u (the tensor-core prefill path is built for %d)",
                        pool->head_dim, PF_HD);
    if (q_dtype != BRC_DTYPE_F32 && q_dtype != BRC_DTYPE_F16)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: q_dtype %d is neither f32 (0) nor f16 (1)", q_dtype);
    if (n_head == 0 || n_head % pool->n_kv_head != 0)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: %u query heads do not divide over %u kv heads", n_head,
                        pool->n_kv_head);
    if (n_head / pool->n_kv_head > 32)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_paged_prefill_attn: %u query heads per kv head (a tile holds up to 32)",
                        n_head / pool->n_kv_head);
    const uint64_t capacity = (uint64_t)table_stride * pool->page_tokens;
    if (max_pos_end > capacity)
        return brc_fail(BRC_ERR_CAPACITY,
                        "brc_paged_prefill_attn would read cells up to %u but each block table holds %llu (%u pages of %u cells)",
                        max_pos_end, (unsigned long long)capacity, table_stride, pool->page_tokens);
    if (gate_dev && gate_head_stride < pool->head_dim)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: gate_head_stride %u < head_dim %u", gate_head_stride, pool->head_dim);
    if (n_seqs == 0 || chunk_len == 0) return BRC_OK;
    if (!q_dev || !block_tables_dev || !pos0_dev || !out_dev)
        return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: NULL query, block table, position or output pointer");
    if ((reinterpret_cast<uintptr_t>(q_dev) & 15u) || (reinterpret_cast<uintptr_t>(out_dev) & 15u))
        return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: query and output pointers must be 16-byte aligned");
    if (n_seqs > 65535u) return brc_fail(BRC_ERR_INVALID, "brc_paged_prefill_attn: %u sequences in one call (limit 65535)", n_seqs);
    brc_device_guard guard(pool->device);
    static bool configured[64] = {};
    if (pool->device < 64 && !configured[pool->device]) {
        BRC_CUDA(cudaFuncSetAttribute(prefill_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
        configured[pool->device] = true;
    }
    PrefillParams p;
    p.q = q_dev;
    p.k_layer = pool->k_base + (uint64_t)layer * pool->layer_bytes;
    p.v_layer = pool->v_base + (uint64_t)layer * pool->v_layer_bytes;
    p.v_q8 = pool->v_q8 ? 1u : 0u;
    p.block_tables = block_tables_dev;
    p.pos0 = pos0_dev;
    p.gate = gate_dev;
    p.out = out_dev;
    p.status = pool->status_dev;
    p.n_seqs = n_seqs;
    p.chunk = chunk_len;
    p.table_stride = table_stride;
    p.max_pos_end = max_pos_end;
    p.n_kv_head = pool->n_kv_head;
    p.group = n_head / pool->n_kv_head;
    p.n_head = n_head;
    p.n_pages = pool->n_pages;
    p.q_f32 = q_dtype == BRC_DTYPE_F32;
    p.gate_head_stride = gate_head_stride;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.head_slots = std::max<uint32_t>(p.group, 8u);
    p.tile_tokens = (uint32_t)PF_ROWS / p.head_slots;
    const uint32_t tiles = (chunk_len + p.tile_tokens - 1) / p.tile_tokens;
    dim3 grid(tiles * pool->n_kv_head, n_seqs);
    brc_stage_begin(pool, BRC_STAGE_PREFILL, brc_stream(stream));
    prefill_attn_kernel<<<grid, PF_THREADS, PF_SMEM, brc_stream(stream)>>>(p);
    brc_stage_end(pool, BRC_STAGE_PREFILL, brc_stream(stream));
    BRC_CUDA(cudaGetLastError());
    return BRC_OK;
}

}  // extern "C"

