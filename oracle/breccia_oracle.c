/*
 * CPU oracle for the paged KV-cache hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the reference's own CPU algorithm for the
 * path (carlkrott/breccia).  Nothing in the product links or calls it: only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg do, and there
 * only as the checker / the timed baseline.
 *
 * Parity pin status
 *   - f16 codec, page layout, pool sizes: pinned by the reference's own
 *     known-answer tests (crates/breccia-kernels/src/qsa/cpu.rs:502-515,
 *     crates/breccia-kernels/shaders/f16_storage.glsl:4-6,
 *     crates/breccia-kernels/src/qsa/mod.rs:2028-2048,2129-2134,
 *     crates/breccia-kernels/tests/attn_conformance.rs:1172-1275).
 *   - attention (`attend`): the reference holds no golden output tensors; its
 *     tests compare GPU results with this same f64 algorithm within a bar.  The
 *     restatement is cross-checked against an independent NumPy float64
 *     restatement.  Parity for the attention values is therefore "unpinned".
 *   - page copy / fork / LSE-combine / causal chunk attention over a shared
 *     pool: the reference has no implementation; these references define the
 *     semantics in this repository ("parity unpinned").
 *
 * The reference is Rust + GLSL; neither toolchain exists here, so it cannot be
 * compiled.  Every function names the reference lines it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define BRC_REF_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* f16 storage codec                                                         */
/* ------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float x)
{
    uint32_t b;
    memcpy(&b, &x, 4);
    return b;
}

static inline float bits_f32(uint32_t b)
{
    float x;
    memcpy(&x, &b, 4);
    return x;
}

/* crates/breccia-kernels/shaders/f16_storage.glsl:26-55
 * Round-to-nearest-even f32 -> binary16 bits by integer arithmetic:
 * |x| >= 65520 -> inf (NaN lands here too), exponent < -14 -> signed zero
 * (decided before rounding, so no subnormal is ever produced). */
BRC_REF_API uint16_t brc_ref_f32_to_f16_bits(float x)
{
    const uint32_t b = f32_bits(x);
    const uint32_t sign = (b >> 16) & 0x8000u;
    const uint32_t mag = b & 0x7fffffffu;
    if (mag >= 0x477ff000u)
        return (uint16_t)(sign | 0x7c00u);
    int e = (int)((mag >> 23) & 0xffu) - 127;
    if (e > 15)
        return (uint16_t)(sign | 0x7c00u);
    if (e < -14)
        return (uint16_t)sign;
    const uint32_t m = mag & 0x7fffffu;
    uint32_t q = (m >> 13) | 0x400u;
    const uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u)))
        q += 1u;
    if (q >= 0x800u) {
        q >>= 1;
        e += 1;
        if (e > 15)
            return (uint16_t)(sign | 0x7c00u);
    }
    return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | (q & 0x3ffu));
}

/* crates/breccia-kernels/shaders/f16_storage.glsl:58-69
 * Exact binary16 bits -> f32; exponent field 0 reads as signed zero. */
BRC_REF_API float brc_ref_f16_bits_to_f32(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = ((uint32_t)h >> 10) & 0x1fu;
    const uint32_t m = (uint32_t)h & 0x3ffu;
    if (e == 0u)
        return bits_f32(sign);
    if (e == 31u)
        return bits_f32(sign | 0x7f800000u | (m << 13));
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* crates/breccia-kernels/src/qsa/cpu.rs:23-53
 * The same rule stated the way the Rust oracle states it (f32 -> f16 grid ->
 * f32), kept as a separate transcription so the two can be held equal. */
BRC_REF_API float brc_ref_to_f16(float x)
{
    const uint32_t b = f32_bits(x);
    const uint32_t sign = b & 0x80000000u;
    const int exp = (int)((b >> 23) & 0xffu) - 127;
    if ((b & 0x7fffffffu) == 0u)
        return bits_f32(sign);
    if (exp > 15)
        return bits_f32(sign | 0x7f800000u);
    if (exp < -14)
        return bits_f32(sign);
    const uint32_t m = (b & 0x007fffffu) | 0x00800000u;
    const uint32_t shift = 13;
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u) == 1u))
        q += 1u;
    int e2 = exp;
    uint32_t q2 = q;
    if (q >= (1u << 11)) {
        e2 = exp + 1;
        q2 = q >> 1;
    }
    if (e2 > 15)
        return bits_f32(sign | 0x7f800000u);
    return bits_f32(sign | ((uint32_t)(e2 + 127) << 23) | ((q2 & 0x3ffu) << 13));
}

/* crates/breccia-kernels/shaders/f16_storage.glsl:72-74: low half = first. */
BRC_REF_API uint32_t brc_ref_pack_f16x2(float lo, float hi)
{
    return ((uint32_t)brc_ref_f32_to_f16_bits(hi) << 16) | brc_ref_f32_to_f16_bits(lo);
}

/* crates/breccia-kernels/src/qsa/cpu.rs:65-82 — q8_0 round trip of a V row:
 * scale = amax/127 per 32 elements (1 for an all-zero block),
 * q = round-half-away(clamp(x/scale, -127, 127)), value read back = q*scale. */
BRC_REF_API int brc_ref_to_q8_0(const float *x, size_t n, float *out)
{
    if (n % 32u)
        return -1;
    for (size_t b = 0; b < n; b += 32) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) {
            const float a = fabsf(x[b + i]);
            amax = a > amax ? a : amax;
        }
        const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        for (int i = 0; i < 32; ++i) {
            float t = x[b + i] / scale;
            t = t < -127.0f ? -127.0f : (t > 127.0f ? 127.0f : t);
            out[b + i] = roundf(t) * scale;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Page layout and sizes                                                     */
/* ------------------------------------------------------------------------- */

/* crates/breccia-kernels/src/qsa/mod.rs:22-28 (element index of the layout). */
BRC_REF_API uint64_t brc_ref_elem_index(uint64_t page, uint64_t kv_head, uint64_t cell_in_page,
                                        uint64_t d, uint64_t n_kv_head, uint64_t page_cells,
                                        uint64_t head_dim)
{
    return ((page * n_kv_head + kv_head) * page_cells + cell_in_page) * head_dim + d;
}

/* crates/breccia-kernels/src/qsa/mod.rs:316-388 (`sizes`), parametric. */
BRC_REF_API uint64_t brc_ref_f16_pool_bytes(uint64_t pages, uint64_t n_kv_head,
                                            uint64_t page_cells, uint64_t head_dim)
{
    return pages * n_kv_head * page_cells * head_dim * 2u;
}

BRC_REF_API uint64_t brc_ref_pool_rows(uint64_t pages, uint64_t n_kv_head, uint64_t page_cells)
{
    return pages * n_kv_head * page_cells;
}

BRC_REF_API uint64_t brc_ref_f16_row_words(uint64_t head_dim) { return head_dim / 2u; }

/* q8_0 V row: head_dim/32 blocks of (32 x i8 + one f32 scale) = 9 words. */
BRC_REF_API uint64_t brc_ref_q8v_row_words(uint64_t head_dim) { return head_dim / 32u * 9u; }

BRC_REF_API uint64_t brc_ref_q8v_pool_bytes(uint64_t pages, uint64_t n_kv_head,
                                            uint64_t page_cells, uint64_t head_dim)
{
    return pages * n_kv_head * page_cells * (head_dim / 32u) * 36u;
}

/* K + V bytes of one page of one layer (crates/.../qsa/mod.rs:237-240). */
BRC_REF_API uint64_t brc_ref_page_bytes(uint64_t n_kv_head, uint64_t page_cells, uint64_t head_dim)
{
    return 2u * brc_ref_f16_pool_bytes(1, n_kv_head, page_cells, head_dim);
}

/* ------------------------------------------------------------------------- */
/* KV append                                                                 */
/* ------------------------------------------------------------------------- */

/* crates/breccia-kernels/shaders/qsa_kv_append.comp:137-161 with the host guard
 * of crates/breccia-kernels/src/qsa/mod.rs:1108-1116.
 * One (token, kv head, d-pair) unit writes one 32-bit word of K and one of V:
 *   cell = pos0 + t; page = PT[cell / page_cells];
 *   word = ((page*n_kv + kvh)*page_cells + cell % page_cells) * (hd/2) + pair.
 * Returns -1 (nothing written) if the write would pass `capacity_cells`. */
BRC_REF_API int brc_ref_kv_append(uint32_t *k_pool, uint32_t *v_pool, const uint32_t *page_table,
                                  const float *k_cur, const float *v_cur, uint32_t tokens,
                                  uint32_t pos0, uint32_t n_kv_head, uint32_t head_dim,
                                  uint32_t page_cells, uint64_t capacity_cells)
{
    if ((uint64_t)pos0 + tokens > capacity_cells)
        return -1;
    const uint32_t pairs = head_dim / 2u;
    const uint64_t total = (uint64_t)tokens * n_kv_head * pairs;
    for (uint64_t unit = 0; unit < total; ++unit) {
        const uint32_t pair = (uint32_t)(unit % pairs);
        const uint64_t rest = unit / pairs;
        const uint32_t kvh = (uint32_t)(rest % n_kv_head);
        const uint32_t t = (uint32_t)(rest / n_kv_head);
        const uint32_t cell = pos0 + t;
        const uint64_t page = page_table[cell / page_cells];
        const uint32_t in_page = cell % page_cells;
        const uint64_t word = ((page * n_kv_head + kvh) * page_cells + in_page) * pairs + pair;
        const uint64_t src = (uint64_t)t * n_kv_head * head_dim + (uint64_t)kvh * head_dim + pair * 2u;
        k_pool[word] = brc_ref_pack_f16x2(k_cur[src], k_cur[src + 1]);
        v_pool[word] = brc_ref_pack_f16x2(v_cur[src], v_cur[src + 1]);
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Gather: paged pool -> logical [cell][kv_head][d]                          */
/* ------------------------------------------------------------------------- */

/* The reference only ever reads pages back through an identity table
 * (crates/breccia-engine/src/graph.rs:2204-2228); this applies the layout
 * formula (qsa/mod.rs:22-28) through a real block table.  `out_bits` receives
 * the raw binary16 bits, `out_f32` (optional) the decoded values the attention
 * reference consumes. */
BRC_REF_API void brc_ref_gather(const uint16_t *pool, const uint32_t *block_table, uint32_t n_cells,
                                uint32_t n_kv_head, uint32_t head_dim, uint32_t page_cells,
                                uint16_t *out_bits, float *out_f32)
{
    for (uint32_t c = 0; c < n_cells; ++c) {
        const uint64_t page = block_table[c / page_cells];
        const uint32_t in_page = c % page_cells;
        for (uint32_t kvh = 0; kvh < n_kv_head; ++kvh) {
            const uint64_t src = brc_ref_elem_index(page, kvh, in_page, 0, n_kv_head, page_cells, head_dim);
            const uint64_t dst = ((uint64_t)c * n_kv_head + kvh) * head_dim;
            for (uint32_t d = 0; d < head_dim; ++d) {
                const uint16_t h = pool[src + d];
                if (out_bits)
                    out_bits[dst + d] = h;
                if (out_f32)
                    out_f32[dst + d] = brc_ref_f16_bits_to_f32(h);
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Attention                                                                 */
/* ------------------------------------------------------------------------- */

static double sigmoid64(double x)
{
    /* crates/breccia-kernels/src/qsa/cpu.rs:84-91 */
    if (x >= 0.0)
        return 1.0 / (1.0 + exp(-x));
    const double e = exp(x);
    return e / (1.0 + e);
}

/* One head of crates/breccia-kernels/src/qsa/cpu.rs:197-246. */
static void attend_head(const float *q, const float *k, const float *v, const uint32_t *cells,
                        size_t n_cells, size_t pos, size_t h, size_t n_head, size_t n_kv_head,
                        size_t head_dim, const float *gate, float *out, double *logits, double *acc)
{
    const double scale = 1.0 / sqrt((double)head_dim);
    const size_t kvh = h * n_kv_head / n_head;
    const size_t row = n_kv_head * head_dim;
    size_t n = 0;
    for (size_t i = 0; i < n_cells; ++i) {
        const size_t c = cells[i];
        if (c > pos)
            continue;
        double dot = 0.0;
        const float *kr = k + c * row + kvh * head_dim;
        const float *qr = q + h * head_dim;
        for (size_t d = 0; d < head_dim; ++d)
            dot += (double)qr[d] * (double)kr[d];
        logits[n++] = dot * scale;
    }
    double mx = -INFINITY;
    for (size_t i = 0; i < n; ++i)
        mx = logits[i] > mx ? logits[i] : mx;
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) {
        logits[i] = exp(logits[i] - mx);
        sum += logits[i];
    }
    for (size_t d = 0; d < head_dim; ++d)
        acc[d] = 0.0;
    size_t j = 0;
    for (size_t i = 0; i < n_cells; ++i) {
        const size_t c = cells[i];
        if (c > pos)
            continue;
        const double p = logits[j++] / sum;
        const float *vr = v + c * row + kvh * head_dim;
        for (size_t d = 0; d < head_dim; ++d)
            acc[d] += p * (double)vr[d];
    }
    for (size_t d = 0; d < head_dim; ++d) {
        /* gate == NULL stands for the reference called with gate = +1e4, whose
         * f64 sigmoid is exactly 1.0. */
        const double g = gate ? sigmoid64((double)gate[h * head_dim + d]) : 1.0;
        out[h * head_dim + d] = (float)(acc[d] * g);
    }
}

/* crates/breccia-kernels/src/qsa/cpu.rs:197-246 (`attend`): dense causal
 * attention over the listed cells with c <= pos, f64 accumulate, softmax over
 * those cells only, sigmoid(gate) last, cast to f32.  k and v are logical
 * arrays [cell][kv_head][d] already on the f16 grid. */
BRC_REF_API int brc_ref_attend(const float *q, const float *k, const float *v, const uint32_t *cells,
                               size_t n_cells, size_t pos, size_t n_head, size_t n_kv_head,
                               size_t head_dim, const float *gate, float *out)
{
    double *logits = (double *)malloc(sizeof(double) * (n_cells + 1));
    double *acc = (double *)malloc(sizeof(double) * head_dim);
    if (!logits || !acc) {
        free(logits);
        free(acc);
        return -1;
    }
    for (size_t h = 0; h < n_head; ++h)
        attend_head(q, k, v, cells, n_cells, pos, h, n_head, n_kv_head, head_dim, gate, out, logits, acc);
    free(logits);
    free(acc);
    return 0;
}

/* crates/breccia-kernels/src/qsa/cpu.rs:249-257 (`cells_of`). */
BRC_REF_API void brc_ref_cells_of(const uint32_t *blocks, size_t n_blocks, size_t idx_block,
                                  uint32_t *out)
{
    for (size_t b = 0; b < n_blocks; ++b)
        for (size_t k = 0; k < idx_block; ++k)
            out[b * idx_block + k] = blocks[b] * (uint32_t)idx_block + (uint32_t)k;
}

/* crates/breccia-kernels/src/ops/cpu.rs:166-183: f64 row softmax (max, exp,
 * normalise), used for a score-level cross-check. */
BRC_REF_API void brc_ref_softmax_rows(const float *x, size_t rows, size_t cols, double *out)
{
    for (size_t r = 0; r < rows; ++r) {
        double mx = -INFINITY;
        for (size_t c = 0; c < cols; ++c)
            mx = (double)x[r * cols + c] > mx ? (double)x[r * cols + c] : mx;
        double sum = 0.0;
        for (size_t c = 0; c < cols; ++c) {
            out[r * cols + c] = exp((double)x[r * cols + c] - mx);
            sum += out[r * cols + c];
        }
        for (size_t c = 0; c < cols; ++c)
            out[r * cols + c] /= sum;
    }
}

/* Batched paged decode step of one layer: for every sequence gather its cells
 * through its block table (layout formula) and run `attend` over cells
 * 0..seq_len-1 with pos = seq_len-1 (the dense selection the reference's
 * `topk_dense` emits, crates/breccia-kernels/src/qsa/mod.rs:1365-1376).
 * Threads split independent (sequence, head) pairs only; arithmetic per pair is
 * the scalar f64 algorithm above.  q: [n_seqs][n_head][hd] f32,
 * gate: same shape or NULL, out: [n_seqs][n_head][hd] f32.  Returns the number
 * of threads used, or -1. */
BRC_REF_API int brc_ref_decode_batch(const uint16_t *k_pool, const uint16_t *v_pool,
                                     const uint32_t *block_tables, uint32_t table_stride,
                                     const uint32_t *seq_lens, uint32_t n_seqs, const float *q,
                                     const float *gate, uint32_t n_head, uint32_t n_kv_head,
                                     uint32_t head_dim, uint32_t page_cells, float *out,
                                     int n_threads)
{
    int used = 1;
#ifdef _OPENMP
    if (n_threads > 0)
        omp_set_num_threads(n_threads);
    used = omp_get_max_threads();
#else
    (void)n_threads;
#endif
    size_t max_len = 0;
    for (uint32_t s = 0; s < n_seqs; ++s)
        max_len = seq_lens[s] > max_len ? seq_lens[s] : max_len;
    const size_t row = (size_t)n_kv_head * head_dim;
    float **kl = (float **)calloc(n_seqs, sizeof(float *));
    float **vl = (float **)calloc(n_seqs, sizeof(float *));
    uint32_t *cells = (uint32_t *)malloc(sizeof(uint32_t) * (max_len + 1));
    if (!kl || !vl || !cells)
        return -1;
    for (size_t c = 0; c < max_len; ++c)
        cells[c] = (uint32_t)c;
    int failed = 0;
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t s = 0; s < n_seqs; ++s) {
        const size_t len = seq_lens[s];
        kl[s] = (float *)malloc(sizeof(float) * (len * row + 1));
        vl[s] = (float *)malloc(sizeof(float) * (len * row + 1));
        if (!kl[s] || !vl[s]) {
            failed = 1;
            continue;
        }
        brc_ref_gather(k_pool, block_tables + (size_t)s * table_stride, (uint32_t)len, n_kv_head,
                       head_dim, page_cells, NULL, kl[s]);
        brc_ref_gather(v_pool, block_tables + (size_t)s * table_stride, (uint32_t)len, n_kv_head,
                       head_dim, page_cells, NULL, vl[s]);
    }
    if (!failed) {
#pragma omp parallel
        {
            double *logits = (double *)malloc(sizeof(double) * (max_len + 1));
            double *acc = (double *)malloc(sizeof(double) * head_dim);
#pragma omp for schedule(dynamic, 1)
            for (uint32_t sh = 0; sh < n_seqs * n_head; ++sh) {
                const uint32_t s = sh / n_head, h = sh % n_head;
                const size_t len = seq_lens[s];
                float *o = out + (size_t)s * n_head * head_dim;
                if (len == 0) {
                    for (uint32_t d = 0; d < head_dim; ++d)
                        o[h * head_dim + d] = 0.0f;
                    continue;
                }
                attend_head(q + (size_t)s * n_head * head_dim, kl[s], vl[s], cells, len, len - 1, h,
                            n_head, n_kv_head, head_dim,
                            gate ? gate + (size_t)s * n_head * head_dim : NULL, o, logits, acc);
            }
            free(logits);
            free(acc);
        }
    }
    for (uint32_t s = 0; s < n_seqs; ++s) {
        free(kl[s]);
        free(vl[s]);
    }
    free(kl);
    free(vl);
    free(cells);
    return failed ? -1 : used;
}

/* Chunked prefill over a paged cache: `chunk` query rows at positions
 * pos0..pos0+chunk-1; row t attends cells 0..=pos0+t.  This is the reference's
 * multi-row rule (all rows' cells appended first, then row t masked by
 * cell <= pos0+t: crates/breccia-kernels/shaders/qsa_attn_scores_small.comp:74-77,
 * crates/breccia-kernels/src/qsa/mod.rs:1617,1638) evaluated with `attend` per
 * row.  q, out: [chunk][n_head][hd]; threads split (row, head) pairs. */
BRC_REF_API int brc_ref_prefill_chunk(const uint16_t *k_pool, const uint16_t *v_pool,
                                      const uint32_t *block_table, uint32_t pos0, uint32_t chunk,
                                      const float *q, const float *gate, uint32_t n_head,
                                      uint32_t n_kv_head, uint32_t head_dim, uint32_t page_cells,
                                      float *out, int n_threads)
{
    int used = 1;
#ifdef _OPENMP
    if (n_threads > 0)
        omp_set_num_threads(n_threads);
    used = omp_get_max_threads();
#else
    (void)n_threads;
#endif
    const size_t len = (size_t)pos0 + chunk;
    const size_t row = (size_t)n_kv_head * head_dim;
    float *kl = (float *)malloc(sizeof(float) * (len * row + 1));
    float *vl = (float *)malloc(sizeof(float) * (len * row + 1));
    uint32_t *cells = (uint32_t *)malloc(sizeof(uint32_t) * (len + 1));
    if (!kl || !vl || !cells)
        return -1;
    for (size_t c = 0; c < len; ++c)
        cells[c] = (uint32_t)c;
    brc_ref_gather(k_pool, block_table, (uint32_t)len, n_kv_head, head_dim, page_cells, NULL, kl);
    brc_ref_gather(v_pool, block_table, (uint32_t)len, n_kv_head, head_dim, page_cells, NULL, vl);
#pragma omp parallel
    {
        double *logits = (double *)malloc(sizeof(double) * (len + 1));
        double *acc = (double *)malloc(sizeof(double) * head_dim);
#pragma omp for schedule(dynamic, 1)
        for (uint32_t th = 0; th < chunk * n_head; ++th) {
            const uint32_t t = th / n_head, h = th % n_head;
            attend_head(q + (size_t)t * n_head * head_dim, kl, vl, cells, len, (size_t)pos0 + t, h,
                        n_head, n_kv_head, head_dim,
                        gate ? gate + (size_t)t * n_head * head_dim : NULL,
                        out + (size_t)t * n_head * head_dim, logits, acc);
        }
        free(logits);
        free(acc);
    }
    free(kl);
    free(vl);
    free(cells);
    return used;
}

/* ------------------------------------------------------------------------- */
/* Operations the reference does not implement (semantics defined here)      */
/* ------------------------------------------------------------------------- */

/* Split-KV partial of one head over a cell range, and the log-sum-exp combine.
 * Partial format (the one the device kernels exchange): m = max logit in base-2
 * units (logit * log2 e), l = sum 2^(logit2 - m), acc[d] = sum 2^(logit2 - m) v[d].
 * An empty range gives m = -inf, l = 0, acc = 0. */
BRC_REF_API void brc_ref_partial_head(const float *q_head, const float *k, const float *v,
                                      size_t cell_begin, size_t cell_end, size_t kvh,
                                      size_t n_kv_head, size_t head_dim, double scale, double *m_out,
                                      double *l_out, double *acc_out)
{
    const double log2e = 1.4426950408889634074;
    const size_t row = n_kv_head * head_dim;
    double m = -INFINITY;
    for (size_t c = cell_begin; c < cell_end; ++c) {
        double dot = 0.0;
        for (size_t d = 0; d < head_dim; ++d)
            dot += (double)q_head[d] * (double)k[c * row + kvh * head_dim + d];
        const double s = dot * scale * log2e;
        m = s > m ? s : m;
    }
    double l = 0.0;
    for (size_t d = 0; d < head_dim; ++d)
        acc_out[d] = 0.0;
    for (size_t c = cell_begin; c < cell_end; ++c) {
        double dot = 0.0;
        for (size_t d = 0; d < head_dim; ++d)
            dot += (double)q_head[d] * (double)k[c * row + kvh * head_dim + d];
        const double p = exp2(dot * scale * log2e - m);
        l += p;
        for (size_t d = 0; d < head_dim; ++d)
            acc_out[d] += p * (double)v[c * row + kvh * head_dim + d];
    }
    *m_out = m;
    *l_out = l;
}

/* out[d] = sum_r 2^(m_r - M) acc_r[d] / sum_r 2^(m_r - M) l_r, M = max_r m_r.
 * Parts with l == 0 (empty ranges) are skipped; all-empty gives zeros. */
BRC_REF_API void brc_ref_lse_combine(const double *m, const double *l, const double *acc,
                                     size_t n_parts, size_t head_dim, double *out)
{
    double M = -INFINITY;
    for (size_t r = 0; r < n_parts; ++r)
        if (l[r] > 0.0 && m[r] > M)
            M = m[r];
    double L = 0.0;
    for (size_t d = 0; d < head_dim; ++d)
        out[d] = 0.0;
    for (size_t r = 0; r < n_parts; ++r) {
        if (!(l[r] > 0.0))
            continue;
        const double w = exp2(m[r] - M);
        L += w * l[r];
        for (size_t d = 0; d < head_dim; ++d)
            out[d] += w * acc[r * head_dim + d];
    }
    if (L > 0.0)
        for (size_t d = 0; d < head_dim; ++d)
            out[d] /= L;
}

/* Page copy across all layers, K and V: plain byte copies of whole pages.
 * Pools are [n_layers][n_pages][page bytes]. */
BRC_REF_API void brc_ref_page_copy(uint8_t *k_pool, uint8_t *v_pool, uint64_t n_layers,
                                   uint64_t n_pages, uint64_t half_page_bytes,
                                   const uint32_t *src_ids, const uint32_t *dst_ids, size_t n)
{
    for (uint64_t layer = 0; layer < n_layers; ++layer) {
        uint8_t *kb = k_pool + layer * n_pages * half_page_bytes;
        uint8_t *vb = v_pool + layer * n_pages * half_page_bytes;
        for (size_t i = 0; i < n; ++i) {
            memmove(kb + (uint64_t)dst_ids[i] * half_page_bytes,
                    kb + (uint64_t)src_ids[i] * half_page_bytes, half_page_bytes);
            memmove(vb + (uint64_t)dst_ids[i] * half_page_bytes,
                    vb + (uint64_t)src_ids[i] * half_page_bytes, half_page_bytes);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Input generators                                                          */
/* ------------------------------------------------------------------------- */

/* crates/breccia-kernels/tests/attn_conformance.rs:110-124 (`normalish`):
 * the reference test-suite's 64-bit LCG, sum of four uniforms, f32 arithmetic. */
BRC_REF_API void brc_ref_normalish(uint64_t seed, size_t n, float *out)
{
    uint64_t s = seed | 1u;
    for (size_t i = 0; i < n; ++i) {
        float acc = 0.0f;
        for (int k = 0; k < 4; ++k) {
            s = s * 6364136223846793005ull + 1442695040888963407ull;
            acc += (float)(s >> 33) / (float)(0xffffffffu >> 1);
        }
        out[i] = (acc - 1.0f) * 1.732f;
    }
}

/* crates/breccia-kernels/tests/attn_conformance.rs:102-108 (`max_rel`):
 * max |got - want| / max(|want|, 1). */
BRC_REF_API double brc_ref_max_rel(const float *got, const double *want, size_t n)
{
    double m = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const double w = fabs(want[i]) > 1.0 ? fabs(want[i]) : 1.0;
        const double e = fabs((double)got[i] - want[i]) / w;
        m = e > m ? e : m;
    }
    return m;
}

/* Whole-range check that the two transcriptions of the f16 rule agree: walks
 * f32 bit patterns from `first` in steps of `stride`, `count` of them, and
 * returns the number of disagreements between brc_ref_to_f16 (Rust form) and
 * decode(encode()) (GLSL form). */
BRC_REF_API uint64_t brc_ref_f16_rule_mismatches(uint32_t first, uint32_t stride, uint64_t count)
{
    uint64_t bad = 0;
    uint32_t b = first;
    for (uint64_t i = 0; i < count; ++i, b += stride) {
        const float x = bits_f32(b);
        const float a = brc_ref_to_f16(x);
        const float c = brc_ref_f16_bits_to_f32(brc_ref_f32_to_f16_bits(x));
        if (f32_bits(a) != f32_bits(c))
            ++bad;
    }
    return bad;
}
