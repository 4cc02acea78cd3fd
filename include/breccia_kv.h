/*
 * libbreccia_kv — C ABI of the B200 (sm_100a) paged KV-cache hot path.
 *
 * Drop-in boundary for the `breccia-kernels::qsa` operator surface of
 * carlkrott/breccia: a caller that today drives `QsaState` / `Qsa::{kv_append,
 * attend, apply}` binds these entry points instead.  Each declaration cites the
 * reference interface it replaces (path inside the reference project : line).
 *
 * Conventions (the reference's, kept):
 *   - every entry point returns a status (0 = OK, negative = error) and never
 *     throws or aborts; `brc_last_error()` gives a thread-local message with
 *     the offending numbers (reference: `anyhow::Result`, qsa/mod.rs:1108-1116);
 *   - shape / capacity violations are refused on the host BEFORE any launch;
 *   - the caller owns state explicitly (create / destroy), nothing here
 *     allocates inside a launch, and launches are asynchronous on the stream
 *     passed as `void*` (a `cudaStream_t`; NULL = the legacy default stream);
 *   - pointers named `*_dev` are device addresses on the pool's GPU, everything
 *     else is host memory;
 *   - there is no CPU fallback: without a usable GPU every compute call fails
 *     with BRC_ERR_CUDA.
 *
 * Page layout (crates/breccia-kernels/src/qsa/mod.rs:22-28, identical):
 *   K and V pools of one layer are arrays of u16 binary16 bits,
 *     element = ((page * n_kv_head + kv_head) * page_tokens + cell_in_page) * head_dim + d
 *   one pool per (GPU, layer) shared by all sequences; a sequence is a block
 *   table of physical page ids.  A page id addresses the same slot in every
 *   layer's K and V pool.
 */
#ifndef BRECCIA_KV_H
#define BRECCIA_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(BRC_BUILDING_LIB)
#define BRC_API __attribute__((visibility("default")))
#else
#define BRC_API
#endif

typedef int32_t brc_status;

#define BRC_OK 0
#define BRC_ERR_INVALID (-1)      /* bad argument / shape                         */
#define BRC_ERR_CAPACITY (-2)     /* write past the block table / pool exhausted  */
#define BRC_ERR_CUDA (-3)         /* a CUDA runtime / driver call failed          */
#define BRC_ERR_NO_PAGES (-4)     /* allocator has too few free pages             */
#define BRC_ERR_TIMEOUT (-5)      /* a bounded device-side wait gave up           */
#define BRC_ERR_DEVICE_CHECK (-6) /* a kernel's own bounds check refused an index */
#define BRC_ERR_UNSUPPORTED (-7)  /* geometry outside what the kernels are built for */
#define BRC_ERR_NOT_RESIDENT (-8) /* page is in the host tier                     */

/* dtype tags for query / source tensors */
#define BRC_DTYPE_F32 0
#define BRC_DTYPE_F16 1

typedef struct brc_pool brc_pool;
typedef struct brc_radix brc_radix;
typedef struct brc_tier brc_tier;
typedef struct brc_cold brc_cold;
typedef struct brc_comm brc_comm;

typedef struct brc_geometry {
    uint32_t n_layers;
    uint32_t n_kv_head;
    uint32_t head_dim;
    uint32_t page_tokens;
    uint32_t n_pages;
    int32_t device;
    uint64_t half_page_bytes; /* bytes of K (or V) of one page of one layer */
    uint64_t total_bytes;     /* K + V, all layers                          */
} brc_geometry;

/* Thread-local text of the last error returned on this thread ("" if none). */
BRC_API const char *brc_last_error(void);
BRC_API int32_t brc_abi_version(void);

/* ---------------------------------------------------------------- pool / state
 * Replaces QsaState::{new, with_layout, reset, bytes, release}
 * (crates/breccia-kernels/src/qsa/mod.rs:393,399,551,572,591) with ONE pool per
 * (GPU, layer set) shared by all sequences.  Pools are zero-filled on creation
 * like the reference (qsa/mod.rs:399-535). */
BRC_API brc_status brc_pool_create(int32_t device, uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim,
                                   uint32_t page_tokens, uint32_t n_pages, brc_pool **out);
/* The same pool with V page bodies stored as q8_0, the reference's VLayout::Q8_0
 * (qsa/mod.rs:245-349; QsaState::with_layout, qsa/mod.rs:399): a V row is
 * head_dim / 32 blocks of one f32 scale followed by 32 signed bytes (36 B for 32
 * values against 64 B: 0.5625x the V bytes), rows in the order of the binary16
 * layout; K stays binary16.  Built for such a pool: brc_kv_append from f32 sources
 * (store rule of shaders/qsa_kv_append.comp:117-133); the dense decode entry
 * points brc_paged_decode_attn(_static), brc_decode_partial, brc_decode_step(_part,
 * _host) with f32 new K/V (the fused append quantises by the same rule) and
 * brc_splitkv_attend / _step - the quanta reach the tensor cores as exact
 * integers and the block scales ride on the probabilities (read rule
 * qsa_attn_apply.comp:60-77), 1600 instead of 2048 bytes per cached cell at
 * 2 kv heads of 256; brc_paged_sparse_attn (in-register dequantisation);
 * brc_page_copy and brc_seq_fork (whole pages, bytes as they are); tiering and
 * the cold store (brc_tier_*, brc_cold_*: a host slot then holds K halves of
 * 16 KiB and V halves of 9 KiB per layer); brc_page_gather (V rows as stored);
 * the page files (brc_state_dump / _load: the reference's `qsa_vq8` part,
 * crates/breccia-engine/src/graph.rs:2183-2186); brc_pool_read /
 * brc_pool_write / brc_pool_v_ptr, the allocator and the prefix tree;
 * brc_qk_prepare_append (V quantised by the append's rule); and
 * brc_paged_prefill_attn, whose loaders dequantise the blocks into the
 * binary16 V tile (scale x quantum rounded to binary16: up to 2^-11 |v| of
 * absolute error on top of the binary16 path's).  Every entry point takes it;
 * only binary16 K/V sources to brc_kv_append are refused (the rule quantises
 * from f32). */
#define BRC_V_F16 0
#define BRC_V_Q8_0 1
BRC_API brc_status brc_pool_create_q8v(int32_t device, uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim,
                                       uint32_t page_tokens, uint32_t n_pages, brc_pool **out);
BRC_API brc_status brc_pool_v_layout(const brc_pool *pool, int32_t *out_layout);
/* A pool without device memory: page ids, refcounts and (later) prefix-tree and
 * tier bookkeeping only.  Every entry point that would touch the GPU refuses it
 * with BRC_ERR_CUDA.  Exists so schedulers and tests can exercise the host-side
 * state machine on a machine without a GPU; it computes nothing. */
BRC_API brc_status brc_pool_create_bookkeeping(uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim,
                                               uint32_t page_tokens, uint32_t n_pages, brc_pool **out);
BRC_API brc_status brc_pool_destroy(brc_pool *pool);
BRC_API brc_status brc_pool_geometry(const brc_pool *pool, brc_geometry *out);
/* qsa/mod.rs:572 (`bytes`) */
BRC_API brc_status brc_pool_bytes(const brc_pool *pool, uint64_t *out);
/* qsa/mod.rs:551-570 (`reset`: pools back to zero) */
BRC_API brc_status brc_pool_zero(brc_pool *pool, void *stream);
/* Test hook: fills every pool byte with 0xFF (binary16 NaN), the analogue of the
 * reference's BRECCIA_FAULT_POISON_QSA flag (qsa/mod.rs:509-523). */
BRC_API brc_status brc_pool_poison_nan(brc_pool *pool, void *stream);
BRC_API brc_status brc_pool_k_ptr(const brc_pool *pool, uint32_t layer, void **out_dev);
BRC_API brc_status brc_pool_v_ptr(const brc_pool *pool, uint32_t layer, void **out_dev);
/* Byte-range read-back / upload of one layer's K (which = 0) or V (which = 1)
 * pool, ordered on `stream` and complete on return (the reference's
 * `gemv::download` / `upload_into`, crates/breccia-kernels/src/gemv.rs:1059-1071).
 * Host memory may be pageable. */
BRC_API brc_status brc_pool_read(brc_pool *pool, int32_t which, uint32_t layer, uint64_t byte_offset, void *dst,
                                 uint64_t bytes, void *stream);
BRC_API brc_status brc_pool_write(brc_pool *pool, int32_t which, uint32_t layer, uint64_t byte_offset,
                                  const void *src, uint64_t bytes, void *stream);
/* Synchronises `stream`, then reports and clears the device-side check word:
 * BRC_OK, BRC_ERR_DEVICE_CHECK (an out-of-range page id or position reached a
 * kernel, which skipped the access) or BRC_ERR_TIMEOUT (a bounded wait gave
 * up).  Mirrors the reference's bounded fence wait
 * (crates/breccia-vk/src/ctx.rs:1541-1561) without aborting the process. */
BRC_API brc_status brc_pool_check(brc_pool *pool, void *stream);

/* ---------------------------------------------------------------- page allocator / refcounts
 * No counterpart in the reference (design note docs/reference-engines/
 * 02-kv-and-context.md:543-581: block = id + refcount + free queue).  Host-side,
 * thread-safe.  Freshly allocated pages have refcount 1. */
BRC_API brc_status brc_pages_alloc(brc_pool *pool, uint32_t n, uint32_t *out_ids);
BRC_API brc_status brc_pages_retain(brc_pool *pool, const uint32_t *ids, uint32_t n);
/* Drops one reference each; a page returns to the free list at refcount 0. */
BRC_API brc_status brc_pages_release(brc_pool *pool, const uint32_t *ids, uint32_t n);
BRC_API brc_status brc_page_refcount(const brc_pool *pool, uint32_t id, uint32_t *out);
BRC_API brc_status brc_pages_free_count(const brc_pool *pool, uint32_t *out);

/* ---------------------------------------------------------------- KV append
 * Replaces Qsa::kv_append (crates/breccia-kernels/src/qsa/mod.rs:1107-1156) and
 * shaders/qsa_kv_append.comp:137-161, batched over sequences.
 *
 * Sequence s appends its tokens at cells pos0_dev[s] .. through its block table
 * row block_tables_dev[s*table_stride ..].  Tokens per sequence are uniform
 * (`tokens_per_seq`, cu_tokens_dev == NULL) or ragged (cu_tokens_dev[n_seqs+1]
 * exclusive prefix of token counts; tokens_per_seq ignored).  Sources are
 * [total_tokens][n_kv_head*head_dim], f32 (reference) or f16 bits already on
 * the storage grid.  f32 sources are encoded by the reference's integer
 * round-to-nearest-even rule (shaders/f16_storage.glsl:26-55), bit-exact.
 *
 * `max_pos_end` is the caller's bound on pos0[s]+tokens(s); the host refuses
 * max_pos_end > table_stride*page_tokens (the reference's capacity check) and
 * the kernel skips, and reports through brc_pool_check, any token beyond it or
 * any block-table entry >= n_pages. */
BRC_API brc_status brc_kv_append(brc_pool *pool, uint32_t layer, const uint32_t *block_tables_dev,
                                 uint32_t table_stride, const uint32_t *pos0_dev, uint32_t n_seqs,
                                 uint32_t tokens_per_seq, const uint32_t *cu_tokens_dev, uint32_t total_tokens,
                                 uint32_t max_pos_end, const void *k_src_dev, const void *v_src_dev,
                                 int32_t src_dtype, void *stream);

/* ---------------------------------------------------------------- page gather / copy / fork
 * Gather: the reference reads pages back only through an identity table
 * (crates/breccia-engine/src/graph.rs:2204-2228, `dump_state`); this reads
 * `n_tokens` cells of one sequence through a real block table into logical
 * [n_tokens][n_kv_head][head_dim] binary16 arrays; on a q8_0 V pool v_out
 * receives the stored rows, [n_tokens][n_kv_head][head_dim / 32 * 36] bytes. */
BRC_API brc_status brc_page_gather(brc_pool *pool, uint32_t layer, const uint32_t *block_table_dev,
                                   uint32_t table_len, uint32_t n_tokens, void *k_out_dev, void *v_out_dev,
                                   void *stream);
/* Copies whole pages src_ids[i] -> dst_ids[i] in every layer, K and V (no
 * counterpart in the reference).  Ids are device arrays; pairs must not chain
 * (no dst that is also a src). */
BRC_API brc_status brc_page_copy(brc_pool *pool, const uint32_t *src_ids_dev, const uint32_t *dst_ids_dev,
                                 uint32_t n, void *stream);
/* Copy-on-write fork of a sequence of `n_tokens` cells (no counterpart in the
 * reference): every full page of the parent is shared (refcount + 1); a
 * partially filled last page is copied into a freshly allocated page.  Host
 * tables in, host table out; `*out_new_page` is the private copy's id or
 * UINT32_MAX when the length is page-aligned. */
BRC_API brc_status brc_seq_fork(brc_pool *pool, const uint32_t *parent_table, uint32_t n_tokens,
                                uint32_t *child_table, uint32_t *out_new_page, void *stream);

/* ---------------------------------------------------------------- paged decode attention
 * Replaces Qsa::topk_dense + Qsa::attend + Qsa::apply at T = 1
 * (crates/breccia-kernels/src/qsa/mod.rs:1365-1376,1382-1462,1466-1580;
 * shaders qsa_attn_scores_small.comp, ops_softmax.comp,
 * qsa_attn_apply_split.comp, qsa_attn_apply_reduce.comp) for a batch of
 * sequences: out[s,h,:] = sigmoid(gate[s,h,:]) * softmax_c(scale * q[s,h].k_c) . v_c
 * over cells c < seq_lens_dev[s] (the dense selection `topk_dense` emits), with
 * kv head = h * n_kv_head / n_head.  Cells at or past seq_len are never read
 * into the result, whatever the pool holds there.  Up to 8 query heads per kv
 * head share one stream of the cache; more (up to 32, e.g. the reference
 * model's 12) are taken in passes of 8, each streaming the cache again.
 *
 *   q_dev     [n_seqs][n_head][head_dim], f16 bits or f32 (reference: f32)
 *   gate_dev  NULL, or f32 with gate[s,h,d] at gate_dev[(s*n_head + h)*gate_head_stride + d]
 *             (the reference reads it in place from the second half of each
 *             head's 2*head_dim block: pass q_full + head_dim, stride 2*head_dim)
 *   out_dev   [n_seqs][n_head][head_dim] f32
 *   scale     the reference uses 1/sqrt(head_dim)
 *   workspace_dev  scratch of at least brc_decode_workspace_bytes(); contents
 *             are undefined afterwards.  Decode calls on one pool (every entry
 *             point of this section, the step and split-KV ones included) share
 *             the pool's arrival counters, so they never overlap in time: calls
 *             on one stream are ordered by the stream, and a call issued on
 *             another stream than the previous one is made to wait for it (an
 *             event recorded behind every decode launch; not while a stream is
 *             being captured - replay a captured decode on its own).
 *   max_seq_len    caller's bound on seq_lens; refused if > table_stride*page_tokens.
 * A sequence of length 0 yields zeros.
 *
 * One launch streams the cache with one CTA per SM, each an equal share of
 * the launch's work.  The SMs of a B200 do not stream at equal rates when all
 * of them do (always the same SMs are slow); with BRC_DECODE_CALIBRATE=1 in
 * the environment the first pool of at least 1 GiB created on a device in
 * this process measures them once (about a millisecond) and every pool of
 * that device then cuts a launch's work in proportion to a part of the
 * measured deviation (measured on B200: 3-4 % faster on long single
 * sequences, +1 .. -2 % on batches, slower on q8_0 V pools; the last bits of
 * the f32 output then depend on the measurement - off by default).
 * brc_decode_share_rates reports what is in force: *out_n = the number of
 * CTAs and rates[i] = CTA i's share relative to the mean, or *out_n = 0 for
 * equal shares (no counterpart in the reference).
 *
 * Two more environment switches, read once per process: BRC_DECODE_UNIT_COST=n
 * (page-units charged per unit when a launch's work is cut into shares; the
 * default is 512 KiB worth) and BRC_DECODE_STAGE_OP=1 (one TMA operation per
 * page-unit through tensor-map views whose strides do not ascend: measured
 * faster - 0.5 % on batches, 9 % on q8_0 V pools - but outside what the
 * driver's documentation allows for a tensor map, hence off by default).
 * The second does not change a result; the first moves the share boundaries
 * and with them the order of the f32 sums (last bits). */
BRC_API brc_status brc_decode_share_rates(const brc_pool *pool, float *rates, uint32_t capacity, uint32_t *out_n);
BRC_API brc_status brc_decode_workspace_bytes(const brc_pool *pool, uint32_t n_seqs, uint32_t n_head,
                                              uint64_t *out_bytes);
BRC_API brc_status brc_paged_decode_attn(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype,
                                         uint32_t n_head, const float *gate_dev, uint32_t gate_head_stride,
                                         const uint32_t *block_tables_dev, uint32_t table_stride,
                                         const uint32_t *seq_lens_dev, uint32_t n_seqs, uint32_t max_seq_len,
                                         float scale, float *out_dev, void *workspace_dev,
                                         uint64_t workspace_bytes, void *stream);

/* The two halves, exposed for split-KV across GPUs (no counterpart in the
 * reference, whose split-K partials stay on one device:
 * qsa/mod.rs:1491-1521).  `brc_decode_partial` runs the same split-KV kernel
 * but emits, per (sequence, head), the un-normalised partial
 *   m = max_c(scale*log2(e) * q.k_c),  l = sum_c 2^(s_c - m),  acc[d] = sum_c 2^(s_c - m) v_c[d]
 * as `partial_dev`: [n_seqs][n_head][head_dim] f32 acc followed by
 * [n_seqs][n_head][2] f32 (m, l); brc_decode_partial_bytes gives the size.
 * `brc_decode_combine` merges `n_parts` such buffers laid `part_stride_bytes`
 * apart (e.g. an all-gather receive buffer), applies the gate and writes out. */
BRC_API brc_status brc_decode_partial_bytes(uint32_t n_seqs, uint32_t n_head, uint32_t head_dim,
                                            uint64_t *out_bytes);
BRC_API brc_status brc_decode_partial(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype,
                                      uint32_t n_head, const uint32_t *block_tables_dev, uint32_t table_stride,
                                      const uint32_t *seq_lens_dev, uint32_t n_seqs, uint32_t max_seq_len,
                                      float scale, void *partial_dev, void *workspace_dev,
                                      uint64_t workspace_bytes, void *stream);
BRC_API brc_status brc_decode_combine(int32_t device, const void *parts_dev, uint32_t n_parts,
                                      uint64_t part_stride_bytes, uint32_t n_seqs, uint32_t n_head,
                                      uint32_t head_dim, const float *gate_dev, uint32_t gate_head_stride,
                                      float *out_dev, void *stream);

/* Paged decode attention without a workspace argument and without any device
 * allocation (no counterpart in the reference).  Same inputs, outputs and
 * results as brc_paged_decode_attn; the split-KV partials go to a fixed array
 * that is part of the library image (4 MiB on every GPU that loads the library,
 * held until the process exits).  It is meant for callers that must not call
 * cudaMalloc: an engine whose arena took the whole HBM budget at start-up, or a
 * decode loop that cannot accept the device-wide synchronisation cudaMalloc
 * implies.
 *   - Limit: the batch must fit the array (about 100 sequences at 2 kv heads on a
 *     148-SM GPU); a larger batch is refused with BRC_ERR_CAPACITY and a message
 *     that names the limit.  Use the workspace variant for those.
 *   - The first call on each device looks up the array's device address (a
 *     host-side query, no allocation).  Make that first call outside any stream
 *     capture.
 *   - All calls on a device share the one array and it keeps whatever the last
 *     call left there; nothing in it needs to start at zero.  Two calls that run
 *     at the same time on one GPU would overwrite each other's partials.  Calls
 *     on ONE pool cannot overlap (see the workspace note above); calls on
 *     different pools of one GPU can: issue those on one stream, or serialise
 *     them. */
BRC_API brc_status brc_paged_decode_attn_static(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype,
                                                uint32_t n_head, const float *gate_dev, uint32_t gate_head_stride,
                                                const uint32_t *block_tables_dev, uint32_t table_stride,
                                                const uint32_t *seq_lens_dev, uint32_t n_seqs, uint32_t max_seq_len,
                                                float scale, float *out_dev, void *stream);

/* ---------------------------------------------------------------- split-KV across GPUs
 * One long sequence whose cells are split into contiguous, page-aligned ranges
 * over the GPUs of one box (rank r holds range r in its own pool).  No
 * counterpart in the reference, whose split-K partials stay on one device
 * (crates/breccia-kernels/src/qsa/mod.rs:1491-1521); the merge rule is the one
 * its reduce shader applies to chunks (qsa_attn_apply_reduce.comp:25-42),
 * extended by the running max.
 *
 * A brc_comm is one rank's end of the exchange: a receive buffer in this rank's
 * HBM with one slot per source rank (and four banks, so that ranks may be a
 * call apart; the separate exchange kernel also keeps release flags there).
 * Peers map it either through CUDA IPC (one
 * process per GPU: pass the 64-byte handles of all ranks, in rank order, to
 * brc_comm_connect_ipc; how they travel between processes is the caller's
 * business) or directly (one process driving several GPUs:
 * brc_comm_connect_local with the handles of all ranks).
 *
 * brc_splitkv_attend = ONE launch of the split-KV attention kernel over this
 * rank's cells in which the exchange rides along: the CTAs that merge a
 * (sequence, kv-head group) unit store its merged partial (16 512 bytes per
 * sequence at 16 heads of 256) into this rank's slot of every rank's receive
 * buffer with ordinary global stores over NVLink.  There are no flags and no
 * fences on that path: an empty slot holds the word 0xFFFFFFFF throughout, and
 * the thread that needs a 16-byte segment polls that very segment in every
 * rank's slot (time limit, default 1 s: on expiry the segment of the output is
 * left untouched and brc_pool_check reports BRC_ERR_TIMEOUT), merges, writes
 * the output and empties the slot again.  Every rank computes the same output.
 * All ranks must make the same sequence of calls with the same n_seqs /
 * n_layers.  No load ever targets peer memory and nothing is multicast.  The
 * workspace must hold the partial slots of the whole call
 * (brc_decode_workspace_bytes() per layer); at most 64 layers and 2048
 * (sequence, kv-head group) units per call.  After a BRC_ERR_TIMEOUT the
 * receive buffers may hold what arrived too late: every rank calls
 * brc_comm_reset (which empties them and restarts the call count) before the
 * group exchanges again.
 * brc_splitkv_exchange_combine is the exchange alone, as a kernel of its own,
 * for a partial the caller already holds (partial_dev NULL = the comm's own
 * buffer). */
#define BRC_IPC_HANDLE_BYTES 64
BRC_API brc_status brc_comm_create(brc_pool *pool, uint32_t world, uint32_t rank, uint32_t max_seqs,
                                   uint32_t n_head, brc_comm **out);
BRC_API brc_status brc_comm_ipc_handle(brc_comm *comm, void *handle_out64);
BRC_API brc_status brc_comm_connect_ipc(brc_comm *comm, const void *handles, uint32_t n_handles);
BRC_API brc_status brc_comm_connect_local(brc_comm *comm, brc_comm *const *comms, uint32_t n_comms);
BRC_API brc_status brc_comm_set_wait_ms(brc_comm *comm, uint32_t ms);
BRC_API brc_status brc_comm_reset(brc_comm *comm, void *stream);
BRC_API brc_status brc_comm_destroy(brc_comm *comm);
BRC_API brc_status brc_splitkv_exchange_combine(brc_comm *comm, const void *partial_dev, uint32_t n_seqs,
                                                const float *gate_dev, uint32_t gate_head_stride,
                                                float *out_dev, void *stream);
BRC_API brc_status brc_splitkv_attend(brc_comm *comm, uint32_t layer, const void *q_dev, int32_t q_dtype,
                                      const float *gate_dev, uint32_t gate_head_stride,
                                      const uint32_t *block_tables_dev, uint32_t table_stride,
                                      const uint32_t *seq_lens_dev, uint32_t n_seqs, uint32_t max_seq_len,
                                      float scale, float *out_dev, void *workspace_dev,
                                      uint64_t workspace_bytes, void *stream);
/* ---------------------------------------------------------------- attention over selected blocks
 * The reference's sparse form of Qsa::attend + Qsa::apply: per query row a list
 * of selected 4-cell blocks, `ids [rows][max_ids]` (ascending) with `counts
 * [rows]` entries in use; slot r * 4 + k names cell ids[r] * 4 + k, and cells
 * beyond the row's own position are masked (crates/breccia-kernels/src/qsa/
 * mod.rs:620-625, 1382-1580; qsa_attn_scores.comp:8-19, 62-118;
 * qsa_attn_apply.comp:85-140; CPU statement: cpu::attend over cpu::cells_of,
 * qsa/cpu.rs:197-257).  The lists are taken as the reference's top-k stage
 * produces them (here: brc_idx_score + brc_topk_blocks).
 * Rows are grouped by sequence: row r belongs to sequence r / rows_per_seq and
 * sits at position pos0[sequence] + r % rows_per_seq (T = 1 decode:
 * rows_per_seq = 1; speculative verify or prefill rows: > 1, causal per row).
 * q [rows][n_head][head_dim] f32 or f16; out [rows][n_head][head_dim] f32;
 * gate as in brc_paged_decode_attn.  Any n_head that divides over the kv heads
 * is accepted (no 8-heads-per-kv-head limit here).  A row whose lists select
 * no live cell yields zeros.  No workspace. */
BRC_API brc_status brc_paged_sparse_attn(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype,
                                         uint32_t n_head, const float *gate_dev, uint32_t gate_head_stride,
                                         const uint32_t *block_tables_dev, uint32_t table_stride,
                                         const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t rows_per_seq,
                                         const uint32_t *ids_dev, uint32_t max_ids, const uint32_t *counts_dev,
                                         uint32_t max_pos_end, float scale, float *out_dev, void *stream);

/* ---------------------------------------------------------------- query / key preparation + append
 * The steps Qsa::forward runs between the projections and the cache
 * (crates/breccia-kernels/src/qsa/mod.rs:1607-1617), five dispatches there, one
 * launch here:
 *   q_norm   per-head RMSNorm of the query half of each head's `q | gate` block
 *            (qsa_q_norm.comp:37-71; q_head_stride = 512 in the reference,
 *            = head_dim when the projection carries no gate half)
 *   k_norm   per-kv-head RMSNorm of k_cur (Qsa::k_norm, qsa/mod.rs:1051-1058)
 *   rope_q / rope_k   partial NEOX rotary, pairs (j, j + n_rot/2), (cos, sin) from
 *            the caller's table [max_pos][n_rot/2][2] f32 built as
 *            ops/cpu.rs:103-117 builds it; the position of token t of sequence s
 *            is pos0[s] + t, clamped into the table (ops_rope.comp:62-95)
 *   kv_append   normalised + rotated K and plain V to cells pos0[s] + t through
 *            the block table, binary16 by the pool's rule (qsa_kv_append.comp:137-161)
 * q_out [n_seqs * tokens_per_seq][n_head][head_dim] (f32 or f16) is what the
 * attention entry points take as their query.  k_cur / v_cur are not modified
 * (the reference normalises and rotates k_cur in place).  Refuses, on the host,
 * writes past the block table with the reference's wording. */
BRC_API brc_status brc_qk_prepare_append(brc_pool *pool, uint32_t layer, const float *q_full_dev,
                                         uint32_t q_head_stride, uint32_t n_head, const float *k_cur_dev,
                                         const float *v_cur_dev, const float *q_gamma_dev,
                                         const float *k_gamma_dev, float eps, const float *rope_table_dev,
                                         uint32_t n_rot, uint32_t max_pos, const uint32_t *block_tables_dev,
                                         uint32_t table_stride, const uint32_t *pos0_dev, uint32_t n_seqs,
                                         uint32_t tokens_per_seq, uint32_t max_pos_end, void *q_out_dev,
                                         int32_t q_out_dtype, void *stream);

/* ---------------------------------------------------------------- page files
 * The reference's state dump (crates/breccia-engine/src/graph.rs:2179-2231,
 * BRECCIA_DUMP_STATE): the first ceil((pos + 1) / 16) pages of a block's K pool
 * and V pool as raw device bytes, <dir>/p<pos:06>-b<block:02>-qsa_k.bin and
 * ...-qsa_v.bin.  Its page table is the identity; here the pages are named by
 * the sequence's block table (HOST array), so the files hold the same bytes the
 * reference writes for the same cache contents.  brc_state_load fills the pages
 * the table names from such a file pair (a persisted prefix).  Lab facility, as
 * in the reference: both calls synchronise `stream`.  The directory must exist. */
BRC_API brc_status brc_state_dump(brc_pool *pool, uint32_t layer, const uint32_t *block_table_host,
                                  uint32_t table_len, uint32_t pos, uint32_t block, const char *dir,
                                  void *stream);
BRC_API brc_status brc_state_load(brc_pool *pool, uint32_t layer, const uint32_t *block_table_host,
                                  uint32_t table_len, uint32_t pos, uint32_t block, const char *dir,
                                  void *stream);

/* One decode token over `n_layers` layers whose attention calls do not depend on
 * one another (the counterpart of brc_decode_step for the split-KV case, append
 * excluded): ONE launch whose flat work list runs over (layer, sequence, kv-head
 * group, page), cut into equal shares per SM, so launch ramp and tail are paid
 * once per token and the exchange of all layers (see brc_splitkv_attend) is one
 * round of stores at the end of the launch.  `workspace_bytes` must be at least n_layers
 * times brc_decode_workspace_bytes(); the comm must have been created with
 * max_seqs >= n_layers * n_seqs.  q is [n_layers] arrays `q_layer_stride_bytes`
 * apart; out is [n_layers][n_seqs][n_head][head_dim] f32, contiguous; gate
 * (nullable) is addressed as gate[row * gate_head_stride + d] with row = (layer,
 * sequence, head) in that order. */
BRC_API brc_status brc_splitkv_step(brc_comm *comm, uint32_t layer0, uint32_t n_layers, const void *q_dev,
                                    int32_t q_dtype, uint64_t q_layer_stride_bytes, const float *gate_dev,
                                    uint32_t gate_head_stride, const uint32_t *block_tables_dev,
                                    uint32_t table_stride, const uint32_t *seq_lens_dev, uint32_t n_seqs,
                                    uint32_t max_seq_len, float scale, float *out_dev, void *workspace_dev,
                                    uint64_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------- one decode step over layers
 * The composition the reference performs per attention layer in Qsa::forward
 * (crates/breccia-kernels/src/qsa/mod.rs:1587-1645: kv_append -> attend ->
 * apply) and the engine repeats for its 12 attention layers
 * (crates/breccia-engine/src/graph.rs:5899-5966), for a batch of sequences:
 *   pos0[s] = seq_lens[s]; seq_lens[s] += 1                (on the device)
 *   for layer in layer0 .. layer0+n_layers:
 *       append k_new/v_new[layer][s] at cell pos0[s];  out[layer] = decode attention
 * q / k_new / v_new / gate / out are per-layer arrays laid `*_layer_stride_bytes`
 * apart ([n_seqs][n_head][head_dim] and [n_seqs][n_kv_head*head_dim]).
 * `max_seq_len_after` bounds seq_lens AFTER the increment.
 * The append is carried out by the attention kernel itself (the CTA about to
 * stream the page of a sequence's newest cell writes that cell first), and the
 * layers of a step do not depend on one another, so a step is one small kernel
 * plus ONE attention launch whose flat work list runs over (layer, sequence,
 * kv-head group, page) when `workspace_bytes` is at least n_layers times
 * brc_decode_workspace_bytes() (up to 64 layers per launch).  With a smaller
 * workspace the layers go in as many launches as it takes, one after another;
 * results agree to rounding (the launches cut their shares differently).  A
 * sequence whose new length exceeds `max_seq_len_after` is reported through
 * brc_pool_check, attended up to the bound, and gets no cell appended. */
BRC_API brc_status brc_decode_step(brc_pool *pool, uint32_t layer0, uint32_t n_layers,
                                   const uint32_t *block_tables_dev, uint32_t table_stride, uint32_t *seq_lens_dev,
                                   uint32_t *pos0_dev, uint32_t n_seqs, uint32_t max_seq_len_after, const void *q_dev,
                                   int32_t q_dtype, uint64_t q_layer_stride_bytes, uint32_t n_head,
                                   const void *k_new_dev, const void *v_new_dev, int32_t kv_dtype,
                                   uint64_t kv_layer_stride_bytes, const float *gate_dev, uint32_t gate_head_stride,
                                   uint64_t gate_layer_stride_bytes, float scale, float *out_dev,
                                   uint64_t out_layer_stride_bytes, void *workspace_dev, uint64_t workspace_bytes,
                                   void *stream);

/* Layers [first, first + count) of the step brc_decode_step would run with the same
 * remaining arguments (every pointer and stride is the whole step's).  The part with
 * first == 0 advances the positions, so the parts of one step go to one stream, that
 * part first.  For a caller whose activations arrive from the host layer by layer
 * (the engine records its layers in order, crates/breccia-engine/src/graph.rs:5899-5966):
 * it can upload the next layers' q / k / v and download the finished layers' output
 * on other streams while this part computes. */
BRC_API brc_status brc_decode_step_part(brc_pool *pool, uint32_t layer0, uint32_t n_layers, uint32_t first,
                                        uint32_t count, const uint32_t *block_tables_dev, uint32_t table_stride,
                                        uint32_t *seq_lens_dev, uint32_t *pos0_dev, uint32_t n_seqs,
                                        uint32_t max_seq_len_after, const void *q_dev, int32_t q_dtype,
                                        uint64_t q_layer_stride_bytes, uint32_t n_head, const void *k_new_dev,
                                        const void *v_new_dev, int32_t kv_dtype, uint64_t kv_layer_stride_bytes,
                                        const float *gate_dev, uint32_t gate_head_stride,
                                        uint64_t gate_layer_stride_bytes, float scale, float *out_dev,
                                        uint64_t out_layer_stride_bytes, void *workspace_dev,
                                        uint64_t workspace_bytes, void *stream);

/* The same step for a caller whose activations live in HOST memory:
 * q_host [n_layers][n_seqs][n_head][head_dim] (q_dtype), k_new_host / v_new_host
 * [n_layers][n_seqs][n_kv_head*head_dim] (kv_dtype), out_host
 * [n_layers][n_seqs][n_head][head_dim] f32, all contiguous.
 *   Pinned buffers (addressable from the device) are used in place: the kernels
 * read q / k / v over PCIe as they reach each (layer, sequence) and store the output
 * straight into out_host, so the step's bytes cross the link while the attention
 * runs, nothing is staged and `staging_dev` may be NULL.  (The three inputs are
 * taken in place together or not at all.)
 *   Pageable buffers, or BRC_STEP_HOST_UPLOAD / BRC_STEP_HOST_DOWNLOAD in `flags`,
 * go through `staging_dev` (256-byte aligned, at least
 * brc_decode_step_host_staging_bytes(); it belongs to the call while it runs): the
 * layers go in `parts` groups (1..8, clamped to n_layers), uploads run ahead on a
 * stream of the pool's own and each group's kernels go to `stream`
 * (brc_decode_step_part); a staged output leaves group by group on a third stream
 * while the next group computes.
 *   Returns when out_host is complete; `stream` is ordered after everything the call
 * issued.  Positions, block tables and the workspace are device-resident as for
 * brc_decode_step. */
BRC_API brc_status brc_decode_step_host_staging_bytes(const brc_pool *pool, uint32_t n_layers, uint32_t n_seqs,
                                                      uint32_t n_head, int32_t q_dtype, int32_t kv_dtype,
                                                      uint64_t *out_bytes);
#define BRC_STEP_HOST_DOWNLOAD 1u /* flags: stage the output on the device and copy it down even when out_host is pinned */
#define BRC_STEP_HOST_UPLOAD 2u   /* flags: copy q / k / v to the device first even when they are pinned */
BRC_API brc_status brc_decode_step_host(brc_pool *pool, uint32_t layer0, uint32_t n_layers, uint32_t parts, uint32_t flags,
                                        const uint32_t *block_tables_dev, uint32_t table_stride,
                                        uint32_t *seq_lens_dev, uint32_t *pos0_dev, uint32_t n_seqs,
                                        uint32_t max_seq_len_after, const void *q_host, int32_t q_dtype,
                                        uint32_t n_head, const void *k_new_host, const void *v_new_host,
                                        int32_t kv_dtype, float scale, float *out_host, void *staging_dev,
                                        uint64_t staging_bytes, void *workspace_dev, uint64_t workspace_bytes,
                                        void *stream);

/* ---------------------------------------------------------------- indexer: pooled-key cache and block scores
 * Replaces shaders/qsa_idx_pool.comp, qsa_idx_tail.comp and qsa_idx_score.comp, driven as Qsa::idx_pool /
 * idx_tail / idx_score (crates/breccia-kernels/src/qsa/mod.rs:1168-1262) in the order of Qsa::forward
 * (:1618-1630): pool, then tail, then score, then brc_topk_blocks.  CPU statements: cpu::pool_keys and
 * cpu::indexer_score (qsa/cpu.rs:97-121, 159-195).  The reference holds one indexer state per sequence;
 * here the state arrays have a leading sequence dimension (caller-owned device memory, f32):
 *   pooled [n_seqs][max_blocks][idx_dim]   one pooled key per COMPLETED 4-cell block
 *   tail   [n_seqs][idx_block - 1][idx_dim]  raw keys of the block being filled
 * and one call serves a batch whose sequences each bring `tokens_per_seq` raw keys
 * raw [n_seqs][tokens_per_seq][idx_dim] at positions pos0[s] .. .
 *   pool : for every block this call completes, pooled[s][b] = rope(rmsnorm(mean(raw keys of cells
 *          4b..4b+3), gamma, eps), position 4b): mean over the RAW keys, NEOX pairs (j, j + n_rot/2) from
 *          the caller's (cos, sin) table [max_pos][n_rot/2][2], rotated at the block's first cell.  Cells
 *          before pos0 come from `tail` (call it BEFORE brc_idx_tail, as the reference does).  Refuses,
 *          with the reference's wording, a call whose blocks would not fit max_blocks (`max_pos_end` is
 *          the caller's bound on pos0[s] + tokens_per_seq, checked on the device too).
 *   tail : stores the raw keys of the call's last, incomplete block (slot = cell % 4 < 3).
 *   score: scores[row][b] = scale * sum_h relu(q[row][h] . pooled[s][b]) for b < n_blocks, row = s *
 *          rows_per_seq + t at position pos0[s] + t; a block whose LAST cell lies beyond the row's
 *          position gets -1e30, which brc_topk_blocks never selects (the shader's rule; the CPU
 *          statement masks on the first cell, the two agree on every block a row fully sees).
 *          q [rows][idx_n_head][idx_dim], idx_n_head <= 8, scale = 1/sqrt(idx_dim) in the reference.
 * Built for idx_dim 128 and idx_block 4 (the reference's constants). */
BRC_API brc_status brc_idx_pool(brc_pool *pool, const float *raw_dev, const float *tail_dev, const float *gamma_dev,
                                const float *rope_table_dev, uint32_t n_rot, uint32_t max_pos, float eps,
                                const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t tokens_per_seq, uint32_t max_pos_end,
                                uint32_t idx_dim, uint32_t idx_block, float *pooled_dev, uint32_t max_blocks, void *stream);
BRC_API brc_status brc_idx_tail(brc_pool *pool, const float *raw_dev, const uint32_t *pos0_dev, uint32_t n_seqs,
                                uint32_t tokens_per_seq, uint32_t idx_dim, uint32_t idx_block, float *tail_dev, void *stream);
BRC_API brc_status brc_idx_score(brc_pool *pool, const float *q_dev, uint32_t idx_n_head, const float *pooled_dev,
                                 uint32_t max_blocks, const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t rows_per_seq,
                                 uint32_t n_blocks, uint32_t idx_dim, uint32_t idx_block, float scale,
                                 float *scores_out_dev, void *stream);

/* ---------------------------------------------------------------- top-k block selection
 * Replaces shaders/qsa_topk.comp (CPU statement cpu::topk_blocks, qsa/cpu.rs:129-151): turns a row's
 * indexer scores into the `ids` / `counts` lists brc_paged_sparse_attn walks.  Per row (row = sequence *
 * rows_per_seq + t, position pos0[sequence] + t): the min(n_blocks, topk_blocks) highest scores in
 * DESCENDING score order, equal scores towards the LOWER block index; a score <= -1e29 or NaN marks a
 * block the row must not see and is never selected; then the row's own block (position / 4) is
 * appended unless already selected.  `dense` != 0 (needs n_blocks <= topk_blocks): every block up to the
 * row's own, ascending, scores not read.  scores [rows][n_blocks] f32 are left untouched (the
 * reference's shader destroys them); ids_out [rows][max_ids], max_ids >= min(n_blocks, topk_blocks) + 1;
 * counts_out [rows].  topk_blocks <= 1024 (the reference selects 512); any n_blocks. */
BRC_API brc_status brc_topk_blocks(brc_pool *pool, const float *scores_dev, uint32_t n_seqs, uint32_t rows_per_seq,
                                   uint32_t n_blocks, uint32_t topk_blocks, uint32_t max_ids,
                                   const uint32_t *pos0_dev, int32_t dense, uint32_t *ids_out_dev,
                                   uint32_t *counts_out_dev, void *stream);

/* ---------------------------------------------------------------- chunked-prefill attention (tensor cores)
 * Replaces the reference's T >= 16 path: qsa_attn_scores_gqa.comp + ops_softmax.comp
 * + qsa_attn_apply_gqa.comp, tiled from Qsa::forward
 * (crates/breccia-kernels/src/qsa/mod.rs:1631-1641; GQA_MIN_TOKENS, ATTN_TILE
 * :116-135).  Every sequence brings `chunk_len` query rows at positions
 * pos0_dev[s] .. pos0_dev[s] + chunk_len - 1; all of the chunk's cells must already
 * be in the cache (the reference appends before it attends, qsa/mod.rs:1617->1638);
 * row t sees cells <= pos0 + t.  Sequences may share prefix pages.
 *   q_dev    [n_seqs][chunk_len][n_head][head_dim], f16 bits or f32 (rounded to f16 for the
 *            tensor cores); out_dev same shape, f32; gate as in brc_paged_decode_attn with
 *            rows (s, t, h).
 *   max_pos_end  caller's bound on pos0[s] + chunk_len; refused if > table_stride*page_tokens.
 * head_dim 256; up to 8 query heads per kv head share a tile of 16 tokens, more (up to 32; the
 * reference model has 12) take floor(128 / heads) tokens per tile.  tcgen05.mma with accumulators in
 * TMEM; K/V pages gathered through the block table. */
BRC_API brc_status brc_paged_prefill_attn(brc_pool *pool, uint32_t layer, const void *q_dev, int32_t q_dtype,
                                          uint32_t n_head, const float *gate_dev, uint32_t gate_head_stride,
                                          const uint32_t *block_tables_dev, uint32_t table_stride,
                                          const uint32_t *pos0_dev, uint32_t n_seqs, uint32_t chunk_len,
                                          uint32_t max_pos_end, float scale, float *out_dev, void *stream);

/* ---------------------------------------------------------------- radix prefix tree (host side)
 * No counterpart in the reference ("Radix/prompt prefix sharing | open",
 * docs/BRIEF.md:287); built to its design note: 16-token blocks identified by
 * their tokens and everything before them, refcounted, with a free queue
 * (docs/reference-engines/02-kv-and-context.md:543-581).  An edge is one full
 * page of token ids; a node holds one reference on the page caching that page
 * of the prefix in every layer.
 *   match  : longest run of full pages of `tokens` present in the tree; each
 *            returned page gets one more reference, owned by the caller.
 *   insert : adds missing nodes for the full pages of `tokens` backed by
 *            `pages`; the tree takes its own reference on the pages it adopts
 *            (`*out_n_new` of them); existing nodes keep their page.
 *   evict  : drops up to n least-recently-used leaves whose page only the tree
 *            holds, returning those pages to the allocator.
 *   release: gives back references `match` handed out (the same as
 *            brc_pages_release on the tree's pool).
 * A page the tree holds is marked in the pool: brc_tier_lru never offers it and
 * brc_tier_demote refuses it, whatever its reference count. */
BRC_API brc_status brc_radix_create(brc_pool *pool, brc_radix **out);
BRC_API brc_status brc_radix_destroy(brc_radix *radix);
BRC_API brc_status brc_radix_match(brc_radix *radix, const uint32_t *tokens, uint32_t n_tokens, uint32_t *out_pages,
                                   uint32_t max_pages, uint32_t *out_n_pages);
BRC_API brc_status brc_radix_insert(brc_radix *radix, const uint32_t *tokens, uint32_t n_tokens, const uint32_t *pages,
                                    uint32_t n_pages, uint32_t *out_n_new);
BRC_API brc_status brc_radix_evict(brc_radix *radix, uint32_t n_pages, uint32_t *out_n_evicted);
BRC_API brc_status brc_radix_release(brc_radix *radix, const uint32_t *pages, uint32_t n_pages);
/* A 64-bit tag per full page of a prompt, the tag of page i a hash of all tokens
 * of pages 0 .. i ("blocks identified by their tokens and everything before
 * them", the design note's hash granularity).  The same prompt gives the same
 * tags in every process: they are the keys under which prefix pages are spilled
 * to a cold store (brc_cold_spill) and found again later (brc_cold_find) - the
 * disk-persisted prefix cache of
 * docs/reference-engines/02-kv-and-context.md:536-548, 617-626.  Never zero. */
BRC_API brc_status brc_radix_prefix_tags(const uint32_t *tokens, uint32_t n_tokens, uint32_t page_tokens,
                                         uint64_t *out_tags, uint32_t capacity, uint32_t *out_n);
BRC_API brc_status brc_radix_stats(brc_radix *radix, uint64_t *out_nodes, uint64_t *out_hit_pages,
                                   uint64_t *out_miss_pages, uint64_t *out_evictions);

/* ---------------------------------------------------------------- HBM <-> pinned host tiering
 * No KV tiering exists in the reference (docs/plan/BRECCIA-PLAN.md:52-56); the
 * nearest code is its H2D transfer ring (crates/breccia-vk/src/transfer.rs:
 * 120-138, 247-369: fixed slots, pinned staging, arrive/release ordering,
 * RingStats) and the rules of its design note: whole pages only, a page lives in
 * exactly one tier, all layers move together, promotion is asynchronous
 * (docs/reference-engines/02-kv-and-context.md:543-581, 617-626).
 *   demote : pages with exactly one holder (not a radix tree; no id twice -
 *            checked before anything is queued) go HBM -> host slots on the tier's
 *            side stream (ordered after `after_stream`'s work so far, if given);
 *            the HBM pages return to the allocator, `out_slots` names the copies.
 *   promote: host slots -> freshly allocated HBM pages (`out_page_ids`), slots freed.
 *   fence  : `stream` waits for every tier copy issued so far (call it before a
 *            stream reads promoted pages or writes pages freed by a demotion).
 *   touch / lru: last-use stamps of resident pages and the n least recently used
 *            single-holder pages, for the caller's demotion policy. */
BRC_API brc_status brc_tier_create(brc_pool *pool, uint32_t host_pages, brc_tier **out);
BRC_API brc_status brc_tier_destroy(brc_tier *tier);
BRC_API brc_status brc_tier_demote(brc_tier *tier, const uint32_t *page_ids, uint32_t n, uint32_t *out_slots,
                                   void *after_stream);
BRC_API brc_status brc_tier_promote(brc_tier *tier, const uint32_t *slots, uint32_t n, uint32_t *out_page_ids);
BRC_API brc_status brc_tier_fence(brc_tier *tier, void *stream);
BRC_API brc_status brc_tier_sync(brc_tier *tier);
BRC_API brc_status brc_tier_touch(brc_tier *tier, const uint32_t *page_ids, uint32_t n);
BRC_API brc_status brc_tier_lru(brc_tier *tier, uint32_t n, uint32_t *out_page_ids, uint32_t *out_n);
BRC_API brc_status brc_tier_stats(brc_tier *tier, uint64_t *out_demoted_pages, uint64_t *out_promoted_pages,
                                  uint64_t *out_d2h_bytes, uint64_t *out_h2d_bytes, uint32_t *out_free_slots);

/* ---------------------------------------------------------------- cold store behind the host tier
 * A file of page records (NVMe in the design note: the third tier, and the disk-persisted prefix cache;
 * docs/reference-engines/02-kv-and-context.md:536-548, item 5 of :617-626; no code in the reference).  A
 * record is byte for byte a host slot of the tier (a page of every layer, K then V), so a page travels
 *     HBM --brc_tier_demote--> host slot --spill--> record --fetch--> host slot --brc_tier_promote--> HBM
 * unchanged.  Each record carries a caller-chosen 64-bit tag (for a cached prefix: a hash of the tokens up
 * to and including the page); tags are stored in the file, so another process can open it later and find
 * the pages again.
 *   open  : create != 0 makes (or truncates) `path` with n_slots records; create == 0 opens an existing
 *           store, refusing one written for another page geometry (n_slots ignored).
 *   spill : host slots -> free records (waits for the demotion that filled the slots), host slots freed.
 *   fetch : records -> free host slots, ready for brc_tier_promote; keep == 0 frees the records.
 *   find  : the record with this tag, or BRC_ERR_NOT_RESIDENT.
 * Synchronous file I/O on the calling thread. */
BRC_API brc_status brc_cold_open(brc_tier *tier, const char *path, uint32_t n_slots, int32_t create, brc_cold **out);
BRC_API brc_status brc_cold_close(brc_cold *cold);
BRC_API brc_status brc_cold_spill(brc_cold *cold, const uint32_t *host_slots, const uint64_t *tags, uint32_t n,
                                  uint32_t *out_cold_slots);
BRC_API brc_status brc_cold_fetch(brc_cold *cold, const uint32_t *cold_slots, uint32_t n, int32_t keep,
                                  uint32_t *out_host_slots);
BRC_API brc_status brc_cold_find(brc_cold *cold, uint64_t tag, uint32_t *out_cold_slot);
BRC_API brc_status brc_cold_stats(brc_cold *cold, uint32_t *out_used, uint32_t *out_total, uint64_t *out_bytes_written,
                                  uint64_t *out_bytes_read);

/* ---------------------------------------------------------------- per-stage GPU timers
 * Counterpart of the reference's BRECCIA_GPU_TIME probe and its stage ids
 * KV_APPEND / ATTN (crates/breccia-kernels/src/dispatch_batch.rs:453-512,
 * qsa/mod.rs:1600-1642).  While enabled, each kernel launch of a stage is
 * bracketed by CUDA events on the launching stream; brc_timing_read waits for
 * them, returns the number of launches and their summed device time since the
 * previous read, and clears the list.  Off by default (event records cost). */
#define BRC_STAGE_KV_APPEND 0
#define BRC_STAGE_ATTN_PARTIAL 1
#define BRC_STAGE_ATTN_COMBINE 2
#define BRC_STAGE_PAGE_COPY 3
#define BRC_STAGE_PAGE_GATHER 4
#define BRC_STAGE_PREFILL 5
BRC_API brc_status brc_timing_enable(brc_pool *pool, int32_t on);
BRC_API brc_status brc_timing_read(brc_pool *pool, int32_t stage, uint32_t *out_launches, double *out_total_ms);

#ifdef __cplusplus
}
#endif
#endif /* BRECCIA_KV_H */
