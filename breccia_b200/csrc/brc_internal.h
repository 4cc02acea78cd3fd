// Internal definitions shared by the translation units of libbreccia_kv.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <vector>

#include "breccia_kv.h"

// Bits of the device-side check word (brc_pool::status_dev).
#define BRC_DEV_BAD_PAGE 1u    // block-table entry >= n_pages
#define BRC_DEV_BAD_POS 2u     // position past the caller's bound
#define BRC_DEV_WAIT_LIMIT 4u  // a bounded mbarrier wait gave up
#define BRC_DEV_BAD_SHAPE 8u   // more work units than a kernel's table holds

// brc_pool::status_dev: 64 words of check state, then the decode kernels' per-unit arrival counters
// (ticket words of the units, never cleared by the kernels: every launch adds a fixed amount per unit).
#define BRC_STATUS_WORDS 64u
#define BRC_DONE_BANK_WORDS 2048u  // one ticket word per unit of a layer (2048 units at most)
#define BRC_DONE_BANKS 64u     // one bank per layer of a launch (a launch covers up to 64 layers)
#define BRC_DONE_WORDS (BRC_DONE_BANK_WORDS * BRC_DONE_BANKS)
#define BRC_STATUS_BYTES ((BRC_STATUS_WORDS + BRC_DONE_WORDS) * 4u)

// Split-KV across GPUs: ranks of one exchange group, and banks of a receive buffer (ranks may be a
// call apart, so a peer's next partial must not land on the one still being merged).
#define BRC_MAX_WORLD 16u
#define BRC_COMM_BANKS 4u

// Stage ids of the optional GPU timers are public (breccia_kv.h); this is their count.
#define BRC_STAGE_COUNT 6

struct brc_pool {
    int32_t device = -1;
    uint32_t n_layers = 0, n_kv_head = 0, head_dim = 0, page_tokens = 0, n_pages = 0;
    uint64_t half_page_bytes = 0;   // K (or V) bytes of one page of one layer
    uint64_t layer_bytes = 0;       // K (or V) bytes of one layer
    uint8_t *k_base = nullptr;      // [n_layers][n_pages][n_kv][page_tokens][head_dim] f16
    uint8_t *v_base = nullptr;      // same allocation as k_base, `layer_bytes * n_layers` further on
    // V page bodies: binary16 like K, or q8_0 (blocks of 32 values: one f32 scale + 32 signed bytes, 36 B;
    // row = head_dim / 32 blocks; rows in the same order as the binary16 layout)
    bool v_q8 = false;
    uint64_t v_layer_bytes = 0;     // V bytes of one layer: layer_bytes, or 9/16 of it for q8_0
    uint32_t *status_dev = nullptr; // device check word
    uint32_t *status_host = nullptr;  // pinned mirror
    uint32_t *ids_dev = nullptr;    // small staging for host-provided id lists
    uint32_t ids_cap = 0;
    int sm_count = 0;
    // TMA views of the whole K / V allocation: 2-D [rows][head_dim] f16, box
    // [page_tokens rows][64 columns], 128-byte swizzle.
    alignas(64) CUtensorMap tm_k;
    alignas(64) CUtensorMap tm_v;
    // 3-D view over both: (column, row, {K, V}); one box = a 64-column group of the K tile and of the V
    // tile of one page of one kv head.
    alignas(64) CUtensorMap tm_kv;
    alignas(64) CUtensorMap tm_kv2;  // same view, box of 2 * page_tokens rows (two kv heads); even n_kv_head only
    // 4-D views (column in a 64-column group, row, K|V, group): one box brings a whole page-unit, every column
    // group of its K and V rows, in ONE operation (opt-in: BRC_DECODE_STAGE_OP=1); stage_maps says whether the driver
    // accepted them
    alignas(64) CUtensorMap tm_kv_stage;
    alignas(64) CUtensorMap tm_kv2_stage;
    alignas(64) CUtensorMap tm_k_stage;    // q8_0 V pools: 3-D view of K alone (column, row, group), all K slabs of a page-unit in one box
    alignas(64) CUtensorMap tm_k2_stage;
    bool stage_maps = false;
    // q8_0 V pools: K alone as [rows][head_dim] f16 with a box of 2 * page_tokens rows (tm_k is the one-kv-head
    // box), and the V rows as [rows][head_dim / 32 * 9] 32-bit words (288 B at head_dim 256), unswizzled,
    // boxes of page_tokens and of 2 * page_tokens whole rows
    alignas(64) CUtensorMap tm_k2;
    alignas(64) CUtensorMap tm_v8;
    alignas(64) CUtensorMap tm_v8_2;
    bool has_tma = false;
    // decode attention: where every CTA's share of a launch begins (fractions x 2^32, device memory owned by the
    // library's per-device cache), from the streaming rates measured on this device; NULL = equal shares
    const uint32_t *cut_prefix = nullptr;
    std::vector<float> cut_rates;   // the rates behind it, relative to their mean (host copy, for reports)

    // per-stage GPU timers (off unless brc_timing_enable)
    bool timing = false;
    struct stage_events {
        std::vector<cudaEvent_t> begin, end;  // recorded pairs since the last read
        std::vector<cudaEvent_t> spare;       // reusable events
    } stages[BRC_STAGE_COUNT];

    // brc_decode_step_host: an upload and a download stream and one event pair per part, made on first use
    static constexpr uint32_t HOST_PARTS_MAX = 8;
    cudaStream_t host_up = nullptr, host_down = nullptr;
    cudaEvent_t host_uploaded[HOST_PARTS_MAX] = {}, host_computed[HOST_PARTS_MAX] = {};
    cudaEvent_t host_all_down = nullptr;

    // decode calls share the arrival counters above: the stream of the last one and an event recorded
    // behind it, so that a call on another stream is ordered after it
    cudaStream_t decode_stream = nullptr;
    bool decode_stream_set = false;
    cudaEvent_t decode_event = nullptr;

    // allocator
    mutable std::mutex mu;
    std::vector<uint32_t> refcount;
    std::vector<uint32_t> tree_refs;  // of those, references held by radix trees (a page whose only holder is a tree
                                      // is not "held by the caller": the tier neither offers nor demotes it)
    std::vector<uint32_t> free_list;  // LIFO
};

void brc_set_error(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
brc_status brc_fail(brc_status code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

#define BRC_CUDA(expr)                                                                           \
    do {                                                                                         \
        cudaError_t _e = (expr);                                                                 \
        if (_e != cudaSuccess)                                                                   \
            return brc_fail(BRC_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                            __FILE__, __LINE__);                                                 \
    } while (0)


// RAII: make the pool's device current for the duration of a call, restore after.
struct brc_device_guard {
    int prev = -1;
    bool ok = true;
    explicit brc_device_guard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; prev = -1; }
        if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~brc_device_guard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// Record a begin/end event pair around a launch when timing is on (no-ops otherwise).
void brc_stage_begin(brc_pool *pool, int stage, cudaStream_t s);
void brc_stage_end(brc_pool *pool, int stage, cudaStream_t s);

// Split-KV across GPUs, as the decode kernel needs it: where this rank's merged partials go and which
// flags announce them (comm.cu owns the buffers).
struct brc_push_args {
    uint32_t world = 1, rank = 0;
    uint8_t *peer_recv[BRC_MAX_WORLD] = {};   // receive buffers of all ranks as mapped here ([rank] = this rank's own)
    uint64_t slot_stride = 0, bank_stride = 0;
    uint64_t push_offset = 0;                 // byte offset, in a receive buffer, of the banks the decode launch stores into
    uint32_t unit_items = 0;                  // units those banks were sized for
    uint32_t *calls = nullptr;                // exchanges completed on this rank
    uint32_t *fin_ticket = nullptr;           // CTAs of the running launch that have finished
    uint64_t wait_ns = 0;
};

// Decode attention over `n_layers` layers of a batch in as few launches as the workspace allows (one,
// when it holds n_layers x brc_decode_workspace_bytes()).  Per-layer arrays lie `*_layer_stride_bytes`
// apart.  k_new / v_new non-NULL: the step's KV append rides in the kernel.  out_ml non-NULL: partial
// mode.  push with world > 1: merged partials go to the peers and the output comes from the cross-rank
// merge inside the same launch (decode_attn.cu).
struct brc_layers_args {
    uint32_t layer0 = 0, n_layers = 1;
    const void *q = nullptr;
    int32_t q_dtype = BRC_DTYPE_F16;
    uint64_t q_layer_stride_bytes = 0;
    uint32_t n_head = 0;
    const float *gate = nullptr;
    uint32_t gate_head_stride = 0;
    uint64_t gate_layer_stride_bytes = 0;
    const uint32_t *block_tables = nullptr;
    uint32_t table_stride = 0;
    const uint32_t *seq_lens = nullptr;
    uint32_t n_seqs = 0, max_seq_len = 0;
    float scale = 0.f;
    float *out = nullptr;
    uint64_t out_layer_stride_bytes = 0;
    float *out_ml = nullptr;
    uint64_t out_ml_layer_stride_bytes = 0;
    void *workspace = nullptr;
    uint64_t workspace_bytes = 0;
    const void *k_new = nullptr, *v_new = nullptr;
    int32_t kv_dtype = BRC_DTYPE_F32;
    uint64_t kv_layer_stride_bytes = 0;
    const brc_push_args *push = nullptr;
};
void brc_decode_calibrate(brc_pool *pool);
brc_status brc_decode_layers(brc_pool *pool, const char *who, const brc_layers_args &args, void *stream);
uint32_t brc_decode_kvb(const brc_pool *pool);   // kv heads that travel together in one unit (1 or 2)

static inline cudaStream_t brc_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }
