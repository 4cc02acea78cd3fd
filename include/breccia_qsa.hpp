// C++ host-side mirror of the reference's `qsa` operator surface over the C ABI of breccia_kv.h.
//
// The reference's host code is Rust (crates/breccia-kernels/src/qsa/mod.rs); this header restates its
// public types with the same names, argument meaning and error behaviour for callers written in a
// compiled language:
//   QsaState      qsa/mod.rs:294-311, ctor 399-535, reset 551-570, bytes 572, release 591-602
//   QsaWorkspace  qsa/mod.rs:606-650 (k_cur, v_cur, q, q_full, attn_out)
//   Qsa           qsa/mod.rs:746 (new), 928 (workspace), 1107 (kv_append), 1365 (topk_dense),
//                 1382 (attend), 1466 (apply)
// What differs, because the pool is shared by all sequences of a GPU: a QsaState is a block table
// over pages taken from a KvPool (the reference gives every state its own identity-mapped pool), and
// attend + apply are one kernel, so `attend` does the work and `apply` is a no-op kept for the call
// sites.  Errors: the reference returns anyhow::Result; here every failing call throws brc::Error
// carrying the status code and the library's message, which has the reference's wording for the
// refusals it shares (capacity check of kv_append, qsa/mod.rs:1108-1116).
//
// Device buffers are plain CUDA device pointers owned by the caller (`DeviceAlloc` is the caller's
// allocator; the library itself allocates nothing inside these calls).  Header-only; link with
// -lbreccia_kv.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "breccia_kv.h"

namespace brc {

struct Error : std::runtime_error {
    brc_status code;
    Error(brc_status c, const std::string &msg) : std::runtime_error(msg), code(c) {}
};

inline void check(brc_status rc) {
    if (rc != BRC_OK) throw Error(rc, brc_last_error());
}

// The caller's device allocator: alloc(bytes) -> device pointer (zero-filled), free(pointer).
struct DeviceAlloc {
    std::function<void *(size_t)> alloc;
    std::function<void(void *)> free;
    // host -> device copy of a small table (block tables, positions), ordered before later launches
    std::function<void(void *dst_dev, const void *src_host, size_t bytes)> upload;
};

constexpr uint32_t PAGE_CELLS = 16;   // qsa/mod.rs:114

// How V page bodies are stored (the reference's VLayout, qsa/mod.rs:245-290): binary16 like K, or q8_0 blocks
// of one f32 scale + 32 signed bytes (0.5625x the V bytes).  K is binary16 in both.
enum class VLayout : int32_t { F16 = BRC_V_F16, Q8_0 = BRC_V_Q8_0 };

class KvPool {
public:
    KvPool(int32_t device, uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim, uint32_t n_pages,
           VLayout v_layout = VLayout::F16) {
        if (v_layout == VLayout::Q8_0)
            check(brc_pool_create_q8v(device, n_layers, n_kv_head, head_dim, PAGE_CELLS, n_pages, &raw_));
        else
            check(brc_pool_create(device, n_layers, n_kv_head, head_dim, PAGE_CELLS, n_pages, &raw_));
        n_layers_ = n_layers, n_kv_head_ = n_kv_head, head_dim_ = head_dim, n_pages_ = n_pages;
    }
    VLayout v_layout() const {
        int32_t v = 0;
        check(brc_pool_v_layout(raw_, &v));
        return static_cast<VLayout>(v);
    }
    // bookkeeping only (allocator + refcounts, no device memory): schedulers and CPU tests
    static KvPool bookkeeping(uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim, uint32_t n_pages) {
        KvPool p;
        check(brc_pool_create_bookkeeping(n_layers, n_kv_head, head_dim, PAGE_CELLS, n_pages, &p.raw_));
        p.n_layers_ = n_layers, p.n_kv_head_ = n_kv_head, p.head_dim_ = head_dim, p.n_pages_ = n_pages;
        return p;
    }
    KvPool(KvPool &&o) noexcept { *this = std::move(o); }
    KvPool &operator=(KvPool &&o) noexcept {
        std::swap(raw_, o.raw_);
        n_layers_ = o.n_layers_, n_kv_head_ = o.n_kv_head_, head_dim_ = o.head_dim_, n_pages_ = o.n_pages_;
        return *this;
    }
    KvPool(const KvPool &) = delete;
    KvPool &operator=(const KvPool &) = delete;
    ~KvPool() {
        if (raw_) brc_pool_destroy(raw_);
    }
    brc_pool *raw() const { return raw_; }
    uint32_t n_layers() const { return n_layers_; }
    uint32_t n_kv_head() const { return n_kv_head_; }
    uint32_t head_dim() const { return head_dim_; }
    uint32_t n_pages() const { return n_pages_; }
    uint64_t bytes() const {
        uint64_t b = 0;
        check(brc_pool_bytes(raw_, &b));
        return b;
    }
    std::vector<uint32_t> alloc(uint32_t n) {
        std::vector<uint32_t> ids(n);
        check(brc_pages_alloc(raw_, n, ids.data()));
        return ids;
    }
    void retain(const std::vector<uint32_t> &ids) { check(brc_pages_retain(raw_, ids.data(), (uint32_t)ids.size())); }
    void release(const std::vector<uint32_t> &ids) { check(brc_pages_release(raw_, ids.data(), (uint32_t)ids.size())); }
    uint32_t refcount(uint32_t page) const {
        uint32_t rc = 0;
        check(brc_page_refcount(raw_, page, &rc));
        return rc;
    }
    uint32_t free_pages() const {
        uint32_t n = 0;
        check(brc_pages_free_count(raw_, &n));
        return n;
    }
    // Reports what the kernels' own bounds checks and bounded waits recorded since the last call.
    void check_device(void *stream = nullptr) { check(brc_pool_check(raw_, stream)); }

private:
    KvPool() = default;
    brc_pool *raw_ = nullptr;
    uint32_t n_layers_ = 0, n_kv_head_ = 0, head_dim_ = 0, n_pages_ = 0;
};

// Per-layer, per-sequence cache state: a block table over pages of the shared pool.
class QsaState {
public:
    // QsaState::new(gpu, capacity_cells, max_pos): pages for capacity_cells come from the pool.
    QsaState(KvPool &pool, const DeviceAlloc &dev, uint32_t layer, size_t capacity_cells)
        : pool_(&pool), dev_(dev), layer_(layer),
          capacity_cells_((capacity_cells + PAGE_CELLS - 1) / PAGE_CELLS * PAGE_CELLS) {   // whole pages, as the reference rounds
        table_ = pool.alloc((uint32_t)(capacity_cells_ / PAGE_CELLS));
        owns_pages_ = true;
        upload_table();
    }
    // A state over an existing block table (prefix reuse, forks): the pages are retained, not allocated.
    QsaState(KvPool &pool, const DeviceAlloc &dev, uint32_t layer, std::vector<uint32_t> block_table)
        : pool_(&pool), dev_(dev), layer_(layer), capacity_cells_(block_table.size() * PAGE_CELLS), table_(std::move(block_table)) {
        pool.retain(table_);
        owns_pages_ = true;
        upload_table();
    }
    QsaState(const QsaState &) = delete;
    QsaState &operator=(const QsaState &) = delete;
    ~QsaState() { release(); }

    // The reference re-uploads zeros and the identity table; here cells past the length are never read,
    // so there is nothing to clear.
    void reset() {}
    size_t bytes() const { return table_.size() * 2ull * pool_->n_kv_head() * PAGE_CELLS * pool_->head_dim() * 2ull; }
    void release() {
        if (owns_pages_) {
            pool_->release(table_);
            owns_pages_ = false;
        }
        if (table_dev_) {
            dev_.free(table_dev_);
            table_dev_ = nullptr;
        }
    }
    size_t capacity_cells() const { return capacity_cells_; }
    uint32_t layer() const { return layer_; }
    const std::vector<uint32_t> &block_table() const { return table_; }
    const uint32_t *block_table_dev() const { return table_dev_; }
    KvPool &pool() const { return *pool_; }

private:
    void upload_table() {
        if (!dev_.alloc) return;   // bookkeeping-only use
        table_dev_ = static_cast<uint32_t *>(dev_.alloc(table_.size() * 4));
        dev_.upload(table_dev_, table_.data(), table_.size() * 4);
    }
    KvPool *pool_;
    DeviceAlloc dev_;
    uint32_t layer_;
    size_t capacity_cells_;
    std::vector<uint32_t> table_;
    uint32_t *table_dev_ = nullptr;
    bool owns_pages_ = false;
};

// Device buffers of one call: `tokens` rows.  Fields as in the reference (qsa/mod.rs:606-650).
struct QsaWorkspace {
    size_t tokens = 0;
    float *k_cur = nullptr;      // [tokens, n_kv * hd] f32
    float *v_cur = nullptr;      // [tokens, n_kv * hd] f32
    float *q = nullptr;          // [tokens, n_head, hd] f32
    float *q_full = nullptr;     // [tokens, n_head * 2 * hd] f32: per head, query half then gate half
    float *attn_out = nullptr;   // [tokens, n_head, hd] f32
    uint32_t *pos_dev = nullptr; // [tokens + 1]: pos0, then per-row lengths
    uint32_t *tables_dev = nullptr;  // [tokens][pages of the state]: every row attends through the same table
    size_t tables_len = 0;       // entries per row tables_dev was sized for
    void *scratch = nullptr;     // split-KV partials
    uint64_t scratch_bytes = 0;
    bool use_gate = false;       // read the gate from q_full (in place, as qsa_attn_apply_reduce.comp:39-41)
};

class Qsa {
public:
    Qsa(KvPool &pool, const DeviceAlloc &dev, uint32_t n_head, void *stream = nullptr)
        : pool_(&pool), dev_(dev), n_head_(n_head), stream_(stream), scale_(1.0f / std::sqrt((float)pool.head_dim())) {}

    QsaWorkspace workspace(size_t tokens) const {
        QsaWorkspace ws;
        ws.tokens = tokens;
        const size_t kv = (size_t)pool_->n_kv_head() * pool_->head_dim(), qh = (size_t)n_head_ * pool_->head_dim();
        ws.k_cur = static_cast<float *>(dev_.alloc(tokens * kv * 4));
        ws.v_cur = static_cast<float *>(dev_.alloc(tokens * kv * 4));
        ws.q = static_cast<float *>(dev_.alloc(tokens * qh * 4));
        ws.q_full = static_cast<float *>(dev_.alloc(tokens * qh * 2 * 4));
        ws.attn_out = static_cast<float *>(dev_.alloc(tokens * qh * 4));
        ws.pos_dev = static_cast<uint32_t *>(dev_.alloc((tokens + 1) * 4));
        check(brc_decode_workspace_bytes(pool_->raw(), (uint32_t)tokens, n_head_, &ws.scratch_bytes));
        ws.scratch = dev_.alloc(ws.scratch_bytes);
        return ws;
    }
    void release(QsaWorkspace &ws) const {
        for (void *p : {(void *)ws.k_cur, (void *)ws.v_cur, (void *)ws.q, (void *)ws.q_full, (void *)ws.attn_out, (void *)ws.pos_dev,
                        (void *)ws.tables_dev, ws.scratch})
            if (p) dev_.free(p);
        ws = QsaWorkspace();
    }

    // Scatter the workspace's `tokens` K/V rows into cells pos0 .. pos0 + tokens of the state.
    void kv_append(const QsaState &st, const QsaWorkspace &ws, size_t pos0) const {
        if (pos0 + ws.tokens > st.capacity_cells())
            throw Error(BRC_ERR_CAPACITY, "kv_append would write cells " + std::to_string(pos0) + ".." +
                                              std::to_string(pos0 + ws.tokens) + " but the cache holds " +
                                              std::to_string(st.capacity_cells()));
        const uint32_t p0 = (uint32_t)pos0;
        dev_.upload(ws.pos_dev, &p0, 4);
        check(brc_kv_append(pool_->raw(), st.layer(), st.block_table_dev(), (uint32_t)st.block_table().size(), ws.pos_dev, 1,
                            (uint32_t)ws.tokens, nullptr, (uint32_t)ws.tokens, (uint32_t)(pos0 + ws.tokens), ws.k_cur, ws.v_cur,
                            BRC_DTYPE_F32, stream_));
    }
    // Dense selection: row t sees cells 0 ..= pos0 + t.  It is carried as per-row lengths; there is no
    // id list to build.
    void topk_dense(const QsaWorkspace &ws, size_t pos0) const {
        std::vector<uint32_t> lens(ws.tokens);
        for (size_t t = 0; t < ws.tokens; ++t) lens[t] = (uint32_t)(pos0 + t + 1);
        dev_.upload(ws.pos_dev + 1, lens.data(), lens.size() * 4);
    }
    // Scores, softmax and the weighted sum of V, gate included: one kernel.  Rows are attended as
    // `tokens` sequences that share the state's block table (causal: row t has length pos0 + t + 1).
    void attend(const QsaState &st, QsaWorkspace &ws, size_t pos0) const {
        if (pos0 + ws.tokens > st.capacity_cells())
            throw Error(BRC_ERR_CAPACITY, "attend would read cells up to " + std::to_string(pos0 + ws.tokens) +
                                              " but the cache holds " + std::to_string(st.capacity_cells()));
        const uint32_t hd = pool_->head_dim();
        const size_t n = st.block_table().size();
        if (ws.tables_len != n) {
            if (ws.tables_dev) dev_.free(ws.tables_dev);
            ws.tables_dev = static_cast<uint32_t *>(dev_.alloc(ws.tokens * n * 4));
            ws.tables_len = n;
        }
        std::vector<uint32_t> rows(ws.tokens * n);
        for (size_t t = 0; t < ws.tokens; ++t) std::copy(st.block_table().begin(), st.block_table().end(), rows.begin() + t * n);
        dev_.upload(ws.tables_dev, rows.data(), rows.size() * 4);
        check(brc_paged_decode_attn(pool_->raw(), st.layer(), ws.q, BRC_DTYPE_F32, n_head_, ws.use_gate ? ws.q_full + hd : nullptr,
                                    ws.use_gate ? 2 * hd : 0, ws.tables_dev, (uint32_t)n, ws.pos_dev + 1, (uint32_t)ws.tokens,
                                    (uint32_t)(pos0 + ws.tokens), scale_, ws.attn_out, ws.scratch, ws.scratch_bytes, stream_));
    }
    void apply(const QsaState &, const QsaWorkspace &, size_t) const {}   // done by attend

    uint32_t n_head() const { return n_head_; }

private:
    KvPool *pool_;
    DeviceAlloc dev_;
    uint32_t n_head_;
    void *stream_;
    float scale_;
};

}  // namespace brc
