// Pool state, page allocator / refcounts, error plumbing.
//
// One pool per (GPU, layer set): K and V are each one contiguous allocation laid out
// [layer][page][kv_head][cell_in_page][d] in binary16, i.e. every layer's slice is exactly the
// reference's per-layer pool (crates/breccia-kernels/src/qsa/mod.rs:22-28), and one physical page id
// names the same slot in all layers.
#include <cstring>
#include <new>
#include <string>

#include "brc_internal.h"

static thread_local std::string g_last_error;

void brc_set_error(const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

brc_status brc_fail(brc_status code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

static cudaEvent_t take_event(brc_pool::stage_events &st) {
    cudaEvent_t e = nullptr;
    if (!st.spare.empty()) {
        e = st.spare.back();
        st.spare.pop_back();
    } else if (cudaEventCreate(&e) != cudaSuccess) {
        e = nullptr;
    }
    return e;
}

void brc_stage_begin(brc_pool *pool, int stage, cudaStream_t s) {
    if (!pool->timing) return;
    brc_pool::stage_events &st = pool->stages[stage];
    cudaEvent_t e = take_event(st);
    if (!e) return;
    cudaEventRecord(e, s);
    st.begin.push_back(e);
}

void brc_stage_end(brc_pool *pool, int stage, cudaStream_t s) {
    if (!pool->timing) return;
    brc_pool::stage_events &st = pool->stages[stage];
    if (st.begin.size() == st.end.size()) return;  // begin failed
    cudaEvent_t e = take_event(st);
    if (!e) {
        st.spare.push_back(st.begin.back());
        st.begin.pop_back();
        return;
    }
    cudaEventRecord(e, s);
    st.end.push_back(e);
}

extern "C" {

const char *brc_last_error(void) { return g_last_error.c_str(); }

int32_t brc_abi_version(void) { return 1; }

}  // extern "C"

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so the library links against the CUDA runtime
// only and still loads on a machine without a driver.
static encode_tiled_fn get_encode_tiled() {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    return reinterpret_cast<encode_tiled_fn>(fn);
}

// 2-D view [rows][head_dim] of a whole K or V allocation; box = one page of one kv head's rows by
// 64 columns (128 bytes, the swizzle span).
static brc_status make_map(CUtensorMap *tm, void *base, uint64_t rows, uint32_t head_dim, uint32_t box_rows) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return brc_fail(BRC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {head_dim, rows};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2u};
    cuuint32_t box[2] = {64u, box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return brc_fail(BRC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows %llu, head_dim %u)",
                        (int)r, (unsigned long long)rows, head_dim);
    return BRC_OK;
}

// 2-D view [rows][row_words] of a q8_0 V allocation in 32-bit words (a row of head_dim / 32 blocks of 9 words);
// box = `box_rows` whole rows, no swizzle (the consumers read single words).
static brc_status make_q8_map(CUtensorMap *tm, void *base, uint64_t rows, uint32_t row_words, uint32_t box_rows) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return brc_fail(BRC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {row_words, rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_words * 4u};
    cuuint32_t box[2] = {row_words, box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return brc_fail(BRC_ERR_CUDA, "cuTensorMapEncodeTiled (q8_0 V view) failed with CUresult %d (rows %llu, %u words per row)",
                        (int)r, (unsigned long long)rows, row_words);
    return BRC_OK;
}

// 3-D view (column, row, K|V) over the single allocation that holds both pools: strides ascend
// (row = head_dim * 2 bytes, K|V = offset of the V pool), and one box [64 columns][page rows][2]
// brings a 64-column group of the K tile and of the V tile of a page in one operation.
static brc_status make_kv_map(CUtensorMap *tm, void *k_base, uint64_t v_offset_bytes, uint64_t rows, uint32_t head_dim,
                              uint32_t page_tokens) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return brc_fail(BRC_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {head_dim, rows, 2u};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2u, v_offset_bytes};
    cuuint32_t box[3] = {64u, page_tokens, 2u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, k_base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return brc_fail(BRC_ERR_CUDA, "cuTensorMapEncodeTiled (3-D K|V view) failed with CUresult %d (rows %llu, V offset %llu)",
                        (int)r, (unsigned long long)rows, (unsigned long long)v_offset_bytes);
    return BRC_OK;
}

// 4-D view (column within a 64-column group, row, K|V, column group): the strides do not ascend (a group lies
// 128 bytes after the one before, inside the row), which lets one box [64][rows][2][head_dim / 64] deliver a
// whole page-unit - laid out in shared memory as [group][K|V][row][64 columns], the order the decode kernel's
// stages have - in a single operation of 16 or 32 KiB.  The encoder accepts it although its documentation asks
// for every stride to be a multiple of the one before; the decode kernel therefore uses these views only when
// asked to (BRC_DECODE_STAGE_OP=1) and otherwise issues one 3-D box per column group.
static bool make_kv_stage_map(CUtensorMap *tm, void *k_base, uint64_t v_offset_bytes, uint64_t rows, uint32_t head_dim,
                              uint32_t box_rows) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[4] = {64u, rows, 2u, head_dim / 64u};
    cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2u, v_offset_bytes, 128u};
    cuuint32_t box[4] = {64u, box_rows, 2u, head_dim / 64u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, k_base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same for K alone (pools with q8_0 V pages): (column within a group, row, group), one box per page-unit.
static bool make_k_stage_map(CUtensorMap *tm, void *k_base, uint64_t rows, uint32_t head_dim, uint32_t box_rows) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[3] = {64u, rows, head_dim / 64u};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2u, 128u};
    cuuint32_t box[3] = {64u, box_rows, head_dim / 64u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, k_base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static brc_status create_pool(int32_t device, uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim,
                              uint32_t page_tokens, uint32_t n_pages, bool v_q8, brc_pool **out) {
    if (!out) return brc_fail(BRC_ERR_INVALID, "brc_pool_create: out is NULL");
    *out = nullptr;
    if (n_layers == 0 || n_kv_head == 0 || n_pages == 0)
        return brc_fail(BRC_ERR_INVALID, "brc_pool_create: n_layers %u, n_kv_head %u, n_pages %u must be non-zero",
                        n_layers, n_kv_head, n_pages);
    if (head_dim != 256 && head_dim != 128)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_pool_create: head_dim %u (kernels are built for 128 and 256)",
                        head_dim);
    if (page_tokens != 16)
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_pool_create: page_tokens %u (the page is 16 cells)", page_tokens);
    const uint64_t rows = (uint64_t)n_layers * n_pages * n_kv_head * page_tokens;
    if (rows >= (1ull << 31))
        return brc_fail(BRC_ERR_UNSUPPORTED, "brc_pool_create: %llu cache rows exceed the 2^31 row coordinate range",
                        (unsigned long long)rows);
    int count = 0;
    BRC_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count)
        return brc_fail(BRC_ERR_INVALID, "brc_pool_create: device %d out of range (%d visible)", device, count);
    brc_device_guard guard(device);
    if (!guard.ok) return brc_fail(BRC_ERR_CUDA, "brc_pool_create: cannot make device %d current", device);

    brc_pool *p = new (std::nothrow) brc_pool();
    if (!p) return brc_fail(BRC_ERR_INVALID, "brc_pool_create: out of host memory");
    p->device = device;
    p->n_layers = n_layers;
    p->n_kv_head = n_kv_head;
    p->head_dim = head_dim;
    p->page_tokens = page_tokens;
    p->n_pages = n_pages;
    p->half_page_bytes = (uint64_t)n_kv_head * page_tokens * head_dim * 2u;
    p->layer_bytes = p->half_page_bytes * n_pages;
    const uint64_t bytes = p->layer_bytes * n_layers;
    p->v_q8 = v_q8;
    p->v_layer_bytes = v_q8 ? p->layer_bytes / 16u * 9u : p->layer_bytes;   // 36 B per 32 values against 64 B
    const uint64_t v_bytes = p->v_layer_bytes * n_layers;
    cudaError_t e;
    // K and V live in one allocation so a single tensor map can address both.
    if ((e = cudaMalloc(&p->k_base, bytes + v_bytes)) != cudaSuccess || (e = cudaMalloc(&p->status_dev, BRC_STATUS_BYTES)) != cudaSuccess ||
        (e = cudaMallocHost(&p->status_host, 256)) != cudaSuccess) {
        brc_status rc = brc_fail(BRC_ERR_CUDA, "brc_pool_create: allocating 2 x %llu bytes on device %d failed: %s",
                                 (unsigned long long)bytes, device, cudaGetErrorString(e));
        brc_pool_destroy(p);
        return rc;
    }
    p->v_base = p->k_base + bytes;
    p->ids_cap = 1u << 16;
    if ((e = cudaMalloc(&p->ids_dev, (size_t)p->ids_cap * 2 * sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMemset(p->k_base, 0, bytes)) != cudaSuccess || (e = cudaMemset(p->v_base, 0, v_bytes)) != cudaSuccess ||
        (e = cudaMemset(p->status_dev, 0, BRC_STATUS_BYTES)) != cudaSuccess || (e = cudaDeviceSynchronize()) != cudaSuccess) {
        brc_status rc = brc_fail(BRC_ERR_CUDA, "brc_pool_create: initialising the pool failed: %s", cudaGetErrorString(e));
        brc_pool_destroy(p);
        return rc;
    }
    cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, device);
    brc_status rc = make_map(&p->tm_k, p->k_base, rows, head_dim, page_tokens);
    // (a q8_0 V pool has no binary16 V rows to map: the kernels that use these views refuse it)
    if (rc == BRC_OK && !v_q8) rc = make_map(&p->tm_v, p->v_base, rows, head_dim, page_tokens);
    if (rc == BRC_OK && !v_q8) rc = make_kv_map(&p->tm_kv, p->k_base, bytes, rows, head_dim, page_tokens);
    // With an even number of kv heads, the rows of two neighbouring kv heads of a page are contiguous:
    // a box of 2 * page_tokens rows brings both (8 KiB per operation instead of 4 KiB).
    if (rc == BRC_OK && !v_q8 && n_kv_head % 2u == 0u)
        rc = make_kv_map(&p->tm_kv2, p->k_base, bytes, rows, head_dim, 2u * page_tokens);
    if (rc == BRC_OK && !v_q8) {
        p->stage_maps = make_kv_stage_map(&p->tm_kv_stage, p->k_base, bytes, rows, head_dim, page_tokens) &&
                        (n_kv_head % 2u != 0u || make_kv_stage_map(&p->tm_kv2_stage, p->k_base, bytes, rows, head_dim, 2u * page_tokens));
    }
    if (rc == BRC_OK && v_q8) {
        const uint32_t row_words = head_dim / 32u * 9u;
        rc = make_q8_map(&p->tm_v8, p->v_base, rows, row_words, page_tokens);
        if (rc == BRC_OK && n_kv_head % 2u == 0u) rc = make_map(&p->tm_k2, p->k_base, rows, head_dim, 2u * page_tokens);
        if (rc == BRC_OK && n_kv_head % 2u == 0u) rc = make_q8_map(&p->tm_v8_2, p->v_base, rows, row_words, 2u * page_tokens);
        if (rc == BRC_OK)
            p->stage_maps = make_k_stage_map(&p->tm_k_stage, p->k_base, rows, head_dim, page_tokens) &&
                            (n_kv_head % 2u != 0u || make_k_stage_map(&p->tm_k2_stage, p->k_base, rows, head_dim, 2u * page_tokens));
    }
    if (rc != BRC_OK) {
        brc_pool_destroy(p);
        return rc;
    }
    p->has_tma = true;
    brc_decode_calibrate(p);   // per-SM streaming rates of this device (measured once per process; large pools only)
    p->refcount.assign(n_pages, 0u);
    p->tree_refs.assign(n_pages, 0u);
    p->free_list.resize(n_pages);
    for (uint32_t i = 0; i < n_pages; ++i) p->free_list[i] = n_pages - 1 - i;  // pop_back yields 0,1,2,...
    *out = p;
    return BRC_OK;
}

extern "C" {

brc_status brc_pool_create(int32_t device, uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim,
                           uint32_t page_tokens, uint32_t n_pages, brc_pool **out) {
    return create_pool(device, n_layers, n_kv_head, head_dim, page_tokens, n_pages, false, out);
}

brc_status brc_pool_create_q8v(int32_t device, uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim,
                               uint32_t page_tokens, uint32_t n_pages, brc_pool **out) {
    return create_pool(device, n_layers, n_kv_head, head_dim, page_tokens, n_pages, true, out);
}

brc_status brc_pool_v_layout(const brc_pool *pool, int32_t *out_layout) {
    if (!pool || !out_layout) return brc_fail(BRC_ERR_INVALID, "brc_pool_v_layout: NULL argument");
    *out_layout = pool->v_q8 ? BRC_V_Q8_0 : BRC_V_F16;
    return BRC_OK;
}

brc_status brc_pool_create_bookkeeping(uint32_t n_layers, uint32_t n_kv_head, uint32_t head_dim, uint32_t page_tokens,
                                       uint32_t n_pages, brc_pool **out) {
    if (!out) return brc_fail(BRC_ERR_INVALID, "brc_pool_create_bookkeeping: out is NULL");
    *out = nullptr;
    if (n_layers == 0 || n_kv_head == 0 || n_pages == 0 || head_dim == 0 || page_tokens == 0)
        return brc_fail(BRC_ERR_INVALID, "brc_pool_create_bookkeeping: zero-sized geometry");
    brc_pool *p = new (std::nothrow) brc_pool();
    if (!p) return brc_fail(BRC_ERR_INVALID, "brc_pool_create_bookkeeping: out of host memory");
    p->device = -1;
    p->n_layers = n_layers;
    p->n_kv_head = n_kv_head;
    p->head_dim = head_dim;
    p->page_tokens = page_tokens;
    p->n_pages = n_pages;
    p->half_page_bytes = (uint64_t)n_kv_head * page_tokens * head_dim * 2u;
    p->layer_bytes = p->half_page_bytes * n_pages;
    p->v_layer_bytes = p->layer_bytes;
    p->refcount.assign(n_pages, 0u);
    p->tree_refs.assign(n_pages, 0u);
    p->free_list.resize(n_pages);
    for (uint32_t i = 0; i < n_pages; ++i) p->free_list[i] = n_pages - 1 - i;
    *out = p;
    return BRC_OK;
}

brc_status brc_pool_destroy(brc_pool *pool) {
    if (!pool) return BRC_OK;
    if (pool->device >= 0) {
        brc_device_guard guard(pool->device);
        if (pool->k_base) cudaFree(pool->k_base);  // V is the second half of the same allocation
        if (pool->status_dev) cudaFree(pool->status_dev);
        if (pool->status_host) cudaFreeHost(pool->status_host);
        if (pool->ids_dev) cudaFree(pool->ids_dev);
        for (auto &st : pool->stages) {
            for (cudaEvent_t e : st.begin) cudaEventDestroy(e);
            for (cudaEvent_t e : st.end) cudaEventDestroy(e);
            for (cudaEvent_t e : st.spare) cudaEventDestroy(e);
        }
        if (pool->host_up) cudaStreamDestroy(pool->host_up);
        if (pool->host_down) cudaStreamDestroy(pool->host_down);
        for (cudaEvent_t e : pool->host_uploaded) if (e) cudaEventDestroy(e);
        for (cudaEvent_t e : pool->host_computed) if (e) cudaEventDestroy(e);
        if (pool->host_all_down) cudaEventDestroy(pool->host_all_down);
        if (pool->decode_event) cudaEventDestroy(pool->decode_event);
    }
    delete pool;
    return BRC_OK;
}

brc_status brc_pool_geometry(const brc_pool *pool, brc_geometry *out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_pool_geometry: NULL argument");
    out->n_layers = pool->n_layers;
    out->n_kv_head = pool->n_kv_head;
    out->head_dim = pool->head_dim;
    out->page_tokens = pool->page_tokens;
    out->n_pages = pool->n_pages;
    out->device = pool->device;
    out->half_page_bytes = pool->half_page_bytes;
    out->total_bytes = (pool->layer_bytes + pool->v_layer_bytes) * pool->n_layers;
    return BRC_OK;
}

brc_status brc_pool_bytes(const brc_pool *pool, uint64_t *out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_pool_bytes: NULL argument");
    *out = (pool->layer_bytes + pool->v_layer_bytes) * pool->n_layers;
    return BRC_OK;
}

static brc_status pool_fill(brc_pool *pool, int value, void *stream, const char *who) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "%s: pool is NULL", who);
    brc_device_guard guard(pool->device);
    const uint64_t bytes = pool->layer_bytes * pool->n_layers;
    BRC_CUDA(cudaMemsetAsync(pool->k_base, value, bytes, brc_stream(stream)));
    BRC_CUDA(cudaMemsetAsync(pool->v_base, value, pool->v_layer_bytes * pool->n_layers, brc_stream(stream)));
    return BRC_OK;
}

brc_status brc_pool_zero(brc_pool *pool, void *stream) { return pool_fill(pool, 0, stream, "brc_pool_zero"); }

brc_status brc_pool_poison_nan(brc_pool *pool, void *stream) {
    return pool_fill(pool, 0xFF, stream, "brc_pool_poison_nan");
}

brc_status brc_pool_k_ptr(const brc_pool *pool, uint32_t layer, void **out_dev) {
    if (!pool || !out_dev) return brc_fail(BRC_ERR_INVALID, "brc_pool_k_ptr: NULL argument");
    if (layer >= pool->n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_pool_k_ptr: layer %u but the pool has %u", layer, pool->n_layers);
    *out_dev = pool->k_base + (uint64_t)layer * pool->layer_bytes;
    return BRC_OK;
}

brc_status brc_pool_v_ptr(const brc_pool *pool, uint32_t layer, void **out_dev) {
    if (!pool || !out_dev) return brc_fail(BRC_ERR_INVALID, "brc_pool_v_ptr: NULL argument");
    if (layer >= pool->n_layers)
        return brc_fail(BRC_ERR_INVALID, "brc_pool_v_ptr: layer %u but the pool has %u", layer, pool->n_layers);
    *out_dev = pool->v_base + (uint64_t)layer * pool->v_layer_bytes;
    return BRC_OK;
}

static brc_status pool_rw(brc_pool *pool, int32_t which, uint32_t layer, uint64_t off, void *host, uint64_t bytes,
                          void *stream, bool read, const char *who) {
    if (!pool || (!host && bytes)) return brc_fail(BRC_ERR_INVALID, "%s: NULL argument", who);
    if (pool->device < 0 || !pool->k_base) return brc_fail(BRC_ERR_CUDA, "%s: this pool holds bookkeeping only", who);
    if (which != 0 && which != 1) return brc_fail(BRC_ERR_INVALID, "%s: which = %d (0 = K, 1 = V)", who, which);
    if (layer >= pool->n_layers) return brc_fail(BRC_ERR_INVALID, "%s: layer %u but the pool has %u", who, layer, pool->n_layers);
    const uint64_t one_layer = which ? pool->v_layer_bytes : pool->layer_bytes;
    if (off > one_layer || bytes > one_layer - off)
        return brc_fail(BRC_ERR_CAPACITY, "%s: bytes %llu..%llu but one layer's pool holds %llu", who,
                        (unsigned long long)off, (unsigned long long)(off + bytes), (unsigned long long)one_layer);
    brc_device_guard guard(pool->device);
    uint8_t *dev = (which ? pool->v_base : pool->k_base) + (uint64_t)layer * one_layer + off;
    cudaStream_t s = brc_stream(stream);
    if (read)
        BRC_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, s));
    else
        BRC_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, s));
    BRC_CUDA(cudaStreamSynchronize(s));
    return BRC_OK;
}

brc_status brc_pool_read(brc_pool *pool, int32_t which, uint32_t layer, uint64_t byte_offset, void *dst, uint64_t bytes,
                         void *stream) {
    return pool_rw(pool, which, layer, byte_offset, dst, bytes, stream, true, "brc_pool_read");
}

brc_status brc_pool_write(brc_pool *pool, int32_t which, uint32_t layer, uint64_t byte_offset, const void *src,
                          uint64_t bytes, void *stream) {
    return pool_rw(pool, which, layer, byte_offset, const_cast<void *>(src), bytes, stream, false, "brc_pool_write");
}

brc_status brc_pool_check(brc_pool *pool, void *stream) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_pool_check: pool is NULL");
    brc_device_guard guard(pool->device);
    cudaStream_t s = brc_stream(stream);
    BRC_CUDA(cudaMemcpyAsync(pool->status_host, pool->status_dev, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    BRC_CUDA(cudaMemsetAsync(pool->status_dev, 0, 4 * sizeof(uint32_t), s));
    BRC_CUDA(cudaStreamSynchronize(s));
    const uint32_t w = pool->status_host[0];
    const uint32_t detail = pool->status_host[1];
    if (w == 0) return BRC_OK;
    // A kernel that gave up or skipped work may have left the decode kernels' per-unit arrival counters
    // (which are otherwise returned to zero by the kernels themselves) in an odd state: clear them.
    cudaMemsetAsync(pool->status_dev, 0, BRC_STATUS_BYTES, s);
    cudaStreamSynchronize(s);
    if (w & BRC_DEV_WAIT_LIMIT)
        return brc_fail(BRC_ERR_TIMEOUT, "a kernel gave up a bounded wait (check word 0x%x, detail %u, at %u of %u)", w, detail,
                        pool->status_host[2], pool->status_host[3]);
    return brc_fail(BRC_ERR_DEVICE_CHECK,
                    "a kernel refused an index: check word 0x%x (%s%s%s), last offending value %u", w,
                    (w & BRC_DEV_BAD_PAGE) ? "page id >= n_pages " : "", (w & BRC_DEV_BAD_POS) ? "position past bound " : "",
                    (w & BRC_DEV_BAD_SHAPE) ? "too many work units" : "", detail);
}

brc_status brc_timing_enable(brc_pool *pool, int32_t on) {
    if (!pool) return brc_fail(BRC_ERR_INVALID, "brc_timing_enable: pool is NULL");
    if (pool->device < 0) return brc_fail(BRC_ERR_CUDA, "brc_timing_enable: this pool holds bookkeeping only");
    pool->timing = on != 0;
    return BRC_OK;
}

brc_status brc_timing_read(brc_pool *pool, int32_t stage, uint32_t *out_launches, double *out_total_ms) {
    if (!pool || !out_launches || !out_total_ms) return brc_fail(BRC_ERR_INVALID, "brc_timing_read: NULL argument");
    if (stage < 0 || stage >= BRC_STAGE_COUNT)
        return brc_fail(BRC_ERR_INVALID, "brc_timing_read: stage %d of %d", stage, BRC_STAGE_COUNT);
    if (pool->device < 0) return brc_fail(BRC_ERR_CUDA, "brc_timing_read: this pool holds bookkeeping only");
    brc_device_guard guard(pool->device);
    brc_pool::stage_events &st = pool->stages[stage];
    double total = 0.0;
    const size_t n = st.end.size();
    for (size_t i = 0; i < n; ++i) {
        BRC_CUDA(cudaEventSynchronize(st.end[i]));
        float ms = 0.f;
        BRC_CUDA(cudaEventElapsedTime(&ms, st.begin[i], st.end[i]));
        total += ms;
    }
    for (cudaEvent_t e : st.begin) st.spare.push_back(e);
    for (cudaEvent_t e : st.end) st.spare.push_back(e);
    st.begin.clear();
    st.end.clear();
    *out_launches = (uint32_t)n;
    *out_total_ms = total;
    return BRC_OK;
}

// ------------------------------------------------------------------------------------ allocator

brc_status brc_pages_alloc(brc_pool *pool, uint32_t n, uint32_t *out_ids) {
    if (!pool || (!out_ids && n)) return brc_fail(BRC_ERR_INVALID, "brc_pages_alloc: NULL argument");
    std::lock_guard<std::mutex> lock(pool->mu);
    if (pool->free_list.size() < n)
        return brc_fail(BRC_ERR_NO_PAGES, "brc_pages_alloc: %u pages requested, %zu free of %u", n,
                        pool->free_list.size(), pool->n_pages);
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t id = pool->free_list.back();
        pool->free_list.pop_back();
        pool->refcount[id] = 1;
        out_ids[i] = id;
    }
    return BRC_OK;
}

brc_status brc_pages_retain(brc_pool *pool, const uint32_t *ids, uint32_t n) {
    if (!pool || (!ids && n)) return brc_fail(BRC_ERR_INVALID, "brc_pages_retain: NULL argument");
    std::lock_guard<std::mutex> lock(pool->mu);
    for (uint32_t i = 0; i < n; ++i) {
        if (ids[i] >= pool->n_pages || pool->refcount[ids[i]] == 0)
            return brc_fail(BRC_ERR_INVALID, "brc_pages_retain: page %u (entry %u) is %s", ids[i], i,
                            ids[i] >= pool->n_pages ? "out of range" : "not allocated");
    }
    for (uint32_t i = 0; i < n; ++i) ++pool->refcount[ids[i]];
    return BRC_OK;
}

brc_status brc_pages_release(brc_pool *pool, const uint32_t *ids, uint32_t n) {
    if (!pool || (!ids && n)) return brc_fail(BRC_ERR_INVALID, "brc_pages_release: NULL argument");
    std::lock_guard<std::mutex> lock(pool->mu);
    // Validate the whole list first (an id may repeat) so a refused call changes nothing.
    std::vector<uint32_t> drop(n ? pool->n_pages : 0, 0u);
    for (uint32_t i = 0; i < n; ++i) {
        if (ids[i] >= pool->n_pages)
            return brc_fail(BRC_ERR_INVALID, "brc_pages_release: page %u (entry %u) is out of range", ids[i], i);
        if (++drop[ids[i]] > pool->refcount[ids[i]])
            return brc_fail(BRC_ERR_INVALID, "brc_pages_release: page %u released more often than it is held (%u)",
                            ids[i], pool->refcount[ids[i]]);
    }
    for (uint32_t i = 0; i < n; ++i)
        if (--pool->refcount[ids[i]] == 0) pool->free_list.push_back(ids[i]);
    return BRC_OK;
}

brc_status brc_page_refcount(const brc_pool *pool, uint32_t id, uint32_t *out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_page_refcount: NULL argument");
    if (id >= pool->n_pages) return brc_fail(BRC_ERR_INVALID, "brc_page_refcount: page %u of %u", id, pool->n_pages);
    std::lock_guard<std::mutex> lock(pool->mu);
    *out = pool->refcount[id];
    return BRC_OK;
}

brc_status brc_pages_free_count(const brc_pool *pool, uint32_t *out) {
    if (!pool || !out) return brc_fail(BRC_ERR_INVALID, "brc_pages_free_count: NULL argument");
    std::lock_guard<std::mutex> lock(pool->mu);
    *out = (uint32_t)pool->free_list.size();
    return BRC_OK;
}

}  // extern "C"
