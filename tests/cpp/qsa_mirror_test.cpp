// Test driver of the C++ host-side mirror (include/breccia_qsa.hpp), built and run by
// tests/test_cpp_mirror_*.py.
//
//   qsa_mirror_test cpu
//       bookkeeping pool only (no GPU): allocator, refcounts, states over shared tables, the host-side
//       capacity refusal of kv_append.  Prints "ok" and exits 0.
//   qsa_mirror_test gpu <dir>
//       the reference's call sequence for one sequence of one layer (kv_append in chunks, one more
//       token, topk_dense, attend, apply), inputs read from <dir>/{table.u32,k_ctx.f32,v_ctx.f32,
//       k_new.f32,v_new.f32,q.f32}, results written to <dir>/{out.f32,k_pool.u16,v_pool.u16}.
//       Geometry: 16 query heads, 2 kv heads, head_dim 256, 256-page pool, 1024 context cells.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "breccia_qsa.hpp"

#define REQUIRE(cond)                                                         \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::fprintf(stderr, "%s:%d: %s failed\n", __FILE__, __LINE__, #cond); \
            return 1;                                                         \
        }                                                                     \
    } while (0)

template <typename T>
static std::vector<T> read_file(const std::string &path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + path);
    const size_t bytes = (size_t)f.tellg();
    std::vector<T> v(bytes / sizeof(T));
    f.seekg(0);
    f.read(reinterpret_cast<char *>(v.data()), (std::streamsize)bytes);
    return v;
}

template <typename T>
static void write_file(const std::string &path, const std::vector<T> &v) {
    std::ofstream f(path, std::ios::binary);
    f.write(reinterpret_cast<const char *>(v.data()), (std::streamsize)(v.size() * sizeof(T)));
}

static int run_cpu() {
    brc::KvPool pool = brc::KvPool::bookkeeping(12, 2, 256, 64);
    REQUIRE(pool.free_pages() == 64);
    REQUIRE(pool.v_layout() == brc::VLayout::F16);
    brc::DeviceAlloc none;   // no device: states keep their tables on the host only
    {
        brc::QsaState a(pool, none, 0, 100);   // 7 pages
        REQUIRE(a.block_table().size() == 7 && pool.free_pages() == 57);
        REQUIRE(a.bytes() == 7ull * 32768);    // page_bytes() == 32768 in the reference (qsa/mod.rs:2133)
        {
            brc::QsaState shared(pool, none, 0, a.block_table());   // a second holder of the same pages
            REQUIRE(pool.refcount(a.block_table()[0]) == 2 && pool.free_pages() == 57);
        }
        REQUIRE(pool.refcount(a.block_table()[0]) == 1);
        // the host-side refusal comes before any device call
        brc::Qsa qsa(pool, none, 16);
        brc::QsaWorkspace ws;
        ws.tokens = 8;
        bool refused = false;
        try {
            qsa.kv_append(a, ws, 110);
        } catch (const brc::Error &e) {
            refused = e.code == BRC_ERR_CAPACITY && std::string(e.what()).find("kv_append would write cells 110..118") != std::string::npos;
        }
        REQUIRE(refused);
    }
    REQUIRE(pool.free_pages() == 64);
    bool exhausted = false;
    try {
        pool.alloc(65);
    } catch (const brc::Error &e) {
        exhausted = e.code == BRC_ERR_NO_PAGES;
    }
    REQUIRE(exhausted);
    std::puts("ok");
    return 0;
}

static int run_gpu(const std::string &dir) {
    using brc::check;
    const uint32_t n_head = 16, n_kv = 2, hd = 256, pool_pages = 256, context = 1024;
    brc::DeviceAlloc dev;
    dev.alloc = [](size_t bytes) {
        void *p = nullptr;
        if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess) throw std::runtime_error("cudaMalloc");
        return p;
    };
    dev.free = [](void *p) { cudaFree(p); };
    dev.upload = [](void *dst, const void *src, size_t bytes) {
        if (cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess) throw std::runtime_error("cudaMemcpy");
    };
    const auto table = read_file<uint32_t>(dir + "/table.u32");
    const auto k_ctx = read_file<float>(dir + "/k_ctx.f32"), v_ctx = read_file<float>(dir + "/v_ctx.f32");
    const auto k_new = read_file<float>(dir + "/k_new.f32"), v_new = read_file<float>(dir + "/v_new.f32");
    const auto q = read_file<float>(dir + "/q.f32");
    REQUIRE(table.size() == 65 && k_ctx.size() == (size_t)context * n_kv * hd && q.size() == (size_t)n_head * hd);

    brc::KvPool pool(0, 1, n_kv, hd, pool_pages);
    check(brc_pool_zero(pool.raw(), nullptr));
    // the block table is the test's permutation, so take exactly those pages
    std::vector<uint32_t> all = pool.alloc(pool_pages);
    brc::QsaState state(pool, dev, 0, table);
    pool.release(all);
    brc::Qsa qsa(pool, dev, n_head);
    brc::QsaWorkspace ws = qsa.workspace(256);
    const size_t row = (size_t)n_kv * hd;
    for (uint32_t start = 0; start < context; start += 256) {
        dev.upload(ws.k_cur, k_ctx.data() + start * row, 256 * row * 4);
        dev.upload(ws.v_cur, v_ctx.data() + start * row, 256 * row * 4);
        qsa.kv_append(state, ws, start);
    }
    brc::QsaWorkspace ws1 = qsa.workspace(1);
    dev.upload(ws1.k_cur, k_new.data(), row * 4);
    dev.upload(ws1.v_cur, v_new.data(), row * 4);
    dev.upload(ws1.q, q.data(), q.size() * 4);
    qsa.kv_append(state, ws1, context);
    qsa.topk_dense(ws1, context);
    qsa.attend(state, ws1, context);
    qsa.apply(state, ws1, context);
    pool.check_device();

    std::vector<float> out((size_t)n_head * hd);
    REQUIRE(cudaMemcpy(out.data(), ws1.attn_out, out.size() * 4, cudaMemcpyDeviceToHost) == cudaSuccess);
    std::vector<uint16_t> kp((size_t)pool_pages * n_kv * 16 * hd), vp(kp.size());
    check(brc_pool_read(pool.raw(), 0, 0, 0, kp.data(), kp.size() * 2, nullptr));
    check(brc_pool_read(pool.raw(), 1, 0, 0, vp.data(), vp.size() * 2, nullptr));
    write_file(dir + "/out.f32", out);
    write_file(dir + "/k_pool.u16", kp);
    write_file(dir + "/v_pool.u16", vp);

    // appending past the table is refused on the host, with the numbers, and nothing is launched
    bool refused = false;
    try {
        qsa.kv_append(state, ws, 65 * 16 - 100);
    } catch (const brc::Error &e) {
        refused = e.code == BRC_ERR_CAPACITY;
    }
    REQUIRE(refused);
    qsa.release(ws);
    qsa.release(ws1);
    std::puts("ok");
    return 0;
}

int main(int argc, char **argv) {
    try {
        if (argc >= 2 && std::strcmp(argv[1], "cpu") == 0) return run_cpu();
        if (argc >= 3 && std::strcmp(argv[1], "gpu") == 0) return run_gpu(argv[2]);
    } catch (const std::exception &e) {
        std::fprintf(stderr, "exception: %s\n", e.what());
        return 2;
    }
    std::fprintf(stderr, "usage: qsa_mirror_test cpu | gpu <dir>\n");
    return 64;
}
