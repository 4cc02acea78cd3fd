// Device-side helpers: the reference's f16 storage codec and thin wrappers over
// the sm_100a PTX this library uses (mbarrier, TMA tiled loads, ldmatrix,
// mma.sync, movmatrix).  Every wait is bounded.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace brc {

// ---------------------------------------------------------------------------------------------
// f16 storage codec — shaders/f16_storage.glsl:26-69 of the reference, bit for bit.  This is NOT
// cvt.rn.f16.f32: magnitudes below 2^-14 store as signed zero (no subnormals), NaN stores as inf.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f32_to_f16_bits(float x) {
    const uint32_t b = __float_as_uint(x);
    const uint32_t sign = (b >> 16) & 0x8000u;
    const uint32_t mag = b & 0x7fffffffu;
    if (mag >= 0x477ff000u) return sign | 0x7c00u;
    if (mag < 0x38800000u) return sign;  // exponent < -14 (includes zero): flushed before rounding
    // Normal range: rebias the exponent (127 -> 15), add half an ulp minus one plus the kept LSB
    // (ties to even) and drop 13 bits; a mantissa carry lands in the exponent field by itself.
    const uint32_t lsb = (mag >> 13) & 1u;
    return sign | ((mag - 0x38000000u + 0xfffu + lsb) >> 13);
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    const uint32_t m = h & 0x3ffu;
    if (e == 0u) return __uint_as_float(sign);
    if (e == 31u) return __uint_as_float(sign | 0x7f800000u | (m << 13));
    return __uint_as_float(sign | ((e + 112u) << 23) | (m << 13));
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    return (f32_to_f16_bits(hi) << 16) | f32_to_f16_bits(lo);
}

// Two binary16 values as stored: an exponent field of zero becomes a signed zero (what the
// reference's loader would read, shaders/f16_storage.glsl:62-64), so the pool never holds subnormals.
__device__ __forceinline__ uint32_t flush_f16x2(uint32_t w) {
    if ((w & 0x7c00u) == 0u) w &= 0xffff8000u;
    if ((w & 0x7c000000u) == 0u) w &= 0x8000ffffu;
    return w;
}

// ---------------------------------------------------------------------------------------------
// shared-memory addressing and mbarriers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: each try_wait already suspends for a hardware-defined slice, so the limit below is
// seconds of wall time, far beyond any legitimate wait here.  Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Order this thread's generic-proxy shared-memory writes before later async-proxy (TMA) accesses.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Order this thread's generic-proxy global-memory writes before later async-proxy (TMA) reads of them.
__device__ __forceinline__ void fence_proxy_async_global() {
    asm volatile("fence.proxy.async.global;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled tensor loads into this CTA's shared memory)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *tm) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
}

// x = innermost (column, elements), y = row.  x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap *tm, int32_t x, int32_t y,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}

// Three coordinates, innermost first.  c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap *tm, int32_t c0, int32_t c1, int32_t c2,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(policy)
        : "memory");
}

// Four coordinates, innermost first.  c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap *tm, int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst_smem),
        "l"(reinterpret_cast<uint64_t>(tm)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy)
        : "memory");
}

// ---------------------------------------------------------------------------------------------
// warp-level matrix helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Transpose an 8x8 matrix of 16-bit elements held one 32-bit register per lane.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace brc
