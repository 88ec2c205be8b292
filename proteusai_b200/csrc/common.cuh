// Shared device helpers: packed fp32x2 arithmetic, mbarrier + bulk-copy (TMA) wrappers with
// bounded waits, and the device status word.  sm_100a only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/proteus_b200.h"

namespace pai {

// One status word per device, written by kernels that give up on a bounded wait.  The library
// is one translation unit, so file scope is library scope.
static __device__ int g_device_status = 0;
static __device__ float g_sink = 0.f;

// ---- packed fp32x2 (Blackwell FFMA2/FMUL2/FADD2) -------------------------------------------
typedef unsigned long long f2_t;  // two fp32 in one 64-bit register pair: {lo, hi}

__device__ __forceinline__ f2_t f2_pack(float lo, float hi) {
    f2_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(f2_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2_t f2_mul(f2_t a, f2_t b) {
    f2_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2_t f2_add(f2_t a, f2_t b) {
    f2_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2_t f2_sub(f2_t a, f2_t b) {
    f2_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2_t f2_fma(f2_t a, f2_t b, f2_t c) {
    f2_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// sin and cos on the SFU (MUFU.SIN / MUFU.COS behind one shared fp32 scaling multiply)
__device__ __forceinline__ void sfu_sincos(float x, float &s, float &c) {
    asm("sin.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(x));
    asm("cos.approx.ftz.f32 %0, %1;" : "=f"(c) : "f"(x));
}

// sin and cos of 2 pi t for a packed pair of phases t given in REVOLUTIONS, entirely on the FMA pipe:
// subtract the nearest integer exactly (magic-number rounding), then even/odd polynomials in the
// fraction f in [-0.5, 0.5] (coefficients: Chebyshev fits of sin(2 pi f)/f and cos(2 pi f) in f^2;
// maximum error in fp32 Horner form 6e-7 and 4e-7).  17 packed instructions, no SFU.
__device__ __forceinline__ void poly_sincos_rev(f2_t t2, f2_t &s2, f2_t &c2) {
    const f2_t big = f2_pack(12582912.f, 12582912.f);  // 1.5 * 2^23
    const f2_t n2 = f2_sub(f2_add(t2, big), big);      // nearest integer
    const f2_t f = f2_sub(t2, n2);                     // exact
    const f2_t u = f2_mul(f, f);
#define PAI_C2(x) f2_pack(x, x)
    f2_t ps = PAI_C2(-12.47124354f);
    ps = f2_fma(ps, u, PAI_C2(41.34288235f));
    ps = f2_fma(ps, u, PAI_C2(-76.61447253f));
    ps = f2_fma(ps, u, PAI_C2(81.59994333f));
    ps = f2_fma(ps, u, PAI_C2(-41.34158923f));
    ps = f2_fma(ps, u, PAI_C2(6.28318492f));
    s2 = f2_mul(ps, f);
    f2_t pc = PAI_C2(6.52865816f);
    pc = f2_fma(pc, u, PAI_C2(-25.96759925f));
    pc = f2_fma(pc, u, PAI_C2(60.16763095f));
    pc = f2_fma(pc, u, PAI_C2(-85.45013953f));
    pc = f2_fma(pc, u, PAI_C2(64.93911746f));
    pc = f2_fma(pc, u, PAI_C2(-19.7392045f));
    c2 = f2_fma(pc, u, PAI_C2(0.99999999f));
#undef PAI_C2
}

// ---- shared-memory addresses, mbarriers, 1-D bulk copies --------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// (re-initialising a barrier that has been in use: invalidate it first)
__device__ __forceinline__ void mbar_inval(uint64_t *bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false after `limit` polls (each poll may itself block for a short,
// hardware-defined time).  The caller records the failure and leaves without touching the data.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 18)) {
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.  Both addresses and the
// size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

}  // namespace pai
