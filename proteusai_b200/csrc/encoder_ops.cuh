// Memory-bound row operations of the encoder block around the attention kernel, bf16 in and out with fp32
// arithmetic: the post-norm step LN(x + y) of the reference's Encoder (old/old_scripts/encoder.py:30-39, which
// runs it as an elementwise add followed by nn.LayerNorm) as one pass, and the exact (erf) GELU of its MLP
// (utils/model_utils/base_modules/base_modules.py:46-52).
//
// Both are HBM-bound: LN(x + y) reads two rows and writes one (6 bytes per element), GELU reads and writes one
// (4 bytes per element).  Rows stay in registers between the statistics and the normalisation, so nothing is
// read twice.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace pai {

constexpr int ENC_THREADS = 256;  // 8 warps, one row per warp

__device__ __forceinline__ void bf16x8_to_float(const uint4 &u, float *f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint32_t float2_to_bf16x2(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&b);
}

// out[r,:] = LayerNorm(x[r,:] + y[r,:]) * gamma + beta over D values, D = 8 * 32 * CHUNKS at most and a multiple of 8.
// gamma/beta are bf16 or fp32 (params_fp32).  Statistics as nn.LayerNorm computes them: mean, then the biased
// variance of the centred values, eps inside the square root.
template <int CHUNKS>
__global__ void __launch_bounds__(ENC_THREADS) add_layernorm_bf16_kernel(const __nv_bfloat16 *__restrict__ x,
                                                                        const __nv_bfloat16 *__restrict__ y,
                                                                        const void *__restrict__ gamma,
                                                                        const void *__restrict__ beta,
                                                                        __nv_bfloat16 *__restrict__ out, long long rows, int D,
                                                                        float eps, int params_fp32) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (ENC_THREADS / 32) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + row * D);
    const uint4 *yr = y ? reinterpret_cast<const uint4 *>(y + row * D) : nullptr;
    float v[CHUNKS][8];
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int e = (c * 32 + lane) * 8;
        if (e < D) {
            float a[8], b[8];
            bf16x8_to_float(xr[c * 32 + lane], a);
            if (yr) {
                bf16x8_to_float(yr[c * 32 + lane], b);
#pragma unroll
                for (int i = 0; i < 8; ++i) a[i] += b[i];
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v[c][i] = a[i];
                sum += a[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[c][i] = 0.f;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / (float)D;
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        if ((c * 32 + lane) * 8 < D) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float d = v[c][i] - mean;
                sq = fmaf(d, d, sq);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / (float)D + eps);
    uint4 *orow = reinterpret_cast<uint4 *>(out + row * D);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int e = (c * 32 + lane) * 8;
        if (e < D) {
            float g[8], b[8];
            if (params_fp32) {
                const float4 *gp = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(gamma) + e);
                const float4 *bp = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(beta) + e);
                const float4 g0 = gp[0], g1 = gp[1], b0 = bp[0], b1 = bp[1];
                g[0] = g0.x, g[1] = g0.y, g[2] = g0.z, g[3] = g0.w, g[4] = g1.x, g[5] = g1.y, g[6] = g1.z, g[7] = g1.w;
                b[0] = b0.x, b[1] = b0.y, b[2] = b0.z, b[3] = b0.w, b[4] = b1.x, b[5] = b1.y, b[6] = b1.z, b[7] = b1.w;
            } else {
                bf16x8_to_float(*reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(gamma) + e), g);
                bf16x8_to_float(*reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(beta) + e), b);
            }
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = fmaf((v[c][i] - mean) * rstd, g[i], b[i]);
            uint4 pk;
            pk.x = float2_to_bf16x2(o[0], o[1]);
            pk.y = float2_to_bf16x2(o[2], o[3]);
            pk.z = float2_to_bf16x2(o[4], o[5]);
            pk.w = float2_to_bf16x2(o[6], o[7]);
            orow[c * 32 + lane] = pk;
        }
    }
}

static int add_layernorm_bf16_launch(const void *x, const void *y, const void *gamma, const void *beta, void *out, long long rows,
                                     int D, float eps, int params_fp32, cudaStream_t stream) {
    const unsigned grid = (unsigned)((rows + ENC_THREADS / 32 - 1) / (ENC_THREADS / 32));
    const int chunks = (D + 255) / 256;
#define PAI_LN_CASE(C)                                                                                                       \
    add_layernorm_bf16_kernel<C><<<grid, ENC_THREADS, 0, stream>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)y, gamma, \
                                                                   beta, (__nv_bfloat16 *)out, rows, D, eps, params_fp32)
    if (chunks <= 1) PAI_LN_CASE(1);
    else if (chunks <= 2) PAI_LN_CASE(2);
    else if (chunks <= 4) PAI_LN_CASE(4);
    else if (chunks <= 8) PAI_LN_CASE(8);
    else PAI_LN_CASE(16);
#undef PAI_LN_CASE
    return (int)cudaPeekAtLastError();
}

// Phi(x) = 0.5 erfc(-x / sqrt 2) from the rational approximation 7.1.26 of Abramowitz & Stegun,
// erfc(z) = t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-z^2), t = 1 / (1 + p z), z >= 0, absolute error below
// 1.5e-7 on erfc -- two SFU operations and a dozen FMAs, against the ~40 instructions of erff, which makes the
// elementwise pass compute-bound.  The negative side is evaluated as 0.5 erfc(|z|) directly, so small values of
// x Phi(x) keep their relative accuracy; the result is rounded to bf16 (2^-9 relative) anyway.
__device__ __forceinline__ float gelu_erf(float x) {
    const float z = fabsf(x) * 0.70710678118654752f;
    const float t = __fdividef(1.f, fmaf(0.3275911f, z, 1.f));
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(t, poly, 1.421413741f);
    poly = fmaf(t, poly, -0.284496736f);
    poly = fmaf(t, poly, 0.254829592f);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * z * z));
    const float half_erfc = 0.5f * t * poly * e;  // 0.5 erfc(|x| / sqrt 2)
    const float phi = x < 0.f ? half_erfc : 1.f - half_erfc;
    return x * phi;
}

__device__ __forceinline__ uint4 gelu_bf16x8(const uint4 &u) {
    float f[8];
    bf16x8_to_float(u, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = gelu_erf(f[k]);
    uint4 pk;
    pk.x = float2_to_bf16x2(f[0], f[1]);
    pk.y = float2_to_bf16x2(f[2], f[3]);
    pk.z = float2_to_bf16x2(f[4], f[5]);
    pk.w = float2_to_bf16x2(f[6], f[7]);
    return pk;
}

// Four independent 16-byte loads per thread and step: a B200 needs several MB of loads in flight to cover the HBM
// latency at full bandwidth, more than one load per resident thread provides.
__global__ void __launch_bounds__(ENC_THREADS) gelu_bf16_kernel(const uint4 *__restrict__ x, uint4 *__restrict__ out, long long n8) {
    constexpr int U = 4;
    const long long stride = (long long)gridDim.x * ENC_THREADS * U;
    for (long long i0 = (long long)blockIdx.x * ENC_THREADS * U + threadIdx.x; i0 < n8; i0 += stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = i0 + (long long)u * ENC_THREADS;
            if (i < n8) v[u] = x[i];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long long i = i0 + (long long)u * ENC_THREADS;
            if (i < n8) out[i] = gelu_bf16x8(v[u]);
        }
    }
}

static int gelu_bf16_launch(const void *x, void *out, long long n, int sms, cudaStream_t stream) {
    const long long n8 = n / 8;
    long long blocks = (n8 + ENC_THREADS * 4 - 1) / (ENC_THREADS * 4);  // four 16-byte words per thread and step
    const long long cap = (long long)sms * 8 * 4;  // 8 resident CTAs per SM, a few waves
    if (blocks > cap) blocks = cap;
    gelu_bf16_kernel<<<(unsigned)blocks, ENC_THREADS, 0, stream>>>((const uint4 *)x, (uint4 *)out, n8);
    return (int)cudaPeekAtLastError();
}

}  // namespace pai
