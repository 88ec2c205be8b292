// Wavefunction Embedding backward w.r.t. the wavenumbers: an HBM-bound reduction over rows,
//   dk[k] = sum_{z,n} dO[z,n,2k+1] * cos_sums[z,n,k] - dO[z,n,2k] * sin_sums[z,n,k]
// (utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding.py:72-81, three elementwise PyTorch
// kernels and a reduction there).  Two passes so that the result is bit-reproducible: pass 1
// writes one partial row per CTA into the workspace, pass 2 adds the partials in CTA order.
#pragma once
#include "common.cuh"

namespace pai {

constexpr int WE_BWD_THREADS = 256;
constexpr int WE_BWD_MAX_BLOCKS = 592;  // 148 SMs x 4

struct WeBwdParams {
    const float *d_out;     // [Z,N,2K]
    const float *cos_sums;  // [Z,N,K]
    const float *sin_sums;  // [Z,N,K]
    float *partial;         // [blocks,K]
    int N, K, row_begin, rows_per_z, total_rows, rows_per_block, kx;
};

__global__ void __launch_bounds__(WE_BWD_THREADS) we_bwd_partial_kernel(const WeBwdParams p) {
    __shared__ float red[WE_BWD_THREADS];
    const int tid = threadIdx.x;
    const int kx = p.kx, ry = WE_BWD_THREADS / kx;
    const int kl = tid % kx, rl = tid / kx;
    const int r0 = blockIdx.x * p.rows_per_block;
    const int r1 = min(r0 + p.rows_per_block, p.total_rows);
    for (int kb = 0; kb < p.K; kb += kx) {
        const int k = kb + kl;
        float acc = 0.f;
        if (k < p.K) {
#pragma unroll 4
            for (int r = r0 + rl; r < r1; r += ry) {
                const int z = r / p.rows_per_z;
                const size_t row = (size_t)z * p.N + p.row_begin + (r - z * p.rows_per_z);
                const float2 g = *reinterpret_cast<const float2 *>(p.d_out + (row * p.K + k) * 2);
                const float c = p.cos_sums[row * p.K + k];
                const float s = p.sin_sums[row * p.K + k];
                acc = fmaf(g.y, c, acc);
                acc = fmaf(-g.x, s, acc);
            }
        }
        if (ry > 1) {
            red[tid] = acc;
            __syncthreads();
            if (rl == 0) {
                for (int q = 1; q < ry; ++q) acc += red[q * kx + kl];
            }
            __syncthreads();
        }
        if (rl == 0 && k < p.K) p.partial[(size_t)blockIdx.x * p.K + k] = acc;
    }
}

// The same pass with two wavenumbers per thread: one 16-byte load of dO (re, im, re, im) and one 8-byte load of each
// stored sum per row, for even K and suitably aligned pointers.  Fixed order of summation as well (bit-reproducible
// from call to call; the grouping of rows differs from the one-wavenumber kernel's, so the two can differ in the last bits).
__global__ void __launch_bounds__(WE_BWD_THREADS) we_bwd_partial2_kernel(const WeBwdParams p) {
    __shared__ float2 red[WE_BWD_THREADS];
    const int tid = threadIdx.x;
    const int kx = p.kx, ry = WE_BWD_THREADS / kx;  // kx threads cover 2 kx wavenumbers of a row
    const int kl = tid % kx, rl = tid / kx;
    const int r0 = blockIdx.x * p.rows_per_block;
    const int r1 = min(r0 + p.rows_per_block, p.total_rows);
    for (int kb = 0; kb < p.K; kb += 2 * kx) {
        const int k = kb + 2 * kl;
        float a0 = 0.f, a1 = 0.f;
        if (k < p.K) {
#pragma unroll 4
            for (int r = r0 + rl; r < r1; r += ry) {
                const int z = r / p.rows_per_z;
                const size_t row = (size_t)z * p.N + p.row_begin + (r - z * p.rows_per_z);
                const float4 g = *reinterpret_cast<const float4 *>(p.d_out + (row * p.K + k) * 2);
                const float2 c = *reinterpret_cast<const float2 *>(p.cos_sums + row * p.K + k);
                const float2 sn = *reinterpret_cast<const float2 *>(p.sin_sums + row * p.K + k);
                a0 = fmaf(g.y, c.x, a0);
                a0 = fmaf(-g.x, sn.x, a0);
                a1 = fmaf(g.w, c.y, a1);
                a1 = fmaf(-g.z, sn.y, a1);
            }
        }
        if (ry > 1) {
            red[tid] = make_float2(a0, a1);
            __syncthreads();
            if (rl == 0) {
                for (int q = 1; q < ry; ++q) {
                    a0 += red[q * kx + kl].x;
                    a1 += red[q * kx + kl].y;
                }
            }
            __syncthreads();
        }
        if (rl == 0 && k < p.K) {
            p.partial[(size_t)blockIdx.x * p.K + k] = a0;
            p.partial[(size_t)blockIdx.x * p.K + k + 1] = a1;
        }
    }
}

__global__ void __launch_bounds__(WE_BWD_THREADS) we_bwd_final_kernel(const float *partial, float *dk, int K, int blocks) {
    const int k = blockIdx.x * WE_BWD_THREADS + threadIdx.x;
    if (k >= K) return;
    float acc = 0.f;
    for (int b = 0; b < blocks; ++b) acc += partial[(size_t)b * K + k];
    dk[k] = acc;
}

static int we_bwd_launch(const float *d_out, const float *cos_sums, const float *sin_sums, float *dk, float *partial,
                         int Z, int N, int K, int row_begin, int row_end, cudaStream_t stream) {
    WeBwdParams p;
    p.d_out = d_out;
    p.cos_sums = cos_sums;
    p.sin_sums = sin_sums;
    p.partial = partial;
    p.N = N;
    p.K = K;
    p.row_begin = row_begin;
    p.rows_per_z = row_end - row_begin;
    p.total_rows = Z * p.rows_per_z;
    // two wavenumbers per thread when the 16-byte / 8-byte loads are aligned for every row
    const bool vec2 = (K % 2) == 0 && ((uintptr_t)d_out % 16) == 0 && ((uintptr_t)cos_sums % 8) == 0 && ((uintptr_t)sin_sums % 8) == 0;
    const int per_thread = vec2 ? 2 : 1;
    int kx = 32;
    while (kx * per_thread < K && kx < WE_BWD_THREADS) kx *= 2;
    p.kx = kx;
    const int ry = WE_BWD_THREADS / kx;
    int rpb = (p.total_rows + WE_BWD_MAX_BLOCKS - 1) / WE_BWD_MAX_BLOCKS;
    if (rpb < 8 * ry) rpb = 8 * ry;
    p.rows_per_block = rpb;
    const int blocks = (p.total_rows + rpb - 1) / rpb;
    if (vec2) we_bwd_partial2_kernel<<<blocks, WE_BWD_THREADS, 0, stream>>>(p);
    else we_bwd_partial_kernel<<<blocks, WE_BWD_THREADS, 0, stream>>>(p);
    we_bwd_final_kernel<<<(K + WE_BWD_THREADS - 1) / WE_BWD_THREADS, WE_BWD_THREADS, 0, stream>>>(partial, dk, K, blocks);
    return (int)cudaPeekAtLastError();
}

}  // namespace pai
