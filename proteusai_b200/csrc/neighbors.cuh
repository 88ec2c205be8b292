// Nearest-neighbour graph and edge features of the reference's FeaturizeProtein
// (utils/model_utils/gnn/gnn.py:97-137), which builds them from an N x N distance matrix, torch.topk and a
// [Z,N,K,4,4,R] broadcast in PyTorch.
//
//   knn_kernel       one warp per node, 8 nodes per CTA: the other nodes' coordinates stream through shared memory in
//                    tiles of 256; each warp keeps its K nearest in a sorted list spread over the lanes (entry r lives
//                    in register r / 32 of lane r % 32) and writes indices and the edge mask.  No N x N matrix exists
//                    anywhere; the coordinates (12 B per node) stay in L2.  Work is N^2 / 32 warp iterations of ~20
//                    instructions: issue bound.
//   edge_rbf_kernel  one warp per edge: the 16 atom-pair distances are computed once per pair and shared by shuffle,
//                    each lane evaluates 8 of the 256 radial basis values and the warp writes the 1 kB feature row
//                    with two fully coalesced 512-byte stores.  HBM-write bound: 4 * A*A*R bytes per edge.
//
// Distances are formed exactly as the reference forms them (differences squared, summed x, y, z in that order, each
// operation rounded to fp32, IEEE square root) so that ordering and thresholds see the same values.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace pai {

constexpr int KNN_THREADS = 256;  // 8 warps = 8 nodes per CTA
constexpr int KNN_MAX_K = 64;

__device__ __forceinline__ float ref_distance2(float ax, float ay, float az, float bx, float by, float bz) {
    const float dx = __fsub_rn(ax, bx), dy = __fsub_rn(ay, by), dz = __fsub_rn(az, bz);
    return __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
}
__device__ __forceinline__ float ref_distance(float ax, float ay, float az, float bx, float by, float bz) {
    return __fsqrt_rn(ref_distance2(ax, ay, az, bx, by, bz));
}

// (value, index) pairs ordered by value, then by index: equal distances keep the lower index first.
__device__ __forceinline__ bool knn_less(float va, int ia, float vb, int ib) { return va < vb || (va == vb && ia < ib); }

// NL = list entries per lane (K <= 32 * NL).
//   valid [Z,N] u8 or nullptr: 0 marks a masked node.  What the reference computes (gnn.py:103-115):
//   * a masked node gets itself as every neighbour and an all-false edge mask;
//   * for an unmasked node i the candidates are all j with d_ij != 0 (masked nodes included: their padding
//     coordinates take part in the selection), the K smallest are taken in ascending order, and an edge is kept when
//     the neighbour is unmasked and d_ij < max_dist; dropped edges point back at i.
template <int NL>
__global__ void __launch_bounds__(KNN_THREADS) knn_kernel(const float *__restrict__ ca, const uint8_t *__restrict__ valid,
                                                          long long *__restrict__ idx_out, uint8_t *__restrict__ mask_out, int N,
                                                          int K, float max_dist) {
    // A CTA is 8 consecutive nodes of one batch element (blockIdx.y), one per warp; the candidates stream through shared
    // memory in tiles of 256 as x / y / z planes, loaded once per CTA and scanned by all 8 warps.
    __shared__ __align__(16) float tx[KNN_THREADS], ty[KNN_THREADS], tz[KNN_THREADS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int z = blockIdx.y;
    const int i = blockIdx.x * (KNN_THREADS / 32) + warp;
    const float *cz = ca + (size_t)z * N * 3;
    const uint8_t *vz = valid ? valid + (size_t)z * N : nullptr;
    const bool in_range = i < N;
    // (a warp without work still takes part in the CTA's barriers)
    const bool active = in_range && !(vz && vz[i] == 0);
    float ix = 0.f, iy = 0.f, iz = 0.f;
    if (active) {
        ix = cz[i * 3];
        iy = cz[i * 3 + 1];
        iz = cz[i * 3 + 2];
    }
    float val[NL];
    int idx[NL];
#pragma unroll
    for (int s = 0; s < NL; ++s) {
        val[s] = INFINITY;
        idx[s] = 0x7fffffff;
    }
    // The admission threshold, kept in every lane: the K-th entry so far, and never more than max_dist -- a neighbour at
    // max_dist or beyond is written as a dropped edge (the node itself, mask 0) whichever node it is, so it need not be
    // found.  thr2 bounds the squared distance from above (with a margin for the rounding of the square root) so that
    // the exact square root is taken only for candidates that can pass.
    float thr_v = max_dist;
    int thr_i = -1;
    float thr2 = max_dist * max_dist * 1.000002f;
    const int ks = (K - 1) >> 5, kl = (K - 1) & 31;  // register and lane of entry K-1

    // Tiles are visited outwards from the CTA's own tile.  The result does not depend on the order (entries are ordered
    // by distance, then index); the cost does: along a chain the sequence neighbours are also the nearest in space, so
    // the threshold is tight after the first tile and almost nothing is inserted later, where a scan from node 0 would
    // meet ever closer candidates and insert most of them.
    const int ntile = (N + KNN_THREADS - 1) / KNN_THREADS;
    const int t_own = (blockIdx.x * (KNN_THREADS / 32)) / KNN_THREADS;
    auto tile_at = [&](int t) {  // t-th tile of the outward order, or -1 when it falls outside the range
        const int tile = (t & 1) ? t_own - ((t + 1) >> 1) : t_own + (t >> 1);
        return (tile < 0 || tile >= ntile) ? -1 : tile;
    };
    float px = 0.f, py = 0.f, pz = 0.f;  // this thread's candidate of the next tile, fetched while the current one is scanned
    auto fetch = [&](int tile) {
        // slots past the end of the batch element hold NaN: their squared distance compares false with every
        // threshold, so the scan needs no bounds test
        const int j = tile * KNN_THREADS + threadIdx.x;
        const bool ok = j < N;
        const float nan = __int_as_float(0x7fc00000);
        px = ok ? cz[j * 3] : nan;
        py = ok ? cz[j * 3 + 1] : nan;
        pz = ok ? cz[j * 3 + 2] : nan;
    };
    int t = 0;
    fetch(t_own);
    while (t < 2 * ntile) {  // (uniform over the CTA)
        const int base = tile_at(t) * KNN_THREADS;
        __syncthreads();  // the previous tile has been scanned by every warp
        tx[threadIdx.x] = px;
        ty[threadIdx.x] = py;
        tz[threadIdx.x] = pz;
        __syncthreads();
        for (++t; t < 2 * ntile && tile_at(t) < 0; ++t) {
        }
        if (t < 2 * ntile) fetch(tile_at(t));
        if (!active) continue;
        const int cnt = min(KNN_THREADS, N - base);
        // 128 candidates per step, four consecutive ones per lane.  The common case costs eight flops and one compare
        // per candidate: squared distances against the squared threshold, one vote of the warp; only when some candidate
        // may enter the list (almost never once the threshold is tight) are square roots taken and candidates looked at
        // one by one.
        for (int b = 0; b < cnt; b += 128) {
            const int l0 = b + 4 * lane;
            const float4 cx = *reinterpret_cast<const float4 *>(&tx[l0]);
            const float4 cy = *reinterpret_cast<const float4 *>(&ty[l0]);
            const float4 cz4 = *reinterpret_cast<const float4 *>(&tz[l0]);
            const float xs[4] = {cx.x, cx.y, cx.z, cx.w}, ys[4] = {cy.x, cy.y, cy.z, cy.w}, zs[4] = {cz4.x, cz4.y, cz4.z, cz4.w};
            bool maybe = false;
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // fused arithmetic is enough for the filter: thr2 carries a margin of 16 ulp
                const float dx = xs[q] - ix, dy = ys[q] - iy, dz = zs[q] - iz;
                maybe |= fmaf(dz, dz, fmaf(dy, dy, dx * dx)) <= thr2;
            }
            if (__ballot_sync(0xffffffffu, maybe) == 0u) continue;
            float d[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {  // now exactly as the reference rounds
                const float s2 = ref_distance2(xs[q], ys[q], zs[q], ix, iy, iz);
                d[q] = INFINITY;
                if (s2 <= thr2 && s2 != 0.f) d[q] = __fsqrt_rn(s2);  // s2 == 0: the node itself and coincident points
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                unsigned pass = __ballot_sync(0xffffffffu, knn_less(d[q], base + l0 + q, thr_v, thr_i));
                while (pass) {
                    const int src = __ffs(pass) - 1;
                    pass &= pass - 1;
                    const float cv = __shfl_sync(0xffffffffu, d[q], src);
                    const int ci = base + b + 4 * src + q;
                    if (!knn_less(cv, ci, thr_v, thr_i)) continue;  // the threshold moved since the vote
                    // rank of the candidate = number of entries below it
                    int p = 0;
#pragma unroll
                    for (int s = 0; s < NL; ++s) p += __popc(__ballot_sync(0xffffffffu, knn_less(val[s], idx[s], cv, ci)));
                    // entries at ranks >= p move up by one, the candidate takes rank p (the last entry falls off)
                    float carry_v = 0.f;
                    int carry_i = 0;
#pragma unroll
                    for (int s = 0; s < NL; ++s) {
                        const int r = s * 32 + lane;
                        float up_v = __shfl_up_sync(0xffffffffu, val[s], 1);
                        int up_i = __shfl_up_sync(0xffffffffu, idx[s], 1);
                        const float last_v = __shfl_sync(0xffffffffu, val[s], 31);
                        const int last_i = __shfl_sync(0xffffffffu, idx[s], 31);
                        if (lane == 0) {
                            up_v = carry_v;  // entry 32 s - 1 lives in lane 31 of the previous register
                            up_i = carry_i;
                        }
                        carry_v = last_v;
                        carry_i = last_i;
                        if (r == p) {
                            val[s] = cv;
                            idx[s] = ci;
                        } else if (r > p) {
                            val[s] = up_v;
                            idx[s] = up_i;
                        }
                    }
#pragma unroll
                    for (int s = 0; s < NL; ++s) {
                        if (s == ks) {
                            const float kv = __shfl_sync(0xffffffffu, val[s], kl);
                            const int ki = __shfl_sync(0xffffffffu, idx[s], kl);
                            if (kv < max_dist) {  // the list holds K entries inside max_dist: its last one is the new threshold
                                thr_v = kv;
                                thr_i = ki;
                                thr2 = kv * kv * 1.000002f;
                            }
                        }
                    }
                }
            }
        }
    }
    if (!in_range) return;
    long long *orow = idx_out + ((long long)z * N + i) * K;
    uint8_t *mrow = mask_out + ((long long)z * N + i) * K;
#pragma unroll
    for (int s = 0; s < NL; ++s) {
        const int r = s * 32 + lane;
        if (r < K) {
            const float v = val[s];
            const int jn = idx[s];
            // A masked node keeps its initial entries; so do the ranks that were not filled from inside max_dist.  Both
            // come out as dropped edges, like the reference's masked rows, its neighbours at max_dist or beyond and its
            // inf values.
            const bool keep = v < max_dist && jn < N && (vz ? vz[jn] != 0 : true);
            orow[r] = keep ? jn : i;
            mrow[r] = keep ? 1 : 0;
        }
    }
}

static int knn_launch(const float *ca, const uint8_t *valid, long long *idx, uint8_t *mask, int Z, int N, int K, float max_dist,
                      cudaStream_t stream) {
    const dim3 grid((unsigned)((N + KNN_THREADS / 32 - 1) / (KNN_THREADS / 32)), (unsigned)Z);
    if (K <= 32) knn_kernel<1><<<grid, KNN_THREADS, 0, stream>>>(ca, valid, idx, mask, N, K, max_dist);
    else knn_kernel<2><<<grid, KNN_THREADS, 0, stream>>>(ca, valid, idx, mask, N, K, max_dist);
    return (int)cudaPeekAtLastError();
}

__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// out[z,i,k,a,b,r] = exp(-(|atoms[z,i,a] - atoms[z,idx[z,i,k],b]| - centers[r])^2 / spread^2), A = 4 atoms per node and
// R = 16 centres (gnn.py:119-131): 256 values per edge, one warp per edge.
// LN: the LayerNorm over the 256 features of an edge that follows in the reference (edge_norm, gnn.py:134) is applied
// before the store -- the warp holds the whole feature row, so mean and variance are two shuffle reductions and the
// features cross HBM once instead of three times (written, read and written again by a separate LayerNorm).
template <bool LN>
__global__ void __launch_bounds__(KNN_THREADS, 8) edge_rbf_4x4x16_kernel(const float *__restrict__ atoms, const long long *__restrict__ idx,
                                                                     const float *__restrict__ centers,
                                                                     float neg_log2e_over_spread2, const float *__restrict__ gamma,
                                                                     const float *__restrict__ beta, float eps,
                                                                     float *__restrict__ out, int N, int K, long long edges) {
    const int lane = threadIdx.x & 31;
    // Lane l computes the distance of atom pair l / 2 (a = l / 8, b = (l / 2) % 4; the two lanes of a pair compute the
    // same value).  It writes features 4 l .. 4 l + 3 (pair l / 4, centres 4 (l % 4) ..) and 128 + 4 l .. (pair 8 + l / 4),
    // so that each of the two stores of a warp covers 512 contiguous bytes.
    const int a = lane >> 3, b = (lane >> 1) & 3, r0 = (lane & 3) * 4;
    const int src_lo = (lane >> 2) * 2, src_hi = 16 + (lane >> 2) * 2;
    float c[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) c[q] = centers[r0 + q];
    // LayerNorm parameters in shared memory (kept out of the registers: 8 CTAs per SM need 32 registers per thread)
    __shared__ float4 s_gamma[64], s_beta[64];
    if (LN) {
        if (threadIdx.x < 64) {
            s_gamma[threadIdx.x] = reinterpret_cast<const float4 *>(gamma)[threadIdx.x];
            s_beta[threadIdx.x] = reinterpret_cast<const float4 *>(beta)[threadIdx.x];
        }
        __syncthreads();
    }
    // 32-bit index arithmetic (the launcher guarantees edges < 2^31): 64-bit divisions cost dozens of instructions each
    const unsigned warps = gridDim.x * (KNN_THREADS / 32);
    const unsigned n_edges = (unsigned)edges, uK = (unsigned)K, uN = (unsigned)N;
    for (unsigned e = blockIdx.x * (KNN_THREADS / 32) + (threadIdx.x >> 5); e < n_edges; e += warps) {
        const unsigned node = e / uK;            // z * N + i
        const unsigned zbase = (node / uN) * uN;  // z * N
        const long long nb = (long long)zbase + idx[e];
        const float *pi = atoms + ((size_t)node * 4 + a) * 3;
        const float *pj = atoms + ((size_t)nb * 4 + b) * 3;
        const float d = ref_distance(pi[0], pi[1], pi[2], pj[0], pj[1], pj[2]);
        const float d_lo = __shfl_sync(0xffffffffu, d, src_lo), d_hi = __shfl_sync(0xffffffffu, d, src_hi);
        float v[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float t0 = d_lo - c[q], t1 = d_hi - c[q];
            v[q] = ex2_fast(t0 * t0 * neg_log2e_over_spread2);
            v[4 + q] = ex2_fast(t1 * t1 * neg_log2e_over_spread2);
        }
        if (LN) {  // biased variance of the centred values, eps inside the square root, as nn.LayerNorm
            float sum = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const float mean = sum * (1.f / 256.f);
            float sq = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                v[q] -= mean;
                sq = fmaf(v[q], v[q], sq);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            const float rstd = rsqrtf(sq * (1.f / 256.f) + eps);
            const float4 g_lo = s_gamma[lane], g_hi = s_gamma[32 + lane], b_lo = s_beta[lane], b_hi = s_beta[32 + lane];
            v[0] = fmaf(v[0] * rstd, g_lo.x, b_lo.x);
            v[1] = fmaf(v[1] * rstd, g_lo.y, b_lo.y);
            v[2] = fmaf(v[2] * rstd, g_lo.z, b_lo.z);
            v[3] = fmaf(v[3] * rstd, g_lo.w, b_lo.w);
            v[4] = fmaf(v[4] * rstd, g_hi.x, b_hi.x);
            v[5] = fmaf(v[5] * rstd, g_hi.y, b_hi.y);
            v[6] = fmaf(v[6] * rstd, g_hi.z, b_hi.z);
            v[7] = fmaf(v[7] * rstd, g_hi.w, b_hi.w);
        }
        float4 *o = reinterpret_cast<float4 *>(out + (size_t)e * 256);
        o[lane] = make_float4(v[0], v[1], v[2], v[3]);
        o[32 + lane] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// any number of atoms per node and centres: one thread per output value (same arithmetic, plain indexing)
__global__ void __launch_bounds__(KNN_THREADS) edge_rbf_generic_kernel(const float *__restrict__ atoms, const long long *__restrict__ idx,
                                                                      const float *__restrict__ centers, float neg_log2e_over_spread2,
                                                                      float *__restrict__ out, int N, int K, int A, int R,
                                                                      long long total) {
    const long long stride = (long long)gridDim.x * KNN_THREADS;
    const int per_edge = A * A * R;
    for (long long t = (long long)blockIdx.x * KNN_THREADS + threadIdx.x; t < total; t += stride) {
        const long long e = t / per_edge;
        const int f = (int)(t - e * per_edge);
        const int a = f / (A * R), b = (f / R) % A, r = f % R;
        const long long node = e / K;
        const long long nb = (node / N) * N + idx[e];
        const float *pi = atoms + (node * A + a) * 3;
        const float *pj = atoms + (nb * A + b) * 3;
        const float d = ref_distance(pi[0], pi[1], pi[2], pj[0], pj[1], pj[2]);
        const float u = d - centers[r];
        out[t] = ex2_fast(u * u * neg_log2e_over_spread2);
    }
}

static int edge_rbf_launch(const float *atoms, const long long *idx, const float *centers, double spread, const float *gamma,
                           const float *beta, float eps, float *out, int Z, int N, int K, int A, int R, int sms,
                           cudaStream_t stream) {
    const long long edges = (long long)Z * N * K;
    // exp(-t^2 / spread^2) = 2^(t^2 * (-log2 e / spread^2)): one multiply and one SFU operation per value.  Against the
    // reference's fp32 division and exp this moves a value by at most ~1e-7 absolute (argument error <= 2 ulp, times
    // arg * exp(-arg) <= 0.37), far inside the 1e-6 the features are compared at.
    const float spread2 = (float)(-1.4426950408889634 / (spread * spread));
    const long long cap = (long long)sms * 8 * 8;
    if (A == 4 && R == 16 && edges < (1ll << 31)) {  // (32-bit edge counter with room for the grid stride)
        long long blocks = (edges + KNN_THREADS / 32 - 1) / (KNN_THREADS / 32);
        if (blocks > cap) blocks = cap;
        if (gamma)
            edge_rbf_4x4x16_kernel<true><<<(unsigned)blocks, KNN_THREADS, 0, stream>>>(atoms, idx, centers, spread2, gamma, beta, eps,
                                                                                        out, N, K, edges);
        else
            edge_rbf_4x4x16_kernel<false><<<(unsigned)blocks, KNN_THREADS, 0, stream>>>(atoms, idx, centers, spread2, nullptr, nullptr,
                                                                                         0.f, out, N, K, edges);
    } else {
        if (gamma) return (int)PAI_ERR_UNSUPPORTED;  // the fused LayerNorm exists for the 4 x 4 x 16 layout only
        const long long total = edges * A * A * R;
        long long blocks = (total + KNN_THREADS - 1) / KNN_THREADS;
        if (blocks > cap) blocks = cap;
        edge_rbf_generic_kernel<<<(unsigned)blocks, KNN_THREADS, 0, stream>>>(atoms, idx, centers, spread2, out, N, K, A, R, total);
    }
    return (int)cudaPeekAtLastError();
}

}  // namespace pai
