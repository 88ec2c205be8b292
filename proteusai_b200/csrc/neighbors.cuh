// Nearest-neighbour graph and edge features of the reference's FeaturizeProtein
// (utils/model_utils/gnn/gnn.py:97-137), which builds them from an N x N distance matrix, torch.topk and a
// [Z,N,K,4,4,R] broadcast in PyTorch.
//
//   knn_kernel       one warp per node: streams the other nodes' coordinates, keeps the K nearest in a sorted list
//                    spread over the lanes (entry r lives in register r / 32 of lane r % 32), and writes indices and
//                    the edge mask.  No N x N matrix exists anywhere; the coordinates (12 B per node) stay in L2.
//                    Work is N^2 / 32 warp iterations of ~25 instructions: latency/issue bound, ~0.2 ms at N = 16384.
//   edge_rbf_kernel  one warp per edge: lane l computes the distance of atom pair l / 2 and 8 of its 16 radial basis
//                    values, so a warp writes the 1 kB feature row of the edge with two coalesced 16-byte stores per
//                    lane.  HBM-write bound: 4 * A*A*R bytes per edge.
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

__device__ __forceinline__ float ref_distance(float ax, float ay, float az, float bx, float by, float bz) {
    const float dx = __fsub_rn(ax, bx), dy = __fsub_rn(ay, by), dz = __fsub_rn(az, bz);
    const float s = __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
    return __fsqrt_rn(s);
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
                                                          long long *__restrict__ idx_out, uint8_t *__restrict__ mask_out, int Z,
                                                          int N, int K, float max_dist) {
    const int lane = threadIdx.x & 31;
    const long long node = (long long)blockIdx.x * (KNN_THREADS / 32) + (threadIdx.x >> 5);
    if (node >= (long long)Z * N) return;
    const int z = (int)(node / N), i = (int)(node - (long long)z * N);
    const float *cz = ca + (size_t)z * N * 3;
    const uint8_t *vz = valid ? valid + (size_t)z * N : nullptr;
    long long *orow = idx_out + node * K;
    uint8_t *mrow = mask_out + node * K;
    if (vz && vz[i] == 0) {
        for (int r = lane; r < K; r += 32) {
            orow[r] = i;
            mrow[r] = 0;
        }
        return;
    }
    const float ix = cz[i * 3], iy = cz[i * 3 + 1], iz = cz[i * 3 + 2];
    float val[NL];
    int idx[NL];
#pragma unroll
    for (int s = 0; s < NL; ++s) {
        val[s] = INFINITY;
        idx[s] = 0x7fffffff;
    }
    // the K-th entry so far (the admission threshold), kept in every lane
    float thr_v = INFINITY;
    int thr_i = 0x7fffffff;
    const int ks = (K - 1) >> 5, kl = (K - 1) & 31;  // register and lane of entry K-1

    for (int j0 = 0; j0 < N; j0 += 32) {
        const int j = j0 + lane;
        float d = INFINITY;
        if (j < N) {
            d = ref_distance(cz[j * 3], cz[j * 3 + 1], cz[j * 3 + 2], ix, iy, iz);
            if (d == 0.f) d = INFINITY;  // the node itself and coincident points
        }
        unsigned pass = __ballot_sync(0xffffffffu, j < N && knn_less(d, j, thr_v, thr_i));
        while (pass) {
            const int src = __ffs(pass) - 1;
            pass &= pass - 1;
            const float cv = __shfl_sync(0xffffffffu, d, src);
            const int ci = j0 + src;
            if (!knn_less(cv, ci, thr_v, thr_i)) continue;  // the threshold moved since the ballot
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
                    thr_v = __shfl_sync(0xffffffffu, val[s], kl);
                    thr_i = __shfl_sync(0xffffffffu, idx[s], kl);
                }
            }
        }
    }
#pragma unroll
    for (int s = 0; s < NL; ++s) {
        const int r = s * 32 + lane;
        if (r < K) {
            const float v = val[s];
            const int jn = idx[s];
            // fewer than K candidates leave (inf, -) entries: they fail the distance test like the reference's inf values
            const bool keep = v < max_dist && jn < N && (vz ? vz[jn] != 0 : true);
            orow[r] = keep ? jn : i;
            mrow[r] = keep ? 1 : 0;
        }
    }
}

static int knn_launch(const float *ca, const uint8_t *valid, long long *idx, uint8_t *mask, int Z, int N, int K, float max_dist,
                      cudaStream_t stream) {
    const long long nodes = (long long)Z * N;
    const unsigned grid = (unsigned)((nodes + KNN_THREADS / 32 - 1) / (KNN_THREADS / 32));
    if (K <= 32) knn_kernel<1><<<grid, KNN_THREADS, 0, stream>>>(ca, valid, idx, mask, Z, N, K, max_dist);
    else knn_kernel<2><<<grid, KNN_THREADS, 0, stream>>>(ca, valid, idx, mask, Z, N, K, max_dist);
    return (int)cudaPeekAtLastError();
}

// out[z,i,k,a,b,r] = exp(-(|atoms[z,i,a] - atoms[z,idx[z,i,k],b]| - centers[r])^2 / spread^2), A = 4 atoms per node and
// R = 16 centres (gnn.py:119-131): 256 values per edge, one warp per edge, lane l -> pair (a, b) = (l / 8, (l / 2) % 4),
// centres 8 (l % 2) .. 8 (l % 2) + 7.
__global__ void __launch_bounds__(KNN_THREADS) edge_rbf_4x4x16_kernel(const float *__restrict__ atoms, const long long *__restrict__ idx,
                                                                     const float *__restrict__ centers, float spread2,
                                                                     float *__restrict__ out, int N, int K, long long edges) {
    const int lane = threadIdx.x & 31;
    const int a = lane >> 3, b = (lane >> 1) & 3, r0 = (lane & 1) * 8;
    float c[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) c[q] = centers[r0 + q];
    const long long warps = (long long)gridDim.x * (KNN_THREADS / 32);
    for (long long e = (long long)blockIdx.x * (KNN_THREADS / 32) + (threadIdx.x >> 5); e < edges; e += warps) {
        const long long node = e / K;          // z * N + i
        const long long zbase = (node / N) * N;  // z * N
        const long long nb = zbase + idx[e];
        const float *pi = atoms + (node * 4 + a) * 3;
        const float *pj = atoms + (nb * 4 + b) * 3;
        const float d = ref_distance(pi[0], pi[1], pi[2], pj[0], pj[1], pj[2]);
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float t = __fsub_rn(d, c[q]);
            v[q] = expf(__fdiv_rn(-__fmul_rn(t, t), spread2));
        }
        float4 *o = reinterpret_cast<float4 *>(out + e * 256 + lane * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// any number of atoms per node and centres: one thread per output value (same arithmetic, plain indexing)
__global__ void __launch_bounds__(KNN_THREADS) edge_rbf_generic_kernel(const float *__restrict__ atoms, const long long *__restrict__ idx,
                                                                      const float *__restrict__ centers, float spread2,
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
        const float u = __fsub_rn(d, centers[r]);
        out[t] = expf(__fdiv_rn(-__fmul_rn(u, u), spread2));
    }
}

static int edge_rbf_launch(const float *atoms, const long long *idx, const float *centers, double spread, float *out, int Z, int N,
                           int K, int A, int R, int sms, cudaStream_t stream) {
    const long long edges = (long long)Z * N * K;
    const float spread2 = (float)(spread * spread);  // the reference squares a Python float, then divides fp32 tensors by it
    const long long cap = (long long)sms * 8 * 8;
    if (A == 4 && R == 16) {
        long long blocks = (edges + KNN_THREADS / 32 - 1) / (KNN_THREADS / 32);
        if (blocks > cap) blocks = cap;
        edge_rbf_4x4x16_kernel<<<(unsigned)blocks, KNN_THREADS, 0, stream>>>(atoms, idx, centers, spread2, out, N, K, edges);
    } else {
        const long long total = edges * A * A * R;
        long long blocks = (total + KNN_THREADS - 1) / KNN_THREADS;
        if (blocks > cap) blocks = cap;
        edge_rbf_generic_kernel<<<(unsigned)blocks, KNN_THREADS, 0, stream>>>(atoms, idx, centers, spread2, out, N, K, A, R, total);
    }
    return (int)cudaPeekAtLastError();
}

}  // namespace pai
