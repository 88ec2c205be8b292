// Per-batch plan of the geometric-attention kernels: which 128-token tiles of every sample hold a valid
// token, and the samples ordered longest first.  The reference kernel visits every tile of the padded
// sequence (old/old_scripts/attn/geometric_attn.py:183-219 loops over all of N); here tiles without a
// valid token are never loaded, and the CTAs of long samples are issued first so that the short ones
// fill the tail.  One plan serves every layer, head, forward and backward call that shares the mask.
//
// Layout (int32 words):
//   [0] Z   [1] N   [2] tiles per sample T = ceil(N / 128)   [3] arrival counter (0 between launches)
//   order [Z]      sample indices by decreasing number of non-empty tiles (ties: lower index first)
//   count [Z]      number of non-empty tiles of the sample
//   nvalid[Z]      number of valid tokens of the sample
//   tiles [Z][T]   the first count[z] entries: tile index, bit 15 set when the tile also holds a padded
//                  (or out-of-range) token
//   info  [Z][T]   per tile: -1 = no valid token; else offset of its first valid token (0..127), bit 15 as above
#pragma once
#include "common.cuh"

namespace pai {

constexpr int GA_PLAN_TILE = 128;
constexpr int GA_PLAN_MAX_TILES = 1024;
constexpr int GA_PLAN_HEADER = 4;

__host__ __device__ inline int ga_plan_tiles_per_sample(int N) { return (N + GA_PLAN_TILE - 1) / GA_PLAN_TILE; }
__host__ __device__ inline size_t ga_plan_words(int Z, int N) {
    return (size_t)GA_PLAN_HEADER + 3 * (size_t)Z + 2 * (size_t)Z * (size_t)ga_plan_tiles_per_sample(N);
}
__host__ __device__ inline const int *ga_plan_order(const int *plan) { return plan + GA_PLAN_HEADER; }
__host__ __device__ inline const int *ga_plan_count(const int *plan, int Z) { return plan + GA_PLAN_HEADER + Z; }
__host__ __device__ inline const int *ga_plan_nvalid(const int *plan, int Z) { return plan + GA_PLAN_HEADER + 2 * Z; }
__host__ __device__ inline const int *ga_plan_tiles(const int *plan, int Z, int N, int z) {
    return plan + GA_PLAN_HEADER + 3 * (size_t)Z + (size_t)z * ga_plan_tiles_per_sample(N);
}

__host__ __device__ inline const int *ga_plan_info(const int *plan, int Z, int N, int z) {
    const size_t T = ga_plan_tiles_per_sample(N);
    return plan + GA_PLAN_HEADER + 3 * (size_t)Z + (size_t)Z * T + (size_t)z * T;
}
// Tile word of a sequence without a mask: every tile is live, the last one may be ragged.
__host__ __device__ inline int ga_plan_info_unmasked(int N, int tile) {
    const int T = ga_plan_tiles_per_sample(N);
    if (tile >= T) return -1;
    return (tile == T - 1 && (N % GA_PLAN_TILE) != 0) ? 0x8000 : 0;
}

// One CTA per sample scans its mask; the CTA that finishes last orders the samples (counting sort by
// tile count, descending, stable) and clears the arrival counter for the next launch.
__global__ void __launch_bounds__(256) geoattn_plan_kernel(const uint8_t *valid, int *plan, int Z, int N) {
    __shared__ unsigned short flags[GA_PLAN_MAX_TILES];
    __shared__ int hist[GA_PLAN_MAX_TILES + 2];
    __shared__ int s_nvalid, s_last;
    const int z = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int T = ga_plan_tiles_per_sample(N);
    const uint8_t *vz = valid + (size_t)z * N;
    if (tid == 0) s_nvalid = 0;
    __syncthreads();
    int mine = 0;
    int *info = plan + GA_PLAN_HEADER + 3 * (size_t)Z + (size_t)Z * T + (size_t)z * T;
    for (int t = warp; t < T; t += 8) {
        int n_ok = 0, first = GA_PLAN_TILE;
        for (int o = lane; o < GA_PLAN_TILE; o += 32) {
            const int j = t * GA_PLAN_TILE + o;
            if (j < N && vz[j] != 0) {
                ++n_ok;
                first = min(first, o);
            }
        }
        n_ok = __reduce_add_sync(0xffffffffu, n_ok);
        first = __reduce_min_sync(0xffffffffu, first);
        if (lane == 0) {
            flags[t] = n_ok == 0 ? (unsigned short)0 : (unsigned short)(1 | (n_ok < GA_PLAN_TILE ? 0x8000 : 0));
            info[t] = n_ok == 0 ? -1 : (first | (n_ok < GA_PLAN_TILE ? 0x8000 : 0));
            mine += n_ok;
        }
    }
    if (lane == 0 && mine) atomicAdd(&s_nvalid, mine);
    __syncthreads();
    int *order = plan + GA_PLAN_HEADER, *count = order + Z, *nvalid = count + Z;
    int *tiles = plan + GA_PLAN_HEADER + 3 * (size_t)Z + (size_t)z * T;
    if (tid == 0) {
        int n = 0;
        for (int t = 0; t < T; ++t)
            if (flags[t]) tiles[n++] = t | (flags[t] & 0x8000);
        count[z] = n;
        nvalid[z] = s_nvalid;
        plan[0] = Z;
        plan[1] = N;
        plan[2] = T;
        __threadfence();
        s_last = (atomicAdd(plan + 3, 1) == Z - 1) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int c = tid; c < T + 2; c += 256) hist[c] = 0;
    __syncthreads();
    if (tid == 0) {
        const volatile int *cnt = count;
        for (int s = 0; s < Z; ++s) hist[cnt[s]]++;
        int start = 0;
        for (int c = T; c >= 0; --c) {  // descending tile count
            const int n = hist[c];
            hist[c] = start;
            start += n;
        }
        for (int s = 0; s < Z; ++s) order[hist[cnt[s]]++] = s;
        plan[3] = 0;
    }
}

}  // namespace pai
