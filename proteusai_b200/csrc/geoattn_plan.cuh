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

// ---- balanced schedule ------------------------------------------------------------------------------
// The attention kernels' work items are (sample, head, 128-token tile) triples whose cost grows with the sample's
// number of non-empty tiles.  A grid with one CTA per item leaves the pairing of long and short items on an SM to
// the order in which SMs happen to fall free; on a batch of mixed lengths the busiest SM then carries a third more
// than the average.  The schedule packs the live items into `bins` persistent CTAs beforehand so that the fullest
// carries as little as possible (every item also pays a fixed set-up cost).  Tiles without a
// valid token only need zeros written: they are listed separately and shared out round-robin.
//
// Layout (int32 words):
//   [0] bins  [1] H  [2] Z  [3] N  [4] cap = slots per bin  [5] number of dead items  [6] number of live items  [7] capacity found
//   count[bins]          live items of the bin
//   items[bins][cap]     (sample * H + head) << 10 | tile
//   dead [Z * H * T]     the first [5] entries: dead items, same packing
constexpr int GA_SCHED_HEADER = 8;
constexpr int GA_SCHED_MAX_BINS = 1024;
__host__ __device__ inline int ga_sched_cap(int Z, int N, int H, int bins) {
    const long long items = (long long)Z * H * ga_plan_tiles_per_sample(N);
    return (int)(4 * ((items + bins - 1) / bins) + 8);
}
__host__ __device__ inline size_t ga_sched_words(int Z, int N, int H, int bins) {
    return (size_t)GA_SCHED_HEADER + (size_t)bins + (size_t)bins * ga_sched_cap(Z, N, H, bins) +
           (size_t)Z * H * ga_plan_tiles_per_sample(N);
}
__host__ __device__ inline const int *ga_sched_count(const int *sched) { return sched + GA_SCHED_HEADER; }
__host__ __device__ inline const int *ga_sched_items(const int *sched, int bin) {
    return sched + GA_SCHED_HEADER + sched[0] + (size_t)bin * sched[4];
}
__host__ __device__ inline const int *ga_sched_dead(const int *sched) {
    return sched + GA_SCHED_HEADER + sched[0] + (size_t)sched[0] * sched[4];
}

// One CTA of 1024 threads; thread b keeps the load of bin b.  `tile_cost`, `item_cost`: cost of one non-empty tile
// of the sample and fixed cost of an item, in the same (arbitrary) unit.
// The items are packed by first fit, longest first, into bins of capacity C, and C is bisected down to the smallest
// capacity for which every item finds a bin (MULTIFIT).  The H x count[z] items of a sample cost the same, and first fit
// places a run of equal items by filling the bins in index order with as many as each has room for: one prefix sum
// over the bins per sample instead of one search per item, which keeps the kernel at a few tens of microseconds
// (it runs once per mask, head count and direction).
// With `pair` the bins of the packing are SMs that run two CTAs each: the items of SM b are dealt, longest first, to the
// lighter of CTAs b and b + bins / 2 (a guess at which CTAs share an SM; where it is wrong only the balance suffers).
__device__ inline int ga_block_scan_1024(int v, int *warp_sums, int &total) {  // exclusive prefix sum over the CTA
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
    }
    __syncthreads();  // (the previous scan's sums have been read)
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int w = warp_sums[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, w, off);
        if (lane >= off) w += n;
    }
    total = __shfl_sync(0xffffffffu, w, 31);
    const int before = __shfl_sync(0xffffffffu, w, max(warp - 1, 0));
    return incl - v + (warp > 0 ? before : 0);
}

__global__ void __launch_bounds__(1024) geoattn_schedule_kernel(const int *plan, int *sched, int Z, int N, int H, int bins, int tile_cost,
                                                                int item_cost, int pair) {
    __shared__ int warp_sums[32];
    __shared__ int dead_n;
    const int tid = threadIdx.x;
    const int T = ga_plan_tiles_per_sample(N);
    const int cap = ga_sched_cap(Z, N, H, bins);
    const int nb = pair ? bins / 2 : bins;        // bins of the packing
    const int limit = pair ? 2 * cap - 2 : cap;   // items a bin of the packing can list
    int *count = sched + GA_SCHED_HEADER, *items = count + bins, *dead = items + (size_t)bins * cap;
    const int *order = ga_plan_order(plan), *cnt = ga_plan_count(plan, Z);
    // totals: lower bound of the capacity
    long long total_cost = 0;
    int biggest = 0, n_live = 0;
    for (int s = 0; s < Z; ++s) {
        const int c = cnt[order[s]];
        const int cost = c * tile_cost + item_cost;
        n_live += c * H;
        total_cost += (long long)c * H * cost;
        if (c > 0) biggest = max(biggest, cost);
    }
    // first fit with capacity 2 x (lower bound) + 1 always succeeds: a bin that refuses an item is more than half full
    int lo = (int)max((long long)biggest, (total_cost + nb - 1) / nb), hi = 2 * lo + 1;
    for (int pass = 0; pass <= 12; ++pass) {  // pass < 12: bisection (nothing is written); the last pass writes the lists
        const bool last = pass == 12;
        const int C = last ? hi : (lo + hi) / 2;
        int load = 0, mine = 0, load2[2] = {0, 0}, mine2[2] = {0, 0};
        bool fail = false;
        for (int s = 0; s < Z && !fail; ++s) {  // samples, longest first: a run of c * H equal items
            const int z = order[s], c = cnt[z];
            if (c == 0) continue;
            const int cost = c * tile_cost + item_cost;
            int m = c * H, done = 0;
            // round 0: by capacity; round 1 (last pass only, cannot happen with the capacity found unless the lists are
            // full): any bin with a free slot, so that no item is ever left out
            for (int round = 0; round < 2 && m > 0; ++round) {
                int room = 0;
                if (tid < nb) room = round == 0 ? (load <= C ? min((C - load) / cost, limit - mine) : 0) : limit - mine;
                int total;
                const int before = ga_block_scan_1024(room, warp_sums, total);
                const int take = max(0, min(room, m - before));
                if (take > 0) {
                    if (last) {
                        const int *tl = ga_plan_tiles(plan, Z, N, z);
                        for (int i = 0; i < take; ++i) {
                            const int idx = done + before + i;  // item of the run: head idx / c, its (idx % c)-th non-empty tile
                            const int item = ((z * H + idx / c) << 10) | (tl[idx % c] & 0x3ff);
                            const int half = (pair && load2[1] < load2[0] && mine2[1] < cap) || (pair && mine2[0] >= cap) ? 1 : 0;
                            items[(size_t)(tid + half * nb) * cap + mine2[half]] = item;
                            ++mine2[half];
                            load2[half] += cost;
                        }
                    }
                    load += take * cost;
                    mine += take;
                }
                done += min(total, m);
                m -= min(total, m);
                if (!last) break;
            }
            if (m > 0) fail = true;  // (the same for every thread)
        }
        if (last) {
            if (tid < nb) {
                count[tid] = mine2[0];
                if (pair) count[tid + nb] = mine2[1];
            }
            if (pair && (bins & 1) && tid == 0) count[bins - 1] = 0;
        } else if (fail) {
            lo = C + 1;
        } else {
            hi = C;
        }
        if (!last && lo >= hi) pass = 11;  // converged: the next pass is the last
    }
    // tiles without a valid token, in any order
    if (tid == 0) dead_n = 0;
    __syncthreads();
    for (int e = tid; e < Z * H * T; e += 1024) {
        const int x = e % T, zh = e / T, z = zh / H;
        if (ga_plan_info(plan, Z, N, z)[x] < 0) dead[atomicAdd(&dead_n, 1)] = (zh << 10) | x;
    }
    __syncthreads();
    if (tid == 0) {
        sched[0] = bins;
        sched[1] = H;
        sched[2] = Z;
        sched[3] = N;
        sched[4] = cap;
        sched[5] = dead_n;
        sched[6] = n_live;
        sched[7] = hi;
    }
}

}  // namespace pai
