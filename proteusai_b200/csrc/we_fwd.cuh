// Wavefunction Embedding forward for sm_100a.
//
// Work decomposition (replaces the reference's one-CTA-per-observer kernel,
// utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding_kernel.cu:49-292):
//   * a lane owns ONE observer row and a register slice of KS wavenumbers, i.e. 4*KS fp32
//     accumulators (sum mag*cos, sum mag*sin, sum mag*r*cos, sum mag*r*sin) held as packed
//     fp32x2 pairs; nothing is reduced across lanes, so the inner loop has no shuffle, no
//     atomic and no shared-memory write;
//   * a warp is 32 consecutive observers x one wavenumber slice; the 4 warps of a CTA share
//     the observers and take 4 consecutive slices.  An "item" is (batch element, 32-observer
//     block, group of 4 slices); it needs all source tiles of its batch element;
//   * the (item, source tile) pairs form one linear sequence which is cut into equal runs, one
//     per CTA of a grid of (SM count x 4 resident CTAs x a few waves).  Every SM therefore gets
//     the same amount of work whatever the shape or the shard size (with a padding mask, whose runs
//     are very unequal, resident CTAs draw the runs from a global counter instead), at the price of items that
//     straddle a cut: each run adds its partial sums into the zero-filled outputs with fp32
//     reductions, so the last bit of a sum can differ from run to run.  A "reproducible" launch
//     mode keeps every run at least one item long: then an output element receives at most two
//     contributions and the result is bit-identical from run to run (when the shard is large
//     enough for that), at a few per cent of speed;
//   * sources stream through shared memory in tiles: the x/y/z planes arrive by 1-D bulk copies
//     (TMA) into a double-buffered staging area, are repacked once per tile into
//     float4 {x,y,z,valid} so the inner loop reads one broadcast LDS.128 per pair, and tiles
//     without a single valid source are skipped;
//   * per pair the distance is evaluated once (rsqrt + one Newton step, so r is within an ulp
//     of sqrt) and reused by all KS wavenumbers; per (pair, wavenumber) the work is one phase
//     multiply, one sin and one cos on the SFU, and four fused multiply-adds, issued as
//     packed fp32x2 instructions.  The kernel is SFU-bound by construction.
#pragma once
#include "common.cuh"

namespace pai {

constexpr int WE_TJ_MAX = 512;    // sources per staged tile (upper bound; smaller for small problems)
constexpr int WE_WARPS = 4;       // warps (wavenumber slices) per CTA
constexpr int WE_THREADS = WE_WARPS * 32;
constexpr int WE_CTAS_PER_SM = 4;
constexpr int WE_MAX_WAVES = 8;

struct WeFwdParams {
    const float *coords;   // [Z,3,N]
    const uint8_t *valid;  // [Z,N] or nullptr
    const float *wn;       // [K]
    float *out;            // [Z,N,2K]   zero-filled over the row range before the launch
    float *cos_sums;       // [Z,N,K]    "
    float *sin_sums;       // [Z,N,K]    "
    int N, K, row_begin, row_end, mag_type, use_tma;
    int tj;                // sources per tile
    int tiles;             // tiles per item = ceil(N / tj)
    int obs_blocks;        // 32-observer blocks per batch element
    int k_groups;          // groups of WE_WARPS * KS wavenumbers
    long long units;       // Z * obs_blocks * k_groups * tiles
    int nruns;             // the unit sequence is cut into this many equal runs
    uint32_t seed;         // dropout: hash seed,
    uint32_t drop_thr;     //   an evaluation is kept when its hash is >= this,
    float drop_scale;      //   and kept evaluations are scaled by this (1 / (1 - p)); 0 = no dropout
    unsigned *counter;     // zeroed before the launch: CTAs draw run indices from it (nullptr: run = blockIdx.x)
};

struct __align__(16) WeSmem {
    float stage[2][3][WE_TJ_MAX];  // x/y/z planes, two stages
    float4 tile[WE_TJ_MAX];        // repacked {x,y,z,valid}
    uint64_t bar[2];
    int hi[2][8];
    unsigned run;
};

// Final mixing of the reference's dropout hash (hash5, wf_embedding_kernel.cu:27-40); the caller has already
// xor-ed the seed with the four index terms.
__device__ __forceinline__ uint32_t we_hash_mix(uint32_t h) {
    h = (h ^ (h >> 16)) * 0x85ebca6bu;
    h ^= h >> 13;
    h = (h ^ (h >> 16)) * 0xc2b2ae35u;
    h ^= h >> 16;
    return h;
}

// KS: wavenumbers per lane (even).  MAG1: compile-time fast path for magnitude_type == 1.
// RR: reduce the phase to [-pi, pi] explicitly (phase in revolutions, subtract the nearest
//     integer exactly) before the SFU sin/cos, instead of leaving the reduction to the
//     fp32 multiply inside sin.approx/cos.approx.
// NP: of the KS/2 wavenumber pairs of a lane, the first NP are evaluated with the FMA-pipe polynomial
//     (poly_sincos_rev) instead of the SFU: the SFU is the bottleneck and the FMA pipe is half idle.
//     Measured at N = 16384: NP = 1 (one eighth of the evaluations) is 5.6 % faster than NP = 0, NP = 2
//     3 %, NP = 3 slower: the long dependent Horner chains share the in-order issue of each warp with the
//     SFU instructions, so the pipes overlap far less than their idle capacities suggest.
//
// DROP: dropout of single evaluations, as the reference kernel does it (wf_embedding_kernel.cu:27-46,227-232): a
//     hash of (batch element, observer, source, wavenumber index, seed) is mapped to [0, 1] and the evaluation is
//     kept when that is >= p; kept real and imaginary parts (and with them the stored sums) are scaled by 1/(1-p).
//     The comparison (float)h / 2^32 >= p is done on the integer: the host passes the smallest h that passes.
// The body of a warp: KS wavenumbers per lane starting `kslice0` wavenumbers into the CTA's group of `GROUP`; the CTA has
// THREADS threads, all of which walk the same runs, units and barriers whatever their KS and NP.
template <int KS, bool MAG1, bool RR, int NP, bool DROP, int THREADS, int GROUP>
__device__ __forceinline__ void we_fwd_body(const WeFwdParams &p, WeSmem &sm, const int kslice0) {
    constexpr int KP = KS / 2;
    constexpr int NWARPS = THREADS / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = p.N, K = p.K;
    const bool tma = p.use_tma != 0;

    auto issue_tile = [&](long long u, int st) {  // thread 0: bulk-copy the three planes of unit u's tile
        const long long item = u / p.tiles;
        const int tile = (int)(u - item * p.tiles);
        const int zz = (int)(item / ((long long)p.k_groups * p.obs_blocks));
        const int j0 = tile * p.tj;
        const uint32_t bytes = (uint32_t)min(p.tj, N - j0) * 4u;
        const float *src = p.coords + (size_t)zz * 3 * N + j0;
        mbar_expect_tx(&sm.bar[st], 3 * bytes);
#pragma unroll
        for (int c = 0; c < 3; ++c) bulk_g2s(&sm.stage[st][c][0], src + (size_t)c * N, bytes, &sm.bar[st]);
    };

    if (tma) {
        if (tid == 0) {
            mbar_init(&sm.bar[0], 1);
            mbar_init(&sm.bar[1], 1);
            mbar_fence_init();
            fence_proxy_async();
        }
        __syncthreads();
    }

    // state of the current item
    long long cur_item = -1;
    int z = 0, row = 0, k0 = 0;
    bool row_in = false, ov = false, item_live = false;
    float ox = 0.f, oy = 0.f, oz = 0.f;
    uint32_t h_zi = 0u, h_k0 = 0u;  // dropout hash: the (seed, batch element, observer) part and the wavenumber term of k0
    f2_t kk[KP];
    f2_t acc_re[KP], acc_im[KP], acc_c[KP], acc_s[KP];
#pragma unroll
    for (int q = 0; q < KP; ++q) kk[q] = acc_re[q] = acc_im[q] = acc_c[q] = acc_s[q] = 0ull;

    auto flush = [&]() {  // add this run's partial sums of the current item into the outputs
        if (cur_item < 0 || !row_in || !ov) return;  // padded observers keep the zeros
        float *orow = p.out + ((size_t)z * N + row) * 2 * K;
        float *crow = p.cos_sums + ((size_t)z * N + row) * K;
        float *srow = p.sin_sums + ((size_t)z * N + row) * K;
#pragma unroll
        for (int q = 0; q < KP; ++q) {
            const int k = k0 + 2 * q;
            if (k >= K) break;
            float re0, re1, im0, im1, c0, c1, s0, s1;
            f2_unpack(acc_re[q], re0, re1);
            f2_unpack(acc_im[q], im0, im1);
            f2_unpack(acc_c[q], c0, c1);
            f2_unpack(acc_s[q], s0, s1);
            atomicAdd(orow + 2 * k, re0);
            atomicAdd(orow + 2 * k + 1, im0);
            atomicAdd(crow + k, c0);
            atomicAdd(srow + k, s0);
            if (k + 1 < K) {
                atomicAdd(orow + 2 * k + 2, re1);
                atomicAdd(orow + 2 * k + 3, im1);
                atomicAdd(crow + k + 1, c1);
                atomicAdd(srow + k + 1, s1);
            }
        }
    };

    // Runs are drawn from a global counter (padded batches make runs very unequal, so a static assignment would
    // leave SMs idle) or, for reproducible sums, assigned by block index.  n counts the units this CTA has staged
    // so far: it selects the staging buffer and the mbarrier phase across runs.
    bool timed_out = false;
    int n = 0;
    for (;;) {
    unsigned run = blockIdx.x;
    if (p.counter) {
        if (tid == 0) sm.run = atomicAdd(p.counter, 1u);
        __syncthreads();  // (the next write of sm.run comes after the barriers inside the run)
        run = sm.run;
    }
    if (run >= (unsigned)p.nruns) break;
    const long long u0 = p.units * run / p.nruns;
    const long long u1 = p.units * (run + 1) / p.nruns;
    if (tma && tid == 0 && u0 < u1) issue_tile(u0, n & 1);  // that buffer was drained two units ago
    for (long long u = u0; u < u1; ++u, ++n) {
        const int st = n & 1;
        if (tma && tid == 0 && u + 1 < u1) issue_tile(u + 1, st ^ 1);  // stage st^1 was drained by the previous repack
        const long long item = u / p.tiles;
        const int tile = (int)(u - item * p.tiles);
        if (item != cur_item) {
            flush();
            cur_item = item;
            const int kg = (int)(item % p.k_groups);
            const long long rest = item / p.k_groups;
            const int ob = (int)(rest % p.obs_blocks);
            z = (int)(rest / p.obs_blocks);
            row = p.row_begin + ob * 32 + lane;
            k0 = kg * GROUP + kslice0;
            row_in = row < p.row_end;
            const float *czi = p.coords + (size_t)z * 3 * N;
            ov = false;
            ox = oy = oz = 0.f;
            if (row_in) {
                ov = p.valid ? (p.valid[(size_t)z * N + row] != 0) : true;
                if (ov) {
                    ox = czi[row];
                    oy = czi[N + row];
                    oz = czi[2 * N + row];
                }
            }
            item_live = __any_sync(0xffffffffu, ov) && k0 < K;  // the same 32 observers in every warp of the CTA
            if (DROP) {
                h_zi = p.seed ^ ((uint32_t)z * 0x85ebca6bu + 0x9e3779b9u) ^ ((uint32_t)row * 0xc2b2ae35u + 0x165667b1u);
                h_k0 = (uint32_t)k0 * 0x85ebca6bu + 0x1b873593u;
            }
#pragma unroll
            for (int q = 0; q < KP; ++q) {
                float a = (k0 + 2 * q < K) ? p.wn[k0 + 2 * q] : 0.f;
                float b = (k0 + 2 * q + 1 < K) ? p.wn[k0 + 2 * q + 1] : 0.f;
                if (RR || q < NP) {  // wavenumber in revolutions per unit length
                    a = (float)((double)a * 0.15915494309189535);
                    b = (float)((double)b * 0.15915494309189535);
                }
                kk[q] = f2_pack(a, b);
                acc_re[q] = acc_im[q] = acc_c[q] = acc_s[q] = 0ull;
            }
        }
        const int j0 = tile * p.tj;
        const int cnt = min(p.tj, N - j0);
        const float *cz = p.coords + (size_t)z * 3 * N;
        const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

        if (tma) {
            const bool ok = mbar_wait_bounded(&sm.bar[st], (uint32_t)((n >> 1) & 1));
            if (__syncthreads_or(ok ? 0 : 1)) {  // also: everyone is done reading sm.tile
                timed_out = true;
                break;
            }
        } else {
            __syncthreads();  // everyone is done reading sm.tile
        }
        // repack to {x,y,z,valid}; find the end of the valid sources of this tile
        int mine = 0;
        for (int j = tid; j < cnt; j += THREADS) {
            float4 s;
            if (tma) {
                s.x = sm.stage[st][0][j];
                s.y = sm.stage[st][1][j];
                s.z = sm.stage[st][2][j];
            } else {
                s.x = cz[j0 + j];
                s.y = cz[N + j0 + j];
                s.z = cz[2 * N + j0 + j];
            }
            const bool v = vz ? (vz[j0 + j] != 0) : true;
            if (!v) s.x = s.y = s.z = 0.f;  // whatever the padding holds (even NaN) never enters the arithmetic
            s.w = v ? 1.f : 0.f;
            if (v) mine = j + 1;
            sm.tile[j] = s;
        }
        mine = __reduce_max_sync(0xffffffffu, mine);
        if (lane == 0) sm.hi[st][warp] = mine;
        __syncthreads();  // also publishes sm.tile (sm.hi[st] is next written two units later, after two more barriers)
        // sources past the last valid one of the tile (the padded tail of a sample) are not looped over
        int hi = 0;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) hi = max(hi, sm.hi[st][w]);
        if (hi == 0 || !item_live) continue;

#pragma unroll 2
        for (int j = 0; j < hi; ++j) {
            const float4 s = sm.tile[j];
            const float dx = ox - s.x, dy = oy - s.y, dz = oz - s.z;
            const float d2 = (dx * dx + dy * dy + dz * dz) * s.w;  // 0 for padded sources
            const bool m = d2 > 0.f;                                 // excludes j == i and coincident points
            const float y = m ? rsqrtf(d2) : 0.f;
            float r = d2 * y;
            r = fmaf(0.5f * y, fmaf(-r, r, d2), r);  // Newton step: r = sqrt(d2) to within an ulp
            float mag, magr;
            if (MAG1) {
                mag = y;
                magr = m ? 1.f : 0.f;
            } else {
                switch (p.mag_type) {
                    case 0: mag = m ? 1.f : 0.f; break;
                    case 1: mag = y; break;
                    case 2: mag = m ? 1.f / log2f(r) : 0.f; break;
                    default: mag = m ? rsqrtf(r) : 0.f; break;
                }
                magr = mag * r;
            }
            const f2_t r2 = f2_pack(r, r), mag2 = f2_pack(mag, mag), magr2 = f2_pack(magr, magr);
            uint32_t h_j = 0u;
            if (DROP) h_j = h_zi ^ ((uint32_t)(j0 + j) * 0x27d4eb2fu + 0xd6e8feb8u);
#pragma unroll
            for (int q = 0; q < KP; ++q) {
                if (q < NP) {  // FMA-pipe evaluation
                    f2_t s2, c2;
                    poly_sincos_rev(f2_mul(r2, kk[q]), s2, c2);
                    acc_re[q] = f2_fma(c2, mag2, acc_re[q]);
                    acc_im[q] = f2_fma(s2, mag2, acc_im[q]);
                    acc_c[q] = f2_fma(c2, magr2, acc_c[q]);
                    acc_s[q] = f2_fma(s2, magr2, acc_s[q]);
                    continue;
                }
                float pa, pb, sa, ca, sb, cb;
                if (RR) {
                    const f2_t big = f2_pack(12582912.f, 12582912.f);        // 1.5 * 2^23
                    const f2_t tau = f2_pack(6.2831853071795865f, 6.2831853071795865f);
                    const f2_t t2 = f2_mul(r2, kk[q]);                       // revolutions
                    const f2_t n2 = f2_sub(f2_add(t2, big), big);            // nearest integer
                    f2_unpack(f2_mul(f2_sub(t2, n2), tau), pa, pb);          // exact fraction -> radians
                } else {
                    f2_unpack(f2_mul(r2, kk[q]), pa, pb);
                }
                sfu_sincos(pa, sa, ca);
                sfu_sincos(pb, sb, cb);
                f2_t c2 = f2_pack(ca, cb), s2 = f2_pack(sa, sb);
                if (DROP) {
                    const uint32_t ha = we_hash_mix(h_j ^ (h_k0 + (uint32_t)(2 * q) * 0x85ebca6bu));
                    const uint32_t hb = we_hash_mix(h_j ^ (h_k0 + (uint32_t)(2 * q + 1) * 0x85ebca6bu));
                    const f2_t keep2 = f2_pack(ha >= p.drop_thr ? p.drop_scale : 0.f, hb >= p.drop_thr ? p.drop_scale : 0.f);
                    c2 = f2_mul(c2, keep2);
                    s2 = f2_mul(s2, keep2);
                }
                acc_re[q] = f2_fma(c2, mag2, acc_re[q]);
                acc_im[q] = f2_fma(s2, mag2, acc_im[q]);
                acc_c[q] = f2_fma(c2, magr2, acc_c[q]);
                acc_s[q] = f2_fma(s2, magr2, acc_s[q]);
            }
        }
    }
    if (timed_out) break;
    flush();
    cur_item = -1;
    if (!p.counter) break;
    }
    if (timed_out && tid == 0) {
        atomicExch(&g_device_status, (int)PAI_ERR_DEVICE_WAIT_TIMEOUT);
        // the one copy that may still be in flight targets this CTA's shared memory: give it a bounded chance to land
        mbar_wait_bounded(&sm.bar[0], (uint32_t)((n >> 1) & 1), 1u << 12);
        mbar_wait_bounded(&sm.bar[1], (uint32_t)((n >> 1) & 1), 1u << 12);
    }
}

template <int KS, bool MAG1, bool RR, int NP, bool DROP = false>
__global__ void __launch_bounds__(WE_THREADS, WE_CTAS_PER_SM) we_fwd_kernel(const WeFwdParams p) {
    __shared__ WeSmem sm;
    we_fwd_body<KS, MAG1, RR, NP, DROP, WE_THREADS, WE_WARPS * KS>(p, sm, (int)(threadIdx.x >> 5) * KS);
}

// The fast path (1/r magnitude, no dropout) with the two pipes fed by DIFFERENT warps: eight warps per CTA, warp w and
// warp w + 4 sit on the same scheduler and share 16 wavenumbers of the CTA's group of 64; warp w evaluates WE_MIX_SFU of
// them with sin.approx / cos.approx (SFU pipe), warp w + 4 the other WE_MIX_POLY with the polynomial (FMA pipe).  Mixed
// inside one warp the long Horner chains and the SFU instructions queue behind each other in the warp's in-order issue;
// in separate warps the scheduler interleaves them and both pipes stay busy.
constexpr int WE_MIX_SFU = 10, WE_MIX_POLY = 6, WE_MIX_THREADS = 256, WE_MIX_CTAS_PER_SM = 2;
static_assert(WE_MIX_SFU + WE_MIX_POLY == 16, "a warp pair covers 16 wavenumbers");

__global__ void __launch_bounds__(WE_MIX_THREADS, WE_MIX_CTAS_PER_SM) we_fwd_mixed_kernel(const WeFwdParams p) {
    __shared__ WeSmem sm;
    const int warp = threadIdx.x >> 5;
    if (warp < 4) we_fwd_body<WE_MIX_SFU, true, false, 0, false, WE_MIX_THREADS, 64>(p, sm, warp * 16);
    else we_fwd_body<WE_MIX_POLY, true, false, WE_MIX_POLY / 2, false, WE_MIX_THREADS, 64>(p, sm, (warp - 4) * 16 + WE_MIX_SFU);
}

template <int KS, int NP>
static void we_fwd_launch_np(const WeFwdParams &p, bool rr, unsigned grid, cudaStream_t stream) {
    dim3 block(WE_THREADS);
    if (p.drop_scale != 0.f) {  // dropout: all evaluations on the SFU, no explicit range reduction
        if (p.mag_type == 1) we_fwd_kernel<KS, true, false, 0, true><<<grid, block, 0, stream>>>(p);
        else we_fwd_kernel<KS, false, false, 0, true><<<grid, block, 0, stream>>>(p);
        return;
    }
    if (p.mag_type == 1) {
        if (rr) we_fwd_kernel<KS, true, true, NP><<<grid, block, 0, stream>>>(p);
        else we_fwd_kernel<KS, true, false, NP><<<grid, block, 0, stream>>>(p);
    } else {
        if (rr) we_fwd_kernel<KS, false, true, NP><<<grid, block, 0, stream>>>(p);
        else we_fwd_kernel<KS, false, false, NP><<<grid, block, 0, stream>>>(p);
    }
}

template <int KS>
static int we_fwd_launch_ks(WeFwdParams p, int Z, bool rr, int sms, int tj_hint, int waves, bool reproducible, int npoly,
                            bool mixed, unsigned *counter, cudaStream_t stream) {
    const int rows = p.row_end - p.row_begin;
    p.obs_blocks = (rows + 31) / 32;
    p.k_groups = (p.K + WE_WARPS * KS - 1) / (WE_WARPS * KS);  // (the mixed kernel's groups are 64 wide like those of KS = 16)
    const long long items = (long long)Z * p.obs_blocks * p.k_groups;
    const long long resident = (long long)sms * (mixed ? WE_MIX_CTAS_PER_SM : WE_CTAS_PER_SM);
    // tile size: as large as possible while every resident CTA still gets several units
    int tj = WE_TJ_MAX;
    if (tj_hint > 0) {
        tj = tj_hint;
    } else {
        while (tj > 64 && items * ((p.N + tj - 1) / tj) < 8 * resident) tj /= 2;
    }
    p.tj = tj;
    p.tiles = (p.N + tj - 1) / tj;
    p.units = items * p.tiles;
    // Grid = resident CTAs x waves.  Several waves of shorter runs let the hardware scheduler even out
    // SM-to-SM differences and stagger the CTAs that share an SM (measured: +4 % over one wave).
    // With `reproducible` the wave count is limited so that a run stays at least one item long: then at
    // most two runs add into any output element and the result is identical from run to run.
    if (waves <= 0) {
        // (with a padding mask the runs are very unequal: twice as many, shorter ones shorten the tail; measured on
        // 64 chains of 64..1024 padded to 1024: 3.71 ms at 8 runs per slot, 3.51 ms at 16, 3.50 ms at 32)
        waves = (p.valid && !reproducible) ? 2 * WE_MAX_WAVES : WE_MAX_WAVES;
        if (reproducible)
            while (waves > 1 && p.units / (resident * waves) < p.tiles) --waves;
    }
    const long long slots = resident * waves;
    p.nruns = (int)(p.units < slots ? p.units : slots);
    // Runs of equal length: with, say, 1.7 units per run half the runs would be twice as long as the others and the
    // last wave of CTAs ragged; rounding the length up to a whole number of units keeps them alike (a row shard of
    // 2048 of 16384 observers, 1.73 units per run before: 4.03 -> 3.91 ms).
    if (!p.valid && p.nruns > 0) {
        const long long len = (p.units + p.nruns - 1) / p.nruns;
        p.nruns = (int)((p.units + len - 1) / len);
    }
    // Without a mask every run costs the same and one CTA per run, placed by the hardware, is the faster
    // form (30.3 against 30.7 ms at N = 16384); with a mask the runs are very unequal and resident CTAs
    // draw them from the counter instead.
    p.counter = (reproducible || !p.valid) ? nullptr : counter;
    unsigned grid = (unsigned)p.nruns;
    if (p.counter) {  // persistent CTAs drawing runs from the counter
        if (grid > (unsigned)resident) grid = (unsigned)resident;
        cudaError_t ce = cudaMemsetAsync(p.counter, 0, sizeof(unsigned), stream);
        if (ce != cudaSuccess) return (int)ce;
    }
    if (mixed) {
        we_fwd_mixed_kernel<<<grid, WE_MIX_THREADS, 0, stream>>>(p);
        return (int)cudaPeekAtLastError();
    }
    // pairs evaluated on the FMA pipe (KS = 16 has 8 pairs per lane)
    if (KS == 16) {
        switch (npoly) {
            case 0: we_fwd_launch_np<KS, 0>(p, rr, grid, stream); break;
            case 2: we_fwd_launch_np<KS, (KS >= 16 ? 2 : 0)>(p, rr, grid, stream); break;
            case 3: we_fwd_launch_np<KS, (KS >= 16 ? 3 : 0)>(p, rr, grid, stream); break;
            default: we_fwd_launch_np<KS, (KS >= 16 ? 1 : 0)>(p, rr, grid, stream); break;
        }
    } else {
        we_fwd_launch_np<KS, 0>(p, rr, grid, stream);
    }
    return (int)cudaPeekAtLastError();
}

// ks_hint: 0 = choose; otherwise 2, 8 or 16.  tj_hint: 0 = choose; otherwise a multiple of 4 in
// [4, 512].  waves: 0 = choose; otherwise CTAs launched per resident CTA slot.  rr: explicit range reduction.  The three outputs must already be zero over the row range.
// `mixed_ok`: the caller asks for the kernel with separate SFU and polynomial warps (it exists for the 1/r magnitude without
// dropout or explicit range reduction at the default lane width of 16; off by default: it measured 12 % slower at N = 16384).
static int we_fwd_launch(const WeFwdParams &p, int Z, int ks_hint, int tj_hint, int waves, bool reproducible, bool rr,
                         int npoly, bool mixed_ok, int sms, unsigned *counter, cudaStream_t stream) {
    int ks = ks_hint;
    if (ks == 0) ks = p.K >= 64 ? 16 : (p.K >= 32 ? 8 : 2);
    if (tj_hint < 0 || tj_hint > WE_TJ_MAX || (tj_hint & 3) || waves < 0 || waves > 64) return (int)PAI_ERR_UNSUPPORTED;
    const bool mixed = mixed_ok && ks == 16 && ks_hint == 0 && p.mag_type == 1 && !rr && p.drop_scale == 0.f;
    switch (ks) {
        case 16: return we_fwd_launch_ks<16>(p, Z, rr, sms, tj_hint, waves, reproducible, npoly, mixed, counter, stream);
        case 8: return we_fwd_launch_ks<8>(p, Z, rr, sms, tj_hint, waves, reproducible, npoly, false, counter, stream);
        case 2: return we_fwd_launch_ks<2>(p, Z, rr, sms, tj_hint, waves, reproducible, npoly, false, counter, stream);
        default: return (int)PAI_ERR_UNSUPPORTED;
    }
}

}  // namespace pai
