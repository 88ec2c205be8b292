// Anisotropic Wavefunction Embedding (per-wavenumber C-beta scaling) forward for sm_100a.
//
// Replaces the reference kernel utils/model_utils/wf_embedding/anisotropic/cb_scaling/learnable_wavenumbers/
// cuda/wf_embedding_kernel.cu:31-225: for observer i and source j with R = A_i - A_j, r = |R|, the phase of
// wavenumber k is k * (r - s_k * (R/r . B_j)), B_j being the source's C-beta direction and s_k a learnable
// magnitude; the outputs are sum_j cos/r and sum_j sin/r interleaved, plus, for the O(N) backward, the
// derivatives of every output element w.r.t. s_k and k.
//
// Same structure as the isotropic kernel (we_fwd.cuh): a lane owns one observer and KS wavenumbers, sources
// stream through shared memory in TMA-staged tiles (here six planes, repacked to two float4 per source), the
// (item, tile) sequence is cut into equal runs whose partial sums are added into the zero-filled outputs.
// Per (pair, wavenumber): one sin and one cos on the SFU and ten packed-pair FMA-pipe operations, six of them
// accumulations; pairs with r == 0 or a padded token get weight 0 and contribute nothing.
#pragma once
#include "we_fwd.cuh"

namespace pai {

constexpr int WEA_KS = 8;  // wavenumbers per lane (6 accumulators each)

struct WeAnisoParams {
    const float *coords_a;  // [Z,3,N]
    const float *coords_b;  // [Z,3,N]
    const uint8_t *valid;   // [Z,N] or nullptr
    const float *cb;        // [K]
    const float *wn;        // [K]
    float *out;             // [Z,N,2K]  zero-filled over the row range before the launch
    float *d_cb;            // [Z,N,2K]  "
    float *d_k;             // [Z,N,2K]  "
    int N, K, row_begin, row_end, use_tma;
    int tj, tiles, obs_blocks, k_groups;
    long long units;
    int nruns;          // the unit sequence is cut into this many equal runs
    unsigned *counter;  // zeroed before the launch: CTAs draw run indices from it (nullptr: run = blockIdx.x)
};

struct __align__(16) WeAnisoSmem {
    float stage[2][6][WE_TJ_MAX];  // A x/y/z and B x/y/z planes, two stages
    float4 ta[WE_TJ_MAX];          // {x, y, z, valid}
    float4 tb[WE_TJ_MAX];          // {bx, by, bz, 0}
    uint64_t bar[2];
    int hi[2][WE_WARPS];
    unsigned run;
};

__global__ void __launch_bounds__(WE_THREADS, WE_CTAS_PER_SM) we_aniso_fwd_kernel(const WeAnisoParams p) {
    __shared__ WeAnisoSmem sm;
    constexpr int KS = WEA_KS, KP = KS / 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int N = p.N, K = p.K;
    const bool tma = p.use_tma != 0;

    auto issue_tile = [&](long long u, int st) {  // thread 0: bulk-copy the six planes of unit u's tile
        const long long item = u / p.tiles;
        const int tile = (int)(u - item * p.tiles);
        const int zz = (int)(item / ((long long)p.k_groups * p.obs_blocks));
        const int j0 = tile * p.tj;
        const uint32_t bytes = (uint32_t)min(p.tj, N - j0) * 4u;
        const float *sa = p.coords_a + (size_t)zz * 3 * N + j0;
        const float *sb = p.coords_b + (size_t)zz * 3 * N + j0;
        mbar_expect_tx(&sm.bar[st], 6 * bytes);
#pragma unroll
        for (int c = 0; c < 3; ++c) {
            bulk_g2s(&sm.stage[st][c][0], sa + (size_t)c * N, bytes, &sm.bar[st]);
            bulk_g2s(&sm.stage[st][3 + c][0], sb + (size_t)c * N, bytes, &sm.bar[st]);
        }
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

    long long cur_item = -1;
    int z = 0, row = 0, k0 = 0;
    bool row_in = false, ov = false, item_live = false;
    float ox = 0.f, oy = 0.f, oz = 0.f;
    f2_t kk[KP], ss[KP];                                            // wavenumbers, negated C-beta magnitudes
    // Sums over the sources of cos / r, sin / r (the output), sin b / r, cos b / r and plain sin, cos, with b = R/r . B_j.
    // The two derivative rows follow from them at the flush, because the factors that depend on the wavenumber slot
    // leave the sums: sum k b sin / r = k sum b sin / r, and (r - s b) / r = 1 - s b / r.  That keeps the inner loop at
    // six accumulations with per-pair scalars only.
    f2_t a_re[KP], a_im[KP], a_sr[KP], a_si[KP], a_kr[KP], a_ki[KP];
#pragma unroll
    for (int q = 0; q < KP; ++q) kk[q] = ss[q] = a_re[q] = a_im[q] = a_sr[q] = a_si[q] = a_kr[q] = a_ki[q] = 0ull;

    auto flush = [&]() {
        if (cur_item < 0 || !row_in || !ov) return;
        const size_t base = ((size_t)z * N + row) * 2 * K;
#pragma unroll
        for (int q = 0; q < KP; ++q) {
            const int k = k0 + 2 * q;
            if (k >= K) break;
            float v[6][2];
            f2_unpack(a_re[q], v[0][0], v[0][1]);
            f2_unpack(a_im[q], v[1][0], v[1][1]);
            // sum k b sin / r, sum k b cos / r;  sum (1 - s b / r) sin, sum (1 - s b / r) cos   (ss holds -s)
            f2_unpack(f2_mul(kk[q], a_sr[q]), v[2][0], v[2][1]);
            f2_unpack(f2_mul(kk[q], a_si[q]), v[3][0], v[3][1]);
            f2_unpack(f2_fma(ss[q], a_sr[q], a_kr[q]), v[4][0], v[4][1]);
            f2_unpack(f2_fma(ss[q], a_si[q], a_ki[q]), v[5][0], v[5][1]);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (k + e >= K) break;
                atomicAdd(p.out + base + 2 * (k + e), v[0][e]);
                atomicAdd(p.out + base + 2 * (k + e) + 1, v[1][e]);
                atomicAdd(p.d_cb + base + 2 * (k + e), v[2][e]);        // d Re / d s_k =  sum k b sin / r
                atomicAdd(p.d_cb + base + 2 * (k + e) + 1, -v[3][e]);   // d Im / d s_k = -sum k b cos / r
                atomicAdd(p.d_k + base + 2 * (k + e), -v[4][e]);        // d Re / d k   = -sum (r - s b) sin / r
                atomicAdd(p.d_k + base + 2 * (k + e) + 1, v[5][e]);     // d Im / d k   =  sum (r - s b) cos / r
            }
        }
    };

    // Runs are assigned by block index or, with a padding mask (very unequal runs), drawn from a global counter by
    // persistent CTAs.  n counts the units this CTA has staged: it selects the buffer and the mbarrier phase.
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
            k0 = (kg * WE_WARPS + warp) * KS;
            row_in = row < p.row_end;
            const float *czi = p.coords_a + (size_t)z * 3 * N;
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
            item_live = __any_sync(0xffffffffu, ov) && k0 < K;
#pragma unroll
            for (int q = 0; q < KP; ++q) {
                const int k = k0 + 2 * q;
                kk[q] = f2_pack(k < K ? p.wn[k] : 0.f, k + 1 < K ? p.wn[k + 1] : 0.f);
                ss[q] = f2_pack(k < K ? -p.cb[k] : 0.f, k + 1 < K ? -p.cb[k + 1] : 0.f);
                a_re[q] = a_im[q] = a_sr[q] = a_si[q] = a_kr[q] = a_ki[q] = 0ull;
            }
        }
        const int j0 = tile * p.tj;
        const int cnt = min(p.tj, N - j0);
        const float *ca = p.coords_a + (size_t)z * 3 * N;
        const float *cb = p.coords_b + (size_t)z * 3 * N;
        const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;
        if (tma) {
            const bool ok = mbar_wait_bounded(&sm.bar[st], (uint32_t)((n >> 1) & 1));
            if (__syncthreads_or(ok ? 0 : 1)) {
                timed_out = true;
                break;
            }
        } else {
            __syncthreads();
        }
        int mine = 0;
        for (int j = tid; j < cnt; j += WE_THREADS) {
            float4 a, b;
            if (tma) {
                a = make_float4(sm.stage[st][0][j], sm.stage[st][1][j], sm.stage[st][2][j], 0.f);
                b = make_float4(sm.stage[st][3][j], sm.stage[st][4][j], sm.stage[st][5][j], 0.f);
            } else {
                a = make_float4(ca[j0 + j], ca[N + j0 + j], ca[2 * N + j0 + j], 0.f);
                b = make_float4(cb[j0 + j], cb[N + j0 + j], cb[2 * N + j0 + j], 0.f);
            }
            const bool v = vz ? (vz[j0 + j] != 0) : true;
            if (!v) {
                a = make_float4(0.f, 0.f, 0.f, 0.f);
                b = a;
            }
            a.w = v ? 1.f : 0.f;
            if (v) mine = j + 1;
            sm.ta[j] = a;
            sm.tb[j] = b;
        }
        mine = __reduce_max_sync(0xffffffffu, mine);
        if (lane == 0) sm.hi[st][warp] = mine;
        __syncthreads();  // also publishes the tile
        // sources past the last valid one of the tile (the padded tail of a sample) are not looped over
        const int hi = max(max(sm.hi[st][0], sm.hi[st][1]), max(sm.hi[st][2], sm.hi[st][3]));
        if (hi == 0 || !item_live) continue;

#pragma unroll 2
        for (int j = 0; j < hi; ++j) {
            const float4 s = sm.ta[j], bj = sm.tb[j];
            const float dx = ox - s.x, dy = oy - s.y, dz = oz - s.z;  // R = A_i - A_j
            const float d2 = (dx * dx + dy * dy + dz * dz) * s.w;
            const bool m = d2 > 0.f;
            const float inv = m ? rsqrtf(d2) : 0.f;
            float r = d2 * inv;
            r = fmaf(0.5f * inv, fmaf(-r, r, d2), r);
            const float binv = (dx * bj.x + dy * bj.y + dz * bj.z) * inv * inv;  // (R/r . B_j) / r
            const float b = binv * r;                                              // R/r . B_j
            const float one = m ? 1.f : 0.f;
            const f2_t r2 = f2_pack(r, r), b2 = f2_pack(b, b), inv2 = f2_pack(inv, inv), binv2 = f2_pack(binv, binv),
                       one2 = f2_pack(one, one);
#pragma unroll
            for (int q = 0; q < KP; ++q) {
                const f2_t w2 = f2_fma(ss[q], b2, r2);  // r - s_k b
                float pa, pb, sa, ca2, sb, cb2;
                f2_unpack(f2_mul(w2, kk[q]), pa, pb);
                sfu_sincos(pa, sa, ca2);
                sfu_sincos(pb, sb, cb2);
                const f2_t c2 = f2_pack(ca2, cb2), s2 = f2_pack(sa, sb);
                a_re[q] = f2_fma(c2, inv2, a_re[q]);
                a_im[q] = f2_fma(s2, inv2, a_im[q]);
                a_sr[q] = f2_fma(s2, binv2, a_sr[q]);
                a_si[q] = f2_fma(c2, binv2, a_si[q]);
                a_kr[q] = f2_fma(s2, one2, a_kr[q]);
                a_ki[q] = f2_fma(c2, one2, a_ki[q]);
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
        // the copies that may still be in flight target this CTA's shared memory: give them a bounded chance to land
        mbar_wait_bounded(&sm.bar[0], (uint32_t)((n >> 1) & 1), 1u << 12);
        mbar_wait_bounded(&sm.bar[1], (uint32_t)((n >> 1) & 1), 1u << 12);
    }
}

static int we_aniso_fwd_launch(WeAnisoParams p, int Z, int sms, unsigned *counter, cudaStream_t stream) {
    const int rows = p.row_end - p.row_begin;
    p.obs_blocks = (rows + 31) / 32;
    p.k_groups = (p.K + WE_WARPS * WEA_KS - 1) / (WE_WARPS * WEA_KS);
    const long long items = (long long)Z * p.obs_blocks * p.k_groups;
    const long long resident = (long long)sms * WE_CTAS_PER_SM;
    int tj = WE_TJ_MAX;
    while (tj > 64 && items * ((p.N + tj - 1) / tj) < 8 * resident) tj /= 2;
    p.tj = tj;
    p.tiles = (p.N + tj - 1) / tj;
    p.units = items * p.tiles;
    const long long slots = resident * (p.valid ? 2 * WE_MAX_WAVES : WE_MAX_WAVES);  // unequal runs: more, shorter ones
    p.nruns = (int)(p.units < slots ? p.units : slots);
    if (!p.valid && p.nruns > 0) {  // runs of equal length (a whole number of units), as in the isotropic launcher
        const long long len = (p.units + p.nruns - 1) / p.nruns;
        p.nruns = (int)((p.units + len - 1) / len);
    }
    p.counter = p.valid ? counter : nullptr;
    unsigned grid = (unsigned)p.nruns;
    if (p.counter) {
        if (grid > (unsigned)resident) grid = (unsigned)resident;
        cudaError_t ce = cudaMemsetAsync(p.counter, 0, sizeof(unsigned), stream);
        if (ce != cudaSuccess) return (int)ce;
    }
    we_aniso_fwd_kernel<<<grid, WE_THREADS, 0, stream>>>(p);
    return (int)cudaPeekAtLastError();
}

// d_cb[k] = sum_{z,n} dO[z,n,2k] P[z,n,2k] + dO[z,n,2k+1] P[z,n,2k+1] for the two stored partial arrays P = d_cb, d_k
// (the reference's backward, .../learnable_wavenumbers/cuda/wf_embedding.py:66-79).  Same two-pass scheme as the
// isotropic backward: per-CTA partial rows, then a fixed-order sum.
struct WeAnisoBwdParams {
    const float *d_out, *pcb, *pk;  // [Z,N,2K] each
    float *partial;                 // [blocks, 2, K]
    int N, K, row_begin, rows_per_z, total_rows, rows_per_block, kx;
};

__global__ void __launch_bounds__(WE_BWD_THREADS) we_aniso_bwd_partial_kernel(const WeAnisoBwdParams p) {
    __shared__ float red[2][WE_BWD_THREADS];
    const int tid = threadIdx.x;
    const int kx = p.kx, ry = WE_BWD_THREADS / kx;
    const int kl = tid % kx, rl = tid / kx;
    const int r0 = blockIdx.x * p.rows_per_block;
    const int r1 = min(r0 + p.rows_per_block, p.total_rows);
    for (int kb = 0; kb < p.K; kb += kx) {
        const int k = kb + kl;
        float acc_s = 0.f, acc_k = 0.f;
        if (k < p.K) {
#pragma unroll 4
            for (int r = r0 + rl; r < r1; r += ry) {
                const int z = r / p.rows_per_z;
                const size_t row = (size_t)z * p.N + p.row_begin + (r - z * p.rows_per_z);
                const size_t off = (row * p.K + k) * 2;
                const float2 g = *reinterpret_cast<const float2 *>(p.d_out + off);
                const float2 a = *reinterpret_cast<const float2 *>(p.pcb + off);
                const float2 b = *reinterpret_cast<const float2 *>(p.pk + off);
                acc_s = fmaf(g.x, a.x, fmaf(g.y, a.y, acc_s));
                acc_k = fmaf(g.x, b.x, fmaf(g.y, b.y, acc_k));
            }
        }
        if (ry > 1) {
            red[0][tid] = acc_s;
            red[1][tid] = acc_k;
            __syncthreads();
            if (rl == 0) {
                for (int q = 1; q < ry; ++q) {
                    acc_s += red[0][q * kx + kl];
                    acc_k += red[1][q * kx + kl];
                }
            }
            __syncthreads();
        }
        if (rl == 0 && k < p.K) {
            p.partial[((size_t)blockIdx.x * 2) * p.K + k] = acc_s;
            p.partial[((size_t)blockIdx.x * 2 + 1) * p.K + k] = acc_k;
        }
    }
}

__global__ void __launch_bounds__(WE_BWD_THREADS) we_aniso_bwd_final_kernel(const float *partial, float *dcb, float *dk, int K,
                                                                             int blocks) {
    const int k = blockIdx.x * WE_BWD_THREADS + threadIdx.x;
    if (k >= K) return;
    float a = 0.f, b = 0.f;
    for (int i = 0; i < blocks; ++i) {
        a += partial[((size_t)i * 2) * K + k];
        b += partial[((size_t)i * 2 + 1) * K + k];
    }
    dcb[k] = a;
    dk[k] = b;
}

static int we_aniso_bwd_launch(const float *d_out, const float *pcb, const float *pk, float *dcb, float *dk, float *partial, int Z,
                               int N, int K, int row_begin, int row_end, cudaStream_t stream) {
    WeAnisoBwdParams p;
    p.d_out = d_out;
    p.pcb = pcb;
    p.pk = pk;
    p.partial = partial;
    p.N = N;
    p.K = K;
    p.row_begin = row_begin;
    p.rows_per_z = row_end - row_begin;
    p.total_rows = Z * p.rows_per_z;
    int kx = 32;
    while (kx < K && kx < WE_BWD_THREADS) kx *= 2;
    p.kx = kx;
    const int ry = WE_BWD_THREADS / kx;
    int rpb = (p.total_rows + WE_BWD_MAX_BLOCKS - 1) / WE_BWD_MAX_BLOCKS;
    if (rpb < 8 * ry) rpb = 8 * ry;
    p.rows_per_block = rpb;
    const int blocks = (p.total_rows + rpb - 1) / rpb;
    we_aniso_bwd_partial_kernel<<<blocks, WE_BWD_THREADS, 0, stream>>>(p);
    we_aniso_bwd_final_kernel<<<(K + WE_BWD_THREADS - 1) / WE_BWD_THREADS, WE_BWD_THREADS, 0, stream>>>(partial, dcb, dk, K, blocks);
    return (int)cudaPeekAtLastError();
}

}  // namespace pai
