// Wavefunction Embedding forward for sm_100a.
//
// Work decomposition (replaces the reference's one-CTA-per-observer kernel,
// utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding_kernel.cu:49-292):
//   * a lane owns ONE observer row and a register slice of KS wavenumbers, i.e. 4*KS fp32
//     accumulators (sum mag*cos, sum mag*sin, sum mag*r*cos, sum mag*r*sin) held as packed
//     fp32x2 pairs; nothing is reduced across lanes, so the inner loop has no shuffle, no
//     atomic and no shared-memory write;
//   * a warp is 32 consecutive observers x one wavenumber slice; the 4 warps of a CTA share
//     the observers and take 4 consecutive slices, so one staged source tile feeds 4*KS
//     wavenumbers of 32 observers;
//   * sources stream through shared memory in tiles of TJ: the x/y/z planes arrive by 1-D
//     bulk copies (TMA) into a double-buffered staging area, are repacked once per tile into
//     float4 {x,y,z,valid} so the inner loop reads one broadcast LDS.128 per pair, and tiles
//     without a single valid source are skipped;
//   * per pair the distance is evaluated once (rsqrt + one Newton step, so r is within an ulp
//     of sqrt) and reused by all KS wavenumbers; per (pair, wavenumber) the work is one phase
//     multiply, one sin and one cos on the SFU, and four fused multiply-adds, issued as
//     packed fp32x2 instructions.  The kernel is SFU-bound by construction.
#pragma once
#include "common.cuh"

namespace pai {

constexpr int WE_TJ = 512;        // sources per staged tile
constexpr int WE_WARPS = 4;       // warps (wavenumber slices) per CTA
constexpr int WE_THREADS = WE_WARPS * 32;

struct WeFwdParams {
    const float *coords;   // [Z,3,N]
    const uint8_t *valid;  // [Z,N] or nullptr
    const float *wn;       // [K]
    float *out;            // [Z,N,2K]
    float *cos_sums;       // [Z,N,K]
    float *sin_sums;       // [Z,N,K]
    int N, K, row_begin, row_end, mag_type, use_tma;
};

struct __align__(16) WeSmem {
    float stage[2][3][WE_TJ];  // x/y/z planes, two stages
    float4 tile[WE_TJ];        // repacked {x,y,z,valid}
    uint64_t bar[2];
    int any_valid;
};

// KS: wavenumbers per lane (even).  MAG1: compile-time fast path for magnitude_type == 1.
// RR: reduce the phase to [-pi, pi] explicitly (phase in revolutions, subtract the nearest
//     integer exactly) before the SFU sin/cos, instead of leaving the reduction to the
//     fp32 multiply inside sin.approx/cos.approx.
template <int KS, bool MAG1, bool RR>
__global__ void __launch_bounds__(WE_THREADS, 4) we_fwd_kernel(const WeFwdParams p) {
    __shared__ WeSmem sm;
    constexpr int KP = KS / 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int z = blockIdx.z;
    const int N = p.N, K = p.K;
    const int row = p.row_begin + blockIdx.x * 32 + lane;
    const int k0 = (blockIdx.y * WE_WARPS + warp) * KS;
    const float *cz = p.coords + (size_t)z * 3 * N;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

    // observer of this lane
    const bool row_in = row < p.row_end;
    float ox = 0.f, oy = 0.f, oz = 0.f;
    bool ov = false;
    if (row_in) {
        ox = cz[row];
        oy = cz[N + row];
        oz = cz[2 * N + row];
        ov = vz ? (vz[row] != 0) : true;
        if (!ov) ox = oy = oz = 0.f;
    }
    const bool cta_has_work = __syncthreads_or(ov ? 1 : 0) != 0;  // same 32 observers in every warp

    // wavenumber slice of this warp (zeros beyond K: harmless, never stored)
    f2_t kk[KP];
#pragma unroll
    for (int q = 0; q < KP; ++q) {
        float a = (k0 + 2 * q < K) ? p.wn[k0 + 2 * q] : 0.f;
        float b = (k0 + 2 * q + 1 < K) ? p.wn[k0 + 2 * q + 1] : 0.f;
        if (RR) {  // wavenumber in revolutions per unit length
            a = (float)((double)a * 0.15915494309189535);
            b = (float)((double)b * 0.15915494309189535);
        }
        kk[q] = f2_pack(a, b);
    }

    f2_t acc_re[KP], acc_im[KP], acc_c[KP], acc_s[KP];
#pragma unroll
    for (int q = 0; q < KP; ++q) acc_re[q] = acc_im[q] = acc_c[q] = acc_s[q] = 0ull;

    bool timed_out = false;
    if (cta_has_work && k0 - warp * KS < K) {
        const int ntiles = (N + WE_TJ - 1) / WE_TJ;
        const bool tma = p.use_tma != 0;
        if (tma) {
            if (tid == 0) {
                mbar_init(&sm.bar[0], 1);
                mbar_init(&sm.bar[1], 1);
                mbar_fence_init();
                fence_proxy_async();
            }
            __syncthreads();
            if (tid == 0) {  // prefetch tile 0
                const uint32_t bytes = (uint32_t)min(WE_TJ, N) * 4u;
                mbar_expect_tx(&sm.bar[0], 3 * bytes);
#pragma unroll
                for (int c = 0; c < 3; ++c) bulk_g2s(&sm.stage[0][c][0], cz + (size_t)c * N, bytes, &sm.bar[0]);
            }
        }
        for (int t = 0; t < ntiles; ++t) {
            const int j0 = t * WE_TJ;
            const int cnt = min(WE_TJ, N - j0);
            const int st = t & 1;
            if (tma) {
                if (tid == 0 && t + 1 < ntiles) {  // stage (t+1)&1 was drained by the repack of tile t-1
                    const int jn = j0 + WE_TJ;
                    const uint32_t bytes = (uint32_t)min(WE_TJ, N - jn) * 4u;
                    mbar_expect_tx(&sm.bar[st ^ 1], 3 * bytes);
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                        bulk_g2s(&sm.stage[st ^ 1][c][0], cz + (size_t)c * N + jn, bytes, &sm.bar[st ^ 1]);
                }
                const bool ok = mbar_wait_bounded(&sm.bar[st], (uint32_t)((t >> 1) & 1));
                if (__syncthreads_or(ok ? 0 : 1)) {  // also: everyone is done reading sm.tile
                    timed_out = true;
                    break;
                }
            } else {
                __syncthreads();  // everyone is done reading sm.tile
            }
            // repack to {x,y,z,valid}; count valid sources of this tile
            int mine = 0;
            for (int j = tid; j < cnt; j += WE_THREADS) {
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
                mine |= v ? 1 : 0;
                sm.tile[j] = s;
            }
            const bool any = __syncthreads_or(mine) != 0;  // also publishes sm.tile
            if (!any) continue;

            if (k0 >= K) continue;  // a slice past the last wavenumber only keeps the barriers company
#pragma unroll 2
            for (int j = 0; j < cnt; ++j) {
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
#pragma unroll
                for (int q = 0; q < KP; ++q) {
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
                    const f2_t c2 = f2_pack(ca, cb), s2 = f2_pack(sa, sb);
                    acc_re[q] = f2_fma(c2, mag2, acc_re[q]);
                    acc_im[q] = f2_fma(s2, mag2, acc_im[q]);
                    acc_c[q] = f2_fma(c2, magr2, acc_c[q]);
                    acc_s[q] = f2_fma(s2, magr2, acc_s[q]);
                }
            }
        }
    }
    if (timed_out) {
        if (tid == 0) atomicExch(&g_device_status, (int)PAI_ERR_DEVICE_WAIT_TIMEOUT);
        return;  // the one copy that may still be in flight targets this CTA's own shared memory
    }

    // epilogue: every row of the shard is written; padded observers get zeros
    if (!row_in) return;
    float *orow = p.out + ((size_t)z * N + row) * 2 * K;
    float *crow = p.cos_sums + ((size_t)z * N + row) * K;
    float *srow = p.sin_sums + ((size_t)z * N + row) * K;
    const bool vec = (K & 1) == 0;
#pragma unroll
    for (int q = 0; q < KP; ++q) {
        const int k = k0 + 2 * q;
        if (k >= K) break;
        float re0, re1, im0, im1, c0, c1, s0, s1;
        f2_unpack(acc_re[q], re0, re1);
        f2_unpack(acc_im[q], im0, im1);
        f2_unpack(acc_c[q], c0, c1);
        f2_unpack(acc_s[q], s0, s1);
        if (!ov) re0 = re1 = im0 = im1 = c0 = c1 = s0 = s1 = 0.f;
        if (vec) {  // K even: k + 1 < K and the addresses are 16- / 8-byte aligned
            *reinterpret_cast<float4 *>(orow + 2 * k) = make_float4(re0, im0, re1, im1);
            *reinterpret_cast<float2 *>(crow + k) = make_float2(c0, c1);
            *reinterpret_cast<float2 *>(srow + k) = make_float2(s0, s1);
        } else {
            orow[2 * k] = re0;
            orow[2 * k + 1] = im0;
            crow[k] = c0;
            srow[k] = s0;
            if (k + 1 < K) {
                orow[2 * k + 2] = re1;
                orow[2 * k + 3] = im1;
                crow[k + 1] = c1;
                srow[k + 1] = s1;
            }
        }
    }
}

template <int KS>
static int we_fwd_launch_ks(const WeFwdParams &p, int Z, bool rr, cudaStream_t stream) {
    const int rows = p.row_end - p.row_begin;
    dim3 grid((rows + 31) / 32, (p.K + WE_WARPS * KS - 1) / (WE_WARPS * KS), Z);
    dim3 block(WE_THREADS);
    if (p.mag_type == 1) {
        if (rr) we_fwd_kernel<KS, true, true><<<grid, block, 0, stream>>>(p);
        else we_fwd_kernel<KS, true, false><<<grid, block, 0, stream>>>(p);
    } else {
        if (rr) we_fwd_kernel<KS, false, true><<<grid, block, 0, stream>>>(p);
        else we_fwd_kernel<KS, false, false><<<grid, block, 0, stream>>>(p);
    }
    return (int)cudaPeekAtLastError();
}

// ks_hint: 0 = choose; otherwise 2, 8 or 16.  rr: explicit range reduction.
static int we_fwd_launch(const WeFwdParams &p, int Z, int ks_hint, bool rr, cudaStream_t stream) {
    int ks = ks_hint;
    if (ks == 0) {
        ks = p.K >= 64 ? 16 : (p.K >= 32 ? 8 : 2);
        // small problems: prefer more, thinner CTAs so that all SMs get work
        const long rows_blocks = (long)((p.row_end - p.row_begin + 31) / 32) * Z;
        if (ks == 16 && rows_blocks * ((p.K + 63) / 64) < 148 * 4) ks = 8;
    }
    switch (ks) {
        case 16: return we_fwd_launch_ks<16>(p, Z, rr, stream);
        case 8: return we_fwd_launch_ks<8>(p, Z, rr, stream);
        case 2: return we_fwd_launch_ks<2>(p, Z, rr, stream);
        default: return (int)PAI_ERR_UNSUPPORTED;
    }
}

}  // namespace pai
