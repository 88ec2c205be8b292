// Geometric attention forward for sm_100a: flash attention on tcgen05 tensor cores with the
// per-head radial-basis scale applied in the softmax stage,
//     SR_ij = (q_i . k_j / sqrt(d)) * (1 + exp(-|r_i - r_j|^2 / (2 sigma_h^2))),
// a pair being valid iff query i and key j are both unpadded.  Replaces the Triton kernel
// `_attn_fwd` (old/old_scripts/attn/geometric_attn.py:57-260) with the logit form the reference's
// README states (README.md:40).
//
// One CTA = 128 query rows of one (batch, head): 8 math warps and one producer warp.
// Query row r = TMEM lane r is shared by two math threads: warp w (0..3) takes key columns 0..63 of a
// tile and output columns 0..31, warp w + 4 takes key columns 64..127 and output columns 32..63 (both
// may touch TMEM lanes 32 (w % 4) ..).  Lane 0 of the producer warp issues every TMA load and MMA.
//   S  = Q K^T : tcgen05.mma, A = Q tile, B = K tile (both K-major, 128-byte swizzle, via TMA),
//                accumulator [128 lanes x 128 columns] fp32 in TMEM;
//   softmax    : each math thread reads its half row with tcgen05.ld and applies scale * (1 + R) in
//                packed fp32x2 arithmetic.  |r_i - r_j|^2 comes from three FMAs on coordinates centred
//                on the tile's first valid query (|q|^2 + |k|^2 - 2 q.k; the centring keeps the
//                cancellation error negligible wherever R is not already ~0).  The two halves of a row
//                exchange their maxima through shared memory; P is written as bf16 into shared memory
//                in the swizzled K-major layout TMA would have produced;
//   O += P V   : tcgen05.mma, A = P tile (K-major), B = V tile (MN-major: keys are the K dimension),
//                accumulated in TMEM [128 x 64] across the key tiles.  The running maximum is only
//                raised when a tile exceeds it by more than 2^8 (then the TMEM accumulator and the row
//                sum are rescaled); otherwise P is computed against the slightly stale maximum, which
//                is exact after the final normalisation.
// K and V are single-buffered: K(t+1) is fetched as soon as S(t) has completed and V(t+1) as soon as
// PV(t) has; S(t+1) is issued ahead of PV(t) so the next softmax can start while PV(t) runs.  Two CTAs
// fit one SM (about 88 kB shared memory, 256 TMEM columns each).  Key tiles without any valid key are
// skipped; tiles without any padded key take a path without the mask; CTAs without any valid query only
// write zeros.
#pragma once
#include "tc.cuh"

namespace pai {

constexpr int GA_BM = 128;  // query rows per CTA
constexpr int GA_BN = 128;  // keys per tile
constexpr int GA_D = 64;    // head dimension
constexpr int GA_MAX_TILES = 1024;
constexpr int GA_FWD_MATH_THREADS = 256;
constexpr int GA_FWD_THREADS = GA_FWD_MATH_THREADS + 32;  // + the producer warp
constexpr float GA_RESCALE_THRESHOLD = 8.f;                 // log2 units
constexpr uint32_t GA_TMEM_COLS = 256;
constexpr uint32_t GA_TILE_BYTES = GA_BN * GA_D * 2;  // 16 KiB

struct GaFwdSmem {
    alignas(1024) uint8_t q[GA_TILE_BYTES];
    alignas(1024) uint8_t k[GA_TILE_BYTES];
    alignas(1024) uint8_t v[GA_TILE_BYTES];
    alignas(1024) uint8_t p[2 * GA_TILE_BYTES];  // [128 x 128] bf16 as two [128 x 64] swizzled sub-tiles
    // centred key coordinates of the current / next tile, two keys per entry:
    float4 ka[2][GA_BN / 2];                      // {x_j, x_j+1, y_j, y_j+1}
    float4 kc[2][GA_BN / 2];                      // {z_j, z_j+1, |k_j|^2, |k_j+1|^2}
    alignas(16) float kb[2][GA_BN];               // additive mask: 0 for a valid key, -inf for a padded one
    float xch[2][GA_BM];                          // row maxima (then row sums) exchanged between the two halves
    uint16_t tiles[GA_MAX_TILES];                 // key tiles with a valid key; bit 15: the tile also has a padded key
    uint64_t bar_q, bar_k, bar_v, bar_s, bar_o, bar_p;
    uint32_t tmem_base;
    int ntiles;
    int first_q;                                  // first valid query row of the tile (origin of the centring)
};

struct GaFwdParams {
    const float *coords;   // [Z,N,3]
    const uint8_t *valid;  // [Z,N] or nullptr
    const float *sigma;    // [H]
    __nv_bfloat16 *out;    // element (z,h,n,:) at out + z*so_z + h*so_h + n*so_n, 64 contiguous values
    long long so_z, so_h, so_n;
    float *lse;            // [Z,H,N]  log-sum-exp of SR (natural log), -inf for padded queries
    int Z, H, N, zh_begin;
    float scale;
    // logit form: 0 = S (1 + R);  1 = S + beta Rn |S| with Rn = 2 (R - min_rbf) / (max_rbf - min_rbf) - 1 and pairs
    // with R outside [min_rbf, max_rbf] masked out (the form of old/old_scripts/attn/geometric_attn.py:193-201)
    int form;
    const float *beta;     // [H], form 1 only
    float min_rbf, max_rbf;
    const int *order;      // [Z] permutation of the samples or nullptr (only with the full (batch, head) range)
};

struct GaForm {  // per-head constants of logit form 1
    float beta, rn_a, rn_b, rmin, rmax;  // Rn = R * rn_a + rn_b
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// Barrier among a subset of the CTA's warps.  The id is an immediate so that the compiler counts the
// barriers the kernel really uses: an SM has 16, and a kernel that indexes them with a register is
// charged all 16, which limits it to one CTA per SM.
template <int ID>
__device__ __forceinline__ void named_bar_sync(int count) {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "r"(count) : "memory");
}
// the two warps w and w + 4 that share 32 query rows
__device__ __forceinline__ void pair_bar_sync(int quarter) {
    switch (quarter) {
        case 0: named_bar_sync<1>(64); break;
        case 1: named_bar_sync<2>(64); break;
        case 2: named_bar_sync<3>(64); break;
        default: named_bar_sync<4>(64); break;
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// One chunk of the first softmax pass: 16 logits (8 key pairs) of one row.  Reads S from TMEM, forms
// SR = (S * c_s) * (1 + R) with R = 2^(c_rbf * d^2), d^2 = |q|^2 + |k|^2 - 2 q.k from the centred
// coordinates, optionally adds the key mask, writes SR back in place and returns the running maximum.
// Written as three stages over the 8 pairs so that the independent chains overlap.
template <bool MASKED, int FORM>
__device__ __forceinline__ float ga_scale_chunk(uint32_t taddr, const float4 *ka, const float4 *kc, const float *kb, f2_t qx2,
                                                f2_t qy2, f2_t qz2, f2_t crbf2, f2_t cqn2, f2_t cs2, const GaForm &fm, float m_loc) {
    uint32_t v[16];
    tmem_ld16(taddr, v);
    f2_t arg[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {  // exponent arguments, independent of S
        const float4 a = ka[e], k4 = kc[e];
        f2_t d2 = f2_fma(qz2, f2_pack(k4.x, k4.y), f2_pack(k4.z, k4.w));
        d2 = f2_fma(qy2, f2_pack(a.z, a.w), d2);
        d2 = f2_fma(qx2, f2_pack(a.x, a.y), d2);
        arg[e] = f2_fma(d2, crbf2, cqn2);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float a0, a1;
        f2_unpack(arg[e], a0, a1);
        if (FORM == 1) {  // keep R <= 1 exactly (the centred d^2 of a coincident pair can round below zero)
            a0 = fminf(a0, 0.f);
            a1 = fminf(a1, 0.f);
        }
        arg[e] = f2_pack(ex2_approx(a0), ex2_approx(a1));  // R
    }
    tmem_wait_ld();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const f2_t t2 = f2_mul(f2_pack(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1])), cs2);
        f2_t sr;
        if (FORM == 0) {
            sr = f2_fma(t2, arg[e], t2);
        } else {
            float t0, t1, r0, r1;
            f2_unpack(t2, t0, t1);
            f2_unpack(arg[e], r0, r1);
            const float s0 = fmaf(fm.beta * fmaf(r0, fm.rn_a, fm.rn_b), fabsf(t0), t0);
            const float s1 = fmaf(fm.beta * fmaf(r1, fm.rn_a, fm.rn_b), fabsf(t1), t1);
            sr = f2_pack((r0 >= fm.rmin && r0 <= fm.rmax) ? s0 : -INFINITY, (r1 >= fm.rmin && r1 <= fm.rmax) ? s1 : -INFINITY);
        }
        if (MASKED) sr = f2_add(sr, *reinterpret_cast<const f2_t *>(kb + 2 * e));
        float v0, v1;
        f2_unpack(sr, v0, v1);
        v[2 * e] = __float_as_uint(v0);
        v[2 * e + 1] = __float_as_uint(v1);
        m_loc = max3(m_loc, v0, v1);
    }
    tmem_st16(taddr, v);
    return m_loc;
}

__global__ void __maxnreg__(80)
geoattn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const GaFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaFwdSmem &sm = *reinterpret_cast<GaFwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_math = warp < GA_FWD_MATH_THREADS / 32;
    const int half = (warp >> 2) & 1;             // 0: key columns 0..63, 1: 64..127
    const int r = (warp & 3) * 32 + lane;         // query row inside the tile = TMEM lane
    int zh_local = blockIdx.y;                    // index into the shard of (batch, head) pairs
    if (p.order) {  // samples in the given order (longest first): neighbouring CTAs get similar amounts of work
        const int zp = zh_local / p.H;
        zh_local = p.order[zp] * p.H + (zh_local - zp * p.H);
    }
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int i0 = blockIdx.x * GA_BM;
    const int N = p.N;
    const int row = i0 + r;
    const float *cz = p.coords + (size_t)z * N * 3;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

    const bool q_ok = is_math && row < N && (vz ? vz[row] != 0 : true);
    if (tid == 0) sm.first_q = 0x7fffffff;
    // ---- key tiles with at least one valid key (bit 15: also a padded or out-of-range key) -----------
    const int all_tiles = (N + GA_BN - 1) / GA_BN;
    for (int t = warp; t < all_tiles; t += GA_FWD_THREADS / 32) {
        bool any = false, hole = false;
        for (int j = t * GA_BN + lane; j < (t + 1) * GA_BN; j += 32) {
            const bool ok = j < N && (vz ? vz[j] != 0 : true);
            any |= ok;
            hole |= !ok;
        }
        any = __any_sync(0xffffffffu, any);
        hole = __any_sync(0xffffffffu, hole);
        if (lane == 0) sm.tiles[t] = any ? (uint16_t)(1 | (hole ? 0x8000 : 0)) : (uint16_t)0;
    }
    __syncthreads();
    if (q_ok && half == 0) atomicMin(&sm.first_q, r);
    const bool cta_has_query = __syncthreads_or(q_ok ? 1 : 0) != 0;
    if (tid == 0) {
        int n = 0;
        for (int t = 0; t < all_tiles; ++t)
            if (sm.tiles[t]) sm.tiles[n++] = (uint16_t)(t | (sm.tiles[t] & 0x8000));  // in place: n <= t
        sm.ntiles = n;
    }
    __syncthreads();
    const int nt = sm.ntiles;

    __nv_bfloat16 *orow = p.out + (long long)z * p.so_z + (long long)h * p.so_h + (long long)row * p.so_n + half * 32;
    if (!cta_has_query || nt == 0) {  // nothing to attend from / to: zeros and -inf
        if (is_math && row < N) {
#pragma unroll
            for (int c = 0; c < 4; ++c) reinterpret_cast<uint4 *>(orow)[c] = make_uint4(0, 0, 0, 0);
            if (half == 0) p.lse[(size_t)zh * N + row] = -INFINITY;
        }
        return;
    }
    // origin of the centred coordinates: the first valid query of this tile
    const int oq = i0 + sm.first_q;
    const float orx = cz[oq * 3], ory = cz[oq * 3 + 1], orz = cz[oq * 3 + 2];

    // ---- set-up: TMEM, barriers, first key coordinates ---------------------------------------------
    if (warp == 8) {
        tmem_alloc(&sm.tmem_base, GA_TMEM_COLS);
        tmem_relinquish();
        if (lane == 0) {
            mbar_init(&sm.bar_q, 1);
            mbar_init(&sm.bar_k, 1);
            mbar_init(&sm.bar_v, 1);
            mbar_init(&sm.bar_s, 1);
            mbar_init(&sm.bar_o, 1);
            mbar_init(&sm.bar_p, GA_FWD_MATH_THREADS);
            mbar_fence_init();
            fence_proxy_async();
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
        }
    }
    auto load_kc = [&](int buf, int tile) {  // threads 0..127 stage key tile*128 + tid, centred
        if (tid < GA_BN) {
            const int j = tile * GA_BN + tid;
            const bool ok = j < N && (vz ? vz[j] != 0 : true);
            const float x = ok ? cz[j * 3] - orx : 0.f, y = ok ? cz[j * 3 + 1] - ory : 0.f, zc = ok ? cz[j * 3 + 2] - orz : 0.f;
            float *a = reinterpret_cast<float *>(&sm.ka[buf][tid >> 1]);
            float *c = reinterpret_cast<float *>(&sm.kc[buf][tid >> 1]);
            a[tid & 1] = x;
            a[2 + (tid & 1)] = y;
            c[tid & 1] = zc;
            c[2 + (tid & 1)] = x * x + y * y + zc * zc;
            sm.kb[buf][tid] = ok ? 0.f : -INFINITY;
        }
    };
    load_kc(0, sm.tiles[0] & 0x7fff);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_s = tmem;          // columns [0,128): S
    const uint32_t tmem_o = tmem + 128;    // columns [128,192): O accumulator
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    if (!is_math) {
        // ================================ producer warp ==============================================
        if (lane == 0) {
            const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);
            constexpr uint32_t IDESC_S = umma_idesc_bf16(GA_BM, GA_BN, false, false);  // Q K^T: both K-major
            constexpr uint32_t IDESC_O = umma_idesc_bf16(GA_BM, GA_D, false, true);    // P V: V is MN-major
            auto issue_s = [&]() {  // 4 MMAs of K = 16 over d = 64: advance 32 B inside the swizzled row
#pragma unroll
                for (int kk = 0; kk < GA_D / 16; ++kk)
                    umma_ss(tmem_s, umma_desc_sw128(q_addr + kk * 32, 16, 1024), umma_desc_sw128(k_addr + kk * 32, 16, 1024),
                            IDESC_S, kk > 0 ? 1u : 0u);
                umma_commit(&sm.bar_s);
            };
            auto issue_pv = [&](bool first) {  // 8 MMAs of K = 16 keys: P advances 32 B (second sub-tile after 64 keys), V 2 KiB
#pragma unroll
                for (int kk = 0; kk < GA_BN / 16; ++kk)
                    umma_ss(tmem_o, umma_desc_sw128(p_addr + (kk >> 2) * GA_TILE_BYTES + (kk & 3) * 32, 16, 1024),
                            umma_desc_sw128(v_addr + kk * 2048, 0, 1024), IDESC_O, (first && kk == 0) ? 0u : 1u);
                umma_commit(&sm.bar_o);
            };
            auto tile_row = [&](int t) { return (int)(sm.tiles[t] & 0x7fff) * GA_BN; };
            mbar_expect_tx(&sm.bar_q, GA_TILE_BYTES);
            tma_load_4d(sm.q, &map_q, 0, i0, h, z, &sm.bar_q);
            mbar_expect_tx(&sm.bar_k, GA_TILE_BYTES);
            tma_load_4d(sm.k, &map_k, 0, tile_row(0), h, z, &sm.bar_k);
            mbar_expect_tx(&sm.bar_v, GA_TILE_BYTES);
            tma_load_4d(sm.v, &map_v, 0, tile_row(0), h, z, &sm.bar_v);
            mbar_wait_timed(&sm.bar_q, 0);
            mbar_wait_timed(&sm.bar_k, 0);
            tc_fence_after();
            issue_s();
            if (nt > 1) {  // the K buffer is free once S(0) has completed
                mbar_wait_timed(&sm.bar_s, 0);
                mbar_expect_tx(&sm.bar_k, GA_TILE_BYTES);
                tma_load_4d(sm.k, &map_k, 0, tile_row(1), h, z, &sm.bar_k);
            }
            for (int t = 0; t < nt; ++t) {
                const uint32_t par = (uint32_t)(t & 1);
                mbar_wait_timed(&sm.bar_p, par);  // P(t) written, S(t) consumed, O rescaled if it had to be
                tc_fence_after();
                if (t + 1 < nt) {
                    mbar_wait_timed(&sm.bar_k, par ^ 1);
                    issue_s();  // S(t+1) first: the next softmax starts while P V(t) runs
                }
                mbar_wait_timed(&sm.bar_v, par);
                issue_pv(t == 0);
                if (t + 2 < nt) {  // K buffer free once S(t+1) has completed
                    mbar_wait_timed(&sm.bar_s, par ^ 1);
                    mbar_expect_tx(&sm.bar_k, GA_TILE_BYTES);
                    tma_load_4d(sm.k, &map_k, 0, tile_row(t + 2), h, z, &sm.bar_k);
                }
                if (t + 1 < nt) {  // V buffer free once P V(t) has completed
                    mbar_wait_timed(&sm.bar_o, par);
                    mbar_expect_tx(&sm.bar_v, GA_TILE_BYTES);
                    tma_load_4d(sm.v, &map_v, 0, tile_row(t + 1), h, z, &sm.bar_v);
                }
            }
        }
        __syncwarp();
    } else {
        // ================================ math warps ==================================================
        const float sig = p.sigma[h];
        const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);  // R = 2^(c_rbf * d^2)
        const float c_s = p.scale * 1.4426950408889634f;               // logits in base-2 units
        float qcx = 0.f, qcy = 0.f, qcz = 0.f;
        if (q_ok) {
            qcx = cz[row * 3] - orx;
            qcy = cz[row * 3 + 1] - ory;
            qcz = cz[row * 3 + 2] - orz;
        }
        // d^2 = |q|^2 + |k|^2 - 2 q.k  ->  c_rbf * d^2 = fma(|k|^2 + (-2q).k, c_rbf, c_rbf |q|^2)
        const f2_t qx2 = f2_pack(-2.f * qcx, -2.f * qcx), qy2 = f2_pack(-2.f * qcy, -2.f * qcy), qz2 = f2_pack(-2.f * qcz, -2.f * qcz);
        const float cqn = c_rbf * (qcx * qcx + qcy * qcy + qcz * qcz);
        const f2_t crbf2 = f2_pack(c_rbf, c_rbf), cqn2 = f2_pack(cqn, cqn), cs2 = f2_pack(c_s, c_s);
        GaForm fm = {0.f, 0.f, 0.f, 0.f, 1.f};
        if (p.form == 1) {
            fm.beta = p.beta[h];
            fm.rn_a = 2.f / (p.max_rbf - p.min_rbf);
            fm.rn_b = -2.f * p.min_rbf / (p.max_rbf - p.min_rbf) - 1.f;
            fm.rmin = p.min_rbf;
            fm.rmax = p.max_rbf;
        }
        float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's half of the row sum

        for (int t = 0; t < nt; ++t) {
            const uint32_t par = (uint32_t)(t & 1);
            const int cb = t & 1;
            const bool has_hole = (sm.tiles[t] & 0x8000) != 0;
            mbar_wait_timed(&sm.bar_s, par);  // S(t) has landed in TMEM
            tc_fence_after();
            // key coordinates of the next tile: issue the global loads now, store after the first pass
            float nx = 0.f, ny = 0.f, nz = 0.f;
            bool nok = false;
            const bool stage_next = t + 1 < nt && tid < GA_BN;
            if (stage_next) {
                const int j = (int)(sm.tiles[t + 1] & 0x7fff) * GA_BN + tid;
                nok = j < N && (vz ? vz[j] != 0 : true);
                if (nok) {
                    nx = cz[j * 3] - orx;
                    ny = cz[j * 3 + 1] - ory;
                    nz = cz[j * 3 + 2] - orz;
                }
            }
            // first pass, 32 logits at a time: scale by (1 + R), mask, write SR back to TMEM, track the maximum
            // (two copies of the loop so that the mask test is not a branch inside the unrolled body)
            float m_loc = -INFINITY;
#define PAI_GA_PASS1(MASKED, FORM)                                                                                          \
    _Pragma("unroll") for (int c = 0; c < 4; ++c) m_loc = ga_scale_chunk<MASKED, FORM>(                                      \
        tmem_s + lane_base + half * 64 + c * 16, &sm.ka[cb][half * 32 + c * 8], &sm.kc[cb][half * 32 + c * 8],               \
        &sm.kb[cb][half * 64 + c * 16], qx2, qy2, qz2, crbf2, cqn2, cs2, fm, m_loc)
            if (p.form == 0) {
                if (has_hole) { PAI_GA_PASS1(true, 0); } else { PAI_GA_PASS1(false, 0); }
            } else {
                if (has_hole) { PAI_GA_PASS1(true, 1); } else { PAI_GA_PASS1(false, 1); }
            }
#undef PAI_GA_PASS1
            tmem_wait_st();
            if (stage_next) {  // the other buffer was last read during tile t-1
                float *a = reinterpret_cast<float *>(&sm.ka[cb ^ 1][tid >> 1]);
                float *k4 = reinterpret_cast<float *>(&sm.kc[cb ^ 1][tid >> 1]);
                a[tid & 1] = nx;
                a[2 + (tid & 1)] = ny;
                k4[tid & 1] = nz;
                k4[2 + (tid & 1)] = nx * nx + ny * ny + nz * nz;
                sm.kb[cb ^ 1][tid] = nok ? 0.f : -INFINITY;
            }
            sm.xch[half][r] = m_loc;
            pair_bar_sync(warp & 3);  // the two warps that share these 32 rows
            // the tile maximum is finite for form 0 (every listed tile holds a valid key); form 1 can mask a whole row of a tile
            const float m_tile = fmaxf(m_loc, sm.xch[half ^ 1][r]);
            float alpha = 1.f;
            bool raise = false;
            if (t == 0) {
                m_run = m_tile;
            } else if (m_tile > m_run + GA_RESCALE_THRESHOLD) {
                raise = true;
                alpha = ex2_approx(m_run - m_tile);
                m_run = m_tile;
            }
            if (t > 0) {  // P V(t-1) has completed: the P buffer is free and the O accumulator is at rest
                mbar_wait_timed(&sm.bar_o, par ^ 1);
                tc_fence_after();
                if (__any_sync(0xffffffffu, raise)) {  // same rows, hence the same decision, in the partner warp
                    uint32_t v[32];
                    tmem_ld32(tmem_o + lane_base + half * 32, v);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                    tmem_st32(tmem_o + lane_base + half * 32, v);
                    tmem_wait_st();
                }
            }
            // second pass: P = 2^(SR - m), row sum, bf16 P into the swizzled tile
            const float m_safe = m_run == -INFINITY ? 0.f : m_run;  // a row without any valid pair so far: P = 2^(-inf) = 0
            const f2_t mn2 = f2_pack(m_safe, m_safe);
            f2_t l2 = 0ull;
            uint32_t va[16], vb[16];  // two chunks in flight: the TMEM load of the next overlaps the exponentials of this one
            tmem_ld16(tmem_s + lane_base + half * 64, va);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t(&v)[16] = (c & 1) ? vb : va;
                uint32_t(&vn)[16] = (c & 1) ? va : vb;
                if (c + 1 < 4) tmem_ld16(tmem_s + lane_base + half * 64 + (c + 1) * 16, vn);
                float ex[16];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float a0, a1;
                    f2_unpack(f2_sub(f2_pack(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1])), mn2), a0, a1);
                    ex[2 * q] = ex2_approx(a0);
                    ex[2 * q + 1] = ex2_approx(a1);
                }
#pragma unroll
                for (int g = 0; g < 2; ++g) {  // 8 keys = one 16-byte chunk of the swizzled row
                    uint32_t w[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        l2 = f2_add(l2, f2_pack(ex[g * 8 + 2 * q], ex[g * 8 + 2 * q + 1]));
                        w[q] = pack_bf16x2(ex[g * 8 + 2 * q], ex[g * 8 + 2 * q + 1]);
                    }
                    *reinterpret_cast<uint4 *>(sm.p + half * GA_TILE_BYTES + sw128_offset(r, c * 2 + g)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                if (c + 1 < 4) tmem_wait_ld();
            }
            float l0, l1;
            f2_unpack(l2, l0, l1);
            l_run = l_run * alpha + (l0 + l1);
            fence_proxy_async();  // P (generic-proxy stores) must be visible to the tensor core
            tc_fence_before();
            mbar_arrive(&sm.bar_p);
            named_bar_sync<5>(GA_FWD_MATH_THREADS);  // key coordinates of the next tile are staged
        }

        // ---- epilogue ----------------------------------------------------------------------------------
        mbar_wait_timed(&sm.bar_o, (uint32_t)((nt - 1) & 1));
        tc_fence_after();
        uint32_t ov[32];
        tmem_ld32(tmem_o + lane_base + half * 32, ov);
        tmem_wait_ld();
        sm.xch[half][r] = l_run;
        pair_bar_sync(warp & 3);
        const float l_tot = l_run + sm.xch[half ^ 1][r];
        if (row < N) {
            const bool live = q_ok && l_tot > 0.f;
            const float inv = live ? 1.f / l_tot : 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint4 pk;
                pk.x = pack_bf16x2(__uint_as_float(ov[c * 8 + 0]) * inv, __uint_as_float(ov[c * 8 + 1]) * inv);
                pk.y = pack_bf16x2(__uint_as_float(ov[c * 8 + 2]) * inv, __uint_as_float(ov[c * 8 + 3]) * inv);
                pk.z = pack_bf16x2(__uint_as_float(ov[c * 8 + 4]) * inv, __uint_as_float(ov[c * 8 + 5]) * inv);
                pk.w = pack_bf16x2(__uint_as_float(ov[c * 8 + 6]) * inv, __uint_as_float(ov[c * 8 + 7]) * inv);
                reinterpret_cast<uint4 *>(orow)[c] = pk;
            }
            if (half == 0) p.lse[(size_t)zh * N + row] = live ? (m_run + lg2_approx(l_tot)) * 0.6931471805599453f : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem, GA_TMEM_COLS);
}

}  // namespace pai
