// Geometric attention backward for sm_100a (tcgen05 / TMEM / TMA).
//
// Replaces the Triton kernel `_attn_bwd` (old/old_scripts/attn/geometric_attn.py:265-543) and the
// PyTorch row-sum in front of it (:616), for the logit form SR = S (1 + R), S = scale q.k,
// R = exp(-d^2 / (2 sigma_h^2)):
//     D_i   = sum_d O_id dO_id                       (pre-kernel, fp32 scratch)
//     P_ij  = exp(SR_ij - L_i)                        (recomputed from the stored log-sum-exp)
//     dV_j  = sum_i P_ij dO_i
//     dP_ij = dO_i . V_j
//     dSR   = P (dP - D)
//     dS    = dSR (1 + R) scale        -> dQ_i = sum_j dS_ij K_j,   dK_j = sum_i dS_ij Q_i
//     dsigma_h = sum_{z,i,j} dSR S R d^2 / sigma_h^3
//
// One CTA = 128 keys of one (batch, head); it loops over the 128-row query tiles.  16 math warps and one
// producer warp: query row r = TMEM lane r of the current tile is shared by four math threads (warps
// w, w+4, w+8, w+12), each taking 32 of the 128 key columns; no row reduction is needed in the backward
// because the log-sum-exp L and D are known.  Lane 0 of the producer warp issues every TMA load and MMA.
// Five MMAs per query tile, all operands straight from the TMA-written swizzled tiles, transposes
// expressed through the operand major-ness:
//     S   = Q_i K_j^T     A K-major,  B K-major     -> TMEM [128 x 128]
//     dP  = dO_i V_j^T    A K-major,  B K-major     -> TMEM [128 x 128]
//     dV += P^T dO_i      A MN-major, B MN-major    -> TMEM [128 x 64], accumulated over i
//     dK += dS^T Q_i      A MN-major, B MN-major    -> TMEM [128 x 64], accumulated over i
//     dQ_i = dS K_j       A K-major,  B MN-major    -> TMEM [128 x 64], read back and added into the global
//                                                      fp32 dQ with 16-byte vector reductions
// P and dS are written by the math threads as bf16 into shared memory in the swizzled [i][j] layout,
// which serves both as K-major (dQ) and MN-major (dV, dK) operand.  The element-wise stage runs in
// packed fp32x2 arithmetic with |r_i - r_j|^2 from centred coordinates (three FMAs).  Query tiles
// without a valid query are skipped, a key tile without a valid key only writes zeros.
#pragma once
#include "geoattn_fwd.cuh"

namespace pai {

constexpr uint32_t GA_BWD_TMEM_COLS = 512;
constexpr int GA_BWD_MATH_THREADS = 512;
constexpr int GA_BWD_THREADS = GA_BWD_MATH_THREADS + 32;  // + the producer warp

struct GaBwdSmem {
    alignas(1024) uint8_t k[GA_TILE_BYTES];
    alignas(1024) uint8_t v[GA_TILE_BYTES];
    alignas(1024) uint8_t q[2][GA_TILE_BYTES];
    alignas(1024) uint8_t dout[2][GA_TILE_BYTES];
    alignas(1024) uint8_t p[2 * GA_TILE_BYTES];
    alignas(1024) uint8_t ds[2 * GA_TILE_BYTES];
    // centred key coordinates, two keys per entry:
    float4 ka[GA_BN / 2];                  // {x_j, x_j+1, y_j, y_j+1}
    float4 kc[GA_BN / 2];                  // {z_j, z_j+1, |k_j|^2, |k_j+1|^2}
    alignas(16) float kb[GA_BN];           // additive mask: 0 for a valid key, -inf for a padded one
    uint16_t tiles[GA_MAX_TILES];          // query tiles that hold at least one valid query
    uint64_t bar_kv, bar_qdo[2], bar_sp, bar_g, bar_vk, bar_pds, bar_dqr;
    uint32_t tmem_base;
    int ntiles;
    int first_k;                           // first valid key of the tile (origin of the centring)
    int has_hole;                          // the key tile holds a padded or out-of-range key
    float dsig[GA_BWD_MATH_THREADS / 32];
    float dbeta[GA_BWD_MATH_THREADS / 32];
};

struct GaBwdParams {
    const float *coords;   // [Z,N,3]
    const uint8_t *valid;  // [Z,N] or nullptr
    const float *sigma;    // [H]
    const float *lse;      // [Z,H,N]
    const float *dsum;     // [nzh,N]   D = rowsum(O * dO), indexed from zh_begin
    float *dq;             // [Z,H,N,64] fp32, zeroed before launch, accumulated here
    float *dk;             // [Z,H,N,64] fp32
    float *dv;             // [Z,H,N,64] fp32
    float *dsigma;         // [H] fp32, zeroed before launch
    float *dbeta;          // [H] fp32, zeroed before launch (form 1 only; may be nullptr for form 0)
    int Z, H, N, zh_begin;
    float scale;
    int form;              // logit form, as in the forward
    const float *beta;     // [H], form 1 only
    float min_rbf, max_rbf;
    const int *order;      // [Z] permutation of the samples or nullptr (only with the full (batch, head) range)
};

// D[zh_local, i] = sum_d O * dO; one warp per row, 2 elements per lane.
__global__ void __launch_bounds__(256) geoattn_bwd_dsum_kernel(const __nv_bfloat16 *o, const __nv_bfloat16 *d_out, float *dsum,
                                                               long long rows) {
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const __nv_bfloat162 a = reinterpret_cast<const __nv_bfloat162 *>(o + row * GA_D)[lane];
    const __nv_bfloat162 b = reinterpret_cast<const __nv_bfloat162 *>(d_out + row * GA_D)[lane];
    float s = __bfloat162float(a.x) * __bfloat162float(b.x) + __bfloat162float(a.y) * __bfloat162float(b.y);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) dsum[row] = s;
}

__device__ __forceinline__ void red_add_v4(float *dst, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

struct GaBwdRow {  // per-thread constants of the current query row, packed for fp32x2 arithmetic
    f2_t qx2, qy2, qz2, cqn2, l22, dsum2;
};

// 16 key columns (8 pairs) of one query row: recompute P, form dS and the spread-gradient term, write P and
// dS as bf16 into the swizzled [i][j] tiles.  `chunk0` is the index of the first 16-byte chunk (8 keys).
template <bool MASKED, int FORM>
__device__ __forceinline__ void ga_bwd_chunk(uint32_t t_s, uint32_t t_dp, const float4 *ka, const float4 *kc, const float *kb,
                                             const GaBwdRow &rw, f2_t crbf2, f2_t cs2, f2_t scale2, const GaForm &fm, f2_t &dsig2,
                                             f2_t &dbeta2, uint8_t *p_tile, uint8_t *ds_tile, int r, int chunk0, uint64_t *gate,
                                             uint32_t gate_parity) {
    uint32_t sv[16], dpv[16];
    tmem_ld16(t_s, sv);
    tmem_ld16(t_dp, dpv);
    const f2_t one2 = f2_pack(1.f, 1.f);
#pragma unroll
    for (int g = 0; g < 2; ++g) {  // 8 keys = one 16-byte chunk
        f2_t arg[4], rb[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float4 a = ka[g * 4 + e], k4 = kc[g * 4 + e];
            f2_t d2 = f2_fma(rw.qz2, f2_pack(k4.x, k4.y), f2_pack(k4.z, k4.w));
            d2 = f2_fma(rw.qy2, f2_pack(a.z, a.w), d2);
            d2 = f2_fma(rw.qx2, f2_pack(a.x, a.y), d2);
            arg[e] = f2_fma(d2, crbf2, rw.cqn2);  // c_rbf * d^2
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float a0, a1;
            f2_unpack(arg[e], a0, a1);
            if (FORM == 1) {
                a0 = fminf(a0, 0.f);
                a1 = fminf(a1, 0.f);
            }
            rb[e] = f2_pack(ex2_approx(a0), ex2_approx(a1));  // R
        }
        if (g == 0) tmem_wait_ld();
        uint32_t pw[4], dw[4];
        f2_t x[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const f2_t s_raw = f2_pack(__uint_as_float(sv[g * 8 + 2 * e]), __uint_as_float(sv[g * 8 + 2 * e + 1]));
            const f2_t t2 = f2_mul(s_raw, cs2);
            f2_t sr;
            if (FORM == 0) {
                sr = f2_fma(t2, rb[e], t2);
            } else {
                float t0, t1, r0, r1;
                f2_unpack(t2, t0, t1);
                f2_unpack(rb[e], r0, r1);
                const float s0 = fmaf(fm.beta * fmaf(r0, fm.rn_a, fm.rn_b), fabsf(t0), t0);
                const float s1 = fmaf(fm.beta * fmaf(r1, fm.rn_a, fm.rn_b), fabsf(t1), t1);
                sr = f2_pack((r0 >= fm.rmin && r0 <= fm.rmax) ? s0 : -INFINITY, (r1 >= fm.rmin && r1 <= fm.rmax) ? s1 : -INFINITY);
            }
            if (MASKED) sr = f2_add(sr, *reinterpret_cast<const f2_t *>(kb + g * 8 + 2 * e));
            x[e] = f2_sub(sr, rw.l22);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float a0, a1;
            f2_unpack(x[e], a0, a1);
            x[e] = f2_pack(ex2_approx(a0), ex2_approx(a1));  // P
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const f2_t s_raw = f2_pack(__uint_as_float(sv[g * 8 + 2 * e]), __uint_as_float(sv[g * 8 + 2 * e + 1]));
            const f2_t dp = f2_pack(__uint_as_float(dpv[g * 8 + 2 * e]), __uint_as_float(dpv[g * 8 + 2 * e + 1]));
            const f2_t dsr = f2_mul(x[e], f2_sub(dp, rw.dsum2));
            f2_t ds;
            if (FORM == 0) {
                ds = f2_mul(f2_mul(dsr, scale2), f2_add(rb[e], one2));
                dsig2 = f2_fma(f2_mul(f2_mul(dsr, s_raw), rb[e]), arg[e], dsig2);
            } else {  // dS = dSR (1 + beta Rn sign(S)),  dR = dSR |S| 2 beta / (max - min),  dbeta = sum dSR Rn |S|
                float s0, s1, r0, r1, g0, g1, a0, a1;
                f2_unpack(s_raw, s0, s1);
                f2_unpack(rb[e], r0, r1);
                f2_unpack(dsr, g0, g1);
                f2_unpack(arg[e], a0, a1);
                const float rn0 = fmaf(r0, fm.rn_a, fm.rn_b), rn1 = fmaf(r1, fm.rn_a, fm.rn_b);
                const float sg0 = (s0 > 0.f) ? 1.f : ((s0 < 0.f) ? -1.f : 0.f), sg1 = (s1 > 0.f) ? 1.f : ((s1 < 0.f) ? -1.f : 0.f);
                float sc0, sc1;
                f2_unpack(scale2, sc0, sc1);
                const float f0 = s0 != 0.f ? fmaf(fm.beta * rn0, sg0, 1.f) : 0.f, f1 = s1 != 0.f ? fmaf(fm.beta * rn1, sg1, 1.f) : 0.f;
                ds = f2_pack(g0 * sc0 * f0, g1 * sc1 * f1);
                dsig2 = f2_fma(f2_pack(g0 * fabsf(s0) * r0, g1 * fabsf(s1) * r1), f2_pack(fminf(a0, 0.f), fminf(a1, 0.f)), dsig2);
                dbeta2 = f2_add(dbeta2, f2_pack(g0 * rn0 * fabsf(s0), g1 * rn1 * fabsf(s1)));
            }
            float p0, p1, d0, d1;
            f2_unpack(x[e], p0, p1);
            f2_unpack(ds, d0, d1);
            pw[e] = pack_bf16x2(p0, p1);
            dw[e] = pack_bf16x2(d0, d1);
        }
        // the previous tile's dV / dK MMAs read the P and dS tiles: no store before they have completed
        if (gate != nullptr && g == 0) mbar_wait_timed(gate, gate_parity);
        const int chunk = chunk0 + g;
        const uint32_t off = (chunk >> 3) * GA_TILE_BYTES + sw128_offset(r, chunk & 7);
        *reinterpret_cast<uint4 *>(p_tile + off) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        *reinterpret_cast<uint4 *>(ds_tile + off) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
    }
}

__global__ void __launch_bounds__(GA_BWD_THREADS, 1)
geoattn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const GaBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaBwdSmem &sm = *reinterpret_cast<GaBwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_math = warp < GA_BWD_MATH_THREADS / 32;
    const int qtr = (warp >> 2) & 3;              // which 32 key columns / which 16 output columns
    const int r = (warp & 3) * 32 + lane;         // row inside a tile = TMEM lane
    int zh_local = blockIdx.y;
    if (p.order) {  // samples in the given order (longest first): neighbouring CTAs get similar amounts of work
        const int zp = zh_local / p.H;
        zh_local = p.order[zp] * p.H + (zh_local - zp * p.H);
    }
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int j0 = blockIdx.x * GA_BN;
    const int N = p.N;
    const float *cz = p.coords + (size_t)z * N * 3;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

    // ---- this CTA's keys ---------------------------------------------------------------------------
    const int jrow = j0 + r;  // the key whose dK / dV row this thread writes (16 of its 64 columns)
    const bool k_ok = is_math && jrow < N && (vz ? vz[jrow] != 0 : true);
    if (tid == 0) {
        sm.first_k = 0x7fffffff;
        sm.has_hole = 0;
    }
    // ---- query tiles with at least one valid query --------------------------------------------------
    const int all_tiles = (N + GA_BM - 1) / GA_BM;
    for (int t = warp; t < all_tiles; t += GA_BWD_THREADS / 32) {
        bool any = false;
        for (int i = t * GA_BM + lane; i < min(N, (t + 1) * GA_BM); i += 32) any |= vz ? (vz[i] != 0) : true;
        any = __any_sync(0xffffffffu, any);
        if (lane == 0) sm.tiles[t] = any ? 1 : 0;
    }
    __syncthreads();
    if (is_math && qtr == 0) {
        if (k_ok) atomicMin(&sm.first_k, r);
        else sm.has_hole = 1;
    }
    const bool cta_has_key = __syncthreads_or(k_ok ? 1 : 0) != 0;
    if (tid == 0) {
        int n = 0;
        for (int t = 0; t < all_tiles; ++t)
            if (sm.tiles[t]) sm.tiles[n++] = (uint16_t)t;
        sm.ntiles = n;
    }
    __syncthreads();
    const int nt = sm.ntiles;

    float *dk_row = p.dk + ((size_t)zh * N + jrow) * GA_D + qtr * 16;
    float *dv_row = p.dv + ((size_t)zh * N + jrow) * GA_D + qtr * 16;
    if (!cta_has_key || nt == 0) {
        if (is_math && jrow < N) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                reinterpret_cast<float4 *>(dk_row)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                reinterpret_cast<float4 *>(dv_row)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        return;
    }
    // origin of the centred coordinates: the first valid key of this tile
    const int ok_row = j0 + sm.first_k;
    const float orx = cz[ok_row * 3], ory = cz[ok_row * 3 + 1], orz = cz[ok_row * 3 + 2];
    const bool has_hole = sm.has_hole != 0;
    if (is_math && qtr == 0) {  // stage the centred keys
        const float x = k_ok ? cz[jrow * 3] - orx : 0.f, y = k_ok ? cz[jrow * 3 + 1] - ory : 0.f, zc = k_ok ? cz[jrow * 3 + 2] - orz : 0.f;
        float *a = reinterpret_cast<float *>(&sm.ka[r >> 1]);
        float *c = reinterpret_cast<float *>(&sm.kc[r >> 1]);
        a[r & 1] = x;
        a[2 + (r & 1)] = y;
        c[r & 1] = zc;
        c[2 + (r & 1)] = x * x + y * y + zc * zc;
        sm.kb[r] = k_ok ? 0.f : -INFINITY;
    }

    // ---- set-up ------------------------------------------------------------------------------------
    if (!is_math) {
        tmem_alloc(&sm.tmem_base, GA_BWD_TMEM_COLS);
        tmem_relinquish();
        if (lane == 0) {
            mbar_init(&sm.bar_kv, 1);
            mbar_init(&sm.bar_qdo[0], 1);
            mbar_init(&sm.bar_qdo[1], 1);
            mbar_init(&sm.bar_sp, 1);
            mbar_init(&sm.bar_g, 1);
            mbar_init(&sm.bar_vk, 1);
            mbar_init(&sm.bar_pds, GA_BWD_MATH_THREADS);
            mbar_init(&sm.bar_dqr, GA_BWD_MATH_THREADS);
            mbar_fence_init();
            fence_proxy_async();
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            tma_prefetch_desc(&map_do);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tm_s = tmem, tm_dp = tmem + 128, tm_dv = tmem + 256, tm_dk = tmem + 320, tm_dq = tmem + 384;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    if (!is_math) {
        // ================================ producer warp ==============================================
        if (lane == 0) {
            const uint32_t k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p), ds_addr = smem_u32(sm.ds);
            constexpr uint32_t IDESC_SP = umma_idesc_bf16(128, 128, false, false);
            constexpr uint32_t IDESC_TT = umma_idesc_bf16(128, GA_D, true, true);   // dV, dK
            constexpr uint32_t IDESC_DQ = umma_idesc_bf16(128, GA_D, false, true);  // dQ
            auto load_qdo = [&](int buf, int tile) {
                mbar_expect_tx(&sm.bar_qdo[buf], 2 * GA_TILE_BYTES);
                tma_load_3d(sm.q[buf], &map_q, 0, tile * GA_BM, zh_local, &sm.bar_qdo[buf]);
                tma_load_3d(sm.dout[buf], &map_do, 0, tile * GA_BM, zh_local, &sm.bar_qdo[buf]);
            };
            auto issue_s_dp = [&](int buf) {
                const uint32_t q_addr = smem_u32(sm.q[buf]), do_addr = smem_u32(sm.dout[buf]);
#pragma unroll
                for (int kk = 0; kk < GA_D / 16; ++kk)
                    umma_ss(tm_s, umma_desc_sw128(q_addr + kk * 32, 16, 1024), umma_desc_sw128(k_addr + kk * 32, 16, 1024),
                            IDESC_SP, kk > 0 ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < GA_D / 16; ++kk)
                    umma_ss(tm_dp, umma_desc_sw128(do_addr + kk * 32, 16, 1024), umma_desc_sw128(v_addr + kk * 32, 16, 1024),
                            IDESC_SP, kk > 0 ? 1u : 0u);
                umma_commit(&sm.bar_sp);
            };
            auto issue_dq = [&]() {  // the math warps wait for this one; K = 16 keys per step
#pragma unroll
                for (int kk = 0; kk < GA_BN / 16; ++kk)
                    umma_ss(tm_dq, umma_desc_sw128(ds_addr + (kk >> 2) * GA_TILE_BYTES + (kk & 3) * 32, 16, 1024),
                            umma_desc_sw128(k_addr + kk * 2048, 0, 1024), IDESC_DQ, kk > 0 ? 1u : 0u);
                umma_commit(&sm.bar_g);
            };
            auto issue_dv_dk = [&](int buf, bool first) {  // K = 16 query rows per step: 2 KiB down the [i][j] tiles
                const uint32_t q_addr = smem_u32(sm.q[buf]), do_addr = smem_u32(sm.dout[buf]);
#pragma unroll
                for (int kk = 0; kk < GA_BM / 16; ++kk) {
                    umma_ss(tm_dv, umma_desc_sw128(p_addr + kk * 2048, GA_TILE_BYTES, 1024),
                            umma_desc_sw128(do_addr + kk * 2048, 0, 1024), IDESC_TT, (first && kk == 0) ? 0u : 1u);
                    umma_ss(tm_dk, umma_desc_sw128(ds_addr + kk * 2048, GA_TILE_BYTES, 1024),
                            umma_desc_sw128(q_addr + kk * 2048, 0, 1024), IDESC_TT, (first && kk == 0) ? 0u : 1u);
                }
                umma_commit(&sm.bar_vk);
            };
            mbar_expect_tx(&sm.bar_kv, 2 * GA_TILE_BYTES);
            tma_load_3d(sm.k, &map_k, 0, j0, zh_local, &sm.bar_kv);
            tma_load_3d(sm.v, &map_v, 0, j0, zh_local, &sm.bar_kv);
            load_qdo(0, sm.tiles[0]);
            if (nt > 1) load_qdo(1, sm.tiles[1]);
            mbar_wait_timed(&sm.bar_kv, 0);
            mbar_wait_timed(&sm.bar_qdo[0], 0);
            tc_fence_after();
            issue_s_dp(0);
            for (int t = 0; t < nt; ++t) {
                const int buf = t & 1;
                const uint32_t par = (uint32_t)(t & 1);
                mbar_wait_timed(&sm.bar_pds, par);  // P, dS(t) written; S, dP(t) consumed
                if (t > 0) mbar_wait_timed(&sm.bar_dqr, par ^ 1);  // dQ(t-1) has been read out of TMEM
                tc_fence_after();
                // dQ(t) first (the math warps stage it next), then the next tile's S and dP so that its element-wise
                // stage can start while dV / dK(t) are still running; P and dS(t) stay untouched until bar_vk(t)
                issue_dq();
                if (t + 1 < nt) {
                    mbar_wait_timed(&sm.bar_qdo[buf ^ 1], (uint32_t)(((t + 1) >> 1) & 1));
                    issue_s_dp(buf ^ 1);
                }
                issue_dv_dk(buf, t == 0);
                if (t + 2 < nt) {  // Q / dO buffer `buf` is free once S, dP(t) and the gradient MMAs(t) are done
                    mbar_wait_timed(&sm.bar_vk, par);
                    load_qdo(buf, sm.tiles[t + 2]);
                }
            }
        }
        __syncwarp();
    } else {
        // ================================ math warps ==================================================
        const float sig = p.sigma[h];
        const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);
        const float c_s = p.scale * 1.4426950408889634f;
        const f2_t crbf2 = f2_pack(c_rbf, c_rbf), cs2 = f2_pack(c_s, c_s), scale2 = f2_pack(p.scale, p.scale);
        f2_t dsig2 = 0ull, dbeta2 = 0ull;
        GaForm fm = {0.f, 0.f, 0.f, 0.f, 1.f};
        if (p.form == 1) {
            fm.beta = p.beta[h];
            fm.rn_a = 2.f / (p.max_rbf - p.min_rbf);
            fm.rn_b = -2.f * p.min_rbf / (p.max_rbf - p.min_rbf) - 1.f;
            fm.rmin = p.min_rbf;
            fm.rmax = p.max_rbf;
        }

        float qcx, qcy, qcz, l2, dsum;
        auto load_row = [&](int tile) {
            const int row = tile * GA_BM + r;
            const bool q_ok = row < N && (vz ? vz[row] != 0 : true);
            qcx = qcy = qcz = 0.f;
            l2 = INFINITY;  // +inf: P = 0 for a padded query
            dsum = 0.f;
            if (q_ok) {
                qcx = cz[row * 3] - orx;
                qcy = cz[row * 3 + 1] - ory;
                qcz = cz[row * 3 + 2] - orz;
                const float lse = p.lse[(size_t)zh * N + row];
                l2 = lse == -INFINITY ? INFINITY : lse * 1.4426950408889634f;  // a row without any valid pair: P = 0
                dsum = p.dsum[(size_t)zh_local * N + row];
            }
        };
        load_row(sm.tiles[0]);
        for (int t = 0; t < nt; ++t) {
            const uint32_t par = (uint32_t)(t & 1);
            const int i0 = sm.tiles[t] * GA_BM;
            // per-row inputs of this query tile (loaded during the previous tile, see the end of the loop body)
            GaBwdRow rw;
            rw.qx2 = f2_pack(-2.f * qcx, -2.f * qcx);
            rw.qy2 = f2_pack(-2.f * qcy, -2.f * qcy);
            rw.qz2 = f2_pack(-2.f * qcz, -2.f * qcz);
            const float cqn = c_rbf * (qcx * qcx + qcy * qcy + qcz * qcz);
            rw.cqn2 = f2_pack(cqn, cqn);
            rw.l22 = f2_pack(l2, l2);
            rw.dsum2 = f2_pack(dsum, dsum);
            mbar_wait_timed(&sm.bar_sp, par);
            tc_fence_after();
#define PAI_GA_BWD(MASKED, FORM)                                                                                             \
    _Pragma("unroll") for (int c = 0; c < 2; ++c) ga_bwd_chunk<MASKED, FORM>(                                                \
        tm_s + lane_base + qtr * 32 + c * 16, tm_dp + lane_base + qtr * 32 + c * 16, &sm.ka[qtr * 16 + c * 8],               \
        &sm.kc[qtr * 16 + c * 8], &sm.kb[qtr * 32 + c * 16], rw, crbf2, cs2, scale2, fm, dsig2, dbeta2, sm.p, sm.ds, r,       \
        qtr * 4 + c * 2, (t > 0 && c == 0) ? &sm.bar_vk : nullptr, par ^ 1)
            if (p.form == 0) {
                if (has_hole) { PAI_GA_BWD(true, 0); } else { PAI_GA_BWD(false, 0); }
            } else {
                if (has_hole) { PAI_GA_BWD(true, 1); } else { PAI_GA_BWD(false, 1); }
            }
#undef PAI_GA_BWD
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(&sm.bar_pds);
            if (t + 1 < nt) load_row(sm.tiles[t + 1]);  // the loads fly while the MMAs run
            // dQ tile: TMEM -> registers -> vector reductions into the global fp32 dQ
            mbar_wait_timed(&sm.bar_g, par);
            tc_fence_after();
            {
                uint32_t v[16];
                tmem_ld16(tm_dq + lane_base + qtr * 16, v);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&sm.bar_dqr);
                const int row = i0 + r;
                if (row < N) {
                    float *dst = p.dq + ((size_t)zh * N + row) * GA_D + qtr * 16;
#pragma unroll
                    for (int e = 0; e < 16; e += 4)
                        red_add_v4(dst + e, __uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]),
                                   __uint_as_float(v[e + 3]));
                }
            }
        }

        // ---- epilogue: dV, dK rows of this key tile; dsigma -------------------------------------------
        mbar_wait_timed(&sm.bar_vk, (uint32_t)((nt - 1) & 1));  // the last dV / dK accumulation has completed
        tc_fence_after();
        {
            uint32_t a[16], b[16];
            tmem_ld16(tm_dv + lane_base + qtr * 16, a);
            tmem_ld16(tm_dk + lane_base + qtr * 16, b);
            tmem_wait_ld();
            if (jrow < N) {
#pragma unroll
                for (int e = 0; e < 16; e += 4) {
                    *reinterpret_cast<uint4 *>(dv_row + e) = make_uint4(a[e], a[e + 1], a[e + 2], a[e + 3]);
                    *reinterpret_cast<uint4 *>(dk_row + e) = make_uint4(b[e], b[e + 1], b[e + 2], b[e + 3]);
                }
            }
        }
        float d0, d1, b0, b1;
        f2_unpack(dsig2, d0, d1);
        f2_unpack(dbeta2, b0, b1);
        float dsig_acc = d0 + d1, dbeta_acc = b0 + b1;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            dsig_acc += __shfl_xor_sync(0xffffffffu, dsig_acc, off);
            dbeta_acc += __shfl_xor_sync(0xffffffffu, dbeta_acc, off);
        }
        if (lane == 0) {
            sm.dsig[warp] = dsig_acc;
            sm.dbeta[warp] = dbeta_acc;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        float tot = 0.f, totb = 0.f;
        for (int w = 0; w < GA_BWD_MATH_THREADS / 32; ++w) {
            tot += sm.dsig[w];
            totb += sm.dbeta[w];
        }
        const float sig = p.sigma[h];
        const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);
        if (p.form == 0) {
            // sum of dSR * S_raw * R * (c_rbf d^2), S = scale * S_raw:  dsigma = sum dSR S R d^2 / sigma^3
            atomicAdd(p.dsigma + h, tot * p.scale / (c_rbf * sig * sig * sig));
        } else {
            // sum of dSR * |S_raw| * R * (c_rbf d^2):  dsigma = sum dR R d^2 / sigma^3 with dR = dSR |S| 2 beta / (max - min)
            atomicAdd(p.dsigma + h, tot * p.scale * 2.f * p.beta[h] / ((p.max_rbf - p.min_rbf) * c_rbf * sig * sig * sig));
            if (p.dbeta) atomicAdd(p.dbeta + h, totb * p.scale);
        }
    }
    if (warp == GA_BWD_MATH_THREADS / 32) tmem_dealloc(tmem, GA_BWD_TMEM_COLS);
}

}  // namespace pai
