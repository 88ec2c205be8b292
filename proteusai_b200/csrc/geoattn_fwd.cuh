// Geometric attention forward for sm_100a: flash attention on tcgen05 tensor cores with the
// per-head radial-basis scale applied in the softmax stage,
//     SR_ij = (q_i . k_j / sqrt(d)) * (1 + exp(-|r_i - r_j|^2 / (2 sigma_h^2))),
// a pair being valid iff query i and key j are both unpadded.  Replaces the Triton kernel
// `_attn_fwd` (old/old_scripts/attn/geometric_attn.py:57-260) with the logit form the reference's
// README states (README.md:40).
//
// One CTA = 128 query rows of one (batch, head); thread t owns row t = TMEM lane t.
//   S  = Q K^T : tcgen05.mma, A = Q tile, B = K tile (both K-major, 128-byte swizzle, via TMA),
//                accumulator [128 lanes x 128 columns] fp32 in TMEM;
//   softmax    : each thread reads its row with tcgen05.ld, applies scale * (1 + R) and the key
//                mask, updates the running maximum / sum, and writes P as bf16 into shared memory
//                in the same swizzled K-major layout TMA would have produced;
//   PV = P V   : tcgen05.mma, A = P tile (K-major), B = V tile (MN-major: keys are the K dimension),
//                accumulator [128 x 64] fp32 in TMEM, read back and folded into the register-held
//                output row with the usual rescale.
// K and V are single-buffered: K(t+1) is fetched as soon as S(t) has completed and V(t+1) as soon
// as PV(t) has, so both loads overlap the softmax of the neighbouring tile; S(t+1) is issued right
// behind PV(t).  Two CTAs fit one SM (84 kB shared memory, 256 TMEM columns each) and overlap one
// CTA's softmax with the other's MMAs.  Key tiles without any valid key are skipped, CTAs without any
// valid query only write zeros.
#pragma once
#include "tc.cuh"

namespace pai {

constexpr int GA_BM = 128;  // query rows per CTA
constexpr int GA_BN = 128;  // keys per tile
constexpr int GA_D = 64;    // head dimension
constexpr int GA_MAX_TILES = 1024;
constexpr uint32_t GA_TMEM_COLS = 256;
constexpr uint32_t GA_TILE_BYTES = GA_BN * GA_D * 2;  // 16 KiB

struct GaFwdSmem {
    alignas(1024) uint8_t q[GA_TILE_BYTES];
    alignas(1024) uint8_t k[GA_TILE_BYTES];
    alignas(1024) uint8_t v[GA_TILE_BYTES];
    alignas(1024) uint8_t p[2 * GA_TILE_BYTES];  // [128 x 128] bf16 as two [128 x 64] swizzled sub-tiles
    float4 kc[2][GA_BN];                          // key {x, y, z, valid} for the current / next tile
    uint16_t tiles[GA_MAX_TILES];                 // key tiles that hold at least one valid key
    uint64_t bar_q, bar_k, bar_v, bar_s, bar_o;
    uint32_t tmem_base;
    int ntiles;
};

struct GaFwdParams {
    const float *coords;   // [Z,N,3]
    const uint8_t *valid;  // [Z,N] or nullptr
    const float *sigma;    // [H]
    __nv_bfloat16 *out;    // [Z,H,N,64]
    float *lse;            // [Z,H,N]  log-sum-exp of SR (natural log), -inf for padded queries
    int Z, H, N, zh_begin;
    float scale;
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

__global__ void __launch_bounds__(128, 2)
geoattn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const GaFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaFwdSmem &sm = *reinterpret_cast<GaFwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int zh_local = blockIdx.y;              // index into the tensor maps (they start at zh_begin)
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int i0 = blockIdx.x * GA_BM;
    const int N = p.N;
    const int row = i0 + tid;
    const float *cz = p.coords + (size_t)z * N * 3;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

    // ---- this thread's query -------------------------------------------------------------------
    const bool q_ok = row < N && (vz ? vz[row] != 0 : true);
    float qx = 0.f, qy = 0.f, qz = 0.f;
    if (q_ok) {
        qx = cz[row * 3];
        qy = cz[row * 3 + 1];
        qz = cz[row * 3 + 2];
    }
    // ---- key tiles with at least one valid key ----------------------------------------------------
    const int all_tiles = (N + GA_BN - 1) / GA_BN;
    for (int t = warp; t < all_tiles; t += 4) {
        bool any = false;
        for (int j = t * GA_BN + lane; j < min(N, (t + 1) * GA_BN); j += 32) any |= vz ? (vz[j] != 0) : true;
        any = __any_sync(0xffffffffu, any);
        if (lane == 0) sm.tiles[t] = any ? 1 : 0;
    }
    const bool cta_has_query = __syncthreads_or(q_ok ? 1 : 0) != 0;
    if (tid == 0) {
        int n = 0;
        for (int t = 0; t < all_tiles; ++t)
            if (sm.tiles[t]) sm.tiles[n++] = (uint16_t)t;  // in place: n <= t
        sm.ntiles = n;
    }
    __syncthreads();
    const int nt = sm.ntiles;

    __nv_bfloat16 *orow = p.out + ((size_t)zh * N + row) * GA_D;
    if (!cta_has_query || nt == 0) {  // nothing to attend from / to: zeros and -inf
        if (row < N) {
#pragma unroll
            for (int c = 0; c < GA_D / 8; ++c) reinterpret_cast<uint4 *>(orow)[c] = make_uint4(0, 0, 0, 0);
            p.lse[(size_t)zh * N + row] = -INFINITY;
        }
        return;
    }

    // ---- set-up: TMEM, barriers, first loads -------------------------------------------------------
    if (warp == 0) {
        tmem_alloc(&sm.tmem_base, GA_TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&sm.bar_q, 1);
        mbar_init(&sm.bar_k, 1);
        mbar_init(&sm.bar_v, 1);
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_fence_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
    }
    auto load_kc = [&](int buf, int tile) {  // thread t stages key tile*128 + t
        const int j = tile * GA_BN + tid;
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < N && (vz ? vz[j] != 0 : true)) c = make_float4(cz[j * 3], cz[j * 3 + 1], cz[j * 3 + 2], 1.f);
        sm.kc[buf][tid] = c;
    };
    load_kc(0, sm.tiles[0]);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_s = tmem;          // columns [0,128): S
    const uint32_t tmem_o = tmem + 128;    // columns [128,192): P V of the current tile
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;

    const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p);
    constexpr uint32_t IDESC_S = umma_idesc_bf16(GA_BM, GA_BN, false, false);  // Q K^T: both K-major
    constexpr uint32_t IDESC_O = umma_idesc_bf16(GA_BM, GA_D, false, true);    // P V: V is MN-major

    auto issue_s = [&]() {  // 4 MMAs of K = 16 over d = 64: advance 32 B inside the swizzled row
#pragma unroll
        for (int kk = 0; kk < GA_D / 16; ++kk)
            umma_ss(tmem_s, umma_desc_sw128(q_addr + kk * 32, 16, 1024), umma_desc_sw128(k_addr + kk * 32, 16, 1024), IDESC_S,
                    kk > 0 ? 1u : 0u);
        umma_commit(&sm.bar_s);
    };
    auto issue_pv = [&]() {  // 8 MMAs of K = 16 keys: P advances 32 B (second sub-tile after 64 keys), V 2 KiB
#pragma unroll
        for (int kk = 0; kk < GA_BN / 16; ++kk)
            umma_ss(tmem_o, umma_desc_sw128(p_addr + (kk >> 2) * GA_TILE_BYTES + (kk & 3) * 32, 16, 1024),
                    umma_desc_sw128(v_addr + kk * 2048, 0, 1024), IDESC_O, kk > 0 ? 1u : 0u);
        umma_commit(&sm.bar_o);
    };

    if (tid == 0) {
        mbar_expect_tx(&sm.bar_q, GA_TILE_BYTES);
        tma_load_3d(sm.q, &map_q, 0, i0, zh_local, &sm.bar_q);
        mbar_expect_tx(&sm.bar_k, GA_TILE_BYTES);
        tma_load_3d(sm.k, &map_k, 0, sm.tiles[0] * GA_BN, zh_local, &sm.bar_k);
        mbar_expect_tx(&sm.bar_v, GA_TILE_BYTES);
        tma_load_3d(sm.v, &map_v, 0, sm.tiles[0] * GA_BN, zh_local, &sm.bar_v);
        mbar_wait_timed(&sm.bar_q, 0);
        mbar_wait_timed(&sm.bar_k, 0);
        tc_fence_after();
        issue_s();
    }

    // ---- main loop ---------------------------------------------------------------------------------
    const float sig = p.sigma[h];
    const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);  // R = 2^(c_rbf * d^2)
    const float c_s = p.scale * 1.4426950408889634f;               // logits in base-2 units
    float m_run = -INFINITY, l_run = 0.f;
    float o[GA_D];
#pragma unroll
    for (int c = 0; c < GA_D; ++c) o[c] = 0.f;

    for (int t = 0; t < nt; ++t) {
        const uint32_t par = (uint32_t)(t & 1);
        const float4 *kc = sm.kc[t & 1];
        // S(t) has landed in TMEM; the K buffer is free again
        mbar_wait_timed(&sm.bar_s, par);
        tc_fence_after();
        if (tid == 0 && t + 1 < nt) {
            mbar_expect_tx(&sm.bar_k, GA_TILE_BYTES);
            tma_load_3d(sm.k, &map_k, 0, sm.tiles[t + 1] * GA_BN, zh_local, &sm.bar_k);
        }
        float s[GA_BN];
#pragma unroll
        for (int c = 0; c < GA_BN / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(tmem_s + lane_base + c * 32, v);
#pragma unroll
            for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(v[e]);
        }
        tmem_wait_ld();
        // scale by (1 + R), mask, running maximum
        float m_new = m_run;
#pragma unroll
        for (int j = 0; j < GA_BN; ++j) {
            const float4 kj = kc[j];
            const float dx = qx - kj.x, dy = qy - kj.y, dz = qz - kj.z;
            const float d2 = dx * dx + dy * dy + dz * dz;
            const float r = ex2_approx(d2 * c_rbf);
            const float t2 = s[j] * c_s;
            const float sr = kj.w != 0.f ? fmaf(t2, r, t2) : -INFINITY;
            s[j] = sr;
            m_new = fmaxf(m_new, sr);
        }
        // every listed tile holds a valid key, so m_new is finite from the first tile on
        const float alpha = ex2_approx(m_run - m_new);
        float l_tile = 0.f;
#pragma unroll
        for (int c = 0; c < GA_BN / 8; ++c) {  // 8 keys = one 16-byte chunk of the swizzled row
            float e[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                e[q] = ex2_approx(s[c * 8 + q] - m_new);
                l_tile += e[q];
            }
            const uint4 pk = make_uint4(pack_bf16x2(e[0], e[1]), pack_bf16x2(e[2], e[3]), pack_bf16x2(e[4], e[5]),
                                        pack_bf16x2(e[6], e[7]));
            *reinterpret_cast<uint4 *>(sm.p + (c >> 3) * GA_TILE_BYTES + sw128_offset(tid, c & 7)) = pk;
        }
        l_run = l_run * alpha + l_tile;
        m_run = m_new;
        fence_proxy_async();  // P (generic-proxy stores) must be visible to the tensor core
        tc_fence_before();
        __syncthreads();      // P complete; everyone has finished reading S(t) from TMEM
        if (tid == 0) {
            tc_fence_after();
            mbar_wait_timed(&sm.bar_v, par);
            issue_pv();
            if (t + 1 < nt) {
                mbar_wait_timed(&sm.bar_k, par ^ 1);
                issue_s();  // S(t+1) runs behind P V(t) while the rows below are folded in
            }
        }
        mbar_wait_timed(&sm.bar_o, par);
        tc_fence_after();
        if (tid == 0 && t + 1 < nt) {  // the V buffer is free again
            mbar_expect_tx(&sm.bar_v, GA_TILE_BYTES);
            tma_load_3d(sm.v, &map_v, 0, sm.tiles[t + 1] * GA_BN, zh_local, &sm.bar_v);
        }
#pragma unroll
        for (int c = 0; c < GA_D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_base + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], alpha, __uint_as_float(v[e]));
        }
        if (t + 1 < nt) load_kc((t + 1) & 1, sm.tiles[t + 1]);
        tc_fence_before();
        __syncthreads();  // key coordinates of the next tile are staged; P V(t) has been read by everyone
    }

    // ---- epilogue ------------------------------------------------------------------------------------
    if (row < N) {
        const bool live = q_ok && l_run > 0.f;
        const float inv = live ? 1.f / l_run : 0.f;
#pragma unroll
        for (int c = 0; c < GA_D / 8; ++c) {
            uint4 pk;
            pk.x = pack_bf16x2(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
            pk.y = pack_bf16x2(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
            pk.z = pack_bf16x2(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
            pk.w = pack_bf16x2(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
            reinterpret_cast<uint4 *>(orow)[c] = pk;
        }
        p.lse[(size_t)zh * N + row] = live ? (m_run + lg2_approx(l_run)) * 0.6931471805599453f : -INFINITY;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, GA_TMEM_COLS);
}

}  // namespace pai
