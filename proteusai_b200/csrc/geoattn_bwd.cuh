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
// One CTA = 128 keys of one (batch, head); it loops over the 128-row query tiles.  Thread t owns
// query row t of the current tile = TMEM lane t.  Five MMAs per query tile, all operands straight
// from the TMA-written swizzled tiles, transposes expressed through the operand major-ness:
//     S   = Q_i K_j^T     A K-major,  B K-major     -> TMEM [128 x 128]
//     dP  = dO_i V_j^T    A K-major,  B K-major     -> TMEM [128 x 128]
//     dV += P^T dO_i      A MN-major, B MN-major    -> TMEM [128 x 64], accumulated over i
//     dK += dS^T Q_i      A MN-major, B MN-major    -> TMEM [128 x 64], accumulated over i
//     dQ_i = dS K_j       A K-major,  B MN-major    -> TMEM [128 x 64], reduced into global fp32 dQ
//                                                      with bulk reduce-add copies (one per warp)
// P and dS are written by the threads as bf16 into shared memory in the swizzled [i][j] layout,
// which serves both as K-major (dQ) and MN-major (dV, dK) operand.  Query tiles without a valid
// query are skipped, a key tile without a valid key only writes zeros.
#pragma once
#include "geoattn_fwd.cuh"

namespace pai {

constexpr uint32_t GA_BWD_TMEM_COLS = 512;

struct GaBwdSmem {
    alignas(1024) uint8_t k[GA_TILE_BYTES];
    alignas(1024) uint8_t v[GA_TILE_BYTES];
    alignas(1024) uint8_t q[2][GA_TILE_BYTES];
    alignas(1024) uint8_t dout[2][GA_TILE_BYTES];
    alignas(1024) uint8_t p[2 * GA_TILE_BYTES];
    alignas(1024) uint8_t ds[2 * GA_TILE_BYTES];
    alignas(1024) float dq[GA_BM * GA_D];  // fp32 staging for the reduce-add, row-major
    float4 kc[GA_BN];                      // key {x, y, z, valid}
    uint16_t tiles[GA_MAX_TILES];          // query tiles that hold at least one valid query
    uint64_t bar_kv, bar_qdo[2], bar_sp, bar_g;
    uint32_t tmem_base;
    int ntiles;
    float dsig[4];
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
    int Z, H, N, zh_begin;
    float scale;
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

__device__ __forceinline__ void bulk_reduce_add_f32(float *dst_gmem, const float *src_smem, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_u32(src_smem)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(128, 1)
geoattn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const GaBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaBwdSmem &sm = *reinterpret_cast<GaBwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int zh_local = blockIdx.y;
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int j0 = blockIdx.x * GA_BN;
    const int N = p.N;
    const float *cz = p.coords + (size_t)z * N * 3;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

    // ---- this thread's key (for the staging of coordinates and the final dK / dV row) -------------
    const int jrow = j0 + tid;
    const bool k_ok = jrow < N && (vz ? vz[jrow] != 0 : true);
    {
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k_ok) c = make_float4(cz[jrow * 3], cz[jrow * 3 + 1], cz[jrow * 3 + 2], 1.f);
        sm.kc[tid] = c;
    }
    // ---- query tiles with at least one valid query --------------------------------------------------
    const int all_tiles = (N + GA_BM - 1) / GA_BM;
    for (int t = warp; t < all_tiles; t += 4) {
        bool any = false;
        for (int i = t * GA_BM + lane; i < min(N, (t + 1) * GA_BM); i += 32) any |= vz ? (vz[i] != 0) : true;
        any = __any_sync(0xffffffffu, any);
        if (lane == 0) sm.tiles[t] = any ? 1 : 0;
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

    float *dk_row = p.dk + ((size_t)zh * N + jrow) * GA_D;
    float *dv_row = p.dv + ((size_t)zh * N + jrow) * GA_D;
    if (!cta_has_key || nt == 0) {
        if (jrow < N) {
#pragma unroll
            for (int c = 0; c < GA_D / 4; ++c) {
                reinterpret_cast<float4 *>(dk_row)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                reinterpret_cast<float4 *>(dv_row)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        return;
    }

    // ---- set-up ------------------------------------------------------------------------------------
    if (warp == 0) {
        tmem_alloc(&sm.tmem_base, GA_BWD_TMEM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        mbar_init(&sm.bar_kv, 1);
        mbar_init(&sm.bar_qdo[0], 1);
        mbar_init(&sm.bar_qdo[1], 1);
        mbar_init(&sm.bar_sp, 1);
        mbar_init(&sm.bar_g, 1);
        mbar_fence_init();
        fence_proxy_async();
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        tma_prefetch_desc(&map_do);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tm_s = tmem, tm_dp = tmem + 128, tm_dv = tmem + 256, tm_dk = tmem + 320, tm_dq = tmem + 384;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const uint32_t k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v), p_addr = smem_u32(sm.p), ds_addr = smem_u32(sm.ds);
    constexpr uint32_t IDESC_SP = umma_idesc_bf16(128, 128, false, false);
    constexpr uint32_t IDESC_TT = umma_idesc_bf16(128, GA_D, true, true);   // dV, dK
    constexpr uint32_t IDESC_DQ = umma_idesc_bf16(128, GA_D, false, true);  // dQ

    auto load_qdo = [&](int buf, int tile) {  // thread 0 only
        mbar_expect_tx(&sm.bar_qdo[buf], 2 * GA_TILE_BYTES);
        tma_load_3d(sm.q[buf], &map_q, 0, tile * GA_BM, zh_local, &sm.bar_qdo[buf]);
        tma_load_3d(sm.dout[buf], &map_do, 0, tile * GA_BM, zh_local, &sm.bar_qdo[buf]);
    };
    auto issue_s_dp = [&](int buf) {
        const uint32_t q_addr = smem_u32(sm.q[buf]), do_addr = smem_u32(sm.dout[buf]);
#pragma unroll
        for (int kk = 0; kk < GA_D / 16; ++kk)
            umma_ss(tm_s, umma_desc_sw128(q_addr + kk * 32, 16, 1024), umma_desc_sw128(k_addr + kk * 32, 16, 1024), IDESC_SP,
                    kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < GA_D / 16; ++kk)
            umma_ss(tm_dp, umma_desc_sw128(do_addr + kk * 32, 16, 1024), umma_desc_sw128(v_addr + kk * 32, 16, 1024), IDESC_SP,
                    kk > 0 ? 1u : 0u);
        umma_commit(&sm.bar_sp);
    };
    auto issue_grads = [&](int buf, bool first) {
        const uint32_t q_addr = smem_u32(sm.q[buf]), do_addr = smem_u32(sm.dout[buf]);
#pragma unroll
        for (int kk = 0; kk < GA_BM / 16; ++kk) {  // K = 16 query rows per step: 2 KiB down the [i][j] tiles
            umma_ss(tm_dv, umma_desc_sw128(p_addr + kk * 2048, GA_TILE_BYTES, 1024), umma_desc_sw128(do_addr + kk * 2048, 0, 1024),
                    IDESC_TT, (first && kk == 0) ? 0u : 1u);
            umma_ss(tm_dk, umma_desc_sw128(ds_addr + kk * 2048, GA_TILE_BYTES, 1024), umma_desc_sw128(q_addr + kk * 2048, 0, 1024),
                    IDESC_TT, (first && kk == 0) ? 0u : 1u);
        }
#pragma unroll
        for (int kk = 0; kk < GA_BN / 16; ++kk)  // K = 16 keys per step
            umma_ss(tm_dq, umma_desc_sw128(ds_addr + (kk >> 2) * GA_TILE_BYTES + (kk & 3) * 32, 16, 1024),
                    umma_desc_sw128(k_addr + kk * 2048, 0, 1024), IDESC_DQ, kk > 0 ? 1u : 0u);
        umma_commit(&sm.bar_g);
    };

    if (tid == 0) {
        mbar_expect_tx(&sm.bar_kv, 2 * GA_TILE_BYTES);
        tma_load_3d(sm.k, &map_k, 0, j0, zh_local, &sm.bar_kv);
        tma_load_3d(sm.v, &map_v, 0, j0, zh_local, &sm.bar_kv);
        load_qdo(0, sm.tiles[0]);
        if (nt > 1) load_qdo(1, sm.tiles[1]);
        mbar_wait_timed(&sm.bar_kv, 0);
        mbar_wait_timed(&sm.bar_qdo[0], 0);
        tc_fence_after();
        issue_s_dp(0);
    }

    const float sig = p.sigma[h];
    const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);
    const float c_s = p.scale * 1.4426950408889634f;
    float dsig_acc = 0.f;
    float *stage = sm.dq + warp * 32 * GA_D;  // this warp's 32 rows of the reduce-add staging

    for (int t = 0; t < nt; ++t) {
        const int buf = t & 1;
        const uint32_t par = (uint32_t)(t & 1);
        const int i0 = sm.tiles[t] * GA_BM;
        const int row = i0 + tid;
        // per-row inputs of this query tile (overlaps the S / dP MMAs)
        const bool q_ok = row < N && (vz ? vz[row] != 0 : true);
        float qx = 0.f, qy = 0.f, qz = 0.f, l2 = 0.f, dsum = 0.f;
        if (q_ok) {
            qx = cz[row * 3];
            qy = cz[row * 3 + 1];
            qz = cz[row * 3 + 2];
            l2 = p.lse[(size_t)zh * N + row] * 1.4426950408889634f;
            dsum = p.dsum[(size_t)zh_local * N + row];
        }
        mbar_wait_timed(&sm.bar_sp, par);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < GA_BN / 32; ++c) {
            uint32_t sv[32], dpv[32];
            tmem_ld32(tm_s + lane_base + c * 32, sv);
            tmem_ld32(tm_dp + lane_base + c * 32, dpv);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < 4; ++g) {  // 8 keys = one 16-byte chunk
                float pe[8], de[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int j = c * 32 + g * 8 + q;
                    const float4 kj = sm.kc[j];
                    const float dx = qx - kj.x, dy = qy - kj.y, dz = qz - kj.z;
                    const float d2 = dx * dx + dy * dy + dz * dz;
                    const float r = ex2_approx(d2 * c_rbf);
                    const float s_raw = __uint_as_float(sv[g * 8 + q]);
                    const float t2 = s_raw * c_s;
                    const bool ok = q_ok && kj.w != 0.f;
                    const float pr = ok ? ex2_approx(fmaf(t2, r, t2) - l2) : 0.f;
                    const float dsr = pr * (__uint_as_float(dpv[g * 8 + q]) - dsum);
                    pe[q] = pr;
                    de[q] = dsr * (1.f + r) * p.scale;
                    dsig_acc = fmaf(dsr * (s_raw * p.scale), r * d2, dsig_acc);
                }
                const int chunk = c * 4 + g;  // 16-byte chunk index along the 128 keys
                const uint32_t off = (chunk >> 3) * GA_TILE_BYTES + sw128_offset(tid, chunk & 7);
                *reinterpret_cast<uint4 *>(sm.p + off) = make_uint4(pack_bf16x2(pe[0], pe[1]), pack_bf16x2(pe[2], pe[3]),
                                                                     pack_bf16x2(pe[4], pe[5]), pack_bf16x2(pe[6], pe[7]));
                *reinterpret_cast<uint4 *>(sm.ds + off) = make_uint4(pack_bf16x2(de[0], de[1]), pack_bf16x2(de[2], de[3]),
                                                                      pack_bf16x2(de[4], de[5]), pack_bf16x2(de[6], de[7]));
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();  // P and dS complete; S and dP have been read by everyone
        if (tid == 0) {
            tc_fence_after();
            issue_grads(buf, t == 0);
            if (t + 1 < nt) {
                mbar_wait_timed(&sm.bar_qdo[buf ^ 1], (uint32_t)(((t + 1) >> 1) & 1));
                issue_s_dp(buf ^ 1);  // next tile's S / dP run behind the gradient MMAs
            }
        }
        mbar_wait_timed(&sm.bar_g, par);
        tc_fence_after();
        if (tid == 0 && t + 2 < nt) load_qdo(buf, sm.tiles[t + 2]);  // Q / dO buffer `buf` is free again
        // dQ tile: TMEM -> fp32 staging -> bulk reduce-add into global dQ (one copy per warp)
        if (lane == 0) bulk_wait_group_read0();  // the previous copy has finished reading the staging
        __syncwarp();
#pragma unroll
        for (int c = 0; c < GA_D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(tm_dq + lane_base + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; e += 4)
                *reinterpret_cast<uint4 *>(stage + lane * GA_D + c * 32 + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            const int r0 = i0 + warp * 32;
            const int nrows = min(32, N - r0);
            if (nrows > 0) {
                bulk_reduce_add_f32(p.dq + ((size_t)zh * N + r0) * GA_D, stage, (uint32_t)nrows * GA_D * 4);
                bulk_commit_group();
            }
        }
        tc_fence_before();
        __syncthreads();  // dQ tile has been read by everyone before the next gradient MMAs overwrite it
    }

    // ---- epilogue: dV, dK rows of this key tile; dsigma -----------------------------------------------
    // (the last bar_g wait above covers the final accumulation)
#pragma unroll
    for (int c = 0; c < GA_D / 32; ++c) {
        uint32_t a[32], b[32];
        tmem_ld32(tm_dv + lane_base + c * 32, a);
        tmem_ld32(tm_dk + lane_base + c * 32, b);
        tmem_wait_ld();
        if (jrow < N) {
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
                *reinterpret_cast<uint4 *>(dv_row + c * 32 + e) = make_uint4(a[e], a[e + 1], a[e + 2], a[e + 3]);
                *reinterpret_cast<uint4 *>(dk_row + c * 32 + e) = make_uint4(b[e], b[e + 1], b[e + 2], b[e + 3]);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dsig_acc += __shfl_xor_sync(0xffffffffu, dsig_acc, off);
    if (lane == 0) sm.dsig[warp] = dsig_acc;
    if (lane == 0) bulk_wait_group0();  // the reduce-add copies of this warp have completed
    tc_fence_before();
    __syncthreads();
    if (tid == 0) atomicAdd(p.dsigma + h, (sm.dsig[0] + sm.dsig[1] + sm.dsig[2] + sm.dsig[3]) / (sig * sig * sig));
    if (warp == 0) tmem_dealloc(tmem, GA_BWD_TMEM_COLS);
}

}  // namespace pai
