// Geometric attention backward for sm_100a (tcgen05 / TMEM / TMA).
//
// Replaces the Triton kernel `_attn_bwd` (old/old_scripts/attn/geometric_attn.py:265-543) and the
// PyTorch row-sum in front of it (:616), for the logit form SR = S (1 + R), S = scale q.k,
// R = exp(-d^2 / (2 sigma_h^2)) (and for the reference tree's own form, FORM = 1):
//     D_i   = sum_d O_id dO_id                       (pre-pass, fp32 scratch; the same pass zeroes dQ)
//     P_ij  = exp(SR_ij - L_i)                        (recomputed from the stored log-sum-exp)
//     dV_j  = sum_i P_ij dO_i
//     dP_ij = dO_i . V_j
//     dSR   = P (dP - D)
//     dS    = dSR (1 + R) scale        -> dQ_i = sum_j dS_ij K_j,   dK_j = sum_i dS_ij Q_i
//     dsigma_h = sum_{z,i,j} dSR S R d^2 / sigma_h^3
//
// One work item = 128 keys of one (batch, head); the CTA loops over the live 128-row query tiles, 64 queries (a
// "sub-tile") at a time.  The logit tile is computed TRANSPOSED, keys on the TMEM lanes and queries along the columns,
// so that a math thread owns a key:
//     S^T  = K_j Q_i^T     A, B K-major                          -> TMEM [128 keys x 64 queries], two stages
//     dP^T = V_j dO_i^T    A, B K-major                          -> TMEM [128 x 64], two stages
//     dV  += P^T dO_i      A = P^T read from TENSOR MEMORY (bf16 pairs written by the math threads), B = dO MN-major
//     dK  += dS^T Q_i      A = dS^T from shared memory, K-major (the math threads write row j = their key, the
//                          queries contiguous: 16-byte stores), B = Q MN-major
//     dQ_i = dS K_j        A = the same dS^T tile read MN-major, B = K MN-major -> TMEM [128 queries x 64], once per
//                          query tile, read back and added into the global fp32 dQ with vector reductions
// Sixteen math warps: key row r = TMEM lane r is shared by four math threads (warps w, w + 4, w + 8, w + 12), each
// taking 16 of the sub-tile's 64 query columns.  A thread reads its S^T and dP^T values into registers and releases
// the stage at once; with two stages the tensor core is a sub-tile ahead and the warps may drift a sub-tile apart
// (their work differs: see the far groups below).  Two threads issue the MMAs, one S^T / dP^T of the sub-tiles
// ahead, one dV / dK / dQ behind and the TMA loads of Q and dO: an MMA holds its issuing thread until the tensor
// core has taken it, and one thread doing all of it, with its waits in between, was the slowest part of the CTA.
// A stager warp keeps the per-query inputs (centred coordinates, log-sum-exp, D, validity, bounding spheres of
// 16 queries) in shared memory up to three query tiles ahead; the pair geometry takes four packed FMAs a pair from
// them (every lane reads the same entry).  Query groups farther than 5.9 sigma_h from a warp's 32 keys skip the RBF
// arithmetic (R < 2^-25 there).  dQ reductions and the dK / dV rows leave through per-warp staging so that every
// instruction covers whole 32-byte sectors.  Query tiles without a valid query are skipped, a key tile without a
// valid key only writes zeros.  Work items come one per CTA or from a balanced schedule (geoattn_plan.cuh).  Every
// wait is bounded and abortable (tc.cuh).
#pragma once
#include "geoattn_fwd.cuh"

namespace pai {

constexpr uint32_t GA_BWD_TMEM_COLS = 512;
constexpr int GA_BWD_MATH_THREADS = 512;
constexpr int GA_BWD_THREADS = GA_BWD_MATH_THREADS + 96;  // + the two issuer warps and the stager warp
constexpr int GA_ROW_BUFS = 3;
constexpr int GA_SUB = 64;  // queries per sub-tile (two sub-tiles per 128-row query tile)

struct GaQueryRows {                  // per-query inputs of one query tile, two queries per entry
    float4 qa[GA_BM / 2];             // centred coordinates {x_i, x_i+1, y_i, y_i+1}
    float4 qc[GA_BM / 2];             // {z_i, z_i+1, |q_i|^2, |q_i+1|^2}
    float4 ld[GA_BM / 2];             // {-L_i, -L_i+1, D_i, D_i+1}: minus the log-sum-exp in base-2 units (-inf: padded query or row
                                      // without a valid pair) and D
    uint32_t qbits[GA_BM / 32];       // bit i of word u: query 32 u + i is valid
    float4 sph[GA_BM / 16];           // bounding sphere of each group of 16 queries (radius < 0: no valid query)
};

struct GaBwdSmem {
    alignas(1024) uint8_t k[GA_TILE_BYTES];
    alignas(1024) uint8_t v[GA_TILE_BYTES];
    alignas(1024) uint8_t q[2][GA_TILE_BYTES];
    alignas(1024) uint8_t dout[2][GA_TILE_BYTES];
    alignas(1024) uint8_t ds[2][2 * GA_TILE_BYTES];  // dS^T [128 keys x 128 queries] bf16: two [128 x 64] swizzled sub-tiles
    GaQueryRows rows[GA_ROW_BUFS];
    alignas(16) float stage[GA_BWD_MATH_THREADS / 32][32 * 16];  // per-warp staging of outgoing rows (ga_warp_rows_out)
    uint16_t tiles[GA_MAX_TILES];          // live query tiles of the range; bit 15: the tile also holds a padded query
    uint64_t bar_kv, bar_qdo[2], bar_sp[2], bar_spfree[2], bar_pds, bar_vk, bar_dq, bar_dqr, bar_rows[GA_ROW_BUFS], bar_rowsfree[GA_ROW_BUFS];
    uint32_t tmem_base;
    int abort;
    float dsig[GA_BWD_MATH_THREADS / 32];
    float dbeta[GA_BWD_MATH_THREADS / 32];
};

struct GaBwdParams {
    const float *coords;   // [Z,N,3]
    const uint8_t *valid;  // [Z,N] or nullptr
    const int *plan;       // batch plan (geoattn_plan.cuh); nullptr iff valid is nullptr
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
    int use_order;         // issue the samples in the plan's longest-first order
    int far_skip;          // skip the RBF arithmetic of far query groups
    const int *sched;      // balanced schedule (geoattn_plan.cuh) or nullptr: one CTA per item
    int qt_begin, qt_end;  // query tiles [qt_begin, qt_end) are visited
};

// Pre-pass: D[pair, i] = sum_d O * dO for the query rows [q_begin, q_begin + q_rows) of every (batch, head) pair of
// the range, and zeros into the same rows of dQ, which the main kernel accumulates with reductions.  Eight threads
// per row (16-byte loads of 8 bf16, two 16-byte stores of zeros each), four rows per warp; o, d_out, dsum and dq point
// at the first pair of the range.
__global__ void __launch_bounds__(256) geoattn_bwd_prep_kernel(const __nv_bfloat16 *o, const __nv_bfloat16 *d_out, float *dsum,
                                                               float *dq, int N, int q_begin, int q_rows, long long rows) {
    const long long idx = (long long)blockIdx.x * 32 + (threadIdx.x >> 3);  // (pair, row inside the range)
    const int part = threadIdx.x & 7;
    float s = 0.f;
    long long row = 0;
    const bool live = idx < rows;
    if (live) {
        const long long pair = idx / q_rows;
        row = pair * N + q_begin + (idx - pair * q_rows);
        const uint4 a = reinterpret_cast<const uint4 *>(o + row * GA_D)[part];
        const uint4 b = reinterpret_cast<const uint4 *>(d_out + row * GA_D)[part];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {  // a bf16 is the upper half of an fp32
            s = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), s);
            s = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), s);
        }
        float4 *z4 = reinterpret_cast<float4 *>(dq + row * GA_D) + part * 2;
        z4[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        z4[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (live && part == 0) dsum[row] = s;
}

__device__ __forceinline__ void red_add_v4(float *dst, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// A warp holds 32 rows x 16 fp32 (one row and 64 B per lane) bound for global rows 256 B apart.  Written lane by lane,
// every store or reduction instruction would touch 32 sectors and fill half of each.  The block goes through 2 KiB of
// shared memory instead (16-byte pieces swizzled by (row >> 1) & 3: conflict-free both ways) and leaves with four lanes
// on the 64 B of one row: 8 rows, 16 whole sectors an instruction.  `dst`: row 0 of the block at the warp's column
// offset; rows >= rows_valid are not written.
template <bool REDUCE>
__device__ __forceinline__ void ga_warp_rows_out(float *stage, const uint32_t (&v)[16], int lane, float *dst, int rows_valid) {
#pragma unroll
    for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4 *>(stage + lane * 16 + ((c ^ ((lane >> 1) & 3)) << 2)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = (lane >> 2) + 8 * i, piece = lane & 3;
        const float4 x = *reinterpret_cast<const float4 *>(stage + row * 16 + ((piece ^ ((row >> 1) & 3)) << 2));
        if (row < rows_valid) {
            float *g = dst + (size_t)row * GA_D + piece * 4;
            if (REDUCE) red_add_v4(g, x.x, x.y, x.z, x.w);
            else *reinterpret_cast<float4 *>(g) = x;
        }
    }
    __syncwarp();  // the staging block may be rewritten
}

struct GaBwdKey {  // per-thread constants of the thread's key (centred coordinates k)
    f2_t ax2, ay2, az2;  // -2 c_rbf k
    f2_t ckn2;           // c_rbf |k|^2
    bool k_ok;
};

// Stages one query of a query tile: centred coordinates, log-sum-exp, D, validity and, with the other 15 queries of its
// half-warp, the bounding sphere of the group of 16.  Executed by whole warps with query = lane + 32 m.
__device__ __forceinline__ void ga_stage_row(GaQueryRows &rw, int i, bool ok, float x, float y, float z, float l2, float dsum) {
    float *qa = reinterpret_cast<float *>(&rw.qa[i >> 1]), *qc = reinterpret_cast<float *>(&rw.qc[i >> 1]);
    float *ld = reinterpret_cast<float *>(&rw.ld[i >> 1]);
    qa[i & 1] = x;
    qa[2 + (i & 1)] = y;
    qc[i & 1] = z;
    qc[2 + (i & 1)] = x * x + y * y + z * z;
    ld[i & 1] = -l2;  // (the exponent of P is SR - L: stored with its sign, one instruction less per pair)
    ld[2 + (i & 1)] = dsum;
    const uint32_t bits = __ballot_sync(0xffffffffu, ok);
    if ((i & 31) == 0) rw.qbits[i >> 5] = bits;
    float n = ok ? 1.f : 0.f, sx = x, sy = y, sz = z;  // padded queries carry 0
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) {
        n += __shfl_xor_sync(0xffffffffu, n, off);
        sx += __shfl_xor_sync(0xffffffffu, sx, off);
        sy += __shfl_xor_sync(0xffffffffu, sy, off);
        sz += __shfl_xor_sync(0xffffffffu, sz, off);
    }
    const float inv = n > 0.f ? 1.f / n : 0.f;
    const float cx = sx * inv, cy = sy * inv, cz = sz * inv;
    float d2 = ok ? (x - cx) * (x - cx) + (y - cy) * (y - cy) + (z - cz) * (z - cz) : 0.f;
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) d2 = fmaxf(d2, __shfl_xor_sync(0xffffffffu, d2, off));
    if ((i & 15) == 0) rw.sph[i >> 4] = make_float4(cx, cy, cz, n > 0.f ? sqrtf(d2) * 1.0001f + 1e-4f : -1.f);
}

// The 16 query columns (8 pairs) of one key row that a thread owns in a sub-tile: recompute P, form dS and the
// spread-gradient term.  sv / dpv hold the raw S^T and dP^T values; the queries' coordinates come from shared memory
// (every lane reads the same entry) and c_rbf |r_k - r_q|^2 = c_rbf |q|^2 - 2 c_rbf k.q + c_rbf |k|^2 takes four packed FMAs a pair;
// the results come back as bf16 pairs in pw / dw.  `p0` is the index of the first of the 8 query pairs inside the
// tile's row arrays.
// `masked` (warp-uniform): the key tile or the query tile holds a padded token; `qbits`: validity of the 16 queries.
// S^T and dP^T of a padded pair are then replaced by 0 and its P by 0, so whatever the padding holds, Inf or NaN
// included, never reaches a result.  `far` (warp-uniform): the 16 queries are too far from the warp's keys for R to
// count; R = 0 then goes through the same arithmetic.  One body serves every case, and every pair goes through the
// whole chain in one pass so that few values are live at a time.
template <int FORM>
__device__ __forceinline__ void ga_bwd_chunk(uint32_t (&sv)[16], uint32_t (&dpv)[16], bool far, bool masked,
                                             uint32_t qbits, const GaQueryRows &rw, int p0, const GaBwdKey &key, f2_t crbf2, f2_t cs2,
                                             f2_t scale2, const GaForm &fm, f2_t &dsig2, f2_t &dbeta2, uint32_t (&pw)[8],
                                             uint32_t (&dw)[8]) {
    const f2_t one2 = f2_pack(1.f, 1.f);
    if (far && FORM == 1 && fm.far_masked) {  // every pair of the group is outside the RBF window: P = 0
#pragma unroll
        for (int e = 0; e < 8; ++e) pw[e] = dw[e] = 0u;
        return;
    }
    const uint32_t ok_bits = masked ? (key.k_ok ? qbits : 0u) : 0xffffu;
    if (masked) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const bool ok = (ok_bits >> i) & 1u;
            sv[i] = ok ? sv[i] : 0u;
            dpv[i] = ok ? dpv[i] : 0u;
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        f2_t arg = 0ull, rb = 0ull;
        if (!far) {  // c_rbf * d^2 and R
            const float4 qa = rw.qa[p0 + e], qc = rw.qc[p0 + e];
            f2_t t = f2_fma(key.ax2, f2_pack(qa.x, qa.y), key.ckn2);
            t = f2_fma(key.ay2, f2_pack(qa.z, qa.w), t);
            t = f2_fma(key.az2, f2_pack(qc.x, qc.y), t);
            float a0, a1;
            f2_unpack(f2_fma(crbf2, f2_pack(qc.z, qc.w), t), a0, a1);
            if (FORM == 1) {
                a0 = fminf(a0, 0.f);
                a1 = fminf(a1, 0.f);
            }
            arg = f2_pack(a0, a1);
            rb = f2_pack(ex2_approx(a0), ex2_approx(a1));
        }
        const f2_t s_raw = f2_pack(__uint_as_float(sv[2 * e]), __uint_as_float(sv[2 * e + 1]));
        const f2_t t2 = f2_mul(s_raw, cs2);
        const f2_t onep = f2_add(rb, one2);
        const float4 l = rw.ld[p0 + e];  // {L pair, D pair}
        f2_t x;
        if (FORM == 0) {
            x = f2_fma(t2, onep, f2_pack(l.x, l.y));
        } else {
            float t0, t1, r0, r1;
            f2_unpack(t2, t0, t1);
            f2_unpack(rb, r0, r1);  // 0 for a far group
            const float s0 = fmaf(fm.beta * fmaf(r0, fm.rn_a, fm.rn_b), fabsf(t0), t0);
            const float s1 = fmaf(fm.beta * fmaf(r1, fm.rn_a, fm.rn_b), fabsf(t1), t1);
            x = f2_add(f2_pack((r0 >= fm.rmin && r0 <= fm.rmax) ? s0 : -INFINITY, (r1 >= fm.rmin && r1 <= fm.rmax) ? s1 : -INFINITY),
                       f2_pack(l.x, l.y));
        }
        float p0v, p1v;
        {
            float a0, a1;
            f2_unpack(x, a0, a1);
            p0v = ex2_approx(a0);  // P
            p1v = ex2_approx(a1);
        }
        if (masked) {
            p0v = (ok_bits >> (2 * e)) & 1u ? p0v : 0.f;
            p1v = (ok_bits >> (2 * e + 1)) & 1u ? p1v : 0.f;
        }
        const f2_t pp = f2_pack(p0v, p1v);
        const f2_t dp = f2_pack(__uint_as_float(dpv[2 * e]), __uint_as_float(dpv[2 * e + 1]));
        const f2_t dsr = f2_mul(pp, f2_sub(dp, f2_pack(l.z, l.w)));  // P = 0 (padding, outside the window): dSR = 0
        f2_t ds;
        if (FORM == 0) {
            ds = f2_mul(f2_mul(dsr, scale2), onep);
            dsig2 = f2_fma(f2_mul(f2_mul(dsr, s_raw), rb), arg, dsig2);
        } else {  // dS = dSR (1 + beta Rn sign(S)),  dR = dSR |S| 2 beta / (max - min),  dbeta = sum dSR Rn |S|
            float s0, s1, r0, r1, g0, g1, a0, a1;
            f2_unpack(s_raw, s0, s1);
            f2_unpack(dsr, g0, g1);
            f2_unpack(rb, r0, r1);
            f2_unpack(arg, a0, a1);
            const float rn0 = fmaf(r0, fm.rn_a, fm.rn_b), rn1 = fmaf(r1, fm.rn_a, fm.rn_b);
            const float sg0 = (s0 > 0.f) ? 1.f : ((s0 < 0.f) ? -1.f : 0.f), sg1 = (s1 > 0.f) ? 1.f : ((s1 < 0.f) ? -1.f : 0.f);
            float sc0, sc1;
            f2_unpack(scale2, sc0, sc1);
            const float f0 = s0 != 0.f ? fmaf(fm.beta * rn0, sg0, 1.f) : 0.f, f1 = s1 != 0.f ? fmaf(fm.beta * rn1, sg1, 1.f) : 0.f;
            ds = f2_pack(g0 * sc0 * f0, g1 * sc1 * f1);
            dsig2 = f2_fma(f2_pack(g0 * fabsf(s0) * r0, g1 * fabsf(s1) * r1), f2_pack(a0, a1), dsig2);  // r = 0 for a far group
            dbeta2 = f2_add(dbeta2, f2_pack(g0 * rn0 * fabsf(s0), g1 * rn1 * fabsf(s1)));
        }
        float d0, d1;
        f2_unpack(ds, d0, d1);
        pw[e] = pack_bf16x2(p0v, p1v);
        dw[e] = pack_bf16x2(d0, d1);
    }
}

// One work item: the key tile `k_tile` of the (batch, head) pair `zh_local` of the launch.  Every thread of the CTA calls
// it; tensor memory is allocated by the caller.  `fresh`: the CTA has not initialised its barriers yet; a live item
// clears it, later ones invalidate the barriers before they initialise them again.
template <int FORM>
__device__ __forceinline__ void geoattn_bwd_item(GaBwdSmem &sm, const CUtensorMap &map_q, const CUtensorMap &map_k, const CUtensorMap &map_v,
                                                 const CUtensorMap &map_do, const GaBwdParams &p, int zh_local, int k_tile, bool &fresh) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_math = warp < GA_BWD_MATH_THREADS / 32;
    const bool is_producer = warp == GA_BWD_MATH_THREADS / 32, is_stager = warp == GA_BWD_MATH_THREADS / 32 + 1;
    const bool is_grad_issuer = warp == GA_BWD_MATH_THREADS / 32 + 2;
    const int grp = (warp >> 2) & 3;              // which 16 query columns of a sub-tile / which 16 output columns
    const int r = (warp & 3) * 32 + lane;         // key row inside the tile = TMEM lane
    const int N = p.N;
    const int tiles_all = (N + GA_BM - 1) / GA_BM;
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int j0 = k_tile * GA_BN;
    const float *cz = p.coords + (size_t)z * N * 3;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;

    // ---- this CTA's keys, the live query tiles of the range ------------------------------------------
    const int jrow = j0 + r;  // the key whose dK / dV row this thread writes (16 of its 64 columns)
    const bool k_ok = is_math && jrow < N && (vz ? vz[jrow] != 0 : true);
    const int k_info = p.plan ? ga_plan_info(p.plan, p.Z, N, z)[j0 / GA_BN] : ga_plan_info_unmasked(N, j0 / GA_BN);
    const int *tl = p.plan ? ga_plan_tiles(p.plan, p.Z, N, z) : nullptr;
    const int nt_all = p.plan ? ga_plan_count(p.plan, p.Z)[z] : tiles_all;
    auto word_g = [&](int t) -> int { return tl ? tl[t] : (ga_plan_info_unmasked(N, t) | t); };
    // the list is ascending: the tiles of [qt_begin, qt_end) are a contiguous run of it
    int first = 0, nt = nt_all;
    if (p.qt_begin > 0 || p.qt_end < tiles_all) {  // (a chain of dependent global loads: only when the range is a part)
        nt = 0;
        while (first < nt_all && (word_g(first) & 0x7fff) < p.qt_begin) ++first;
        while (first + nt < nt_all && (word_g(first + nt) & 0x7fff) < p.qt_end) ++nt;
    }
    float *dk_row = p.dk + ((size_t)zh * N + jrow) * GA_D + grp * 16;
    float *dv_row = p.dv + ((size_t)zh * N + jrow) * GA_D + grp * 16;
    if (k_info < 0 || nt == 0) {  // no valid key here, or no query to hear from: zeros
        if (is_math && jrow < N) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                reinterpret_cast<float4 *>(dk_row)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                reinterpret_cast<float4 *>(dv_row)[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        return;
    }
    for (int t = tid; t < nt; t += GA_BWD_THREADS) sm.tiles[t] = (uint16_t)word_g(first + t);
    auto tile_word = [&](int t) -> int { return (int)sm.tiles[t]; };  // (published by the barrier below)
    const bool key_hole = (k_info & 0x8000) != 0;
    // origin of the centred coordinates: the first valid key of this tile
    const int ok_row = j0 + (k_info & 0x7f);
    const float orx = cz[ok_row * 3], ory = cz[ok_row * 3 + 1], orz = cz[ok_row * 3 + 2];
    volatile int *abort_flag = &sm.abort;
    const int nsub = 2 * nt;  // sub-tiles of 64 queries: u = 2 t + s

    // ---- set-up ------------------------------------------------------------------------------------
    if (is_producer) {
        if (lane == 0) {
            if (!fresh) {
                mbar_inval(&sm.bar_kv);
                mbar_inval(&sm.bar_pds);
                mbar_inval(&sm.bar_vk);
                mbar_inval(&sm.bar_dq);
                mbar_inval(&sm.bar_dqr);
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    mbar_inval(&sm.bar_qdo[b]);
                    mbar_inval(&sm.bar_sp[b]);
                    mbar_inval(&sm.bar_spfree[b]);
                }
#pragma unroll
                for (int b = 0; b < GA_ROW_BUFS; ++b) {
                    mbar_inval(&sm.bar_rows[b]);
                    mbar_inval(&sm.bar_rowsfree[b]);
                }
            }
            mbar_init(&sm.bar_kv, 1);
            mbar_init(&sm.bar_qdo[0], 1);
            mbar_init(&sm.bar_qdo[1], 1);
            mbar_init(&sm.bar_sp[0], 1);
            mbar_init(&sm.bar_sp[1], 1);
            mbar_init(&sm.bar_vk, 1);
            mbar_init(&sm.bar_dq, 1);
            mbar_init(&sm.bar_spfree[0], GA_BWD_MATH_THREADS);
            mbar_init(&sm.bar_spfree[1], GA_BWD_MATH_THREADS);
            mbar_init(&sm.bar_pds, GA_BWD_MATH_THREADS);
            mbar_init(&sm.bar_dqr, GA_BWD_MATH_THREADS);
#pragma unroll
            for (int b = 0; b < GA_ROW_BUFS; ++b) {
                mbar_init(&sm.bar_rows[b], 32);
                mbar_init(&sm.bar_rowsfree[b], GA_BWD_MATH_THREADS);
            }
            mbar_fence_init();
            fence_proxy_async();
            // the first loads leave before anything else is set up
            mbar_expect_tx(&sm.bar_kv, 2 * GA_TILE_BYTES);
            tma_load_3d(sm.k, &map_k, 0, j0, zh_local, &sm.bar_kv);
            tma_load_3d(sm.v, &map_v, 0, j0, zh_local, &sm.bar_kv);
            for (int t = 0; t < 2 && t < nt; ++t) {
                const int i0 = (word_g(first + t) & 0x7fff) * GA_BM;
                mbar_expect_tx(&sm.bar_qdo[t], 2 * GA_TILE_BYTES);
                tma_load_3d(sm.q[t], &map_q, 0, i0, zh_local, &sm.bar_qdo[t]);
                tma_load_3d(sm.dout[t], &map_do, 0, i0, zh_local, &sm.bar_qdo[t]);
            }
        }
        __syncwarp();
    }
    // Per-query inputs of four queries per stager lane (queries lane + 32 m of a tile): the loads are issued at once
    // from clamped indices, none waits for the validity bytes.
    struct RowLoad {
        float gx[4], gy[4], gz[4], lse[4], ds[4];
        uint8_t vb[4];
    };
    auto row_load = [&](int tile, RowLoad &q) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int ic = min(tile * GA_BM + lane + 32 * m, N - 1);
            q.vb[m] = vz ? vz[ic] : (uint8_t)1;
            q.gx[m] = cz[ic * 3];
            q.gy[m] = cz[ic * 3 + 1];
            q.gz[m] = cz[ic * 3 + 2];
            q.lse[m] = p.lse[(size_t)zh * N + ic];
            q.ds[m] = p.dsum[(size_t)zh_local * N + ic];
        }
    };
    auto row_stage = [&](int tile, int buf, const RowLoad &q) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int i = tile * GA_BM + lane + 32 * m;
            const bool ok = i < N && q.vb[m] != 0;
            // +inf: P = 0 for a padded query and for a row without any valid pair
            const float l2 = (ok && q.lse[m] != -INFINITY) ? q.lse[m] * 1.4426950408889634f : INFINITY;
            ga_stage_row(sm.rows[buf], lane + 32 * m, ok, ok ? q.gx[m] - orx : 0.f, ok ? q.gy[m] - ory : 0.f, ok ? q.gz[m] - orz : 0.f, l2,
                         ok ? q.ds[m] : 0.f);
        }
    };
    // this thread's key, centred
    float kcx = 0.f, kcy = 0.f, kcz = 0.f;
    if (k_ok) {
        kcx = cz[jrow * 3] - orx;
        kcy = cz[jrow * 3 + 1] - ory;
        kcz = cz[jrow * 3 + 2] - orz;
    }
    RowLoad rl;
    if (is_stager) row_load(word_g(first) & 0x7fff, rl);  // in flight across the barrier
    tc_fence_before();
    __syncthreads();  // barriers initialised, TMEM allocated, tile list in place
    fresh = false;
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    // two stages of S^T [0,64) [64,128) and dP^T [128,192) [192,256) (sub-tile u uses stage u & 1), P^T [256,288), dV [320,384),
    // dK [384,448), dQ [448,512)
    const uint32_t tm_s = tmem, tm_dp = tmem + 128, tm_p = tmem + 256, tm_dv = tmem + 320, tm_dk = tmem + 384, tm_dq = tmem + 448;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    if (is_stager) {
        // ================================ stager warp ================================================
        // Runs up to GA_ROW_BUFS query tiles ahead of the math warps.
        for (int t = 0; t < nt; ++t) {
            const int b = t % GA_ROW_BUFS;
            if (t > 0) row_load(tile_word(t) & 0x7fff, rl);
            // buffer b was last used by tile t - GA_ROW_BUFS: every math thread has left it
            if (t >= GA_ROW_BUFS && !__all_sync(0xffffffffu, mbar_wait_abortable(&sm.bar_rowsfree[b], (uint32_t)((t / GA_ROW_BUFS - 1) & 1), abort_flag) ? 1 : 0))
                break;  // (decided by the whole warp: the staging below shuffles across all 32 lanes)
            row_stage(tile_word(t) & 0x7fff, b, rl);
            mbar_arrive(&sm.bar_rows[b]);
        }
    } else if (is_producer || is_grad_issuer) {
        // ================================ issuer warps ===============================================
        // Two threads issue the MMAs: an MMA instruction holds its issuing thread until the tensor core has taken it
        // (about 55 cycles each in a stream, 400 to 500 cycles until the first of a batch completes), so one thread
        // issuing all 22 MMAs of a sub-tile in turn, with its waits in between, was busy for longer than the math warps
        // need for the sub-tile.  The first thread issues S^T, dP^T, G^T of the next sub-tile, the second dV, dK, dQ of
        // this one and the TMA loads of Q / dO.
        if (lane == 0) {
            const uint32_t k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v);
            constexpr uint32_t IDESC_SP = umma_idesc_bf16(128, GA_SUB, false, false);  // S^T, dP^T, G^T of a sub-tile: [128 x 64]
            constexpr uint32_t IDESC_KN = umma_idesc_bf16(128, GA_D, false, true);     // dV (A in TMEM), dK: A K-major, B MN-major
            constexpr uint32_t IDESC_NN = umma_idesc_bf16(128, GA_D, true, true);      // dQ: A MN-major, B MN-major
            // descriptors are built once; a step of K = 16 adds to the 16-byte-granular address field
            const uint64_t k_km = umma_desc_sw128(k_addr, 16, 1024), v_km = umma_desc_sw128(v_addr, 16, 1024);  // K-major operands
            const uint64_t k_mn = umma_desc_sw128(k_addr, 0, 1024);                                              // B of dQ
            constexpr uint64_t BUF = (uint64_t)GA_TILE_BYTES >> 4;  // the second buffer of a pair follows the first
            const uint64_t q_km = umma_desc_sw128(smem_u32(sm.q[0]), 16, 1024), do_km = umma_desc_sw128(smem_u32(sm.dout[0]), 16, 1024);
            const uint64_t q_mn = umma_desc_sw128(smem_u32(sm.q[0]), 0, 1024), do_mn = umma_desc_sw128(smem_u32(sm.dout[0]), 0, 1024);
            const uint64_t ds_km = umma_desc_sw128(smem_u32(sm.ds[0]), 16, 1024), ds_mn = umma_desc_sw128(smem_u32(sm.ds[0]), GA_TILE_BYTES, 1024);
            constexpr uint64_t SUB_ROWS = (uint64_t)(GA_SUB * 128) >> 4;  // 64 rows of a swizzled tile, in 16-byte units
            if (is_producer) {
                // Sub-tile u = 2 t + s (queries 64 s .. 64 s + 63 of tile t): S^T = K Q^T and dP^T = V dO^T, 4 + 4 MMAs of K = 16
                // over d = 64, into stage s.  B operands start 64 rows into their tiles for s = 1.
                auto issue_sdp = [&](int u) {
                    const int t = u >> 1, sub = u & 1, b = t & 1;
                    const uint64_t qd = q_km + b * BUF + sub * SUB_ROWS, dd = do_km + b * BUF + sub * SUB_ROWS;
#pragma unroll
                    for (int kk = 0; kk < GA_D / 16; ++kk)
                        umma_ss(tm_s + sub * GA_SUB, k_km + (uint64_t)(kk * 2), qd + (uint64_t)(kk * 2), IDESC_SP, kk > 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < GA_D / 16; ++kk)
                        umma_ss(tm_dp + sub * GA_SUB, v_km + (uint64_t)(kk * 2), dd + (uint64_t)(kk * 2), IDESC_SP, kk > 0 ? 1u : 0u);
                    umma_commit(&sm.bar_sp[sub]);
                };
                bool ok = mbar_wait_abortable(&sm.bar_kv, 0, abort_flag);
                for (int u = 0; ok && u < nsub; ++u) {
                    const int t = u >> 1, sub = u & 1, b = t & 1;
                    // stage `sub` was last used by sub-tile u - 2: every math thread holds its S^T, dP^T in registers
                    if (u >= 2 && !(ok = mbar_wait_abortable(&sm.bar_spfree[sub], (uint32_t)((t - 1) & 1), abort_flag))) break;
                    if (sub == 0 && !(ok = mbar_wait_abortable(&sm.bar_qdo[b], (uint32_t)((t >> 1) & 1), abort_flag))) break;
                    tc_fence_after();
                    issue_sdp(u);
                }
            } else {
                auto load_qdo = [&](int t) {
                    const int b = t & 1;
                    const int i0 = (tile_word(t) & 0x7fff) * GA_BM;
                    mbar_expect_tx(&sm.bar_qdo[b], 2 * GA_TILE_BYTES);
                    tma_load_3d(sm.q[b], &map_q, 0, i0, zh_local, &sm.bar_qdo[b]);
                    tma_load_3d(sm.dout[b], &map_do, 0, i0, zh_local, &sm.bar_qdo[b]);
                };
                auto issue_dv_dk = [&](int u) {  // K = 16 queries per step, 4 steps per sub-tile
                    const int t = u >> 1, sub = u & 1, b = t & 1;
#pragma unroll
                    for (int kk = 0; kk < GA_SUB / 16; ++kk)  // dV += P^T dO: P^T advances 8 TMEM columns, dO 2 KiB (16 rows)
                        umma_ts(tm_dv, tm_p + kk * 8, do_mn + b * BUF + sub * SUB_ROWS + (uint64_t)(kk * 128), IDESC_KN, (u == 0 && kk == 0) ? 0u : 1u);
#pragma unroll
                    for (int kk = 0; kk < GA_SUB / 16; ++kk)  // dK += dS^T Q: the sub-tile of dS^T, 32 B per step inside the swizzled row
                        umma_ss(tm_dk, ds_km + b * 2 * BUF + (uint64_t)(sub * (GA_TILE_BYTES >> 4) + kk * 2),
                                q_mn + b * BUF + sub * SUB_ROWS + (uint64_t)(kk * 128), IDESC_KN, (u == 0 && kk == 0) ? 0u : 1u);
                    umma_commit(&sm.bar_vk);
                };
                auto issue_dq = [&](int b) {  // dQ = dS K: K = 16 keys per step, 2 KiB down the dS^T tile (M = queries: two sub-tiles)
#pragma unroll
                    for (int kk = 0; kk < GA_BN / 16; ++kk)
                        umma_ss(tm_dq, ds_mn + b * 2 * BUF + (uint64_t)(kk * 128), k_mn + (uint64_t)(kk * 128), IDESC_NN, kk > 0 ? 1u : 0u);
                    umma_commit(&sm.bar_dq);
                };
                bool ok = mbar_wait_abortable(&sm.bar_kv, 0, abort_flag);
                for (int u = 0; ok && u < nsub; ++u) {
                    const int t = u >> 1, sub = u & 1, b = t & 1;
                    const uint32_t par = (uint32_t)(u & 1);
                    if (!(ok = mbar_wait_abortable(&sm.bar_pds, par, abort_flag))) break;  // P^T(u) in TMEM, dS^T(u) in shared memory
                    if (sub == 0 && !(ok = mbar_wait_abortable(&sm.bar_qdo[b], (uint32_t)((t >> 1) & 1), abort_flag))) break;  // (long landed)
                    tc_fence_after();
                    issue_dv_dk(u);
                    if (sub == 1) {
                        if (t > 0 && !(ok = mbar_wait_abortable(&sm.bar_dqr, (uint32_t)((t - 1) & 1), abort_flag))) break;  // dQ(t-1) read out
                        tc_fence_after();
                        issue_dq(b);
                        if (t + 2 < nt) {  // Q / dO buffer b is free once the sub-tile MMAs of tile t are done
                            if (!(ok = mbar_wait_abortable(&sm.bar_vk, par, abort_flag))) break;
                            load_qdo(t + 2);
                        }
                    }
                }
                if (!ok || *abort_flag) {  // gave up: let the copies already issued land before the CTA exits (bounded)
                    mbar_wait_bounded(&sm.bar_kv, 0, 1u << 12);
                    mbar_wait_bounded(&sm.bar_qdo[0], 0, 1u << 12);
                    mbar_wait_bounded(&sm.bar_qdo[1], 0, 1u << 12);
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
        GaForm fm;
        ga_form_setup(fm, FORM, FORM == 1 ? p.beta[h] : 0.f, p.min_rbf, p.max_rbf);
        GaBwdKey key;
        const float ckn = c_rbf * (kcx * kcx + kcy * kcy + kcz * kcz);
        key.ckn2 = f2_pack(ckn, ckn);
        key.ax2 = f2_pack(-2.f * c_rbf * kcx, -2.f * c_rbf * kcx);
        key.ay2 = f2_pack(-2.f * c_rbf * kcy, -2.f * c_rbf * kcy);
        key.az2 = f2_pack(-2.f * c_rbf * kcz, -2.f * c_rbf * kcz);
        key.k_ok = k_ok;
        // bounding sphere of the warp's valid keys; wk_reach = (distance beyond which R does not count) + radius
        float wkx, wky, wkz, wk_reach;
        {
            float n = k_ok ? 1.f : 0.f, sx = kcx, sy = kcy, sz = kcz;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                n += __shfl_xor_sync(0xffffffffu, n, off);
                sx += __shfl_xor_sync(0xffffffffu, sx, off);
                sy += __shfl_xor_sync(0xffffffffu, sy, off);
                sz += __shfl_xor_sync(0xffffffffu, sz, off);
            }
            const float inv = n > 0.f ? 1.f / n : 0.f;
            wkx = sx * inv;
            wky = sy * inv;
            wkz = sz * inv;
            float d2 = k_ok ? (kcx - wkx) * (kcx - wkx) + (kcy - wky) * (kcy - wky) + (kcz - wkz) * (kcz - wkz) : 0.f;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) d2 = fmaxf(d2, __shfl_xor_sync(0xffffffffu, d2, off));
            wk_reach = fm.far_cut * sig + sqrtf(d2) * 1.0001f + 1e-4f;
            if (!p.far_skip || !(fm.far_cut < INFINITY)) wk_reach = -INFINITY;  // test off
        }
        // `ok` is kept uniform across the warp: tcgen05.ld / st need all 32 lanes
        bool ok = true;
        auto wait_w = [&](uint64_t *bar, uint32_t parity) -> bool {
            return __all_sync(0xffffffffu, mbar_wait_abortable(bar, parity, abort_flag) ? 1 : 0) != 0;
        };
        auto read_dq = [&](int t) {  // dQ tile of query tile t: TMEM -> registers -> vector reductions into the global fp32 dQ
            uint32_t v[16];
            tmem_ld16(tm_dq + lane_base + grp * 16, v);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&sm.bar_dqr);
            const int row0 = (tile_word(t) & 0x7fff) * GA_BM + (warp & 3) * 32;  // first query row of this warp's block
            ga_warp_rows_out<true>(sm.stage[warp], v, lane, p.dq + ((size_t)zh * N + row0) * GA_D + grp * 16, N - row0);
        };

#pragma unroll 1
        for (int u = 0; ok && u < nsub; ++u) {
            const int t = u >> 1, sub = u & 1, rbuf = t % GA_ROW_BUFS;
            const uint32_t par = (uint32_t)(u & 1);
            const bool masked = key_hole || (tile_word(t) & 0x8000) != 0;
            const GaQueryRows &rw = sm.rows[rbuf];
            uint8_t *ds_tile = sm.ds[t & 1];
            if (sub == 0 && !(ok = wait_w(&sm.bar_rows[rbuf], (uint32_t)((t / GA_ROW_BUFS) & 1)))) break;  // the tile's staged rows
            if (!(ok = wait_w(&sm.bar_sp[sub], (uint32_t)(t & 1)))) break;  // S^T, dP^T(u) have landed in TMEM
            tc_fence_after();
            const int col0 = sub * GA_SUB + grp * 16;  // first query column (inside the tile) of this thread's 16
            uint32_t sv[16], dpv[16];
            tmem_ld16(tm_s + sub * GA_SUB + lane_base + grp * 16, sv);  // (in flight under the far test)
            tmem_ld16(tm_dp + sub * GA_SUB + lane_base + grp * 16, dpv);
            bool far;
            {  // the thread's group of 16 queries against this warp's keys
                const float4 sp = rw.sph[col0 / 16];
                const float dx = sp.x - wkx, dy = sp.y - wky, dz = sp.z - wkz;
                const float reach = wk_reach + sp.w;
                far = sp.w < 0.f || (dx * dx + dy * dy + dz * dz > reach * reach && reach > 0.f);
            }
            const uint32_t qbits = (rw.qbits[col0 / 32] >> (col0 & 16)) & 0xffffu;
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&sm.bar_spfree[sub]);  // the stage may be overwritten with sub-tile u + 2
            uint32_t pw[8], dw[8];
            ga_bwd_chunk<FORM>(sv, dpv, far, masked, qbits, rw, col0 / 2, key, crbf2, cs2, scale2, fm, dsig2, dbeta2, pw, dw);
            // P^T(u-1) is read by dV(u-1): no store before it has completed (the dS^T buffer of this tile was last read
            // by dK / dQ two query tiles ago)
            if (u > 0 && !(ok = wait_w(&sm.bar_vk, par ^ 1))) break;
            tmem_st8(tm_p + lane_base + grp * 8, pw);
#pragma unroll
            for (int c = 0; c < 2; ++c)  // 8 queries = one 16-byte chunk of the swizzled key row, sub-tile `sub`
                *reinterpret_cast<uint4 *>(ds_tile + sub * GA_TILE_BYTES + sw128_offset(r, grp * 2 + c)) =
                    make_uint4(dw[4 * c], dw[4 * c + 1], dw[4 * c + 2], dw[4 * c + 3]);
            tmem_wait_st();
            fence_proxy_async();  // dS^T (generic-proxy stores) must be visible to the tensor core
            tc_fence_before();
            mbar_arrive(&sm.bar_pds);
            if (sub == 1) {
                mbar_arrive(&sm.bar_rowsfree[rbuf]);  // the stager may reuse this tile's row buffer
                if (t > 0) {  // dQ(t-1) completed long ago: read it out now, off the tensor core's critical path
                    if (!(ok = wait_w(&sm.bar_dq, (uint32_t)((t - 1) & 1)))) break;
                    tc_fence_after();
                    read_dq(t - 1);
                }
            }
        }

        // ---- epilogue: dV, dK rows of this key tile (their last accumulation was issued before the last dQ MMAs, which run
        // underneath these stores); the last dQ tile; dsigma ---------------------------------------------------------
        if (ok) ok = wait_w(&sm.bar_vk, (uint32_t)((nsub - 1) & 1));  // the last dV / dK accumulation has completed
        if (ok) {
            tc_fence_after();
            uint32_t a[16], b[16];
            tmem_ld16(tm_dv + lane_base + grp * 16, a);
            tmem_ld16(tm_dk + lane_base + grp * 16, b);
            tmem_wait_ld();
            // (a padded key row holds exact zeros: its P and dS were selected to 0)
            const int row0 = j0 + (warp & 3) * 32;
            const size_t off = ((size_t)zh * N + row0) * GA_D + grp * 16;
            ga_warp_rows_out<false>(sm.stage[warp], a, lane, p.dv + off, N - row0);
            ga_warp_rows_out<false>(sm.stage[warp], b, lane, p.dk + off, N - row0);
            ok = wait_w(&sm.bar_dq, (uint32_t)((nt - 1) & 1));
        }
        if (ok) {
            tc_fence_after();
            read_dq(nt - 1);
        }
        float d0, d1, b0, b1;
        f2_unpack(dsig2, d0, d1);
        f2_unpack(dbeta2, b0, b1);
        float dsig_acc = ok ? d0 + d1 : 0.f, dbeta_acc = ok ? b0 + b1 : 0.f;
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
    if (tid == 0 && !sm.abort) {
        float tot = 0.f, totb = 0.f;
        for (int w = 0; w < GA_BWD_MATH_THREADS / 32; ++w) {
            tot += sm.dsig[w];
            totb += sm.dbeta[w];
        }
        const float sig = p.sigma[h];
        const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);
        if (FORM == 0) {
            // sum of dSR * S_raw * R * (c_rbf d^2), S = scale * S_raw:  dsigma = sum dSR S R d^2 / sigma^3
            atomicAdd(p.dsigma + h, tot * p.scale / (c_rbf * sig * sig * sig));
        } else {
            // sum of dSR * |S_raw| * R * (c_rbf d^2):  dsigma = sum dR R d^2 / sigma^3 with dR = dSR |S| 2 beta / (max - min)
            atomicAdd(p.dsigma + h, tot * p.scale * 2.f * p.beta[h] / ((p.max_rbf - p.min_rbf) * c_rbf * sig * sig * sig));
            if (p.dbeta) atomicAdd(p.dbeta + h, totb * p.scale);
        }
    }
}

// Grid without a schedule: one CTA per (key tile, (batch, head) pair), the samples longest first when the plan's order
// applies.  With a schedule (geoattn_plan.cuh): `bins` persistent CTAs, each working through the items assigned to it and
// writing the zeros of its share of the key tiles without a valid key.
template <int FORM>
__global__ void __launch_bounds__(GA_BWD_THREADS, 1)
geoattn_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const GaBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaBwdSmem &sm = *reinterpret_cast<GaBwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    if (warp == GA_BWD_MATH_THREADS / 32) {
        if (threadIdx.x == GA_BWD_MATH_THREADS) sm.abort = 0;
        __syncwarp();
        tmem_alloc(&sm.tmem_base, GA_BWD_TMEM_COLS);
        tmem_relinquish();
    }
    // one loop (and one copy of the item's code) for both kinds of launch
    // (little state is kept across an item: the lists are looked up again for every item)
    int total = 1;
    if (p.sched != nullptr) {
        const int bins = p.sched[0];
        if (bins != (int)gridDim.x || p.sched[1] != p.H || p.sched[2] != p.Z || p.sched[3] != p.N) {
            // not the schedule of this problem: do nothing and say so (pai_device_status)
            if (threadIdx.x == 0 && blockIdx.x == 0) atomicExch(&g_device_status, (int)PAI_ERR_BAD_SHAPE);
            total = 0;
        } else {
            total = (p.sched[5] - (int)blockIdx.x + bins - 1) / bins + ga_sched_count(p.sched)[blockIdx.x];
        }
    }
    bool fresh = true;  // the barriers have not been initialised yet
#pragma unroll 1
    for (int k = 0; k < total; ++k) {
        int zh_local, tile;
        if (p.sched == nullptr) {
            zh_local = blockIdx.y;  // index into the shard of (batch, head) pairs
            tile = blockIdx.x;
            if (p.use_order) {      // samples longest first: the short ones fill the tail of the launch
                const int zp = zh_local / p.H;
                zh_local = ga_plan_order(p.plan)[zp] * p.H + (zh_local - zp * p.H);
            }
        } else {
            const int bins = p.sched[0];
            const int n_dead = (p.sched[5] - (int)blockIdx.x + bins - 1) / bins;  // this CTA's share of the tiles that only need zeros
            const int item = k < n_dead ? ga_sched_dead(p.sched)[blockIdx.x + k * bins] : ga_sched_items(p.sched, blockIdx.x)[k - n_dead];
            zh_local = item >> 10;
            tile = item & 1023;
        }
        geoattn_bwd_item<FORM>(sm, map_q, map_k, map_v, map_do, p, zh_local, tile, fresh);
        if (!fresh) {
            __syncthreads();  // (after a live item: thread 0 has read the item's partial sums; sm.abort is settled)
            if (sm.abort) break;
        }
    }
    // (a CTA that ran no live item has not synchronised since the allocation)
    tc_fence_before();
    __syncthreads();
    if (warp == GA_BWD_MATH_THREADS / 32) tmem_dealloc(sm.tmem_base, GA_BWD_TMEM_COLS);
}

}  // namespace pai
