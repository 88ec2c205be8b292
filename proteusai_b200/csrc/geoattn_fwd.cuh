// Geometric attention forward for sm_100a: flash attention on tcgen05 tensor cores with the
// per-head radial-basis scale applied in the softmax stage,
//     SR_ij = (q_i . k_j / sqrt(d)) * (1 + exp(-|r_i - r_j|^2 / (2 sigma_h^2))),
// a pair being valid iff query i and key j are both unpadded.  Replaces the Triton kernel
// `_attn_fwd` (old/old_scripts/attn/geometric_attn.py:57-260) with the logit form the reference's
// README states (README.md:40); the form the reference tree's kernel implements is the second
// instantiation (FORM = 1).
//
// One CTA = 128 query rows of one (batch, head): four math warps (one thread per query row = TMEM lane, so a row
// needs no exchange between threads), a producer warp (lane 0 issues every TMA load and MMA) and a stager warp.  Two
// CTAs share an SM: their phases drift apart, so the SFU-heavy and FMA-heavy stretches of one overlap the waits of
// the other, and a CTA's set-up hides behind its neighbour's work.  Keys are taken 64 at a time (a "step"; two steps
// per 128-key tile of the batch plan).
// Tensor memory (256 columns): S [0,64) fp32, G [64,128) fp32, O [128,192) fp32, P [192,224) bf16 pairs.
//   S  = Q K^T : tcgen05.mma, A = Q tile, B = K step (both K-major, 128-byte swizzle, via TMA);
//   G          : the geometry of the step comes from the tensor core as well: G_ij = |k_j|^2 - 2 q_i . k_j
//                (coordinates centred on the tile's first valid query) is a product of two narrow operand tiles
//                that the threads write themselves, each fp32 coordinate split into three bf16 terms
//                (ga_write_geo_row), so that |r_i - r_j|^2 = G_ij + |q_i|^2 to fp32 accuracy.  Reading key
//                coordinates from shared memory instead costs every warp a broadcast load per key pair, which
//                made the shared-memory pipe, not the SFU, the limiter of this stage;
//   softmax    : a math thread reads the 64 logits of its row ONCE into registers (tcgen05.ld), G group by group,
//                and releases the columns, so the tensor core computes the next step underneath the softmax of
//                this one.  R = 2^(c G + c |q|^2), SR = S scale (1 + R) in packed fp32x2 arithmetic.
//                A group of 16 keys whose bounding sphere lies farther than 5.9 sigma_h from the bounding sphere
//                of the warp's 32 queries has R < 2^-25 for every pair, where S (1 + R) == S in fp32: there
//                the exponential is skipped (most of the off-diagonal work of the narrow heads).  P is written
//                as bf16 straight into tensor memory;
//   O += P V   : tcgen05.mma with the A operand (P) read from tensor memory, B = V step (MN-major: keys
//                are the K dimension), accumulated in TMEM [128 x 64] across the steps.  The running
//                maximum is only raised when a step exceeds it by more than 2^8 (then the accumulator and
//                the row sum are rescaled); otherwise P is computed against the slightly stale maximum,
//                which is exact after the final normalisation.
// K and V are double-buffered.  The stager warp runs up to three key tiles ahead: geometry operand rows, masks and
// bounding spheres.  Key tiles without any valid key are never loaded (list from the batch plan, geoattn_plan.cuh);
// tiles without a padded key take a path without the mask; CTAs without any valid query only write zeros.  Every
// wait is bounded and abortable (tc.cuh).
#pragma once
#include "geoattn_plan.cuh"
#include "tc.cuh"

namespace pai {

constexpr int GA_BM = 128;  // query rows per CTA
constexpr int GA_BN = 128;  // tokens per tile of the batch plan (and per query / key tile of the backward)
constexpr int GA_BS = 64;   // keys per step of the forward
constexpr int GA_D = 64;    // head dimension
constexpr int GA_MAX_TILES = GA_PLAN_MAX_TILES;
constexpr int GA_FWD_MATH_THREADS = 128;
constexpr int GA_FWD_THREADS = GA_FWD_MATH_THREADS + 64;  // + the producer warp and the stager warp
constexpr float GA_RESCALE_THRESHOLD = 8.f;                 // log2 units
constexpr uint32_t GA_TMEM_COLS = 256;
constexpr uint32_t GA_TILE_BYTES = GA_BN * GA_D * 2;  // 16 KiB
constexpr uint32_t GA_STEP_BYTES = GA_BS * GA_D * 2;  // 8 KiB
constexpr int GA_KC_BUFS = 3;                           // staged key tiles in flight
constexpr float GA_FAR_SIGMAS = 5.9f;                   // exp(-d^2 / 2 sigma^2) < 2^-25 beyond 5.887 sigma

constexpr int GA_GEO_K = 32;                            // bf16 columns of the geometry operands (24 used)

struct GaKeyCoords {                  // per-key side data of one tile
    alignas(16) float kb[GA_BN];      // 0 for a valid key, -inf for a padded one
    float4 sph[GA_BN / 16];           // bounding sphere of each group of 16 keys: centre, radius (< 0: no valid key)
};

struct GaFwdSmem {
    alignas(1024) uint8_t q[GA_TILE_BYTES];
    alignas(1024) uint8_t k[2][GA_STEP_BYTES];
    alignas(1024) uint8_t v[2][GA_STEP_BYTES];
    // Geometry operands: rows of 128 B of which an operand uses 64 (GA_GEO_K bf16), so one buffer holds two of them side by
    // side (column blocks 0 and 1).  Slot 0: the queries; slots 1..3: the ring of staged key tiles.
    alignas(1024) uint8_t geo[2][GA_TILE_BYTES];
    GaKeyCoords kc[GA_KC_BUFS];
    uint64_t bar_q, bar_k[2], bar_v[2], bar_s, bar_sfree, bar_p, bar_o, bar_kc[GA_KC_BUFS], bar_kcfree[GA_KC_BUFS];
    uint16_t tiles[GA_MAX_TILES];                 // key tiles with a valid key; bit 15: the tile also has a padded key
    uint32_t tmem_base;
    int abort;                                    // raised by the first wait that expires
};

struct GaFwdParams {
    const float *coords;   // [Z,N,3]
    const uint8_t *valid;  // [Z,N] or nullptr
    const int *plan;       // batch plan (geoattn_plan.cuh); nullptr iff valid is nullptr
    const float *sigma;    // [H]
    __nv_bfloat16 *out;    // element (z,h,n,:) at out + z*so_z + h*so_h + n*so_n, 64 contiguous values
    long long so_z, so_h, so_n;
    float *lse;            // [Z,H,N]  log-sum-exp of SR (natural log), -inf for padded queries
    int Z, H, N, zh_begin;
    int q_begin;           // first query row of the launch (a multiple of 128); blockIdx.x counts tiles from it
    int use_order;         // issue the samples in the plan's longest-first order (full sample range only)
    int far_skip;          // skip the RBF arithmetic of far key groups
    float scale;
    // logit form: 0 = S (1 + R);  1 = S + beta Rn |S| with Rn = 2 (R - min_rbf) / (max_rbf - min_rbf) - 1 and pairs
    // with R outside [min_rbf, max_rbf] masked out (the form of old/old_scripts/attn/geometric_attn.py:193-201)
    int form;
    const float *beta;     // [H], form 1 only
    float min_rbf, max_rbf;
};

struct GaForm {  // per-head constants of logit form 1
    float beta, rn_a, rn_b, rmin, rmax;  // Rn = R * rn_a + rn_b
    float far_cut;                       // distance (in units of sigma) beyond which a key group needs no R
    int far_masked;                      // beyond it: 1 = every pair is outside the window (masked), 0 = R counts as 0
};

// Distance beyond which the RBF of a whole key group can be dropped, and what "dropped" means.
//   form 0: R < 2^-25, S (1 + R) == S.
//   form 1: min_rbf > 0: R < min_rbf, the pair is outside the window; min_rbf <= 0: R < 2^-25 counts as 0
//           (Rn changes by < 2^-24).  A positive min_rbf below 2^-25 switches the test off.
__device__ __forceinline__ void ga_form_setup(GaForm &fm, int form, float beta, float min_rbf, float max_rbf) {
    fm.beta = 0.f;
    fm.rn_a = fm.rn_b = 0.f;
    fm.rmin = 0.f;
    fm.rmax = 1.f;
    fm.far_cut = GA_FAR_SIGMAS;
    fm.far_masked = 0;
    if (form == 1) {
        fm.beta = beta;
        fm.rn_a = 2.f / (max_rbf - min_rbf);
        fm.rn_b = -2.f * min_rbf / (max_rbf - min_rbf) - 1.f;
        fm.rmin = min_rbf;
        fm.rmax = max_rbf;
        if (min_rbf > 0.f) {
            if (min_rbf > 3.0e-8f) {
                fm.far_cut = sqrtf(-2.f * logf(min_rbf)) * 1.002f + 1e-3f;
                fm.far_masked = 1;
            } else {
                fm.far_cut = INFINITY;
            }
        }
    }
}

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
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// fp32 -> three bf16 terms whose sum reproduces the value to about 2^-24 relative
__device__ __forceinline__ void ga_split3(float a, uint32_t &h, uint32_t &m, uint32_t &l) {
    const __nv_bfloat16 bh = __float2bfloat16_rn(a);
    const float r1 = a - __bfloat162float(bh);
    const __nv_bfloat16 bm = __float2bfloat16_rn(r1);
    const __nv_bfloat16 bl = __float2bfloat16_rn(r1 - __bfloat162float(bm));
    h = (uint32_t)__bfloat16_as_ushort(bh);
    m = (uint32_t)__bfloat16_as_ushort(bm);
    l = (uint32_t)__bfloat16_as_ushort(bl);
}

// One row (GA_GEO_K bf16 values) of a geometry operand tile, in the 128-byte-swizzled K-major layout the tensor core
// reads.  The product of a LEFT row (a, e) and a RIGHT row (b, n) is  a.b + e n  to fp32 accuracy: every fp32 factor
// is split into bf16 terms h + m + l and the six products of combined order <= 2 are laid out side by side,
//     LEFT  per coordinate: a_h a_h a_m a_h a_l a_m        then e_h e_h e_m e_h e_l e_m   (zeros after that)
//     RIGHT per coordinate: b_h b_m b_h b_l b_h b_m        then n_h n_m n_h n_l n_h n_m
// (dropped terms are below 2^-24 of |a||b|).  In the forward LEFT = (-2 q, 1), RIGHT = (k, |k|^2): G = |k|^2 - 2 q.k.
template <bool LEFT>
__device__ __forceinline__ void ga_write_geo_row(uint8_t *tile, int block, int row, float x, float y, float z, float e) {
    uint32_t w[16];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t h, m, l;
        ga_split3(c == 0 ? x : c == 1 ? y : c == 2 ? z : e, h, m, l);
        if (LEFT) {
            w[3 * c + 0] = h | (h << 16);
            w[3 * c + 1] = m | (h << 16);
            w[3 * c + 2] = l | (m << 16);
        } else {
            w[3 * c + 0] = h | (m << 16);
            w[3 * c + 1] = h | (l << 16);
            w[3 * c + 2] = h | (m << 16);
        }
    }
    w[12] = w[13] = w[14] = w[15] = 0u;
#pragma unroll
    for (int c = 0; c < 4; ++c)  // `block` selects the half of the 128-byte row (16-byte chunks 0..3 or 4..7)
        *reinterpret_cast<uint4 *>(tile + sw128_offset(row, 4 * block + c)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}
// geometry slot -> buffer and column block (two slots share a buffer)
template <typename Smem>
__device__ __forceinline__ uint8_t *ga_geo_tile(Smem &sm, int slot) { return sm.geo[slot >> 1]; }
__device__ __forceinline__ int ga_geo_block(int slot) { return slot & 1; }

// Stages one key of a key tile: its geometry operand row, its mask entry and, with the other 15 keys of its half-warp,
// the bounding sphere of the group of 16.  Executed by whole warps with key = (lane + 32 m): the 16 lanes of a half-warp
// hold 16 consecutive keys.  `x, y, z` are the centred coordinates (0 for a padded key).
__device__ __forceinline__ void ga_stage_key(GaKeyCoords &kc, uint8_t *geo_tile, int geo_block, int key, bool ok, float x, float y, float z) {
    ga_write_geo_row<false>(geo_tile, geo_block, key, x, y, z, x * x + y * y + z * z);
    kc.kb[key] = ok ? 0.f : -INFINITY;
    // bounding sphere of the 16 keys of this half-warp (valid keys only): centre = mean, radius = largest distance
    float n = ok ? 1.f : 0.f, sx = x, sy = y, sz = z;  // padded keys carry 0
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
    if ((key & 15) == 0) kc.sph[key >> 4] = make_float4(cx, cy, cz, n > 0.f ? sqrtf(d2) * 1.0001f + 1e-4f : -1.f);
}

// 16 logits (8 key pairs) of one row, held in registers: v[] holds raw S on entry and SR on return, g[] the matching
// G values; returns the maximum.  SR = (S * c_s) * (1 + R) with R = 2^(c_rbf * (G + |q|^2)).
// FAR: 0 = the group is near (R evaluated), 1 = far (R does not count), 2 = decided at run time by `far_rt`
// (warp-uniform).  With 0 or 1 the body has no branch, so the four groups of a row form one straight-line block.
template <bool MASKED, int FORM, int OFF, int FAR>
__device__ __forceinline__ float ga_sr_chunk(uint32_t (&w)[32], uint32_t g_taddr, bool far_rt, const float *kb, f2_t crbf2,
                                             f2_t cqn2, f2_t cs2, const GaForm &fm) {
#define v(i) w[OFF + (i)]
    const bool far = FAR == 2 ? far_rt : (FAR == 1);
    float m_loc = -INFINITY;
    f2_t rb[8];
    if (!far) {
        uint32_t gw[16];  // the 16 G values of the group, straight from tensor memory
        tmem_ld16(g_taddr + OFF, gw);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float a0, a1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(gw[2 * e]), __uint_as_float(gw[2 * e + 1])), crbf2, cqn2), a0, a1);
            if (FORM == 1) {  // keep R <= 1 exactly (the d^2 of a coincident pair can round below zero)
                a0 = fminf(a0, 0.f);
                a1 = fminf(a1, 0.f);
            }
            rb[e] = f2_pack(ex2_approx(a0), ex2_approx(a1));  // R
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const f2_t t2 = f2_mul(f2_pack(__uint_as_float(v(2 * e)), __uint_as_float(v(2 * e + 1))), cs2);
        f2_t sr;
        if (FORM == 0) {
            sr = far ? t2 : f2_fma(t2, rb[e], t2);
        } else if (far && fm.far_masked) {
            sr = f2_pack(-INFINITY, -INFINITY);
        } else {
            float t0, t1, r0 = 0.f, r1 = 0.f;  // a far group inside the window (min_rbf <= 0): R counts as 0
            f2_unpack(t2, t0, t1);
            if (!far) f2_unpack(rb[e], r0, r1);
            const float s0 = fmaf(fm.beta * fmaf(r0, fm.rn_a, fm.rn_b), fabsf(t0), t0);
            const float s1 = fmaf(fm.beta * fmaf(r1, fm.rn_a, fm.rn_b), fabsf(t1), t1);
            sr = f2_pack((r0 >= fm.rmin && r0 <= fm.rmax) ? s0 : -INFINITY, (r1 >= fm.rmin && r1 <= fm.rmax) ? s1 : -INFINITY);
        }
        float v0, v1;
        f2_unpack(sr, v0, v1);
        if (MASKED) {  // select, do not add: a padded key may hold Inf / NaN
            const float2 b = *reinterpret_cast<const float2 *>(kb + 2 * e);
            v0 = b.x == 0.f ? v0 : -INFINITY;
            v1 = b.y == 0.f ? v1 : -INFINITY;
        }
        v(2 * e) = __float_as_uint(v0);
        v(2 * e + 1) = __float_as_uint(v1);
        m_loc = max3(m_loc, v0, v1);
    }
    return m_loc;
#undef v
}

// 32 logits of one thread (two groups of 16 keys; H = which 32 of the thread's 64 = of the step's keys).  MODE 0: every
// group of the step is near, 1: every group is far, 2: per group (`far`).  `kb`: the mask entries of the step's 64 keys.
template <bool MASKED, int FORM, int MODE, int H>
__device__ __forceinline__ float ga_sr_half(uint32_t (&sv)[32], uint32_t gv, const float *kb, const bool (&far)[4], f2_t crbf2, f2_t cqn2,
                                            f2_t cs2, const GaForm &fm) {
    const float m0 = ga_sr_chunk<MASKED, FORM, 0, MODE>(sv, gv, far[2 * H], kb + (2 * H) * 16, crbf2, cqn2, cs2, fm);
    const float m1 = ga_sr_chunk<MASKED, FORM, 16, MODE>(sv, gv, far[2 * H + 1], kb + (2 * H + 1) * 16, crbf2, cqn2, cs2, fm);
    return fmaxf(m0, m1);
}

template <int FORM>
__global__ void __launch_bounds__(GA_FWD_THREADS, 2)
geoattn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const GaFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaFwdSmem &sm = *reinterpret_cast<GaFwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_math = warp < GA_FWD_MATH_THREADS / 32;
    const bool is_producer = warp == GA_FWD_MATH_THREADS / 32, is_stager = warp == GA_FWD_MATH_THREADS / 32 + 1;
    const int r = tid & (GA_BM - 1);              // math threads: query row inside the tile = TMEM lane
    const int N = p.N;
    const int tiles_all = (N + GA_BN - 1) / GA_BN;
    int zh_local = blockIdx.y;                    // index into the shard of (batch, head) pairs
    if (p.use_order) {  // samples longest first: the short ones fill the tail of the launch
        const int zp = zh_local / p.H;
        zh_local = ga_plan_order(p.plan)[zp] * p.H + (zh_local - zp * p.H);
    }
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int i0 = p.q_begin + blockIdx.x * GA_BM;
    const int row = i0 + r;
    const float *cz = p.coords + (size_t)z * N * 3;
    const uint8_t *vz = p.valid ? p.valid + (size_t)z * N : nullptr;
    // key tiles with at least one valid key (bit 15: also a padded or out-of-range key)
    const int *tl = p.plan ? ga_plan_tiles(p.plan, p.Z, N, z) : nullptr;
    const int nt = p.plan ? ga_plan_count(p.plan, p.Z)[z] : tiles_all;
    auto tile_word_g = [&](int t) -> int { return tl ? tl[t] : ga_plan_info_unmasked(N, t) | t; };
    // this CTA's query tile: dead (no valid query) or the offset of its first valid query
    const int q_info = p.plan ? ga_plan_info(p.plan, p.Z, N, z)[i0 / GA_BM] : ga_plan_info_unmasked(N, i0 / GA_BM);
    const bool q_ok = is_math && row < N && (vz ? vz[row] != 0 : true);
    __nv_bfloat16 *orow = p.out + (long long)z * p.so_z + (long long)h * p.so_h + (long long)row * p.so_n;
    if (q_info < 0 || nt == 0) {  // nothing to attend from / to: zeros and -inf
        if (is_math && row < N) {
#pragma unroll
            for (int c = 0; c < 8; ++c) reinterpret_cast<uint4 *>(orow)[c] = make_uint4(0, 0, 0, 0);
            p.lse[(size_t)zh * N + row] = -INFINITY;
        }
        return;
    }
    // steps of 64 keys: u = 2 t + sub; the second half of the sequence's last tile may lie entirely past N
    const int nu = 2 * nt - (((tile_word_g(nt - 1) & 0x7fff) * GA_BN + GA_BS >= N) ? 1 : 0);
    if (is_producer) {
        if (lane == 0) {
            mbar_init(&sm.bar_q, 1);
            mbar_init(&sm.bar_k[0], 1);
            mbar_init(&sm.bar_k[1], 1);
            mbar_init(&sm.bar_v[0], 1);
            mbar_init(&sm.bar_v[1], 1);
            mbar_init(&sm.bar_s, 1);
            mbar_init(&sm.bar_o, 1);
            mbar_init(&sm.bar_sfree, GA_FWD_MATH_THREADS);
            mbar_init(&sm.bar_p, GA_FWD_MATH_THREADS);
#pragma unroll
            for (int b = 0; b < GA_KC_BUFS; ++b) {
                mbar_init(&sm.bar_kc[b], 32);
                mbar_init(&sm.bar_kcfree[b], GA_FWD_MATH_THREADS);
            }
            mbar_fence_init();
            fence_proxy_async();
            // the first loads leave before anything else is set up
            mbar_expect_tx(&sm.bar_q, GA_TILE_BYTES);
            tma_load_4d(sm.q, &map_q, 0, i0, h, z, &sm.bar_q);
            for (int u = 0; u < 2 && u < nu; ++u) {
                const int j0 = (tile_word_g(u >> 1) & 0x7fff) * GA_BN + (u & 1) * GA_BS;
                mbar_expect_tx(&sm.bar_k[u], GA_STEP_BYTES);
                tma_load_4d(sm.k[u], &map_k, 0, j0, h, z, &sm.bar_k[u]);
                mbar_expect_tx(&sm.bar_v[u], GA_STEP_BYTES);
                tma_load_4d(sm.v[u], &map_v, 0, j0, h, z, &sm.bar_v[u]);
            }
            sm.abort = 0;
        }
        __syncwarp();
        tmem_alloc(&sm.tmem_base, GA_TMEM_COLS);
        tmem_relinquish();
    }
    for (int t = tid; t < nt; t += GA_FWD_THREADS) sm.tiles[t] = (uint16_t)tile_word_g(t);
    auto tile_word = [&](int t) -> int { return (int)sm.tiles[t]; };  // (published by the barrier below)
    // origin of the centred coordinates: the first valid query of this tile
    const int oq = i0 + (q_info & 0x7f);
    const float orx = cz[oq * 3], ory = cz[oq * 3 + 1], orz = cz[oq * 3 + 2];
    volatile int *abort_flag = &sm.abort;

    // Coordinates of four keys per stager lane (keys lane, lane + 32, lane + 64, lane + 96 of a tile): the loads are
    // issued at once from clamped indices, none waits for the validity bytes.
    struct KeyLoad {
        float gx[4], gy[4], gz[4];
        uint8_t vb[4];
    };
    auto key_load = [&](int tile, KeyLoad &k) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int jc = min(tile * GA_BN + lane + 32 * m, N - 1);
            k.vb[m] = vz ? vz[jc] : (uint8_t)1;
            k.gx[m] = cz[jc * 3];
            k.gy[m] = cz[jc * 3 + 1];
            k.gz[m] = cz[jc * 3 + 2];
        }
    };
    auto key_stage = [&](int tile, int buf, const KeyLoad &k) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int j = tile * GA_BN + lane + 32 * m;
            const bool ok = j < N && k.vb[m] != 0;
            ga_stage_key(sm.kc[buf], ga_geo_tile(sm, 1 + buf), ga_geo_block(1 + buf), lane + 32 * m, ok, ok ? k.gx[m] - orx : 0.f,
                         ok ? k.gy[m] - ory : 0.f, ok ? k.gz[m] - orz : 0.f);
        }
        fence_proxy_async();  // the geometry rows (generic-proxy stores) must be visible to the tensor core
    };
    // this thread's query, centred
    float qcx = 0.f, qcy = 0.f, qcz = 0.f;
    if (q_ok) {
        qcx = cz[row * 3] - orx;
        qcy = cz[row * 3 + 1] - ory;
        qcz = cz[row * 3 + 2] - orz;
    }
    if (is_math) {  // the queries' geometry operand: (-2 q, 1)
        ga_write_geo_row<true>(ga_geo_tile(sm, 0), ga_geo_block(0), r, -2.f * qcx, -2.f * qcy, -2.f * qcz, 1.f);
        fence_proxy_async();
    }
    KeyLoad kl;
    if (is_stager) key_load(tile_word_g(0) & 0x7fff, kl);  // in flight across the barrier
    tc_fence_before();
    __syncthreads();  // barriers initialised, TMEM allocated, tile list and the queries' geometry operand in place
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_s = tmem;          // columns [0,64): S
    const uint32_t tmem_g = tmem + 64;     // columns [64,128): G = |k|^2 - 2 q.k
    const uint32_t tmem_o = tmem + 128;    // columns [128,192): O accumulator
    const uint32_t tmem_p = tmem + 192;    // columns [192,224): P as bf16 pairs (A operand of P V)
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;

    if (is_stager) {
        // ================================ stager warp ================================================
        // Runs up to GA_KC_BUFS key tiles ahead of the math warps: geometry operand rows, masks and bounding spheres.
        for (int t = 0; t < nt; ++t) {
            const int b = t % GA_KC_BUFS;
            if (t > 0) key_load(tile_word(t) & 0x7fff, kl);
            // buffer b was last used by tile t - GA_KC_BUFS: every math thread has left it (and its G MMAs have completed)
            if (t >= GA_KC_BUFS && !__all_sync(0xffffffffu, mbar_wait_abortable(&sm.bar_kcfree[b], (uint32_t)((t / GA_KC_BUFS - 1) & 1), abort_flag) ? 1 : 0))
                break;  // (decided by the whole warp: the staging below shuffles across all 32 lanes)
            key_stage(tile_word(t) & 0x7fff, b, kl);
            mbar_arrive(&sm.bar_kc[b]);
        }
    } else if (is_producer) {
        // ================================ producer warp ==============================================
        if (lane == 0) {
            constexpr uint32_t IDESC_S = umma_idesc_bf16(GA_BM, GA_BS, false, false);  // Q K^T and G: both K-major, N = 64
            constexpr uint32_t IDESC_O = umma_idesc_bf16(GA_BM, GA_D, false, true);    // P V: V is MN-major
            // descriptors are built once; a step of K = 16 adds to the 16-byte-granular address field
            const uint64_t q_desc = umma_desc_sw128(smem_u32(sm.q), 16, 1024);
            const uint64_t k_desc[2] = {umma_desc_sw128(smem_u32(sm.k[0]), 16, 1024), umma_desc_sw128(smem_u32(sm.k[1]), 16, 1024)};
            const uint64_t v_desc[2] = {umma_desc_sw128(smem_u32(sm.v[0]), 0, 1024), umma_desc_sw128(smem_u32(sm.v[1]), 0, 1024)};
            const uint64_t geo_desc[2] = {umma_desc_sw128(smem_u32(sm.geo[0]), 16, 1024), umma_desc_sw128(smem_u32(sm.geo[1]), 16, 1024)};
            auto geo_slot_desc = [&](int slot) -> uint64_t { return geo_desc[slot >> 1] + (uint64_t)(ga_geo_block(slot) * 4); };
            constexpr uint64_t STEP_ROWS = (uint64_t)(GA_BS * 128) >> 4;  // 64 rows of a swizzled tile, in 16-byte units
            // S(u) = Q K^T: 4 MMAs of K = 16 over d = 64 (32 B per step inside the swizzled row); G(u): 2 more over the
            // geometry operands (the keys' rows start 64 rows into the staged tile for the second step of a tile)
            auto issue_s = [&](int u) {
                const int b = u & 1, t = u >> 1;
#pragma unroll
                for (int kk = 0; kk < GA_D / 16; ++kk)
                    umma_ss(tmem_s, q_desc + (uint64_t)(kk * 2), k_desc[b] + (uint64_t)(kk * 2), IDESC_S, kk > 0 ? 1u : 0u);
                const uint64_t qg = geo_slot_desc(0), kg = geo_slot_desc(1 + t % GA_KC_BUFS) + (uint64_t)(u & 1) * STEP_ROWS;
#pragma unroll
                for (int kk = 0; kk < GA_GEO_K / 16; ++kk)
                    umma_ss(tmem_g, qg + (uint64_t)(kk * 2), kg + (uint64_t)(kk * 2), IDESC_S, kk > 0 ? 1u : 0u);
                umma_commit(&sm.bar_s);
            };
            auto issue_pv = [&](int u) {  // 4 MMAs of K = 16 keys: P advances 8 TMEM columns, V 2 KiB
                const int b = u & 1;
#pragma unroll
                for (int kk = 0; kk < GA_BS / 16; ++kk)
                    umma_ts(tmem_o, tmem_p + kk * 8, v_desc[b] + (uint64_t)(kk * 128), IDESC_O, (u == 0 && kk == 0) ? 0u : 1u);
                umma_commit(&sm.bar_o);
            };
            auto key0 = [&](int u) -> int { return (tile_word(u >> 1) & 0x7fff) * GA_BN + (u & 1) * GA_BS; };
            auto load_k = [&](int u) {
                const int b = u & 1;
                mbar_expect_tx(&sm.bar_k[b], GA_STEP_BYTES);
                tma_load_4d(sm.k[b], &map_k, 0, key0(u), h, z, &sm.bar_k[b]);
            };
            auto load_v = [&](int u) {
                const int b = u & 1;
                mbar_expect_tx(&sm.bar_v[b], GA_STEP_BYTES);
                tma_load_4d(sm.v[b], &map_v, 0, key0(u), h, z, &sm.bar_v[b]);
            };
            bool ok = mbar_wait_abortable(&sm.bar_q, 0, abort_flag) && mbar_wait_abortable(&sm.bar_k[0], 0, abort_flag) &&
                      mbar_wait_abortable(&sm.bar_kc[0], 0, abort_flag);
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int u = 0; ok && u < nu; ++u) {
                const uint32_t par = (uint32_t)(u & 1);
                const int b = u & 1;
                if (u + 1 < nu) {
                    // every math thread holds S(u), G(u) in registers: their columns and K buffer b are free
                    if (!(ok = mbar_wait_abortable(&sm.bar_sfree, par, abort_flag))) break;
                    if (u + 2 < nu) load_k(u + 2);
                    if (!(ok = mbar_wait_abortable(&sm.bar_k[b ^ 1], (uint32_t)(((u + 1) >> 1) & 1), abort_flag))) break;
                    if (b == 1) {  // the next step opens key tile t + 1: its staged geometry operand
                        const int t1 = (u + 1) >> 1;
                        if (!(ok = mbar_wait_abortable(&sm.bar_kc[t1 % GA_KC_BUFS], (uint32_t)((t1 / GA_KC_BUFS) & 1), abort_flag))) break;
                    }
                    tc_fence_after();
                    issue_s(u + 1);  // S, G(u+1) run underneath the softmax of step u
                }
                if (!(ok = mbar_wait_abortable(&sm.bar_p, par, abort_flag))) break;  // P(u) in TMEM, O rescaled if need be
                if (!(ok = mbar_wait_abortable(&sm.bar_v[b], (uint32_t)((u >> 1) & 1), abort_flag))) break;
                tc_fence_after();
                issue_pv(u);
                if (u + 2 < nu) {  // V buffer b is free once P V(u) has completed
                    if (!(ok = mbar_wait_abortable(&sm.bar_o, par, abort_flag))) break;
                    load_v(u + 2);
                }
            }
            if (!ok) {
                // Gave up: the copies already issued may still be landing in this CTA's shared memory.  Wait for
                // them (bounded) so that the CTA does not exit underneath them.
                for (int b = 0; b < 2; ++b) {
                    mbar_wait_bounded(&sm.bar_k[b], 0, 1u << 12);
                    mbar_wait_bounded(&sm.bar_v[b], 0, 1u << 12);
                }
                mbar_wait_bounded(&sm.bar_q, 0, 1u << 12);
            }
        }
        __syncwarp();
    } else {
        // ================================ math warps ==================================================
        const float sig = p.sigma[h];
        const float c_rbf = -1.4426950408889634f / (2.f * sig * sig);  // R = 2^(c_rbf * d^2)
        const float c_s = p.scale * 1.4426950408889634f;               // logits in base-2 units
        // R = 2^(c_rbf d^2) with d^2 = G + |q|^2
        const float cqn = c_rbf * (qcx * qcx + qcy * qcy + qcz * qcz);
        const f2_t crbf2 = f2_pack(c_rbf, c_rbf), cqn2 = f2_pack(cqn, cqn), cs2 = f2_pack(c_s, c_s);
        GaForm fm;
        ga_form_setup(fm, FORM, FORM == 1 ? p.beta[h] : 0.f, p.min_rbf, p.max_rbf);
        // bounding sphere of the warp's valid queries; wq_reach = (distance beyond which R does not count) + radius
        float wqx, wqy, wqz, wq_reach;
        {
            float n = q_ok ? 1.f : 0.f, sx = qcx, sy = qcy, sz = qcz;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                n += __shfl_xor_sync(0xffffffffu, n, off);
                sx += __shfl_xor_sync(0xffffffffu, sx, off);
                sy += __shfl_xor_sync(0xffffffffu, sy, off);
                sz += __shfl_xor_sync(0xffffffffu, sz, off);
            }
            const float inv = n > 0.f ? 1.f / n : 0.f;
            wqx = sx * inv;
            wqy = sy * inv;
            wqz = sz * inv;
            float d2 = q_ok ? (qcx - wqx) * (qcx - wqx) + (qcy - wqy) * (qcy - wqy) + (qcz - wqz) * (qcz - wqz) : 0.f;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) d2 = fmaxf(d2, __shfl_xor_sync(0xffffffffu, d2, off));
            wq_reach = fm.far_cut * sig + sqrtf(d2) * 1.0001f + 1e-4f;
            if (!p.far_skip || !(fm.far_cut < INFINITY)) wq_reach = -INFINITY;  // test off
        }
        float m_run = -INFINITY, l_run = 0.f;
        // `ok` is kept uniform across the warp (tcgen05.ld / st and the votes below need all 32 lanes)
        bool ok = true;
        auto wait_w = [&](uint64_t *bar, uint32_t parity) -> bool {
            return __all_sync(0xffffffffu, mbar_wait_abortable(bar, parity, abort_flag) ? 1 : 0) != 0;
        };

        for (int u = 0; ok && u < nu; ++u) {
            const uint32_t par = (uint32_t)(u & 1);
            const int t = u >> 1, sub = u & 1, cb = t % GA_KC_BUFS;
            const bool has_hole = (tile_word(t) & 0x8000) != 0;
            uint32_t s0[32], s1[32];
            if (!(ok = wait_w(&sm.bar_s, par))) break;  // S(u), G(u) have landed in TMEM (the producer waited for the staged key tile)
            tc_fence_after();
            const GaKeyCoords &kc = sm.kc[cb];
            const float *kb = kc.kb + sub * GA_BS;
            bool far[4];
            int nfar = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // far test of the step's four key groups against this warp's queries (warp-uniform)
                const float4 sp = kc.sph[sub * 4 + c];
                const float dx = sp.x - wqx, dy = sp.y - wqy, dz = sp.z - wqz;
                const float reach = wq_reach + sp.w;  // wq_reach = cut + radius of the query sphere (-inf: test off)
                far[c] = sp.w < 0.f || (dx * dx + dy * dy + dz * dz > reach * reach && reach > 0.f);
                nfar += far[c] ? 1 : 0;
            }
            // S of the row into registers, G group by group, SR in place (it stays for the P phase)
            uint32_t gv = tmem_g + lane_base;
            float m_a, m_b;
#define PAI_GA_HALF(H, SV, MASKED, MODE) ga_sr_half<MASKED, FORM, MODE, H>(SV, gv, kb, far, crbf2, cqn2, cs2, fm)
#define PAI_GA_DISPATCH(H, SV, OUT)                                                                       \
    if (FORM == 0 && nfar == 0) {                                                                         \
        if (has_hole) OUT = PAI_GA_HALF(H, SV, true, 0); else OUT = PAI_GA_HALF(H, SV, false, 0);         \
    } else if (FORM == 0 && nfar == 4) {                                                                  \
        if (has_hole) OUT = PAI_GA_HALF(H, SV, true, 1); else OUT = PAI_GA_HALF(H, SV, false, 1);         \
    } else {                                                                                              \
        if (has_hole) OUT = PAI_GA_HALF(H, SV, true, 2); else OUT = PAI_GA_HALF(H, SV, false, 2);         \
    }
            tmem_ld32(tmem_s + lane_base, s0);
            tmem_ld32(tmem_s + lane_base + 32, s1);
            tmem_wait_ld();
            PAI_GA_DISPATCH(0, s0, m_a)
            gv += 32;
            PAI_GA_DISPATCH(1, s1, m_b)
#undef PAI_GA_DISPATCH
#undef PAI_GA_HALF
            tc_fence_before();
            mbar_arrive(&sm.bar_sfree);  // S and G are in registers: the tensor core may overwrite them with the next step's
            if (sub == 1 || u + 1 == nu) mbar_arrive(&sm.bar_kcfree[cb]);  // ... and the stager may reuse this key tile's buffer
            // the row maximum of the step (finite for form 0: every listed tile holds a valid key, though a step of it may
            // not; form 1 can mask a whole row)
            const float m_tile = fmaxf(m_a, m_b);
            float alpha = 1.f;
            bool raise = false;
            if (m_run == -INFINITY) {
                m_run = m_tile;
            } else if (m_tile > m_run + GA_RESCALE_THRESHOLD) {
                raise = true;
                alpha = ex2_approx(m_run - m_tile);
                m_run = m_tile;
            }
            // P = 2^(SR - m), row sum, bf16 pairs
            const float m_safe = m_run == -INFINITY ? 0.f : m_run;  // a row without any valid pair so far: P = 2^(-inf) = 0
            const f2_t mn2 = f2_pack(m_safe, m_safe);
            f2_t l2 = 0ull, l2b = 0ull;
            uint32_t pw[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                float a0, a1;
                const f2_t sr2 = e < 16 ? f2_pack(__uint_as_float(s0[2 * e]), __uint_as_float(s0[2 * e + 1]))
                                        : f2_pack(__uint_as_float(s1[2 * e - 32]), __uint_as_float(s1[2 * e - 31]));
                f2_unpack(f2_sub(sr2, mn2), a0, a1);
                const float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
                if (e & 1) l2b = f2_add(l2b, f2_pack(p0, p1));
                else l2 = f2_add(l2, f2_pack(p0, p1));
                pw[e] = pack_bf16x2(p0, p1);
            }
            float l0, l1;
            f2_unpack(f2_add(l2, l2b), l0, l1);
            l_run = l_run * alpha + (l0 + l1);
            if (u > 0) {  // P V(u-1) has completed: the P columns are free and the O accumulator is at rest
                if (!(ok = wait_w(&sm.bar_o, par ^ 1))) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, raise)) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tmem_o + lane_base + c * 32, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                        tmem_st32(tmem_o + lane_base + c * 32, v);
                    }
                }
            }
            tmem_st32(tmem_p + lane_base, pw);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sm.bar_p);
        }

        // ---- epilogue ----------------------------------------------------------------------------------
        if (ok) ok = wait_w(&sm.bar_o, (uint32_t)((nu - 1) & 1));
        if (ok) {  // (warp-uniform: tcgen05.ld needs all 32 lanes, rows past N included; only the stores are per row)
            tc_fence_after();
            // select, do not multiply by 0: padding may hold Inf / NaN in Q, K or V
            const bool live = q_ok && l_run > 0.f;
            const float inv = live ? 1.f / l_run : 0.f;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                uint32_t ov[32];
                tmem_ld32(tmem_o + lane_base + hh * 32, ov);
                tmem_wait_ld();
                if (row < N) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint4 pk;
                        pk.x = pack_bf16x2(__uint_as_float(ov[c * 8 + 0]) * inv, __uint_as_float(ov[c * 8 + 1]) * inv);
                        pk.y = pack_bf16x2(__uint_as_float(ov[c * 8 + 2]) * inv, __uint_as_float(ov[c * 8 + 3]) * inv);
                        pk.z = pack_bf16x2(__uint_as_float(ov[c * 8 + 4]) * inv, __uint_as_float(ov[c * 8 + 5]) * inv);
                        pk.w = pack_bf16x2(__uint_as_float(ov[c * 8 + 6]) * inv, __uint_as_float(ov[c * 8 + 7]) * inv);
                        reinterpret_cast<uint4 *>(orow)[hh * 4 + c] = live ? pk : make_uint4(0, 0, 0, 0);
                    }
                }
            }
            if (row < N) p.lse[(size_t)zh * N + row] = live ? (m_run + lg2_approx(l_run)) * 0.6931471805599453f : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (is_producer) tmem_dealloc(tmem, GA_TMEM_COLS);
}

}  // namespace pai
