// Geometric attention forward for sm_100a: flash attention on tcgen05 tensor cores with the
// per-head radial-basis scale applied in the softmax stage,
//     SR_ij = (q_i . k_j / sqrt(d)) * (1 + exp(-|r_i - r_j|^2 / (2 sigma_h^2))),
// a pair being valid iff query i and key j are both unpadded.  Replaces the Triton kernel
// `_attn_fwd` (old/old_scripts/attn/geometric_attn.py:57-260) with the logit form the reference's
// README states (README.md:40); the form the reference tree's kernel implements is the second
// instantiation (FORM = 1).
//
// One CTA = 128 query rows of one (batch, head): four math warps (one thread per query row = TMEM lane, so a row
// needs no exchange between threads) and three helper warps: one thread issues the MMAs, one the TMA loads of K and V, and
// a whole warp stages the keys' geometry.  Two CTAs share an SM.  Keys are taken 32 at a time (a "unit"; four
// units per 128-key tile of the batch plan, two per 64-key TMA box), and every per-unit buffer in tensor memory is
// doubled, so the tensor core works on unit w + 1 while the math warps hold unit w:
// Tensor memory (256 columns): S 2 x [32] fp32 at 0, G 2 x [32] fp32 at 64, O [64] fp32 at 128, P 2 x [16] bf16 pairs at 192.
//   S  = Q K^T : tcgen05.mma, A = Q tile, B = 32 rows of a K box (both K-major, 128-byte swizzle, via TMA);
//   G          : the geometry of the unit comes from the tensor core as well: G_ij = |k_j|^2 - 2 q_i . k_j
//                (coordinates centred on the tile's first valid query) is a product of two narrow operand tiles
//                that the threads write themselves, each fp32 coordinate split into three bf16 terms
//                (ga_write_geo_row), so that |r_i - r_j|^2 = G_ij + |q_i|^2 to fp32 accuracy.  Reading key
//                coordinates from shared memory instead costs every warp a broadcast load per key pair, which
//                made the shared-memory pipe, not the SFU, the limiter of this stage;
//   softmax    : the loop over units is NOT unrolled and has one body for every case (far / near groups and the
//                key mask are warp-uniform branches inside it): the whole loop is a few hundred instructions.
//                An unrolled loop with one specialised copy per case ran 30 % slower although it executed
//                fewer instructions, because the warps of an SM were fetching many different copies.
//                A math thread reads the 32 logits of its row and their G into registers (tcgen05.ld), so the
//                columns are free for unit w + 2 at once.  R = 2^(c G + c |q|^2), SR = S scale (1 + R) in packed
//                fp32x2 arithmetic.  A group of 16 keys whose bounding sphere lies farther than 5.9 sigma_h from
//                the bounding sphere of the warp's 32 queries has R < 2^-25 for every pair, where S (1 + R) == S
//                in fp32: there the exponential is skipped (most of the off-diagonal work of the narrow heads).
//                P is written as bf16 straight into tensor memory;
//   O += P V   : tcgen05.mma with the A operand (P) read from tensor memory, B = 32 rows of a V box (MN-major:
//                keys are the K dimension), accumulated in TMEM [128 x 64] across the units.  The running
//                maximum is only raised when a unit exceeds it by more than 2^GA_RESCALE_THRESHOLD (then the
//                accumulator and the row sum are rescaled); otherwise P is computed against the stale maximum,
//                which is exact after the final normalisation (floating point keeps the relative accuracy).
// The stager warp runs up to three key tiles ahead: geometry operand rows, mask bits and bounding spheres.  Key
// tiles without any valid key are never loaded (list from the batch plan, geoattn_plan.cuh); CTAs without any
// valid query only write zeros.  Every wait is bounded and abortable (tc.cuh).
#pragma once
#include "geoattn_plan.cuh"
#include "tc.cuh"

namespace pai {

constexpr int GA_BM = 128;  // query rows per CTA
constexpr int GA_BN = 128;  // tokens per tile of the batch plan (and per query / key tile of the backward)
constexpr int GA_BS = 64;   // keys per TMA box of the forward
constexpr int GA_UNIT = 32; // keys per unit of the forward
constexpr int GA_D = 64;    // head dimension
constexpr int GA_MAX_TILES = GA_PLAN_MAX_TILES;
constexpr int GA_FWD_MATH_THREADS = 128;
constexpr int GA_FWD_THREADS = GA_FWD_MATH_THREADS + 96;  // + the issuer, stager and loader warps
constexpr float GA_RESCALE_THRESHOLD = 24.f;                // log2 units
constexpr uint32_t GA_TMEM_COLS = 256;
constexpr uint32_t GA_TILE_BYTES = GA_BN * GA_D * 2;  // 16 KiB
constexpr uint32_t GA_STEP_BYTES = GA_BS * GA_D * 2;  // 8 KiB
constexpr int GA_KC_BUFS = 3;                           // staged key tiles in flight
constexpr float GA_FAR_SIGMAS = 5.9f;                   // exp(-d^2 / 2 sigma^2) < 2^-25 beyond 5.887 sigma

constexpr int GA_GEO_K = 32;                            // bf16 columns of the geometry operands (24 used)

struct GaKeyCoords {                  // per-key side data of one tile
    uint32_t vbits[GA_BN / 32];       // bit i of word u: key 32 u + i is valid
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
    uint64_t bar_q, bar_k[2], bar_v[2], bar_kfree[2], bar_vfree[2], bar_s[2], bar_p[2], bar_o[2], bar_kc[GA_KC_BUFS], bar_kcfree[GA_KC_BUFS];
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
    const int *sched;      // balanced schedule (geoattn_plan.cuh) or nullptr: one CTA per item
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

// Stages one key of a key tile: its geometry operand row, its mask bit and, with the other 15 keys of its half-warp,
// the bounding sphere of the group of 16.  Executed by whole warps with key = (lane + 32 m): the 16 lanes of a half-warp
// hold 16 consecutive keys.  `x, y, z` are the centred coordinates (0 for a padded key).
__device__ __forceinline__ void ga_stage_key(GaKeyCoords &kc, uint8_t *geo_tile, int geo_block, int key, bool ok, float x, float y, float z) {
    ga_write_geo_row<false>(geo_tile, geo_block, key, x, y, z, x * x + y * y + z * z);
    const uint32_t bits = __ballot_sync(0xffffffffu, ok);
    if ((key & 31) == 0) kc.vbits[key >> 5] = bits;
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

// 16 logits (8 key pairs) of one row, held in registers: s[OFF..OFF+16) holds raw S on entry and SR on return,
// g[] the matching G values; returns the maximum.  SR = (S * c_s) * (1 + R) with R = 2^(c_rbf * (G + |q|^2)).
// `far` (warp-uniform): the group's R does not count.
template <int FORM, int OFF>
__device__ __forceinline__ float ga_sr_chunk(uint32_t (&s)[32], const uint32_t (&g)[32], bool far, f2_t crbf2, f2_t cqn2, f2_t cs2,
                                             const GaForm &fm) {
    float m_loc = -INFINITY;
    if (!far) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float a0, a1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(g[OFF + 2 * e]), __uint_as_float(g[OFF + 2 * e + 1])), crbf2, cqn2), a0, a1);
            if (FORM == 1) {  // keep R <= 1 exactly (the d^2 of a coincident pair can round below zero)
                a0 = fminf(a0, 0.f);
                a1 = fminf(a1, 0.f);
            }
            const float r0 = ex2_approx(a0), r1 = ex2_approx(a1);  // R
            const f2_t t2 = f2_mul(f2_pack(__uint_as_float(s[OFF + 2 * e]), __uint_as_float(s[OFF + 2 * e + 1])), cs2);
            float v0, v1;
            if (FORM == 0) {
                f2_unpack(f2_fma(t2, f2_pack(r0, r1), t2), v0, v1);
            } else {
                float t0, t1;
                f2_unpack(t2, t0, t1);
                const float s0 = fmaf(fm.beta * fmaf(r0, fm.rn_a, fm.rn_b), fabsf(t0), t0);
                const float s1 = fmaf(fm.beta * fmaf(r1, fm.rn_a, fm.rn_b), fabsf(t1), t1);
                v0 = (r0 >= fm.rmin && r0 <= fm.rmax) ? s0 : -INFINITY;
                v1 = (r1 >= fm.rmin && r1 <= fm.rmax) ? s1 : -INFINITY;
            }
            s[OFF + 2 * e] = __float_as_uint(v0);
            s[OFF + 2 * e + 1] = __float_as_uint(v1);
            m_loc = max3(m_loc, v0, v1);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const f2_t t2 = f2_mul(f2_pack(__uint_as_float(s[OFF + 2 * e]), __uint_as_float(s[OFF + 2 * e + 1])), cs2);
            float v0, v1;
            f2_unpack(t2, v0, v1);
            if (FORM == 1) {
                if (fm.far_masked) {
                    v0 = v1 = -INFINITY;
                } else {  // a far group inside the window (min_rbf <= 0): R counts as 0
                    v0 = (0.f >= fm.rmin && 0.f <= fm.rmax) ? fmaf(fm.beta * fm.rn_b, fabsf(v0), v0) : -INFINITY;
                    v1 = (0.f >= fm.rmin && 0.f <= fm.rmax) ? fmaf(fm.beta * fm.rn_b, fabsf(v1), v1) : -INFINITY;
                }
            }
            s[OFF + 2 * e] = __float_as_uint(v0);
            s[OFF + 2 * e + 1] = __float_as_uint(v1);
            m_loc = max3(m_loc, v0, v1);
        }
    }
    return m_loc;
}

// One work item: the query tile `q_tile` (counted from q_begin) of the (batch, head) pair `zh_local` of the launch.  Every
// thread of the CTA calls it; tensor memory is allocated by the caller.  `fresh`: the CTA has not initialised its barriers
// yet; a live item clears it, later ones invalidate the barriers before they initialise them again.
template <int FORM>
__device__ __forceinline__ void geoattn_fwd_item(GaFwdSmem &sm, const CUtensorMap &map_q, const CUtensorMap &map_k, const CUtensorMap &map_v,
                                                 const GaFwdParams &p, int zh_local, int q_tile, bool &fresh) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_math = warp < GA_FWD_MATH_THREADS / 32;
    const bool is_producer = warp == GA_FWD_MATH_THREADS / 32, is_stager = warp == GA_FWD_MATH_THREADS / 32 + 1;
    const int r = tid & (GA_BM - 1);              // math threads: query row inside the tile = TMEM lane
    const int N = p.N;
    const int tiles_all = (N + GA_BN - 1) / GA_BN;
    const int zh = p.zh_begin + zh_local;
    const int z = zh / p.H, h = zh - z * p.H;
    const int i0 = p.q_begin + q_tile * GA_BM;
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
    // units of 32 keys: w = 4 t + quarter; the trailing units of the sequence's last tile may lie entirely past N
    const int last_keys = min(GA_BN, N - (tile_word_g(nt - 1) & 0x7fff) * GA_BN);
    const int nw = 4 * (nt - 1) + (last_keys + GA_UNIT - 1) / GA_UNIT;
    const int nbox = (nw + 1) >> 1;  // TMA boxes of 64 keys
    if (is_producer) {
        if (lane == 0) {
            if (!fresh) {
                mbar_inval(&sm.bar_q);
                mbar_inval(&sm.bar_o[0]);
                mbar_inval(&sm.bar_o[1]);
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    mbar_inval(&sm.bar_k[b]);
                    mbar_inval(&sm.bar_v[b]);
                    mbar_inval(&sm.bar_kfree[b]);
                    mbar_inval(&sm.bar_vfree[b]);
                    mbar_inval(&sm.bar_s[b]);
                    mbar_inval(&sm.bar_p[b]);
                }
#pragma unroll
                for (int b = 0; b < GA_KC_BUFS; ++b) {
                    mbar_inval(&sm.bar_kc[b]);
                    mbar_inval(&sm.bar_kcfree[b]);
                }
            }
            mbar_init(&sm.bar_q, 1);
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                mbar_init(&sm.bar_k[b], 1);
                mbar_init(&sm.bar_v[b], 1);
                mbar_init(&sm.bar_kfree[b], 1);
                mbar_init(&sm.bar_vfree[b], 1);
                mbar_init(&sm.bar_s[b], 1);
                mbar_init(&sm.bar_o[b], 1);
                mbar_init(&sm.bar_p[b], GA_FWD_MATH_THREADS);
            }
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
            for (int j = 0; j < 2 && j < nbox; ++j) {
                const int j0 = (tile_word_g(j >> 1) & 0x7fff) * GA_BN + (j & 1) * GA_BS;
                mbar_expect_tx(&sm.bar_k[j], GA_STEP_BYTES);
                tma_load_4d(sm.k[j], &map_k, 0, j0, h, z, &sm.bar_k[j]);
                mbar_expect_tx(&sm.bar_v[j], GA_STEP_BYTES);
                tma_load_4d(sm.v[j], &map_v, 0, j0, h, z, &sm.bar_v[j]);
            }
        }
        __syncwarp();
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
    fresh = false;
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_s = tmem;          // columns [0,64): S of units w (even) and w + 1 (odd), 32 each
    const uint32_t tmem_g = tmem + 64;     // columns [64,128): G = |k|^2 - 2 q.k, likewise
    const uint32_t tmem_o = tmem + 128;    // columns [128,192): O accumulator
    const uint32_t tmem_p = tmem + 192;    // columns [192,224): P as bf16 pairs (A operand of P V), 16 per unit parity
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const bool is_loader = warp == GA_FWD_MATH_THREADS / 32 + 2;
    // Every warp waits as a whole and keeps `ok` uniform: tcgen05.ld / st and the votes need all 32 lanes, and a helper
    // warp whose lanes 1..31 sit at a reconvergence point while lane 0 loops runs several times slower than a
    // converged warp in which lane 0 alone issues the copy or MMA.
    auto wait_w = [&](uint64_t *bar, uint32_t parity) -> bool {
        return __all_sync(0xffffffffu, mbar_wait_abortable(bar, parity, abort_flag) ? 1 : 0) != 0;
    };

    if (is_stager) {
        // ================================ stager warp ================================================
        // Runs up to GA_KC_BUFS key tiles ahead of the math warps: geometry operand rows, mask bits and bounding spheres.
        for (int t = 0; t < nt; ++t) {
            const int b = t % GA_KC_BUFS;
            if (t > 0) key_load(tile_word(t) & 0x7fff, kl);
            // buffer b was last used by tile t - GA_KC_BUFS: every math thread has left it (and its G MMAs have completed)
            if (t >= GA_KC_BUFS && !wait_w(&sm.bar_kcfree[b], (uint32_t)((t / GA_KC_BUFS - 1) & 1))) break;
            key_stage(tile_word(t) & 0x7fff, b, kl);
            mbar_arrive(&sm.bar_kc[b]);
        }
    } else if (is_loader) {
        // ================================ loader warp ================================================
        // K / V box j goes into buffer j & 1 once the MMAs that read box j - 2 have completed.
        bool ok = true;
        for (int j = 2; ok && j < nbox; ++j) {
            const int b = j & 1;
            const uint32_t par = (uint32_t)(((j >> 1) - 1) & 1);
            const int j0 = (tile_word(j >> 1) & 0x7fff) * GA_BN + (j & 1) * GA_BS;
            if (!(ok = wait_w(&sm.bar_kfree[b], par))) break;
            if (lane == 0) {
                mbar_expect_tx(&sm.bar_k[b], GA_STEP_BYTES);
                tma_load_4d(sm.k[b], &map_k, 0, j0, h, z, &sm.bar_k[b]);
            }
            if (!(ok = wait_w(&sm.bar_vfree[b], par))) break;
            if (lane == 0) {
                mbar_expect_tx(&sm.bar_v[b], GA_STEP_BYTES);
                tma_load_4d(sm.v[b], &map_v, 0, j0, h, z, &sm.bar_v[b]);
            }
        }
        // the commits behind the last S and P V MMAs also arrive on the buffers' release barriers: see them land before the
        // item ends (the barriers are re-initialised for the CTA's next item)
        for (int b = 0; ok && b < 2; ++b) {
            const int nb = (nbox + 1 - b) >> 1;  // boxes that went through buffer b
            if (nb > 0) ok = wait_w(&sm.bar_kfree[b], (uint32_t)((nb - 1) & 1)) && wait_w(&sm.bar_vfree[b], (uint32_t)((nb - 1) & 1));
        }
        if (lane == 0 && (!ok || *abort_flag)) {
            // Gave up: the copies already issued may still be landing in this CTA's shared memory.  Wait for
            // them (bounded) so that the CTA does not exit underneath them.
            for (int b = 0; b < 2; ++b) {
                mbar_wait_bounded(&sm.bar_k[b], 0, 1u << 12);
                mbar_wait_bounded(&sm.bar_v[b], 0, 1u << 12);
            }
            mbar_wait_bounded(&sm.bar_q, 0, 1u << 12);
        }
        __syncwarp();
    } else if (is_producer) {
        // ================================ issuer warp ================================================
        // One thread issues every MMA, in the order S(0), S(1), P V(0), S(2), P V(1), S(3), ...: S(w+2) follows P V(w) into
        // the columns that unit w has left, a whole unit before the math warps want it.  The tensor core works through
        // its queue in order, so a math thread that sees S(w) complete knows that P V(w-2) is complete too, and writes
        // P(w) over P(w-2) without a further wait.
        {
            constexpr uint32_t IDESC_S = umma_idesc_bf16(GA_BM, GA_UNIT, false, false);  // Q K^T and G: both K-major, N = 32
            // descriptors are built once; a step of K = 16 adds to the 16-byte-granular address field
            const uint64_t q_desc = umma_desc_sw128(smem_u32(sm.q), 16, 1024);
            // (the second buffer of a pair follows the first: its descriptor is the first one's plus the distance)
            const uint64_t k_desc0 = umma_desc_sw128(smem_u32(sm.k[0]), 16, 1024), geo_desc0 = umma_desc_sw128(smem_u32(sm.geo[0]), 16, 1024);
            auto geo_slot_desc = [&](int slot) -> uint64_t {
                return geo_desc0 + (uint64_t)(slot >> 1) * (GA_TILE_BYTES >> 4) + (uint64_t)(ga_geo_block(slot) * 4);
            };
            constexpr uint64_t UNIT_ROWS = (uint64_t)(GA_UNIT * 128) >> 4;  // 32 rows of a swizzled tile, in 16-byte units
            // S(w) = Q K^T: 4 MMAs of K = 16 over d = 64 (32 B per step inside the swizzled row); G(w): 2 more over the
            // geometry operands (the keys' rows start 32 (w mod 4) rows into the staged tile)
            auto issue_s = [&](int w) {
                const int sb = w & 1, kb = (w >> 1) & 1, t = w >> 2;
                const uint64_t kd = k_desc0 + (uint64_t)kb * (GA_STEP_BYTES >> 4) + (uint64_t)(w & 1) * UNIT_ROWS;
#pragma unroll
                for (int kk = 0; kk < GA_D / 16; ++kk)
                    umma_ss(tmem_s + sb * GA_UNIT, q_desc + (uint64_t)(kk * 2), kd + (uint64_t)(kk * 2), IDESC_S, kk > 0 ? 1u : 0u);
                const uint64_t qg = geo_slot_desc(0), kg = geo_slot_desc(1 + t % GA_KC_BUFS) + (uint64_t)(w & 3) * UNIT_ROWS;
#pragma unroll
                for (int kk = 0; kk < GA_GEO_K / 16; ++kk)
                    umma_ss(tmem_g + sb * GA_UNIT, qg + (uint64_t)(kk * 2), kg + (uint64_t)(kk * 2), IDESC_S, kk > 0 ? 1u : 0u);
                umma_commit(&sm.bar_s[sb]);
                if ((w & 1) || w + 1 == nw) umma_commit(&sm.bar_kfree[kb]);  // the box's last reader
            };
            constexpr uint32_t IDESC_O = umma_idesc_bf16(GA_BM, GA_D, false, true);      // P V: V is MN-major
            const uint64_t v_desc0 = umma_desc_sw128(smem_u32(sm.v[0]), 0, 1024);
            auto issue_pv = [&](int w) {  // 2 MMAs of K = 16 keys: P advances 8 TMEM columns, V 2 KiB
                const int pb = w & 1, vb = (w >> 1) & 1;
#pragma unroll
                for (int kk = 0; kk < GA_UNIT / 16; ++kk)
                    umma_ts(tmem_o, tmem_p + pb * (GA_UNIT / 2) + kk * 8, v_desc0 + (uint64_t)vb * (GA_STEP_BYTES >> 4) + (uint64_t)(((w & 1) * 2 + kk) * 128), IDESC_O,
                            (w == 0 && kk == 0) ? 0u : 1u);
                umma_commit(&sm.bar_o[pb]);
                if ((w & 1) || w + 1 == nw) umma_commit(&sm.bar_vfree[vb]);
            };
            bool ok = wait_w(&sm.bar_q, 0) && wait_w(&sm.bar_k[0], 0) && wait_w(&sm.bar_kc[0], 0);
            if (ok) {
                tc_fence_after();
                if (lane == 0) {
                    issue_s(0);
                    if (nw > 1) issue_s(1);
                }
                __syncwarp();
            }
            for (int w = 0; ok && w < nw; ++w) {
                // P(w) in TMEM (and O rescaled if need be); its arrival also says that every math thread holds S(w), G(w)
                // in registers, so that their columns can take unit w + 2
                if (!(ok = wait_w(&sm.bar_p[w & 1], (uint32_t)((w >> 1) & 1)))) break;
                if ((w & 1) == 0 && !(ok = wait_w(&sm.bar_v[(w >> 1) & 1], (uint32_t)((w >> 2) & 1)))) break;
                const int w2 = w + 2, t2 = w2 >> 2;
                if (w2 < nw) {
                    if ((w2 & 1) == 0 && !(ok = wait_w(&sm.bar_k[(w2 >> 1) & 1], (uint32_t)((w2 >> 2) & 1)))) break;
                    if ((w2 & 3) == 0 && !(ok = wait_w(&sm.bar_kc[t2 % GA_KC_BUFS], (uint32_t)((t2 / GA_KC_BUFS) & 1)))) break;
                }
                tc_fence_after();
                if (lane == 0) {
                    issue_pv(w);
                    if (w2 < nw) issue_s(w2);
                }
                __syncwarp();
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
        bool ok = true;

#pragma unroll 1
        for (int w = 0; ok && w < nw; ++w) {
            const int sb = w & 1, t = w >> 2, qd = w & 3, cb = t % GA_KC_BUFS;
            const bool has_hole = (tile_word(t) & 0x8000) != 0;
            if (!(ok = wait_w(&sm.bar_s[sb], (uint32_t)((w >> 1) & 1)))) break;  // S(w), G(w) have landed in TMEM
            tc_fence_after();
            const GaKeyCoords &kc = sm.kc[cb];
            uint32_t s[32], g[32];
            tmem_ld32(tmem_s + sb * GA_UNIT + lane_base, s);  // (in flight under the far test)
            bool far[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {  // far test of the unit's two key groups against this warp's queries (warp-uniform)
                const float4 sp = kc.sph[qd * 2 + c];
                const float dx = sp.x - wqx, dy = sp.y - wqy, dz = sp.z - wqz;
                const float reach = wq_reach + sp.w;  // wq_reach = cut + radius of the query sphere (-inf: test off)
                far[c] = sp.w < 0.f || (dx * dx + dy * dy + dz * dz > reach * reach && reach > 0.f);
            }
            const uint32_t vbits = kc.vbits[qd];
            if (!(far[0] && far[1])) tmem_ld32(tmem_g + sb * GA_UNIT + lane_base, g);
            tmem_wait_ld();
            tc_fence_before();
            if (qd == 3 || w + 1 == nw) mbar_arrive(&sm.bar_kcfree[cb]);  // the stager may reuse this key tile's buffer
            float m_unit = fmaxf(ga_sr_chunk<FORM, 0>(s, g, far[0], crbf2, cqn2, cs2, fm), ga_sr_chunk<FORM, 16>(s, g, far[1], crbf2, cqn2, cs2, fm));
            if (has_hole) {  // select, do not add: a padded key may hold Inf / NaN
                m_unit = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float v = (vbits >> i) & 1u ? __uint_as_float(s[i]) : -INFINITY;
                    s[i] = __float_as_uint(v);
                    m_unit = fmaxf(m_unit, v);
                }
            }
            // the row maximum (finite for form 0 once the row has met a valid key; form 1 can mask a whole row)
            float alpha = 1.f;
            bool raise = false;
            if (m_run == -INFINITY) {
                m_run = m_unit;
            } else if (m_unit > m_run + GA_RESCALE_THRESHOLD) {
                raise = true;
                alpha = ex2_approx(m_run - m_unit);
                m_run = m_unit;
            }
            if (__any_sync(0xffffffffu, raise)) {  // rare: rescale the row sum and the accumulator
                l_run *= alpha;
                if (w > 0) {  // P V(w-1) must have completed: the O accumulator is at rest
                    if (!(ok = wait_w(&sm.bar_o[(w - 1) & 1], (uint32_t)(((w - 1) >> 1) & 1)))) break;
                    tc_fence_after();
#pragma unroll 1
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
            // P = 2^(SR - m), row sum, bf16 pairs
            const float m_safe = m_run == -INFINITY ? 0.f : m_run;  // a row without any valid pair so far: P = 2^(-inf) = 0
            const f2_t mn2 = f2_pack(m_safe, m_safe);
            f2_t l2 = 0ull, l2b = 0ull;
            uint32_t pw[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                float a0, a1;
                f2_unpack(f2_sub(f2_pack(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1])), mn2), a0, a1);
                const float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
                if (e & 1) l2b = f2_add(l2b, f2_pack(p0, p1));
                else l2 = f2_add(l2, f2_pack(p0, p1));
                pw[e] = pack_bf16x2(p0, p1);
            }
            float l0, l1;
            f2_unpack(f2_add(l2, l2b), l0, l1);
            l_run += l0 + l1;
            // (P V(w-2), the last reader of these P columns, completed before S(w): the tensor core works in issue order)
            tmem_st16(tmem_p + sb * (GA_UNIT / 2) + lane_base, pw);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&sm.bar_p[sb]);
        }

        // ---- epilogue ----------------------------------------------------------------------------------
        if (ok) ok = wait_w(&sm.bar_o[(nw - 1) & 1], (uint32_t)(((nw - 1) >> 1) & 1));  // (the units' P V complete in issue order)
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
    __syncthreads();  // every role has left the item: its barriers, buffers and tensor-memory columns can be reused
}

// Grid without a schedule: one CTA per (query tile, (batch, head) pair), the samples longest first when the plan's order
// applies.  With a schedule (geoattn_plan.cuh): `bins` persistent CTAs, each working through the items assigned to it and
// writing the zeros of its share of the tiles without a valid query.
template <int FORM>
__global__ void __launch_bounds__(GA_FWD_THREADS, 2)
geoattn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const GaFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    GaFwdSmem &sm = *reinterpret_cast<GaFwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    if (warp == GA_FWD_MATH_THREADS / 32) {
        if (threadIdx.x == GA_FWD_MATH_THREADS) sm.abort = 0;
        __syncwarp();
        tmem_alloc(&sm.tmem_base, GA_TMEM_COLS);
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
        geoattn_fwd_item<FORM>(sm, map_q, map_k, map_v, p, zh_local, tile, fresh);
        if (!fresh) {
            __syncthreads();  // (after a live item: thread 0 has read the item's partial sums; sm.abort is settled)
            if (sm.abort) break;
        }
    }
    // (a CTA that ran no live item has not synchronised since the allocation)
    tc_fence_before();
    __syncthreads();
    if (warp == GA_FWD_MATH_THREADS / 32) tmem_dealloc(sm.tmem_base, GA_TMEM_COLS);
}

}  // namespace pai
