// C ABI of the proteus_b200 library (see include/proteus_b200.h).  Single translation unit:
// the kernels are header files so that the device status word needs no relocatable device code.
#include "common.cuh"

#include "geoattn_bwd.cuh"
#include "encoder_ops.cuh"
#include "neighbors.cuh"
#include "geoattn_fwd.cuh"
#include "we_bwd.cuh"
#include "we_fwd.cuh"
#include "we_aniso_fwd.cuh"

#include <cstring>

namespace {

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Compute capability of the current device, cached per device ordinal.
int current_device_cc(int *cc_out) {
    static int cache[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64 && cache[dev]) {
        *cc_out = cache[dev];
        return 0;
    }
    int major = 0, minor = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (e != cudaSuccess) return (int)e;
    *cc_out = major * 10 + minor;
    if (dev >= 0 && dev < 64) cache[dev] = *cc_out;
    return 0;
}

// Run counters of the WE forward (one 4-byte slot per launch in flight, handed out round-robin): part of the
// library image so that the entry point needs no workspace argument.
static __device__ unsigned g_we_run_counters[256];

int next_we_counter(unsigned **slot) {
    static unsigned *base[64];
    static unsigned next[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)PAI_ERR_UNSUPPORTED;
    if (!base[dev]) {
        unsigned *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_we_run_counters);
        if (e != cudaSuccess) return (int)e;
        base[dev] = p;
    }
    *slot = base[dev] + (__atomic_fetch_add(&next[dev], 1u, __ATOMIC_RELAXED) & 255u);
    return 0;
}

int current_device_sms(int *sms_out) {
    static int cache[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64 && cache[dev]) {
        *sms_out = cache[dev];
        return 0;
    }
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (sms < 1) return (int)PAI_ERR_UNSUPPORTED;
    *sms_out = sms;
    if (dev >= 0 && dev < 64) cache[dev] = sms;
    return 0;
}

int require_sm100() {
    int cc = 0;
    int e = current_device_cc(&cc);
    if (e) return e;
    return cc == 100 ? 0 : (int)PAI_ERR_NOT_SM100;
}

// Tuning knobs of the test-only entry pai_tune_set (plain process-wide integers; the hot entry points read
// them without any environment lookup).  Defaults are what the library ships with.
int g_tune[PAI_TUNE_COUNT] = {
    /* PAI_TUNE_WE_KS */ 0,        /* PAI_TUNE_WE_TJ */ 0,          /* PAI_TUNE_WE_WAVES */ 0,
    /* PAI_TUNE_WE_RANGE_REDUCE */ 0, /* PAI_TUNE_WE_POLY_PAIRS */ 2, /* PAI_TUNE_WE_NO_TMA */ 0,
    /* PAI_TUNE_GA_NO_FAR_SKIP */ 0,  /* PAI_TUNE_GA_NO_ORDER */ 0,   /* PAI_TUNE_WE_MIXED */ 0,
};

// register-only sin+cos loop: 8 independent chains per thread
__global__ void __launch_bounds__(256) sfu_peak_kernel(int iters, float seed) {
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = seed + 0.001f * (threadIdx.x + 17 * i);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float s, c;
            pai::sfu_sincos(x[i], s, c);
            x[i] = s + c;
        }
    }
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += x[i];
    if (t == 123456.789f) pai::g_sink = t;
}

}  // namespace

extern "C" {

int pai_abi_version(void) { return 6; }  // 6: balanced attention schedules (5: WE flags, batch plan, query-row ranges, test-only entries)

const char *pai_status_str(int status) {
    switch (status) {
        case PAI_OK: return "ok";
        case PAI_ERR_NULL_POINTER: return "null pointer argument";
        case PAI_ERR_BAD_SHAPE: return "bad shape (sizes must be positive and within limits)";
        case PAI_ERR_MISALIGNED: return "pointer not aligned as required";
        case PAI_ERR_UNSUPPORTED: return "unsupported option";
        case PAI_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
        case PAI_ERR_BAD_ROW_RANGE: return "bad row range (need 0 <= begin <= end <= N)";
        case PAI_ERR_NOT_SM100: return "current device is not sm_100 (B200)";
        case PAI_ERR_DEVICE_WAIT_TIMEOUT: return "a kernel gave up on a bounded device-side wait";
        case PAI_ERR_EXCEEDS_STATIC_SCRATCH:
            return "size exceeds the built-in scratch of the allocation-free entry point (K > 1024); use the workspace variant";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

int pai_device_status(void *stream) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, pai::g_device_status, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(pai::g_device_status, &zero, sizeof(int));
        if (e != cudaSuccess) return (int)e;
    }
    return v;
}

int pai_we_fwd(const float *coords_soa, const uint8_t *valid, const float *wavenumbers, float *out, float *cos_sums,
               float *sin_sums, int Z, int N, int K, int row_begin, int row_end, int magnitude_type, float dropout_p,
               uint32_t seed, uint32_t flags, void *stream) {
    if (!coords_soa || !wavenumbers || !out || !cos_sums || !sin_sums) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || Z > 65535 || N < 1 || K < 1 || (long long)N * K > (1ll << 40)) return PAI_ERR_BAD_SHAPE;
    if (row_begin < 0 || row_end > N || row_begin > row_end) return PAI_ERR_BAD_ROW_RANGE;
    if (magnitude_type < 0 || magnitude_type > 3) return PAI_ERR_UNSUPPORTED;
    if (!(dropout_p >= 0.0f && dropout_p < 1.0f)) return PAI_ERR_UNSUPPORTED;
    if (flags & ~(uint32_t)PAI_WE_REPRODUCIBLE) return PAI_ERR_UNSUPPORTED;
    if (!aligned(coords_soa, 4) || !aligned(wavenumbers, 4)) return PAI_ERR_MISALIGNED;
    if ((K & 1) == 0 ? (!aligned(out, 16) || !aligned(cos_sums, 8) || !aligned(sin_sums, 8))
                     : (!aligned(out, 4) || !aligned(cos_sums, 4) || !aligned(sin_sums, 4)))
        return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    if (row_begin == row_end) return PAI_OK;
    pai::WeFwdParams p;
    p.coords = coords_soa;
    p.valid = valid;
    p.wn = wavenumbers;
    p.out = out;
    p.cos_sums = cos_sums;
    p.sin_sums = sin_sums;
    p.N = N;
    p.K = K;
    p.row_begin = row_begin;
    p.row_end = row_end;
    p.mag_type = magnitude_type;
    p.seed = seed;
    p.drop_thr = 0u;
    p.drop_scale = 0.f;
    if (dropout_p != 0.0f) {
        // The reference keeps an evaluation when (float)h / (float)UINT32_MAX >= p, where (float)UINT32_MAX is 2^32
        // and the conversion of h rounds to nearest.  That conversion is monotonic in h, so the test equals
        // h >= (the smallest h that passes), found here by bisection with the same float arithmetic.
        const float t = dropout_p * 4294967296.0f;  // exact (a power-of-two scaling)
        uint32_t lo = 0u, hi = 0xffffffffu;          // invariant: hi passes (p < 1), everything below lo fails
        while (lo < hi) {
            const uint32_t mid = lo + (hi - lo) / 2u;
            if ((float)mid >= t) hi = mid;
            else lo = mid + 1u;
        }
        p.drop_thr = lo;
        p.drop_scale = 1.0f / (1.0f - dropout_p);
    }
    // bulk copies need 16-byte aligned plane segments: base aligned and N a multiple of 4
    p.use_tma = (aligned(coords_soa, 16) && (N % 4) == 0 && g_tune[PAI_TUNE_WE_NO_TMA] == 0) ? 1 : 0;
    // the kernel adds partial sums into the outputs: zero the rows of the shard first
    cudaStream_t st = (cudaStream_t)stream;
    const size_t rows = (size_t)(row_end - row_begin);
    cudaError_t ce = cudaMemset2DAsync(out + (size_t)row_begin * 2 * K, (size_t)N * 2 * K * sizeof(float), 0,
                                       rows * 2 * K * sizeof(float), (size_t)Z, st);
    if (ce != cudaSuccess) return (int)ce;
    ce = cudaMemset2DAsync(cos_sums + (size_t)row_begin * K, (size_t)N * K * sizeof(float), 0, rows * K * sizeof(float),
                           (size_t)Z, st);
    if (ce != cudaSuccess) return (int)ce;
    ce = cudaMemset2DAsync(sin_sums + (size_t)row_begin * K, (size_t)N * K * sizeof(float), 0, rows * K * sizeof(float),
                           (size_t)Z, st);
    if (ce != cudaSuccess) return (int)ce;
    int sms = 0;
    if (int e = current_device_sms(&sms)) return e;
    unsigned *counter = nullptr;
    if (int e = next_we_counter(&counter)) return e;
    return pai::we_fwd_launch(p, Z, g_tune[PAI_TUNE_WE_KS], g_tune[PAI_TUNE_WE_TJ], g_tune[PAI_TUNE_WE_WAVES],
                              (flags & PAI_WE_REPRODUCIBLE) != 0, g_tune[PAI_TUNE_WE_RANGE_REDUCE] != 0,
                              g_tune[PAI_TUNE_WE_POLY_PAIRS], g_tune[PAI_TUNE_WE_MIXED] != 0, sms, counter, st);
}

size_t pai_we_bwd_dk_workspace_bytes(int Z, int N, int K) {
    (void)Z;
    (void)N;
    if (K < 1) return 0;
    return (size_t)pai::WE_BWD_MAX_BLOCKS * (size_t)K * sizeof(float);
}

int pai_we_bwd_dk(const float *dO, const float *cos_sums, const float *sin_sums, float *dk, void *workspace,
                  size_t workspace_bytes, int Z, int N, int K, int row_begin, int row_end, void *stream) {
    if (!dO || !cos_sums || !sin_sums || !dk || !workspace) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || N < 1 || K < 1 || (long long)Z * N > (1ll << 30)) return PAI_ERR_BAD_SHAPE;
    if (row_begin < 0 || row_end > N || row_begin > row_end) return PAI_ERR_BAD_ROW_RANGE;
    if (!aligned(dO, 8) || !aligned(cos_sums, 4) || !aligned(sin_sums, 4) || !aligned(dk, 4) || !aligned(workspace, 16))
        return PAI_ERR_MISALIGNED;
    if (workspace_bytes < pai_we_bwd_dk_workspace_bytes(Z, N, K)) return PAI_ERR_WORKSPACE_TOO_SMALL;
    if (int e = require_sm100()) return e;
    if (row_begin == row_end) {
        cudaError_t e = cudaMemsetAsync(dk, 0, (size_t)K * sizeof(float), (cudaStream_t)stream);
        return (int)e;
    }
    return pai::we_bwd_launch(dO, cos_sums, sin_sums, dk, (float *)workspace, Z, N, K, row_begin, row_end,
                              (cudaStream_t)stream);
}

size_t pai_geoattn_plan_bytes(int Z, int N) {
    if (Z < 1 || N < 1) return 0;
    return pai::ga_plan_words(Z, N) * sizeof(int);
}

int pai_geoattn_plan(const uint8_t *valid, int Z, int N, void *plan, size_t plan_bytes, void *stream) {
    if (!valid || !plan) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || Z > 65535 || N < 1 || N > pai::GA_BN * pai::GA_MAX_TILES) return PAI_ERR_BAD_SHAPE;
    if (!aligned(plan, 16)) return PAI_ERR_MISALIGNED;
    if (plan_bytes < pai_geoattn_plan_bytes(Z, N)) return PAI_ERR_WORKSPACE_TOO_SMALL;
    if (int e = require_sm100()) return e;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce = cudaMemsetAsync(plan, 0, pai::GA_PLAN_HEADER * sizeof(int), st);  // the arrival counter starts at 0
    if (ce != cudaSuccess) return (int)ce;
    pai::geoattn_plan_kernel<<<Z, 256, 0, st>>>(valid, (int *)plan, Z, N);
    return (int)cudaPeekAtLastError();
}

size_t pai_geoattn_schedule_bytes(int Z, int N, int H, int bins) {
    if (Z < 1 || N < 1 || H < 1 || bins < 1 || bins > pai::GA_SCHED_MAX_BINS) return 0;
    return pai::ga_sched_words(Z, N, H, bins) * sizeof(int);
}

int pai_geoattn_schedule(const void *plan, int Z, int N, int H, int bins, int backward, void *sched, size_t sched_bytes, void *stream) {
    if (!plan || !sched) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || H < 1 || (long long)Z * H > 65535 || N < 1 || N > pai::GA_BN * pai::GA_MAX_TILES) return PAI_ERR_BAD_SHAPE;
    if (bins < 1 || bins > pai::GA_SCHED_MAX_BINS) return PAI_ERR_BAD_SHAPE;
    if (!aligned(plan, 16) || !aligned(sched, 16)) return PAI_ERR_MISALIGNED;
    if (sched_bytes < pai_geoattn_schedule_bytes(Z, N, H, bins)) return PAI_ERR_WORKSPACE_TOO_SMALL;
    if (int e = require_sm100()) return e;
    // cost of a work item in eighths of a (128 x 128) tile: the tiles it visits plus its set-up and epilogue
    // (measured: set-up, first loads and epilogue of an item take as long as 1.5 tiles in the backward, 0.6 in the forward)
    // (the forward runs two CTAs per SM and packs per SM; a single bin has no second CTA to pair with)
    pai::geoattn_schedule_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>((const int *)plan, (int *)sched, Z, N, H, bins, 8,
                                                                       backward ? 12 : 5, (backward || bins < 2) ? 0 : 1);
    return (int)cudaPeekAtLastError();
}

namespace {
// argument checks shared by the attention entry points; *qt0, *qt1: query tiles of the row range
int check_attn_common(int Z, int H, int N, int d, int logit_form, const float *betas, float min_rbf, float max_rbf,
                      const uint8_t *valid, const void *plan, int zh_begin, int zh_end, int q_begin, int q_end) {
    if (logit_form != 0 && logit_form != 1) return PAI_ERR_UNSUPPORTED;
    if (logit_form == 1 && !betas) return PAI_ERR_NULL_POINTER;
    if (logit_form == 1 && !(max_rbf > min_rbf)) return PAI_ERR_BAD_SHAPE;
    if (Z < 1 || H < 1 || N < 1 || (long long)Z * H > 65535 || N > pai::GA_BN * pai::GA_MAX_TILES) return PAI_ERR_BAD_SHAPE;
    if (d != pai::GA_D) return PAI_ERR_UNSUPPORTED;
    if (zh_begin < 0 || zh_end > Z * H || zh_begin > zh_end) return PAI_ERR_BAD_ROW_RANGE;
    if (q_begin < 0 || q_end > N || q_begin > q_end || (q_begin % pai::GA_BM) != 0 || (q_end != N && (q_end % pai::GA_BM) != 0))
        return PAI_ERR_BAD_ROW_RANGE;
    if (valid && !plan) return PAI_ERR_NULL_POINTER;  // a mask needs its plan
    if (plan && !aligned(plan, 16)) return PAI_ERR_MISALIGNED;
    return 0;
}
// the plan's longest-first order applies when the range covers whole samples from the first to the last
bool order_applies(const void *plan, int Z, int H, int zh_begin, int zh_end) {
    return plan != nullptr && zh_begin == 0 && zh_end == Z * H && g_tune[PAI_TUNE_GA_NO_ORDER] == 0;
}
// a schedule covers the whole problem: every (batch, head) pair and every query row
int check_sched(const void *plan, const void *sched, int sched_bins, int Z, int H, int N, int zh_begin, int zh_end, int q_begin, int q_end) {
    if (!sched) return 0;
    if (!plan) return PAI_ERR_NULL_POINTER;
    if (!aligned(sched, 16)) return PAI_ERR_MISALIGNED;
    if (sched_bins < 1 || sched_bins > pai::GA_SCHED_MAX_BINS) return PAI_ERR_BAD_SHAPE;
    if (zh_begin != 0 || zh_end != Z * H || q_begin != 0 || q_end != N) return PAI_ERR_BAD_ROW_RANGE;
    return 0;
}
}  // namespace

int pai_geoattn_fwd_strided(const void *Q, const int64_t *q_strides, const void *K, const int64_t *k_strides, const void *V,
                            const int64_t *v_strides, const float *coords, const float *sigma, const float *betas,
                            const uint8_t *valid, const void *plan, const void *sched, int sched_bins, void *O, const int64_t *o_strides,
                            float *L, int Z, int H,
                            int N, int d, float scale, float min_rbf, float max_rbf, int logit_form, int zh_begin, int zh_end,
                            int q_begin, int q_end, void *stream) {
    if (!Q || !K || !V || !coords || !sigma || !O || !L || !q_strides || !k_strides || !v_strides || !o_strides)
        return PAI_ERR_NULL_POINTER;
    if (int e = check_attn_common(Z, H, N, d, logit_form, betas, min_rbf, max_rbf, valid, plan, zh_begin, zh_end, q_begin, q_end))
        return e;
    if (int e = check_sched(valid ? plan : nullptr, sched, sched_bins, Z, H, N, zh_begin, zh_end, q_begin, q_end)) return e;
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16) || !aligned(coords, 4) ||
        !aligned(sigma, 4) || !aligned(L, 4))
        return PAI_ERR_MISALIGNED;
    for (const int64_t *st : {q_strides, k_strides, v_strides, o_strides})
        for (int a = 0; a < 3; ++a) {
            // rows are moved 16 bytes at a time; an axis of extent 1 may carry any stride (it is never stepped)
            const int extent = a == 0 ? Z : a == 1 ? H : N;
            if (st[a] < 0 || st[a] >= (1ll << 38)) return PAI_ERR_BAD_SHAPE;
            if ((st[a] & 7) != 0 && extent > 1) return PAI_ERR_MISALIGNED;
            if (st[a] < d && extent > 1) return PAI_ERR_BAD_SHAPE;  // rows of d elements must not overlap
        }
    if (int e = require_sm100()) return e;
    if (zh_begin == zh_end || q_begin == q_end) return PAI_OK;
    const int nzh = zh_end - zh_begin;
    auto stride_of = [&](const int64_t *st, int a, int extent) { return extent > 1 ? (long long)st[a] : (long long)d; };
    CUtensorMap mq, mk, mv;
    if (int e = pai::make_map_bf16_zhnd(&mq, Q, Z, H, N, d, stride_of(q_strides, 0, Z), stride_of(q_strides, 1, H),
                                        stride_of(q_strides, 2, N), pai::GA_BM))
        return e;
    if (int e = pai::make_map_bf16_zhnd(&mk, K, Z, H, N, d, stride_of(k_strides, 0, Z), stride_of(k_strides, 1, H),
                                        stride_of(k_strides, 2, N), pai::GA_BS))
        return e;
    if (int e = pai::make_map_bf16_zhnd(&mv, V, Z, H, N, d, stride_of(v_strides, 0, Z), stride_of(v_strides, 1, H),
                                        stride_of(v_strides, 2, N), pai::GA_BS))
        return e;
    const int smem = (int)sizeof(pai::GaFwdSmem) + 1024;
    static bool attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(pai::geoattn_fwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(pai::geoattn_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    pai::GaFwdParams p;
    p.coords = coords;
    p.valid = valid;
    p.plan = valid ? (const int *)plan : nullptr;
    p.sigma = sigma;
    p.out = (__nv_bfloat16 *)O;
    p.so_z = stride_of(o_strides, 0, Z);
    p.so_h = stride_of(o_strides, 1, H);
    p.so_n = stride_of(o_strides, 2, N);
    p.lse = L;
    p.Z = Z;
    p.H = H;
    p.N = N;
    p.zh_begin = zh_begin;
    p.q_begin = q_begin;
    p.use_order = order_applies(p.plan, Z, H, zh_begin, zh_end) ? 1 : 0;
    p.far_skip = g_tune[PAI_TUNE_GA_NO_FAR_SKIP] == 0 ? 1 : 0;
    p.scale = scale;
    p.form = logit_form;
    p.beta = betas;
    p.min_rbf = min_rbf;
    p.max_rbf = max_rbf;
    p.sched = (valid && g_tune[PAI_TUNE_GA_NO_ORDER] == 0) ? (const int *)sched : nullptr;
    dim3 grid((q_end - q_begin + pai::GA_BM - 1) / pai::GA_BM, nzh, 1);
    if (p.sched) grid = dim3(sched_bins, 1, 1);
    if (logit_form == 0) pai::geoattn_fwd_kernel<0><<<grid, pai::GA_FWD_THREADS, smem, (cudaStream_t)stream>>>(mq, mk, mv, p);
    else pai::geoattn_fwd_kernel<1><<<grid, pai::GA_FWD_THREADS, smem, (cudaStream_t)stream>>>(mq, mk, mv, p);
    return (int)cudaPeekAtLastError();
}

int pai_geoattn_fwd(const void *Q, const void *K, const void *V, const float *coords, const float *sigma,
                    const float *betas, const uint8_t *valid, const void *plan, const void *sched, int sched_bins, void *O, float *L,
                    int Z, int H, int N, int d, float scale, float min_rbf, float max_rbf, int logit_form, int zh_begin, int zh_end,
                    int q_begin, int q_end, void *stream) {
    const int64_t st[3] = {(int64_t)H * N * d, (int64_t)N * d, (int64_t)d};  // contiguous [Z,H,N,d]
    return pai_geoattn_fwd_strided(Q, st, K, st, V, st, coords, sigma, betas, valid, plan, sched, sched_bins, O, st, L, Z, H, N, d, scale,
                                   min_rbf, max_rbf, logit_form, zh_begin, zh_end, q_begin, q_end, stream);
}

size_t pai_geoattn_bwd_workspace_bytes(int Z, int H, int N, int d) {
    (void)d;
    if (Z < 1 || H < 1 || N < 1) return 0;
    return (size_t)Z * H * N * sizeof(float);
}

int pai_geoattn_bwd(const void *Q, const void *K, const void *V, const void *O, const void *dO, const float *L,
                    const float *coords, const float *sigma, const float *betas, const uint8_t *valid,
                    const void *plan, const void *sched, int sched_bins, float *dQ, float *dK, float *dV, float *dsigma, float *dbetas,
                    void *workspace,
                    size_t workspace_bytes, int Z, int H, int N, int d, float scale, float min_rbf, float max_rbf,
                    int logit_form, int zh_begin, int zh_end, int q_begin, int q_end, void *stream) {
    if (!Q || !K || !V || !O || !dO || !L || !coords || !sigma || !dQ || !dK || !dV || !dsigma || !workspace)
        return PAI_ERR_NULL_POINTER;
    if (logit_form == 1 && !dbetas) return PAI_ERR_NULL_POINTER;
    if (int e = check_attn_common(Z, H, N, d, logit_form, betas, min_rbf, max_rbf, valid, plan, zh_begin, zh_end, q_begin, q_end))
        return e;
    if (int e = check_sched(valid ? plan : nullptr, sched, sched_bins, Z, H, N, zh_begin, zh_end, q_begin, q_end)) return e;
    if (!aligned(Q, 16) || !aligned(K, 16) || !aligned(V, 16) || !aligned(O, 16) || !aligned(dO, 16) || !aligned(dQ, 16) ||
        !aligned(dK, 16) || !aligned(dV, 16) || !aligned(L, 4) || !aligned(coords, 4) || !aligned(sigma, 4) ||
        !aligned(dsigma, 4) || !aligned(workspace, 16))
        return PAI_ERR_MISALIGNED;
    if (workspace_bytes < pai_geoattn_bwd_workspace_bytes(Z, H, N, d)) return PAI_ERR_WORKSPACE_TOO_SMALL;
    if (int e = require_sm100()) return e;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t ce = cudaMemsetAsync(dsigma, 0, (size_t)H * sizeof(float), st);
    if (ce != cudaSuccess) return (int)ce;
    if (dbetas) {
        ce = cudaMemsetAsync(dbetas, 0, (size_t)H * sizeof(float), st);
        if (ce != cudaSuccess) return (int)ce;
    }
    if (zh_begin == zh_end) return PAI_OK;
    const int nzh = zh_end - zh_begin;
    const size_t rows0 = (size_t)zh_begin * N;
    const size_t off = rows0 * d * 2;
    CUtensorMap mq, mk, mv, mdo;
    if (int e = pai::make_map_bf16_rows(&mq, (const char *)Q + off, nzh, N, d, pai::GA_BM)) return e;
    if (int e = pai::make_map_bf16_rows(&mk, (const char *)K + off, nzh, N, d, pai::GA_BN)) return e;
    if (int e = pai::make_map_bf16_rows(&mv, (const char *)V + off, nzh, N, d, pai::GA_BN)) return e;
    if (int e = pai::make_map_bf16_rows(&mdo, (const char *)dO + off, nzh, N, d, pai::GA_BM)) return e;
    const int smem = (int)sizeof(pai::GaBwdSmem) + 1024;
    static bool attr_done[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        ce = cudaFuncSetAttribute(pai::geoattn_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (ce != cudaSuccess) return (int)ce;
        ce = cudaFuncSetAttribute(pai::geoattn_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (ce != cudaSuccess) return (int)ce;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    // pre-pass: D = rowsum(O * dO) and zeros into dQ, both over the query rows of the range
    float *dsum = (float *)workspace;
    if (q_end > q_begin) {
        const int q_rows = q_end - q_begin;
        const long long rows = (long long)nzh * q_rows;
        pai::geoattn_bwd_prep_kernel<<<(unsigned)((rows + 31) / 32), 256, 0, st>>>(
            (const __nv_bfloat16 *)O + rows0 * d, (const __nv_bfloat16 *)dO + rows0 * d, dsum, dQ + rows0 * d, N, q_begin, q_rows, rows);
    }
    pai::GaBwdParams p;
    p.coords = coords;
    p.valid = valid;
    p.sigma = sigma;
    p.lse = L;
    p.dsum = dsum;
    p.dq = dQ;
    p.dk = dK;
    p.dv = dV;
    p.dsigma = dsigma;
    p.dbeta = dbetas;
    p.form = logit_form;
    p.beta = betas;
    p.min_rbf = min_rbf;
    p.max_rbf = max_rbf;
    p.plan = valid ? (const int *)plan : nullptr;
    p.use_order = order_applies(p.plan, Z, H, zh_begin, zh_end) ? 1 : 0;
    p.far_skip = g_tune[PAI_TUNE_GA_NO_FAR_SKIP] == 0 ? 1 : 0;
    p.qt_begin = q_begin / pai::GA_BM;
    p.qt_end = (q_end + pai::GA_BM - 1) / pai::GA_BM;
    p.Z = Z;
    p.H = H;
    p.N = N;
    p.zh_begin = zh_begin;
    p.scale = scale;
    p.sched = (valid && g_tune[PAI_TUNE_GA_NO_ORDER] == 0) ? (const int *)sched : nullptr;
    dim3 grid((N + pai::GA_BN - 1) / pai::GA_BN, nzh, 1);
    if (p.sched) grid = dim3(sched_bins, 1, 1);
    if (p.form == 0) pai::geoattn_bwd_kernel<0><<<grid, pai::GA_BWD_THREADS, smem, st>>>(mq, mk, mv, mdo, p);
    else pai::geoattn_bwd_kernel<1><<<grid, pai::GA_BWD_THREADS, smem, st>>>(mq, mk, mv, mdo, p);
    return (int)cudaPeekAtLastError();
}

int pai_we_aniso_fwd(const float *coords_a_soa, const float *coords_b_soa, const uint8_t *valid, const float *cb_magnitudes,
                     const float *wavenumbers, float *out, float *d_cb, float *d_k, int Z, int N, int K, int row_begin,
                     int row_end, void *stream) {
    if (!coords_a_soa || !coords_b_soa || !cb_magnitudes || !wavenumbers || !out || !d_cb || !d_k) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || Z > 65535 || N < 1 || K < 1 || (long long)N * K > (1ll << 40)) return PAI_ERR_BAD_SHAPE;
    if (row_begin < 0 || row_end > N || row_begin > row_end) return PAI_ERR_BAD_ROW_RANGE;
    if (!aligned(coords_a_soa, 4) || !aligned(coords_b_soa, 4) || !aligned(cb_magnitudes, 4) || !aligned(wavenumbers, 4) ||
        !aligned(out, 4) || !aligned(d_cb, 4) || !aligned(d_k, 4))
        return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    if (row_begin == row_end) return PAI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t rows = (size_t)(row_end - row_begin), pitch = (size_t)N * 2 * K * sizeof(float), width = rows * 2 * K * sizeof(float);
    float *bufs[3] = {out, d_cb, d_k};
    for (float *b : bufs) {
        cudaError_t ce = cudaMemset2DAsync(b + (size_t)row_begin * 2 * K, pitch, 0, width, (size_t)Z, st);
        if (ce != cudaSuccess) return (int)ce;
    }
    int sms = 0;
    if (int e = current_device_sms(&sms)) return e;
    pai::WeAnisoParams p;
    p.coords_a = coords_a_soa;
    p.coords_b = coords_b_soa;
    p.valid = valid;
    p.cb = cb_magnitudes;
    p.wn = wavenumbers;
    p.out = out;
    p.d_cb = d_cb;
    p.d_k = d_k;
    p.N = N;
    p.K = K;
    p.row_begin = row_begin;
    p.row_end = row_end;
    p.use_tma = (aligned(coords_a_soa, 16) && aligned(coords_b_soa, 16) && (N % 4) == 0 && g_tune[PAI_TUNE_WE_NO_TMA] == 0) ? 1 : 0;
    unsigned *counter = nullptr;
    if (valid)
        if (int e = next_we_counter(&counter)) return e;
    return pai::we_aniso_fwd_launch(p, Z, sms, counter, st);
}

size_t pai_we_aniso_bwd_workspace_bytes(int Z, int N, int K) {
    (void)Z;
    (void)N;
    if (K < 1) return 0;
    return (size_t)pai::WE_BWD_MAX_BLOCKS * 2 * (size_t)K * sizeof(float);
}

int pai_we_aniso_bwd(const float *dO, const float *d_cb, const float *d_k, float *grad_cb, float *grad_wavenumbers, void *workspace,
                     size_t workspace_bytes, int Z, int N, int K, int row_begin, int row_end, void *stream) {
    if (!dO || !d_cb || !d_k || !grad_cb || !grad_wavenumbers || !workspace) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || N < 1 || K < 1 || (long long)Z * N > (1ll << 30)) return PAI_ERR_BAD_SHAPE;
    if (row_begin < 0 || row_end > N || row_begin > row_end) return PAI_ERR_BAD_ROW_RANGE;
    if (!aligned(dO, 8) || !aligned(d_cb, 8) || !aligned(d_k, 8) || !aligned(grad_cb, 4) || !aligned(grad_wavenumbers, 4) ||
        !aligned(workspace, 16))
        return PAI_ERR_MISALIGNED;
    if (workspace_bytes < pai_we_aniso_bwd_workspace_bytes(Z, N, K)) return PAI_ERR_WORKSPACE_TOO_SMALL;
    if (int e = require_sm100()) return e;
    cudaStream_t st = (cudaStream_t)stream;
    if (row_begin == row_end) {
        cudaError_t ce = cudaMemsetAsync(grad_cb, 0, (size_t)K * sizeof(float), st);
        if (ce != cudaSuccess) return (int)ce;
        return (int)cudaMemsetAsync(grad_wavenumbers, 0, (size_t)K * sizeof(float), st);
    }
    return pai::we_aniso_bwd_launch(dO, d_cb, d_k, grad_cb, grad_wavenumbers, (float *)workspace, Z, N, K, row_begin, row_end, st);
}

// ---- allocation-free variant of the WE backward --------------------------------------------------
// Scratch for the per-block partial sums lives in the library image instead of a caller buffer.
// Every GPU that loads the library carries this array (about 2.3 MiB) until the process exits.
#define PAI_WE_BWD_STATIC_MAX_K 1024
static __device__ __align__(256) float g_we_bwd_static_scratch[pai::WE_BWD_MAX_BLOCKS * PAI_WE_BWD_STATIC_MAX_K];

int pai_we_bwd_dk_static_max_k(void) { return PAI_WE_BWD_STATIC_MAX_K; }

int pai_we_bwd_dk_static(const float *dO, const float *cos_sums, const float *sin_sums, float *dk, int Z, int N, int K,
                         int row_begin, int row_end, void *stream) {
    if (!dO || !cos_sums || !sin_sums || !dk) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || N < 1 || K < 1 || (long long)Z * N > (1ll << 30)) return PAI_ERR_BAD_SHAPE;
    if (K > PAI_WE_BWD_STATIC_MAX_K) return PAI_ERR_EXCEEDS_STATIC_SCRATCH;
    if (row_begin < 0 || row_end > N || row_begin > row_end) return PAI_ERR_BAD_ROW_RANGE;
    if (!aligned(dO, 8) || !aligned(cos_sums, 4) || !aligned(sin_sums, 4) || !aligned(dk, 4)) return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    // The array's name is only a host-side handle here; the kernels need its device address, which
    // differs per GPU.  Looked up once per device, with that device current, and kept.
    static float *scratch_on_device[64];
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return (int)ce;
    if (dev < 0 || dev >= 64) return PAI_ERR_UNSUPPORTED;
    float *scratch = scratch_on_device[dev];
    if (!scratch) {
        ce = cudaGetSymbolAddress((void **)&scratch, g_we_bwd_static_scratch);
        if (ce != cudaSuccess) return (int)ce;
        if (!scratch) return PAI_ERR_UNSUPPORTED;
        scratch_on_device[dev] = scratch;
    }
    if (row_begin == row_end) {
        // nothing to sum: the result is zero; written by the final-pass kernel over zero partial rows
        pai::we_bwd_final_kernel<<<(K + pai::WE_BWD_THREADS - 1) / pai::WE_BWD_THREADS, pai::WE_BWD_THREADS, 0,
                                   (cudaStream_t)stream>>>(scratch, dk, K, 0);
        return (int)cudaPeekAtLastError();
    }
    // Pass 1 overwrites every partial row that pass 2 reads, so nothing in the array has to start at zero.
    return pai::we_bwd_launch(dO, cos_sums, sin_sums, dk, scratch, Z, N, K, row_begin, row_end, (cudaStream_t)stream);
}

int pai_add_layernorm_bf16(const void *x, const void *y, const void *gamma, const void *beta, int params_fp32, void *out,
                           long long rows, int D, float eps, void *stream) {
    if (!x || !gamma || !beta || !out) return PAI_ERR_NULL_POINTER;
    if (rows < 0 || D < 8 || (D & 7) != 0 || D > 4096 || !(eps >= 0.f)) return PAI_ERR_BAD_SHAPE;
    if (!aligned(x, 16) || (y && !aligned(y, 16)) || !aligned(out, 16) || !aligned(gamma, 16) || !aligned(beta, 16))
        return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    if (rows == 0) return PAI_OK;
    if ((rows + 7) / 8 > 0x7fffffffll) return PAI_ERR_BAD_SHAPE;
    return pai::add_layernorm_bf16_launch(x, y, gamma, beta, out, rows, D, eps, params_fp32 ? 1 : 0, (cudaStream_t)stream);
}

int pai_gelu_bf16(const void *x, void *out, long long n, void *stream) {
    if (!x || !out) return PAI_ERR_NULL_POINTER;
    if (n < 0 || (n & 7) != 0) return PAI_ERR_BAD_SHAPE;
    if (!aligned(x, 16) || !aligned(out, 16)) return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    if (n == 0) return PAI_OK;
    int sms = 0;
    if (int e = current_device_sms(&sms)) return e;
    return pai::gelu_bf16_launch(x, out, n, sms, (cudaStream_t)stream);
}

int pai_knn_neighbors(const float *ca, const uint8_t *valid, int64_t *idx, uint8_t *edge_mask, int Z, int N, int K, float max_dist,
                      void *stream) {
    if (!ca || !idx || !edge_mask) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || Z > 65535 || N < 1 || K < 1 || K > N || (long long)Z * N > (1ll << 31)) return PAI_ERR_BAD_SHAPE;
    if (K > pai::KNN_MAX_K) return PAI_ERR_UNSUPPORTED;
    if (!aligned(ca, 4) || !aligned(idx, 8)) return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    static_assert(sizeof(long long) == sizeof(int64_t), "index type");
    return pai::knn_launch(ca, valid, (long long *)idx, edge_mask, Z, N, K, max_dist, (cudaStream_t)stream);
}

int pai_edge_rbf(const float *atoms, const int64_t *idx, const float *centers, double spread, const float *ln_gamma,
                 const float *ln_beta, float ln_eps, float *out, int Z, int N, int K, int A, int R, void *stream) {
    if (!atoms || !idx || !centers || !out) return PAI_ERR_NULL_POINTER;
    if ((ln_gamma == nullptr) != (ln_beta == nullptr)) return PAI_ERR_NULL_POINTER;
    if (Z < 1 || N < 1 || K < 1 || A < 1 || R < 1 || A > 64 || R > 4096 || !(spread > 0.0) || !(ln_eps >= 0.f)) return PAI_ERR_BAD_SHAPE;
    if (ln_gamma && !(A == 4 && R == 16)) return PAI_ERR_UNSUPPORTED;
    if (!aligned(atoms, 4) || !aligned(idx, 8) || !aligned(centers, 4) || !aligned(out, 16)) return PAI_ERR_MISALIGNED;
    if (ln_gamma && (!aligned(ln_gamma, 16) || !aligned(ln_beta, 16))) return PAI_ERR_MISALIGNED;
    if (int e = require_sm100()) return e;
    int sms = 0;
    if (int e = current_device_sms(&sms)) return e;
    return pai::edge_rbf_launch(atoms, (const long long *)idx, centers, spread, ln_gamma, ln_beta, ln_eps, out, Z, N, K, A, R, sms,
                                (cudaStream_t)stream);
}

int pai_measure_sfu_peak(double *sincos_pairs_per_s, double *elapsed_ms) {
    if (!sincos_pairs_per_s || !elapsed_ms) return PAI_ERR_NULL_POINTER;
    if (int e = require_sm100()) return e;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int blocks = sms * 8, threads = 256, iters = 4096;
    cudaEvent_t a, b;
    cudaError_t e = cudaEventCreate(&a);
    if (e != cudaSuccess) return (int)e;
    e = cudaEventCreate(&b);
    if (e != cudaSuccess) {
        cudaEventDestroy(a);
        return (int)e;
    }
    sfu_peak_kernel<<<blocks, threads>>>(256, 0.5f);  // warm-up
    float best = 1e30f;
    for (int rep = 0; rep < 3; ++rep) {
        cudaEventRecord(a);
        sfu_peak_kernel<<<blocks, threads>>>(iters, 0.5f);
        cudaEventRecord(b);
        e = cudaEventSynchronize(b);
        if (e != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, a, b);
        if (ms < best) best = ms;
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    *elapsed_ms = best;
    *sincos_pairs_per_s = (double)blocks * threads * iters * 8.0 / (best * 1e-3);
    return PAI_OK;
}

// ---- test-only entries ---------------------------------------------------------------------------
int pai_tune_set(int key, int value) {
    if (key < 0 || key >= PAI_TUNE_COUNT) return PAI_ERR_UNSUPPORTED;
    g_tune[key] = value;
    return PAI_OK;
}

int pai_selftest_wait_timeout(void *stream) {
    if (int e = require_sm100()) return e;
    pai::selftest_wait_timeout_kernel<<<1, 64, 0, (cudaStream_t)stream>>>();
    return (int)cudaPeekAtLastError();
}

}  // extern "C"
