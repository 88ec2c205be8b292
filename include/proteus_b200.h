/*
 * proteus_b200 -- C ABI of the B200 (sm_100a) kernels for proteusAI's two hot paths:
 * the isotropic Wavefunction Embedding (WE) and the Geometric Attention.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current CUDA device unless stated otherwise;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - calls are asynchronous: they enqueue work on `stream` and return;
 *   - the caller allocates every buffer; the callee writes every element of the outputs it
 *     owns (rows of padded tokens are written as zeros), so outputs need no zero-fill;
 *   - return value: 0 = ok, negative = argument error (pai_status), positive = cudaError_t;
 *     nothing throws, aborts or traps across this boundary;
 *   - the library allocates no device memory.
 *
 * Each entry point cites the reference interface it replaces (path inside jaimec00/proteusAI).
 */
#ifndef PROTEUS_B200_H
#define PROTEUS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum pai_status {
    PAI_OK = 0,
    PAI_ERR_NULL_POINTER = -1,
    PAI_ERR_BAD_SHAPE = -2,
    PAI_ERR_MISALIGNED = -3,
    PAI_ERR_UNSUPPORTED = -4,
    PAI_ERR_WORKSPACE_TOO_SMALL = -5,
    PAI_ERR_BAD_ROW_RANGE = -6,
    PAI_ERR_NOT_SM100 = -7,
    PAI_ERR_DEVICE_WAIT_TIMEOUT = -8,
    PAI_ERR_EXCEEDS_STATIC_SCRATCH = -9
};

/* Bits of the `flags` argument of pai_we_fwd. */
enum pai_we_flags {
    PAI_WE_REPRODUCIBLE = 1 /* bit-identical sums from run to run (see pai_we_fwd) */
};

/* ABI version of this header (bumped on any signature change). */
int pai_abi_version(void);

/* Human-readable text for a value returned by any entry point (static storage). */
const char *pai_status_str(int status);

/* Synchronises `stream` and returns, then clears, the device-side status word of the
 * current device: PAI_OK, PAI_ERR_DEVICE_WAIT_TIMEOUT when a kernel gave up on a
 * bounded wait (it then wrote nothing further and returned), or PAI_ERR_BAD_SHAPE when an
 * attention launch was handed a schedule made for another problem (it did nothing). */
int pai_device_status(void *stream);

/* ---------------------------------------------------------------------------------------
 * Wavefunction Embedding, forward.
 * Replaces wf_embedding_kernel_forward()
 *   (utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding_kernel.cu:295-344), the function
 *   behind the pybind11 entry `wf_embedding_kernel.forward`
 *   (utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding_if.cpp:20-77).
 *
 *   coords_soa  [Z,3,N] fp32   coordinates, x/y/z planes (the reference's transposed layout)
 *   valid       [Z,N]   u8     1 = real token, 0 = padding; NULL = all valid
 *                              (replaces the reference's x == 12345 sentinel)
 *   wavenumbers [K]     fp32
 *   out         [Z,N,2K] fp32  interleaved: [2k] = sum_j mag*cos(k r_ij), [2k+1] = sum_j mag*sin(k r_ij)
 *   cos_sums    [Z,N,K] fp32   sum_j mag*r*cos(k r_ij)   (stored for the backward)
 *   sin_sums    [Z,N,K] fp32   sum_j mag*r*sin(k r_ij)
 *   row_begin,row_end          observer rows [row_begin,row_end) of every batch element are
 *                              computed and written; other rows are not touched (multi-GPU shard)
 *   magnitude_type             0: 1, 1: 1/r, 2: 1/log2(r), 3: 1/sqrt(r)
 *   dropout_p, seed            0 <= dropout_p < 1 (PAI_ERR_UNSUPPORTED otherwise).  With dropout_p > 0 single
 *                              (observer, source, wavenumber) evaluations are dropped as the reference kernel
 *                              does (wf_embedding_kernel.cu:27-46,227-232): a hash of (z, i, j, k, seed) mapped to
 *                              [0,1] keeps the evaluation when >= dropout_p; kept terms, in `out` and in both
 *                              stored sums, are scaled by 1/(1-dropout_p).  The same seed gives the same pattern
 *                              for any row range, shard or launch configuration.
 *   flags                      0, or PAI_WE_REPRODUCIBLE: by default the kernel cuts the work into equal runs that add
 *                              their partial sums into the outputs with fp32 reductions in arrival order, so the
 *                              last bit of a sum can differ from one launch to the next; with this flag every run
 *                              covers whole items, at most two runs touch an output element and the results are
 *                              bit-identical from launch to launch (a few per cent slower on small shards).  Other
 *                              bits: PAI_ERR_UNSUPPORTED.
 * Pairs with j == i, coincident points (r == 0) and padded tokens contribute nothing.
 * Requires 1 <= N, 1 <= K, 1 <= Z <= 65535.
 *
 * Launches with a padding mask draw their work from one of 256 four-byte counters inside the library image,
 * handed out round-robin per call (pai_we_aniso_fwd shares them).  Consequences for the caller:
 *   - more than 256 masked launches in flight at once on one device would share a counter and give wrong sums;
 *   - the first call on a device looks the counters up (cudaGetSymbolAddress), which is not allowed during stream
 *     capture: make one warm-up call per device before capturing;
 *   - a captured masked launch has its counter baked into the graph: do not let two replays of that graph (or a
 *     replay and more than 255 other masked launches) overlap in time.
 */
int pai_we_fwd(const float *coords_soa, const uint8_t *valid, const float *wavenumbers,
               float *out, float *cos_sums, float *sin_sums,
               int Z, int N, int K, int row_begin, int row_end,
               int magnitude_type, float dropout_p, uint32_t seed, uint32_t flags, void *stream);

/* ---------------------------------------------------------------------------------------
 * Wavefunction Embedding, backward w.r.t. the wavenumbers.
 * Replaces the PyTorch expression in _wf_embedding.backward
 *   (utils/model_utils/wf_embedding/isotropic/cuda/wf_embedding.py:64-83):
 *   dk[k] = sum_{z, n in [row_begin,row_end)} dO[z,n,2k+1]*cos_sums[z,n,k] - dO[z,n,2k]*sin_sums[z,n,k]
 *
 *   dO [Z,N,2K], cos_sums/sin_sums [Z,N,K], dk [K] (overwritten), all fp32.
 *   workspace: scratch of at least pai_we_bwd_dk_workspace_bytes(Z,N,K) bytes, 16-byte aligned;
 *   it holds per-block partial sums that a second pass adds in a fixed order (bit-reproducible).
 */
size_t pai_we_bwd_dk_workspace_bytes(int Z, int N, int K);
int pai_we_bwd_dk(const float *dO, const float *cos_sums, const float *sin_sums, float *dk,
                  void *workspace, size_t workspace_bytes,
                  int Z, int N, int K, int row_begin, int row_end, void *stream);

/* ---------------------------------------------------------------------------------------
 * Anisotropic Wavefunction Embedding with per-wavenumber C-beta scaling, forward.
 * Replaces wf_embedding_kernel_forward() of the variant the reference's model calls by default
 *   (utils/model_utils/wf_embedding/anisotropic/cb_scaling/learnable_wavenumbers/cuda/wf_embedding_kernel.cu,
 *   pybind entry in .../cuda/wf_embedding_if.cpp; Python side .../cuda/wf_embedding.py:16-64).
 *   Phase of wavenumber k for observer i, source j:  k * (r - s_k * (R/r . B_j)),  R = A_i - A_j, r = |R|.
 *
 *   coords_a_soa [Z,3,N] fp32   C-alpha coordinates, x/y/z planes
 *   coords_b_soa [Z,3,N] fp32   C-beta directions (unit vectors), x/y/z planes
 *   valid        [Z,N]   u8     1 = real token, 0 = padding; NULL = all valid
 *   cb_magnitudes [K], wavenumbers [K] fp32
 *   out          [Z,N,2K] fp32  interleaved sum_j cos(phase)/r, sum_j sin(phase)/r
 *   d_cb, d_k    [Z,N,2K] fp32  derivative of every output element w.r.t. s_k and w.r.t. k (kept for the backward)
 *   row_begin,row_end           as in pai_we_fwd
 */
int pai_we_aniso_fwd(const float *coords_a_soa, const float *coords_b_soa, const uint8_t *valid,
                     const float *cb_magnitudes, const float *wavenumbers, float *out, float *d_cb, float *d_k,
                     int Z, int N, int K, int row_begin, int row_end, void *stream);

/* Anisotropic Wavefunction Embedding, backward.  Replaces the PyTorch expressions in _wf_embedding.backward
 *   (.../learnable_wavenumbers/cuda/wf_embedding.py:66-79):
 *   grad_cb[k] = sum_{z,n} dO[z,n,2k] d_cb[z,n,2k] + dO[z,n,2k+1] d_cb[z,n,2k+1], and the same with d_k.
 *   workspace: at least pai_we_aniso_bwd_workspace_bytes(Z,N,K) bytes, 16-byte aligned; results are bit-reproducible. */
size_t pai_we_aniso_bwd_workspace_bytes(int Z, int N, int K);
int pai_we_aniso_bwd(const float *dO, const float *d_cb, const float *d_k, float *grad_cb, float *grad_wavenumbers,
                     void *workspace, size_t workspace_bytes, int Z, int N, int K, int row_begin, int row_end,
                     void *stream);

/* ---------------------------------------------------------------------------------------
 * Wavefunction Embedding, backward w.r.t. the wavenumbers, without any caller-provided scratch.
 * No counterpart in the reference: this entry point exists for callers that cannot allocate device
 * memory at the time of the call, for example a serving process that handed the whole GPU to its own
 * memory pool at start-up and treats any later cudaMalloc as an error, or code that runs where the
 * implicit device-wide synchronisation of cudaMalloc/cudaFree is not acceptable.  Such a caller has no
 * buffer to pass as `workspace` to pai_we_bwd_dk, so the partial sums go to an array that is part of
 * the library image.
 *
 * Same arguments, same arithmetic and same result as pai_we_bwd_dk minus (workspace, workspace_bytes).
 *   - Limit: K <= pai_we_bwd_dk_static_max_k() (1024, i.e. d_model <= 2048); a larger K returns
 *     PAI_ERR_EXCEEDS_STATIC_SCRATCH and nothing is launched.  Every GPU that loads the library holds the
 *     array (592 * 1024 floats, about 2.3 MiB) until the process exits, used or not.
 *   - The call itself performs no cudaMalloc, cudaFree or other allocation.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and keeps it; make that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps whatever the last call left in it.
 *     Nothing in it needs clearing between calls (each call overwrites every element it later reads),
 *     but two calls that overlap in time on the same GPU, e.g. on two streams, race on it and
 *     give wrong results: serialise them, or use pai_we_bwd_dk with separate workspaces.
 */
int pai_we_bwd_dk_static_max_k(void);
int pai_we_bwd_dk_static(const float *dO, const float *cos_sums, const float *sin_sums, float *dk,
                         int Z, int N, int K, int row_begin, int row_end, void *stream);

/* ---------------------------------------------------------------------------------------
 * Geometric attention: batch plan.
 * No counterpart in the reference, whose kernel walks every tile of the padded sequence
 *   (old/old_scripts/attn/geometric_attn.py:183-219).  The plan lists, per sample, the 128-token tiles that hold a
 *   valid token and orders the samples longest first; the attention kernels then never load a tile of padding and
 *   issue the long samples first.  One plan serves every call (all layers and heads, forward and backward) that
 *   uses the same mask; a call that passes `valid` must pass the plan made from it (with the same Z and N).
 *
 *   valid [Z,N] u8; plan: at least pai_geoattn_plan_bytes(Z,N) bytes, 16-byte aligned, written by the call.
 */
size_t pai_geoattn_plan_bytes(int Z, int N);
int pai_geoattn_plan(const uint8_t *valid, int Z, int N, void *plan, size_t plan_bytes, void *stream);

/* ---------------------------------------------------------------------------------------
 * Geometric attention: balanced schedule.
 * No counterpart in the reference, which launches one program per (query block, batch x head) pair
 *   (old/old_scripts/attn/geometric_attn.py:582-585).  The work items of the attention kernels, (sample, head, 128-token
 *   tile) triples, cost as much as their sample has non-empty tiles; with one CTA per item the SM that happens to get
 *   two long items finishes a third later than the average on a batch of mixed lengths.  A schedule assigns the
 *   items of a plan to `bins` persistent CTAs beforehand, longest first, each to the bin with the least work.
 *   One schedule serves every call with the same plan, H and direction.
 *
 *   plan       from pai_geoattn_plan (same Z, N)
 *   bins       CTAs of the launch, at most 1024: twice the SM count for the forward (two CTAs share an SM), the SM
 *              count for the backward
 *   backward   0: for pai_geoattn_fwd*, 1: for pai_geoattn_bwd (the fixed cost of an item differs)
 *   sched      at least pai_geoattn_schedule_bytes(Z,N,H,bins) bytes, 16-byte aligned, written by the call
 * The attention calls take the schedule as (sched, sched_bins); sched = NULL launches one CTA per item.  A schedule
 *   needs `valid` and its plan, and only applies to a call over the whole problem (zh_begin = 0, zh_end = Z*H,
 *   q_begin = 0, q_end = N): other ranges with a schedule are PAI_ERR_BAD_ROW_RANGE.
 *   A schedule made for another Z, N, H or number of CTAs is not followed: the launch does nothing and pai_device_status
 *   reports PAI_ERR_BAD_SHAPE.
 */
size_t pai_geoattn_schedule_bytes(int Z, int N, int H, int bins);
int pai_geoattn_schedule(const void *plan, int Z, int N, int H, int bins, int backward, void *sched, size_t sched_bytes,
                         void *stream);

/* ---------------------------------------------------------------------------------------
 * Geometric attention, forward.
 * Replaces the Triton launch `_attn_fwd[grid](...)` in _geometric_attn.forward
 *   (old/old_scripts/attn/geometric_attn.py:553-607; kernel :57-260).  Two logit forms:
 *   logit_form 0  SR_ij = S_ij * (1 + R_ij), the form of the reference README (README.md:40);
 *                 betas, min_rbf, max_rbf are ignored (betas may be NULL);
 *   logit_form 1  SR_ij = S_ij + beta_h * Rn_ij * |S_ij|, Rn = 2 (R - min_rbf) / (max_rbf - min_rbf) - 1, and pairs with
 *                 R outside [min_rbf, max_rbf] masked out: the form the reference tree's kernel and test implement
 *                 (geometric_attn.py:193-201, tests/attn/geo_attn.py:202-207);
 *   with S_ij = q_i.k_j * scale, R_ij = exp(-|r_i-r_j|^2 / (2 sigma_h^2)), softmax over the keys j, a pair (i,j) valid
 *   iff both tokens are unpadded.
 *
 *   Q, K, V  [Z,H,N,d] bf16, contiguous     (d must be 64; a caller with narrower heads zero-pads Q, K, V to 64 and
 *                                            passes the scale of the true width, as the Python wrapper does)
 *   coords   [Z,N,3]   fp32                 C-alpha coordinates
 *   sigma    [H]       fp32                 per-head RBF spread
 *   betas    [H]       fp32                 per-head RBF weight (logit_form 1)
 *   valid    [Z,N]     u8                   1 = real token, 0 = padding; NULL = all valid
 *   plan                                    from pai_geoattn_plan for this `valid` (required with `valid`, ignored without)
 *   sched, sched_bins                       from pai_geoattn_schedule(..., backward = 0), or NULL, 0
 *   O        [Z,H,N,d] bf16                 rows of padded queries are written as zeros (whatever Q, K, V hold there)
 *   L        [Z,H,N]   fp32                 log-sum-exp of SR over the keys (natural log); -inf for rows without a valid pair
 *   scale                                    softmax scale, 1/sqrt(d) in the reference
 *   zh_begin, zh_end                         only the (batch, head) pairs z*H + h in [zh_begin, zh_end) are
 *                                            computed and written (multi-GPU shard); other rows are not touched
 *   q_begin, q_end                           only the query rows [q_begin, q_end) of those pairs are computed and written
 *                                            (multi-GPU shard by query blocks, the reference grid's first axis,
 *                                            geometric_attn.py:582-585); q_begin a multiple of 128, q_end a multiple of
 *                                            128 or N.  Keys and values are always read in full.
 * bf16 x bf16 -> fp32 tensor-core products, fp32 softmax, P rounded to bf16 before P V.
 */
int pai_geoattn_fwd(const void *Q, const void *K, const void *V, const float *coords, const float *sigma,
                    const float *betas, const uint8_t *valid, const void *plan, const void *sched, int sched_bins,
                    void *O, float *L,
                    int Z, int H, int N, int d, float scale, float min_rbf, float max_rbf, int logit_form,
                    int zh_begin, int zh_end, int q_begin, int q_end, void *stream);

/* ---------------------------------------------------------------------------------------
 * Geometric attention, forward, on strided tensors.
 * The reference kernel takes a stride for every axis of Q, K, V and O (`_attn_fwd` arguments stride_Q_Z ... stride_O_D,
 *   old/old_scripts/attn/geometric_attn.py:58-62, passed from tensor.stride() at :588-591), so a caller can hand it
 *   views such as the [Z,H,N,d] permutation of a fused projection output [Z,N,3,H,d] without a copy.  Same here:
 *
 *   q_strides, k_strides, v_strides, o_strides   int64[3] on the host: element strides of the z, h and n axes; the d
 *                                                axis must be contiguous (stride 1).  Strides of axes longer than 1
 *                                                must be multiples of 8 elements (rows move 16 bytes at a time) and
 *                                                at least d.
 *   Everything else as in pai_geoattn_fwd, which is this call with the strides of a contiguous [Z,H,N,d] tensor.
 *   L is always contiguous [Z,H,N].
 */
int pai_geoattn_fwd_strided(const void *Q, const int64_t *q_strides, const void *K, const int64_t *k_strides,
                            const void *V, const int64_t *v_strides, const float *coords, const float *sigma,
                            const float *betas, const uint8_t *valid, const void *plan, const void *sched, int sched_bins,
                            void *O, const int64_t *o_strides, float *L,
                            int Z, int H, int N, int d, float scale, float min_rbf, float max_rbf, int logit_form,
                            int zh_begin, int zh_end, int q_begin, int q_end, void *stream);

/* ---------------------------------------------------------------------------------------
 * Geometric attention, backward.
 * Replaces _geometric_attn.backward (old/old_scripts/attn/geometric_attn.py:610-660): the PyTorch row-sum
 *   D = sum(O * dO) (:616) and the Triton launch `_attn_bwd[grid](...)` (:640-657; kernel :265-543), for the
 *   logit forms of pai_geoattn_fwd.
 *
 *   Q, K, V, O, dO [Z,H,N,d] bf16 contiguous (d must be 64); L [Z,H,N] fp32 as written by the forward
 *   dQ, dK, dV     [Z,H,N,d] fp32, like the reference's gradients (:626-628).  Of the (batch, head) range: every
 *                  row of dK and dV is written, and the rows [q_begin, q_end) of dQ; rows of padded tokens as zeros;
 *                  dQ is accumulated across key tiles with fp32 reductions, so its summation order is not fixed
 *   dsigma         [H] fp32, overwritten: gradient w.r.t. the spreads summed over the (batch, head) range
 *   dbetas         [H] fp32, overwritten: gradient w.r.t. betas (logit_form 1; may be NULL for logit_form 0)
 *   workspace      scratch of at least pai_geoattn_bwd_workspace_bytes(Z,H,N,d) bytes, 16-byte aligned
 *                  (holds D, one fp32 per query row)
 *   valid, plan, zh_begin, zh_end  as in the forward
 *   sched, sched_bins  from pai_geoattn_schedule(..., backward = 1), or NULL, 0
 *   q_begin, q_end only the query rows [q_begin, q_end) contribute: dK, dV, dsigma, dbetas are then partial sums
 *                  that the caller adds over the query shards (an all-reduce across ranks); same alignment rule
 */
size_t pai_geoattn_bwd_workspace_bytes(int Z, int H, int N, int d);
int pai_geoattn_bwd(const void *Q, const void *K, const void *V, const void *O, const void *dO, const float *L,
                    const float *coords, const float *sigma, const float *betas, const uint8_t *valid,
                    const void *plan, const void *sched, int sched_bins,
                    float *dQ, float *dK, float *dV, float *dsigma, float *dbetas,
                    void *workspace, size_t workspace_bytes,
                    int Z, int H, int N, int d, float scale, float min_rbf, float max_rbf, int logit_form,
                    int zh_begin, int zh_end, int q_begin, int q_end, void *stream);

/* ---------------------------------------------------------------------------------------
 * Row operations of the encoder block on either side of the attention kernel (bf16 in and out, fp32 arithmetic).
 * The reference runs them as PyTorch operators, so there is no reference FFI to replace:
 *   pai_add_layernorm_bf16   out[r,:] = LayerNorm(x[r,:] + y[r,:]) * gamma + beta, the post-norm steps
 *                            `norm(q + dropout(attn))` and `norm(q + dropout(ffn))` of Encoder.forward
 *                            (old/old_scripts/encoder.py:30-39) with dropout inactive, as one pass over the rows.
 *                            x, y, out [rows, D] bf16 (y may be NULL: plain LayerNorm; out may alias x or y);
 *                            gamma, beta [D] bf16, or fp32 when params_fp32 != 0; D a multiple of 8, at most 4096;
 *                            biased variance, eps inside the square root, as nn.LayerNorm.
 *   pai_gelu_bf16            out[i] = x[i] * Phi(x[i]), the erf form of GELU used by the reference MLP
 *                            (utils/model_utils/base_modules/base_modules.py:46-52, F.gelu); n a multiple of 8;
 *                            out may alias x.  Phi is evaluated to ~1e-7 absolute, below bf16 resolution.
 */
int pai_add_layernorm_bf16(const void *x, const void *y, const void *gamma, const void *beta, int params_fp32,
                           void *out, long long rows, int D, float eps, void *stream);
int pai_gelu_bf16(const void *x, void *out, long long n, void *stream);

/* ---------------------------------------------------------------------------------------
 * Nearest-neighbour graph and radial-basis edge features: FeaturizeProtein.get_neighbors and the tensor part of
 * FeaturizeProtein.get_edges (utils/model_utils/gnn/gnn.py:97-117 and :119-131), which the reference evaluates in
 * PyTorch through an N x N distance matrix, torch.topk and a [Z,N,K,4,4,R] broadcast (no reference FFI to replace).
 *
 * pai_knn_neighbors
 *   ca        [Z,N,3] fp32   C-alpha coordinates
 *   valid     [Z,N]   u8     1 = real node, 0 = masked (the inverse of the reference's node_mask); NULL = all real
 *   idx       [Z,N,K] i64    the K nearest nodes of each node in ascending order of distance (ties: lower index first);
 *                            an edge that is dropped points back at its own node, as in the reference
 *   edge_mask [Z,N,K] u8     1 = edge kept: both nodes real and distance < max_dist (12 in the reference)
 *   Candidates of a real node are all nodes at non-zero distance, masked ones included (their padding coordinates take
 *   part in the selection exactly as in the reference, and such edges are then dropped); a masked node gets itself K
 *   times and no edge.  Distances are rounded as PyTorch rounds them (fp32 differences, squares, sum in x, y, z order,
 *   IEEE square root).  Requires K <= N (the reference asserts it) and K <= 64.
 * pai_edge_rbf
 *   atoms     [Z,N,A,3] fp32  backbone atoms per node (A = 4 in the reference: N, C-alpha, C, C-beta)
 *   idx       [Z,N,K]   i64   neighbour indices (within the batch element), e.g. from pai_knn_neighbors
 *   centers   [R]       fp32  RBF centres; spread as the reference's Python float
 *   out       [Z,N,K,A*A*R] fp32  out[..., (a*A + b)*R + r] = exp(-(|atoms[z,i,a] - atoms[z,idx,b]| - centers[r])^2 / spread^2)
 *   ln_gamma, ln_beta [A*A*R] fp32, ln_eps   optional (both NULL = off): the LayerNorm over the features of each edge that
 *                             follows in the reference (`edge_norm`, gnn.py:134) applied before the store, so the features
 *                             cross HBM once; available for A = 4, R = 16 (PAI_ERR_UNSUPPORTED otherwise).
 */
int pai_knn_neighbors(const float *ca, const uint8_t *valid, int64_t *idx, uint8_t *edge_mask,
                      int Z, int N, int K, float max_dist, void *stream);
int pai_edge_rbf(const float *atoms, const int64_t *idx, const float *centers, double spread,
                 const float *ln_gamma, const float *ln_beta, float ln_eps, float *out,
                 int Z, int N, int K, int A, int R, void *stream);

/* ---------------------------------------------------------------------------------------
 * Measured SFU (MUFU) throughput of the current device: runs a register-only sin+cos loop and
 * returns results per second through *sincos_pairs_per_s (one pair = one sin and one cos, which is
 * what one WE evaluation needs) and the elapsed device time.  Synchronous.  Used as the
 * denominator of the WE roofline; has no counterpart in the reference.
 */
int pai_measure_sfu_peak(double *sincos_pairs_per_s, double *elapsed_ms);

/* ---------------------------------------------------------------------------------------
 * Test-only entries (no counterpart in the reference; not for production callers).
 *
 * pai_tune_set            sets a process-wide tuning knob of the kernels (launch geometry and kernel variants that
 *                         do not change results beyond rounding); the hot entry points read the knobs as plain
 *                         integers, there is no environment lookup anywhere.  Value 0 = the library's own choice
 *                         unless stated.  PAI_ERR_UNSUPPORTED for an unknown key.
 * pai_selftest_wait_timeout  launches one CTA whose warps wait, with a limit of a few thousand cycles, on an mbarrier
 *                         that nobody arrives on: exercises the path a kernel takes when a bounded device-side wait
 *                         runs out.  The kernel returns normally; afterwards pai_device_status() reports
 *                         PAI_ERR_DEVICE_WAIT_TIMEOUT once and the device is usable as before.
 */
enum pai_tune_key {
    PAI_TUNE_WE_KS = 0,           /* wavenumbers per lane: 2, 8 or 16 */
    PAI_TUNE_WE_TJ = 1,           /* sources per staged tile: multiple of 4 up to 512 */
    PAI_TUNE_WE_WAVES = 2,        /* runs per resident CTA slot */
    PAI_TUNE_WE_RANGE_REDUCE = 3, /* 1: explicit range reduction of the phase before the SFU */
    PAI_TUNE_WE_POLY_PAIRS = 4,   /* wavenumber pairs per lane evaluated on the FMA pipe (default 2) */
    PAI_TUNE_WE_NO_TMA = 5,       /* 1: plain loads instead of bulk copies for the source tiles */
    PAI_TUNE_GA_NO_FAR_SKIP = 6,  /* 1: evaluate the RBF of every key group, however far */
    PAI_TUNE_GA_NO_ORDER = 7,     /* 1: issue the samples in natural order instead of longest first */
    PAI_TUNE_WE_MIXED = 8,        /* 1: separate SFU and polynomial warps (we_fwd_mixed_kernel) instead of both pipes in every warp;
                                     measured 12 % slower at N = 16384, kept for comparison (default 0) */
    PAI_TUNE_COUNT = 9
};
int pai_tune_set(int key, int value);
int pai_selftest_wait_timeout(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* PROTEUS_B200_H */
