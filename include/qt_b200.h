/*
 * qt_b200.h -- C ABI of the B200 (sm_100a) quantize + scaled low-precision GEMM library.
 *
 * Every entry point takes plain device pointers, sizes, strides (in ELEMENTS) and a CUDA
 * stream handle (a cudaStream_t passed as void*; NULL = the legacy default stream). Nothing
 * here allocates device memory unless its comment says so; all launches are asynchronous on
 * the given stream. A return value of 0 means the work was enqueued; any other value is an
 * error code (QT_ERR_*) and qt_last_error() holds a human-readable message for the calling
 * thread. Pointers are borrowed for the duration of the enqueued work.
 *
 * The "replaces" notes cite the gau-nernst/quantized-training source (path:line inside that
 * project) whose behaviour the entry point reproduces.
 */
#ifndef QT_B200_H
#define QT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums ------------------------------------------------------------------------------ */

/* element types of tensors crossing the boundary */
enum {
    QT_BF16 = 0,    /* bfloat16 */
    QT_F32 = 1,     /* float    */
    QT_I8 = 2,      /* int8     */
    QT_E4M3 = 3,    /* float8 e4m3fn (finite, no inf; max 448) */
    QT_E5M2 = 4,    /* float8 e5m2   */
    QT_I32 = 5,     /* int32    */
    QT_F16 = 6      /* half     */
};

/* error codes */
enum {
    QT_OK = 0,
    QT_ERR_INVALID = 1,     /* bad argument: shape, stride, alignment, dtype      */
    QT_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed                */
    QT_ERR_UNSUPPORTED = 3, /* valid request outside what the kernels implement   */
    QT_ERR_DEVICE = 4       /* a kernel reported a bounded wait that ran out      */
};

/* ---- library -------------------------------------------------------------------------------- */

/* Message of the last error on the calling thread ("" if none). Never NULL. */
const char* qt_last_error(void);

/* Library version, e.g. "qt_b200 0.1 sm_100a". */
const char* qt_version(void);

/*
 * Reads and clears the device-side status word of the current device (synchronises the
 * device). 0 = no kernel has given up on a bounded wait since the last call. Non-zero values
 * encode (role << 8 | barrier id) of the wait that ran out.
 */
int qt_device_status(int* status_out);

/*
 * The same word without synchronising: kernels copy the code they record into a pinned host word, and
 * this reads that word. A non-zero value means some earlier GEMM gave up on a wait and its output is not
 * valid; a zero says nothing about kernels still running. Does not clear the word (qt_device_status
 * does). The Python operators call this after every GEMM launch and raise RuntimeError, the counterpart
 * of the reference's TORCH_CHECK failures (kernels/csrc/cutlass_sm89_fp8.cu:15-16,181) for a failure that
 * is only known once the kernel has run.
 */
int qt_device_status_peek(int* status_out);

/* ---- piece 1: absmax quantize ----------------------------------------------------------- */

/*
 * Row-wise symmetric absmax quantize.
 *   scale[r]  = max_c |x[r,c]| / qmax            (fp32 math; qmax = 127 for QT_I8, 448 for QT_E4M3)
 *   q[r,c]    = cast(round(x[r,c] / max(scale[r], eps)))   clamped to [-128,127] (int8) or [-448,448]
 * round = round-half-to-even, or floor(v + u) with u ~ U[0,1) from Philox4x32-10 keyed by
 * (seed, offset) when stochastic != 0 (int8 only).
 * x: [rows, cols], element (r,c) at x + r*x_row_stride + c, dtype x_dtype (QT_BF16 | QT_F32).
 * q: [rows, cols] contiguous. scale: [rows] of scale_dtype (QT_BF16 | QT_F32) -- the value
 * stored is the UNCLAMPED scale rounded to scale_dtype.
 * replaces: subclasses/int8.py:12-26 (quantize_int8 with dim=-1).
 */
int qt_quantize_rowwise(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                        void* q, int q_dtype, void* scale, int scale_dtype, float eps,
                        int stochastic, uint64_t seed, uint64_t offset, void* stream);

/*
 * qt_quantize_rowwise (round-half-even) fused with the all-gather of a row-sharded tensor: the rows of
 * this shard and their scales are written at row offset dst_row0 into n_dst gathered buffers
 * q_dst[d] ([total_rows, cols] contiguous) and scale_dst[d] ([total_rows]) -- this GPU's own buffer and
 * its peers' (device pointers into peer memory mapped into this process, e.g. the buffers of a symmetric
 * allocation; plain peer-to-peer stores over NVLink, no multicast). q_dst and scale_dst are HOST arrays
 * of n_dst <= 16 device pointers. The caller orders the consumers after every rank's kernel (a barrier
 * across the ranks on the same streams). bf16 input, rows 16-byte aligned, cols a multiple of 8 and at
 * most 32768; otherwise QT_ERR_UNSUPPORTED (quantize locally and use a library all-gather).
 * replaces: quantize_int8 of the FSDP2 shard followed by the all-gather of the reference's
 * fsdp_pre_all_gather (subclasses/bitnet.py:83-90 is its only instance); no kernel of the reference
 * writes to peer memory.
 */
int qt_quantize_rowwise_scatter(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                                int n_dst, void* const* q_dst, void* const* scale_dst, int64_t dst_row0,
                                int q_dtype, int scale_dtype, float eps, void* stream);

/*
 * Same as qt_quantize_rowwise and, in the same pass over x, the per-column absolute maximum
 * col_absmax[c] = max_r |x[r,c]| (fp32, [cols]). col_absmax is zeroed by this call (on the
 * stream) before the kernel runs. Lets a later qt_quantize_colwise_t skip its reduction pass.
 * replaces: the pair of quantize_int8 calls on one activation in
 * subclasses/mixed_precision.py:100-108,147-193 (row-wise in forward, column-wise in backward).
 */
int qt_quantize_rowwise_colabsmax(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                  int64_t x_row_stride, void* q, int q_dtype, void* scale,
                                  int scale_dtype, float* col_absmax, float eps, int stochastic,
                                  uint64_t seed, uint64_t offset, void* stream);

/*
 * Per-column absolute maximum: col_absmax[c] = max_r |x[r,c]| (fp32, [cols]); zeroed first.
 * replaces: the amax reduction of quantize_int8(x.T, dim=1), subclasses/int8.py:16.
 */
int qt_col_absmax(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                  float* col_absmax, void* stream);

/*
 * Column-wise quantize with the transpose materialised: for x [rows, cols],
 *   scale[c] = col_absmax[c] / qmax ; qt[c, r] = cast(round(x[r,c] / max(scale[c], eps)))
 * qt: [cols, rows] contiguous; scale: [cols]. col_absmax must hold the per-column absmax of x
 * (from qt_col_absmax or qt_quantize_rowwise_colabsmax).
 * The Philox counter of element (r,c) is that of the transposed element index c*rows + r, so
 * stochastic results equal qt_quantize_rowwise applied to a materialised transpose.
 * replaces: quantize_int8(B.T, sr, dim=1) followed by .contiguous(),
 * subclasses/mixed_precision.py:102-105.
 */
int qt_quantize_colwise_t(const void* x, int x_dtype, int64_t rows, int64_t cols,
                          int64_t x_row_stride, const float* col_absmax, void* qt, int q_dtype,
                          void* scale, int scale_dtype, float eps, int stochastic, uint64_t seed,
                          uint64_t offset, void* stream);

/*
 * The same column-wise quantization without the transpose: q [rows, cols] contiguous with
 * q[r][c] = round(x[r][c] / max(col_absmax[c] / qmax, eps)), scale [cols]. col_absmax is the caller's
 * (for a row-sharded weight: the element-wise maximum of every rank's qt_col_absmax, which makes the
 * gathered rows bit-identical to quantizing the whole weight). Stochastic rounding draws the uniform of
 * element r * cols + c.
 * replaces: quantize_int8(weight.T, dim=1) of the grad-input product (subclasses/mixed_precision.py:102
 * called from :176-178), applied per FSDP2 shard; the reference has no sharded form of it.
 */
int qt_quantize_colwise(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                        const float* col_absmax, void* q, int q_dtype, void* scale, int scale_dtype,
                        float eps, int stochastic, uint64_t seed, uint64_t offset, void* stream);

/*
 * qt_col_absmax + qt_quantize_colwise_t in one call that allocates nothing, for hosts that cannot
 * give this library memory at call time: a serving or training runtime that has already claimed the
 * whole device for its own pool (a cudaMalloc from a plugin would fail or fragment it), or a caller
 * inside a region where allocation is forbidden. The per-column absmax that the two-call form keeps
 * in a caller buffer lives in a fixed 256 KB array inside the library instead, so at most 65536
 * columns are accepted (more returns QT_ERR_UNSUPPORTED; use the two-call form with your own
 * buffer). x, qt and scale are still the caller's. No cudaMalloc / cudaFree or allocating library
 * routine is called.
 *   - The first call on each device looks up the array's device address (a one-time set-up step):
 *     make that first call outside any stream capture.
 *   - Every call on a device shares the one array: calls that may overlap on the GPU (different
 *     streams) race on it; keep them on one stream or serialise them. The array keeps the previous
 *     call's maxima between calls; each call clears the columns it uses before reducing into them.
 * Results are bit-identical to qt_col_absmax followed by qt_quantize_colwise_t.
 * No counterpart in the reference (its quantize is eager PyTorch and allocates freely).
 */
int qt_quantize_colwise_t_noalloc(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                  int64_t x_row_stride, void* qt, int q_dtype, void* scale,
                                  int scale_dtype, float eps, int stochastic, uint64_t seed,
                                  uint64_t offset, void* stream);

/*
 * Tile-wise absmax quantize: one scale per (tile_r x tile_c) tile of x [rows, cols];
 * scale is [ceil(rows/tile_r), ceil(cols/tile_c)] contiguous. tile_r in {1, 128}, tile_c = 128
 * (1x128 activations, 128x128 weights). Round-half-to-even only.
 * replaces: no function in the reference (its benchmark draws tile scales at random,
 * benchmark_mm.py:87-89); the arithmetic is quantize_int8's (subclasses/int8.py:15-25) per tile.
 */
int qt_quantize_tile(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t x_row_stride,
                     int tile_r, int tile_c, void* q, int q_dtype, void* scale, int scale_dtype,
                     float eps, void* stream);

/* ---- piece 2: tcgen05 GEMMs ----------------------------------------------------------------- */

/*
 * Operand addressing for all GEMMs: A is [M,K] with element (m,k) at a + m*a_sm + k*a_sk and B is
 * [K,N] with element (k,n) at b + k*b_sk + n*b_sn. Exactly one stride of each operand must be 1:
 *   a_sk == 1 : A row-major (K-major)        a_sm == 1 : A column-major (M-major)
 *   b_sk == 1 : B column-major (K-major)     b_sn == 1 : B row-major (N-major)
 * so A@B.T is (a_sk=1,b_sk=1), A@B is (a_sk=1,b_sn=1), A.T@B is (a_sm=1,b_sn=1).
 * The non-unit stride must be a multiple of 16 and the base pointers 16-byte aligned (TMA).
 * C is [M,N] row-major with row stride ldc (elements).
 */

/*
 * How many CTAs cooperate on one MMA in the GEMMs below: 0 = chosen per problem (a 2-CTA pair
 * sharing a 256 x 256 tile when M > 128 and the reduction is at least 512 bytes long, else one CTA per
 * 128 x 256 tile), 1 or 2 = forced.
 * Process-wide; meant for tests and tuning. Results are identical either way for int8.
 * No counterpart in the reference (Triton autotunes its own tile shapes, triton_mm.py:9-43).
 */
int qt_set_gemm_cta_group(int cta_group);

/*
 * Rasterisation of the persistent GEMM grids: `group_m` row-tiles sweep all column-tiles before the next group
 * starts, so the group's A panel stays in L2 while B streams past once per group. 0 = the default of 8,
 * otherwise forced. Process-wide; for tests and tuning.
 * Results do not depend on it. No counterpart in the reference (Triton's kernels use a fixed GROUP_M = 8,
 * kernels/gn_kernels/triton_mm.py:66,72-77).
 */
int qt_set_gemm_group_m(int group_m);

/*
 * Number of SMs the persistent GEMM grids leave unused (default 0), so that a kernel which has to
 * run at the same time -- an NCCL collective prefetching the next weight -- finds free SMs instead
 * of queueing behind a grid that holds every SM until it finishes. Process-wide.
 * No counterpart in the reference (it leaves overlap to FSDP2's streams and Triton's non-persistent grids).
 */
int qt_set_gemm_sm_margin(int sms);

/*
 * C(int32) = A(int8) @ B(int8), exact.
 * replaces: gn_kernels int8_mm, kernels/gn_kernels/triton_mm.py:112-128 (_matmul_kernel :53-109).
 */
int qt_int8_mm(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn,
               int32_t* c, int64_t ldc, int64_t M, int64_t N, int64_t K, void* stream);

/*
 * C = cast( (fp32(A @ B) * scale_a[m]) * scale_b[n] ) with A, B both int8 (int32 accumulate) or
 * both fp8 (ab_dtype QT_E4M3 / QT_E5M2 per operand, fp32 accumulate). scale_a: [M]; scale_b: [N],
 * or one element when bit 0 of scale_b_is_scalar is set. Bit 1 of scale_b_is_scalar swaps the order of
 * the two multiplications to (acc * scale_b[n]) * scale_a[m]: a product computed in transposed form
 * (C^T = B^T A^T, e.g. a grad-weight written directly in the weight's layout) then rounds exactly like the
 * untransposed one. Scales and C share scale_dtype (QT_BF16 | QT_F32).
 * replaces: gn_kernels scaled_mm, kernels/gn_kernels/triton_mm.py:345,349-373,382-407
 * (_scaled_mm_kernel :146-220).
 */
int qt_scaled_mm(const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b, int b_dtype,
                 int64_t b_sk, int64_t b_sn, const void* scale_a, const void* scale_b,
                 int scale_b_is_scalar, int scale_dtype, void* c, int64_t ldc, int64_t M, int64_t N,
                 int64_t K, void* stream);

/*
 * C = bf16( bf16(A @ B^T) * col_scale[n] ) for bf16 A [M, K] (row pitch lda) and B [N, K] (row pitch ldb), bf16
 * col_scale [N], bf16 C: a bf16 matmul (fp32 accumulate on tcgen05 kind::f16, rounded to bf16) followed by
 * the bf16 multiply with a per-column scale, fused into the epilogue with both roundings kept. K, lda and ldb
 * multiples of 8.
 * replaces: the INT8 weight-only forward `(input @ weight.int_data.T.to(input.dtype)) * weight.scale.T`
 * (subclasses/int8.py:147) once the int8 weight has been widened to bf16 (exact): the reference runs it as a
 * bf16 cuBLAS matmul plus an element-wise multiply over the output.
 */
int qt_bf16_mm_colscale(const void* a, int64_t lda, const void* b, int64_t ldb, const void* col_scale, void* c,
                        int64_t ldc, int64_t M, int64_t N, int64_t K, void* stream);

/*
 * Split-K forms. When the output is small and the reduction long (the grad-weight GEMMs: a
 * [hidden, hidden] result reduced over tens of thousands of tokens) there are too few output tiles
 * to occupy the GPU; given a workspace, these variants let several CTA pairs share one tile, each
 * reducing a slice of K into a raw partial plane, and a finishing kernel sums the planes and applies
 * the epilogue. int8 results stay bit-identical (integer partials add exactly); fp8 partials add in
 * fp32. qt_gemm_workspace_bytes returns the bytes the library would like for (M, N, K): 0 means no
 * split would be used. A null, misaligned (32 bytes) or too-small workspace falls back to the
 * unsplit kernel. The workspace contents are undefined afterwards.
 * No counterpart in the reference (Triton's kernels there never split K).
 */
int64_t qt_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int qt_int8_mm_ws(const void* a, int64_t a_sm, int64_t a_sk, const void* b, int64_t b_sk, int64_t b_sn,
                  int32_t* c, int64_t ldc, int64_t M, int64_t N, int64_t K, void* workspace,
                  int64_t workspace_bytes, void* stream);
int qt_scaled_mm_ws(const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b, int b_dtype,
                    int64_t b_sk, int64_t b_sn, const void* scale_a, const void* scale_b,
                    int scale_b_is_scalar, int scale_dtype, void* c, int64_t ldc, int64_t M, int64_t N,
                    int64_t K, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Tile-scaled GEMM: for each block kb of qk reduction elements
 *   acc[m,n] += fp32(A[m,kb] @ B[kb,n]) * scale_a[m/qm, kb] * scale_b[kb, n/qn]
 * scale_a: [ceil(M/qm), K/qk] with strides (sa_s0, sa_s1); scale_b: [K/qk, ceil(N/qn)] with strides
 * (sb_s0, sb_s1). Supported: qk a multiple of 128 with K % qk == 0, any qm >= 1, qn one of 16, 32, 64
 * or a multiple of 128 (the reference benchmark's 1x128 activation / 128x128 weight tiles,
 * benchmark_mm.py:87-89, take the fastest instantiation); other shapes return QT_ERR_UNSUPPORTED. The per-block term is evaluated as one fused multiply-add with
 * the product of the two scales, so results agree with the reference's two multiplies to rounding.
 * replaces: gn_kernels tile_scaled_mm, kernels/gn_kernels/triton_mm.py:346,410-441
 * (_tile_scaled_mm_kernel :223-342).
 */
int qt_tile_scaled_mm(const void* a, int a_dtype, int64_t a_sm, int64_t a_sk, const void* b,
                      int b_dtype, int64_t b_sk, int64_t b_sn, const void* scale_a, int64_t sa_s0,
                      int64_t sa_s1, const void* scale_b, int64_t sb_s0, int64_t sb_s1, int qm, int qn,
                      int qk, int scale_dtype, void* c, int64_t ldc, int64_t M, int64_t N, int64_t K,
                      void* stream);

/* ---- BitNet b1.58 weight path ------------------------------------------------------------------ */

/*
 * out[0] = mean(|x|) in fp32 over numel elements (deterministic two-stage reduction).
 * workspace: caller-provided scratch of at least 8192 bytes, 8-byte aligned; contents undefined
 * afterwards. replaces: get_bitnet_scale, subclasses/bitnet.py:110-112.
 */
int qt_abs_mean(const void* x, int x_dtype, int64_t numel, float* out, void* workspace,
                int64_t workspace_bytes, void* stream);

/*
 * Ternary weight quantize: q = clip(round_half_even(w / max(scale[0], eps)), -1, 1), scale a device
 * fp32 scalar. pack_2bit == 0: out is int8 [numel]. pack_2bit != 0: out is int8 [numel/4], four
 * 2-bit two's-complement values per byte, the first in the top bits (numel % 4 == 0; rows of a
 * [N,K] weight pack along K when K % 4 == 0).
 * replaces: quantize_bitnet_weight + _pack_i2_in_i8, subclasses/bitnet.py:115-118,185-195.
 */
int qt_bitnet_quantize_weight(const void* w, int w_dtype, int64_t numel, const float* scale, float eps,
                              void* out, int pack_2bit, void* stream);

/*
 * Inverse of the 2-bit packing: int8 [numel_packed] -> int8 [4 * numel_packed], sign-extended.
 * replaces: _unpack_i2_in_i8, subclasses/bitnet.py:198-201.
 */
int qt_unpack_i2(const void* packed, int64_t numel_packed, void* out, void* stream);

/* ---- optimizer ------------------------------------------------------------------------------- */

/*
 * One AdamW step on one parameter tensor with bf16 states: fp32 math, states written back in bf16,
 * a bf16 parameter written back with stochastic rounding (bits + 16 random bits, truncated) when
 * stochastic != 0, otherwise round-to-nearest; an fp32 parameter is written back as is.
 * beta1/beta2 are doubles because the reference forms the lerp weight (1 - beta) in double before
 * it is rounded to fp32. bias_correction1 = 1 - beta1^step and sqrt_bias_correction2 =
 * sqrt(1 - beta2^step) are computed by the caller in fp32. exp_avg / exp_avg_sq are bf16 [numel].
 * Tensors are contiguous; 16-byte aligned ones move four elements per access, others one (same values).
 * replaces: other_optim/bf16_sr.py:78-124 (adamw), called per parameter from AdamWBF16SR.step :30-75.
 */
int qt_adamw_bf16_sr(void* p, int p_dtype, const void* grad, int grad_dtype, void* exp_avg,
                     void* exp_avg_sq, int64_t numel, float lr, double beta1, double beta2,
                     float weight_decay, float eps, float bias_correction1,
                     float sqrt_bias_correction2, int stochastic, uint64_t seed, uint64_t offset,
                     void* stream);

/*
 * In-place optimizer update of an INT8 weight [rows, cols] with bf16 per-row scales [rows]: what the
 * reference does in three eager steps -- de-quantize, add_/addcdiv_, re-quantize row-wise with
 * stochastic rounding and copy back (subclasses/int8.py:114-133) -- in one pass that reads q, scale and
 * the operands once and overwrites q and scale:
 *   w = bf16(float(q) * scale[row])
 *   mode 0: y = bf16(w + value * t1)              (add_(t1, alpha=value))
 *   mode 1: y = bf16(w + value * (t1 / t2))       (addcdiv_(t1, t2, value=value))
 *   q, scale <- stochastic row-wise INT8 quantization of y, random bits of (seed, offset) exactly as
 *   qt_quantize_rowwise draws them for a contiguous [rows, cols] tensor.
 * t1, t2: contiguous bf16 [rows, cols] (t2 unused in mode 0). Needs cols % 8 == 0, cols <= 32768,
 * q 8-byte and t1/t2 16-byte aligned: otherwise QT_ERR_UNSUPPORTED and the caller runs the three steps.
 */
int qt_int8_weight_update(void* q, void* scale, int64_t rows, int64_t cols, int mode, const void* t1,
                          const void* t2, float value, float eps, uint64_t seed, uint64_t offset,
                          void* stream);

/*
 * The same update for n_tensors parameter tensors in as few launches as possible (a launch covers up
 * to 160 tensors, 8192 elements per block). p, grad, exp_avg, exp_avg_sq and numel are HOST
 * arrays of n_tensors device pointers / lengths; all tensors share the dtypes and the scalars (the
 * reference steps every parameter of a group with the same hyper-parameters, other_optim/
 * bf16_sr.py:37-74, and launches one compiled kernel per parameter). Tensor t gets exactly the result
 * of qt_adamw_bf16_sr(..., seed, offset + t, ...). Tensors of length 0 are skipped.
 */
int qt_adamw_bf16_sr_multi(int n_tensors, void* const* p, const void* const* grad, void* const* exp_avg,
                           void* const* exp_avg_sq, const int64_t* numel, int p_dtype, int grad_dtype,
                           float lr, double beta1, double beta2, float weight_decay, float eps,
                           float bias_correction1, float sqrt_bias_correction2, int stochastic,
                           uint64_t seed, uint64_t offset, void* stream);

/* ---- producer-fused activation quantize ------------------------------------------------------------ */

/*
 * RMSNorm with the activation quantize of the following INT8 linear layers folded in: one pass over x
 * writes y = weight * bf16(x * rstd) (rstd = 1 / sqrt(mean(x^2) + norm_eps), the arithmetic of an eager
 * RMSNorm module on bf16 input), rstd per row (may be NULL), and -- when q is not NULL -- the row-wise
 * quantization of y exactly as qt_quantize_rowwise_colabsmax(y) would produce it: q, scale and the
 * per-column |y| maxima (zeroed here, reached by atomic max). x, y bf16; y is [rows, cols] contiguous.
 * Needs 16-byte aligned rows, cols a multiple of 8 and at most 16384, rows a multiple of the rows one
 * CTA holds at that width (8 up to 1024 columns, 4 / 2 / 1 for up to 2048 / 4096 / more): otherwise
 * QT_ERR_UNSUPPORTED and the caller runs the norm and the quantize separately.
 * replaces: nothing the reference has as a kernel. It is the fusion its source names as the open
 * optimisation ("output is not quantized ... optimization opportunity", subclasses/int8.py:155-156):
 * RMSNorm (a module of the model, compiled by torch.compile at llm_pretrain.py:138) followed by
 * quantize_int8 (subclasses/int8.py:12-26) at the entry of _Int8MixedPrecisionLinear.forward
 * (subclasses/mixed_precision.py:146-160).
 */
int qt_rmsnorm_quantize(const void* x, int64_t rows, int64_t cols, int64_t x_row_stride, const void* weight,
                        float norm_eps, void* y, float* rstd, void* q, int q_dtype, void* scale,
                        int scale_dtype, float* col_absmax, float eps, void* stream);

/*
 * Number of rows of fp32 scratch ([partial_rows, cols]) qt_rmsnorm_backward needs for a [rows, cols] input.
 */
int64_t qt_rmsnorm_backward_partial_rows(int64_t rows, int64_t cols);

/*
 * Backward of the RMSNorm above: dx = rstd * (g - n * mean(g * n)) with g = dy * weight, n = x * rstd, and
 * dweight[c] = sum over rows of dy * bf16(n), all in fp32 from the bf16 inputs; dx bf16 [rows, cols]
 * contiguous, dweight [cols] of dweight_dtype (QT_BF16 | QT_F32). dw_partial is caller-provided scratch
 * whose rows are summed in a fixed order (results do not depend on scheduling). Same shape limits as the
 * forward, any row count.
 * replaces: the autograd backward of the model's RMSNorm module (no kernel of the reference).
 */
int qt_rmsnorm_backward(const void* dy, int64_t dy_row_stride, const void* x, int64_t x_row_stride,
                        const void* weight, const float* rstd, int64_t rows, int64_t cols, void* dx,
                        float* dw_partial, int64_t partial_rows, void* dweight, int dweight_dtype, void* stream);

/*
 * y = bf16(bf16(silu(gate)) * up), the gated activation of a SwiGLU MLP, with the quantize of the
 * following INT8 linear layer folded in like qt_rmsnorm_quantize (q, scale, col_absmax; q may be NULL).
 * gate, up, y bf16; same shape limits.
 * replaces: act_fn(gate_proj(x)) * up_proj(x) of the model's MLP followed by quantize_int8 at the entry
 * of the down projection (subclasses/mixed_precision.py:146-160, subclasses/int8.py:155-156).
 */
int qt_silu_mul_quantize(const void* gate, const void* up, int64_t rows, int64_t cols, int64_t gate_row_stride,
                         int64_t up_row_stride, void* y, void* q, int q_dtype, void* scale, int scale_dtype,
                         float* col_absmax, float eps, void* stream);

/*
 * Backward of the gated activation: dup = dh * bf16(silu(gate)), dgate = dh * up * d silu(gate), fp32
 * arithmetic, bf16 out ([rows, cols] contiguous). 16-byte aligned rows, cols a multiple of 8.
 * replaces: the autograd backward of the model's MLP activation (no kernel of the reference).
 */
int qt_silu_mul_backward(const void* dh, int64_t dh_row_stride, const void* gate, int64_t gate_row_stride,
                         const void* up, int64_t up_row_stride, int64_t rows, int64_t cols, void* dgate,
                         void* dup, void* stream);

/*
 * Rotary position embedding of x [tokens, heads, head_dim] (bf16, contiguous) with cos / sin
 * [batch or 1, seq_len, head_dim] (bf16; cos_batch_stride = 0 when one table serves every sequence):
 * y1 = x1 * cos1 - x2 * sin1, y2 = x2 * cos2 + x1 * sin2 over the two halves of each head; inverse != 0
 * applies the transpose (the backward pass). head_dim a multiple of 16.
 * replaces: apply_rotary_pos_emb of the model code the reference trains (transformers' Llama, compiled by
 * llm_pretrain.py:138); no kernel of the reference.
 */
int qt_rope(const void* x, int64_t tokens, int heads, int head_dim, const void* cos, const void* sin,
            int64_t seq_len, int64_t cos_batch_stride, int inverse, void* y, void* stream);

/* ---- self-tests ------------------------------------------------------------------------------ */

/*
 * Exhaustive check of the quantize kernels' bf16 division (correctly rounded reciprocal + one
 * fused correction) against IEEE division, over every finite bf16 absmax a >= 0 and every bf16 x
 * with |x| <= a, for d = max(a / qmax(q_dtype), eps). mismatches[0] = quotients that differ in any
 * bit, mismatches[1] = quantized bytes that differ. Allocates 16 bytes of device memory and
 * synchronises the device. Test utility; no counterpart in the reference.
 */
int qt_selftest_division(int q_dtype, float eps, unsigned long long* mismatches);

/*
 * Exercises the bounded-wait path of the GEMM kernels without a GEMM: one warp waits on an mbarrier
 * that nothing arrives on, gives up after 50 ms, records the code 0x7E57 in the device status word
 * and returns. *observed_status receives the word (0x7E57 when the mechanism works); the word is reset
 * to zero before the call returns unless leave_set is non-zero (then the next qt_device_status call
 * clears it). Fails if the word was already set. Synchronises the device.
 * Test utility; no counterpart in the reference.
 */
int qt_selftest_wait_timeout(int* observed_status, int leave_set);

#ifdef __cplusplus
}
#endif
#endif /* QT_B200_H */
