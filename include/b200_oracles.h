/*
 * C ABI of libb200_oracles.so: hand-written sm_100a CUDA kernels for the memory-bound fused
 * regions of the better-benchmark corpus (row/column reductions, softmax, LayerNorm / RMSNorm /
 * BatchNorm forward and backward, permutes with pointwise epilogues).
 *
 * The reference has no native code: each fused region is a Python function
 *     oracle_forward(inputs, **launch_kwargs)            (oracle_harness.py:1777-1779)
 * in repros/canonical/<id>/oracle.py that launches Triton kernels on torch tensors. An entry
 * point below is what such a function binds instead; the comment on each names the Triton
 * kernels it replaces (paths inside the reference repository).
 *
 * Conventions
 *   - All pointers are device pointers; sizes and strides are in ELEMENTS unless a name says
 *     bytes. Nothing is allocated, freed or synchronised; every launch goes to `stream`
 *     (a cudaStream_t passed as void*), so calls may be captured into a CUDA graph.
 *   - dtype codes: 0 = float32, 1 = bfloat16, 2 = float16.
 *   - Return value: 0 on success; < 0 an argument error found before anything was launched
 *     (B200_ERR_*); > 0 the cudaError_t of a rejected launch. b200_last_error() returns the text
 *     of the calling thread's last failure.
 *   - Kernels that combine per-CTA partial results take a caller-provided `scratch` buffer
 *     (16-byte aligned). Its first 256 bytes hold grid-barrier words that must be zero before
 *     the first use; every kernel leaves them zero. Concurrent launches on different streams
 *     need different scratch buffers.
 *   - Accumulation is fp32 (fp64 where partial results of many CTAs are combined), no fast-math,
 *     no fused multiply-add contraction; reductions have a fixed order (bit-reproducible).
 */
#ifndef B200_ORACLES_H
#define B200_ORACLES_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_F32 0
#define B200_BF16 1
#define B200_F16 2

#define B200_OK 0
#define B200_ERR_INVALID -1
#define B200_ERR_UNSUPPORTED -2
#define B200_ERR_ALIGNMENT -3
#define B200_ERR_WORKSPACE -4
#define B200_ERR_DEVICE_WAIT -5

/* Text of the calling thread's last error ("" if none). Python exceptions in the reference
 * (oracle_harness.py:1116-1125, scripts/bench_parallel.py:3115-3118) map onto this. */
const char* b200_last_error(void);

/* ABI version of this library. */
int32_t b200_version(void);

/* Multiprocessor count and L2 size of the current device. The reference reads the same facts
 * through torch in oracle_harness.get_hardware_info (oracle_harness.py:46-56). */
int32_t b200_sm_count(void);
int32_t b200_l2_bytes(void);

/* Kernels launched by this library in this process so far. No counterpart in the reference; the
 * benchmark reports the count of launches inside its timed region. */
int64_t b200_launch_count(void);

/* Name of the kernel the calling thread launched last, with the variant its launcher chose in
 * brackets ("b200_row_reduce [vector, warp per row]"); "" before the first launch. No counterpart
 * in the reference (its oracle files name their Triton kernels in source); sweep reports use it to
 * tell the tuned paths from the element-wise ones. */
const char* b200_last_kernel(void);

/* Reads the status words of a scratch buffer; returns B200_ERR_DEVICE_WAIT if a grid-wide wait
 * inside a cooperative kernel ran out. Synchronises `stream`: diagnostic use only. No
 * counterpart in the reference (its kernels never wait on one another). */
int32_t b200_check_status(const void* scratch, void* stream);

/* Row reduction over the last (unit-stride) dimension: op 0 sum, 1 mean, 2 amax, 3 amin.
 * x is [rows, n] with rows = d0*d1*d2 addressed through x_strides[3] (row = (i0*d1+i1)*d2+i2);
 * out[row * out_stride] has dtype out_dtype.
 * Replaces repros/canonical/mean_c9e1a8113328/oracle.py:11-76 (contiguous case) and the row
 * max/sum loops of amax_sum_7079889cfc04/oracle.py:20-29. */
int32_t b200_row_reduce(const void* x, void* out, int64_t rows, int64_t n, int64_t d1, int64_t d2,
                        const int64_t* x_strides, int64_t out_stride, int32_t x_dtype,
                        int32_t out_dtype, int32_t op, void* stream);

/* softmax / log_softmax over the last dimension of x [* scale] [+ mask]; mask (nullable, x's
 * dtype) broadcasts over the outer dimensions through mask_strides (0 = broadcast).
 * flags: 1 log_softmax, 2 apply scale, 4 run the multiply/add in the 16-bit input dtype with
 * rounding (what a 16-bit aten graph does) instead of in fp32.
 * Replaces amax_sum_20ccc18dda60/oracle.py:11-58, amax_sum_d16035e7b826/oracle.py:14-33,
 * amax_sum_7079889cfc04/oracle.py:10-36. */
int32_t b200_softmax(const void* x, const void* mask, void* y, int64_t rows, int64_t n, int64_t d1,
                     int64_t d2, const int64_t* x_strides, const int64_t* mask_strides,
                     const int64_t* y_strides, int32_t in_dtype, int32_t out_dtype, double scale,
                     int32_t flags, void* stream);

/* LayerNorm (rms = 0) / RMSNorm (rms = 1) forward over the last dimension; also row var_mean
 * (y = NULL). weight, bias, y, mean_out, rstd_out, var_out may each be NULL; statistics are fp32
 * [rows]. var uses the divisor n - correction. Adding 2 to rms puts the exact (erf) GELU in front:
 * the rows that are normalised are gelu(x) rounded to x's dtype, as the graph of
 * var_mean_af505388b035/repro.py:27-33 materialises them.
 * Replaces var_mean_f8ec553e339e/oracle.py:50-84, var_mean_af505388b035/oracle.py:11-40,
 * var_mean_f7906a6c6957/oracle.py:14-50, mean_f667cd8901af/oracle.py:36-72. */
int32_t b200_norm_fwd(const void* x, const void* weight, const void* bias, void* y, float* mean_out,
                      float* rstd_out, float* var_out, int64_t rows, int64_t n, int64_t x_row_stride,
                      int64_t y_row_stride, int32_t x_dtype, int32_t w_dtype, int32_t y_dtype,
                      double eps, double correction, int32_t rms, void* stream);

/* b200_norm_fwd with a residual prologue: the rows that are normalised are x + residual
 * (var_mean_0ada225c0a04/repro.py:26-27). The sum stays in fp32, as in Inductor's fused kernel (the
 * form the reference's fp64-anchored gate accepts); adding 4 to rms rounds it to x's dtype first, as
 * the eager graph materialises it; adding 8 instead (plain LayerNorm only) normalises both forms,
 * each with its own statistics, and gives every element the fp32 form where that form's rounded
 * output exceeds 3 in magnitude and the rounded form elsewhere - what the reference's oracles for
 * these regions return (var_mean_45f7dfd4a983/oracle.py:96-107). The statistics that are returned
 * are those of the fp32 sum in every mode but 4. residual: x's dtype, x's row stride; sum_out (may be NULL):
 * receives the sum rounded to x's dtype, rows of n contiguous elements; y must have x's dtype.
 * residual = NULL is b200_norm_fwd. Replaces var_mean_0ada225c0a04/oracle.py, var_mean_f4578c128d74/oracle.py. */
int32_t b200_norm_fwd_residual(const void* x, const void* residual, void* sum_out, const void* weight,
                               const void* bias, void* y, float* mean_out, float* rstd_out, float* var_out,
                               int64_t rows, int64_t n, int64_t x_row_stride, int64_t y_row_stride,
                               int32_t x_dtype, int32_t w_dtype, int32_t y_dtype, double eps, double correction,
                               int32_t rms, void* stream);

/* Number of bounded device-side waits of b200_norm_fwd's streaming kernel that ran out since the
 * library was loaded: 0 in normal operation. Synchronises the device (diagnostic). No counterpart
 * in the reference. */
int64_t b200_norm_fwd_wait_timeouts(void);

/* Same counter for b200_norm_bwd's streaming kernel. */
int64_t b200_norm_bwd_wait_timeouts(void);

/* Scratch bytes that let b200_norm_bwd run its largest grid for rows of n elements. */
int64_t b200_norm_bwd_scratch_bytes(int64_t n);

/* LayerNorm / RMSNorm backward in one pass over x and dy: dx rows, dweight and dbias (fp32 [n],
 * nullable) as column reductions over all rows. dx element (r, c) is stored at
 *   (r / seq) * dx_batch_stride + (r % seq) * dx_seq_stride + (c / head_dim) * dx_head_stride + c % head_dim
 * which covers both the plain [rows, n] layout (seq = 1, head_dim = n, dx_batch_stride = n) and the
 * fused head-major (B,S,H,D) -> (B,H,S,D) store. flags: 1 = two launches (main + finalize)
 * instead of one cooperative launch; 2 = dy points at ONE element that stands for the whole
 * tensor (the reference's captured graphs expand a 0-dim gradient,
 * sum_sum_2cd99e5eb23e/repro.py:26): dy_row_stride is ignored and nothing but that element is read.
 * Replaces sum_sum_2cd99e5eb23e/oracle.py:48-117, sum_sum_sum_3cac3bbf4e8f/oracle.py:100-193 and
 * the head-split copy of pointwise_c0d19d490a2f/oracle.py:10-33. */
int32_t b200_norm_bwd(const void* x, const void* dy, const void* weight, const float* mean,
                      const float* rstd, void* dx, float* dweight, float* dbias, int64_t rows,
                      int64_t n, int64_t x_row_stride, int64_t dy_row_stride, int32_t x_dtype,
                      int32_t w_dtype, int32_t rms, int64_t seq, int64_t head_dim,
                      int64_t dx_batch_stride, int64_t dx_seq_stride, int64_t dx_head_stride,
                      void* scratch, int64_t scratch_bytes, int32_t flags, void* stream);

/* Same counter for b200_batch_norm_fwd's fused kernel. */
int64_t b200_batch_norm_wait_timeouts(void);

/* Scratch bytes b200_batch_norm_fwd needs for `channels` channels. */
int64_t b200_batch_norm_scratch_bytes(int64_t channels);

/* BatchNorm2d training forward (+ ReLU when relu != 0): x and y are [batch, channels, spatial]
 * with element strides (stride_n, stride_c, stride_s) - NCHW and channels-last both fit; y uses
 * x's strides. running_mean/var (fp32 [C], nullable together) are updated in place;
 * save_mean/save_invstd (fp32 [C], nullable) receive the batch statistics.
 * Replaces var_mean_42fad1ece813/oracle.py:11-46, :49-87, :90-119 and :122-182. */
int32_t b200_batch_norm_fwd(const void* x, void* y, const void* weight, const void* bias,
                            float* running_mean, float* running_var, float* save_mean,
                            float* save_invstd, int64_t batch, int64_t channels, int64_t spatial,
                            int64_t stride_n, int64_t stride_c, int64_t stride_s, int32_t x_dtype,
                            int32_t w_dtype, double eps, double momentum, int32_t relu, void* scratch,
                            int64_t scratch_bytes, void* stream);

/* Column reduction: x is [batch, rows, cols] with cols unit-stride; out[b, c] = reduce over rows
 * (op 0 sum, 1 mean, 2 amax). Tall inputs are split over several CTAs whose fp32 partials (in
 * `scratch`, batch*cols floats per split; may be NULL for a single split) are combined in fp64 by
 * a second launch. No atomics.
 * Replaces sum_eb86a17deab9/oracle.py:20-70, sum_c2bf513c1ebf/oracle.py:10-29 and the
 * channels-last spatial mean of mean_c9e1a8113328/oracle.py:11-76. */
int32_t b200_col_reduce(const void* x, void* out, int64_t batch, int64_t rows, int64_t cols,
                        int64_t x_batch_stride, int64_t x_row_stride, int64_t out_batch_stride,
                        int32_t x_dtype, int32_t out_dtype, int32_t op, void* scratch, int64_t scratch_bytes,
                        void* stream);

/* Permuting copy into a contiguous output of shape out_shape[4]; in_strides[i] is the input
 * stride (elements) of output dimension i. Optional scale (fp32 multiply) and dtype conversion.
 * Replaces pointwise_c0d19d490a2f/oracle.py:10-33 (head split) and other permute + clone regions. */
int32_t b200_permute_copy(const void* x, void* y, const int64_t* out_shape, const int64_t* in_strides,
                          int32_t in_dtype, int32_t out_dtype, double scale, int32_t has_scale, void* stream);

/* Transpose of the two innermost dimensions: input [batch, rows, cols] (cols unit-stride, given row
 * and batch strides) -> contiguous output [batch, cols, rows], through a shared-memory tile.
 * Replaces pointwise_021e90d9c17d/oracle.py:10-51. */
int32_t b200_transpose_copy(const void* x, void* y, int64_t batch, int64_t rows, int64_t cols,
                            int64_t in_batch_stride, int64_t in_row_stride, int32_t in_dtype,
                            int32_t out_dtype, double scale, int32_t has_scale, void* stream);

/* Dropout -> residual add -> RMSNorm -> dropout over rows of `cols` elements (a multiple of 8, at most
 * 2048): keep0 = T(u0) > p; s = T(T(keep0 * x) * 1/(1-p)); sum = residual + s;
 * rstd = rsqrt(mean(sum^2) + eps); keep1 = u1 > p; y = T((keep1 * (weight * (sum * rstd))) * 1/(1-p)).
 * x, y: x_dtype (bf16 or fp16) [rows, cols]; residual, sum: fp32 [rows, cols]; weight: fp32 [cols];
 * rstd: fp32 [rows]; keep0, keep1: one byte per element (0 or 1). u0, u1 are Philox4x32-10 uniforms keyed by
 * seeds[seed_index0] and seeds[seed_index1] (read on the device), counter = (element index / 4, mask number).
 * Replaces mean_014afd4984e6/oracle.py:14-130 (kernel) and :201-260 (wrapper); the masks are stochastic
 * outputs for the reference's check (oracle_harness.py stochastic-output skip), all other outputs follow
 * from them. */
int32_t b200_dropout_rms_norm(const void* x, const void* residual, const void* weight, const int64_t* seeds,
                              int32_t seed_index0, int32_t seed_index1, double p, double eps, void* keep0,
                              void* sum, void* rstd, void* keep1, void* y, int64_t rows, int64_t cols,
                              int32_t x_dtype, void* stream);

/* Dropout -> residual add -> LayerNorm over rows of `cols` elements (a multiple of 8, at most 2048):
 * keep = T(u) > p; sum = T(T(keep * x) * 1/(1-p)) + residual; var, mean = var_mean(sum);
 * rstd = rsqrt(var + eps); xhat = (sum - mean) * rstd; y = xhat * weight + bias.
 * x: x_dtype (bf16 or fp16) [rows, cols]; residual, xhat, y: fp32 [rows, cols]; weight, bias: fp32 [cols];
 * rstd_over_n: fp32 [rows] = rstd / cols; keep: one byte per element. u as in b200_dropout_rms_norm (mask
 * number 0, key seeds[seed_index]).
 * Replaces var_mean_01fbd6c1b27f/oracle.py (kernel and wrapper); graph var_mean_01fbd6c1b27f/repro.py:24-44. */
int32_t b200_dropout_layer_norm(const void* x, const void* residual, const void* weight, const void* bias,
                                const int64_t* seeds, int32_t seed_index, double p, double eps, void* keep,
                                void* xhat, void* y, void* rstd_over_n, int64_t rows, int64_t cols,
                                int32_t x_dtype, void* stream);

/* Dropout -> residual add over n elements (a multiple of 8): keep = T(u) > p;
 * sum = residual + T(T(keep * x) * 1/(1-p)). x: x_dtype (bf16 or fp16); residual, sum: fp32; keep: one byte per
 * element; u as in b200_dropout_rms_norm (mask number 0, key seeds[seed_index]).
 * Replaces pointwise_4b076ed1ff41/oracle.py, pointwise_7bd204513fbb/oracle.py, pointwise_6e7efb08a440/oracle.py
 * (kernel and wrapper); graph pointwise_4b076ed1ff41/repro.py:24-32. */
int32_t b200_dropout_add(const void* x, const void* residual, const int64_t* seeds, int32_t seed_index, double p,
                         void* keep, void* sum, int64_t n, int32_t x_dtype, void* stream);

/* softmax(x + bias) -> dropout over rows of `cols` scores (a multiple of 8, at most 1024):
 *   logits = T(x + bias); amax = max(logits); sum = sum(exp(logits - amax)); prob = T(exp(..) / sum);
 *   keep = T(u) > p; y = T(T(keep * prob) * 1/(1-p)).
 * x: contiguous [batch*heads, seq_q, cols], x_dtype (bf16 or fp16); bias: fp32 [batch, heads, seq_q, cols] with
 * the four element strides given (any layout); outputs contiguous: logits and y x_dtype, amax and sum fp32
 * [batch*heads*seq_q], keep one byte per element. u as in b200_dropout_rms_norm (mask number 0, key
 * seeds[seed_index], counter = flat element index).
 * Replaces amax_sum_089fdab8f22b/oracle.py (kernels and wrapper); graph amax_sum_089fdab8f22b/repro.py:24-46. */
int32_t b200_softmax_dropout(const void* x, const void* bias, int64_t batch, int64_t heads, int64_t seq_q,
                             int64_t cols, int64_t bias_stride_b, int64_t bias_stride_h, int64_t bias_stride_q,
                             int64_t bias_stride_k, const int64_t* seeds, int32_t seed_index, double p,
                             void* logits, void* amax, void* sum, void* keep, void* y, int32_t x_dtype,
                             void* stream);

/* Contiguous cast / scale / activation of n elements: y = Tout(op(x)). has_scale is a mode word: bit 0
 * multiplies by scale (in fp32); then bit 1 applies ReLU (a NaN stays a NaN), bit 2 the exact GELU
 * (x * 0.5) * (erf(x * 0.7071067811865476) + 1), bit 3 SiLU x / (exp(-x) + 1), all in fp32.
 * Replaces pointwise_8bb40810003c/oracle.py:11-15, pointwise_95ed2ef35da9/oracle.py:10-44, and the
 * storage-order kernels of pointwise_04d85912d998/oracle.py, pointwise_ccd411f2a45d/oracle.py
 * (parameter casts), pointwise_3abc926270f6/oracle.py (ReLU), pointwise_826ea0b5f6e4/oracle.py (GELU) and
 * pointwise_795cdbe23b17/oracle.py (SiLU). */
int32_t b200_cast_scale(const void* x, void* y, int64_t n, int32_t in_dtype, int32_t out_dtype, double scale,
                        int32_t has_scale, void* stream);

/* BatchNorm2d training backward. dy, x, (act) and dx share the element strides (n, c, spatial);
 * mean / invstd are the statistics saved by the forward pass (fp32 [C]). Outputs: dx (may be NULL:
 * sums only), dweight = sum(dy * (x - mean)) * invstd and dbias = sum(dy), fp32 [C] (each may be
 * NULL). `act` (may be NULL) enables the activation-backward prologue dy' = act > 0 ? dy : dy * slope
 * (slope 0: ReLU), rounded to the tensor dtype. One launch for contiguous NCHW tensors; three
 * launches (sums, fp64 finalize, apply) for channels-last tensors (flat 16-byte vectors, any channel
 * count) and for other strides (element-wise). No atomics. Scratch: b200_batch_norm_bwd_scratch_bytes(channels), 16-byte aligned, no initial state.
 * Replaces sum_sum_183b124c731f/oracle.py (partial sums, finalize, apply) and, with the prologue,
 * sum_sum_12fc8ebf8180/oracle.py. */
int64_t b200_batch_norm_bwd_scratch_bytes(int64_t channels);
int32_t b200_batch_norm_bwd(const void* dy, const void* x, const void* act, const float* mean,
                            const float* invstd, const void* weight, void* dx, float* dweight,
                            float* dbias, int64_t batch, int64_t channels, int64_t spatial,
                            int64_t stride_n, int64_t stride_c, int64_t stride_s, int32_t x_dtype,
                            int32_t w_dtype, double slope, void* scratch, int64_t scratch_bytes,
                            void* stream);

/* The two entry points above with a constant of the captured graph passed in instead of derived
 * from the sizes. The reference's eager modules are graphs captured at ONE shape point; numbers that
 * depended on that shape are literals in them (var_mean_42fad1ece813/repro.py:40 multiplies the
 * batch variance by 1.0001220852154804 = 8192/8191, sum_sum_183b124c731f/repro.py:33 multiplies the
 * sums by 6.228077168367346e-07 = 1/1605632) and are applied unchanged at every other point of
 * shapes.json, as the reference's own oracles do (sum_sum_183b124c731f/oracle.py:10). unbiased_factor
 * / inv_count <= 0 select the value derived from the sizes. */
int32_t b200_batch_norm_fwd_ex(const void* x, void* y, const void* weight, const void* bias,
                               float* running_mean, float* running_var, float* save_mean,
                               float* save_invstd, int64_t batch, int64_t channels, int64_t spatial,
                               int64_t stride_n, int64_t stride_c, int64_t stride_s, int32_t x_dtype,
                               int32_t w_dtype, double eps, double momentum, double unbiased_factor,
                               int32_t relu, void* scratch, int64_t scratch_bytes, void* stream);
int32_t b200_batch_norm_bwd_ex(const void* dy, const void* x, const void* act, const float* mean,
                               const float* invstd, const void* weight, void* dx, float* dweight,
                               float* dbias, int64_t batch, int64_t channels, int64_t spatial,
                               int64_t stride_n, int64_t stride_c, int64_t stride_s, int32_t x_dtype,
                               int32_t w_dtype, double slope, double inv_count, void* scratch,
                               int64_t scratch_bytes, void* stream);

/* b200_batch_norm_fwd for callers that may not allocate device memory (a host framework that owns
 * the only arena and forbids plug-ins to call cudaMalloc, or a caller that owns nothing but the
 * tensors it was handed): the scratch lives in a fixed array inside the library's device image
 * instead of a caller-provided buffer. Same arguments minus scratch. Limits: at most 1024 channels
 * (larger requests return B200_ERR_UNSUPPORTED); every GPU that loads the library holds the array
 * (about 1.3 MB) until the process exits. The first call on each device looks up the array's
 * device address and should be made before any stream capture. All calls on a device share the
 * array: calls that overlap on the GPU race and must be ordered by the caller. Allocates nothing.
 * The caller has no scratch pointer to hand to b200_check_status here (and the barrier words are
 * cleared at every call): a bounded device-side wait that ran out shows in
 * b200_batch_norm_wait_timeouts(), which stays at 0 in normal operation.
 * This entry point has no counterpart in the reference. */
int32_t b200_batch_norm_fwd_static_scratch(const void* x, void* y, const void* weight, const void* bias,
                                           float* running_mean, float* running_var, float* save_mean,
                                           float* save_invstd, int64_t batch, int64_t channels,
                                           int64_t spatial, int64_t stride_n, int64_t stride_c,
                                           int64_t stride_s, int32_t x_dtype, int32_t w_dtype, double eps,
                                           double momentum, int32_t relu, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* B200_ORACLES_H */
