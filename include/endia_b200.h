/*
 * endia_b200.h — C ABI of the B200 (sm_100a) device path for Endia's reverse-mode
 * hot path: the ops of an MLP training step (matmul and its VJPs, elementwise and
 * reduction VJPs, fused Adam) and the complex FFT family with its VJPs.
 *
 * Conventions
 *   - Every entry point returns 0 on success and a negative ENDIA_B200_E* code on
 *     failure; endia_b200_last_error() then returns a thread-local message. Nothing
 *     throws across this boundary (Endia's ops `raise "string"`; the binding turns a
 *     non-zero status into such a raise).
 *   - All data pointers are DEVICE pointers to float32 storage. A complex element is
 *     an interleaved (re, im) float pair (endia/_array/_array.mojo:126-128, 528-536).
 *   - Every launch takes an explicit `stream` (a cudaStream_t passed as void*;
 *     NULL = the legacy default stream). Calls are asynchronous unless stated.
 *   - A tensor descriptor carries Endia's ArrayShape semantics: shape, stride and
 *     storage offset counted in ELEMENTS (one complex element counts 1),
 *     row-major default strides (endia/utils/_array_shape.mojo:24-30).
 *   - There is no CPU fallback: without a usable sm_100 device every compute entry
 *     point fails with ENDIA_B200_ENODEV.
 */
#ifndef ENDIA_B200_H
#define ENDIA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ENDIA_B200_MAX_DIMS 8

enum {
  ENDIA_B200_OK = 0,
  ENDIA_B200_EINVAL = -1,   /* bad shape / stride / NULL pointer / unsupported flag  */
  ENDIA_B200_ECUDA = -2,    /* a CUDA runtime call failed                            */
  ENDIA_B200_ENODEV = -3,   /* no CUDA device / not an sm_100 part                   */
  ENDIA_B200_ENOMEM = -4,   /* device allocation failed                              */
  ENDIA_B200_ESHAPE = -5,   /* operand shapes are not compatible                     */
  ENDIA_B200_EPOW2 = -6,    /* FFT length is not a power of two
                               (endia/functional/fft_ops/fft_cooley_tukey.mojo:227-235) */
  ENDIA_B200_ETIMEOUT = -7, /* a bounded device-side wait gave up                    */
  ENDIA_B200_ELIMIT = -8    /* size beyond a documented fixed limit                  */
};

/* Strided view of device storage. Replaces Array/ArrayShape as seen by an op's
 * `fwd` callable (endia/_array/_array.mojo:56-113; endia/utils/_array_shape.mojo:85-250). */
typedef struct endia_b200_tensor {
  void *data;                           /* base of the float32 buffer              */
  int64_t shape[ENDIA_B200_MAX_DIMS];
  int64_t stride[ENDIA_B200_MAX_DIMS];  /* in elements; 0 = broadcast dimension    */
  int64_t offset;                       /* storage offset in elements              */
  int32_t ndim;
  int32_t is_complex;                   /* 1: elements are (re, im) float pairs    */
} endia_b200_tensor;

/* ---------------------------------------------------------------- runtime ---- */

/* Select `device`, verify compute capability 10.x, create the per-device state.
 * Replaces nothing in the reference (its arrays live in host memory); it is the hook the
 * device-resident Node storage needs (endia/_array/_array.mojo:125-131). */
int endia_b200_init(int device);
int endia_b200_shutdown(void);
const char *endia_b200_last_error(void);
/* ABI version (major*1000 + minor). */
int endia_b200_version(void);
/* Number of kernels this library has launched in this process (all threads); a benchmark
 * reads it before and after its timed region. */
uint64_t endia_b200_launch_count(void);
/* 1 when the library was built with the tcgen05 GEMM and the device accepts it. */
int endia_b200_has_tcgen05(void);

/* Synchronises `stream` and reports whether any kernel of this library gave up a bounded
 * device-side wait since the last call (ENDIA_B200_ETIMEOUT, flag cleared), else 0. Kernels that
 * wait on barriers never spin without a limit; a wait that runs out records a code, lets the
 * kernel drain and return, and is reported here. */
int endia_b200_device_status(void *stream);
/* Self-test of that give-up path: launches one small kernel whose only wait (the library's bounded
 * barrier wait, limited to `polls` polls, at most 2^20) is on a barrier that nothing arrives at. The
 * wait runs out, the kernel returns, and the next endia_b200_device_status reports
 * ENDIA_B200_ETIMEOUT once; the context stays usable. */
int endia_b200_selftest_wait_timeout(int32_t polls, void *stream);

/* Stream-ordered device memory. Replaces UnsafePointer.alloc/free + memset_zero in
 * Node.__init__/__del__ (endia/_array/_array.mojo:127-128, 177-179) and
 * setup_shape_and_data (endia/functional/_utils.mojo:319-326). */
int endia_b200_malloc(void **ptr, size_t bytes, void *stream);
/* Upper bound on the bytes endia_b200_malloc may have live at one time (0 = none, the default). A
 * request beyond it fails with ENDIA_B200_ENOMEM before the driver is asked: the budget of a host
 * that shares the device, and the way a caller's out-of-memory handling is exercised without
 * exhausting a GPU. */
int endia_b200_set_malloc_quota(size_t bytes);
int endia_b200_free(void *ptr, void *stream);
int endia_b200_memset0(void *ptr, size_t bytes, void *stream);
int endia_b200_h2d(void *dst_dev, const void *src_host, size_t bytes, void *stream);
int endia_b200_d2h(void *dst_host, const void *src_dev, size_t bytes, void *stream);
int endia_b200_d2d(void *dst_dev, const void *src_dev, size_t bytes, void *stream);

int endia_b200_stream_create(void **stream);
int endia_b200_stream_destroy(void *stream);
int endia_b200_stream_sync(void *stream);
int endia_b200_event_create(void **event);
int endia_b200_event_destroy(void *event);
int endia_b200_event_record(void *event, void *stream);
int endia_b200_stream_wait_event(void *stream, void *event);
/* Milliseconds between two recorded events (both must have completed). */
int endia_b200_event_elapsed_ms(void *start, void *stop, float *ms);

/* ------------------------------------------------------------------ GEMM ---- */

enum { ENDIA_B200_ACT_NONE = 0, ENDIA_B200_ACT_RELU = 1, ENDIA_B200_ACT_TANH = 2,
       ENDIA_B200_ACT_SIGMOID = 3 };

enum { ENDIA_B200_GEMM_AUTO = 0,   /* a tcgen05 split-precision kernel when the shape allows, else FFMA */
       ENDIA_B200_GEMM_FFMA = 1,   /* fp32 FFMA tiles                                 */
       ENDIA_B200_GEMM_3XTF32 = 2, /* tcgen05 tf32 MMAs, hi/lo split, fp32 accumulate */
       /* a_hi*b_hi as one tf32 MMA; the two correction products a_lo*b + a*b_lo as bf16 MMAs
        * (their operands only need 8 bits: error 2^-19 of |a||b| per product instead of 2^-22,
        * far inside the 1e-4 bound on gradients). Two thirds of the tensor-core time of 3xTF32.
        * Needs N >= 256. */
       ENDIA_B200_GEMM_TF32_BF16X2 = 3 };

/* Work fused into the GEMM's store, applied in this order to acc = op(A)·op(B):
 *   v = alpha*acc
 *   v += bias[n]                           (bias != NULL)          Add after matmul,
 *                                           endia/nn/modules/_mlp.mojo:50-51
 *   v  = act(v)                            (act != NONE)           relu_op.mojo:115,
 *                                           tanh_op.mojo:112-115, sigmoid_op.mojo:118-121
 *   v *= act'(dact_src[m,n])               (dact != NONE)          the VJP masks:
 *        RELU:    dact_src = pre-activation s, factor (s > 0)      relu_op.mojo:95
 *        TANH:    dact_src = activation   a, factor 1 - a*a        tanh_op.mojo:92
 *        SIGMOID: dact_src = activation   a, factor a*(1-a)        sigmoid_op.mojo:98
 *   v += beta*C[m,n]                       (beta != 0; gradient accumulation,
 *                                           endia/autograd/functional.mojo:55-57)
 *   C[m,n] = v
 *   colsum[n] = sum_m v                    (colsum != NULL; the bias gradient that
 *                                           Expand.vjp reduces, expand_op.mojo:121-126)
 * colsum is reduced deterministically: per-row-tile partials go to `colsum_scratch`
 * (at least endia_b200_gemm_colsum_scratch_bytes(M, N) bytes) and a second small kernel
 * adds them in a fixed order. */
typedef struct endia_b200_epilogue {
  float alpha;
  float beta;
  const float *bias;
  int32_t act;
  int32_t dact;
  const float *dact_src;
  int64_t ld_dact;
  float *colsum;
  float *colsum_scratch;
  /* Optional, used only by the 3xTF32 kernel: the low parts x - tf32(x) of A and/or B, laid out
   * exactly like A / B (same leading dimension), e.g. as endia_b200_tf32_split or
   * endia_b200_adam_step_multi_lo wrote them. NULL = computed inside the call. */
  const float *a_lo;
  const float *b_lo;
  /* Optional, used only by the TF32_BF16X2 kernel: the bf16 split of A and/or B as
   * endia_b200_bf16_split wrote it for the operand's whole [rows, ld] storage. NULL = computed
   * inside the call. */
  const void *a16;
  const void *b16;
  /* Optional output: the bf16 split of the stored C (endia_b200_bf16_split's layout for the [M, N]
   * array; needs batch == 1, ldc == N, M*N a multiple of 8), for the products that will read C as an
   * operand. Written by the two-CTA kernel's epilogue from the values it stores; when another
   * kernel runs the call ends with one split pass over C, so the parts are valid either way. */
  void *c16;
} endia_b200_epilogue;

size_t endia_b200_gemm_colsum_scratch_bytes(int64_t M, int64_t N);

/* lo[i] = x[i] - (x[i] with its 13 low mantissa bits cleared), for `rows` rows of `cols` floats
 * (cols and both leading dimensions multiples of 4, 16-byte aligned pointers): the second operand
 * part of the 3xTF32 product, for callers that reuse it over several GEMMs. */
int endia_b200_tf32_split(const float *x, float *lo, int64_t rows, int64_t cols, int64_t ld_in,
                          int64_t ld_out, void *stream);

/* The operand parts of the TF32_BF16X2 product for an array of `numel` floats (numel a multiple
 * of 8, 16-byte aligned pointers): pair16[0 .. numel) = bf16(x) and pair16[numel .. 2*numel) =
 * bf16(x - tf32(x)), round to nearest, 2 bytes each, laid out like x. `pair16` holds
 * 4*numel bytes. */
int endia_b200_bf16_split(const float *x, void *pair16, int64_t numel, void *stream);

/* C[M,N] = epilogue(op(A)[M,K] · op(B)[K,N]), fp32, row-major storage.
 *   trans_a = 0: A is stored [M,K] with leading dimension lda >= K
 *   trans_a = 1: A is stored [K,M] with leading dimension lda >= M   (Xᵀ·dY without a copy)
 *   trans_b = 0: B is stored [K,N], ldb >= N;  trans_b = 1: B is stored [N,K], ldb >= K (dY·Wᵀ)
 * `batch` independent products with element strides stride_a/b/c between them
 * (a stride of 0 broadcasts that operand over the batch).
 * Replaces matmul_fwd (endia/functional/binary_ops/matmul_op.mojo:93-254) and the
 * transposing copies it makes of `.T()` operands (matmul_op.mojo:107-136), so that the
 * two products of matmul_vjp (matmul_op.mojo:278-284) need no materialised transpose.
 * `epi` may be NULL (alpha = 1, nothing fused). `algo` is one of ENDIA_B200_GEMM_*. */
int endia_b200_gemm(int trans_a, int trans_b, int64_t M, int64_t N, int64_t K,
                    const float *A, int64_t lda, const float *B, int64_t ldb,
                    float *C, int64_t ldc, int64_t batch, int64_t stride_a,
                    int64_t stride_b, int64_t stride_c, const endia_b200_epilogue *epi,
                    int algo, void *stream);

/* Complex (interleaved) matmul, same storage conventions, no epilogue.
 * Replaces the complex branch of matmul_fwd (matmul_op.mojo:200-238). */
int endia_b200_gemm_complex(int trans_a, int trans_b, int64_t M, int64_t N, int64_t K,
                            const float *A, int64_t lda, const float *B, int64_t ldb,
                            float *C, int64_t ldc, int64_t batch, int64_t stride_a,
                            int64_t stride_b, int64_t stride_c, void *stream);

/* ------------------------------------------------------------ elementwise ---- */

enum {
  ENDIA_B200_UN_COPY = 0,   /* strided gather → `out` (contiguous(), functional/_utils.mojo:79-205) */
  ENDIA_B200_UN_NEG, ENDIA_B200_UN_RELU, ENDIA_B200_UN_TANH, ENDIA_B200_UN_SIGMOID,
  ENDIA_B200_UN_SQUARE, ENDIA_B200_UN_SQRT, ENDIA_B200_UN_ABS, ENDIA_B200_UN_SIGN,
  ENDIA_B200_UN_CONJ, ENDIA_B200_UN_EXP, ENDIA_B200_UN_LOG, ENDIA_B200_UN_SIN,
  ENDIA_B200_UN_COS, ENDIA_B200_UN_RECIPROCAL,
  ENDIA_B200_UN_SINH, ENDIA_B200_UN_COSH, ENDIA_B200_UN_TAN, ENDIA_B200_UN_ASIN, ENDIA_B200_UN_ACOS,
  ENDIA_B200_UN_ATAN,        /* unary_ops/{sinh,cosh,tan,asin,acos,atan}_op.mojo */
  ENDIA_B200_UN_COUNT
};
enum {
  ENDIA_B200_BIN_ADD = 0, ENDIA_B200_BIN_SUB, ENDIA_B200_BIN_MUL, ENDIA_B200_BIN_DIV,
  ENDIA_B200_BIN_POW, ENDIA_B200_BIN_GREATER,
  /* fused VJP forms (one pass instead of the reference's op chains):           */
  ENDIA_B200_BIN_RELU_BWD,     /* out = (a > 0) * b          a = pre-activation, b = grad */
  ENDIA_B200_BIN_TANH_BWD,     /* out = (1 - tanh(a)^2) * b  a = pre-activation           */
  ENDIA_B200_BIN_SIGMOID_BWD,  /* out = a*(1-a) * b          a = sigmoid output           */
  ENDIA_B200_BIN_COMPLEX,      /* out = a + i*b, a and b real, out complex (`complex(re, im)`,
                                  init_ops.mojo:419-433)                                      */
  ENDIA_B200_BIN_ABS_BWD,      /* out = a/|a| * b            Abs.vjp sign(x)*grad, abs_op.mojo:93          */
  ENDIA_B200_BIN_SQUARE_BWD,   /* out = 2*a*b                Square.vjp, square_op.mojo:96                 */
  /* the other comparisons of comparison_ops/: 1.0 / 0.0, real operands */
  ENDIA_B200_BIN_GREATER_EQUAL, ENDIA_B200_BIN_LESS, ENDIA_B200_BIN_LESS_EQUAL, ENDIA_B200_BIN_EQUAL,
  ENDIA_B200_BIN_NOT_EQUAL,
  ENDIA_B200_BIN_TANH_OUT_BWD,   /* out = (1 - a^2) * b   a = tanh OUTPUT, b = grad (tanh_op.mojo:92), real only */
  ENDIA_B200_BIN_TANH_OUT_BWD2,  /* out = -2 * a * b      the derivative of the line above w.r.t. a, real only   */
  ENDIA_B200_BIN_COUNT
};

/* out[i] = f(in[i]) over in's logical shape; `out` must have the same shape. `in` may be any
 * strided view (broadcast strides included); complex inputs use the complex formulas of the
 * op files under endia/functional/unary_ops/. Replaces execute_unary_op
 * (endia/functional/unary_ops/_utils.mojo:77-134) and execute_copy_raw
 * (endia/functional/_utils.mojo:79-163). */
int endia_b200_ew_unary(int op, const endia_b200_tensor *in, const endia_b200_tensor *out,
                        void *stream);

/* out = a (op) b. a and b must already be expanded to out's shape (stride 0 on stretched
 * dims, as Endia's `expand` view produces, expand_op.mojo:62-84); nothing is materialised.
 * Replaces execute_binary_op (endia/functional/binary_ops/_utils.mojo:93-177). */
int endia_b200_ew_binary(int op, const endia_b200_tensor *a, const endia_b200_tensor *b,
                         const endia_b200_tensor *out, void *stream);

/* Fill a contiguous float buffer with a constant (endia `full`/`ones`/`zeros`,
 * init_ops.mojo:85-205). For complex buffers pass re/im. */
int endia_b200_fill(float *dst, int64_t n_elements, int is_complex, float re, float im,
                    void *stream);
/* n×n identity (init_ops.mojo `eye`), used as the Jacobian seed of non-scalar outputs
 * (endia/autograd/functional.mojo:34-38). */
int endia_b200_eye(float *dst, int64_t n, void *stream);

/* -------------------------------------------------------------- reductions ---- */

/* out = sum of `in` over the axes set in `axes_mask` (bit d = reduce dim d); `out` is a
 * contiguous buffer with the reduced dims kept as 1. Deterministic (fixed tree order).
 * `scratch` must hold endia_b200_reduce_scratch_bytes(in, axes_mask) bytes (may be NULL when
 * that is 0). Replaces ReduceAdd.__call__ (endia/functional/reduce_ops/reduce_add_op.mojo:65-210). */
size_t endia_b200_reduce_scratch_bytes(const endia_b200_tensor *in, uint32_t axes_mask);
int endia_b200_reduce_add(const endia_b200_tensor *in, uint32_t axes_mask, float *out,
                          void *scratch, void *stream);

/* The same with a product instead of a sum (ReduceMul.__call__,
 * endia/functional/reduce_ops/reduce_mul_op.mojo); real arrays only. Same scratch size. */
int endia_b200_reduce_mul(const endia_b200_tensor *in, uint32_t axes_mask, float *out,
                          void *scratch, void *stream);

/* Fused mean-squared-error forward and backward on contiguous [n] buffers:
 *   loss[0] = sum((p-t)^2) / n ;  dpred[i] = gscale * 2 (p[i]-t[i]) / n   (dpred may be NULL)
 * `scratch` >= endia_b200_mse_scratch_bytes(n). Replaces the op chain of mse
 * (endia/functional/loss_ops/mse_op.mojo:18-20) and its five VJP passes. */
size_t endia_b200_mse_scratch_bytes(int64_t n);
int endia_b200_mse_fwd_bwd(const float *pred, const float *target, int64_t n, float gscale,
                           float *loss, float *dpred, void *scratch, void *stream);

/* Allocation-free form of endia_b200_mse_fwd_bwd. It has no counterpart in the reference.
 * It exists for hosts that must not allocate device memory around a call: a runtime that owns
 * the whole device heap and hands out no more of it, or a caller inside a section where
 * cudaMalloc is forbidden. Same results as endia_b200_mse_fwd_bwd, but the per-block partial sums
 * go to a fixed 16 KiB array inside the library (held by every GPU that loads the library until the
 * process exits) instead of caller-provided scratch, and the call allocates nothing.
 *   - Limit: n <= 16,777,216 elements (4096 partials of 4096 elements); larger n returns
 *     ENDIA_B200_ELIMIT and the message names the limit.
 *   - The first call on each device looks up the array's device address; make that first call
 *     before any stream capture begins.
 *   - All calls share the one array (its old contents are simply overwritten), so two calls that
 *     may run on the GPU at the same time (different streams) race: order them on one stream. */
int endia_b200_mse_fwd_bwd_noalloc(const float *pred, const float *target, int64_t n,
                                   float gscale, float *loss, float *dpred, void *stream);

/* Fused activation backward and bias gradient of one layer, on contiguous [M, N] buffers:
 *   ds[m,n] = grad[m,n] * act'(act_out[m,n])   (factors as in endia_b200_epilogue; act = NONE
 *                                               leaves ds untouched and only sums grad)
 *   colsum[n] = sum_m ds[m,n]                   (colsum may be NULL)
 * `scratch` >= endia_b200_act_bwd_colsum_scratch_bytes(M, N) when colsum is given. Replaces the
 * VJP chains of relu/tanh/sigmoid (relu_op.mojo:95, tanh_op.mojo:92, sigmoid_op.mojo:98) followed by
 * Expand.vjp's reduce_add for the bias (expand_op.mojo:121-126). */
size_t endia_b200_act_bwd_colsum_scratch_bytes(int64_t M, int64_t N);
int endia_b200_act_bwd_colsum(int act, const float *act_out, const float *grad, float *ds,
                              float *colsum, int64_t M, int64_t N, void *scratch, void *stream);

/* The same, also writing the bf16 split of dS (endia_b200_bf16_split's layout, 4*M*N bytes at
 * `pair16`, NULL = not written) that the TF32_BF16X2 products consuming dS read, in the same pass
 * (needs act != NONE, N % 4 == 0, M*N % 8 == 0). */
int endia_b200_act_bwd_colsum_parts(int act, const float *act_out, const float *grad, float *ds,
                                    float *colsum, int64_t M, int64_t N, void *scratch, void *pair16,
                                    void *stream);

/* --------------------------------------------------------------- optimizer ---- */

/* One fused Adam step over n_tensors parameter tensors (device pointers passed in HOST arrays):
 *   g' = grad_scale*g; m = b1*m + (1-b1)*g'; v = b2*v + ((1-b2)*g')*g';
 *   p -= (lr * (m/(1-b1^t))) / (sqrt(v/(1-b2^t)) + eps)
 * with every scalar evaluated in fp32 and t an fp32 step count that starts at 1
 * (endia/optim/adam.mojo:40, 47-65). Replaces ~14 array passes per tensor. */
int endia_b200_adam_step_multi(int32_t n_tensors, float *const *params, const float *const *grads,
                               float *const *m, float *const *v, const int64_t *numel, float lr,
                               float beta1, float beta2, float eps, float t, float grad_scale,
                               void *stream);

/* One whole training step of a small MLP (forward, MSE loss, backward, optional Adam update) in
 * a single launch of one CTA, every activation in shared memory: for networks whose step is bound
 * by launch latency (the reference's own benchmark sizes). x is [batch, dims[0]], y is
 * [batch, dims[n_layers]], W[l] is [dims[l], dims[l+1]] row-major, b[l] is [dims[l+1]]; `act` is
 * applied to all but the last layer. Writes loss[0], the gradients gW[l] / gb[l], and, with
 * do_adam, updates W, b and the moments in place (t as in endia_b200_adam_step_multi). Limits:
 * at most 8 layers, widths <= 256, and batch * (sum of widths + 2 * max width) + max weight matrix
 * within 200 KiB of floats (ENDIA_B200_ELIMIT otherwise).
 * Replaces, for such sizes, the op sequence of MLP.forward + mse + backward + Adam.step
 * (endia/nn/modules/_mlp.mojo:47-53, loss_ops/mse_op.mojo:18-20, autograd/functional.mojo:26-67,
 * optim/adam.mojo:47-65; the loop of benchmarks/mlp_benchmarks/mlp_imp.mojo:47-75). */
int endia_b200_mlp_small_step(int32_t n_layers, const int32_t *dims, int32_t batch, int32_t act,
                              const float *x, const float *y, float *const *W, float *const *b,
                              float *const *gW, float *const *gb, float *const *mW,
                              float *const *vW, float *const *mb, float *const *vb, float *loss,
                              int32_t do_adam, float lr, float beta1, float beta2, float eps,
                              float t, void *stream);

/* endia_b200_adam_step_multi that also writes, for every tensor with a non-NULL entry in `p_lo`,
 * the tf32 low part of the UPDATED parameter (same layout), so that the GEMMs of the next step
 * need not recompute it for the weights. */
int endia_b200_adam_step_multi_lo(int32_t n_tensors, float *const *params, const float *const *grads,
                                  float *const *m, float *const *v, float *const *p_lo,
                                  const int64_t *numel, float lr, float beta1, float beta2, float eps,
                                  float t, float grad_scale, void *stream);

/* The same with the bf16 split of the updated parameter (endia_b200_bf16_split's layout, numel a
 * multiple of 8) for every tensor with a non-NULL entry in `p16`. */
int endia_b200_adam_step_multi_bf16(int32_t n_tensors, float *const *params, const float *const *grads,
                                    float *const *m, float *const *v, void *const *p16,
                                    const int64_t *numel, float lr, float beta1, float beta2, float eps,
                                    float t, float grad_scale, void *stream);

/* endia_b200_adam_step_multi_bf16 for a step that is replayed from a CUDA graph, where a host value
 * of t would be frozen at capture: t is read from t_dev[0] (a device float, >= 1) when the kernel
 * runs, the bias corrections 1 - beta^t are formed on the device (the power in double, rounded to
 * fp32), and, with `advance` != 0, a second one-thread launch adds 1 to t_dev[0] (a step whose
 * tensors go in several calls advances with the last one; n_tensors = 0 only advances).
 * `p16` may be NULL or hold NULL entries. */
int endia_b200_adam_step_multi_graph(int32_t n_tensors, float *const *params, const float *const *grads,
                                     float *const *m, float *const *v, void *const *p16,
                                     const int64_t *numel, float lr, float beta1, float beta2, float eps,
                                     float *t_dev, int32_t advance, float grad_scale, void *stream);

/* The other optimizers of the reference as single multi-tensor launches, same conventions as
 * endia_b200_adam_step_multi (flat numel per tensor, gradients multiplied by grad_scale first):
 *   sgd      (endia/optim/sgd.mojo:40-63): g' = g + weight_decay * p when weight_decay > 0;
 *            momentum > 0: velocity = momentum * velocity - lr * g', p += velocity (`velocity`
 *            required); momentum == 0: p -= lr * g' (`velocity` may be NULL)
 *   rmsprop  (endia/optim/rmsprop.mojo:39-53): cache = alpha * cache + (1 - alpha) * g * g,
 *            p -= lr * g / (sqrt(cache) + eps)
 *   adagrad  (endia/optim/adagrad.mojo:36-45): cache += g * g, p -= lr * g / (sqrt(cache) + eps) */
int endia_b200_sgd_step_multi(int32_t n_tensors, float *const *params, const float *const *grads,
                              float *const *velocity, const int64_t *numel, float lr, float momentum,
                              float weight_decay, float grad_scale, void *stream);
int endia_b200_rmsprop_step_multi(int32_t n_tensors, float *const *params, const float *const *grads,
                                  float *const *cache, const int64_t *numel, float lr, float alpha,
                                  float eps, float grad_scale, void *stream);
int endia_b200_adagrad_step_multi(int32_t n_tensors, float *const *params, const float *const *grads,
                                  float *const *cache, const int64_t *numel, float lr, float eps,
                                  float grad_scale, void *stream);

/* --------------------------------------------------------------------- FFT ---- */

/* Complex-to-complex FFT over the listed dims of `in` (contiguous or strided complex, or
 * contiguous real: read as complex with a zero imaginary part, fft_cooley_tukey.mojo:204-206)
 * into `out` (contiguous complex, same shape):
 *   inverse = 0: sign -  (forward DFT),  inverse = 1: sign +  (conjugate-direction transform,
 *   i.e. conj(fft(conj(x))), which is both FFTN.vjp and the core of ifftn)
 *   every output element is multiplied by `scale`.
 * Each transformed length must be a power of two (ENDIA_B200_EPOW2 otherwise).
 * `scratch` must hold endia_b200_fft_scratch_bytes(...) bytes (NULL when that is 0).
 * Replaces fft_cooley_tukey_parallel (endia/functional/fft_ops/fft_cooley_tukey.mojo:179-313)
 * as called by FFTN/IFFTN and their VJPs (fftn_op.mojo:43-60, ifftn_op.mojo:42-77). */
size_t endia_b200_fft_scratch_bytes(const endia_b200_tensor *in, const int32_t *dims,
                                    int32_t n_dims);
int endia_b200_fft_c2c(const endia_b200_tensor *in, const endia_b200_tensor *out,
                       const int32_t *dims, int32_t n_dims, int inverse, float scale,
                       void *scratch, void *stream);

/* The same transform with work fused into its last pass, so that a loss on the result and the
 * gradient that flows back into the VJP transform cost no passes of their own:
 *   scale_dev     (optional) device scalar multiplied into `scale` when the last pass runs: the
 *                 incoming gradient of a loss, folded into the VJP transform
 *   reduce = 1    reduce_out[0] = reduce_scale * sum |y|^2          the chain
 *                 sum(square(to_abs(y))) (abs_op.mojo:114-157, real_op.mojo:43-52,
 *                 square_op.mojo:117-119, sum_op.mojo:35-62)
 *   reduce = 2    reduce_out[0] = reduce_scale * sum real(y) * reduce_w   the chain
 *                 sum(real(y) * w) (real_op.mojo:43-52, mul_op.mojo, sum_op.mojo:35-62);
 *                 reduce_w: contiguous float array of the output's shape
 * over the stored output y (after `scale`). The sum is deterministic: one partial per CTA of the
 * last pass in `reduce_scratch` (endia_b200_fft_fusion_scratch_bytes() bytes), added in a fixed
 * order. Where the last pass has no fused form the loss term takes one more pass over `out`.
 * `fusion` = NULL is endia_b200_fft_c2c. */
typedef struct endia_b200_fft_fusion {
  const float *scale_dev;
  int32_t reduce;
  const float *reduce_w;
  float *reduce_out;
  float reduce_scale;
  void *reduce_scratch;
} endia_b200_fft_fusion;
size_t endia_b200_fft_fusion_scratch_bytes(void);
int endia_b200_fft_c2c_fused(const endia_b200_tensor *in, const endia_b200_tensor *out,
                             const int32_t *dims, int32_t n_dims, int inverse, float scale,
                             void *scratch, const endia_b200_fft_fusion *fusion, void *stream);
/* The same loss term (reduce = 1 or 2, as above) in one pass over a contiguous complex array `y`
 * that exists already. */
int endia_b200_fft_loss_term(const endia_b200_tensor *y, int reduce, const float *reduce_w,
                             float *reduce_out, float reduce_scale, void *reduce_scratch, void *stream);

/* ------------------------------------------------------------- collectives ---- */

/* One NCCL communicator per (process, device); libnccl.so.2 is opened at first use
 * (ENDIA_B200_ENODEV when it cannot be). The reference has no communication layer
 * (single-process, single-threaded graph walk, endia/autograd/functional.mojo:26-67); these are the
 * two exchange steps of its sharded forms: the sum of the per-rank gradients of a data-parallel
 * train step (matmul_vjp's dW, endia/functional/binary_ops/matmul_op.mojo:278-284, summed before
 * Adam.step, endia/optim/adam.mojo:47-65) and the slab transpose between the axes of fftn
 * (the per-dimension gather of endia/functional/fft_ops/fft_cooley_tukey.mojo:251-257).
 *   comm_unique_id: rank 0 fills a 128-byte id and hands it to the other ranks by any host channel.
 *   comm_init:      collective over the ranks; endia_b200_init must have selected the device.
 *   allreduce_sum_f32: recv[i] = sum over ranks of send[i]; send == recv allowed.
 *   alltoall_bytes: block p (bytes_per_peer bytes) of `send` goes to rank p, whose block with this
 *                   rank's index lands in block p of `recv`; send and recv must not overlap.
 * All calls are ordered on `stream`. */
#define ENDIA_B200_COMM_ID_BYTES 128
int endia_b200_comm_unique_id(void *id128);
int endia_b200_comm_init(int32_t rank, int32_t nranks, const void *id128, void **comm_out);
int endia_b200_comm_destroy(void *comm);
int endia_b200_allreduce_sum_f32(void *comm, const float *send, float *recv, int64_t count, void *stream);
int endia_b200_alltoall_bytes(void *comm, const void *send, void *recv, int64_t bytes_per_peer,
                              void *stream);

/* ---------------------------------------------- memory shared between ranks ---- */

/* dst = src for two views of the same shape that may both be strided (the last dim contiguous on
 * both sides); 128-bit accesses when the runs allow. Either side may lie in another GPU's memory
 * mapped with endia_b200_ipc_open (plain loads and stores over NVLink). Used by the slab-
 * decomposed fftn to write each rank's block of the transpose straight into its place in the
 * receiving rank's array (the gather of fft_cooley_tukey.mojo:251-257, across GPUs). */
int endia_b200_copy_strided(const endia_b200_tensor *src, const endia_b200_tensor *dst, void *stream);

/* The receiving side of an all-gather done with peer copies (dist.ShardedAdam): `w` holds this
 * rank's updated slice [rank * numel/world, (rank+1) * numel/world); the other ranks have copied
 * theirs into `inbox` (numel floats, laid out like w) with endia_b200_d2d. Moves those slices
 * into w and, when pair16 is not NULL, writes the bf16 operand parts of the whole of w
 * ([bf16(w) | bf16(w - tf32(w))], as endia_b200_bf16_split) in the same pass.
 * numel must be a multiple of 8 * world. No counterpart in the reference (it has no multi-GPU path). */
int endia_b200_gather_slices(float *w, const float *inbox, int64_t numel, int32_t rank, int32_t world,
                             void *pair16, void *stream);

/* A device allocation that other processes on the same machine can map (CUDA IPC):
 *   ipc_alloc: allocates `bytes` and fills a 64-byte handle to pass to the other ranks
 *   ipc_open:  maps another process's allocation from its handle (peer access over NVLink)
 *   ipc_close / ipc_free: unmap a peer's allocation / free an own one (after all peers closed it)
 * The caller orders accesses between ranks itself (a collective on the stream serves as barrier). */
#define ENDIA_B200_IPC_HANDLE_BYTES 64
int endia_b200_ipc_alloc(size_t bytes, void **ptr, void *handle64);
int endia_b200_ipc_open(const void *handle64, void **ptr);
int endia_b200_ipc_close(void *ptr);
int endia_b200_ipc_free(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* ENDIA_B200_H */
