// Parameters shared by the GEMM kernels and the epilogue they all apply.
#pragma once
#include "common.cuh"

namespace eb {

struct EpiParams {
  float alpha, beta;
  const float *bias;
  int act, dact;
  const float *dact_src;
  int64_t ld_dact;
  float *colsum_partial;  // [row tiles (x batch), N] partial column sums, or NULL
  // optional: the bf16 split of the stored values (bf16(c) at c16[m*ldc + n], bf16(c - tf32(c)) at
  // c16[c16_lo + m*ldc + n], in bf16 elements), written by the two-CTA kernel's epilogue
  void *c16;
  int64_t c16_lo;
};

struct GemmParams {
  const float *A, *B;
  float *C;
  int64_t M, N, K, lda, ldb, ldc;
  int64_t stride_a, stride_b, stride_c;
  bool vec_a, vec_b, vec_c;  // 16-byte aligned base, leading dimension and batch stride
  EpiParams epi;
  // split-K: partial[split][M][ld_partial] receives the raw sums of each K range
  float *partial;
  int64_t ld_partial;
  int64_t partial_rows;   // rows per slice of `partial` (0: M)
  // optional precomputed tf32 low parts, laid out like A / B
  const float *a_lo, *b_lo;
  // optional precomputed bf16 splits of the operands' storage (endia_b200_bf16_split)
  const void *a16, *b16;
  // 0 = 3xTF32, 1 = one tf32 MMA + two bf16 correction MMAs per product
  int scheme;
  bool scheme_forced;   // the caller named the algorithm (GEMM_AUTO may fall back to 3xTF32 split-K)
};

__device__ __forceinline__ float act_fwd(int act, float v) {
  switch (act) {
    case ENDIA_B200_ACT_RELU: return fmaxf(v, 0.f);                 // relu_op.mojo:115
    case ENDIA_B200_ACT_TANH: return tanhf(v);                      // tanh_op.mojo:112-115
    case ENDIA_B200_ACT_SIGMOID: return 1.f / (1.f + expf(-v));     // sigmoid_op.mojo:118-121
    default: return v;
  }
}
// Derivative factor from the saved tensor (see endia_b200_epilogue in the public header).
__device__ __forceinline__ float act_bwd(int dact, float s) {
  switch (dact) {
    case ENDIA_B200_ACT_RELU: return s > 0.f ? 1.f : 0.f;           // relu_op.mojo:95
    case ENDIA_B200_ACT_TANH: return 1.f - s * s;                   // tanh_op.mojo:92
    case ENDIA_B200_ACT_SIGMOID: return s * (1.f - s);              // sigmoid_op.mojo:98
    default: return 1.f;
  }
}

// v = acc after the fused steps, for output element (m, n); `c_old` points at C[m,n].
__device__ __forceinline__ float apply_epilogue(const EpiParams &e, float acc, int64_t m, int64_t n,
                                                const float *c_old) {
  float v = e.alpha * acc;
  if (e.bias) v += __ldg(e.bias + n);
  if (e.act) v = act_fwd(e.act, v);
  if (e.dact) v *= act_bwd(e.dact, __ldg(e.dact_src + m * e.ld_dact + n));
  if (e.beta != 0.f) v += e.beta * (*c_old);
  return v;
}

int launch_gemm_ffma(const GemmParams &p, int trans_a, int trans_b, int64_t batch, cudaStream_t s);
int launch_colsum_finish(const float *partial, float *out, int64_t N, int tiles, int64_t batch,
                         cudaStream_t s);
// Degenerate shapes (N <= 8, K <= 8, or M <= 8 with a row-major B): one pass over the large operand.
bool skinny_gemm_supported(const GemmParams &p, int trans_b, int64_t batch);
int launch_gemm_skinny(const GemmParams &p, int trans_a, int trans_b, cudaStream_t s);
int launch_tf32_split(const float *x, float *lo, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                      cudaStream_t s);
// hi16 = bf16(x), lo16 = bf16(x - tf32(x)) for rows of `cols` floats (cols % 4 == 0).
int launch_bf16_split(const float *x, void *hi16, void *lo16, int64_t rows, int64_t cols, int64_t ld_in,
                      int64_t ld_out, cudaStream_t s);
// C = epilogue(sum over `splits` slices of p.partial, in order).
int launch_splitk_finish(const GemmParams &p, int splits, cudaStream_t s);
// tcgen05 3xTF32 path: true when the shape/alignment is one it handles.
bool tc_gemm_supported(const GemmParams &p, int trans_a, int trans_b, int64_t batch,
                       bool explicit_request);
int launch_gemm_tc(const GemmParams &p, int trans_a, int trans_b, cudaStream_t s, bool *c16_written = nullptr);
// Scheme GEMM_AUTO uses on the two-CTA kernel (1 unless ENDIA_B200_TC_SCHEME=3xtf32).
int tc_default_scheme();

}  // namespace eb
