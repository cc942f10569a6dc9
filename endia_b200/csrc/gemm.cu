// endia_b200_gemm: argument checks, algorithm choice and the second stage of the fused
// column sum. Replaces matmul_fwd and the two products of matmul_vjp
// (endia/functional/binary_ops/matmul_op.mojo:93-254, 257-284).
#include "common.cuh"
#include "gemm.cuh"

using namespace eb;

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" {

size_t endia_b200_gemm_colsum_scratch_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  // One row of partial sums per 32 rows of C: the tensor-core epilogue writes one per warp (32
  // rows), the FFMA kernel one per 128-row tile.
  return sizeof(float) * (size_t)ceil_div(M, 32) * (size_t)N;
}

int endia_b200_gemm(int trans_a, int trans_b, int64_t M, int64_t N, int64_t K, const float *A,
                    int64_t lda, const float *B, int64_t ldb, float *C, int64_t ldc, int64_t batch,
                    int64_t stride_a, int64_t stride_b, int64_t stride_c,
                    const endia_b200_epilogue *epi, int algo, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, ENDIA_B200_EINVAL, "gemm: negative size");
  if (M == 0 || N == 0 || batch == 0) return ENDIA_B200_OK;
  EB_REQUIRE(C != nullptr && (K == 0 || (A && B)), ENDIA_B200_EINVAL, "gemm: NULL pointer");
  EB_REQUIRE(lda >= (trans_a ? M : K) && ldb >= (trans_b ? K : N) && ldc >= N, ENDIA_B200_EINVAL,
             "gemm: leading dimension too small (lda %lld, ldb %lld, ldc %lld)", (long long)lda,
             (long long)ldb, (long long)ldc);
  EB_REQUIRE(stride_a >= 0 && stride_b >= 0 && stride_c >= 0, ENDIA_B200_EINVAL,
             "gemm: negative batch stride");
  EB_REQUIRE(algo >= ENDIA_B200_GEMM_AUTO && algo <= ENDIA_B200_GEMM_TF32_BF16X2, ENDIA_B200_EINVAL,
             "gemm: unknown algo %d", algo);
  GemmParams p{};
  p.A = A; p.B = B; p.C = C;
  p.M = M; p.N = N; p.K = K; p.lda = lda; p.ldb = ldb; p.ldc = ldc;
  p.stride_a = stride_a; p.stride_b = stride_b; p.stride_c = stride_c;
  p.vec_a = aligned16(A) && lda % 4 == 0 && stride_a % 4 == 0;
  p.vec_b = aligned16(B) && ldb % 4 == 0 && stride_b % 4 == 0;
  p.vec_c = aligned16(C) && ldc % 4 == 0 && stride_c % 4 == 0;
  p.epi.alpha = 1.f;
  float *colsum = nullptr;
  if (epi) {
    p.epi.alpha = epi->alpha; p.epi.beta = epi->beta; p.epi.bias = epi->bias;
    p.epi.act = epi->act; p.epi.dact = epi->dact; p.epi.dact_src = epi->dact_src;
    p.epi.ld_dact = epi->ld_dact;
    p.a_lo = epi->a_lo; p.b_lo = epi->b_lo;
    p.a16 = epi->a16; p.b16 = epi->b16;
    if (epi->c16) {
      EB_REQUIRE(batch == 1 && ldc == N && (M * N) % 8 == 0 && aligned16(C) && aligned16(epi->c16), ENDIA_B200_EINVAL,
                 "gemm: c16 needs batch == 1, ldc == N, M*N %% 8 == 0 and 16-byte aligned C and c16");
      p.epi.c16 = epi->c16;
      p.epi.c16_lo = M * N;
    }
    EB_REQUIRE(epi->act >= 0 && epi->act <= ENDIA_B200_ACT_SIGMOID && epi->dact >= 0 &&
                   epi->dact <= ENDIA_B200_ACT_SIGMOID, ENDIA_B200_EINVAL, "gemm: unknown activation");
    EB_REQUIRE(epi->dact == 0 || (epi->dact_src && epi->ld_dact >= N), ENDIA_B200_EINVAL,
               "gemm: dact needs dact_src with ld_dact >= N");
    if (epi->colsum) {
      EB_REQUIRE(epi->colsum_scratch != nullptr, ENDIA_B200_EINVAL,
                 "gemm: colsum needs colsum_scratch (endia_b200_gemm_colsum_scratch_bytes)");
      EB_REQUIRE(batch == 1, ENDIA_B200_EINVAL, "gemm: colsum supports batch == 1 only");
      colsum = epi->colsum;
      p.epi.colsum_partial = epi->colsum_scratch;
    }
  }
  cudaStream_t s = as_stream(stream);
  bool use_tc = false;
  if (algo != ENDIA_B200_GEMM_FFMA) {
    use_tc = tc_gemm_supported(p, trans_a, trans_b, batch, algo != ENDIA_B200_GEMM_AUTO);
    // AUTO takes the bf16-compensated scheme where the two-CTA kernel applies (N >= 256).
    p.scheme_forced = algo != ENDIA_B200_GEMM_AUTO;
    p.scheme = algo == ENDIA_B200_GEMM_3XTF32 ? 0 : (algo == ENDIA_B200_GEMM_TF32_BF16X2 ? 1 : tc_default_scheme());
    if (N < 256) {
      EB_REQUIRE(algo != ENDIA_B200_GEMM_TF32_BF16X2, ENDIA_B200_EINVAL, "gemm: TF32_BF16X2 needs N >= 256");
      p.scheme = 0;
    }
    EB_REQUIRE(use_tc || algo == ENDIA_B200_GEMM_AUTO, ENDIA_B200_EINVAL,
               "gemm: the 3xTF32 tcgen05 kernel does not take this shape/alignment "
               "(M %lld N %lld K %lld batch %lld)", (long long)M, (long long)N, (long long)K,
               (long long)batch);
  }
  // rows of C per partial column sum: 32 in the two-CTA tensor-core kernel, 128 in the FFMA kernel
  int tile_m = (use_tc && colsum) ? 32 : 128;
  bool c16_written = false;
  void *c16 = p.epi.c16;
  if (!use_tc && algo == ENDIA_B200_GEMM_AUTO && skinny_gemm_supported(p, trans_b, batch)) {
    p.epi.c16 = nullptr;
    if ((st = launch_gemm_skinny(p, trans_a, trans_b, s))) return st;
    if (c16) return launch_bf16_split(C, c16, static_cast<char *>(c16) + 2 * M * N, 1, M * N, M * N, M * N, s);
    return ENDIA_B200_OK;
  }
  if (use_tc) {
    st = launch_gemm_tc(p, trans_a, trans_b, s, &c16_written);
  } else {
    p.epi.c16 = nullptr;
    st = launch_gemm_ffma(p, trans_a, trans_b, batch, s);
  }
  if (st) return st;
  if (c16 && !c16_written &&      // a kernel without that epilogue ran: one pass over C
      (st = launch_bf16_split(C, c16, static_cast<char *>(c16) + 2 * M * N, 1, M * N, M * N, M * N, s)))
    return st;
  if (colsum) return launch_colsum_finish(p.epi.colsum_partial, colsum, N, (int)ceil_div(M, tile_m), 1, s);
  return ENDIA_B200_OK;
}

}  // extern "C"

extern "C" int endia_b200_bf16_split(const float *x, void *pair16, int64_t numel, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(numel >= 0, ENDIA_B200_EINVAL, "bf16_split: negative size");
  if (numel == 0) return ENDIA_B200_OK;
  EB_REQUIRE(x && pair16 && numel % 8 == 0 && aligned16(x) && aligned16(pair16), ENDIA_B200_EINVAL,
             "bf16_split: numel must be a multiple of 8 and the pointers 16-byte aligned");
  return launch_bf16_split(x, pair16, static_cast<char *>(pair16) + 2 * numel, 1, numel, numel, numel,
                           as_stream(stream));
}

extern "C" int endia_b200_tf32_split(const float *x, float *lo, int64_t rows, int64_t cols, int64_t ld_in,
                                     int64_t ld_out, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(rows >= 0 && cols >= 0, ENDIA_B200_EINVAL, "tf32_split: negative size");
  if (rows == 0 || cols == 0) return ENDIA_B200_OK;
  EB_REQUIRE(x && lo, ENDIA_B200_EINVAL, "tf32_split: NULL pointer");
  EB_REQUIRE(cols % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && ld_in >= cols && ld_out >= cols &&
                 aligned16(x) && aligned16(lo), ENDIA_B200_EINVAL,
             "tf32_split: cols and leading dimensions must be multiples of 4 and pointers 16-byte aligned");
  return launch_tf32_split(x, lo, rows, cols, ld_in, ld_out, as_stream(stream));
}
