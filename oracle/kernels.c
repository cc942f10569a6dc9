/*
 * CPU restatement of the hot loops of Endia's reference implementation, used ONLY as the
 * checker for the CUDA path (tests, the smoke test and the CPU-baseline leg of the benchmark).
 * It is test infrastructure, not a product path: nothing under endia_b200/ may call it.
 *
 * Every function follows one reference loop (file:line given at the function); arithmetic is
 * float32 except the FFT core, which the reference runs in float64.
 *
 * Build: gcc -O3 -ffp-contract=off -fopenmp -shared -fPIC kernels.c -o _build/liboracle.so -lm
 * (no FMA contraction, so results do not depend on the host's instruction set).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Horizontal add of a SIMD vector by repeated halving (Mojo SIMD.reduce_add as used at
 * endia/functional/binary_ops/matmul_op.mojo:189). */
static float hadd(float *p, int n) {
  for (int h = n / 2; h >= 1; h /= 2)
    for (int i = 0; i < h; ++i) p[i] += p[i + h];
  return p[0];
}

/* C[m,n] = sum_k A[m,k] * Bt[n,k]; A is [M,K] contiguous and Bt the transposed-contiguous rhs
 * the reference materialises first (matmul_op.mojo:107-136). Per output element: `nelts`-wide
 * partial sums over k, a horizontal add, then a scalar tail (matmul_op.mojo:170-199).
 * Single-threaded, like the reference (its parallelize call is commented out, :168-169). */
void oracle_matmul_f32(const float *A, const float *Bt, float *C, int64_t M, int64_t N, int64_t K,
                       int nelts) {
  if (nelts < 1 || nelts > 64) nelts = 16;
  const int64_t k_end = K - (K % nelts);
  for (int64_t m = 0; m < M; ++m) {
    const float *a = A + m * K;
    for (int64_t n = 0; n < N; ++n) {
      const float *b = Bt + n * K;
      float part[64];
      for (int i = 0; i < nelts; ++i) part[i] = 0.f;
      for (int64_t k = 0; k < k_end; k += nelts)
        for (int i = 0; i < nelts; ++i) part[i] += a[k + i] * b[k + i];
      float s = hadd(part, nelts);
      for (int64_t k = k_end; k < K; ++k) s += a[k] * b[k];
      C[m * N + n] = s;
    }
  }
}

/* Same product with float64 accumulation and all cores: the "fast" mode that checks the large
 * configurations; it must agree with oracle_matmul_f32 on small shapes. */
void oracle_matmul_fast(const float *A, const float *Bt, float *C, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const float *a = A + m * K;
    for (int64_t n = 0; n < N; ++n) {
      const float *b = Bt + n * K;
      double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
      int64_t k = 0;
      for (; k + 3 < K; k += 4) {
        s0 += (double)a[k] * b[k];
        s1 += (double)a[k + 1] * b[k + 1];
        s2 += (double)a[k + 2] * b[k + 2];
        s3 += (double)a[k + 3] * b[k + 3];
      }
      for (; k < K; ++k) s0 += (double)a[k] * b[k];
      C[m * N + n] = (float)((s0 + s1) + (s2 + s3));
    }
  }
}

/* Complex variant: real and imaginary sums kept separately (matmul_op.mojo:200-238);
 * interleaved (re, im) storage. */
void oracle_matmul_c64(const float *A, const float *Bt, float *C, int64_t M, int64_t N, int64_t K,
                       int nelts) {
  if (nelts < 1 || nelts > 64) nelts = 16;
  const int64_t k_end = K - (K % nelts);
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      const float *a = A + 2 * m * K, *b = Bt + 2 * n * K;
      float pr[64], pi[64];
      for (int i = 0; i < nelts; ++i) pr[i] = pi[i] = 0.f;
      for (int64_t k = 0; k < k_end; k += nelts)
        for (int i = 0; i < nelts; ++i) {
          const float ar = a[2 * (k + i)], ai = a[2 * (k + i) + 1];
          const float br = b[2 * (k + i)], bi = b[2 * (k + i) + 1];
          pr[i] += ar * br - ai * bi;
          pi[i] += ar * bi + ai * br;
        }
      float sr = hadd(pr, nelts), si = hadd(pi, nelts);
      for (int64_t k = k_end; k < K; ++k) {
        const float ar = a[2 * k], ai = a[2 * k + 1], br = b[2 * k], bi = b[2 * k + 1];
        sr += ar * br - ai * bi;
        si += ar * bi + ai * br;
      }
      C[2 * (m * N + n)] = sr;
      C[2 * (m * N + n) + 1] = si;
    }
}

/* Sum of a contiguous float array over the axes flagged in `reduce`: the input is walked in
 * row-major order and every element is added into its slot of the zero-initialised output, whose
 * strides are those of the kept-dims shape with 0 on reduced axes
 * (endia/functional/reduce_ops/reduce_add_op.mojo:96-160). `width` = floats per element
 * (2 for complex). The 1-D case sums nelts-wide chunks horizontally into slot 0, then a scalar
 * tail (:162-193). */
void oracle_reduce_add(const float *in, float *out, int ndim, const int64_t *shape,
                       const int32_t *reduce, int width, int nelts) {
  int64_t tstride[16], idx[16], total = 1, out_n = 1;
  int64_t acc = 1;
  for (int d = ndim - 1; d >= 0; --d) {
    tstride[d] = reduce[d] ? 0 : acc;
    if (!reduce[d]) acc *= shape[d];
    total *= shape[d];
  }
  out_n = acc;
  memset(out, 0, sizeof(float) * (size_t)(out_n * width));
  if (total == 0) return;
  if (ndim == 1 && reduce[0] && width == 1) {
    if (nelts < 1 || nelts > 64) nelts = 16;
    const int64_t end = total - (total % nelts);
    float s = 0.f;
    for (int64_t i = 0; i < end; i += nelts) {
      float part[64];
      for (int j = 0; j < nelts; ++j) part[j] = in[i + j];
      s += hadd(part, nelts);
    }
    for (int64_t i = end; i < total; ++i) s += in[i];
    out[0] = s;
    return;
  }
  for (int d = 0; d < ndim; ++d) idx[d] = 0;
  for (int64_t i = 0; i < total; ++i) {
    int64_t t = 0;
    for (int d = 0; d < ndim; ++d) t += idx[d] * tstride[d];
    for (int w = 0; w < width; ++w) out[t * width + w] += in[i * width + w];
    for (int d = ndim - 1; d >= 0; --d) {
      if (++idx[d] < shape[d]) break;
      idx[d] = 0;
    }
  }
}

static uint32_t reverse_bits(uint32_t y) {  /* fft_ops/utils.mojo:26-38 */
  y = ((y >> 1) & 0x55555555u) | ((y & 0x55555555u) << 1);
  y = ((y >> 2) & 0x33333333u) | ((y & 0x33333333u) << 2);
  y = ((y >> 4) & 0x0F0F0F0Fu) | ((y & 0x0F0F0F0Fu) << 4);
  y = ((y >> 8) & 0x00FF00FFu) | ((y & 0x00FF00FFu) << 8);
  return (y >> 16) | (y << 16);
}

/* In-place radix-2 decimation-in-time FFT of `rows` contiguous rows of n complex float64 values:
 * bit-reversal permutation (table from a 32-bit reverse shifted by 32 - log2 n,
 * fft_ops/utils.mojo:41-69), then log2 n stages m = 2, 4, ..., n with w = cis(-2*pi/m) and the
 * twiddle u advanced by complex multiplication per k
 * (endia/functional/fft_ops/fft_cooley_tukey.mojo:133-176). Rows are independent; the reference
 * spreads them over worker threads (:272-280), here over OpenMP threads when `threads` > 1. */
void oracle_fft_rows_f64(double *data, int64_t rows, int64_t n, int threads) {
  if (n <= 1) return;
  int log2n = 0;
  while (((int64_t)1 << log2n) < n) ++log2n;
  uint32_t *rev = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)n);
  for (int64_t i = 0; i < n; ++i) rev[i] = reverse_bits((uint32_t)i) >> (32 - log2n);
  const double pi = 3.14159265358979323846;
  if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
  for (int64_t r = 0; r < rows; ++r) {
    double *x = data + 2 * r * n;
    for (int64_t i = 0; i < n; ++i) {
      const int64_t j = rev[i];
      if (i < j) {
        const double tr = x[2 * i], ti = x[2 * i + 1];
        x[2 * i] = x[2 * j]; x[2 * i + 1] = x[2 * j + 1];
        x[2 * j] = tr; x[2 * j + 1] = ti;
      }
    }
    for (int64_t m = 2; m <= n; m *= 2) {
      double ur = 1.0, ui = 0.0;
      const double angle = -2 * pi / (double)m;
      const double wr = cos(angle), wi = sin(angle);
      for (int64_t k = 0; k < m / 2; ++k) {
        for (int64_t j = k; j < n; j += m) {
          double *z = x + 2 * j, *d = x + 2 * j + m;
          const double tr = ur * d[0] - ui * d[1], ti = ur * d[1] + ui * d[0];
          d[0] = z[0] - tr; d[1] = z[1] - ti;
          z[0] = z[0] + tr; z[1] = z[1] + ti;
        }
        const double nr = ur * wr - ui * wi, ni = ur * wi + ui * wr;
        ur = nr; ui = ni;
      }
    }
  }
  free(rev);
}
