// fp32 FFMA GEMM (128x128x16 tiles, 8x8 outputs per thread) with the fused epilogue of
// endia_b200_epilogue. It serves every shape (any M, N, K, leading dimension, alignment) and is
// the exact-fp32 arm beside the tcgen05 3xTF32 kernel. Replaces the dot-product loops of
// matmul_fwd (endia/functional/binary_ops/matmul_op.mojo:162-199) and the transposing copies
// in front of them (matmul_op.mojo:107-136).
#include "common.cuh"
#include "gemm.cuh"

namespace eb {

constexpr int BM = 128, BN = 128, BK = 16;

// One operand tile (BK x 128 in shared memory, k-major rows) fetched as 2 float4 per thread.
// MN_CONTIG: the operand's m (or n) index is contiguous in global memory.
template <bool MN_CONTIG>
struct TileLoader {
  float4 r[2];
  __device__ __forceinline__ void load(const float *__restrict__ g, int64_t ld, int64_t mn0,
                                       int64_t k0, int64_t MN, int64_t K, bool vec_ok) {
    const int tid = threadIdx.x;
    const bool full = vec_ok && (mn0 + 128 <= MN) && (k0 + BK <= K);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int f = tid + i * 256;
      if constexpr (MN_CONTIG) {
        const int k = f >> 5, c4 = (f & 31) * 4;
        const float *src = g + (k0 + k) * ld + mn0 + c4;
        if (full) {
          r[i] = __ldg(reinterpret_cast<const float4 *>(src));
        } else {
          float v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[j] = (k0 + k < K && mn0 + c4 + j < MN) ? __ldg(src + j) : 0.f;
          r[i] = make_float4(v[0], v[1], v[2], v[3]);
        }
      } else {
        const int mn = f & 127, k4 = (f >> 7) * 4;
        const float *src = g + (mn0 + mn) * ld + k0 + k4;
        if (full) {
          r[i] = __ldg(reinterpret_cast<const float4 *>(src));
        } else {
          float v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[j] = (mn0 + mn < MN && k0 + k4 + j < K) ? __ldg(src + j) : 0.f;
          r[i] = make_float4(v[0], v[1], v[2], v[3]);
        }
      }
    }
  }
  __device__ __forceinline__ void store(float (*s)[128]) const {
    const int tid = threadIdx.x;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int f = tid + i * 256;
      if constexpr (MN_CONTIG) {
        const int k = f >> 5, c4 = (f & 31) * 4;
        *reinterpret_cast<float4 *>(&s[k][c4]) = r[i];
      } else {
        const int mn = f & 127, k4 = (f >> 7) * 4;
        s[k4 + 0][mn] = r[i].x; s[k4 + 1][mn] = r[i].y;
        s[k4 + 2][mn] = r[i].z; s[k4 + 3][mn] = r[i].w;
      }
    }
  }
};

template <bool TA, bool TB>
__global__ void __launch_bounds__(256, 2) gemm_ffma_kernel(GemmParams p) {
  __shared__ __align__(16) float As[2][BK][128];
  __shared__ __align__(16) float Bs[2][BK][128];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int64_t bz = blockIdx.z;
  const float *A = p.A + bz * p.stride_a;
  const float *B = p.B + bz * p.stride_b;
  float *C = p.C + bz * p.stride_c;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  // A is m-contiguous when stored [K,M] (trans_a); B is n-contiguous when stored [K,N].
  TileLoader<TA> la;
  TileLoader<!TB> lb;
  const int64_t nk = (p.K + BK - 1) / BK;
  la.load(A, p.lda, m0, 0, p.M, p.K, p.vec_a);
  lb.load(B, p.ldb, n0, 0, p.N, p.K, p.vec_b);
  la.store(As[0]);
  lb.store(Bs[0]);
  __syncthreads();
  int buf = 0;
  for (int64_t kt = 0; kt < nk; ++kt) {
    if (kt + 1 < nk) {
      la.load(A, p.lda, m0, (kt + 1) * BK, p.M, p.K, p.vec_a);
      lb.load(B, p.ldb, n0, (kt + 1) * BK, p.N, p.K, p.vec_b);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[8], b[8];
      *reinterpret_cast<float4 *>(&a[0]) = *reinterpret_cast<const float4 *>(&As[buf][k][ty * 4]);
      *reinterpret_cast<float4 *>(&a[4]) = *reinterpret_cast<const float4 *>(&As[buf][k][64 + ty * 4]);
      *reinterpret_cast<float4 *>(&b[0]) = *reinterpret_cast<const float4 *>(&Bs[buf][k][tx * 4]);
      *reinterpret_cast<float4 *>(&b[4]) = *reinterpret_cast<const float4 *>(&Bs[buf][k][64 + tx * 4]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < nk) {
      la.store(As[buf ^ 1]);
      lb.store(Bs[buf ^ 1]);
    }
    __syncthreads();
    buf ^= 1;
  }

  // ---- fused epilogue
  float colpart[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) colpart[j] = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t m = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
    if (m >= p.M) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int64_t nb = n0 + tx * 4 + jh * 64;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t n = nb + j;
        float x = acc[i][jh * 4 + j];
        if (n < p.N) x = apply_epilogue(p.epi, x, m, n, C + m * p.ldc + n);
        else x = 0.f;
        v[j] = x;
        colpart[jh * 4 + j] += x;
      }
      if (p.vec_c && nb + 3 < p.N) {
        *reinterpret_cast<float4 *>(C + m * p.ldc + nb) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (nb + j < p.N) C[m * p.ldc + nb + j] = v[j];
      }
    }
  }
  if (p.epi.colsum_partial) {
    // Sum the 16 row-groups of this tile in a fixed order, then one row of partials per tile.
    float(*red)[128] = As[0];  // 16 x 128 floats, free after the main loop
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) red[ty][tx * 4 + (j & 3) + (j >> 2) * 64] = colpart[j];
    __syncthreads();
    if (tid < 128) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < 16; ++r) s += red[r][tid];
      const int64_t n = n0 + tid;
      if (n < p.N)
        p.epi.colsum_partial[(bz * gridDim.y + blockIdx.y) * p.N + n] = s;
    }
  }
}

// Complex product, 16x16 tiles in shared memory; operands addressed through element strides.
__global__ void __launch_bounds__(256)
gemm_complex_kernel(const float2 *A, const float2 *B, float2 *C, int64_t M, int64_t N, int64_t K,
                    int64_t sam, int64_t sak, int64_t sbk, int64_t sbn, int64_t ldc,
                    int64_t stride_a, int64_t stride_b, int64_t stride_c) {
  __shared__ float2 As[16][17], Bs[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m = (int64_t)blockIdx.y * 16 + ty, n = (int64_t)blockIdx.x * 16 + tx;
  A += blockIdx.z * stride_a; B += blockIdx.z * stride_b; C += blockIdx.z * stride_c;
  float re = 0.f, im = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += 16) {
    As[ty][tx] = (m < M && k0 + tx < K) ? A[m * sam + (k0 + tx) * sak] : make_float2(0.f, 0.f);
    Bs[ty][tx] = (k0 + ty < K && n < N) ? B[(k0 + ty) * sbk + n * sbn] : make_float2(0.f, 0.f);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float2 a = As[ty][k], b = Bs[k][tx];
      re += a.x * b.x - a.y * b.y;  // matmul_op.mojo:216-217
      im += a.x * b.y + a.y * b.x;
    }
    __syncthreads();
  }
  if (m < M && n < N) C[m * ldc + n] = make_float2(re, im);
}

__global__ void __launch_bounds__(256)
gemm_colsum_finish_kernel(const float *partial, float *out, int64_t N, int tiles, int64_t batch) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += step) {
    float acc = 0.f;
    for (int64_t t = 0; t < (int64_t)tiles * batch; ++t) acc += partial[t * N + i];
    out[i] = acc;
  }
}

int launch_colsum_finish(const float *partial, float *out, int64_t N, int tiles, int64_t batch,
                         cudaStream_t s) {
  gemm_colsum_finish_kernel<<<grid_for(N, 256), 256, 0, s>>>(partial, out, N, tiles, batch);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

int launch_gemm_ffma(const GemmParams &p, int trans_a, int trans_b, int64_t batch, cudaStream_t s) {
  dim3 grid((unsigned)ceil_div(p.N, BN), (unsigned)ceil_div(p.M, BM), (unsigned)batch);
  EB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, ENDIA_B200_ELIMIT,
             "gemm: M/128 and batch must each stay below 65536");
  if (trans_a && trans_b) gemm_ffma_kernel<true, true><<<grid, 256, 0, s>>>(p);
  else if (trans_a) gemm_ffma_kernel<true, false><<<grid, 256, 0, s>>>(p);
  else if (trans_b) gemm_ffma_kernel<false, true><<<grid, 256, 0, s>>>(p);
  else gemm_ffma_kernel<false, false><<<grid, 256, 0, s>>>(p);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

}  // namespace eb

using namespace eb;

extern "C" {

int endia_b200_gemm_complex(int trans_a, int trans_b, int64_t M, int64_t N, int64_t K,
                            const float *A, int64_t lda, const float *B, int64_t ldb, float *C,
                            int64_t ldc, int64_t batch, int64_t stride_a, int64_t stride_b,
                            int64_t stride_c, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(M >= 0 && N >= 0 && K >= 0 && batch >= 0, ENDIA_B200_EINVAL, "gemm_complex: negative size");
  if (M == 0 || N == 0 || batch == 0) return ENDIA_B200_OK;
  EB_REQUIRE(A && B && C, ENDIA_B200_EINVAL, "gemm_complex: NULL pointer");
  EB_REQUIRE(lda >= (trans_a ? M : K) && ldb >= (trans_b ? K : N) && ldc >= N, ENDIA_B200_EINVAL,
             "gemm_complex: leading dimension too small");
  dim3 grid((unsigned)ceil_div(N, 16), (unsigned)ceil_div(M, 16), (unsigned)batch);
  EB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, ENDIA_B200_ELIMIT, "gemm_complex: grid too large");
  gemm_complex_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      reinterpret_cast<const float2 *>(A), reinterpret_cast<const float2 *>(B),
      reinterpret_cast<float2 *>(C), M, N, K, trans_a ? 1 : lda, trans_a ? lda : 1,
      trans_b ? 1 : ldb, trans_b ? ldb : 1, ldc, stride_a, stride_b, stride_c);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

}  // extern "C"
