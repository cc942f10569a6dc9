// GEMMs with a degenerate dimension: N <= 8 (matrix times a few vectors: a layer with one output,
// its dW = a^T g) and K <= 8 (a sum of a few outer products: dX = g W^T through such a layer).
// Tiled kernels waste almost all of a 128 x 128 tile on them; these are bound by reading (or
// writing) the one large operand once. Same operand conventions and fused epilogue (without the
// column sum) as the other GEMM kernels; sums run in a fixed order.
// Replaces matmul_fwd (endia/functional/binary_ops/matmul_op.mojo:93-254) for these shapes.
#include "common.cuh"
#include "gemm.cuh"

namespace eb {

constexpr int SKINNY_MAX = 8;

__device__ __forceinline__ float b_at(const GemmParams &p, int tb, int64_t k, int64_t n) {
  return tb ? __ldg(p.B + n * p.ldb + k) : __ldg(p.B + k * p.ldb + n);
}

// A stored [M, K] (rows contiguous): one warp per output row, lanes stride over k.
__global__ void __launch_bounds__(256) gemm_small_n_rows_kernel(GemmParams p, int tb) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t m = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); m < p.M; m += warps) {
    float acc[SKINNY_MAX];
#pragma unroll
    for (int n = 0; n < SKINNY_MAX; ++n) acc[n] = 0.f;
    const float *arow = p.A + m * p.lda;
    for (int64_t k = lane; k < p.K; k += 32) {
      const float a = __ldg(arow + k);
#pragma unroll
      for (int n = 0; n < SKINNY_MAX; ++n)
        if (n < p.N) acc[n] = fmaf(a, b_at(p, tb, k, n), acc[n]);
    }
#pragma unroll
    for (int n = 0; n < SKINNY_MAX; ++n) {
      float v = acc[n];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == n && n < p.N) p.C[m * p.ldc + n] = apply_epilogue(p.epi, v, m, n, p.C + m * p.ldc + n);
    }
  }
}

// A stored [K, M] (columns of the logical A contiguous): 32 rows x 8 k-slices per CTA, the slices
// are added in a fixed order through shared memory.
__global__ void __launch_bounds__(256) gemm_small_n_cols_kernel(GemmParams p, int tb, int64_t k_per_split) {
  __shared__ float part[8][32][SKINNY_MAX + 1];
  const int mx = threadIdx.x & 31, ky = threadIdx.x >> 5;
  const int64_t m = (int64_t)blockIdx.x * 32 + mx;
  const int64_t k_begin = (int64_t)blockIdx.y * k_per_split;
  const int64_t k_end = k_begin + k_per_split < p.K ? k_begin + k_per_split : p.K;
  float acc[SKINNY_MAX];
#pragma unroll
  for (int n = 0; n < SKINNY_MAX; ++n) acc[n] = 0.f;
  if (m < p.M) {
    for (int64_t k = k_begin + ky; k < k_end; k += 8) {
      const float a = __ldg(p.A + k * p.lda + m);
#pragma unroll
      for (int n = 0; n < SKINNY_MAX; ++n)
        if (n < p.N) acc[n] = fmaf(a, b_at(p, tb, k, n), acc[n]);
    }
  }
#pragma unroll
  for (int n = 0; n < SKINNY_MAX; ++n) part[ky][mx][n] = acc[n];
  __syncthreads();
  if (ky == 0 && m < p.M) {
    for (int n = 0; n < p.N; ++n) {
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < 8; ++s) v += part[s][mx][n];
      if (gridDim.y > 1) p.partial[((int64_t)blockIdx.y * p.M + m) * p.ld_partial + n] = v;
      else p.C[m * p.ldc + n] = apply_epilogue(p.epi, v, m, n, p.C + m * p.ldc + n);
    }
  }
}

// K <= 8: every output element is a short sum of products; consecutive threads write
// consecutive n.
__global__ void __launch_bounds__(256) gemm_small_k_kernel(GemmParams p, int ta, int tb) {
  const int64_t total = p.M * p.N;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t m = i / p.N, n = i - m * p.N;
    float v = 0.f;
    for (int64_t k = 0; k < p.K; ++k) {
      const float a = ta ? __ldg(p.A + k * p.lda + m) : __ldg(p.A + m * p.lda + k);
      v = fmaf(a, b_at(p, tb, k, n), v);
    }
    p.C[m * p.ldc + n] = apply_epilogue(p.epi, v, m, n, p.C + m * p.ldc + n);
  }
}

// M <= 8 with B stored [K, N]: threads run over n (coalesced rows of B), CTAs also split K; the
// slices are added by the split-K finishing kernel.
__global__ void __launch_bounds__(256) gemm_small_m_kernel(GemmParams p, int ta, int64_t k_per_split) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t k_begin = (int64_t)blockIdx.y * k_per_split;
  const int64_t k_end = k_begin + k_per_split < p.K ? k_begin + k_per_split : p.K;
  if (n >= p.N) return;
  float acc[SKINNY_MAX];
#pragma unroll
  for (int m = 0; m < SKINNY_MAX; ++m) acc[m] = 0.f;
  for (int64_t k = k_begin; k < k_end; ++k) {
    const float b = __ldg(p.B + k * p.ldb + n);
#pragma unroll
    for (int m = 0; m < SKINNY_MAX; ++m)
      if (m < p.M) acc[m] = fmaf(ta ? __ldg(p.A + k * p.lda + m) : __ldg(p.A + m * p.lda + k), b, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < SKINNY_MAX; ++m)
    if (m < p.M) p.partial[((int64_t)blockIdx.y * p.M + m) * p.ld_partial + n] = acc[m];
}

bool skinny_gemm_supported(const GemmParams &p, int trans_b, int64_t batch) {
  if (batch != 1 || p.epi.colsum_partial) return false;
  if (p.N <= SKINNY_MAX && p.M >= 32) return true;
  if (p.K <= SKINNY_MAX && p.K >= 1 && p.M * p.N >= 4096) return true;
  return p.M <= SKINNY_MAX && !trans_b && p.N >= 256 && p.K >= 64;
}

int launch_gemm_skinny(const GemmParams &p, int trans_a, int trans_b, cudaStream_t s) {
  const bool small_n = p.N <= SKINNY_MAX && p.M >= 32 && !(p.K <= SKINNY_MAX && p.N > 2);
  const bool small_k = !small_n && p.K <= SKINNY_MAX && p.K >= 1 && p.M * p.N >= 4096;
  if (small_n && !trans_a) {
    gemm_small_n_rows_kernel<<<grid_for(p.M * 32, 256), 256, 0, s>>>(p, trans_b);
    EB_LAUNCH_CHECK();
    return ENDIA_B200_OK;
  }
  if (small_k) {
    gemm_small_k_kernel<<<grid_for(p.M * p.N, 256), 256, 0, s>>>(p, trans_a, trans_b);
    EB_LAUNCH_CHECK();
    return ENDIA_B200_OK;
  }
  // The remaining two shapes split K over CTAs to fill the machine.
  const int64_t ctas_x = small_n ? ceil_div(p.M, 32) : ceil_div(p.N, 256);
  int64_t splits = ceil_div((int64_t)2 * 148, ctas_x);
  if (splits > p.K / 64) splits = p.K / 64;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  const int64_t k_per = ceil_div(p.K, splits);
  splits = ceil_div(p.K, k_per);
  GemmParams q = p;
  float *partial = nullptr;
  if (splits > 1 || !small_n) {
    q.ld_partial = p.N;
    EB_CUDA(cudaMallocAsync(&partial, sizeof(float) * (size_t)splits * p.M * p.N, s));
    q.partial = partial;
  }
  if (small_n) {
    gemm_small_n_cols_kernel<<<dim3((unsigned)ctas_x, (unsigned)splits), 256, 0, s>>>(q, trans_b, k_per);
  } else {
    gemm_small_m_kernel<<<dim3((unsigned)ctas_x, (unsigned)splits), 256, 0, s>>>(q, trans_a, k_per);
  }
  EB_LAUNCH_CHECK();
  int st = ENDIA_B200_OK;
  if (partial) {
    st = launch_splitk_finish(q, (int)splits, s);
    cudaFreeAsync(partial, s);
  }
  return st;
}

}  // namespace eb
