// GEMMs with a degenerate dimension: N <= 8 (matrix times a few vectors: a layer with one output,
// its dW = a^T g), M <= 8 (a few vectors times a matrix) and K <= 8 (a sum of a few outer products:
// dX = g W^T through such a layer). Tiled kernels waste almost all of a 128 x 128 tile on them;
// these are bound by reading (or writing) the one large operand once, with 16-byte accesses and
// four of them in flight per thread. Same operand conventions and fused epilogue (without the
// column sum) as the other GEMM kernels; sums run in a fixed order.
// Replaces matmul_fwd (endia/functional/binary_ops/matmul_op.mojo:93-254) for these shapes.
#include "common.cuh"
#include "gemm.cuh"

namespace eb {

constexpr int SKINNY_MAX = 8;

// The product seen from its large operand `big`; the other operand has S <= 8 vectors of length K.
struct SkinnyArgs {
  const float *big;
  int64_t ld_big;       // rows kernel: big is [R][K]; tall kernel: big is [K][R]
  const float *small;
  int64_t sk, ss;       // small(k, s) = small[k * sk + s * ss]
  int64_t R, K;
  int S;
  int swap;             // the sum for (r, s) is C[r, s] (0) or C[s, r] (1)
  int vec_big;          // 16-byte aligned base and leading dimension of big
  int vec_small;        // sk == 1 and every vector of small starts on a 16-byte boundary
};

__device__ __forceinline__ void skinny_store(const GemmParams &p, const SkinnyArgs &a, int split, bool to_partial,
                                             int64_t r, int s, float v) {
  const int64_t m = a.swap ? s : r, n = a.swap ? r : s;
  if (to_partial) p.partial[((int64_t)split * p.M + m) * p.ld_partial + n] = v;
  else p.C[m * p.ldc + n] = apply_epilogue(p.epi, v, m, n, p.C + m * p.ldc + n);
}

// big stored [R, K] (the reduction runs along its rows): one warp per row, lanes stride over k.
template <int SS>
__global__ void __launch_bounds__(256) skinny_rows_kernel(GemmParams p, SkinnyArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < a.R; r += warps) {
    float acc[SS];
#pragma unroll
    for (int s = 0; s < SS; ++s) acc[s] = 0.f;
    const float *row = a.big + r * a.ld_big;
    if (a.vec_big && (a.K & 3) == 0) {
      const int64_t K4 = a.K >> 2;
      const float4 *row4 = reinterpret_cast<const float4 *>(row);
      for (int64_t q0 = lane; q0 < K4; q0 += 128) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t q = q0 + 32 * u;
          v[u] = q < K4 ? __ldg(row4 + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int64_t k = (q0 + 32 * u) * 4;
          if (k < a.K) {
#pragma unroll
            for (int s = 0; s < SS; ++s) {
              if (s < a.S) {
                float4 b;
                if (a.vec_small) {
                  b = __ldg(reinterpret_cast<const float4 *>(a.small + s * a.ss + k));
                } else {
                  const float *bp = a.small + k * a.sk + s * a.ss;
                  b = make_float4(__ldg(bp), __ldg(bp + a.sk), __ldg(bp + 2 * a.sk), __ldg(bp + 3 * a.sk));
                }
                acc[s] = fmaf(v[u].w, b.w, fmaf(v[u].z, b.z, fmaf(v[u].y, b.y, fmaf(v[u].x, b.x, acc[s]))));
              }
            }
          }
        }
      }
    } else {
      for (int64_t k = lane; k < a.K; k += 32) {
        const float x = __ldg(row + k);
#pragma unroll
        for (int s = 0; s < SS; ++s)
          if (s < a.S) acc[s] = fmaf(x, __ldg(a.small + k * a.sk + s * a.ss), acc[s]);
      }
    }
#pragma unroll
    for (int s = 0; s < SS; ++s) {
      float v = acc[s];
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == s && s < a.S) skinny_store(p, a, 0, false, r, s, v);
    }
  }
}

// big stored [K, R] (the reduction runs down its columns): a CTA takes 128 columns x one K range,
// a thread four columns x every eighth k of the range; the eight slices are added in order through
// shared memory. With gridDim.y > 1 the sums of the K ranges go to p.partial.
template <int SS>
__global__ void __launch_bounds__(256) skinny_tall_kernel(GemmParams p, SkinnyArgs a, int64_t k_per_split) {
  __shared__ float part[8][SS][128];
  const int xq = threadIdx.x & 31, ky = threadIdx.x >> 5;
  const int64_t x0 = (int64_t)blockIdx.x * 128 + xq * 4;
  const int64_t k_begin = (int64_t)blockIdx.y * k_per_split;
  const int64_t k_end = k_begin + k_per_split < a.K ? k_begin + k_per_split : a.K;
  const bool full = a.vec_big && x0 + 4 <= a.R;
  float acc[SS][4];
#pragma unroll
  for (int s = 0; s < SS; ++s)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[s][j] = 0.f;
  for (int64_t k = k_begin + ky; k < k_end; k += 32) {
    float4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t kk = k + 8 * u;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (kk < k_end) {
        const float *src = a.big + kk * a.ld_big + x0;
        if (full) {
          v[u] = __ldg(reinterpret_cast<const float4 *>(src));
        } else {
          if (x0 < a.R) v[u].x = __ldg(src);
          if (x0 + 1 < a.R) v[u].y = __ldg(src + 1);
          if (x0 + 2 < a.R) v[u].z = __ldg(src + 2);
          if (x0 + 3 < a.R) v[u].w = __ldg(src + 3);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t kk = k + 8 * u;
      if (kk < k_end) {
#pragma unroll
        for (int s = 0; s < SS; ++s) {
          if (s < a.S) {
            const float b = __ldg(a.small + kk * a.sk + s * a.ss);
            acc[s][0] = fmaf(v[u].x, b, acc[s][0]);
            acc[s][1] = fmaf(v[u].y, b, acc[s][1]);
            acc[s][2] = fmaf(v[u].z, b, acc[s][2]);
            acc[s][3] = fmaf(v[u].w, b, acc[s][3]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int s = 0; s < SS; ++s)
    *reinterpret_cast<float4 *>(&part[ky][s][xq * 4]) = make_float4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]);
  __syncthreads();
  const bool to_partial = gridDim.y > 1;
  for (int o = threadIdx.x; o < SS * 128; o += 256) {
    const int s = o >> 7, xl = o & 127;
    const int64_t x = (int64_t)blockIdx.x * 128 + xl;
    if (s < a.S && x < a.R) {
      float v = 0.f;
#pragma unroll
      for (int y = 0; y < 8; ++y) v += part[y][s][xl];
      skinny_store(p, a, (int)blockIdx.y, to_partial, x, s, v);
    }
  }
}

// K <= 8: every output element is a short sum of products; a thread writes four consecutive n.
__global__ void __launch_bounds__(256) skinny_outer_kernel(GemmParams p, int ta, int tb, int vec) {
  const int64_t N4 = (p.N + 3) >> 2, total = p.M * N4;
  const bool narrow = total < ((int64_t)1 << 31);
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int64_t m = narrow ? (int64_t)((uint32_t)i / (uint32_t)N4) : i / N4;
    const int64_t n0 = (i - m * N4) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < SKINNY_MAX; ++k) {
      if (k < p.K) {
        const float x = ta ? __ldg(p.A + k * p.lda + m) : __ldg(p.A + m * p.lda + k);
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (vec && !tb) {
          b = __ldg(reinterpret_cast<const float4 *>(p.B + k * p.ldb + n0));
        } else {
          const int64_t sn = tb ? p.ldb : 1;
          const float *bp = tb ? p.B + n0 * p.ldb + k : p.B + k * p.ldb + n0;
          b.x = __ldg(bp);
          if (n0 + 1 < p.N) b.y = __ldg(bp + sn);
          if (n0 + 2 < p.N) b.z = __ldg(bp + 2 * sn);
          if (n0 + 3 < p.N) b.w = __ldg(bp + 3 * sn);
        }
        acc[0] = fmaf(x, b.x, acc[0]);
        acc[1] = fmaf(x, b.y, acc[1]);
        acc[2] = fmaf(x, b.z, acc[2]);
        acc[3] = fmaf(x, b.w, acc[3]);
      }
    }
    float *c = p.C + m * p.ldc + n0;
    if (vec) {
      float4 o;
      o.x = apply_epilogue(p.epi, acc[0], m, n0, c);
      o.y = apply_epilogue(p.epi, acc[1], m, n0 + 1, c + 1);
      o.z = apply_epilogue(p.epi, acc[2], m, n0 + 2, c + 2);
      o.w = apply_epilogue(p.epi, acc[3], m, n0 + 3, c + 3);
      *reinterpret_cast<float4 *>(c) = o;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + j < p.N) c[j] = apply_epilogue(p.epi, acc[j], m, n0 + j, c + j);
    }
  }
}

bool skinny_gemm_supported(const GemmParams &p, int trans_b, int64_t batch) {
  (void)trans_b;
  if (batch != 1 || p.epi.colsum_partial) return false;
  if (p.N <= SKINNY_MAX && p.M >= 32) return true;
  if (p.K <= SKINNY_MAX && p.K >= 1 && p.M * p.N >= 4096) return true;
  return p.M <= SKINNY_MAX && p.N >= 256 && p.K >= 64;
}

static bool aligned16(const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

template <int SS>
static int launch_rows(const GemmParams &p, const SkinnyArgs &a, cudaStream_t s) {
  skinny_rows_kernel<SS><<<grid_for(a.R * 32, 256), 256, 0, s>>>(p, a);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

template <int SS>
static int launch_tall(const GemmParams &p, const SkinnyArgs &a, cudaStream_t s) {
  // K ranges over CTAs until the machine is filled twice; a range keeps at least 32 k (eight
  // slices of four loads in flight)
  const int64_t ctas_x = ceil_div(a.R, 128);
  int64_t splits = ceil_div((int64_t)2 * (sm_count() > 0 ? sm_count() : 148), ctas_x);
  if (splits > a.K / 32) splits = a.K / 32;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  const int64_t k_per = ceil_div(a.K, splits);
  splits = ceil_div(a.K, k_per);
  GemmParams q = p;
  float *partial = nullptr;
  if (splits > 1) {
    q.ld_partial = (p.N + 3) / 4 * 4;
    EB_CUDA(cudaMallocAsync(&partial, sizeof(float) * (size_t)splits * p.M * q.ld_partial, s));
    q.partial = partial;
  }
  skinny_tall_kernel<SS><<<dim3((unsigned)ctas_x, (unsigned)splits), 256, 0, s>>>(q, a, k_per);
  count_launch();
  cudaError_t e = cudaGetLastError();
  int st = ENDIA_B200_OK;
  if (e != cudaSuccess) {
    set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e), __FILE__, __LINE__);
    st = ENDIA_B200_ECUDA;
  }
  if (partial) {
    if (st == ENDIA_B200_OK) st = launch_splitk_finish(q, (int)splits, s);
    cudaFreeAsync(partial, s);
  }
  return st;
}

int launch_gemm_skinny(const GemmParams &p, int trans_a, int trans_b, cudaStream_t s) {
  const bool small_n = p.N <= SKINNY_MAX && p.M >= 32 && !(p.K <= SKINNY_MAX && p.N > 2);
  const bool small_k = !small_n && p.K <= SKINNY_MAX && p.K >= 1 && p.M * p.N >= 4096;
  if (small_k) {
    const int vec = p.vec_c && p.N % 4 == 0 && (trans_b || p.vec_b);
    skinny_outer_kernel<<<grid_for(p.M * ceil_div(p.N, 4), 256), 256, 0, s>>>(p, trans_a, trans_b, vec);
    EB_LAUNCH_CHECK();
    return ENDIA_B200_OK;
  }
  SkinnyArgs a;
  bool rows;
  if (small_n) {
    // the large operand is A; the vectors are the columns of the logical B
    a.big = p.A; a.ld_big = p.lda; a.R = p.M; a.S = (int)p.N; a.swap = 0; a.vec_big = p.vec_a;
    a.small = p.B; a.sk = trans_b ? 1 : p.ldb; a.ss = trans_b ? p.ldb : 1;
    rows = !trans_a;
  } else {
    // the large operand is B; the vectors are the rows of the logical A
    a.big = p.B; a.ld_big = p.ldb; a.R = p.N; a.S = (int)p.M; a.swap = 1; a.vec_big = p.vec_b;
    a.small = p.A; a.sk = trans_a ? p.lda : 1; a.ss = trans_a ? 1 : p.lda;
    rows = trans_b != 0;
  }
  a.K = p.K;
  a.vec_small = a.sk == 1 && aligned16(a.small) && (a.S == 1 || a.ss % 4 == 0);
  const int ss = a.S <= 1 ? 1 : a.S <= 2 ? 2 : a.S <= 4 ? 4 : 8;
  if (rows) {
    switch (ss) {
      case 1: return launch_rows<1>(p, a, s);
      case 2: return launch_rows<2>(p, a, s);
      case 4: return launch_rows<4>(p, a, s);
      default: return launch_rows<8>(p, a, s);
    }
  }
  switch (ss) {
    case 1: return launch_tall<1>(p, a, s);
    case 2: return launch_tall<2>(p, a, s);
    case 4: return launch_tall<4>(p, a, s);
    default: return launch_tall<8>(p, a, s);
  }
}

}  // namespace eb
