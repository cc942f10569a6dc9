// Sum reductions with a fixed (deterministic) summation tree, and the fused MSE loss.
// Replaces ReduceAdd.__call__ (endia/functional/reduce_ops/reduce_add_op.mojo:65-210), which
// accumulates sequentially in fp32, and the op chain of mse (loss_ops/mse_op.mojo:18-20).
#include "common.cuh"
#include <cuda_bf16.h>
#include <mutex>

namespace eb {

constexpr int RD = ENDIA_B200_MAX_DIMS + 1;  // +1: complex arrays get an inner (re, im) dim

struct RedParams {
  const float *in;
  float *dst;           // partials [n_out, splits] (or the output itself when splits == 1)
  int nk, nr;
  int64_t kshape[RD], kstride[RD];
  int64_t rshape[RD], rstride[RD];
  int64_t n_out, n_red;
  int splits;
  int64_t red_per_split;
  int mul;              // 1: product instead of sum (reduce_mul_op.mojo)
};

__device__ __forceinline__ int64_t offs(const int64_t *shape, const int64_t *stride, int n,
                                        int64_t i) {
  int64_t o = 0;
  for (int d = n - 1; d >= 0; --d) {
    int64_t q = i / shape[d];
    o += (i - q * shape[d]) * stride[d];
    i = q;
  }
  return o;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum of `v` over the CTA (blockDim.x a multiple of 32, at most 1024); valid in thread 0.
__device__ __forceinline__ float block_sum(float v) {
  __shared__ float warp_part[32];
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) warp_part[w] = v;
  __syncthreads();
  float r = 0.f;
  if (w == 0) {
    r = lane < (int)(blockDim.x >> 5) ? warp_part[lane] : 0.f;
    r = warp_sum(r);
  }
  return r;
}

// Product over the warp / the CTA, same shape as the sums above.
__device__ __forceinline__ float warp_prod(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v *= __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_prod(float v) {
  __shared__ float warp_part[32];
  v = warp_prod(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) warp_part[w] = v;
  __syncthreads();
  float r = 1.f;
  if (w == 0) {
    r = lane < (int)(blockDim.x >> 5) ? warp_part[lane] : 1.f;
    r = warp_prod(r);
  }
  return r;
}

// GROUP threads cooperate on one (output element, split): GROUP = 256 (a CTA), 32 (a warp) or 1.
template <int GROUP>
__global__ void __launch_bounds__(256) reduce_generic_kernel(RedParams p) {
  const int64_t n_groups = p.n_out * p.splits;
  const int groups_per_cta = 256 / GROUP;
  const int g_in_cta = threadIdx.x / GROUP;
  const int t_in_g = threadIdx.x % GROUP;
  for (int64_t gbase = (int64_t)blockIdx.x * groups_per_cta; gbase < n_groups;
       gbase += (int64_t)gridDim.x * groups_per_cta) {
    const int64_t g = gbase + g_in_cta;
    float acc = p.mul ? 1.f : 0.f;
    if (g < n_groups && p.mul) {
      const int64_t o = g / p.splits;
      const int s = (int)(g - o * p.splits);
      const int64_t base = offs(p.kshape, p.kstride, p.nk, o);
      const int64_t r0 = (int64_t)s * p.red_per_split;
      int64_t r1 = r0 + p.red_per_split;
      if (r1 > p.n_red) r1 = p.n_red;
      for (int64_t r = r0 + t_in_g; r < r1; r += GROUP)
        acc *= p.in[base + offs(p.rshape, p.rstride, p.nr, r)];
    } else if (g < n_groups) {
      const int64_t o = g / p.splits;
      const int s = (int)(g - o * p.splits);
      const int64_t base = offs(p.kshape, p.kstride, p.nk, o);
      const int64_t r0 = (int64_t)s * p.red_per_split;
      int64_t r1 = r0 + p.red_per_split;
      if (r1 > p.n_red) r1 = p.n_red;
      if (p.nr == 1 && p.rstride[0] == 1) {
        // one contiguous run: 128-bit loads over the aligned middle, scalars at the ends
        const float *src = p.in + base;
        int64_t a0 = r0, a1 = r1;
        while (a0 < a1 && (reinterpret_cast<uintptr_t>(src + a0) & 15)) ++a0;
        a1 = a0 + ((a1 - a0) & ~int64_t(3));
        for (int64_t r = r0 + t_in_g; r < a0; r += GROUP) acc += src[r];
        float a2 = 0.f, a3 = 0.f, a4 = 0.f;
        for (int64_t r = a0 + 4 * (int64_t)t_in_g; r < a1; r += 4 * GROUP) {
          const float4 v = __ldg(reinterpret_cast<const float4 *>(src + r));
          acc += v.x; a2 += v.y; a3 += v.z; a4 += v.w;
        }
        acc = (acc + a2) + (a3 + a4);
        for (int64_t r = a1 + t_in_g; r < r1; r += GROUP) acc += src[r];
      } else {
        for (int64_t r = r0 + t_in_g; r < r1; r += GROUP)
          acc += p.in[base + offs(p.rshape, p.rstride, p.nr, r)];
      }
    }
    if constexpr (GROUP == 256) {
      acc = p.mul ? block_prod(acc) : block_sum(acc);
      if (threadIdx.x == 0 && g < n_groups) p.dst[g] = acc;
    } else if constexpr (GROUP == 32) {
      acc = p.mul ? warp_prod(acc) : warp_sum(acc);
      if (t_in_g == 0 && g < n_groups) p.dst[g] = acc;
    } else {
      if (g < n_groups) p.dst[g] = acc;
    }
  }
}

// out[o] = sum_s partial[o*splits + s] (or the product, mul = 1), sequential in s.
__global__ void __launch_bounds__(256)
reduce_finish_kernel(const float *partial, float *out, int64_t n_out, int splits, float scale, int mul = 0) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; o < n_out; o += step) {
    float acc = mul ? 1.f : 0.f;
    for (int s = 0; s < splits; ++s) acc = mul ? acc * partial[o * splits + s] : acc + partial[o * splits + s];
    out[o] = acc * scale;
  }
}

// out[0] = scale * sum of `count` partials, one CTA: thread t adds partial[t], partial[t + 256], ...
// in that order and the CTA adds the 256 thread sums in a fixed tree, so the result does not depend
// on timing. (A single thread walking thousands of partials costs more than the pass that made them.)
__global__ void __launch_bounds__(256)
scalar_finish_kernel(const float *partial, float *out, int count, float scale) {
  float acc = 0.f;
  for (int i = threadIdx.x; i < count; i += 256) acc += partial[i];
  acc = block_sum(acc);
  if (threadIdx.x == 0) out[0] = acc * scale;
}

// Layout [A, R, C] with C contiguous: dst[(a*chunks + chunk)*C + c] = sum over the chunk's rows.
// VEC = 4: one thread owns 4 adjacent columns (128-bit loads).
template <int VEC>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const float *in, float *dst, int64_t R, int64_t C, int64_t a_stride,
                      int64_t r_stride, int64_t rows_per_chunk) {
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= C) return;
  const int64_t chunk = blockIdx.y, a = blockIdx.z;
  const int64_t r0 = chunk * rows_per_chunk;
  int64_t r1 = r0 + rows_per_chunk;
  if (r1 > R) r1 = R;
  const float *src = in + a * a_stride + c;
  // Eight rows are in flight per thread (eight independent 128-bit loads before the first add):
  // with two the kernel reached 47 % of the HBM copy rate. Row r goes to accumulator r % 8 and the
  // eight are added in a fixed order, so the sum does not depend on timing.
  constexpr int U = 8;
  float acc[U][VEC];
#pragma unroll
  for (int u = 0; u < U; ++u)
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[u][j] = 0.f;
  int64_t r = r0;
  for (; r + U <= r1; r += U) {
    if constexpr (VEC == 4) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = __ldg(reinterpret_cast<const float4 *>(src + (r + u) * r_stride));
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[u][0] += v[u].x; acc[u][1] += v[u].y; acc[u][2] += v[u].z; acc[u][3] += v[u].w;
      }
    } else {
      float v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = src[(r + u) * r_stride];
#pragma unroll
      for (int u = 0; u < U; ++u) acc[u][0] += v[u];
    }
  }
#pragma unroll
  for (int u = 0; u < U - 1; ++u) {      // the last rows (fewer than eight)
    if (r + u < r1) {
      if constexpr (VEC == 4) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(src + (r + u) * r_stride));
        acc[u][0] += v.x; acc[u][1] += v.y; acc[u][2] += v.z; acc[u][3] += v.w;
      } else {
        acc[u][0] += src[(r + u) * r_stride];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    const float s01 = acc[0][j] + acc[1][j], s23 = acc[2][j] + acc[3][j];
    const float s45 = acc[4][j] + acc[5][j], s67 = acc[6][j] + acc[7][j];
    dst[(a * gridDim.y + chunk) * C + c + j] = (s01 + s23) + (s45 + s67);
  }
}
// out[a*C + c] = sum over chunks in a fixed order: 32 columns x 8 chunk slices per CTA, each slice
// summed sequentially, the 8 slice sums added in order through shared memory.
__global__ void __launch_bounds__(256)
colsum_finish_kernel(const float *partial, float *out, int64_t A, int64_t C, int chunks) {
  __shared__ float part[8][33];
  const int cx = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int64_t col_blocks = (C + 31) / 32;
  for (int64_t blk = blockIdx.x; blk < A * col_blocks; blk += gridDim.x) {
    const int64_t a = blk / col_blocks, c = (blk - a * col_blocks) * 32 + cx;
    float acc = 0.f;
    if (c < C) {
      // eight loads in flight, added in the order of k
      const float *src = partial + a * chunks * C + c;
      for (int k0 = sl; k0 < chunks; k0 += 64) {
        float t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) t[u] = k0 + 8 * u < chunks ? __ldcs(src + (int64_t)(k0 + 8 * u) * C) : 0.f;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (k0 + 8 * u < chunks) acc += t[u];
      }
    }
    part[sl][cx] = acc;
    __syncthreads();
    if (sl == 0 && c < C) {
      float v = 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q) v += part[q][cx];
      out[a * C + c] = v;
    }
    __syncthreads();
  }
}

// Per-CTA partial of sum((p-t)^2); optionally writes dpred = g2n*(p-t).
__global__ void __launch_bounds__(256)
mse_partial_kernel(const float *pred, const float *target, int64_t n, float g2n, float *dpred,
                   float *partial) {
  float acc = 0.f;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  const int64_t n4 = ((reinterpret_cast<uintptr_t>(pred) | reinterpret_cast<uintptr_t>(target) |
                       reinterpret_cast<uintptr_t>(dpred)) & 15) == 0 ? n / 4 : 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += step) {
    float4 p = reinterpret_cast<const float4 *>(pred)[i];
    float4 t = reinterpret_cast<const float4 *>(target)[i];
    float4 d = make_float4(p.x - t.x, p.y - t.y, p.z - t.z, p.w - t.w);
    acc += (d.x * d.x + d.y * d.y) + (d.z * d.z + d.w * d.w);
    if (dpred)
      reinterpret_cast<float4 *>(dpred)[i] = make_float4(g2n * d.x, g2n * d.y, g2n * d.z, g2n * d.w);
  }
  for (int64_t i = n4 * 4 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    float d = pred[i] - target[i];
    acc += d * d;
    if (dpred) dpred[i] = g2n * d;
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}


// Fused activation backward + bias gradient over a contiguous [M, N] layer output:
//   dS[m,n] = grad[m,n] * act'(a[m,n]);  partial[chunk][n] = sum over the chunk's rows of dS.
// One thread owns 4 adjacent columns (VEC) or 1 and walks its chunk of rows.
template <int VEC>
__global__ void __launch_bounds__(256)
act_bwd_colsum_kernel(int act, const float *a, const float *grad, float *ds, float *partial,
                      int64_t M, int64_t N, int64_t rows_per_chunk, __nv_bfloat16 *hi16, __nv_bfloat16 *lo16) {
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= N) return;
  const int64_t r0 = (int64_t)blockIdx.y * rows_per_chunk;
  int64_t r1 = r0 + rows_per_chunk;
  if (r1 > M) r1 = M;
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  for (int64_t r = r0; r < r1; ++r) {
    float g[VEC], s[VEC];
    if constexpr (VEC == 4) {
      *reinterpret_cast<float4 *>(g) = __ldg(reinterpret_cast<const float4 *>(grad + r * N + c));
      if (act) *reinterpret_cast<float4 *>(s) = __ldg(reinterpret_cast<const float4 *>(a + r * N + c));
    } else {
      g[0] = grad[r * N + c];
      if (act) s[0] = a[r * N + c];
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float f = 1.f;
      if (act == ENDIA_B200_ACT_RELU) f = s[j] > 0.f ? 1.f : 0.f;          // relu_op.mojo:95
      else if (act == ENDIA_B200_ACT_TANH) f = 1.f - s[j] * s[j];          // tanh_op.mojo:92
      else if (act == ENDIA_B200_ACT_SIGMOID) f = s[j] * (1.f - s[j]);     // sigmoid_op.mojo:98
      g[j] *= f;
      acc[j] += g[j];
    }
    if (ds) {
      if constexpr (VEC == 4) *reinterpret_cast<float4 *>(ds + r * N + c) = *reinterpret_cast<float4 *>(g);
      else ds[r * N + c] = g[0];
    }
    if constexpr (VEC == 4) {
      if (hi16) {
        // bf16(dS) and bf16(dS - tf32(dS)): the operand parts the GEMMs that consume dS read
        float l[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) l[j] = g[j] - __uint_as_float(__float_as_uint(g[j]) & 0xFFFFE000u);
        __nv_bfloat162 h01 = __floats2bfloat162_rn(g[0], g[1]), h23 = __floats2bfloat162_rn(g[2], g[3]);
        __nv_bfloat162 l01 = __floats2bfloat162_rn(l[0], l[1]), l23 = __floats2bfloat162_rn(l[2], l[3]);
        uint2 hv, lv;
        hv.x = *reinterpret_cast<uint32_t *>(&h01); hv.y = *reinterpret_cast<uint32_t *>(&h23);
        lv.x = *reinterpret_cast<uint32_t *>(&l01); lv.y = *reinterpret_cast<uint32_t *>(&l23);
        *reinterpret_cast<uint2 *>(hi16 + r * N + c) = hv;
        *reinterpret_cast<uint2 *>(lo16 + r * N + c) = lv;
      }
    }
  }
  if (partial) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) partial[(int64_t)blockIdx.y * N + c + j] = acc[j];
  }
}

static int act_bwd_chunks(int64_t M, int64_t N) {
  const int64_t ctas_x = ceil_div(ceil_div(N, 4), 256);
  int64_t want = ceil_div((int64_t)4 * 148, ctas_x);
  const int64_t max_chunks = ceil_div(M, 8);
  if (want > max_chunks) want = max_chunks;
  if (want < 1) want = 1;
  if (want > 4096) want = 4096;
  const int64_t rows = ceil_div(M, want);
  return (int)ceil_div(M, rows);
}

struct RedPlan {
  RedParams p;
  bool colsum;       // [A, R, C] fast path
  int64_t A, R, C, a_stride, r_stride;
  int chunks;
  int64_t rows_per_chunk;
  int group;
  size_t scratch_bytes;
};

static int make_plan(const endia_b200_tensor *in, uint32_t axes_mask, RedPlan &pl, bool generic_only = false) {
  int st = check_tensor(in, "reduce_add: in");
  if (st) return st;
  // Float view of the input: complex arrays get an extra kept (re, im) dim.
  int nd = 0;
  int64_t shape[RD], stride[RD];
  bool red[RD];
  const int w = in->is_complex ? 2 : 1;
  for (int d = 0; d < in->ndim; ++d) {
    shape[nd] = in->shape[d]; stride[nd] = in->stride[d] * w;
    red[nd] = (axes_mask >> d) & 1u; ++nd;
  }
  if (in->is_complex) { shape[nd] = 2; stride[nd] = 1; red[nd] = false; ++nd; }
  RedParams &p = pl.p;
  p = RedParams{};
  p.in = static_cast<const float *>(in->data) + in->offset * w;
  p.n_out = 1; p.n_red = 1;
  // Kept and reduced dims, each collapsed where adjacent dims form one longer dim.
  for (int d = 0; d < nd; ++d) {
    if (shape[d] == 1) continue;
    if (red[d]) {
      if (p.nr > 0 && p.rstride[p.nr - 1] == stride[d] * shape[d] && d > 0 && red[d - 1]) {
        p.rshape[p.nr - 1] *= shape[d]; p.rstride[p.nr - 1] = stride[d];
      } else { p.rshape[p.nr] = shape[d]; p.rstride[p.nr] = stride[d]; ++p.nr; }
      p.n_red *= shape[d];
    } else {
      if (p.nk > 0 && p.kstride[p.nk - 1] == stride[d] * shape[d] && d > 0 && !red[d - 1]) {
        p.kshape[p.nk - 1] *= shape[d]; p.kstride[p.nk - 1] = stride[d];
      } else { p.kshape[p.nk] = shape[d]; p.kstride[p.nk] = stride[d]; ++p.nk; }
      p.n_out *= shape[d];
    }
  }
  for (int d = 0; d < nd; ++d)
    if (shape[d] == 0) { p.n_out = red[d] ? p.n_out : 0; p.n_red = red[d] ? 0 : p.n_red; }
  pl.colsum = false;
  pl.scratch_bytes = 0;
  // Column-sum fast path: one reduced dim, innermost kept dim contiguous and inside it.
  if (!generic_only && p.nr == 1 && p.nk >= 1 && p.nk <= 2 && p.kstride[p.nk - 1] == 1 &&
      p.kshape[p.nk - 1] >= 32 && p.n_red > 1) {
    pl.C = p.kshape[p.nk - 1];
    pl.R = p.rshape[0]; pl.r_stride = p.rstride[0];
    pl.A = p.nk == 2 ? p.kshape[0] : 1;
    pl.a_stride = p.nk == 2 ? p.kstride[0] : 0;
    const int64_t ctas_x = ceil_div(ceil_div(pl.C, 4), 256) * pl.A;
    int64_t want = ceil_div((int64_t)8 * 148, ctas_x);
    int64_t max_chunks = ceil_div(pl.R, 16);
    if (want > max_chunks) want = max_chunks;
    if (want < 1) want = 1;
    if (want > 65535) want = 65535;
    pl.rows_per_chunk = ceil_div(pl.R, want);
    pl.chunks = (int)ceil_div(pl.R, pl.rows_per_chunk);
    if (pl.A <= 65535) {
      pl.colsum = true;
      pl.scratch_bytes = pl.chunks > 1 ? sizeof(float) * pl.A * pl.chunks * pl.C : 0;
      return ENDIA_B200_OK;
    }
  }
  // Generic path: pick the group size from the amount of work per output element.
  pl.group = p.n_red >= 2048 ? 256 : (p.n_red >= 64 ? 32 : 1);
  p.splits = 1;
  if (pl.group == 256) {
    const int64_t target = 4 * 148;
    if (p.n_out < target) {
      int64_t s = target / (p.n_out > 0 ? p.n_out : 1);
      int64_t max_s = ceil_div(p.n_red, 4096);
      if (s > max_s) s = max_s;
      if (s < 1) s = 1;
      if (s > 4096) s = 4096;
      p.splits = (int)s;
    }
  }
  p.red_per_split = ceil_div(p.n_red > 0 ? p.n_red : 1, p.splits);
  p.splits = (int)ceil_div(p.n_red > 0 ? p.n_red : 1, p.red_per_split);
  pl.scratch_bytes = p.splits > 1 ? sizeof(float) * p.n_out * p.splits : 0;
  return ENDIA_B200_OK;
}

int launch_scalar_finish(const float *partial, float *out, int count, float scale, cudaStream_t s) {
  scalar_finish_kernel<<<1, 256, 0, s>>>(partial, out, count, scale);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

static int mse_ctas(int64_t n) {
  int64_t c = ceil_div(n, 256 * 16);
  if (c > 1024) c = 1024;
  if (c < 1) c = 1;
  return (int)c;
}

}  // namespace eb

using namespace eb;

extern "C" {

size_t endia_b200_reduce_scratch_bytes(const endia_b200_tensor *in, uint32_t axes_mask) {
  // (enough for the sum and for the product, which always takes the generic kernel)
  RedPlan pl, pg;
  if (make_plan(in, axes_mask, pl) || make_plan(in, axes_mask, pg, true)) return 0;
  return pl.scratch_bytes > pg.scratch_bytes ? pl.scratch_bytes : pg.scratch_bytes;
}

static int reduce_impl(const endia_b200_tensor *in, uint32_t axes_mask, float *out, void *scratch,
                       void *stream, int mul);

int endia_b200_reduce_add(const endia_b200_tensor *in, uint32_t axes_mask, float *out, void *scratch,
                          void *stream) {
  return reduce_impl(in, axes_mask, out, scratch, stream, 0);
}

int endia_b200_reduce_mul(const endia_b200_tensor *in, uint32_t axes_mask, float *out, void *scratch,
                          void *stream) {
  EB_REQUIRE(in && !in->is_complex, ENDIA_B200_EINVAL, "reduce_mul: real arrays only");
  return reduce_impl(in, axes_mask, out, scratch, stream, 1);
}

static int reduce_impl(const endia_b200_tensor *in, uint32_t axes_mask, float *out, void *scratch,
                       void *stream, int mul) {
  int st = require_device();
  if (st) return st;
  RedPlan pl;
  if ((st = make_plan(in, axes_mask, pl, mul != 0))) return st;
  pl.p.mul = mul;
  if (pl.p.n_out == 0) return ENDIA_B200_OK;
  EB_REQUIRE(out != nullptr, ENDIA_B200_EINVAL, "reduce_add: out is NULL");
  EB_REQUIRE(pl.scratch_bytes == 0 || scratch != nullptr, ENDIA_B200_EINVAL,
             "reduce_add: %zu bytes of scratch are required", pl.scratch_bytes);
  cudaStream_t s = as_stream(stream);
  if (pl.p.n_red == 0) {
    if (mul) return endia_b200_fill(out, pl.p.n_out, 0, 1.f, 0.f, stream);     // the empty product
    EB_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * pl.p.n_out, s));
    return ENDIA_B200_OK;
  }
  if (pl.colsum) {
    float *dst = pl.chunks > 1 ? static_cast<float *>(scratch) : out;
    const bool vec = pl.C % 4 == 0 && pl.a_stride % 4 == 0 && pl.r_stride % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(pl.p.in) & 15) == 0;
    if (vec) {
      dim3 grid((unsigned)ceil_div(pl.C / 4, 256), (unsigned)pl.chunks, (unsigned)pl.A);
      colsum_partial_kernel<4><<<grid, 256, 0, s>>>(pl.p.in, dst, pl.R, pl.C, pl.a_stride, pl.r_stride,
                                                    pl.rows_per_chunk);
    } else {
      dim3 grid((unsigned)ceil_div(pl.C, 256), (unsigned)pl.chunks, (unsigned)pl.A);
      colsum_partial_kernel<1><<<grid, 256, 0, s>>>(pl.p.in, dst, pl.R, pl.C, pl.a_stride, pl.r_stride,
                                                    pl.rows_per_chunk);
    }
    EB_LAUNCH_CHECK();
    if (pl.chunks > 1) {
      colsum_finish_kernel<<<grid_for(pl.A * ceil_div(pl.C, 32) * 256, 256), 256, 0, s>>>(
          static_cast<const float *>(scratch), out, pl.A, pl.C, pl.chunks);
      EB_LAUNCH_CHECK();
    }
    return ENDIA_B200_OK;
  }
  RedParams p = pl.p;
  p.dst = p.splits > 1 ? static_cast<float *>(scratch) : out;
  const int64_t n_groups = p.n_out * p.splits;
  if (pl.group == 256) {
    int64_t g = n_groups < (int64_t)148 * 16 ? n_groups : (int64_t)148 * 16;
    reduce_generic_kernel<256><<<(unsigned)g, 256, 0, s>>>(p);
  } else if (pl.group == 32) {
    reduce_generic_kernel<32><<<grid_for(n_groups * 32, 256), 256, 0, s>>>(p);
  } else {
    reduce_generic_kernel<1><<<grid_for(n_groups, 256), 256, 0, s>>>(p);
  }
  EB_LAUNCH_CHECK();
  if (p.splits > 1) {
    if (p.n_out == 1 && !mul)
      scalar_finish_kernel<<<1, 256, 0, s>>>(static_cast<const float *>(scratch), out, p.splits, 1.f);
    else
      reduce_finish_kernel<<<grid_for(p.n_out, 256), 256, 0, s>>>(static_cast<const float *>(scratch),
                                                                  out, p.n_out, p.splits, 1.f, mul);
    EB_LAUNCH_CHECK();
  }
  return ENDIA_B200_OK;
}

size_t endia_b200_mse_scratch_bytes(int64_t n) { return sizeof(float) * (size_t)mse_ctas(n); }

int endia_b200_mse_fwd_bwd(const float *pred, const float *target, int64_t n, float gscale,
                           float *loss, float *dpred, void *scratch, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n > 0, ENDIA_B200_EINVAL, "mse: n must be positive");
  EB_REQUIRE(pred && target && loss && scratch, ENDIA_B200_EINVAL, "mse: NULL pointer");
  cudaStream_t s = as_stream(stream);
  const int ctas = mse_ctas(n);
  // 2/n as the reference forms it: two products d*g with g = 1/n, added (mul_op.mojo:125-128,
  // autograd/functional.mojo:55-57).
  const float inv_n = 1.f / (float)n;
  const float g2n = gscale * (inv_n + inv_n);
  mse_partial_kernel<<<ctas, 256, 0, s>>>(pred, target, n, g2n, dpred, static_cast<float *>(scratch));
  EB_LAUNCH_CHECK();
  scalar_finish_kernel<<<1, 256, 0, s>>>(static_cast<const float *>(scratch), loss, ctas, inv_n);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

size_t endia_b200_act_bwd_colsum_scratch_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  return sizeof(float) * (size_t)act_bwd_chunks(M, N) * (size_t)N;
}

int endia_b200_act_bwd_colsum(int act, const float *act_out, const float *grad, float *ds,
                              float *colsum, int64_t M, int64_t N, void *scratch, void *stream) {
  return endia_b200_act_bwd_colsum_parts(act, act_out, grad, ds, colsum, M, N, scratch, nullptr, stream);
}

int endia_b200_act_bwd_colsum_parts(int act, const float *act_out, const float *grad, float *ds,
                                    float *colsum, int64_t M, int64_t N, void *scratch, void *pair16,
                                    void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(M >= 0 && N >= 0, ENDIA_B200_EINVAL, "act_bwd_colsum: negative size");
  EB_REQUIRE(act >= 0 && act <= ENDIA_B200_ACT_SIGMOID, ENDIA_B200_EINVAL,
             "act_bwd_colsum: unknown activation %d", act);
  if (M == 0 || N == 0) return ENDIA_B200_OK;
  EB_REQUIRE(grad != nullptr && (act == 0 || (act_out && ds)), ENDIA_B200_EINVAL,
             "act_bwd_colsum: NULL pointer");
  EB_REQUIRE(!colsum || scratch, ENDIA_B200_EINVAL, "act_bwd_colsum: colsum needs scratch");
  cudaStream_t s = as_stream(stream);
  const int chunks = act_bwd_chunks(M, N);
  const int64_t rows = ceil_div(M, chunks);
  float *partial = colsum ? static_cast<float *>(scratch) : nullptr;
  const bool vec = N % 4 == 0 && ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(act_out) |
                                   reinterpret_cast<uintptr_t>(ds)) & 15) == 0;
  EB_REQUIRE(!pair16 || (vec && (M * N) % 8 == 0 && (reinterpret_cast<uintptr_t>(pair16) & 15) == 0),
             ENDIA_B200_EINVAL, "act_bwd_colsum: the bf16 parts need N %% 4 == 0, M*N %% 8 == 0 and aligned arrays");
  __nv_bfloat16 *hi16 = static_cast<__nv_bfloat16 *>(pair16), *lo16 = hi16 ? hi16 + M * N : nullptr;
  if (vec) {
    dim3 grid((unsigned)ceil_div(N / 4, 256), (unsigned)chunks);
    act_bwd_colsum_kernel<4><<<grid, 256, 0, s>>>(act, act_out, grad, act ? ds : nullptr, partial, M, N, rows,
                                                  hi16, lo16);
  } else {
    dim3 grid((unsigned)ceil_div(N, 256), (unsigned)chunks);
    act_bwd_colsum_kernel<1><<<grid, 256, 0, s>>>(act, act_out, grad, act ? ds : nullptr, partial, M, N, rows,
                                                  nullptr, nullptr);
  }
  EB_LAUNCH_CHECK();
  if (colsum) {
    colsum_finish_kernel<<<grid_for(ceil_div(N, 32) * 256, 256), 256, 0, s>>>(partial, colsum, 1, N, chunks);
    EB_LAUNCH_CHECK();
  }
  return ENDIA_B200_OK;
}

// ---- allocation-free MSE --------------------------------------------------------------------
// Partial sums of the allocation-free variant live in this fixed device array instead of a
// caller-provided buffer. One partial per 4096 elements, so the array bounds the problem size.
#define EB_MSE_NOALLOC_MAX_PARTIALS 4096
#define EB_MSE_NOALLOC_ELEMS_PER_PARTIAL 4096
static __device__ __align__(256) float g_mse_noalloc_scratch[EB_MSE_NOALLOC_MAX_PARTIALS];
// Device address of the array above, looked up once per device (indexed by device ordinal).
static float *g_mse_noalloc_addr[64] = {nullptr};
static std::mutex g_mse_noalloc_mutex;

int endia_b200_mse_fwd_bwd_noalloc(const float *pred, const float *target, int64_t n, float gscale,
                                   float *loss, float *dpred, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n > 0, ENDIA_B200_EINVAL, "mse_noalloc: n must be positive");
  EB_REQUIRE(pred && target && loss, ENDIA_B200_EINVAL, "mse_noalloc: NULL pointer");
  const int64_t max_n = (int64_t)EB_MSE_NOALLOC_MAX_PARTIALS * EB_MSE_NOALLOC_ELEMS_PER_PARTIAL;
  EB_REQUIRE(n <= max_n, ENDIA_B200_ELIMIT,
             "mse_noalloc: n = %lld exceeds the fixed scratch of this entry point (at most %lld "
             "elements); use endia_b200_mse_fwd_bwd with caller-provided scratch",
             (long long)n, (long long)max_n);
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  EB_REQUIRE(dev >= 0 && dev < 64, ENDIA_B200_ELIMIT, "mse_noalloc: device ordinal %d not supported", dev);
  float *scratch = nullptr;
  {
    // Set-up on the first call per device: the array's name is only a host-side handle, the
    // kernels need its device address.
    std::lock_guard<std::mutex> lock(g_mse_noalloc_mutex);
    if (!g_mse_noalloc_addr[dev]) {
      void *addr = nullptr;
      EB_CUDA(cudaGetSymbolAddress(&addr, g_mse_noalloc_scratch));
      g_mse_noalloc_addr[dev] = static_cast<float *>(addr);
    }
    scratch = g_mse_noalloc_addr[dev];
  }
  cudaStream_t s = as_stream(stream);
  const int ctas = (int)ceil_div(n, EB_MSE_NOALLOC_ELEMS_PER_PARTIAL);
  const float inv_n = 1.f / (float)n;
  const float g2n = gscale * (inv_n + inv_n);
  // Every partial slot in [0, ctas) is overwritten by this call, so nothing has to be cleared.
  mse_partial_kernel<<<ctas, 256, 0, s>>>(pred, target, n, g2n, dpred, scratch);
  EB_LAUNCH_CHECK();
  scalar_finish_kernel<<<1, 256, 0, s>>>(scratch, loss, ctas, inv_n);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

}  // extern "C"
