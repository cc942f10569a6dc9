// Complex64 FFT: shared-memory Stockham kernels (radix 16/8/4/2 butterflies in registers),
// tiled over lines so that strided axes are read and written in contiguous segments, and a
// four-step split (two passes with a twiddle in between) for lengths that do not fit in shared
// memory. Replaces the float64 radix-2 Cooley-Tukey core and the per-axis transposing gathers of
// fft_cooley_tukey_parallel (endia/functional/fft_ops/fft_cooley_tukey.mojo:133-176, 241-297).
// The inverse direction is conj -> forward -> conj, as IFFTN and FFTN.vjp state it
// (ifftn_op.mojo:60-77, fftn_op.mojo:43-49), fused into the first load and the last store.
#include "common.cuh"
#include <map>
#include <mutex>
#include <vector>
#include <math.h>
#include <stdlib.h>

namespace eb {

constexpr int FFT_E = 16;            // complex elements held by one thread
constexpr int FFT_MAX_SMEM_N = 4096; // longest line transformed inside one CTA
constexpr int FFT_MAX_STAGES = 6;

struct FftParams {
  const float2 *in;
  float2 *out;
  int N;
  int T, logT;                   // lines per tile (power of two)
  int n_stages;
  int radix[FFT_MAX_STAGES];
  int64_t n_tiles, lines_per_outer, tiles_per_outer;
  int64_t in_outer_stride, in_line_stride, in_elem_stride;
  int64_t out_outer_stride, out_line_stride, out_elem_stride;
  const float2 *tw;              // W_N^q, q in [0, N)
  int conj_in, conj_out;
  float scale;
  // Four-step twiddle applied at the store: element j of line l is multiplied by
  // W_big^(j*l) = tw_hi[(j*l) >> lo_bits] * tw_lo[(j*l) & mask].
  const float2 *tw_hi, *tw_lo;
  int lo_bits;
  int in_real;                   // `in` points at floats (one per element): the imaginary part is 0
  // Work fused into the LAST pass of a transform (all zero otherwise):
  const float *scale_dev;        // a device scalar multiplied into `scale`
  int red_mode;                  // 1: sum |y|^2, 2: sum real(y) * red_w[index of y], over the stored values y
  const float *red_w;
  float *red_partial;            // one partial sum per CTA
};

// Sum over the CTA of `v` (blockDim.x a multiple of 32); valid in thread 0.
__device__ __forceinline__ float fft_block_sum(float v) {
  __shared__ float part[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) part[w] = v;
  __syncthreads();
  float r = 0.f;
  if (w == 0) {
    r = lane < (int)((blockDim.x + 31) >> 5) ? part[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  }
  return r;
}

// Element `idx` (in elements from `base`) of the input, which is complex or, with `real`, real.
__device__ __forceinline__ float2 load_in(const float2 *base, int64_t idx, int real) {
  if (real) return make_float2(reinterpret_cast<const float *>(base)[idx], 0.f);
  return base[idx];
}

__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
// multiply by -i
__device__ __forceinline__ float2 mul_mi(float2 a) { return make_float2(a.y, -a.x); }

template <int R>
__device__ __forceinline__ void dft(float2 *u);

template <>
__device__ __forceinline__ void dft<2>(float2 *u) {
  float2 a = u[0], b = u[1];
  u[0] = cadd(a, b);
  u[1] = csub(a, b);
}
template <>
__device__ __forceinline__ void dft<4>(float2 *u) {
  float2 a = cadd(u[0], u[2]), b = csub(u[0], u[2]);
  float2 c = cadd(u[1], u[3]), d = mul_mi(csub(u[1], u[3]));
  u[0] = cadd(a, c); u[1] = cadd(b, d); u[2] = csub(a, c); u[3] = csub(b, d);
}
template <>
__device__ __forceinline__ void dft<8>(float2 *u) {
  float2 e[4] = {u[0], u[2], u[4], u[6]};
  float2 o[4] = {u[1], u[3], u[5], u[7]};
  dft<4>(e);
  dft<4>(o);
  const float h = 0.70710678118654752440f;
  o[1] = make_float2(h * (o[1].x + o[1].y), h * (o[1].y - o[1].x));   // * (1 - i)/sqrt2
  o[2] = mul_mi(o[2]);
  o[3] = make_float2(h * (o[3].y - o[3].x), -h * (o[3].x + o[3].y));  // * (-1 - i)/sqrt2
#pragma unroll
  for (int k = 0; k < 4; ++k) { u[k] = cadd(e[k], o[k]); u[k + 4] = csub(e[k], o[k]); }
}
template <>
__device__ __forceinline__ void dft<16>(float2 *u) {
  // 4 x 4 decomposition: DFT-4 over m of u[j + 4m], twiddle W16^(j q), DFT-4 over j.
  float2 a[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int m = 0; m < 4; ++m) a[j][m] = u[j + 4 * m];
    dft<4>(a[j]);
  }
  const float c1 = 0.92387953251128675613f, s1 = 0.38268343236508977173f;  // cos, sin(pi/8)
  const float h = 0.70710678118654752440f;
  const float2 w[10] = {
      make_float2(1.f, 0.f),  make_float2(c1, -s1), make_float2(h, -h),  make_float2(s1, -c1),
      make_float2(0.f, -1.f), make_float2(-s1, -c1), make_float2(-h, -h), make_float2(-c1, -s1),
      make_float2(-1.f, 0.f), make_float2(-c1, s1)};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float2 b[4];
    b[0] = a[0][q];
#pragma unroll
    for (int j = 1; j < 4; ++j) b[j] = (q == 0) ? a[j][q] : cmul(a[j][q], w[j * q]);
    dft<4>(b);
#pragma unroll
    for (int s = 0; s < 4; ++s) u[q + 4 * s] = b[s];
  }
}

// One Stockham stage of radix R over every line of the tile. `p` is the product of the radices
// of the earlier stages. Every thread owns FFT_E/R butterflies; all reads of the stage happen
// before the barrier and all writes after it, so the stage runs in place.
template <int R>
__device__ __forceinline__ void stage(float2 *sm, const FftParams &P, int p, int tid) {
  constexpr int ITEMS = FFT_E / R;
  const int T = P.T, LS = T + 1;
  const int per_line = P.N / R;        // butterflies per line
  const int tw_step = P.N / (p * R);
  float2 u[ITEMS][R];
  int jout[ITEMS];
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
    const int w = tid + it * blockDim.x;  // t fastest
    const int t = w & (T - 1), i = w >> P.logT;
    const int k = i & (p - 1);
#pragma unroll
    for (int r = 0; r < R; ++r) u[it][r] = sm[(i + r * per_line) * LS + t];
    if (p > 1) {
#pragma unroll
      for (int r = 1; r < R; ++r) u[it][r] = cmul(u[it][r], __ldg(P.tw + r * k * tw_step));
    }
    dft<R>(u[it]);
    jout[it] = ((i - k) * R + k) * LS + t;
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) {
#pragma unroll
    for (int r = 0; r < R; ++r) sm[jout[it] + r * p * LS] = u[it][r];
  }
  __syncthreads();
}

__global__ void __launch_bounds__(1024, 1) fft_tile_kernel(const __grid_constant__ FftParams P) {
  extern __shared__ float2 sm[];
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int T = P.T, LS = T + 1, N = P.N;
  const int total = T * N;
  const float scale = P.scale_dev ? P.scale * __ldg(P.scale_dev) : P.scale;
  float red = 0.f;
  for (int64_t tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
    const int64_t o = tile / P.tiles_per_outer;
    const int64_t line0 = (tile - o * P.tiles_per_outer) * T;
    int64_t nl64 = P.lines_per_outer - line0;
    const int nl = nl64 < T ? (int)nl64 : T;
    // ---- load
    const int64_t src0 = o * P.in_outer_stride + line0 * P.in_line_stride;
    if (P.in_elem_stride == 1) {
      for (int w = tid; w < total; w += nthr) {
        const int t = w / N, j = w - t * N;
        float2 v = make_float2(0.f, 0.f);
        if (t < nl) v = load_in(P.in, src0 + (int64_t)t * P.in_line_stride + j, P.in_real);
        if (P.conj_in) v.y = -v.y;
        sm[j * LS + t] = v;
      }
    } else {
      for (int w = tid; w < total; w += nthr) {
        const int t = w & (T - 1), j = w >> P.logT;
        float2 v = make_float2(0.f, 0.f);
        if (t < nl) v = load_in(P.in, src0 + (int64_t)t * P.in_line_stride + (int64_t)j * P.in_elem_stride, P.in_real);
        if (P.conj_in) v.y = -v.y;
        sm[j * LS + t] = v;
      }
    }
    __syncthreads();
    // ---- stages
    int p = 1;
    for (int s = 0; s < P.n_stages; ++s) {
      const int R = P.radix[s];
      if (R == 16) stage<16>(sm, P, p, tid);
      else if (R == 8) stage<8>(sm, P, p, tid);
      else if (R == 4) stage<4>(sm, P, p, tid);
      else stage<2>(sm, P, p, tid);
      p *= R;
    }
    // ---- store
    float2 *dst = P.out + o * P.out_outer_stride + line0 * P.out_line_stride;
    const bool t_fast = P.out_elem_stride != 1;
    for (int w = tid; w < total; w += nthr) {
      int t, j;
      if (t_fast) { t = w & (T - 1); j = w >> P.logT; }
      else { t = w / N; j = w - t * N; }
      if (t >= nl) continue;
      float2 v = sm[j * LS + t];
      if (P.tw_hi) {
        const int64_t q = (int64_t)j * (line0 + t);
        v = cmul(v, cmul(__ldg(P.tw_hi + (q >> P.lo_bits)),
                         __ldg(P.tw_lo + (q & ((int64_t(1) << P.lo_bits) - 1)))));
      }
      v.x *= scale; v.y *= scale;
      if (P.conj_out) v.y = -v.y;
      const int64_t at = (int64_t)t * P.out_line_stride + (int64_t)j * P.out_elem_stride;
      dst[at] = v;
      if (P.red_mode == 1) red += v.x * v.x + v.y * v.y;
      else if (P.red_mode == 2) red += v.x * __ldg(P.red_w + (dst - P.out) + at);
    }
    __syncthreads();
  }
  if (P.red_mode) {
    red = fft_block_sum(red);
    if (tid == 0) P.red_partial[blockIdx.x] = red;
  }
}

// ------------------------------------------------------------------- fast path
// Lines of 256 / 512 / 1024 / 2048 points, 8 lines per tile, sizes known at compile time, plan
// 16 x 16 x (N/256). Thread (t, i) owns 16 points of line t. The first radix-16 stage reads its
// inputs straight from global memory and the last stage writes its outputs straight back, so only
// the two exchanges between stages go through shared memory. Two thread mappings:
//   COL (strided axis; the 8 lines are adjacent in memory): lanes run over the lines first, so a
//       warp touches 64-byte segments; shared layout [point][line] with an XOR swizzle that keeps
//       both line-major and point-major accesses free of bank conflicts;
//   ROW (contiguous axis): lanes run over the points of one line, so a warp touches 256 contiguous
//       bytes; shared layout [line][point] with the low 4 bits of the point index XORed by the
//       next 4 (the Stockham write patterns of this plan then never collide).
// COL with STAGE_IN reads contiguous lines through shared memory (coalesced) and writes strided:
// the transposing second pass of the four-step split.
// Twiddles W_N^q sit in shared memory for the lifetime of the (persistent) CTA.
struct FastParams {
  const float2 *in;
  float2 *out;
  int64_t n_tiles, tiles_per_outer;
  int64_t in_outer, in_line, in_elem;
  int64_t out_outer, out_line, out_elem;
  const float2 *tw, *tw_hi, *tw_lo;
  int lo_bits;
  int conj_in, conj_out;
  float scale;
  int in_real;                   // as in FftParams
  const float *scale_dev;        // as in FftParams (last pass only)
  const float *red_w;
  float *red_partial;
};

enum { FAST_COL = 0, FAST_ROW = 1, FAST_COL_STAGED_IN = 2 };
enum { RED_NONE = 0, RED_ABS2 = 1, RED_RE_W = 2 };

template <int LOGN, int MODE, int T>
__device__ __forceinline__ int fast_phys(int j, int t) {
  if constexpr (MODE == FAST_ROW) {
    return (t << LOGN) + (j ^ ((j >> 4) & 15));
  } else if constexpr (T == 16) {
    // one row = one 128-byte bank line; rotating the slot by the row index keeps point-major
    // accesses (same line, consecutive points) conflict-free too
    return (j << 4) + (t ^ (j & 15));
  } else {
    // rows 2m and 2m+1 share a 128-byte bank line: which half is flipped by bit 4 of the row,
    // and the slot inside the half is rotated by the line-pair index
    const int m = j >> 1;
    return (m << 4) + (((j ^ (j >> 4)) & 1) << 3) + (t ^ (m & 7));
  }
}

// Four-step twiddle W_big^q from the two small tables.
__device__ __forceinline__ float2 fast_bigtw(const FastParams &P, int q) {
  return cmul(__ldg(P.tw_hi + (q >> P.lo_bits)), __ldg(P.tw_lo + (q & ((1 << P.lo_bits) - 1))));
}
// Store of output point j of the line at `dst`; RED accumulates the loss term of the stored value
// (`wl` = the line of red_w that lies under `dst`).
template <int RED>
__device__ __forceinline__ void fast_store(const FastParams &P, float2 *dst, int j, float2 v, float sc,
                                           float &red, const float *wl) {
  v.x *= sc; v.y *= sc;
  if (P.conj_out) v.y = -v.y;
  dst[(int64_t)j * P.out_elem] = v;
  if constexpr (RED == RED_ABS2) red += v.x * v.x + v.y * v.y;
  if constexpr (RED == RED_RE_W) red += v.x * __ldg(wl + (int64_t)j * P.out_elem);
}

template <int LOGN, int MODE, bool TW, int T, bool REAL, int RED = RED_NONE>
__global__ void __launch_bounds__((T << LOGN) / 16, 16384 / (T << LOGN))
fft_fast_kernel(const __grid_constant__ FastParams P) {
  constexpr int N = 1 << LOGN, NT = T * N / 16, Q = N / 16, R3 = N / 256;
  constexpr int LOGT = T == 16 ? 4 : 3;
  extern __shared__ float2 sm[];
  float2 *tws = sm + N * T;
  const int tid = threadIdx.x;
  const int t = MODE == FAST_ROW ? tid / Q : (tid & (T - 1));
  const int i0 = MODE == FAST_ROW ? tid % Q : (tid >> LOGT);
  for (int q = tid; q < N; q += NT) tws[q] = __ldg(P.tw + q);
  __syncthreads();
  const float sc = P.scale_dev ? P.scale * __ldg(P.scale_dev) : P.scale;
  float red = 0.f;
  for (int64_t tile = blockIdx.x; tile < P.n_tiles; tile += gridDim.x) {
    const int64_t o = tile / P.tiles_per_outer;
    const int line0 = (int)(tile - o * P.tiles_per_outer) * T;
    const int line = line0 + t;
    float2 *dst = P.out + o * P.out_outer + (int64_t)line * P.out_line;
    const float *wl = RED == RED_RE_W ? P.red_w + (dst - P.out) : nullptr;
    float2 u[16];
    if constexpr (MODE == FAST_COL_STAGED_IN) {
      // contiguous lines: a warp reads 32 consecutive points of one line, the swizzle makes the
      // point-major shared store conflict-free as well
      const int64_t src0 = o * P.in_outer + (int64_t)line0 * P.in_line;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int w = tid + e * NT, j = w & (N - 1), tt = w >> LOGN;
        float2 v = load_in(P.in, src0 + (int64_t)tt * P.in_line + j, REAL ? 1 : 0);
        if (P.conj_in) v.y = -v.y;
        sm[fast_phys<LOGN, MODE, T>(j, tt)] = v;
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < 16; ++r) u[r] = sm[fast_phys<LOGN, MODE, T>(i0 + r * Q, t)];
      __syncthreads();
    } else {
      const int64_t src0 = o * P.in_outer + (int64_t)line * P.in_line;
      if constexpr (REAL) {
        const float *srcr = reinterpret_cast<const float *>(P.in) + src0;
#pragma unroll
        for (int r = 0; r < 16; ++r) u[r] = make_float2(srcr[(int64_t)(i0 + r * Q) * P.in_elem], 0.f);
      } else {
        const float2 *src = P.in + src0;
#pragma unroll
        for (int r = 0; r < 16; ++r) u[r] = src[(int64_t)(i0 + r * Q) * P.in_elem];
      }
      if (P.conj_in) {
#pragma unroll
        for (int r = 0; r < 16; ++r) u[r].y = -u[r].y;
      }
    }
    // stage 1: radix 16 on inputs i0 + r*N/16
    dft<16>(u);
#pragma unroll
    for (int r = 0; r < 16; ++r) sm[fast_phys<LOGN, MODE, T>(i0 * 16 + r, t)] = u[r];
    __syncthreads();
    // stage 2: radix 16, p = 16
#pragma unroll
    for (int r = 0; r < 16; ++r) u[r] = sm[fast_phys<LOGN, MODE, T>(i0 + r * Q, t)];
    const int k = i0 & 15;
#pragma unroll
    for (int r = 1; r < 16; ++r) u[r] = cmul(u[r], tws[r * k * R3]);
    dft<16>(u);
    if constexpr (R3 == 1) {
      // last stage: output point i0 + 16 r; its four-step twiddle is base * step^r
      if constexpr (TW) {
        float2 w = fast_bigtw(P, i0 * line);
        const float2 step = fast_bigtw(P, 16 * line);
#pragma unroll
        for (int r = 0; r < 16; ++r) { u[r] = cmul(u[r], w); w = cmul(w, step); }
      }
#pragma unroll
      for (int r = 0; r < 16; ++r) fast_store<RED>(P, dst, i0 + 16 * r, u[r], sc, red, wl);
    } else {
      __syncthreads();
#pragma unroll
      for (int r = 0; r < 16; ++r) sm[fast_phys<LOGN, MODE, T>((i0 - k) * 16 + k + 16 * r, t)] = u[r];
      __syncthreads();
      // stage 3: radix R3, p = 256; 16/R3 butterflies per thread, outputs straight to global
      float2 step = make_float2(1.f, 0.f);
      if constexpr (TW) step = fast_bigtw(P, 256 * line);
#pragma unroll
      for (int it = 0; it < 16 / R3; ++it) {
        const int i = i0 + it * Q;
        float2 v[R3];
#pragma unroll
        for (int r = 0; r < R3; ++r) v[r] = sm[fast_phys<LOGN, MODE, T>(i + r * 256, t)];
#pragma unroll
        for (int r = 1; r < R3; ++r) v[r] = cmul(v[r], tws[r * i]);
        dft<R3>(v);
        if constexpr (TW) {
          float2 w = fast_bigtw(P, i * line);
#pragma unroll
          for (int r = 0; r < R3; ++r) { v[r] = cmul(v[r], w); w = cmul(w, step); }
        }
#pragma unroll
        for (int r = 0; r < R3; ++r) fast_store<RED>(P, dst, i + r * 256, v[r], sc, red, wl);
      }
    }
    __syncthreads();
  }
  if constexpr (RED != RED_NONE) {
    red = fft_block_sum(red);
    if (tid == 0) P.red_partial[blockIdx.x] = red;
  }
}

// Standalone form of the fused loss term, for transforms whose last pass has no fused variant:
// one pass over the stored result.
__global__ void __launch_bounds__(256) fft_reduce_kernel(const float2 *y, const float *w, int64_t n, int mode,
                                                         float *partial) {
  float red = 0.f;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const float2 v = y[i];
    red += mode == RED_ABS2 ? v.x * v.x + v.y * v.y : v.x * __ldg(w + i);
  }
  red = fft_block_sum(red);
  if (threadIdx.x == 0) partial[blockIdx.x] = red;
}

// ------------------------------------------------------------------ host side
static std::mutex g_tw_mutex;
static std::map<std::pair<int, int64_t>, float2 *> g_tw_cache;  // (device, key) -> table

// Table of `count` entries: entry q = exp(-2*pi*i * q * mult / n), evaluated in float64.
static int twiddle_table(int64_t n, int64_t mult, int64_t count, int kind, const float2 **out) {
  int dev = 0;
  EB_CUDA(cudaGetDevice(&dev));
  const int64_t key = (n << 8) | (int64_t)kind;
  std::lock_guard<std::mutex> lock(g_tw_mutex);
  auto it = g_tw_cache.find({dev, key});
  if (it != g_tw_cache.end()) { *out = it->second; return ENDIA_B200_OK; }
  std::vector<float2> host((size_t)count);
  const long double two_pi = 6.283185307179586476925286766559L;
  for (int64_t q = 0; q < count; ++q) {
    // Reduce the angle to an exact fraction of the circle before the float64 evaluation.
    const int64_t num = (q * mult) % n;
    const long double ang = -two_pi * (long double)num / (long double)n;
    host[(size_t)q] = make_float2((float)cosl(ang), (float)sinl(ang));
  }
  float2 *dev_ptr = nullptr;
  cudaError_t e = cudaMalloc(&dev_ptr, sizeof(float2) * (size_t)count);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error("fft: twiddle table allocation failed");
    return ENDIA_B200_ENOMEM;
  }
  EB_CUDA(cudaMemcpy(dev_ptr, host.data(), sizeof(float2) * (size_t)count, cudaMemcpyHostToDevice));
  g_tw_cache[{dev, key}] = dev_ptr;
  *out = dev_ptr;
  return ENDIA_B200_OK;
}

static void plan_radices(int N, FftParams &P) {
  int L = ilog2(N);
  P.n_stages = 0;
  while (L > 0) {
    int l = L >= 4 ? 4 : L;
    if (L == 5) l = 3;  // 8 * 4 rather than 16 * 2
    P.radix[P.n_stages++] = 1 << l;
    L -= l;
  }
}

// Lines per tile for a line length N: at least 2048 elements per CTA (128 threads), 16 lines
// (128-byte segments on strided axes) where shared memory allows.
static int pick_T(int N) {
  int T = 16;
  while (T * N < 2048) T *= 2;
  while (T > 1 && (size_t)N * (T + 1) * sizeof(float2) > 200 * 1024) T /= 2;
  if (N == 1024) T = 8;  // 3 CTAs per SM instead of 1
  return T;
}

constexpr int FFT_RED_MAX_PARTIALS = 4096;   // CTAs of a last pass never exceed this

// What the last pass of a transform does besides the transform (see endia_b200_fft_fusion).
struct LastPass {
  const float *scale_dev = nullptr;
  int red_mode = RED_NONE;
  const float *red_w = nullptr;
  float *red_partial = nullptr;
  int n_partials = 0;            // out: CTAs that wrote a partial sum (0: the pass had no fused variant)
};

template <int LOGN, int MODE, bool TW, int T, bool REAL, int RED = RED_NONE>
static int launch_fast_variant(FastParams F, int64_t lines_per_outer, int64_t n_outer, cudaStream_t s,
                               LastPass *lp = nullptr) {
  constexpr int N = 1 << LOGN;
  constexpr size_t SMEM = sizeof(float2) * (size_t)N * (T + 1);   // T lines of data + the twiddle table
  F.tiles_per_outer = lines_per_outer / T;
  F.n_tiles = F.tiles_per_outer * n_outer;
  auto kern = fft_fast_kernel<LOGN, MODE, TW, T, REAL, RED>;
  static bool attr = false;
  if (!attr) {
    EB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    attr = true;
  }
  const int per_sm = 16384 / (T * N);   // 1024 threads (16 points each) per SM
  const int64_t cap = (int64_t)(sm_count() > 0 ? sm_count() : 148) * per_sm;
  const int grid = (int)(F.n_tiles < cap ? F.n_tiles : cap);
  if (lp) {
    F.scale_dev = lp->scale_dev;
    if constexpr (RED != RED_NONE) {
      F.red_w = lp->red_w; F.red_partial = lp->red_partial;
      lp->n_partials = grid;
    }
  }
  kern<<<grid, T * N / 16, SMEM, s>>>(F);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

// The variants that can end a transform exist with the fused loss terms as well (complex source,
// no four-step twiddle: that pass is never the last).
template <int LOGN, int MODE, int T>
static int launch_fast_last(const FastParams &F, int64_t lpo, int64_t no, cudaStream_t s, LastPass *lp) {
  const int red = lp ? lp->red_mode : RED_NONE;
  if (red == RED_ABS2) return launch_fast_variant<LOGN, MODE, false, T, false, RED_ABS2>(F, lpo, no, s, lp);
  if (red == RED_RE_W) return launch_fast_variant<LOGN, MODE, false, T, false, RED_RE_W>(F, lpo, no, s, lp);
  return launch_fast_variant<LOGN, MODE, false, T, false>(F, lpo, no, s, lp);
}

template <int LOGN, bool REAL>
static int launch_fast_nr(const FastParams &F, bool tw, int64_t lpo, int64_t no, cudaStream_t s, LastPass *lp) {
  const bool row_in = F.in_elem == 1, row_out = F.out_elem == 1;
  if (row_in && row_out) {
    if constexpr (!REAL) return launch_fast_last<LOGN, FAST_ROW, 8>(F, lpo, no, s, lp);
    return launch_fast_variant<LOGN, FAST_ROW, false, 8, REAL>(F, lpo, no, s, lp);
  }
  // 16 lines per tile give 128-byte segments on the strided side; they fit next to 2 CTAs per SM
  // for lines up to 512 points (and, with one 1024-thread CTA per SM, for 1024 points: measured
  // faster than two 512-thread CTAs of 8 lines, whose segments are 64 bytes).
  static const int wide_max = []() { const char *e = getenv("ENDIA_B200_FFT_WIDE_MAX"); return e ? atoi(e) : 1024; }();
  if constexpr (LOGN <= 10) {
    if ((1 << LOGN) <= wide_max && lpo % 16 == 0) {
      if (row_in) {
        if constexpr (!REAL) return launch_fast_last<LOGN, FAST_COL_STAGED_IN, 16>(F, lpo, no, s, lp);
        return launch_fast_variant<LOGN, FAST_COL_STAGED_IN, false, 16, REAL>(F, lpo, no, s, lp);
      }
      if (tw) return launch_fast_variant<LOGN, FAST_COL, true, 16, REAL>(F, lpo, no, s, lp);
      if constexpr (!REAL) return launch_fast_last<LOGN, FAST_COL, 16>(F, lpo, no, s, lp);
      return launch_fast_variant<LOGN, FAST_COL, false, 16, REAL>(F, lpo, no, s, lp);
    }
  }
  if (row_in) {
    if constexpr (!REAL) return launch_fast_last<LOGN, FAST_COL_STAGED_IN, 8>(F, lpo, no, s, lp);
    return launch_fast_variant<LOGN, FAST_COL_STAGED_IN, false, 8, REAL>(F, lpo, no, s, lp);
  }
  if (tw) return launch_fast_variant<LOGN, FAST_COL, true, 8, REAL>(F, lpo, no, s, lp);
  if constexpr (!REAL) return launch_fast_last<LOGN, FAST_COL, 8>(F, lpo, no, s, lp);
  return launch_fast_variant<LOGN, FAST_COL, false, 8, REAL>(F, lpo, no, s, lp);
}

template <int LOGN>
static int launch_fast_n(const FastParams &F, bool tw, int64_t lpo, int64_t no, cudaStream_t s, LastPass *lp) {
  // a real source (read with a zero imaginary part) has kernels of its own, so that the complex
  // ones keep their register budget
  return F.in_real ? launch_fast_nr<LOGN, true>(F, tw, lpo, no, s, lp) : launch_fast_nr<LOGN, false>(F, tw, lpo, no, s, lp);
}

// Supported combinations: strided in and out (optionally with the four-step twiddle), contiguous
// in and out, contiguous in with strided out.
static bool fast_supported(int64_t in_elem, int64_t out_elem, bool tw) {
  const bool row_in = in_elem == 1, row_out = out_elem == 1;
  if (row_in) return !tw;
  return !row_out;
}

static int launch_fast(const FastParams &F, int N, bool tw, int64_t lpo, int64_t no, cudaStream_t s, LastPass *lp) {
  switch (N) {
    case 256: return launch_fast_n<8>(F, tw, lpo, no, s, lp);
    case 512: return launch_fast_n<9>(F, tw, lpo, no, s, lp);
    case 1024: return launch_fast_n<10>(F, tw, lpo, no, s, lp);
    default: return launch_fast_n<11>(F, tw, lpo, no, s, lp);
  }
}

struct Pass {
  int N;
  int64_t n_outer, lines_per_outer;
  int64_t in_outer, in_line, in_elem, out_outer, out_line, out_elem;
  int conj_in, conj_out;
  float scale;
  int64_t big_n;  // > 0: four-step twiddle W_big^(j*line) at the store
};

// `lp` is given for the last pass of a transform only.
static int launch_pass(const Pass &ps, const float2 *in, float2 *out, cudaStream_t s, bool in_real = false,
                       LastPass *lp = nullptr) {
  FftParams P{};
  P.in = in; P.out = out; P.N = ps.N;
  P.in_real = in_real ? 1 : 0;
  P.T = pick_T(ps.N); P.logT = ilog2(P.T);
  plan_radices(ps.N, P);
  P.lines_per_outer = ps.lines_per_outer;
  P.tiles_per_outer = ceil_div(ps.lines_per_outer, P.T);
  P.n_tiles = P.tiles_per_outer * ps.n_outer;
  P.in_outer_stride = ps.in_outer; P.in_line_stride = ps.in_line; P.in_elem_stride = ps.in_elem;
  P.out_outer_stride = ps.out_outer; P.out_line_stride = ps.out_line; P.out_elem_stride = ps.out_elem;
  P.conj_in = ps.conj_in; P.conj_out = ps.conj_out; P.scale = ps.scale;
  if (P.n_tiles == 0) return ENDIA_B200_OK;
  int st = twiddle_table(ps.N, 1, ps.N, 0, &P.tw);
  if (st) return st;
  if (ps.N >= 256 && ps.N <= 2048 && ps.lines_per_outer % 8 == 0 && ps.big_n < ((int64_t)1 << 23) &&
      fast_supported(ps.in_elem, ps.out_elem, ps.big_n > 0)) {
    FastParams F{};
    F.in = in; F.out = out;
    F.in_real = in_real ? 1 : 0;
    F.tiles_per_outer = ps.lines_per_outer / 8;
    F.n_tiles = F.tiles_per_outer * ps.n_outer;
    F.in_outer = ps.in_outer; F.in_line = ps.in_line; F.in_elem = ps.in_elem;
    F.out_outer = ps.out_outer; F.out_line = ps.out_line; F.out_elem = ps.out_elem;
    F.tw = P.tw; F.conj_in = ps.conj_in; F.conj_out = ps.conj_out; F.scale = ps.scale;
    if (ps.big_n > 0) {
      const int lb = ilog2(ps.big_n);
      F.lo_bits = (lb + 1) / 2;
      if ((st = twiddle_table(ps.big_n, 1, int64_t(1) << F.lo_bits, 1, &F.tw_lo))) return st;
      if ((st = twiddle_table(ps.big_n, int64_t(1) << F.lo_bits, int64_t(1) << (lb - F.lo_bits), 2,
                              &F.tw_hi))) return st;
    }
    return launch_fast(F, ps.N, ps.big_n > 0, ps.lines_per_outer, ps.n_outer, s, lp);
  }
  if (ps.big_n > 0) {
    const int lb = ilog2(ps.big_n);
    P.lo_bits = (lb + 1) / 2;
    if ((st = twiddle_table(ps.big_n, 1, int64_t(1) << P.lo_bits, 1, &P.tw_lo))) return st;
    if ((st = twiddle_table(ps.big_n, int64_t(1) << P.lo_bits, int64_t(1) << (lb - P.lo_bits), 2,
                            &P.tw_hi))) return st;
  }
  int threads = P.T * ps.N / FFT_E;
  if (threads < 32) threads = 32;  // short tiles: surplus threads own no butterfly
  const size_t smem = sizeof(float2) * (size_t)ps.N * (P.T + 1);
  static bool attr_set = false;
  if (!attr_set) {
    // (the kernel also has 128 bytes of static shared memory for its block sum)
    EB_CUDA(cudaFuncSetAttribute(fft_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024 - 1024));
    attr_set = true;
  }
  int64_t cap = (int64_t)(sm_count() > 0 ? sm_count() : 148) * 4;
  int grid = (int)(P.n_tiles < cap ? P.n_tiles : cap);
  if (lp) {
    P.scale_dev = lp->scale_dev;
    if (lp->red_mode) {
      P.red_mode = lp->red_mode; P.red_w = lp->red_w; P.red_partial = lp->red_partial;
      lp->n_partials = grid;
    }
  }
  fft_tile_kernel<<<grid, threads, smem, s>>>(P);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

// Splits a long line length into N1 * N2 with both factors <= FFT_MAX_SMEM_N.
static bool split_len(int64_t N, int &N1, int &N2) {
  const int L = ilog2(N);
  int l1 = (L + 1) / 2;
  static const int forced = []() { const char *e = getenv("ENDIA_B200_FFT_SPLIT_L1"); return e ? atoi(e) : 0; }();
  if (forced > 0 && forced < L) l1 = forced;
  N1 = 1 << l1; N2 = 1 << (L - l1);
  return N1 <= FFT_MAX_SMEM_N && N2 <= FFT_MAX_SMEM_N;
}

struct AxisInfo { int64_t outer, n, inner; };

// Signals per four-step group. Grouping so that the intermediate stays in L2 measured slower than
// two full-size passes (the passes are not HBM-bound and small launches fill the machine
// badly), so by default a group is the whole batch; ENDIA_B200_FFT_GROUP_MIB overrides.
static int64_t four_step_group(int64_t n, int64_t outer) {
  static const int64_t mib = []() { const char *e = getenv("ENDIA_B200_FFT_GROUP_MIB"); return (int64_t)(e ? atoi(e) : 1 << 20); }();
  int64_t g = (mib << 20) / (n * (int64_t)sizeof(float2));
  if (g < 1) g = 1;
  return g < outer ? g : outer;
}

static int collect_axes(const endia_b200_tensor *in, const int32_t *dims, int32_t n_dims,
                        std::vector<AxisInfo> &axes, bool &need_scratch) {
  need_scratch = false;
  uint32_t seen = 0;
  for (int a = 0; a < n_dims; ++a) {
    int d = dims[a] < 0 ? dims[a] + in->ndim : dims[a];
    EB_REQUIRE(d >= 0 && d < in->ndim, ENDIA_B200_EINVAL, "fft: dim %d out of range for rank %d",
               dims[a], in->ndim);
    EB_REQUIRE(!((seen >> d) & 1u), ENDIA_B200_EINVAL, "fft: dim %d listed twice", dims[a]);
    seen |= 1u << d;
    const int64_t n = in->shape[d];
    // fft_cooley_tukey.mojo:227-235 raises for lengths that are not powers of two.
    EB_REQUIRE(is_pow2(n), ENDIA_B200_EPOW2, "fft: length %lld of dim %d is not a power of two",
               (long long)n, d);
    AxisInfo ai{1, n, 1};
    for (int e = 0; e < d; ++e) ai.outer *= in->shape[e];
    for (int e = d + 1; e < in->ndim; ++e) ai.inner *= in->shape[e];
    if (n > FFT_MAX_SMEM_N) {
      int n1, n2;
      EB_REQUIRE(split_len(n, n1, n2), ENDIA_B200_ELIMIT, "fft: length %lld exceeds the limit %lld",
                 (long long)n, (long long)FFT_MAX_SMEM_N * FFT_MAX_SMEM_N);
      EB_REQUIRE(ai.inner == 1, ENDIA_B200_ELIMIT,
                 "fft: lengths above %d are supported on the innermost axis only", FFT_MAX_SMEM_N);
      need_scratch = true;
    }
    if (n > 1) axes.push_back(ai);
  }
  return ENDIA_B200_OK;
}

}  // namespace eb

using namespace eb;

extern "C" {

size_t endia_b200_fft_scratch_bytes(const endia_b200_tensor *in, const int32_t *dims,
                                    int32_t n_dims) {
  if (!in || (n_dims > 0 && !dims)) return 0;
  std::vector<AxisInfo> axes;
  bool need = false;
  if (collect_axes(in, dims, n_dims, axes, need)) return 0;
  if (!need) return 0;
  size_t bytes = 0;
  for (const AxisInfo &ai : axes)
    if (ai.n > FFT_MAX_SMEM_N) {
      const size_t b = sizeof(float2) * (size_t)ai.n * (size_t)four_step_group(ai.n, ai.outer);
      if (b > bytes) bytes = b;
    }
  return bytes;
}

size_t endia_b200_fft_fusion_scratch_bytes(void) { return sizeof(float) * FFT_RED_MAX_PARTIALS; }

int endia_b200_fft_loss_term(const endia_b200_tensor *y, int reduce, const float *reduce_w, float *reduce_out,
                             float reduce_scale, void *reduce_scratch, void *stream) {
  int st = require_device();
  if (st) return st;
  if ((st = check_tensor(y, "fft_loss_term: y"))) return st;
  EB_REQUIRE(y->is_complex && is_contiguous(y), ENDIA_B200_EINVAL, "fft_loss_term: y must be contiguous complex");
  EB_REQUIRE(reduce == RED_ABS2 || reduce == RED_RE_W, ENDIA_B200_EINVAL, "fft_loss_term: unknown reduction %d", reduce);
  EB_REQUIRE(reduce_out && reduce_scratch && (reduce != RED_RE_W || reduce_w), ENDIA_B200_EINVAL,
             "fft_loss_term: NULL pointer");
  cudaStream_t s = as_stream(stream);
  const int64_t total = numel(y);
  if (total == 0) {
    EB_CUDA(cudaMemsetAsync(reduce_out, 0, sizeof(float), s));
    return ENDIA_B200_OK;
  }
  const int ctas = grid_for(total, 256, 8);
  fft_reduce_kernel<<<ctas, 256, 0, s>>>(reinterpret_cast<const float2 *>(y->data) + y->offset, reduce_w, total, reduce,
                                         static_cast<float *>(reduce_scratch));
  EB_LAUNCH_CHECK();
  return launch_scalar_finish(static_cast<float *>(reduce_scratch), reduce_out, ctas, reduce_scale, s);
}

int endia_b200_fft_c2c(const endia_b200_tensor *in, const endia_b200_tensor *out,
                       const int32_t *dims, int32_t n_dims, int inverse, float scale, void *scratch,
                       void *stream) {
  return endia_b200_fft_c2c_fused(in, out, dims, n_dims, inverse, scale, scratch, nullptr, stream);
}

int endia_b200_fft_c2c_fused(const endia_b200_tensor *in, const endia_b200_tensor *out,
                             const int32_t *dims, int32_t n_dims, int inverse, float scale, void *scratch,
                             const endia_b200_fft_fusion *fusion, void *stream) {
  int st = require_device();
  if (st) return st;
  LastPass lp;
  const bool fused = fusion != nullptr;
  if (fused) {
    EB_REQUIRE(fusion->reduce >= 0 && fusion->reduce <= 2, ENDIA_B200_EINVAL, "fft: unknown reduction %d", fusion->reduce);
    EB_REQUIRE(!fusion->reduce || (fusion->reduce_out && fusion->reduce_scratch), ENDIA_B200_EINVAL,
               "fft: the fused reduction needs reduce_out and reduce_scratch");
    EB_REQUIRE(fusion->reduce != 2 || fusion->reduce_w, ENDIA_B200_EINVAL, "fft: reduce = 2 needs reduce_w");
    lp.scale_dev = fusion->scale_dev;
    lp.red_mode = fusion->reduce;
    lp.red_w = fusion->reduce_w;
    lp.red_partial = static_cast<float *>(fusion->reduce_scratch);
  }
  if ((st = check_tensor(in, "fft: in"))) return st;
  if ((st = check_tensor(out, "fft: out"))) return st;
  // A real `in` (contiguous) is read as complex with a zero imaginary part by the first pass.
  EB_REQUIRE(out->is_complex, ENDIA_B200_EINVAL, "fft: out must be complex");
  bool real_in = !in->is_complex;
  EB_REQUIRE(!real_in || is_contiguous(in), ENDIA_B200_EINVAL, "fft: a real input must be contiguous");
  EB_REQUIRE(n_dims >= 0 && n_dims <= ENDIA_B200_MAX_DIMS && (n_dims == 0 || dims), ENDIA_B200_EINVAL,
             "fft: bad dims list");
  EB_REQUIRE(in->ndim == out->ndim, ENDIA_B200_ESHAPE, "fft: rank mismatch");
  for (int d = 0; d < in->ndim; ++d)
    EB_REQUIRE(in->shape[d] == out->shape[d], ENDIA_B200_ESHAPE, "fft: shape mismatch in dim %d", d);
  EB_REQUIRE(is_contiguous(out), ENDIA_B200_EINVAL, "fft: out must be contiguous");
  std::vector<AxisInfo> axes;
  bool need_scratch = false;
  if ((st = collect_axes(in, dims, n_dims, axes, need_scratch))) return st;
  EB_REQUIRE(!need_scratch || scratch, ENDIA_B200_EINVAL,
             "fft: scratch of endia_b200_fft_scratch_bytes() bytes is required");
  const int64_t total = numel(in);
  cudaStream_t s = as_stream(stream);
  if (total == 0) {
    if (fused && fusion->reduce) EB_CUDA(cudaMemsetAsync(fusion->reduce_out, 0, sizeof(float), s));
    return ENDIA_B200_OK;
  }
  // After the last pass: add up the per-CTA partial sums, or, where that pass had no fused variant
  // (or ran as several launches), take the loss term in one more pass over the result.
  int last_launches = 0;
  auto finish_reduction = [&]() -> int {
    if (!fused || !fusion->reduce) return ENDIA_B200_OK;
    float2 *y = reinterpret_cast<float2 *>(out->data) + out->offset;
    if (lp.n_partials == 0 || last_launches != 1) {
      lp.n_partials = grid_for(total, 256, 8);
      fft_reduce_kernel<<<lp.n_partials, 256, 0, s>>>(y, lp.red_w, total, lp.red_mode, lp.red_partial);
      EB_LAUNCH_CHECK();
    }
    return launch_scalar_finish(lp.red_partial, fusion->reduce_out, lp.n_partials, fusion->reduce_scale, s);
  };
  const float2 *src = real_in ? reinterpret_cast<const float2 *>(static_cast<const float *>(in->data) + in->offset)
                              : reinterpret_cast<const float2 *>(in->data) + in->offset;
  float2 *dst = reinterpret_cast<float2 *>(out->data) + out->offset;
  if (!is_contiguous(in)) {
    // Gather the strided view once; the transform then runs in place on `out`.
    if ((st = endia_b200_ew_unary(ENDIA_B200_UN_COPY, in, out, stream))) return st;
    src = dst;
  }
  if (axes.empty()) {
    // Nothing to transform: out = scale * in (the inverse of a length-1 transform is itself).
    Pass ps{1, 1, total, 0, 1, 1, 0, 1, 1, 0, 0, scale, 0};
    ++last_launches;
    if ((st = launch_pass(ps, src, dst, s, real_in, fused ? &lp : nullptr))) return st;
    return finish_reduction();
  }
  // Innermost axis first: its pass reads `in` in long contiguous runs.
  for (size_t a = axes.size(); a-- > 0;) {
    const AxisInfo &ai = axes[a];
    const bool first = (a + 1 == axes.size()), last = (a == 0);
    const int cin = (inverse && first) ? 1 : 0, cout = (inverse && last) ? 1 : 0;
    const float sc = last ? scale : 1.f;
    if (ai.n <= FFT_MAX_SMEM_N) {
      Pass ps{};
      ps.N = (int)ai.n; ps.conj_in = cin; ps.conj_out = cout; ps.scale = sc; ps.big_n = 0;
      if (ai.inner == 1) {
        ps.n_outer = 1; ps.lines_per_outer = ai.outer;
        ps.in_outer = ps.out_outer = 0; ps.in_line = ps.out_line = ai.n; ps.in_elem = ps.out_elem = 1;
      } else {
        ps.n_outer = ai.outer; ps.lines_per_outer = ai.inner;
        ps.in_outer = ps.out_outer = ai.n * ai.inner; ps.in_line = ps.out_line = 1;
        ps.in_elem = ps.out_elem = ai.inner;
      }
      if (last) ++last_launches;
      if ((st = launch_pass(ps, src, dst, s, real_in, (fused && last) ? &lp : nullptr))) return st;
    } else {
      int n1, n2;
      split_len(ai.n, n1, n2);
      float2 *tmp = reinterpret_cast<float2 *>(scratch);
      // The two passes run group by group over the signals, through one group-sized scratch
      // buffer that is rewritten for every group: the intermediate then lives in L2 and HBM sees
      // one read of the input and one write of the output.
      const int64_t group = four_step_group(ai.n, ai.outer);
      for (int64_t g0 = 0; g0 < ai.outer; g0 += group) {
        const int64_t ng = ai.outer - g0 < group ? ai.outer - g0 : group;
        // Pass A: for every n2, transform over n1 (stride n2), then multiply by W_n^(k1*n2).
        Pass pa{};
        pa.N = n1; pa.n_outer = ng; pa.lines_per_outer = n2;
        pa.in_outer = pa.out_outer = ai.n; pa.in_line = pa.out_line = 1; pa.in_elem = pa.out_elem = n2;
        pa.conj_in = cin; pa.conj_out = 0; pa.scale = 1.f; pa.big_n = ai.n;
        // (a real source is indexed in floats: the group offset is applied in those units)
        const float2 *src_g = real_in ? reinterpret_cast<const float2 *>(reinterpret_cast<const float *>(src) + g0 * ai.n)
                                      : src + g0 * ai.n;
        if ((st = launch_pass(pa, src_g, tmp, s, real_in))) return st;
        // Pass B: for every k1, transform the contiguous row over n2; X[k1 + n1*k2] = row[k2].
        Pass pb{};
        pb.N = n2; pb.n_outer = ng; pb.lines_per_outer = n1;
        pb.in_outer = pb.out_outer = ai.n; pb.in_line = n2; pb.in_elem = 1;
        pb.out_line = 1; pb.out_elem = n1;
        pb.conj_in = 0; pb.conj_out = cout; pb.scale = sc; pb.big_n = 0;
        if (last) ++last_launches;
        if ((st = launch_pass(pb, tmp, dst + g0 * ai.n, s, false, (fused && last) ? &lp : nullptr))) return st;
      }
    }
    src = dst;
    real_in = false;
  }
  return finish_reduction();
}

}  // extern "C"
