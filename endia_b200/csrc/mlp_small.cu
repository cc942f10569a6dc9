// Whole training step of a small MLP in ONE launch of ONE CTA: forward, MSE loss, backward and
// the Adam update, with every activation held in shared memory. For networks as small as the
// reference's own benchmark (widths <= 64, batch of a few hundred: endia/nn/modules/_mlp.mojo:47-53,
// benchmarks/mlp_benchmarks/mlp_imp.mojo:47-75) the step is bound by launch latency, not by
// arithmetic, so the ~60 separate op launches of the eager path are replaced by one.
// Arithmetic follows the op chain of the reference: pred = act(a @ W + b) per layer
// (_mlp.mojo:50-52), loss = sum((p-t)^2)/size (loss_ops/mse_op.mojo:18-20), the VJPs of
// matmul/add/relu/tanh/sigmoid (matmul_op.mojo:278-284, expand_op.mojo:121-126, relu_op.mojo:95,
// tanh_op.mojo:92, sigmoid_op.mojo:98) and Adam (optim/adam.mojo:47-65). Sums run in a fixed order.
#include "common.cuh"

namespace eb {

constexpr int SM_MAX_LAYERS = 8;
constexpr int SM_THREADS = 512;

struct SmallMlpArgs {
  int n_layers, batch, act;
  int dims[SM_MAX_LAYERS + 1];
  const float *x, *y;
  float *W[SM_MAX_LAYERS], *b[SM_MAX_LAYERS];
  float *gW[SM_MAX_LAYERS], *gb[SM_MAX_LAYERS];
  float *mW[SM_MAX_LAYERS], *vW[SM_MAX_LAYERS], *mb[SM_MAX_LAYERS], *vb[SM_MAX_LAYERS];
  float *loss;
  int do_adam;
  float lr, b1, b2, eps, omb1, omb2, c1, c2;
  int act_off[SM_MAX_LAYERS + 2];  // float offsets of the activations in shared memory
  int d_off[2], w_off;             // two gradient buffers and the weight staging buffer
  int red_off;                     // slice sums of the weight gradients: max over layers of slices * K * N floats
  int slices[SM_MAX_LAYERS];       // batch slices of each layer's weight-gradient sum (1: no slice sums)
  // resident != 0: every layer's weights and biases have a place of their own in shared memory and
  // are read from global memory once, at the start (one memory latency instead of one per layer
  // and pass); otherwise each layer's weights go through the staging buffer when they are needed
  int resident;
  int w_offs[SM_MAX_LAYERS], b_offs[SM_MAX_LAYERS];
};

__device__ __forceinline__ float small_act(int act, float v) {
  if (act == ENDIA_B200_ACT_RELU) return fmaxf(v, 0.f);
  if (act == ENDIA_B200_ACT_TANH) return tanhf(v);
  if (act == ENDIA_B200_ACT_SIGMOID) return 1.f / (1.f + expf(-v));
  return v;
}
__device__ __forceinline__ float small_dact(int act, float a) {
  if (act == ENDIA_B200_ACT_RELU) return a > 0.f ? 1.f : 0.f;
  if (act == ENDIA_B200_ACT_TANH) return 1.f - a * a;
  if (act == ENDIA_B200_ACT_SIGMOID) return a * (1.f - a);
  return 1.f;
}
__device__ __forceinline__ void small_adam(const SmallMlpArgs &a, float &p, float g, float &m, float &v) {
  m = a.b1 * m + a.omb1 * g;
  v = a.b2 * v + (a.omb2 * g) * g;
  p = p - (a.lr * (m / a.c1)) / (sqrtf(v / a.c2) + a.eps);
}

__global__ void __launch_bounds__(SM_THREADS, 1) mlp_small_step_kernel(const __grid_constant__ SmallMlpArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[SM_THREADS / 32];
  const int tid = threadIdx.x, B = a.batch, L = a.n_layers;
  float *Ws = sm + a.w_off;
  // ---- forward
  for (int i = tid; i < B * a.dims[0]; i += SM_THREADS) sm[a.act_off[0] + i] = a.x[i];
  if (a.resident) {
    for (int l = 0; l < L; ++l) {
      const int KN = a.dims[l] * a.dims[l + 1], N = a.dims[l + 1];
      for (int i = tid; i < KN; i += SM_THREADS) sm[a.w_offs[l] + i] = a.W[l][i];
      for (int i = tid; i < N; i += SM_THREADS) sm[a.b_offs[l] + i] = a.b[l][i];
    }
  }
  for (int l = 0; l < L; ++l) {
    const int K = a.dims[l], N = a.dims[l + 1];
    const float *bias = a.resident ? sm + a.b_offs[l] : a.b[l];
    if (a.resident) Ws = sm + a.w_offs[l];
    else
      for (int i = tid; i < K * N; i += SM_THREADS) Ws[i] = a.W[l][i];
    __syncthreads();
    const float *in = sm + a.act_off[l];
    float *out = sm + a.act_off[l + 1];
    const int act = l < L - 1 ? a.act : ENDIA_B200_ACT_NONE;
    if ((N & 3) == 0) {
      // four adjacent outputs of two batch rows per thread: two broadcast reads of the input and
      // one 128-bit read of the weights feed eight FMAs (the second row is masked at an odd batch)
      const int N4 = N >> 2, B2 = (B + 1) >> 1;
      for (int i = tid; i < B2 * N4; i += SM_THREADS) {
        const int bp = i / N4, n = (i - bp * N4) * 4;
        const int r0 = 2 * bp, r1 = r0 + 1 < B ? r0 + 1 : r0;
        float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
        int k = 0;
        if ((K & 3) == 0) {
          // (128-bit reads of the inputs as well: six shared-memory loads per 32 FMAs)
#pragma unroll 2
          for (; k < K; k += 4) {
            const float4 xa = *reinterpret_cast<const float4 *>(in + r0 * K + k);
            const float4 xb = *reinterpret_cast<const float4 *>(in + r1 * K + k);
            const float xs0[4] = {xa.x, xa.y, xa.z, xa.w}, xs1[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float4 w = *reinterpret_cast<const float4 *>(Ws + (k + u) * N + n);
              s0.x = fmaf(xs0[u], w.x, s0.x); s0.y = fmaf(xs0[u], w.y, s0.y);
              s0.z = fmaf(xs0[u], w.z, s0.z); s0.w = fmaf(xs0[u], w.w, s0.w);
              s1.x = fmaf(xs1[u], w.x, s1.x); s1.y = fmaf(xs1[u], w.y, s1.y);
              s1.z = fmaf(xs1[u], w.z, s1.z); s1.w = fmaf(xs1[u], w.w, s1.w);
            }
          }
        }
#pragma unroll 8
        for (; k < K; ++k) {
          const float x0 = in[r0 * K + k], x1 = in[r1 * K + k];
          const float4 w = *reinterpret_cast<const float4 *>(Ws + k * N + n);
          s0.x = fmaf(x0, w.x, s0.x); s0.y = fmaf(x0, w.y, s0.y); s0.z = fmaf(x0, w.z, s0.z); s0.w = fmaf(x0, w.w, s0.w);
          s1.x = fmaf(x1, w.x, s1.x); s1.y = fmaf(x1, w.y, s1.y); s1.z = fmaf(x1, w.z, s1.z); s1.w = fmaf(x1, w.w, s1.w);
        }
        const float4 bb = *reinterpret_cast<const float4 *>(bias + n);
        float4 o;
        o.x = small_act(act, s0.x + bb.x); o.y = small_act(act, s0.y + bb.y);
        o.z = small_act(act, s0.z + bb.z); o.w = small_act(act, s0.w + bb.w);
        *reinterpret_cast<float4 *>(out + r0 * N + n) = o;
        if (r1 != r0) {
          o.x = small_act(act, s1.x + bb.x); o.y = small_act(act, s1.y + bb.y);
          o.z = small_act(act, s1.z + bb.z); o.w = small_act(act, s1.w + bb.w);
          *reinterpret_cast<float4 *>(out + r1 * N + n) = o;
        }
      }
    } else {
      for (int i = tid; i < B * N; i += SM_THREADS) {
        const int bi = i / N, n = i - bi * N;
        float s = 0.f;
        for (int k = 0; k < K; ++k) s = fmaf(in[bi * K + k], Ws[k * N + n], s);
        out[i] = small_act(act, s + bias[n]);
      }
    }
    __syncthreads();
  }
  // ---- loss and its gradient w.r.t. the prediction
  const int NL = a.dims[L], total = B * NL;
  const float inv = 1.f / (float)total;
  float *dcur = sm + a.d_off[0], *dnext = sm + a.d_off[1];
  float part = 0.f;
  for (int i = tid; i < total; i += SM_THREADS) {
    const float d = sm[a.act_off[L] + i] - a.y[i];
    part += d * d;
    dcur[i] = d * (inv + inv);
  }
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((tid & 31) == 0) red[tid >> 5] = part;
  __syncthreads();
  if (tid == 0) {
    float s = 0.f;
    for (int w = 0; w < SM_THREADS / 32; ++w) s += red[w];
    a.loss[0] = s * inv;
  }
  // ---- backward, last layer first
  for (int l = L - 1; l >= 0; --l) {
    const int K = a.dims[l], N = a.dims[l + 1];
    const float *in = sm + a.act_off[l], *outp = sm + a.act_off[l + 1];
    const int act = l < L - 1 ? a.act : ENDIA_B200_ACT_NONE;
    if (a.resident) Ws = sm + a.w_offs[l];      // (the forward pass's copy: untouched by Adam)
    else
      for (int i = tid; i < K * N; i += SM_THREADS) Ws[i] = a.W[l][i];
    if (act != ENDIA_B200_ACT_NONE)
      for (int i = tid; i < B * N; i += SM_THREADS) dcur[i] *= small_dact(act, outp[i]);
    __syncthreads();
    // gradient w.r.t. the layer input, with the weights as they were in the forward pass
    if (l > 0) {
      if ((N & 3) == 0) {
        // two adjacent inputs k of one batch row per thread: one 128-bit read of the gradient and
        // two of the weights feed eight FMAs (the second is masked at an odd K)
        const int K2 = (K + 1) >> 1;
        for (int i = tid; i < B * K2; i += SM_THREADS) {
          const int bi = i / K2, k0 = (i - bi * K2) * 2, k1 = k0 + 1 < K ? k0 + 1 : k0;
          float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
          for (int n = 0; n < N; n += 4) {
            const float4 d = *reinterpret_cast<const float4 *>(dcur + bi * N + n);
            const float4 w0 = *reinterpret_cast<const float4 *>(Ws + k0 * N + n);
            const float4 w1 = *reinterpret_cast<const float4 *>(Ws + k1 * N + n);
            s0 = fmaf(d.x, w0.x, s0); s0 = fmaf(d.y, w0.y, s0); s0 = fmaf(d.z, w0.z, s0); s0 = fmaf(d.w, w0.w, s0);
            s1 = fmaf(d.x, w1.x, s1); s1 = fmaf(d.y, w1.y, s1); s1 = fmaf(d.z, w1.z, s1); s1 = fmaf(d.w, w1.w, s1);
          }
          dnext[bi * K + k0] = s0;
          if (k1 != k0) dnext[bi * K + k1] = s1;
        }
      } else {
        for (int i = tid; i < B * K; i += SM_THREADS) {
          const int bi = i / K, k = i - bi * K;
          float s = 0.f;
          for (int n = 0; n < N; ++n) s = fmaf(dcur[bi * N + n], Ws[k * N + n], s);
          dnext[i] = s;
        }
      }
    }
    // weight gradient, then Adam. The batch rows are cut into S slices so that every thread has a
    // share: a thread sums one slice for one group of outputs (4 inputs x 4 columns as an outer
    // product of two 128-bit reads, or four columns, or one); with S > 1 the slice sums go through
    // shared memory and are added in slice order.
    {
      const bool vec = (N & 3) == 0, quad = vec && (K & 3) == 0;
      const int groups = quad ? (K >> 2) * (N >> 2) : (vec ? K * (N >> 2) : K * N);
      const int S = a.slices[l];
      const int rows = (B + S - 1) / S;
      float *part = sm + a.red_off;                 // [S][K * N]
      for (int i = tid; i < groups * S; i += SM_THREADS) {
        const int sl = i / groups, g = i - sl * groups;
        const int b0 = sl * rows, b1 = b0 + rows < B ? b0 + rows : B;
        if (quad) {
          const int N4 = N >> 2;
          const int k = (g / N4) * 4, n = (g - (g / N4) * N4) * 4;
          float4 acc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
          for (int bi = b0; bi < b1; ++bi) {
            const float4 x = *reinterpret_cast<const float4 *>(in + bi * K + k);
            const float4 d = *reinterpret_cast<const float4 *>(dcur + bi * N + n);
            const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              acc[u].x = fmaf(xs[u], d.x, acc[u].x); acc[u].y = fmaf(xs[u], d.y, acc[u].y);
              acc[u].z = fmaf(xs[u], d.z, acc[u].z); acc[u].w = fmaf(xs[u], d.w, acc[u].w);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (S > 1) {
              *reinterpret_cast<float4 *>(part + sl * K * N + (k + u) * N + n) = acc[u];
            } else {
              const float gv[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int idx = (k + u) * N + n + j;
                a.gW[l][idx] = gv[j];
                if (a.do_adam) small_adam(a, a.W[l][idx], gv[j], a.mW[l][idx], a.vW[l][idx]);
              }
            }
          }
        } else if (vec) {
          const int N4 = N >> 2;
          const int k = g / N4, n = (g - k * N4) * 4;
          float4 p[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) p[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          int bi = b0;
          for (; bi + 4 <= b1; bi += 4) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float x = in[(bi + u) * K + k];
              const float4 d = *reinterpret_cast<const float4 *>(dcur + (bi + u) * N + n);
              p[u].x = fmaf(x, d.x, p[u].x); p[u].y = fmaf(x, d.y, p[u].y);
              p[u].z = fmaf(x, d.z, p[u].z); p[u].w = fmaf(x, d.w, p[u].w);
            }
          }
          for (; bi < b1; ++bi) {
            const float x = in[bi * K + k];
            const float4 d = *reinterpret_cast<const float4 *>(dcur + bi * N + n);
            p[0].x = fmaf(x, d.x, p[0].x); p[0].y = fmaf(x, d.y, p[0].y);
            p[0].z = fmaf(x, d.z, p[0].z); p[0].w = fmaf(x, d.w, p[0].w);
          }
          const float4 gsum = make_float4((p[0].x + p[1].x) + (p[2].x + p[3].x), (p[0].y + p[1].y) + (p[2].y + p[3].y),
                                          (p[0].z + p[1].z) + (p[2].z + p[3].z), (p[0].w + p[1].w) + (p[2].w + p[3].w));
          if (S > 1) {
            *reinterpret_cast<float4 *>(part + sl * K * N + k * N + n) = gsum;
          } else {
            const float gv[4] = {gsum.x, gsum.y, gsum.z, gsum.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int idx = k * N + n + j;
              a.gW[l][idx] = gv[j];
              if (a.do_adam) small_adam(a, a.W[l][idx], gv[j], a.mW[l][idx], a.vW[l][idx]);
            }
          }
        } else {
          const int k = g / N, n = g - k * N;
          float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
          int bi = b0;
          for (; bi + 4 <= b1; bi += 4) {
            p0 = fmaf(in[(bi + 0) * K + k], dcur[(bi + 0) * N + n], p0);
            p1 = fmaf(in[(bi + 1) * K + k], dcur[(bi + 1) * N + n], p1);
            p2 = fmaf(in[(bi + 2) * K + k], dcur[(bi + 2) * N + n], p2);
            p3 = fmaf(in[(bi + 3) * K + k], dcur[(bi + 3) * N + n], p3);
          }
          for (; bi < b1; ++bi) p0 = fmaf(in[bi * K + k], dcur[bi * N + n], p0);
          const float gv = (p0 + p1) + (p2 + p3);
          if (S > 1) {
            part[sl * K * N + g] = gv;
          } else {
            a.gW[l][g] = gv;
            if (a.do_adam) small_adam(a, a.W[l][g], gv, a.mW[l][g], a.vW[l][g]);
          }
        }
      }
      if (S > 1) {
        __syncthreads();
        for (int o = tid; o < K * N; o += SM_THREADS) {
          float v = 0.f;
          for (int sl = 0; sl < S; ++sl) v += part[sl * K * N + o];
          a.gW[l][o] = v;
          if (a.do_adam) small_adam(a, a.W[l][o], v, a.mW[l][o], a.vW[l][o]);
        }
      }
    }
    // bias gradient: 16 lanes per column (rows bi = j (mod 16)), added by a fixed shuffle tree
    for (int base = 0; base < N; base += SM_THREADS / 16) {
      const int n = base + (tid >> 4), j = tid & 15;
      float s = 0.f;
      if (n < N)
        for (int bi = j; bi < B; bi += 16) s += dcur[bi * N + n];
      for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (n < N && j == 0) {
        a.gb[l][n] = s;
        if (a.do_adam) small_adam(a, a.b[l][n], s, a.mb[l][n], a.vb[l][n]);
      }
    }
    __syncthreads();
    float *t = dcur; dcur = dnext; dnext = t;
  }
}

}  // namespace eb

using namespace eb;

extern "C" int endia_b200_mlp_small_step(int32_t n_layers, const int32_t *dims, int32_t batch, int32_t act,
                                         const float *x, const float *y, float *const *W, float *const *b,
                                         float *const *gW, float *const *gb, float *const *mW,
                                         float *const *vW, float *const *mb, float *const *vb, float *loss,
                                         int32_t do_adam, float lr, float beta1, float beta2, float eps,
                                         float t, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n_layers >= 1 && n_layers <= SM_MAX_LAYERS, ENDIA_B200_ELIMIT,
             "mlp_small_step: 1..%d layers are supported, got %d", SM_MAX_LAYERS, n_layers);
  EB_REQUIRE(dims && x && y && W && b && gW && gb && loss, ENDIA_B200_EINVAL, "mlp_small_step: NULL argument");
  EB_REQUIRE(!do_adam || (mW && vW && mb && vb), ENDIA_B200_EINVAL, "mlp_small_step: Adam state is NULL");
  EB_REQUIRE(batch >= 1 && act >= 0 && act <= ENDIA_B200_ACT_SIGMOID, ENDIA_B200_EINVAL,
             "mlp_small_step: bad batch or activation");
  EB_REQUIRE(!do_adam || t >= 1.f, ENDIA_B200_EINVAL, "mlp_small_step: step count t starts at 1");
  SmallMlpArgs a{};
  a.n_layers = n_layers; a.batch = batch; a.act = act; a.x = x; a.y = y; a.loss = loss;
  int off = 0, dmax = 0, wmax = 0;
  for (int l = 0; l <= n_layers; ++l) {
    EB_REQUIRE(dims[l] >= 1 && dims[l] <= 256, ENDIA_B200_ELIMIT, "mlp_small_step: width %d outside [1, 256]", dims[l]);
    a.dims[l] = dims[l];
    a.act_off[l] = off;
    off += (batch * dims[l] + 3) / 4 * 4;
    if (l > 0 && dims[l] > dmax) dmax = dims[l];
    if (l > 0 && dims[l - 1] > dmax) dmax = dims[l - 1];
    if (l > 0 && dims[l - 1] * dims[l] > wmax) wmax = dims[l - 1] * dims[l];
  }
  a.d_off[0] = off; off += (batch * dmax + 3) / 4 * 4;
  a.d_off[1] = off; off += (batch * dmax + 3) / 4 * 4;
  // batch slices of the weight-gradient sums (same grouping as the kernel), and their scratch
  int red = 0;
  for (int l = 0; l < n_layers; ++l) {
    const int K = dims[l], N = dims[l + 1];
    const bool vec = (N & 3) == 0, quad = vec && (K & 3) == 0;
    const int groups = quad ? (K >> 2) * (N >> 2) : (vec ? K * (N >> 2) : K * N);
    int S = SM_THREADS / groups;
    S = S < 1 ? 1 : (S > 16 ? 16 : S);
    if (S > batch) S = batch;
    a.slices[l] = S;
    if (S > 1 && S * K * N > red) red = S * K * N;
  }
  if (sizeof(float) * (size_t)(off + red + wmax) > 200 * 1024) {   // no room: every layer in one slice
    for (int l = 0; l < n_layers; ++l) a.slices[l] = 1;
    red = 0;
  }
  a.red_off = off; off += (red + 3) / 4 * 4;
  a.w_off = off; off += wmax;
  int res = off - wmax;            // resident layout: every layer's weights and biases instead of one staging buffer
  for (int l = 0; l < n_layers; ++l) {
    a.w_offs[l] = res; res += (dims[l] * dims[l + 1] + 3) / 4 * 4;
    a.b_offs[l] = res; res += (dims[l + 1] + 3) / 4 * 4;
  }
  if (sizeof(float) * (size_t)res <= 200 * 1024) {
    a.resident = 1;
    off = res > off ? res : off;
  }
  const size_t smem = sizeof(float) * (size_t)off;
  EB_REQUIRE(smem <= 200 * 1024, ENDIA_B200_ELIMIT,
             "mlp_small_step: the network's activations need %zu bytes of shared memory (limit %d); "
             "use the layer-by-layer path", smem, 200 * 1024);
  for (int l = 0; l < n_layers; ++l) {
    EB_REQUIRE(W[l] && b[l] && gW[l] && gb[l], ENDIA_B200_EINVAL, "mlp_small_step: NULL pointer for layer %d", l);
    a.W[l] = W[l]; a.b[l] = b[l]; a.gW[l] = gW[l]; a.gb[l] = gb[l];
    if (do_adam) {
      EB_REQUIRE(mW[l] && vW[l] && mb[l] && vb[l], ENDIA_B200_EINVAL, "mlp_small_step: NULL Adam state for layer %d", l);
      a.mW[l] = mW[l]; a.vW[l] = vW[l]; a.mb[l] = mb[l]; a.vb[l] = vb[l];
    }
  }
  a.do_adam = do_adam;
  a.lr = lr; a.b1 = beta1; a.b2 = beta2; a.eps = eps;
  a.omb1 = 1.f - beta1; a.omb2 = 1.f - beta2;
  a.c1 = do_adam ? 1.f - powf(beta1, t) : 1.f;
  a.c2 = do_adam ? 1.f - powf(beta2, t) : 1.f;
  static size_t attr_bytes = 0;
  if (smem > attr_bytes) {
    EB_CUDA(cudaFuncSetAttribute(mlp_small_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_bytes = 200 * 1024;
  }
  mlp_small_step_kernel<<<1, SM_THREADS, smem, as_stream(stream)>>>(a);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}
