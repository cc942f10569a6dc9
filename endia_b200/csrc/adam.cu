// Fused multi-tensor optimizer steps. One launch over all parameter tensors replaces the array
// expressions per tensor of Adam.step (endia/optim/adam.mojo:47-65, ~14 of them), SGD.step
// (endia/optim/sgd.mojo:40-63), RMSprop.step (endia/optim/rmsprop.mojo:39-53) and Adagrad.step
// (endia/optim/adagrad.mojo:36-45); the operation order inside an element follows the reference
// so that fp32 results agree to rounding.
#include "common.cuh"
#include <cuda_bf16.h>

namespace eb {

constexpr int ADAM_MAX_TENSORS = 40;  // per launch; longer lists are issued in groups
constexpr int ADAM_CHUNK = 256 * 4 * 8;  // elements per CTA work item

struct AdamArgs {
  float *p[ADAM_MAX_TENSORS];
  const float *g[ADAM_MAX_TENSORS];
  float *m[ADAM_MAX_TENSORS];
  float *v[ADAM_MAX_TENSORS];
  float *lo[ADAM_MAX_TENSORS];   // optional: tf32 low part of the updated parameter, or its bf16 split
  int lo_is_bf16;                // lo[t] holds [numel bf16(p)][numel bf16(p - tf32(p))] instead
  int64_t chunk_start[ADAM_MAX_TENSORS + 1];  // prefix sum of chunks per tensor
  int64_t numel[ADAM_MAX_TENSORS];
  int n;
  float lr, b1, b2, eps, omb1, omb2, c1, c2, gscale;
  // SGD: b1 = momentum, b2 = weight decay. RMSprop: b1 = alpha, omb1 = 1 - alpha. Adagrad: lr, eps.
  const float *t_dev;            // Adam: the step count lives on the device (c1, c2 are formed there)
};

enum { OPT_ADAM = 0, OPT_SGD = 1, OPT_SGD_MOMENTUM = 2, OPT_RMSPROP = 3, OPT_ADAGRAD = 4 };

__device__ __forceinline__ float tf32_lo(float x) {
  return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

__device__ __forceinline__ void adam_one(float &p, float g, float &m, float &v, const AdamArgs &a, float c1,
                                         float c2) {
  g *= a.gscale;
  m = a.b1 * m + a.omb1 * g;           // adam.mojo:49-51
  v = a.b2 * v + (a.omb2 * g) * g;     // adam.mojo:52-56, (1-b2)*g*g left to right
  const float mhat = m / c1;           // adam.mojo:57-58
  const float vhat = v / c2;
  p = p - (a.lr * mhat) / (sqrtf(vhat) + a.eps);  // adam.mojo:61-63
}

// One element of the other optimizers; `s` is the velocity (SGD) or the cache (RMSprop, Adagrad).
template <int KIND>
__device__ __forceinline__ void opt_one(float &p, float g, float &s, const AdamArgs &a) {
  g *= a.gscale;
  if (KIND == OPT_SGD || KIND == OPT_SGD_MOMENTUM) {
    if (a.b2 > 0.f) g = g + a.b2 * p;               // sgd.mojo:42-54: grad + weight_decay * param
    if (KIND == OPT_SGD_MOMENTUM) {
      s = a.b1 * s - a.lr * g;                      // sgd.mojo:43-47, 55-58
      p = p + s;
    } else {
      p = p - a.lr * g;                             // sgd.mojo:50-53, 62
    }
  } else if (KIND == OPT_RMSPROP) {
    s = a.b1 * s + (a.omb1 * g) * g;                // rmsprop.mojo:41-46
    p = p - (a.lr * g) / (sqrtf(s) + a.eps);        // rmsprop.mojo:48-52
  } else {
    s = s + g * g;                                  // adagrad.mojo:38
    p = p - (a.lr * g) / (sqrtf(s) + a.eps);        // adagrad.mojo:40-44
  }
}

template <int KIND>
__global__ void __launch_bounds__(256) opt_kernel(const __grid_constant__ AdamArgs a) {
  constexpr bool HAS_S = KIND != OPT_SGD;
  const int64_t total = a.chunk_start[a.n];
  for (int64_t c = blockIdx.x; c < total; c += gridDim.x) {
    int t = 0;
    while (t + 1 < a.n && a.chunk_start[t + 1] <= c) ++t;
    const int64_t n = a.numel[t];
    const int64_t e0 = (c - a.chunk_start[t]) * ADAM_CHUNK;
    int64_t e1 = e0 + ADAM_CHUNK;
    if (e1 > n) e1 = n;
    float *p = a.p[t]; const float *g = a.g[t]; float *s = a.m[t];
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       (HAS_S ? reinterpret_cast<uintptr_t>(s) : 0)) & 15) == 0;
    int64_t v1 = e0;
    if (vec) {
      v1 = e1 & ~int64_t(3);
      for (int64_t i = e0 + threadIdx.x * 4; i < v1; i += 256 * 4) {
        float4 pp = *reinterpret_cast<float4 *>(p + i);
        const float4 gg = __ldg(reinterpret_cast<const float4 *>(g + i));
        float4 ss = make_float4(0.f, 0.f, 0.f, 0.f);
        if (HAS_S) ss = *reinterpret_cast<float4 *>(s + i);
        opt_one<KIND>(pp.x, gg.x, ss.x, a); opt_one<KIND>(pp.y, gg.y, ss.y, a);
        opt_one<KIND>(pp.z, gg.z, ss.z, a); opt_one<KIND>(pp.w, gg.w, ss.w, a);
        *reinterpret_cast<float4 *>(p + i) = pp;
        if (HAS_S) *reinterpret_cast<float4 *>(s + i) = ss;
      }
    }
    for (int64_t i = v1 + threadIdx.x; i < e1; i += 256) {
      float ss = HAS_S ? s[i] : 0.f;
      opt_one<KIND>(p[i], g[i], ss, a);
      if (HAS_S) s[i] = ss;
    }
  }
}

// t_dev[0] += 1: the step count of a step that is replayed from a CUDA graph advances on the device.
__global__ void adam_bump_kernel(float *t_dev) { t_dev[0] += 1.f; }

__global__ void __launch_bounds__(256) adam_kernel(const __grid_constant__ AdamArgs a) {
  float c1 = a.c1, c2 = a.c2;
  if (a.t_dev) {
    // 1 - beta^t with the power correctly rounded to fp32 (evaluated in double), as the host forms it
    const double t = (double)__ldg(a.t_dev);
    c1 = 1.f - (float)pow((double)a.b1, t);
    c2 = 1.f - (float)pow((double)a.b2, t);
  }
  const int64_t total = a.chunk_start[a.n];
  for (int64_t c = blockIdx.x; c < total; c += gridDim.x) {
    int t = 0;
    while (t + 1 < a.n && a.chunk_start[t + 1] <= c) ++t;
    const int64_t n = a.numel[t];
    const int64_t e0 = (c - a.chunk_start[t]) * ADAM_CHUNK;
    int64_t e1 = e0 + ADAM_CHUNK;
    if (e1 > n) e1 = n;
    float *p = a.p[t]; const float *g = a.g[t]; float *m = a.m[t]; float *v = a.v[t];
    float *lo = a.lo[t];
    const bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                       reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    if (vec) {
      const int64_t v1 = e1 & ~int64_t(3);
      for (int64_t i = e0 + threadIdx.x * 4; i < v1; i += 256 * 4) {
        float4 pp = *reinterpret_cast<float4 *>(p + i);
        float4 gg = __ldg(reinterpret_cast<const float4 *>(g + i));
        float4 mm = *reinterpret_cast<float4 *>(m + i);
        float4 vv = *reinterpret_cast<float4 *>(v + i);
        adam_one(pp.x, gg.x, mm.x, vv.x, a, c1, c2); adam_one(pp.y, gg.y, mm.y, vv.y, a, c1, c2);
        adam_one(pp.z, gg.z, mm.z, vv.z, a, c1, c2); adam_one(pp.w, gg.w, mm.w, vv.w, a, c1, c2);
        *reinterpret_cast<float4 *>(p + i) = pp;
        *reinterpret_cast<float4 *>(m + i) = mm;
        *reinterpret_cast<float4 *>(v + i) = vv;
        if (lo && !a.lo_is_bf16) {
          lo[i + 0] = tf32_lo(pp.x); lo[i + 1] = tf32_lo(pp.y);
          lo[i + 2] = tf32_lo(pp.z); lo[i + 3] = tf32_lo(pp.w);
        } else if (lo) {
          __nv_bfloat16 *h16 = reinterpret_cast<__nv_bfloat16 *>(lo), *l16 = h16 + n;
          __nv_bfloat162 h01 = __floats2bfloat162_rn(pp.x, pp.y), h23 = __floats2bfloat162_rn(pp.z, pp.w);
          __nv_bfloat162 l01 = __floats2bfloat162_rn(tf32_lo(pp.x), tf32_lo(pp.y));
          __nv_bfloat162 l23 = __floats2bfloat162_rn(tf32_lo(pp.z), tf32_lo(pp.w));
          uint2 hv, lv;
          hv.x = *reinterpret_cast<uint32_t *>(&h01); hv.y = *reinterpret_cast<uint32_t *>(&h23);
          lv.x = *reinterpret_cast<uint32_t *>(&l01); lv.y = *reinterpret_cast<uint32_t *>(&l23);
          *reinterpret_cast<uint2 *>(h16 + i) = hv;
          *reinterpret_cast<uint2 *>(l16 + i) = lv;
        }
      }
      for (int64_t i = v1 + threadIdx.x; i < e1; i += 256) {
        adam_one(p[i], g[i], m[i], v[i], a, c1, c2);
        if (lo && !a.lo_is_bf16) {
          lo[i] = tf32_lo(p[i]);
        } else if (lo) {
          __nv_bfloat16 *h16 = reinterpret_cast<__nv_bfloat16 *>(lo);
          h16[i] = __float2bfloat16_rn(p[i]);
          h16[n + i] = __float2bfloat16_rn(tf32_lo(p[i]));
        }
      }
    } else {
      for (int64_t i = e0 + threadIdx.x; i < e1; i += 256) {
        adam_one(p[i], g[i], m[i], v[i], a, c1, c2);
        if (lo && !a.lo_is_bf16) {
          lo[i] = tf32_lo(p[i]);
        } else if (lo) {
          __nv_bfloat16 *h16 = reinterpret_cast<__nv_bfloat16 *>(lo);
          h16[i] = __float2bfloat16_rn(p[i]);
          h16[n + i] = __float2bfloat16_rn(tf32_lo(p[i]));
        }
      }
    }
  }
}

}  // namespace eb

using namespace eb;

static int adam_launch(int32_t n_tensors, float *const *params, const float *const *grads, float *const *m,
                       float *const *v, float *const *p_lo, int lo_is_bf16, const int64_t *numel, float lr,
                       float beta1, float beta2, float eps, float t, float grad_scale, void *stream,
                       float *t_dev = nullptr, bool bump = true) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n_tensors >= 0, ENDIA_B200_EINVAL, "adam: negative tensor count");
  if (n_tensors == 0) return ENDIA_B200_OK;
  EB_REQUIRE(params && grads && m && v && numel, ENDIA_B200_EINVAL, "adam: NULL argument array");
  EB_REQUIRE(t_dev || t >= 1.f, ENDIA_B200_EINVAL, "adam: step count t starts at 1 (adam.mojo:40)");
  for (int i0 = 0; i0 < n_tensors; i0 += ADAM_MAX_TENSORS) {
    AdamArgs a{};
    a.n = 0;
    a.chunk_start[0] = 0;
    for (int i = i0; i < n_tensors && a.n < ADAM_MAX_TENSORS; ++i) {
      EB_REQUIRE(numel[i] >= 0, ENDIA_B200_EINVAL, "adam: negative numel for tensor %d", i);
      if (numel[i] == 0) continue;
      EB_REQUIRE(params[i] && grads[i] && m[i] && v[i], ENDIA_B200_EINVAL,
                 "adam: NULL pointer for tensor %d", i);
      a.p[a.n] = params[i]; a.g[a.n] = grads[i]; a.m[a.n] = m[i]; a.v[a.n] = v[i];
      a.lo[a.n] = p_lo ? p_lo[i] : nullptr;
      EB_REQUIRE(!(lo_is_bf16 && a.lo[a.n]) || (numel[i] % 8 == 0 && (reinterpret_cast<uintptr_t>(params[i]) & 15) == 0 &&
                                                (reinterpret_cast<uintptr_t>(a.lo[a.n]) & 15) == 0),
                 ENDIA_B200_EINVAL, "adam: the bf16 split needs numel %% 8 == 0 and 16-byte aligned arrays (tensor %d)", i);
      a.numel[a.n] = numel[i];
      a.chunk_start[a.n + 1] = a.chunk_start[a.n] + ceil_div(numel[i], ADAM_CHUNK);
      ++a.n;
    }
    if (a.n == 0) continue;
    a.lr = lr; a.b1 = beta1; a.b2 = beta2; a.eps = eps; a.gscale = grad_scale;
    a.lo_is_bf16 = lo_is_bf16;
    // fp32 scalars exactly as the reference forms them (adam.mojo:50, 54, 57-58).
    a.omb1 = 1.f - beta1;
    a.omb2 = 1.f - beta2;
    a.c1 = 1.f - powf(beta1, t);
    a.c2 = 1.f - powf(beta2, t);
    a.t_dev = t_dev;
    int64_t total = a.chunk_start[a.n];
    int64_t cap = (int64_t)(sm_count() > 0 ? sm_count() : 148) * 8;
    int grid = (int)(total < cap ? total : cap);
    adam_kernel<<<grid, 256, 0, as_stream(stream)>>>(a);
    EB_LAUNCH_CHECK();
  }
  if (t_dev && bump) {
    adam_bump_kernel<<<1, 1, 0, as_stream(stream)>>>(t_dev);
    EB_LAUNCH_CHECK();
  }
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_adam_step_multi_graph(int32_t n_tensors, float *const *params,
                                                const float *const *grads, float *const *m,
                                                float *const *v, void *const *p16, const int64_t *numel,
                                                float lr, float beta1, float beta2, float eps, float *t_dev,
                                                int32_t advance, float grad_scale, void *stream) {
  EB_REQUIRE(t_dev != nullptr, ENDIA_B200_EINVAL, "adam: t_dev is NULL");
  if (n_tensors == 0 && advance) {      // only the count: the tensors of this step went in earlier calls
    int st = require_device();
    if (st) return st;
    adam_bump_kernel<<<1, 1, 0, as_stream(stream)>>>(t_dev);
    EB_LAUNCH_CHECK();
    return ENDIA_B200_OK;
  }
  return adam_launch(n_tensors, params, grads, m, v, reinterpret_cast<float *const *>(p16), 1, numel, lr, beta1,
                     beta2, eps, 1.f, grad_scale, stream, t_dev, advance != 0);
}

extern "C" int endia_b200_adam_step_multi_lo(int32_t n_tensors, float *const *params,
                                             const float *const *grads, float *const *m,
                                             float *const *v, float *const *p_lo, const int64_t *numel,
                                             float lr, float beta1, float beta2, float eps, float t,
                                             float grad_scale, void *stream) {
  return adam_launch(n_tensors, params, grads, m, v, p_lo, 0, numel, lr, beta1, beta2, eps, t, grad_scale, stream);
}

extern "C" int endia_b200_adam_step_multi_bf16(int32_t n_tensors, float *const *params,
                                               const float *const *grads, float *const *m,
                                               float *const *v, void *const *p16, const int64_t *numel,
                                               float lr, float beta1, float beta2, float eps, float t,
                                               float grad_scale, void *stream) {
  return adam_launch(n_tensors, params, grads, m, v, reinterpret_cast<float *const *>(p16), 1, numel, lr, beta1,
                     beta2, eps, t, grad_scale, stream);
}

extern "C" int endia_b200_adam_step_multi(int32_t n_tensors, float *const *params,
                                          const float *const *grads, float *const *m,
                                          float *const *v, const int64_t *numel, float lr,
                                          float beta1, float beta2, float eps, float t,
                                          float grad_scale, void *stream) {
  return endia_b200_adam_step_multi_lo(n_tensors, params, grads, m, v, nullptr, numel, lr, beta1, beta2,
                                       eps, t, grad_scale, stream);
}

namespace eb {

// Shared host side of the SGD / RMSprop / Adagrad entry points: `state` is the velocity or cache
// array list (NULL for SGD without momentum).
static int launch_opt(int kind, const char *what, int32_t n_tensors, float *const *params,
                      const float *const *grads, float *const *state, const int64_t *numel, AdamArgs h,
                      cudaStream_t stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n_tensors >= 0, ENDIA_B200_EINVAL, "%s: negative tensor count", what);
  if (n_tensors == 0) return ENDIA_B200_OK;
  EB_REQUIRE(params && grads && numel && (state || kind == OPT_SGD), ENDIA_B200_EINVAL,
             "%s: NULL argument array", what);
  for (int i0 = 0; i0 < n_tensors; i0 += ADAM_MAX_TENSORS) {
    AdamArgs a = h;
    a.n = 0;
    a.chunk_start[0] = 0;
    for (int i = i0; i < n_tensors && a.n < ADAM_MAX_TENSORS; ++i) {
      EB_REQUIRE(numel[i] >= 0, ENDIA_B200_EINVAL, "%s: negative numel for tensor %d", what, i);
      if (numel[i] == 0) continue;
      EB_REQUIRE(params[i] && grads[i] && (kind == OPT_SGD || state[i]), ENDIA_B200_EINVAL,
                 "%s: NULL pointer for tensor %d", what, i);
      a.p[a.n] = params[i]; a.g[a.n] = grads[i]; a.m[a.n] = kind == OPT_SGD ? nullptr : state[i];
      a.numel[a.n] = numel[i];
      a.chunk_start[a.n + 1] = a.chunk_start[a.n] + ceil_div(numel[i], ADAM_CHUNK);
      ++a.n;
    }
    if (a.n == 0) continue;
    const int64_t total = a.chunk_start[a.n];
    const int64_t cap = (int64_t)(sm_count() > 0 ? sm_count() : 148) * 8;
    const int grid = (int)(total < cap ? total : cap);
    switch (kind) {
      case OPT_SGD: opt_kernel<OPT_SGD><<<grid, 256, 0, stream>>>(a); break;
      case OPT_SGD_MOMENTUM: opt_kernel<OPT_SGD_MOMENTUM><<<grid, 256, 0, stream>>>(a); break;
      case OPT_RMSPROP: opt_kernel<OPT_RMSPROP><<<grid, 256, 0, stream>>>(a); break;
      default: opt_kernel<OPT_ADAGRAD><<<grid, 256, 0, stream>>>(a); break;
    }
    EB_LAUNCH_CHECK();
  }
  return ENDIA_B200_OK;
}

}  // namespace eb

extern "C" int endia_b200_sgd_step_multi(int32_t n_tensors, float *const *params, const float *const *grads,
                                         float *const *velocity, const int64_t *numel, float lr,
                                         float momentum, float weight_decay, float grad_scale, void *stream) {
  EB_REQUIRE(momentum >= 0.f && weight_decay >= 0.f, ENDIA_B200_EINVAL,
             "sgd: momentum and weight decay must not be negative");
  EB_REQUIRE(momentum == 0.f || velocity, ENDIA_B200_EINVAL, "sgd: momentum needs the velocity arrays");
  AdamArgs h{};
  h.lr = lr; h.b1 = momentum; h.b2 = weight_decay; h.gscale = grad_scale;
  return launch_opt(momentum > 0.f ? OPT_SGD_MOMENTUM : OPT_SGD, "sgd", n_tensors, params, grads, velocity, numel,
                    h, as_stream(stream));
}

extern "C" int endia_b200_rmsprop_step_multi(int32_t n_tensors, float *const *params,
                                             const float *const *grads, float *const *cache,
                                             const int64_t *numel, float lr, float alpha, float eps,
                                             float grad_scale, void *stream) {
  AdamArgs h{};
  h.lr = lr; h.b1 = alpha; h.omb1 = 1.f - alpha; h.eps = eps; h.gscale = grad_scale;
  return launch_opt(OPT_RMSPROP, "rmsprop", n_tensors, params, grads, cache, numel, h, as_stream(stream));
}

extern "C" int endia_b200_adagrad_step_multi(int32_t n_tensors, float *const *params,
                                             const float *const *grads, float *const *cache,
                                             const int64_t *numel, float lr, float eps, float grad_scale,
                                             void *stream) {
  AdamArgs h{};
  h.lr = lr; h.eps = eps; h.gscale = grad_scale;
  return launch_opt(OPT_ADAGRAD, "adagrad", n_tensors, params, grads, cache, numel, h, as_stream(stream));
}
