// Elementwise kernels: one templated, 128-bit vectorised kernel for every unary/binary op,
// reading broadcast operands through stride-0 dimensions instead of materialising them.
// Formulas follow the per-op `unary_simd_op` / `binary_simd_op` of the reference
// (endia/functional/unary_ops/*_op.mojo, endia/functional/binary_ops/*_op.mojo); the driver
// loops they replace are execute_unary_op (unary_ops/_utils.mojo:77-134), execute_binary_op
// (binary_ops/_utils.mojo:93-177) and execute_copy_raw (functional/_utils.mojo:79-163).
#include "common.cuh"

namespace eb {

constexpr int EW_MAX_DIMS = 6;

// Collapsed iteration space: `nd` dims, innermost last. Strides in floats for real data and in
// complex elements for complex data.
struct EwParams {
  const float *a;
  const float *b;
  float *out;
  int64_t total;  // number of work items (vectors of VEC elements)
  int nd;
  int64_t shape[EW_MAX_DIMS];  // innermost extent is in units of VEC
  int64_t sa[EW_MAX_DIMS];
  int64_t sb[EW_MAX_DIMS];
};

struct c32 {
  float re, im;
};

// ---------------------------------------------------------------- real functors
template <int OP>
__device__ __forceinline__ float un_real(float x) {
  if constexpr (OP == ENDIA_B200_UN_COPY) return x;
  if constexpr (OP == ENDIA_B200_UN_NEG) return -x;
  if constexpr (OP == ENDIA_B200_UN_RELU) return fmaxf(x, 0.f);           // relu_op.mojo:115
  if constexpr (OP == ENDIA_B200_UN_TANH) return tanhf(x);                // tanh_op.mojo:112-115
  if constexpr (OP == ENDIA_B200_UN_SIGMOID) return 1.f / (1.f + expf(-x));  // sigmoid_op.mojo:118-121
  if constexpr (OP == ENDIA_B200_UN_SQUARE) return x * x;                 // square_op.mojo:117
  if constexpr (OP == ENDIA_B200_UN_SQRT) return sqrtf(x);                // sqrt_op.mojo:111-113
  if constexpr (OP == ENDIA_B200_UN_ABS) return fabsf(x);                 // abs_op.mojo:114
  if constexpr (OP == ENDIA_B200_UN_SIGN) return x / fabsf(x);            // sign_op.mojo:78-80
  if constexpr (OP == ENDIA_B200_UN_CONJ) return x;
  if constexpr (OP == ENDIA_B200_UN_EXP) return expf(x);
  if constexpr (OP == ENDIA_B200_UN_LOG) return logf(fabsf(x));           // log_op.mojo:111-113
  if constexpr (OP == ENDIA_B200_UN_SIN) return sinf(x);
  if constexpr (OP == ENDIA_B200_UN_COS) return cosf(x);
  if constexpr (OP == ENDIA_B200_UN_RECIPROCAL) return 1.f / x;
  if constexpr (OP == ENDIA_B200_UN_SINH) return sinhf(x);                // sinh_op.mojo:108
  if constexpr (OP == ENDIA_B200_UN_COSH) return coshf(x);                // cosh_op.mojo:109
  if constexpr (OP == ENDIA_B200_UN_TAN) return tanf(x);                  // tan_op.mojo:101
  if constexpr (OP == ENDIA_B200_UN_ASIN) return asinf(x);                // asin_op.mojo:103
  if constexpr (OP == ENDIA_B200_UN_ACOS) return acosf(x);                // acos_op.mojo:111
  if constexpr (OP == ENDIA_B200_UN_ATAN) return atanf(x);                // atan_op.mojo:105
  return x;
}

template <int OP>
__device__ __forceinline__ float bin_real(float a, float b) {
  if constexpr (OP == ENDIA_B200_BIN_ADD) return a + b;
  if constexpr (OP == ENDIA_B200_BIN_SUB) return a - b;
  if constexpr (OP == ENDIA_B200_BIN_MUL) return a * b;
  if constexpr (OP == ENDIA_B200_BIN_DIV) return a / b;
  if constexpr (OP == ENDIA_B200_BIN_POW) {
    // Polar form of the reference, real lane (pow_op.mojo:139-147): a negative base gives
    // |a|^b * cos(pi*b).
    float lm = logf(fabsf(a));
    float u = expf(lm * b);
    if (a >= 0.f) return u;
    return u * cosf(3.14159265358979323846f * b);
  }
  if constexpr (OP == ENDIA_B200_BIN_GREATER) return a > b ? 1.f : 0.f;  // greater_op.mojo:55-60
  if constexpr (OP == ENDIA_B200_BIN_GREATER_EQUAL) return a >= b ? 1.f : 0.f;   // greater_equal_op.mojo
  if constexpr (OP == ENDIA_B200_BIN_LESS) return a < b ? 1.f : 0.f;             // less_op.mojo
  if constexpr (OP == ENDIA_B200_BIN_LESS_EQUAL) return a <= b ? 1.f : 0.f;      // less_equal_op.mojo
  if constexpr (OP == ENDIA_B200_BIN_EQUAL) return a == b ? 1.f : 0.f;           // equal_op.mojo
  if constexpr (OP == ENDIA_B200_BIN_NOT_EQUAL) return a != b ? 1.f : 0.f;       // not_equal_op.mojo
  if constexpr (OP == ENDIA_B200_BIN_RELU_BWD) return a > 0.f ? b : 0.f;  // relu_op.mojo:95
  if constexpr (OP == ENDIA_B200_BIN_TANH_BWD) {                          // tanh_op.mojo:92
    float t = tanhf(a);
    return (1.f - t * t) * b;
  }
  if constexpr (OP == ENDIA_B200_BIN_SIGMOID_BWD) return a * (1.f - a) * b;  // sigmoid_op.mojo:98
  if constexpr (OP == ENDIA_B200_BIN_ABS_BWD) return (a / fabsf(a)) * b;     // abs_op.mojo:93, sign_op.mojo:78-80
  if constexpr (OP == ENDIA_B200_BIN_SQUARE_BWD) return (2.f * a) * b;       // square_op.mojo:96
  if constexpr (OP == ENDIA_B200_BIN_TANH_OUT_BWD) return (1.f - a * a) * b;  // tanh_op.mojo:92, a = tanh output
  if constexpr (OP == ENDIA_B200_BIN_TANH_OUT_BWD2) return (-2.f * a) * b;
  return a;
}

// ------------------------------------------------------------- complex functors
template <int OP>
__device__ __forceinline__ c32 un_cplx(c32 z) {
  c32 r = z;
  if constexpr (OP == ENDIA_B200_UN_NEG) { r.re = -z.re; r.im = -z.im; }
  if constexpr (OP == ENDIA_B200_UN_CONJ) { r.im = -z.im; }
  if constexpr (OP == ENDIA_B200_UN_SQUARE) { r.re = z.re * z.re - z.im * z.im; r.im = 2.f * z.re * z.im; }
  if constexpr (OP == ENDIA_B200_UN_ABS) { r.re = sqrtf(z.re * z.re + z.im * z.im); r.im = 0.f; }
  if constexpr (OP == ENDIA_B200_UN_SIGN) {
    float n = sqrtf(z.re * z.re + z.im * z.im);
    r.re = z.re / n; r.im = z.im / n;
  }
  if constexpr (OP == ENDIA_B200_UN_SQRT) {
    float m = sqrtf(z.re * z.re + z.im * z.im);
    r.re = sqrtf((m + z.re) * 0.5f);
    r.im = copysignf(sqrtf((m - z.re) * 0.5f), z.im);
  }
  if constexpr (OP == ENDIA_B200_UN_EXP) {
    float e = expf(z.re), s, c;
    sincosf(z.im, &s, &c);
    r.re = e * c; r.im = e * s;
  }
  if constexpr (OP == ENDIA_B200_UN_LOG) {
    r.re = logf(sqrtf(z.re * z.re + z.im * z.im));
    r.im = atan2f(z.im, z.re);
  }
  if constexpr (OP == ENDIA_B200_UN_TANH) {
    float d = coshf(2.f * z.re) + cosf(2.f * z.im);
    r.re = sinhf(2.f * z.re) / d; r.im = sinf(2.f * z.im) / d;
  }
  if constexpr (OP == ENDIA_B200_UN_SIN) {
    r.re = sinf(z.re) * coshf(z.im); r.im = cosf(z.re) * sinhf(z.im);
  }
  if constexpr (OP == ENDIA_B200_UN_COS) {
    r.re = cosf(z.re) * coshf(z.im); r.im = -sinf(z.re) * sinhf(z.im);
  }
  if constexpr (OP == ENDIA_B200_UN_RECIPROCAL) {
    float d = z.re * z.re + z.im * z.im;
    r.re = z.re / d; r.im = -z.im / d;
  }
  if constexpr (OP == ENDIA_B200_UN_SINH) {   // sinh_op.mojo:108-109
    r.re = sinhf(z.re) * cosf(z.im); r.im = coshf(z.re) * sinf(z.im);
  }
  if constexpr (OP == ENDIA_B200_UN_COSH) {   // cosh_op.mojo:109-110
    r.re = coshf(z.re) * cosf(z.im); r.im = sinhf(z.re) * sinf(z.im);
  }
  // tan, acos and atan act on the real part and give a zero imaginary part, asin uses the
  // reference's own pair of formulas (tan_op.mojo:101-102, acos_op.mojo:111-112,
  // atan_op.mojo:105-106, asin_op.mojo:103-104)
  if constexpr (OP == ENDIA_B200_UN_TAN) { r.re = tanf(z.re); r.im = 0.f; }
  if constexpr (OP == ENDIA_B200_UN_ACOS) { r.re = acosf(z.re); r.im = 0.f; }
  if constexpr (OP == ENDIA_B200_UN_ATAN) { r.re = atanf(z.re); r.im = 0.f; }
  if constexpr (OP == ENDIA_B200_UN_ASIN) {
    r.re = asinf(z.re) * coshf(z.im); r.im = -acosf(z.re) * sinhf(z.im);
  }
  return r;
}

template <int OP>
__device__ __forceinline__ c32 bin_cplx(c32 a, c32 b) {
  c32 r = a;
  if constexpr (OP == ENDIA_B200_BIN_ADD) { r.re = a.re + b.re; r.im = a.im + b.im; }
  if constexpr (OP == ENDIA_B200_BIN_SUB) { r.re = a.re - b.re; r.im = a.im - b.im; }
  if constexpr (OP == ENDIA_B200_BIN_MUL) {  // mul_op.mojo:152-155
    r.re = a.re * b.re - a.im * b.im; r.im = a.re * b.im + a.im * b.re;
  }
  if constexpr (OP == ENDIA_B200_BIN_DIV) {  // div_op.mojo:138-142
    float d = b.re * b.re + b.im * b.im;
    r.re = (a.re * b.re + a.im * b.im) / d; r.im = (a.im * b.re - a.re * b.im) / d;
  }
  if constexpr (OP == ENDIA_B200_BIN_POW) {  // pow_op.mojo:139-147
    float lm = logf(sqrtf(a.re * a.re + a.im * a.im));
    float ar = atan2f(a.im, a.re);
    float u = expf(lm * b.re - ar * b.im);
    float v = lm * b.im + ar * b.re;
    float s, c;
    sincosf(v, &s, &c);
    r.re = u * c; r.im = u * s;
  }
  if constexpr (OP == ENDIA_B200_BIN_COMPLEX) { r.re = a.re; r.im = b.re; }
  if constexpr (OP == ENDIA_B200_BIN_ABS_BWD) {   // sign(a) * b as a complex product (no conjugation)
    const float nrm = sqrtf(a.re * a.re + a.im * a.im);
    const float sr = a.re / nrm, si = a.im / nrm;
    r.re = sr * b.re - si * b.im; r.im = sr * b.im + si * b.re;
  }
  if constexpr (OP == ENDIA_B200_BIN_SQUARE_BWD) {
    const float tr = 2.f * a.re, ti = 2.f * a.im;
    r.re = tr * b.re - ti * b.im; r.im = tr * b.im + ti * b.re;
  }
  return r;
}

// ---------------------------------------------------------------------- kernels
__device__ __forceinline__ void decompose(const EwParams &p, int64_t i, int64_t &oa, int64_t &ob) {
  oa = 0; ob = 0;
#pragma unroll
  for (int d = EW_MAX_DIMS - 1; d >= 0; --d) {
    if (d < p.nd) {
      int64_t q = (d == 0) ? 0 : i / p.shape[d];
      int64_t r = (d == 0) ? i : i - q * p.shape[d];
      oa += r * p.sa[d];
      ob += r * p.sb[d];
      i = q;
    }
  }
}

// Real data, VEC floats per work item along the innermost dim (inner strides are 0 or 1 when
// VEC > 1; a stride-0 inner operand is splatted).
template <int OP, bool BINARY, int VEC>
__global__ void __launch_bounds__(256) ew_real_kernel(EwParams p) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += step) {
    int64_t oa, ob;
    if (p.nd == 1) {
      oa = i * p.sa[0]; ob = i * p.sb[0];
    } else {
      decompose(p, i, oa, ob);
    }
    if constexpr (VEC == 4) {
      // Innermost strides were pre-multiplied by VEC on the host (0 stays 0).
      float4 va, vb, vo;
      const int in = p.nd - 1;
      if (p.sa[in] != 0) va = *reinterpret_cast<const float4 *>(p.a + oa);
      else { float s = p.a[oa]; va = make_float4(s, s, s, s); }
      if constexpr (BINARY) {
        if (p.sb[in] != 0) vb = *reinterpret_cast<const float4 *>(p.b + ob);
        else { float s = p.b[ob]; vb = make_float4(s, s, s, s); }
        vo.x = bin_real<OP>(va.x, vb.x); vo.y = bin_real<OP>(va.y, vb.y);
        vo.z = bin_real<OP>(va.z, vb.z); vo.w = bin_real<OP>(va.w, vb.w);
      } else {
        vo.x = un_real<OP>(va.x); vo.y = un_real<OP>(va.y);
        vo.z = un_real<OP>(va.z); vo.w = un_real<OP>(va.w);
      }
      *reinterpret_cast<float4 *>(p.out + i * 4) = vo;
    } else {
      float x = p.a[oa];
      if constexpr (BINARY) p.out[i] = bin_real<OP>(x, p.b[ob]);
      else p.out[i] = un_real<OP>(x);
    }
  }
}

// Complex data: one (re, im) pair per work item, strides in complex elements. A real operand
// of a binary op (a_real / b_real) contributes a zero imaginary part.
template <int OP, bool BINARY>
__global__ void __launch_bounds__(256)
ew_cplx_kernel(EwParams p, int a_real, int b_real) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.total; i += step) {
    int64_t oa, ob;
    decompose(p, i, oa, ob);
    c32 x, y, r;
    if (a_real) { x.re = p.a[oa]; x.im = 0.f; }
    else { float2 t = *reinterpret_cast<const float2 *>(p.a + 2 * oa); x.re = t.x; x.im = t.y; }
    if constexpr (BINARY) {
      if (b_real) { y.re = p.b[ob]; y.im = 0.f; }
      else { float2 t = *reinterpret_cast<const float2 *>(p.b + 2 * ob); y.re = t.x; y.im = t.y; }
      r = bin_cplx<OP>(x, y);
    } else {
      r = un_cplx<OP>(x);
    }
    *reinterpret_cast<float2 *>(p.out + 2 * i) = make_float2(r.re, r.im);
  }
}

__global__ void __launch_bounds__(256) fill_kernel(float *dst, int64_t n_floats, float re, float im,
                                                   int is_complex) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_floats; i += step)
    dst[i] = (is_complex && (i & 1)) ? im : re;
}
__global__ void __launch_bounds__(256) eye_kernel(float *dst, int64_t n) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n * n; i += step)
    dst[i] = (i / n == i % n) ? 1.f : 0.f;
}

// ------------------------------------------------------------------ host side
// Builds the collapsed iteration space of `out`'s shape with the operand strides; adjacent dims
// are merged when both operands step through them like one longer dim.
static void collapse(const endia_b200_tensor *out, const endia_b200_tensor *a,
                     const endia_b200_tensor *b, EwParams &p, bool &ok) {
  int nd = 0;
  int64_t shp[ENDIA_B200_MAX_DIMS], sa[ENDIA_B200_MAX_DIMS], sb[ENDIA_B200_MAX_DIMS];
  for (int d = 0; d < out->ndim; ++d) {
    if (out->shape[d] == 1) continue;
    int64_t e = out->shape[d], xa = a->stride[d], xb = b->stride[d];
    if (nd > 0 && sa[nd - 1] == xa * e && sb[nd - 1] == xb * e) {
      shp[nd - 1] *= e; sa[nd - 1] = xa; sb[nd - 1] = xb;
    } else {
      shp[nd] = e; sa[nd] = xa; sb[nd] = xb; ++nd;
    }
  }
  if (nd == 0) { shp[0] = 1; sa[0] = 0; sb[0] = 0; nd = 1; }
  ok = nd <= EW_MAX_DIMS;
  if (!ok) return;
  p.nd = nd;
  for (int d = 0; d < nd; ++d) { p.shape[d] = shp[d]; p.sa[d] = sa[d]; p.sb[d] = sb[d]; }
}

static bool aligned16(const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

template <int OP, bool BINARY>
static int launch_real(EwParams p, cudaStream_t st) {
  // Vectorise by 4 when the innermost dim allows it for every operand.
  const int in = p.nd - 1;
  bool vec = (p.shape[in] % 4 == 0) && aligned16(p.out);
  auto operand_ok = [&](const float *base, const int64_t *s) {
    if (s[in] == 0) {
      return true;
    }
    if (s[in] != 1 || !aligned16(base)) return false;
    for (int d = 0; d < in; ++d)
      if (s[d] % 4 != 0) return false;
    return true;
  };
  vec = vec && operand_ok(p.a, p.sa) && (!BINARY || operand_ok(p.b, p.sb));
  int64_t n = 1;
  for (int d = 0; d < p.nd; ++d) n *= p.shape[d];
  if (n == 0) return ENDIA_B200_OK;
  if (vec) {
    p.shape[in] /= 4;
    p.sa[in] *= 4;
    p.sb[in] *= 4;
    p.total = n / 4;
    ew_real_kernel<OP, BINARY, 4><<<grid_for(p.total, 256), 256, 0, st>>>(p);
  } else {
    p.total = n;
    ew_real_kernel<OP, BINARY, 1><<<grid_for(p.total, 256), 256, 0, st>>>(p);
  }
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

template <int OP, bool BINARY>
static int launch_cplx(EwParams p, int a_real, int b_real, cudaStream_t st) {
  int64_t n = 1;
  for (int d = 0; d < p.nd; ++d) n *= p.shape[d];
  if (n == 0) return ENDIA_B200_OK;
  p.total = n;
  ew_cplx_kernel<OP, BINARY><<<grid_for(p.total, 256), 256, 0, st>>>(p, a_real, b_real);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

template <int OP>
static int dispatch_unary(const EwParams &p, bool cplx, cudaStream_t st) {
  if (!cplx) return launch_real<OP, false>(p, st);
  if constexpr (OP == ENDIA_B200_UN_RELU || OP == ENDIA_B200_UN_SIGMOID) {
    // relu_op.mojo:51-52 and sigmoid_op.mojo:49-50 raise for complex input.
    set_error("ew_unary: op %d is not defined for complex input", OP);
    return ENDIA_B200_EINVAL;
  } else {
    return launch_cplx<OP, false>(p, 0, 0, st);
  }
}

template <int OP>
static int dispatch_binary(const EwParams &p, bool a_c, bool b_c, cudaStream_t st) {
  if constexpr (OP == ENDIA_B200_BIN_COMPLEX) {
    if (a_c || b_c) {
      set_error("ew_binary: complex(re, im) takes two real operands");
      return ENDIA_B200_EINVAL;
    }
    return launch_cplx<OP, true>(p, 1, 1, st);
  }
  if (!a_c && !b_c) return launch_real<OP, true>(p, st);
  if constexpr (OP <= ENDIA_B200_BIN_POW || OP == ENDIA_B200_BIN_ABS_BWD || OP == ENDIA_B200_BIN_SQUARE_BWD) {
    return launch_cplx<OP, true>(p, !a_c, !b_c, st);
  } else {
    set_error("ew_binary: op %d is not defined for complex input", OP);
    return ENDIA_B200_EINVAL;
  }
}

}  // namespace eb

using namespace eb;

extern "C" {

int endia_b200_ew_unary(int op, const endia_b200_tensor *in, const endia_b200_tensor *out,
                        void *stream) {
  int st = require_device();
  if (st) return st;
  if ((st = check_tensor(in, "ew_unary: in"))) return st;
  if ((st = check_tensor(out, "ew_unary: out"))) return st;
  EB_REQUIRE(op >= 0 && op < ENDIA_B200_UN_COUNT, ENDIA_B200_EINVAL, "ew_unary: unknown op %d", op);
  EB_REQUIRE(in->ndim == out->ndim, ENDIA_B200_ESHAPE, "ew_unary: rank mismatch %d vs %d", in->ndim,
             out->ndim);
  for (int d = 0; d < in->ndim; ++d)
    EB_REQUIRE(in->shape[d] == out->shape[d], ENDIA_B200_ESHAPE, "ew_unary: shape mismatch in dim %d",
               d);
  EB_REQUIRE(is_contiguous(out), ENDIA_B200_EINVAL, "ew_unary: out must be contiguous");
  const bool cplx = in->is_complex != 0;
  // abs keeps a complex layout with a zero imaginary part (abs_op.mojo:114-115).
  EB_REQUIRE((out->is_complex != 0) == cplx, ENDIA_B200_EINVAL,
             "ew_unary: in/out complex flags differ");
  EwParams p{};
  bool ok;
  collapse(out, in, in, p, ok);
  EB_REQUIRE(ok, ENDIA_B200_EINVAL, "ew_unary: more than %d non-mergeable dims", EW_MAX_DIMS);
  const int w = cplx ? 2 : 1;
  p.a = static_cast<const float *>(in->data) + w * in->offset;
  p.b = p.a;
  p.out = static_cast<float *>(out->data) + w * out->offset;
  cudaStream_t s = as_stream(stream);
  switch (op) {
#define EB_CASE(OPC) case OPC: return dispatch_unary<OPC>(p, cplx, s);
    EB_CASE(ENDIA_B200_UN_COPY) EB_CASE(ENDIA_B200_UN_NEG) EB_CASE(ENDIA_B200_UN_RELU)
    EB_CASE(ENDIA_B200_UN_TANH) EB_CASE(ENDIA_B200_UN_SIGMOID) EB_CASE(ENDIA_B200_UN_SQUARE)
    EB_CASE(ENDIA_B200_UN_SQRT) EB_CASE(ENDIA_B200_UN_ABS) EB_CASE(ENDIA_B200_UN_SIGN)
    EB_CASE(ENDIA_B200_UN_CONJ) EB_CASE(ENDIA_B200_UN_EXP) EB_CASE(ENDIA_B200_UN_LOG)
    EB_CASE(ENDIA_B200_UN_SIN) EB_CASE(ENDIA_B200_UN_COS) EB_CASE(ENDIA_B200_UN_RECIPROCAL)
    EB_CASE(ENDIA_B200_UN_SINH) EB_CASE(ENDIA_B200_UN_COSH) EB_CASE(ENDIA_B200_UN_TAN)
    EB_CASE(ENDIA_B200_UN_ASIN) EB_CASE(ENDIA_B200_UN_ACOS) EB_CASE(ENDIA_B200_UN_ATAN)
#undef EB_CASE
  }
  return ENDIA_B200_EINVAL;
}

int endia_b200_ew_binary(int op, const endia_b200_tensor *a, const endia_b200_tensor *b,
                         const endia_b200_tensor *out, void *stream) {
  int st = require_device();
  if (st) return st;
  if ((st = check_tensor(a, "ew_binary: a"))) return st;
  if ((st = check_tensor(b, "ew_binary: b"))) return st;
  if ((st = check_tensor(out, "ew_binary: out"))) return st;
  EB_REQUIRE(op >= 0 && op < ENDIA_B200_BIN_COUNT, ENDIA_B200_EINVAL, "ew_binary: unknown op %d", op);
  EB_REQUIRE(a->ndim == out->ndim && b->ndim == out->ndim, ENDIA_B200_ESHAPE,
             "ew_binary: operands must be expanded to the result rank (%d, %d vs %d)", a->ndim,
             b->ndim, out->ndim);
  for (int d = 0; d < out->ndim; ++d)
    EB_REQUIRE(a->shape[d] == out->shape[d] && b->shape[d] == out->shape[d], ENDIA_B200_ESHAPE,
               "ew_binary: operands must be expanded to the result shape (dim %d)", d);
  EB_REQUIRE(is_contiguous(out), ENDIA_B200_EINVAL, "ew_binary: out must be contiguous");
  const bool ac = a->is_complex != 0, bc = b->is_complex != 0;
  const bool out_c = out->is_complex != 0;
  EB_REQUIRE(out_c == (ac || bc || op == ENDIA_B200_BIN_COMPLEX), ENDIA_B200_EINVAL,
             "ew_binary: out must be complex exactly when an operand is");
  EwParams p{};
  bool ok;
  collapse(out, a, b, p, ok);
  EB_REQUIRE(ok, ENDIA_B200_EINVAL, "ew_binary: more than %d non-mergeable dims", EW_MAX_DIMS);
  p.a = static_cast<const float *>(a->data) + (ac ? 2 : 1) * a->offset;
  p.b = static_cast<const float *>(b->data) + (bc ? 2 : 1) * b->offset;
  p.out = static_cast<float *>(out->data) + (out_c ? 2 : 1) * out->offset;
  cudaStream_t s = as_stream(stream);
  switch (op) {
#define EB_CASE(OPC) case OPC: return dispatch_binary<OPC>(p, ac, bc, s);
    EB_CASE(ENDIA_B200_BIN_ADD) EB_CASE(ENDIA_B200_BIN_SUB) EB_CASE(ENDIA_B200_BIN_MUL)
    EB_CASE(ENDIA_B200_BIN_DIV) EB_CASE(ENDIA_B200_BIN_POW) EB_CASE(ENDIA_B200_BIN_GREATER)
    EB_CASE(ENDIA_B200_BIN_RELU_BWD) EB_CASE(ENDIA_B200_BIN_TANH_BWD)
    EB_CASE(ENDIA_B200_BIN_SIGMOID_BWD) EB_CASE(ENDIA_B200_BIN_COMPLEX)
    EB_CASE(ENDIA_B200_BIN_ABS_BWD) EB_CASE(ENDIA_B200_BIN_SQUARE_BWD)
    EB_CASE(ENDIA_B200_BIN_GREATER_EQUAL) EB_CASE(ENDIA_B200_BIN_LESS) EB_CASE(ENDIA_B200_BIN_LESS_EQUAL)
    EB_CASE(ENDIA_B200_BIN_EQUAL) EB_CASE(ENDIA_B200_BIN_NOT_EQUAL)
    EB_CASE(ENDIA_B200_BIN_TANH_OUT_BWD) EB_CASE(ENDIA_B200_BIN_TANH_OUT_BWD2)
#undef EB_CASE
  }
  return ENDIA_B200_EINVAL;
}

int endia_b200_fill(float *dst, int64_t n_elements, int is_complex, float re, float im,
                    void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n_elements >= 0, ENDIA_B200_EINVAL, "fill: negative size");
  if (n_elements == 0) return ENDIA_B200_OK;
  EB_REQUIRE(dst != nullptr, ENDIA_B200_EINVAL, "fill: dst is NULL");
  int64_t nf = n_elements * (is_complex ? 2 : 1);
  fill_kernel<<<grid_for(nf, 256), 256, 0, as_stream(stream)>>>(dst, nf, re, im, is_complex);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

int endia_b200_eye(float *dst, int64_t n, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(n >= 0, ENDIA_B200_EINVAL, "eye: negative size");
  if (n == 0) return ENDIA_B200_OK;
  EB_REQUIRE(dst != nullptr, ENDIA_B200_EINVAL, "eye: dst is NULL");
  eye_kernel<<<grid_for(n * n, 256), 256, 0, as_stream(stream)>>>(dst, n);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

}  // extern "C"
