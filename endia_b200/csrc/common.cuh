// Shared helpers of the device library: status/error plumbing and launch utilities.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "../../include/endia_b200.h"

namespace eb {

// Thread-local error text returned by endia_b200_last_error().
void set_error(const char *fmt, ...);
// Device properties captured by endia_b200_init (0 SMs before init).
int sm_count();
bool device_ready();
// Checks that init() succeeded; sets the error and returns a status otherwise.
int require_device();
// Every kernel launch of this library is counted (endia_b200_launch_count).
void count_launch();

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

#define EB_CUDA(call)                                                               \
  do {                                                                              \
    cudaError_t _e = (call);                                                        \
    if (_e != cudaSuccess) {                                                        \
      eb::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e), __FILE__, \
                    __LINE__);                                                      \
      return ENDIA_B200_ECUDA;                                                      \
    }                                                                               \
  } while (0)

#define EB_LAUNCH_CHECK()                                                           \
  do {                                                                              \
    eb::count_launch();                                                             \
    cudaError_t _e = cudaGetLastError();                                            \
    if (_e != cudaSuccess) {                                                        \
      eb::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e),     \
                    __FILE__, __LINE__);                                            \
      return ENDIA_B200_ECUDA;                                                      \
    }                                                                               \
  } while (0)

#define EB_REQUIRE(cond, code, ...)                                                 \
  do {                                                                              \
    if (!(cond)) {                                                                  \
      eb::set_error(__VA_ARGS__);                                                   \
      return (code);                                                                \
    }                                                                               \
  } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool is_pow2(int64_t n) { return n > 0 && (n & (n - 1)) == 0; }
inline int ilog2(int64_t n) {
  int l = 0;
  while ((int64_t(1) << l) < n) ++l;
  return l;
}

// Number of logical elements of a descriptor.
inline int64_t numel(const endia_b200_tensor *t) {
  int64_t n = 1;
  for (int d = 0; d < t->ndim; ++d) n *= t->shape[d];
  return n;
}
// True when strides are the row-major defaults of the shape (size-1 dims are ignored).
inline bool is_contiguous(const endia_b200_tensor *t) {
  int64_t expect = 1;
  for (int d = t->ndim - 1; d >= 0; --d) {
    if (t->shape[d] != 1 && t->stride[d] != expect) return false;
    expect *= t->shape[d];
  }
  return true;
}
int check_tensor(const endia_b200_tensor *t, const char *what);

// out[0] = scale * (sum of `count` floats at `partial`), one CTA, fixed summation order (reduce.cu).
int launch_scalar_finish(const float *partial, float *out, int count, float scale, cudaStream_t s);

// Grid size for a grid-stride kernel: enough CTAs to fill the machine a few times over.
inline int grid_for(int64_t work_items, int threads, int ctas_per_sm = 8) {
  int64_t want = ceil_div(work_items, threads);
  int64_t cap = (int64_t)sm_count() * ctas_per_sm;
  if (cap <= 0) cap = 148 * ctas_per_sm;
  if (want < 1) want = 1;
  return (int)(want < cap ? want : cap);
}

}  // namespace eb
