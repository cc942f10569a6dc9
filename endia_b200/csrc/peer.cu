// Device memory shared between the ranks of one machine (CUDA IPC) and a copy kernel whose source
// and destination may both be strided views, so that a rank can write its blocks of a slab
// transpose straight into the other ranks' memory over NVLink: the block packing, the exchange and
// the unpacking of the slab-decomposed fftn become one pass (the reference gathers per dimension
// on one host, endia/functional/fft_ops/fft_cooley_tukey.mojo:251-257). Plain loads and stores
// only; no bulk or multicast copy touches peer memory.
#include "common.cuh"
#include <string.h>
#include <cuda_bf16.h>

namespace eb {

constexpr int CP_MAX_DIMS = ENDIA_B200_MAX_DIMS;

struct CopyParams {
  const float *src;
  float *dst;
  int64_t outer[CP_MAX_DIMS];       // extents of the outer dims (innermost run excluded)
  int64_t sstride[CP_MAX_DIMS];     // in floats
  int64_t dstride[CP_MAX_DIMS];
  int n_outer;
  int64_t rows;                     // product of the outer extents
  int64_t run;                      // floats per contiguous run
};

template <int VEC>
__global__ void __launch_bounds__(256) copy_strided_kernel(const CopyParams p) {
  const int64_t per_row = p.run / VEC;
  const int64_t total = p.rows * per_row;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    int64_t row = i / per_row;
    const int64_t c = (i - row * per_row) * VEC;
    int64_t so = 0, dof = 0;
#pragma unroll 1
    for (int d = p.n_outer - 1; d >= 0; --d) {
      const int64_t q = row / p.outer[d], r = row - q * p.outer[d];
      so += r * p.sstride[d];
      dof += r * p.dstride[d];
      row = q;
    }
    if (VEC == 4) {
      *reinterpret_cast<float4 *>(p.dst + dof + c) = *reinterpret_cast<const float4 *>(p.src + so + c);
    } else {
      p.dst[dof + c] = p.src[so + c];
    }
  }
}

}  // namespace eb

using namespace eb;

extern "C" int endia_b200_copy_strided(const endia_b200_tensor *src, const endia_b200_tensor *dst, void *stream) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(src && dst && src->data && dst->data, ENDIA_B200_EINVAL, "copy_strided: NULL tensor");
  EB_REQUIRE(src->ndim == dst->ndim && src->ndim >= 1 && src->ndim <= CP_MAX_DIMS, ENDIA_B200_ESHAPE,
             "copy_strided: ranks %d and %d", src->ndim, dst->ndim);
  EB_REQUIRE((src->is_complex != 0) == (dst->is_complex != 0), ENDIA_B200_EINVAL,
             "copy_strided: complex flags differ");
  const int nd = src->ndim;
  const int64_t w = src->is_complex ? 2 : 1;
  int64_t total = 1;
  for (int d = 0; d < nd; ++d) {
    EB_REQUIRE(src->shape[d] == dst->shape[d] && src->shape[d] >= 0, ENDIA_B200_ESHAPE,
               "copy_strided: shape mismatch in dim %d", d);
    total *= src->shape[d];
  }
  if (total == 0) return ENDIA_B200_OK;
  EB_REQUIRE((src->stride[nd - 1] == 1 || src->shape[nd - 1] == 1) &&
                 (dst->stride[nd - 1] == 1 || dst->shape[nd - 1] == 1),
             ENDIA_B200_EINVAL, "copy_strided: the last dim must be contiguous on both sides");
  CopyParams p{};
  p.src = static_cast<const float *>(src->data) + w * src->offset;
  p.dst = static_cast<float *>(dst->data) + w * dst->offset;
  p.run = src->shape[nd - 1] * w;
  p.rows = 1;
  p.n_outer = 0;
  // merge outer dims that are contiguous with the run on both sides into the run
  int d = nd - 2;
  int64_t run_elems = src->shape[nd - 1];
  for (; d >= 0; --d) {
    if (src->shape[d] == 1) continue;
    if (src->stride[d] == run_elems && dst->stride[d] == run_elems) {
      run_elems *= src->shape[d];
      p.run = run_elems * w;
    } else {
      break;
    }
  }
  for (int k = 0; k <= d; ++k) {
    if (src->shape[k] == 1) continue;
    p.outer[p.n_outer] = src->shape[k];
    p.sstride[p.n_outer] = src->stride[k] * w;
    p.dstride[p.n_outer] = dst->stride[k] * w;
    p.rows *= src->shape[k];
    ++p.n_outer;
  }
  bool vec = p.run % 4 == 0 && (reinterpret_cast<uintptr_t>(p.src) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(p.dst) & 15) == 0;
  for (int k = 0; k < p.n_outer; ++k) vec = vec && p.sstride[k] % 4 == 0 && p.dstride[k] % 4 == 0;
  const int64_t work = p.rows * (vec ? p.run / 4 : p.run);
  int64_t blocks = ceil_div(work, 256);
  const int64_t cap = (int64_t)(sm_count() > 0 ? sm_count() : 148) * 16;
  if (blocks > cap) blocks = cap;
  if (vec) copy_strided_kernel<4><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(p);
  else copy_strided_kernel<1><<<(unsigned)blocks, 256, 0, as_stream(stream)>>>(p);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

// The receiving side of an all-gather done with peer copies: the other ranks' slices of a
// parameter have landed in `inbox` (laid out like the parameter); they are moved into the
// parameter, and the bf16 operand parts of the whole parameter are written in the same pass.
__global__ void __launch_bounds__(256)
gather_slices_kernel(float *__restrict__ w, const float *__restrict__ inbox, int64_t n4, int64_t slice4, int rank,
                     __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += step) {
    const bool own = i / slice4 == rank;
    float4 v;
    if (own) {
      v = reinterpret_cast<const float4 *>(w)[i];
    } else {
      v = __ldcs(reinterpret_cast<const float4 *>(inbox) + i);
      reinterpret_cast<float4 *>(w)[i] = v;
    }
    if (hi) {
      const float l0 = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
      const float l1 = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
      const float l2 = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
      const float l3 = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
      __nv_bfloat162 h01 = __floats2bfloat162_rn(v.x, v.y), h23 = __floats2bfloat162_rn(v.z, v.w);
      __nv_bfloat162 l01 = __floats2bfloat162_rn(l0, l1), l23 = __floats2bfloat162_rn(l2, l3);
      uint2 hv, lv;
      hv.x = *reinterpret_cast<uint32_t *>(&h01); hv.y = *reinterpret_cast<uint32_t *>(&h23);
      lv.x = *reinterpret_cast<uint32_t *>(&l01); lv.y = *reinterpret_cast<uint32_t *>(&l23);
      reinterpret_cast<uint2 *>(hi)[i] = hv;
      reinterpret_cast<uint2 *>(lo)[i] = lv;
    }
  }
}

extern "C" int endia_b200_gather_slices(float *w, const float *inbox, int64_t numel, int32_t rank, int32_t world,
                                        void *pair16, void *stream) {
  int st = eb::require_device();
  if (st) return st;
  EB_REQUIRE(w && inbox && numel > 0 && world >= 1 && rank >= 0 && rank < world, ENDIA_B200_EINVAL,
             "gather_slices: bad arguments");
  EB_REQUIRE(numel % ((int64_t)8 * world) == 0, ENDIA_B200_EINVAL,
             "gather_slices: numel must be a multiple of 8 * world");
  EB_REQUIRE(((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(inbox) |
               reinterpret_cast<uintptr_t>(pair16)) & 15) == 0, ENDIA_B200_EINVAL,
             "gather_slices: pointers must be 16-byte aligned");
  __nv_bfloat16 *hi = static_cast<__nv_bfloat16 *>(pair16);
  gather_slices_kernel<<<eb::grid_for(numel / 4, 256), 256, 0, eb::as_stream(stream)>>>(
      w, inbox, numel / 4, numel / world / 4, rank, hi, hi ? hi + numel : nullptr);
  EB_LAUNCH_CHECK();
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_ipc_alloc(size_t bytes, void **ptr, void *handle64) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(ptr && handle64 && bytes > 0, ENDIA_B200_EINVAL, "ipc_alloc: NULL argument or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == ENDIA_B200_IPC_HANDLE_BYTES, "handle size");
  *ptr = nullptr;
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    set_error("ipc_alloc: device allocation of %zu bytes failed", bytes);
    return ENDIA_B200_ENOMEM;
  }
  EB_CUDA(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
    set_error("ipc_alloc: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    cudaGetLastError();
    return ENDIA_B200_ECUDA;
  }
  memcpy(handle64, &h, sizeof(h));
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_ipc_open(const void *handle64, void **ptr) {
  int st = require_device();
  if (st) return st;
  EB_REQUIRE(ptr && handle64, ENDIA_B200_EINVAL, "ipc_open: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  EB_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_ipc_close(void *ptr) {
  if (!ptr) return ENDIA_B200_OK;
  EB_CUDA(cudaIpcCloseMemHandle(ptr));
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_ipc_free(void *ptr) {
  if (!ptr) return ENDIA_B200_OK;
  EB_CUDA(cudaFree(ptr));
  return ENDIA_B200_OK;
}
