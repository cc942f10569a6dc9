// Runtime part of the C ABI: device selection, stream-ordered memory, streams and events.
// The reference keeps every Array in host memory (endia/_array/_array.mojo:125-131); these
// entry points are what a device-resident Node needs instead.
#include "common.cuh"
#include <mutex>
#include <unordered_map>
#include <string.h>
#include <atomic>

namespace eb {

static thread_local char g_err[512] = "";
static int g_sm_count = 0;
static int g_device = -1;
static bool g_ready = false;
static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
uint64_t launches() { return g_launches.load(std::memory_order_relaxed); }

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int sm_count() { return g_sm_count; }
bool device_ready() { return g_ready; }

int require_device() {
  if (g_ready) return ENDIA_B200_OK;
  // Lazy init on the current device keeps the entry points usable for callers that have
  // already chosen a device through another runtime in the same process.
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    set_error("no CUDA device is available; this library has no CPU fallback");
    return ENDIA_B200_ENODEV;
  }
  return endia_b200_init(dev);
}

int check_tensor(const endia_b200_tensor *t, const char *what) {
  EB_REQUIRE(t != nullptr, ENDIA_B200_EINVAL, "%s: descriptor is NULL", what);
  EB_REQUIRE(t->ndim >= 0 && t->ndim <= ENDIA_B200_MAX_DIMS, ENDIA_B200_EINVAL,
             "%s: ndim %d outside [0, %d]", what, t->ndim, ENDIA_B200_MAX_DIMS);
  for (int d = 0; d < t->ndim; ++d) {
    EB_REQUIRE(t->shape[d] >= 0, ENDIA_B200_EINVAL, "%s: negative extent in dim %d", what, d);
    EB_REQUIRE(t->stride[d] >= 0, ENDIA_B200_EINVAL, "%s: negative stride in dim %d", what, d);
  }
  EB_REQUIRE(t->offset >= 0, ENDIA_B200_EINVAL, "%s: negative storage offset", what);
  EB_REQUIRE(t->data != nullptr || numel(t) == 0, ENDIA_B200_EINVAL, "%s: data pointer is NULL",
             what);
  return ENDIA_B200_OK;
}

}  // namespace eb

using namespace eb;

extern "C" {

int endia_b200_init(int device) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    set_error("no CUDA device is available (%s); this library has no CPU fallback",
              e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    return ENDIA_B200_ENODEV;
  }
  EB_REQUIRE(device >= 0 && device < count, ENDIA_B200_EINVAL, "device %d outside [0, %d)", device,
             count);
  cudaDeviceProp prop;
  EB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    set_error("device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major,
              prop.minor);
    return ENDIA_B200_ENODEV;
  }
  EB_CUDA(cudaSetDevice(device));
  // Stream-ordered allocations (endia_b200_malloc, GEMM work buffers) come from the device's
  // default pool; keep freed blocks cached across synchronisation points instead of returning
  // them to the driver, which would make the next allocation cost milliseconds.
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
    uint64_t keep = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  cudaGetLastError();
  g_sm_count = prop.multiProcessorCount;
  g_device = device;
  g_ready = true;
  return ENDIA_B200_OK;
}

int endia_b200_shutdown(void) {
  g_ready = false;
  g_sm_count = 0;
  g_device = -1;
  return ENDIA_B200_OK;
}

const char *endia_b200_last_error(void) { return g_err; }
int endia_b200_version(void) { return 1000; }
uint64_t endia_b200_launch_count(void) { return eb::launches(); }

// Bytes handed out by endia_b200_malloc and not yet freed, and the optional quota on them.
static std::mutex g_alloc_mutex;
static std::unordered_map<void *, size_t> g_alloc_sizes;
static size_t g_alloc_live = 0, g_alloc_quota = 0;

int endia_b200_set_malloc_quota(size_t bytes) {
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  g_alloc_quota = bytes;
  return ENDIA_B200_OK;
}

int endia_b200_malloc(void **ptr, size_t bytes, void *stream) {
  EB_REQUIRE(ptr != nullptr, ENDIA_B200_EINVAL, "malloc: ptr is NULL");
  int st = require_device();
  if (st) return st;
  *ptr = nullptr;
  if (bytes == 0) return ENDIA_B200_OK;
  {
    std::lock_guard<std::mutex> lock(g_alloc_mutex);
    if (g_alloc_quota && g_alloc_live + bytes > g_alloc_quota) {
      set_error("device allocation of %zu bytes refused: %zu bytes are live and the quota is %zu", bytes,
                g_alloc_live, g_alloc_quota);
      return ENDIA_B200_ENOMEM;
    }
  }
  cudaError_t e = cudaMallocAsync(ptr, bytes, as_stream(stream));
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    set_error("device allocation of %zu bytes failed", bytes);
    return ENDIA_B200_ENOMEM;
  }
  EB_CUDA(e);
  std::lock_guard<std::mutex> lock(g_alloc_mutex);
  g_alloc_sizes[*ptr] = bytes;
  g_alloc_live += bytes;
  return ENDIA_B200_OK;
}
int endia_b200_free(void *ptr, void *stream) {
  if (!ptr) return ENDIA_B200_OK;
  {
    std::lock_guard<std::mutex> lock(g_alloc_mutex);
    auto it = g_alloc_sizes.find(ptr);
    if (it != g_alloc_sizes.end()) {
      g_alloc_live -= it->second;
      g_alloc_sizes.erase(it);
    }
  }
  EB_CUDA(cudaFreeAsync(ptr, as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_memset0(void *ptr, size_t bytes, void *stream) {
  if (bytes == 0) return ENDIA_B200_OK;
  EB_REQUIRE(ptr != nullptr, ENDIA_B200_EINVAL, "memset0: ptr is NULL");
  EB_CUDA(cudaMemsetAsync(ptr, 0, bytes, as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_h2d(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return ENDIA_B200_OK;
  EB_REQUIRE(dst && src, ENDIA_B200_EINVAL, "h2d: NULL pointer");
  EB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_d2h(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return ENDIA_B200_OK;
  EB_REQUIRE(dst && src, ENDIA_B200_EINVAL, "d2h: NULL pointer");
  EB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_d2d(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return ENDIA_B200_OK;
  EB_REQUIRE(dst && src, ENDIA_B200_EINVAL, "d2d: NULL pointer");
  EB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
  return ENDIA_B200_OK;
}

int endia_b200_stream_create(void **stream) {
  EB_REQUIRE(stream != nullptr, ENDIA_B200_EINVAL, "stream_create: NULL");
  int st = require_device();
  if (st) return st;
  cudaStream_t s;
  EB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *stream = s;
  return ENDIA_B200_OK;
}
int endia_b200_stream_destroy(void *stream) {
  if (stream) EB_CUDA(cudaStreamDestroy(as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_stream_sync(void *stream) {
  EB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_event_create(void **event) {
  EB_REQUIRE(event != nullptr, ENDIA_B200_EINVAL, "event_create: NULL");
  int st = require_device();
  if (st) return st;
  cudaEvent_t e;
  EB_CUDA(cudaEventCreate(&e));
  *event = e;
  return ENDIA_B200_OK;
}
int endia_b200_event_destroy(void *event) {
  if (event) EB_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
  return ENDIA_B200_OK;
}
int endia_b200_event_record(void *event, void *stream) {
  EB_REQUIRE(event != nullptr, ENDIA_B200_EINVAL, "event_record: NULL event");
  EB_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
  return ENDIA_B200_OK;
}
int endia_b200_stream_wait_event(void *stream, void *event) {
  EB_REQUIRE(event != nullptr, ENDIA_B200_EINVAL, "stream_wait_event: NULL event");
  EB_CUDA(cudaStreamWaitEvent(as_stream(stream), reinterpret_cast<cudaEvent_t>(event), 0));
  return ENDIA_B200_OK;
}
int endia_b200_event_elapsed_ms(void *start, void *stop, float *ms) {
  EB_REQUIRE(start && stop && ms, ENDIA_B200_EINVAL, "event_elapsed_ms: NULL argument");
  EB_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start),
                               reinterpret_cast<cudaEvent_t>(stop)));
  return ENDIA_B200_OK;
}

}  // extern "C"
