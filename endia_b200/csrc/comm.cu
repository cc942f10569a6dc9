// Collectives of the C ABI: a thin layer over NCCL for callers that do not run inside a
// torch.distributed process group (the reference has no communication layer at all; a Mojo host
// would bind these). libnccl.so.2 is opened at first use, so the library loads and every other
// entry point works on machines without NCCL; inside a process that already holds NCCL (torch)
// the same copy is reused.
#include "common.cuh"
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

namespace eb {

struct NcclApi {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

static NcclApi &nccl() {
  static NcclApi api = []() {
    NcclApi a;
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) return a;
#define EB_SYM(field, name)                                                       \
  a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.handle, name));           \
  if (!a.field) return a
    EB_SYM(GetUniqueId, "ncclGetUniqueId");
    EB_SYM(CommInitRank, "ncclCommInitRank");
    EB_SYM(CommDestroy, "ncclCommDestroy");
    EB_SYM(AllReduce, "ncclAllReduce");
    EB_SYM(Send, "ncclSend");
    EB_SYM(Recv, "ncclRecv");
    EB_SYM(GroupStart, "ncclGroupStart");
    EB_SYM(GroupEnd, "ncclGroupEnd");
    EB_SYM(GetErrorString, "ncclGetErrorString");
#undef EB_SYM
    a.ok = true;
    return a;
  }();
  return api;
}

static int require_nccl() {
  if (!nccl().ok) {
    set_error("collectives need libnccl.so.2, which could not be opened: %s", dlerror() ? dlerror() : "symbol missing");
    return ENDIA_B200_ENODEV;
  }
  return ENDIA_B200_OK;
}

#define EB_NCCL(call)                                                                     \
  do {                                                                                    \
    ncclResult_t _r = (call);                                                             \
    if (_r != ncclSuccess) {                                                              \
      eb::set_error("%s failed: %s", #call, eb::nccl().GetErrorString(_r));               \
      return ENDIA_B200_ECUDA;                                                            \
    }                                                                                     \
  } while (0)

struct Comm {
  ncclComm_t comm;
  int rank, nranks;
};

}  // namespace eb

using namespace eb;

extern "C" int endia_b200_comm_unique_id(void *id128) {
  int st = require_nccl();
  if (st) return st;
  EB_REQUIRE(id128, ENDIA_B200_EINVAL, "comm_unique_id: NULL buffer");
  static_assert(sizeof(ncclUniqueId) == ENDIA_B200_COMM_ID_BYTES, "id size");
  ncclUniqueId id;
  EB_NCCL(nccl().GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_comm_init(int32_t rank, int32_t nranks, const void *id128, void **comm_out) {
  int st = require_device();
  if (st) return st;
  if ((st = require_nccl())) return st;
  EB_REQUIRE(id128 && comm_out, ENDIA_B200_EINVAL, "comm_init: NULL pointer");
  EB_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, ENDIA_B200_EINVAL,
             "comm_init: rank %d outside [0, %d)", (int)rank, (int)nranks);
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  Comm *c = new Comm{nullptr, rank, nranks};
  ncclResult_t r = nccl().CommInitRank(&c->comm, nranks, id, rank);
  if (r != ncclSuccess) {
    set_error("ncclCommInitRank failed: %s", nccl().GetErrorString(r));
    delete c;
    return ENDIA_B200_ECUDA;
  }
  *comm_out = c;
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_comm_destroy(void *comm) {
  if (!comm) return ENDIA_B200_OK;
  int st = require_nccl();
  if (st) return st;
  Comm *c = static_cast<Comm *>(comm);
  ncclResult_t r = nccl().CommDestroy(c->comm);
  delete c;
  if (r != ncclSuccess) {
    set_error("ncclCommDestroy failed: %s", nccl().GetErrorString(r));
    return ENDIA_B200_ECUDA;
  }
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_allreduce_sum_f32(void *comm, const float *send, float *recv, int64_t count,
                                            void *stream) {
  int st = require_nccl();
  if (st) return st;
  EB_REQUIRE(comm, ENDIA_B200_EINVAL, "allreduce_sum_f32: NULL communicator");
  EB_REQUIRE(count >= 0, ENDIA_B200_EINVAL, "allreduce_sum_f32: negative count");
  if (count == 0) return ENDIA_B200_OK;
  EB_REQUIRE(send && recv, ENDIA_B200_EINVAL, "allreduce_sum_f32: NULL buffer");
  Comm *c = static_cast<Comm *>(comm);
  EB_NCCL(nccl().AllReduce(send, recv, (size_t)count, ncclFloat32, ncclSum, c->comm, as_stream(stream)));
  return ENDIA_B200_OK;
}

extern "C" int endia_b200_alltoall_bytes(void *comm, const void *send, void *recv, int64_t bytes_per_peer,
                                         void *stream) {
  int st = require_nccl();
  if (st) return st;
  EB_REQUIRE(comm, ENDIA_B200_EINVAL, "alltoall_bytes: NULL communicator");
  EB_REQUIRE(bytes_per_peer >= 0, ENDIA_B200_EINVAL, "alltoall_bytes: negative size");
  if (bytes_per_peer == 0) return ENDIA_B200_OK;
  EB_REQUIRE(send && recv && send != recv, ENDIA_B200_EINVAL,
             "alltoall_bytes: NULL buffer or send == recv (in-place exchange is not supported)");
  Comm *c = static_cast<Comm *>(comm);
  const char *s = static_cast<const char *>(send);
  char *r = static_cast<char *>(recv);
  EB_NCCL(nccl().GroupStart());
  for (int peer = 0; peer < c->nranks; ++peer) {
    ncclResult_t a = nccl().Send(s + (size_t)peer * bytes_per_peer, (size_t)bytes_per_peer, ncclInt8, peer, c->comm,
                                 as_stream(stream));
    ncclResult_t b = a == ncclSuccess ? nccl().Recv(r + (size_t)peer * bytes_per_peer, (size_t)bytes_per_peer,
                                                    ncclInt8, peer, c->comm, as_stream(stream))
                                      : a;
    if (b != ncclSuccess) {
      nccl().GroupEnd();
      set_error("alltoall_bytes: send/recv with rank %d failed: %s", peer, nccl().GetErrorString(b));
      return ENDIA_B200_ECUDA;
    }
  }
  EB_NCCL(nccl().GroupEnd());
  return ENDIA_B200_OK;
}
