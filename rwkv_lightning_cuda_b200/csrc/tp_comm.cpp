// NCCL bound at run time through dlopen; see tp_comm.h.
#include "tp_comm.h"

#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace rk {
namespace {

// Mirrors of the public NCCL C API (nccl.h): opaque communicator, 128-byte id, enum values.
struct NcclId {
  char bytes[kTpUniqueIdBytes];
};
constexpr int kNcclSuccess = 0;
constexpr int kNcclFloat32 = 7;  // ncclFloat32
constexpr int kNcclSum = 0;      // ncclSum

struct Api {
  int (*get_unique_id)(NcclId*) = nullptr;
  int (*comm_init_rank)(void**, int, NcclId, int) = nullptr;
  int (*comm_destroy)(void*) = nullptr;
  int (*all_reduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*all_gather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  const char* (*error_string)(int) = nullptr;
  bool ok = false;
};

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = nullptr;
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (h) break;
    }
    if (!h) return;
    a.get_unique_id = reinterpret_cast<decltype(a.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
    a.comm_init_rank = reinterpret_cast<decltype(a.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
    a.comm_destroy = reinterpret_cast<decltype(a.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
    a.all_reduce = reinterpret_cast<decltype(a.all_reduce)>(dlsym(h, "ncclAllReduce"));
    a.all_gather = reinterpret_cast<decltype(a.all_gather)>(dlsym(h, "ncclAllGather"));
    a.error_string = reinterpret_cast<decltype(a.error_string)>(dlsym(h, "ncclGetErrorString"));
    a.ok = a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.all_reduce && a.all_gather && a.error_string;
  });
  return a;
}

int nccl_status(int rc, const char* what) {
  if (rc == kNcclSuccess) return kOk;
  set_error("%s: NCCL error %d (%s)", what, rc, api().error_string ? api().error_string(rc) : "?");
  return kNccl;
}

int need_api() {
  RK_REQUIRE(api().ok, kNccl, "tensor parallelism needs libnccl.so.2, which could not be loaded");
  return kOk;
}

}  // namespace

TpComm::~TpComm() {
  if (comm_ && api().ok) api().comm_destroy(comm_);
}

int TpComm::make_unique_id(void* out128) {
  RK_REQUIRE(out128, kBadArg, "tp_unique_id: null buffer");
  if (int s = need_api()) return s;
  NcclId id;
  if (int s = nccl_status(api().get_unique_id(&id), "ncclGetUniqueId")) return s;
  memcpy(out128, id.bytes, kTpUniqueIdBytes);
  return kOk;
}

int TpComm::init(const void* unique_id, int rank, int size) {
  RK_REQUIRE(unique_id && size > 1 && rank >= 0 && rank < size, kBadArg, "tp_init: bad rank/size or null id");
  RK_REQUIRE(!comm_, kBadArg, "tp_init: the communicator exists already");
  if (int s = need_api()) return s;
  NcclId id;
  memcpy(id.bytes, unique_id, kTpUniqueIdBytes);
  if (int s = nccl_status(api().comm_init_rank(&comm_, size, id, rank), "ncclCommInitRank")) {
    comm_ = nullptr;
    return s;
  }
  size_ = size;
  return kOk;
}

int TpComm::all_reduce_sum(float* buf, size_t count, cudaStream_t stream) {
  RK_REQUIRE(comm_, kNotReady, "tensor-parallel model used before rwkv7_b200_model_tp_init");
  return nccl_status(api().all_reduce(buf, buf, count, kNcclFloat32, kNcclSum, comm_, stream), "ncclAllReduce");
}

int TpComm::all_gather(const float* send, float* recv, size_t count, cudaStream_t stream) {
  RK_REQUIRE(comm_, kNotReady, "tensor-parallel model used before rwkv7_b200_model_tp_init");
  return nccl_status(api().all_gather(send, recv, count, kNcclFloat32, comm_, stream), "ncclAllGather");
}

}  // namespace rk
