// NCCL bound at run time through dlopen; see tp_comm.h.
#include "tp_comm.h"

#include <dlfcn.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <thread>

#include "common.cuh"
#include "kernels.h"

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
  release_peer();
  if (comm_ && api().ok) api().comm_destroy(comm_);
}

// Before this rank's region goes away, every rank must be done reading it, and this rank must be done reading theirs.
// The ranks tell each other through the "closed" marks of the control blocks, from the host: own device idle first,
// then a mark in every peer's block, then a wait (at most two seconds: a peer that has died never answers) for all
// peers' marks here.  Ranks therefore have to drop (or grow) their tensor-parallel models at the same point of the
// program, like every other collective.
void TpComm::release_peer() {
  if (peer_count_ > 0 && region_) {
    cudaDeviceSynchronize();
    const unsigned one = 1;
    for (int p = 0; p < size_; ++p)
      if (peer_region_[p]) cudaMemcpy(static_cast<unsigned*>(peer_region_[p]) + 16 + rank_, &one, sizeof(one), cudaMemcpyHostToDevice);
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      unsigned marks[kTpMaxRanks] = {};
      if (cudaMemcpy(marks, static_cast<unsigned*>(region_) + 16, sizeof(marks), cudaMemcpyDeviceToHost) != cudaSuccess) break;
      bool all = true;
      for (int p = 0; p < size_; ++p) all = all && marks[p] == 1;
      if (all || std::chrono::steady_clock::now() - t0 > std::chrono::seconds(2)) break;
      std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    cudaGetLastError();
  }
  for (int p = 0; p < kTpMaxRanks; ++p) {
    if (peer_region_[p] && p != rank_) cudaIpcCloseMemHandle(peer_region_[p]);
    peer_region_[p] = nullptr;
  }
  if (region_) cudaFree(region_);
  region_ = nullptr;
  local_partial_[0] = local_partial_[1] = nullptr;
  peer_count_ = 0;
}

namespace {
constexpr size_t kCtrlBytes = 512;
}

int TpComm::ensure_peer(size_t count) {
  RK_REQUIRE(comm_, kNotReady, "tensor-parallel model used before rwkv7_b200_model_tp_init");
  // One-shot all-reduce: every rank reads every other rank's plane, (G - 1) x the message over NVLink per rank.  At
  // two ranks that is the minimum and beats NCCL (7.2B prefill chunk 5.81 -> 5.46 ms); at eight it moves four times
  // what a reduce-scatter + all-gather moves and loses (6.75 against 5.32 ms), so from `tp_peer_ranks` + 1 ranks on the
  // all-reduce stays with NCCL.
  if (peer_failed_ || size_ > kTpMaxRanks || size_ > options().tp_peer_ranks) return kOk;
  count = (count + 3) & ~static_cast<size_t>(3);
  if (count <= peer_count_) return kOk;
  // (every rank gets here with the same count: they all run the same calls)
  RK_CUDA(cudaDeviceSynchronize());
  release_peer();
  const size_t bytes = kCtrlBytes + 2 * count * sizeof(float);
  auto give_up = [&]() {  // the NCCL path stays in use; the ranks decide alike because they see each other's handles
    cudaGetLastError();
    release_peer();
    peer_failed_ = true;
    return kOk;
  };
  // (no early return before the exchange below: it is a collective, every rank has to take part)
  cudaIpcMemHandle_t mine;
  memset(&mine, 0, sizeof(mine));
  bool have = cudaMalloc(&region_, bytes) == cudaSuccess;
  if (!have) region_ = nullptr;
  have = have && cudaMemset(region_, 0, kCtrlBytes) == cudaSuccess && cudaIpcGetMemHandle(&mine, region_) == cudaSuccess;
  if (!have) cudaGetLastError();
  // exchange the handles (and whether each rank has one) with an all-gather of 64 + 4 bytes, padded to 80
  constexpr size_t kSlot = 80;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
  char host[kTpMaxRanks * kSlot] = {};
  memcpy(host + rank_ * kSlot, &mine, 64);
  host[rank_ * kSlot + 64] = have ? 1 : 0;
  void* dev = nullptr;
  RK_CUDA(cudaMalloc(&dev, kTpMaxRanks * kSlot));
  RK_CUDA(cudaMemcpy(dev, host, kTpMaxRanks * kSlot, cudaMemcpyHostToDevice));
  int s = nccl_status(api().all_gather(static_cast<char*>(dev) + rank_ * kSlot, dev, kSlot / sizeof(float), kNcclFloat32, comm_, nullptr),
                      "ncclAllGather (peer handles)");
  if (s == kOk) s = cuda_status(cudaDeviceSynchronize(), "sync after the handle exchange");
  if (s == kOk) s = cuda_status(cudaMemcpy(host, dev, kTpMaxRanks * kSlot, cudaMemcpyDeviceToHost), "copy peer handles");
  cudaFree(dev);
  if (s != kOk) return s;
  bool all = true;
  for (int p = 0; p < size_; ++p) all = all && host[p * kSlot + 64] == 1;
  if (!all) return give_up();
  for (int p = 0; p < size_; ++p) {
    if (p == rank_) { peer_region_[p] = region_; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, host + p * kSlot, 64);
    if (cudaIpcOpenMemHandle(&peer_region_[p], h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      peer_region_[p] = nullptr;
      // the other ranks may have succeeded: agree on the outcome below
      all = false;
    }
  }
  // agree: everyone must have every mapping, or nobody uses the path (one more tiny all-reduce through NCCL)
  float flag_host = all ? 0.f : 1.f, *flag_dev = nullptr;
  RK_CUDA(cudaMalloc(reinterpret_cast<void**>(&flag_dev), sizeof(float)));
  RK_CUDA(cudaMemcpy(flag_dev, &flag_host, sizeof(float), cudaMemcpyHostToDevice));
  s = nccl_status(api().all_reduce(flag_dev, flag_dev, 1, kNcclFloat32, kNcclSum, comm_, nullptr), "ncclAllReduce (peer agreement)");
  if (s == kOk) s = cuda_status(cudaDeviceSynchronize(), "sync after the peer agreement");
  if (s == kOk) s = cuda_status(cudaMemcpy(&flag_host, flag_dev, sizeof(float), cudaMemcpyDeviceToHost), "copy peer agreement");
  cudaFree(flag_dev);
  if (s != kOk) return s;
  if (flag_host != 0.f) return give_up();
  local_partial_[0] = reinterpret_cast<float*>(static_cast<char*>(region_) + kCtrlBytes);
  local_partial_[1] = local_partial_[0] + count;
  peer_count_ = count;
  return kOk;
}

int TpComm::all_reduce_peer(int buf, size_t count, float* out, int* timeout_word, cudaStream_t stream) {
  RK_REQUIRE(peer_count_ > 0 && count <= peer_count_ && count % 4 == 0, kBadArg, "peer all-reduce: not set up for %zu floats", count);
  PeerReduceArgs a = {};
  a.rank = rank_; a.size = size_;
  a.ctrl = static_cast<unsigned*>(region_);
  for (int p = 0; p < size_; ++p) {
    a.peer_flags[p] = static_cast<unsigned*>(peer_region_[p]);
    a.partial[p] = reinterpret_cast<const float*>(static_cast<const char*>(peer_region_[p]) + kCtrlBytes) + (buf & 1) * peer_count_;
  }
  a.out = out; a.count = count; a.timeout = timeout_word;
  return peer_reduce_launch(stream, a);
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
  rank_ = rank;
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
