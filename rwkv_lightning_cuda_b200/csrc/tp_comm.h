// Tensor-parallel communicator: a thin wrapper over NCCL, bound at run time.
//
// The library does not link NCCL.  When a model is created with tp_size > 1 the NCCL shared object that the
// process already holds (the one torch.distributed loaded, else the system one) is opened with dlopen and the
// handful of entry points used here are looked up by name.  Only NCCL's public C API is used.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

namespace rk {

constexpr int kTpUniqueIdBytes = 128;  // sizeof(ncclUniqueId)

class TpComm {
 public:
  TpComm() = default;
  ~TpComm();
  TpComm(const TpComm&) = delete;
  TpComm& operator=(const TpComm&) = delete;

  // Fills 128 bytes that rank 0 hands to every other rank (over any host channel) before init().
  static int make_unique_id(void* out128);
  // Collective: every rank of the group calls it with the same id.  The current device is the rank's GPU.
  int init(const void* unique_id, int rank, int size);
  bool ready() const { return comm_ != nullptr; }
  int size() const { return size_; }

  int all_reduce_sum(float* buf, size_t count, cudaStream_t stream);                 // in place
  int all_gather(const float* send, float* recv, size_t count, cudaStream_t stream);  // recv: [size][count]

 private:
  void* comm_ = nullptr;
  int size_ = 1;
};

}  // namespace rk
