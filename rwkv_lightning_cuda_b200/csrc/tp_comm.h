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

  // ---- all-reduce through peer memory (tp_allreduce.cu): every rank keeps two buffers of partial sums in a region the
  // other ranks of the node have mapped (CUDA IPC); one kernel publishes this rank's partial (a flag in every peer's
  // region), waits -- bounded -- for the peers' flags and adds all partials in rank order, reading the peers' over
  // NVLink.  For the 2 MiB sums of a tensor-parallel prefill chunk this takes a few microseconds where an NCCL call
  // costs tens.  Consecutive calls must alternate the buffer (0, 1, 0, ...): a rank may run one call ahead of its
  // peers, never two.
  // Collective (all ranks, same count, no stream capture in progress): makes room for `count` floats per buffer and
  // exchanges the mappings.  Leaves peer_ready() false when the GPUs cannot map each other's memory.
  int ensure_peer(size_t count);
  bool peer_ready() const { return peer_count_ > 0; }
  float* peer_partial(int buf) const { return local_partial_[buf & 1]; }  // where the producer writes this rank's partial
  int all_reduce_peer(int buf, size_t count, float* out, int* timeout_word, cudaStream_t stream);

 private:
  void release_peer();
  void* comm_ = nullptr;
  int size_ = 1, rank_ = 0;
  bool peer_failed_ = false;
  size_t peer_count_ = 0;            // floats per partial buffer; 0: not set up
  void* region_ = nullptr;           // this rank's region: [control 512 B][partial 0][partial 1]
  void* peer_region_[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  float* local_partial_[2] = {nullptr, nullptr};
};

// tp_allreduce.cu
constexpr int kTpMaxRanks = 8;
struct PeerReduceArgs {
  int rank, size;
  unsigned* ctrl;                        // this rank's control block: flags[8], epoch, done counter
  unsigned* peer_flags[kTpMaxRanks];     // every rank's flags array (entry [rank] is ours there)
  const float* partial[kTpMaxRanks];     // every rank's partial buffer of this call (ours included)
  float* out;
  size_t count;                          // floats, a multiple of 4
  int* timeout;
};
int peer_reduce_launch(cudaStream_t stream, const PeerReduceArgs& a);

}  // namespace rk
