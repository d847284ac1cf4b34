// All-reduce (sum, fp32) of one buffer per rank through peer-mapped memory, for the ranks of one node.
// See TpComm in tp_comm.h for the protocol.  No counterpart in the reference, which drives one GPU.
//
// One kernel per call and rank:
//   1. this rank's partial sums were written by the kernel before this one; a system-scope fence, then the call's
//      epoch number is stored into slot [rank] of every peer's flag array;
//   2. every CTA waits until all slots of the LOCAL flag array have reached the epoch (bounded: on a time-out the
//      failure word gets its bit and the sums are left incomplete -- nothing hangs);
//   3. out[i] = partial_0[i] + partial_1[i] + ... in rank order, the peers' values read over NVLink with plain
//      16-byte loads (the same order on every rank, so all ranks hold bit-identical sums);
//   4. the last CTA to finish advances the epoch counter (a device-side counter: the kernel replays from CUDA graphs).
#include <algorithm>

#include "kernels.h"
#include "tp_comm.h"

namespace rk {
namespace {

constexpr uint32_t kPeerPolls = 1u << 22;

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(256) peer_reduce_kernel(const PeerReduceArgs a) {
  __shared__ unsigned s_epoch;
  __shared__ int s_ok;
  pdl_wait();  // the partial sums of this rank are complete
  pdl_trigger();
  unsigned* flags = a.ctrl;        // [8]
  unsigned* epoch_ctr = a.ctrl + 8;
  unsigned* done_ctr = a.ctrl + 9;
  if (threadIdx.x == 0) {
    const unsigned e = *reinterpret_cast<volatile unsigned*>(epoch_ctr) + 1;  // this call's number (1, 2, ...)
    s_epoch = e;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int p = 0; p < a.size; ++p) st_release_sys(a.peer_flags[p] + a.rank, e);
    }
    int ok = 1;
    for (int p = 0; p < a.size && ok; ++p) {
      uint32_t n = 0;
      while (static_cast<int>(ld_acquire_sys(flags + p) - e) < 0) {
        if (++n > kPeerPolls) { ok = 0; break; }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const size_t n4 = a.count >> 2;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
      float4 acc = reinterpret_cast<const float4*>(a.partial[0])[i];
      for (int p = 1; p < a.size; ++p) {
        const float4 t = reinterpret_cast<const float4*>(a.partial[p])[i];
        acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
      }
      reinterpret_cast<float4*>(a.out)[i] = acc;
    }
  } else if (threadIdx.x == 0 && a.timeout) {
    atomicOr(a.timeout, kTimeoutPeer);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_ctr, 1u) == gridDim.x - 1) {  // every CTA of this call has read the epoch: move on
      *done_ctr = 0;
      *reinterpret_cast<volatile unsigned*>(epoch_ctr) = s_epoch;
      __threadfence();
    }
  }
}

}  // namespace

int peer_reduce_launch(cudaStream_t stream, const PeerReduceArgs& a) {
  RK_REQUIRE(a.size >= 2 && a.size <= kTpMaxRanks && a.count % 4 == 0, kBadArg, "peer all-reduce: 2..8 ranks, count %% 4 == 0");
  const size_t n4 = a.count / 4;
  const int grid = static_cast<int>(std::min<size_t>(148, (n4 + 255) / 256));
  RK_CUDA(launch_pdl(peer_reduce_kernel, dim3(grid > 0 ? grid : 1), dim3(256), 0, stream, a));
  RK_LAUNCH_CHECK("peer all-reduce launch");
  return kOk;
}

}  // namespace rk
