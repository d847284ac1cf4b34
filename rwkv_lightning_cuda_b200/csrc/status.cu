// Device-side failure word and the library's few run-time options.
//
// Every kernel of this library that waits on an mbarrier does so with a poll limit; when the limit runs out the
// kernel ORs its bit into one word in device memory and returns (it does not trap and does not hang).  The host
// reads that word where it synchronises anyway (forward_to_host, decode_greedy with a host buffer, the C++
// adapter) and reports RWKV7_B200_TIMEOUT; asynchronous callers use rwkv7_b200_timeout_flags().
#include <cstring>
#include <mutex>

#include "kernels.h"

namespace rk {
namespace {

// word 0: the failure bits; words 1..15: where the first tensor-core GEMM wait ran out (a diagnostic, see timeout_detail)
__device__ int g_timeout_word[16] = {0};

std::mutex g_mu;
int* g_word_ptr[64] = {nullptr};
Options g_options;

// Waits (bounded) on a barrier that nothing ever completes: the one way to see the time-out path work without
// losing a copy or stalling the GPU.  One thread, no memory traffic, no copy in flight when it gives up.
__global__ void wait_probe_kernel(int* word, unsigned polls) {
  __shared__ __align__(8) uint64_t bar;
  mbar_init(smem_u32(&bar), 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  bool done = false;
  for (unsigned i = 0; i < polls && !done; ++i) done = mbar_try_wait(smem_u32(&bar), 0);
  if (!done) atomicOr(word, kTimeoutProbe);
}

}  // namespace

int timeout_word(int** out) {
  int dev = 0;
  RK_CUDA(cudaGetDevice(&dev));
  RK_REQUIRE(dev >= 0 && dev < 64, kBadArg, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_word_ptr[dev]) {
    void* p = nullptr;
    RK_CUDA(cudaGetSymbolAddress(&p, g_timeout_word));  // the symbol's address on the current device
    g_word_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_word_ptr[dev];
  return kOk;
}

int* timeout_word_or_null() {
  int* p = nullptr;
  return timeout_word(&p) == kOk ? p : nullptr;
}

int timeout_read(int* flags, bool clear) {
  int* p = nullptr;
  int s = timeout_word(&p);
  if (s != kOk) return s;
  RK_CUDA(cudaMemcpy(flags, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (clear && *flags) RK_CUDA(cudaMemset(p, 0, sizeof(int)));
  return kOk;
}

// The record a GEMM kernel leaves with its first expired wait: {1, role (1 producer, 2 MMA, 3 dequantisation, 4
// epilogue), CTA, work unit, K-block counter, stages, total units, product index, M, N, K, format, row tile, splits, 0}.
int timeout_detail(int* out15, bool clear) {
  int* p = nullptr;
  int s = timeout_word(&p);
  if (s != kOk) return s;
  RK_CUDA(cudaMemcpy(out15, p + 1, 15 * sizeof(int), cudaMemcpyDeviceToHost));
  if (clear) RK_CUDA(cudaMemset(p + 1, 0, 15 * sizeof(int)));
  return kOk;
}

int timeout_status(int flags) {
  if (!flags) return kOk;
  set_error("a bounded wait inside a kernel ran out (flags 0x%x:%s%s%s%s); the results of that call are incomplete", flags,
            (flags & kTimeoutGemv) ? " weight-streaming GEMV" : "", (flags & kTimeoutGemm) ? " tensor-core GEMM" : "",
            (flags & kTimeoutTmix) ? " time-mix core" : "", (flags & (kTimeoutProbe | kTimeoutPeer)) ? " wait probe / peer all-reduce" : "");
  return kTimeout;
}

int wait_probe(cudaStream_t stream, unsigned polls) {
  int* p = nullptr;
  int s = timeout_word(&p);
  if (s != kOk) return s;
  RK_REQUIRE(polls <= (1u << 20), kBadArg, "wait_probe: at most 2^20 polls");
  wait_probe_kernel<<<1, 1, 0, stream>>>(p, polls);
  RK_LAUNCH_CHECK("wait_probe launch");
  return kOk;
}

Options& options() { return g_options; }

int set_option(const char* name, int value) {
  RK_REQUIRE(name, kBadArg, "set_option: null name");
  struct Slot { const char* name; int* v; int lo, hi; };
  Options& o = g_options;
  const Slot slots[] = {
      {"gemm_cta_pair", &o.gemm_cta_pair, 0, 1},
      {"quant_tc_rows", &o.quant_tc_rows, 0, 1 << 20},   {"fp16_tc_rows", &o.fp16_tc_rows, 0, 1 << 20},
      {"decode_graphs", &o.decode_graphs, 0, 1},         {"wkv_chunked", &o.wkv_chunked, 0, 1},
      {"gemv_mma", &o.gemv_mma, 0, 4},
      {"tp_peer_ranks", &o.tp_peer_ranks, 0, 64},
      {"gemv_mma_tall", &o.gemv_mma_tall, 0, 3},
  };
  for (const Slot& s : slots) {
    if (std::strcmp(name, s.name) != 0) continue;
    RK_REQUIRE(value >= s.lo && value <= s.hi, kBadArg, "set_option: %s must be in [%d, %d]", name, s.lo, s.hi);
    *s.v = value;
    return kOk;
  }
  set_error("set_option: unknown option '%s'", name);
  return kBadArg;
}

}  // namespace rk
