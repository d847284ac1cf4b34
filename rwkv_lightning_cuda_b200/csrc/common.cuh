// Shared device/host helpers for the sm_100a RWKV-7 forward kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rk {

constexpr int kHead = 64;  // head size; the model family fixes it

// Status codes returned through the C ABI.
enum Status : int {
  kOk = 0,
  kBadArg = 1,
  kShape = 2,
  kPrecision = 3,
  kCuda = 4,
  kNccl = 5,
  kTimeout = 6,
  kNotReady = 7,
};

void set_error(const char* fmt, ...);
int cuda_status(cudaError_t err, const char* what);
long long& launch_counter();  // thread-local count of kernels enqueued by this library

#define RK_CUDA(expr)                                   \
  do {                                                  \
    int _s = ::rk::cuda_status((expr), #expr);          \
    if (_s != ::rk::kOk) return _s;                     \
  } while (0)

#define RK_LAUNCH_CHECK(what)                           \
  do {                                                  \
    int _s = ::rk::cuda_status(cudaGetLastError(), what); \
    if (_s != ::rk::kOk) return _s;                     \
    ++::rk::launch_counter();                           \
  } while (0)

#define RK_REQUIRE(cond, code, ...)                     \
  do {                                                  \
    if (!(cond)) {                                      \
      ::rk::set_error(__VA_ARGS__);                     \
      return (code);                                    \
    }                                                   \
  } while (0)

// Input activation applied to x before a linear layer, and epilogues applied to the
// fp32 accumulator.  The numeric codes are part of the C ABI.
enum InAct : int { kActNone = 0, kActTanh = 1, kActSigmoid = 2 };
enum Epilogue : int {
  kEpiNone = 0,    // y = half(acc)
  kEpiRelu2 = 1,   // h = half(acc); y = half(relu(h)^2)
  kEpiVres = 2,    // y = half(v + (v_first - v) * sigmoid(v0 + acc))
  kEpiF32 = 3,     // y32 = float(half(acc))   (logits)
  kEpiRawF32 = 4,  // y32 = acc, not rounded: a partial sum another rank's partial is added to
  // internal to the library (tensor-core path only): LoRA activations of the many-row path
  kEpiTanhH = 100,     // h = half(acc); y = half(tanh(h))
  kEpiSigmoidH = 101,  // h = half(acc); y = half(sigmoid(h))
};

struct EpiArgs {
  const half* v = nullptr;        // kEpiVres
  const half* v_first = nullptr;  // kEpiVres
  const half* v0 = nullptr;       // kEpiVres, per output channel
};

#ifdef __CUDACC__

// Launch with programmatic stream serialization: the kernel may be scheduled while its
// predecessor in the stream is still running; it must call pdl_wait() before it reads anything
// the predecessor wrote (every CTA calls it, so completion stays transitive along the stream).
// Works the same in eager streams and under stream capture (the edge becomes a programmatic
// graph dependency).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Sum over a CTA of kThreads threads; every thread receives the total.
template <int kThreads>
__device__ __forceinline__ float block_sum(float x, float* scratch /* >= kThreads/32 floats */) {
  x = warp_sum(x);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) t += scratch[w];
  return t;
}

__device__ __forceinline__ float sigmoid_fast(float x) { return 1.0f / (1.0f + __expf(-x)); }

__device__ __forceinline__ float apply_in_act(float x, int act) {
  if (act == kActTanh) return tanhf(x);
  if (act == kActSigmoid) return 1.0f / (1.0f + expf(-x));
  return x;
}

// 16-byte global load that bypasses L1 allocation: weights are streamed exactly once.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// Programmatic dependent launch: a kernel may start while its predecessor drains.
// wait() blocks until the predecessor has completed and its memory is visible; trigger() lets the
// successor be scheduled.  Kernels here call trigger() only after wait(): then the successor cannot
// start before the predecessor's predecessor has completed, so what a kernel reads before its own
// wait() may be anything except the output of its immediate predecessor.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

// ---- mbarrier + bulk-copy (TMA engine) primitives
constexpr uint32_t kSpinLimit = 1u << 24;
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kSpinLimit polls instead of hanging the GPU; callers record the
// failure in a device flag and return.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ float2 h2f2(uint32_t u) {
  return __half22float2(*reinterpret_cast<const __half2*>(&u));
}

#endif  // __CUDACC__

}  // namespace rk
