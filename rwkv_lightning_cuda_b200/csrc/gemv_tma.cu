// fp16 weight-streaming GEMV (M <= 4) with the weights staged through shared memory by the
// bulk-copy engine: every warp owns a ring of kSlots buffers, one lane requests the next piece of
// the warp's contiguous weight stream with cp.async.bulk (completion on an mbarrier), the warp
// consumes pieces in order with 128-bit shared-memory loads and re-arms the slot it has just read.
// About kSlots * 4 KiB per warp (96 KiB per CTA) are in flight without holding registers, which is
// what it takes to keep HBM3e busy from 148 SMs; the first kSlots pieces are requested before the
// programmatic-dependency wait, so a kernel's weight stream starts while its predecessor drains.
// Same arithmetic and rounding as the register-staged kernel in linear.cu.
#include <algorithm>

#include "gemv.h"
#include "kernels.h"

namespace rk {
namespace {

constexpr int kWarps = 8;
constexpr int kSlots = 3;
constexpr int kPieceCap = 4096;  // bytes
constexpr uint32_t kSpinLimit = 1u << 24;

__device__ int g_gemv_timeout = 0;  // set when a bounded mbarrier wait gives up

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
// Bounded wait: gives up after kSpinLimit polls instead of hanging the GPU.
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

template <int kM>
__global__ void __launch_bounds__(kWarps * 32) gemv_tma_kernel(const GemvBatch p, int x_bytes) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[kWarps][kSlots];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSeg; ++i)
    if (i < p.n_seg && static_cast<int>(blockIdx.x) >= p.seg[i].cta_begin) s = i;
  const GemvSeg& sg = p.seg[s];
  const int row0 = (blockIdx.x - sg.cta_begin) * sg.rows_per_cta;
  const int rows_end = min(sg.N, row0 + sg.rows_per_cta);
  const int rows_cta = max(rows_end - row0, 0);
  const int rpw = (rows_cta + kWarps - 1) / kWarps;
  const int r_begin = row0 + warp * rpw;
  const int r_end = min(rows_end, r_begin + rpw);
  const int parts = sg.parts, piece = sg.piece_bytes;
  const int total = r_end > r_begin ? (r_end - r_begin) * parts : 0;
  const size_t row_bytes = static_cast<size_t>(sg.K) * 2;
  const char* stream = static_cast<const char*>(sg.w) + static_cast<size_t>(r_begin) * row_bytes;

  half* xs16 = sg.in_act == kActNone ? reinterpret_cast<half*>(smem_raw) : nullptr;
  float* xs32 = sg.in_act == kActNone ? nullptr : reinterpret_cast<float*>(smem_raw);
  unsigned char* ring = smem_raw + x_bytes + static_cast<size_t>(warp) * kSlots * kPieceCap;

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kSlots; ++i) mbar_init(smem_u32(&bars[warp][i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  auto issue = [&](int pc) {
    if (lane == 0) {
      const int slot = pc % kSlots;
      const uint32_t bar = smem_u32(&bars[warp][slot]);
      mbar_expect_tx(bar, piece);
      bulk_g2s(smem_u32(ring + slot * kPieceCap), stream + static_cast<size_t>(pc) * piece, piece, bar);
    }
  };
  // weights do not depend on the previous kernel: fill the ring before waiting for it
  for (int pc = 0; pc < kSlots && pc < total; ++pc) issue(pc);

  pdl_wait();
  stage_activations<kM, kWarps * 32>(sg, xs16, xs32);
  __syncthreads();

  const int chunks = piece >> 4;  // 16-byte chunks per piece
  float acc[kM];
  for (int pc = 0; pc < total; ++pc) {
    const int slot = pc % kSlots;
    const int row = pc / parts, part = pc - row * parts;
    if (!mbar_wait(smem_u32(&bars[warp][slot]), (pc / kSlots) & 1)) {
      if (lane == 0) atomicExch(&g_gemv_timeout, 1);
      return;
    }
    if (part == 0) {
#pragma unroll
      for (int m = 0; m < kM; ++m) acc[m] = 0.f;
    }
    const uint4* wsm = reinterpret_cast<const uint4*>(ring + slot * kPieceCap);
    const int k0 = part * (piece >> 1);
#pragma unroll
    for (int it = 0; it < kPieceCap / 16 / 32; ++it) {
      const int c = it * 32 + lane;
      if (c < chunks) {
        const uint4 q = wsm[c];
        const uint32_t wu[4] = {q.x, q.y, q.z, q.w};
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = h2f2(wu[i]);
          wf[2 * i] = f.x;
          wf[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int m = 0; m < kM; ++m) {
          float xf[8];
          if (xs32) {
            const float4 a = *reinterpret_cast<const float4*>(xs32 + static_cast<size_t>(m) * sg.K + k0 + c * 8);
            const float4 b = *reinterpret_cast<const float4*>(xs32 + static_cast<size_t>(m) * sg.K + k0 + c * 8 + 4);
            xf[0] = a.x; xf[1] = a.y; xf[2] = a.z; xf[3] = a.w; xf[4] = b.x; xf[5] = b.y; xf[6] = b.z; xf[7] = b.w;
          } else {
            const uint4 xq = *reinterpret_cast<const uint4*>(xs16 + static_cast<size_t>(m) * sg.K + k0 + c * 8);
            const uint32_t xu[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = h2f2(xu[i]);
              xf[2 * i] = f.x;
              xf[2 * i + 1] = f.y;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[m] = fmaf(xf[i], wf[i], acc[m]);
        }
      }
    }
    __syncwarp();  // every lane has read the slot: it may be overwritten
    if (pc + kSlots < total) issue(pc + kSlots);
    if (part == parts - 1) {
#pragma unroll
      for (int m = 0; m < kM; ++m) {
        const float a = warp_sum(acc[m]);
        if (lane == 0) store_result(sg, m, r_begin + row, a);
      }
    }
  }
}

}  // namespace

// Fills cta_begin / rows_per_cta / parts / piece_bytes for the bulk-copy kernel.  Returns false when
// a problem does not fit it (non-fp16 weights, or a row that cannot be cut into 16-byte multiples).
bool gemv_tma_plan(GemvBatch& b, int M, size_t* smem_bytes, int* grid) {
  size_t x_bytes = 0;
  double total_bytes = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    GemvSeg& g = b.seg[i];
    if (g.fmt != 0) return false;
    const int row_bytes = g.K * 2;
    int parts = (row_bytes + kPieceCap - 1) / kPieceCap;
    while (parts <= 64 && (row_bytes % (parts * 16) != 0)) ++parts;
    if (parts > 64) return false;
    g.parts = parts;
    g.piece_bytes = row_bytes / parts;
    x_bytes = std::max(x_bytes, static_cast<size_t>(M) * g.K * (g.in_act == kActNone ? 2 : 4));
    total_bytes += static_cast<double>(g.N) * row_bytes;
  }
  x_bytes = (x_bytes + 127) & ~static_cast<size_t>(127);
  const size_t smem = x_bytes + static_cast<size_t>(kWarps) * kSlots * kPieceCap;
  if (smem > 200 * 1024) return false;
  // two CTAs per SM when the shared memory allows it, CTAs shared out by weight bytes
  const int per_sm = smem <= 110 * 1024 ? 2 : 1;
  const int budget = 148 * per_sm;
  int cta = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    GemvSeg& g = b.seg[i];
    const double share = static_cast<double>(g.N) * g.K * 2 / total_bytes;
    int n = static_cast<int>(share * budget + 0.5);
    n = std::max(1, std::min(n, (g.N + kWarps - 1) / kWarps));
    g.rows_per_cta = (g.N + n - 1) / n;
    g.cta_begin = cta;
    cta += (g.N + g.rows_per_cta - 1) / g.rows_per_cta;
  }
  *smem_bytes = smem;
  *grid = cta;
  return true;
}

int gemv_tma_launch(cudaStream_t stream, const GemvBatch& b, int M, size_t smem_bytes, int grid) {
  const int x_bytes = static_cast<int>(smem_bytes - static_cast<size_t>(kWarps) * kSlots * kPieceCap);
  auto launch = [&](auto kernel) -> int {
    RK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RK_CUDA(launch_pdl(kernel, dim3(grid), dim3(kWarps * 32), smem_bytes, stream, b, x_bytes));
    return kOk;
  };
  int s;
  switch (M) {
    case 1: s = launch(gemv_tma_kernel<1>); break;
    case 2: s = launch(gemv_tma_kernel<2>); break;
    case 3: s = launch(gemv_tma_kernel<3>); break;
    default: s = launch(gemv_tma_kernel<4>); break;
  }
  if (s != kOk) return s;
  RK_LAUNCH_CHECK("gemv_tma launch");
  return kOk;
}

// Non-zero when a bounded wait inside a bulk-copy kernel has timed out since the last call.
int gemv_timeout_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_timeout, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace rk
