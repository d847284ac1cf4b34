// Tensor-core GEMM for row counts above the weight-streaming GEMV range (batched decode, prefill
// chunks): y[M,N] = epi(x[M,K] W[N,K]^T), fp16 operands, fp32 accumulation in tensor memory.
//
// sm_100a design: the weight matrix takes the MMA's M side ("swap AB"), so a CTA owns 128 output
// channels (weight rows) and a tile of up to 256 activation rows; tiles of 128x64 (weights) and
// Nt x 64 (activations) are brought into 128-byte-swizzled shared memory by TMA
// (cp.async.bulk.tensor), one elected thread issues tcgen05.mma (cta_group::1, kind::f16,
// M=128, N=Nt, K=16) into a TMEM accumulator, tcgen05.commit releases the stage, and four epilogue
// warps read the accumulator back with tcgen05.ld, apply the epilogue and store y (one rounding to
// half, the reference's rounding point for its cuBLAS calls, cuda/rwkv7_v3a_ops.cu:2235-2302).
// Replaces rwkv7_v3a_linear_f16_orig_launch / _lt_cfg_launch / linear_orig_rows_* for rows > 4.
//
// Every mbarrier wait is bounded; on a time-out the kernel records it in a device flag, still
// reaches its final barrier, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

constexpr int kBM = 128;  // weight rows (output channels) per CTA = MMA M
constexpr int kBK = 64;   // halves per K block = one 128-byte swizzle row
constexpr int kThreads = 192;

__device__ int g_gemm_timeout = 0;

struct GemmDev {
  int M, N, K, Nt, stages, epi;
  int splits, kb_per_split;  // split-K: grid.z CTAs share an output tile, kb_per_split K blocks each
  float* partial;            // [splits, M, N] fp32 partial sums (scratch), used when splits > 1
  void* y;
  const half* scale;    // optional per-output-channel factor applied to the accumulator
  const half* v;        // kEpiVres
  const half* v_first;
  const half* v0;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(1) << 16;           // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;   // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;           // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;           // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// Applies the epilogue to one fp32 result: the layer's single rounding to half.
__device__ __forceinline__ void emit(const GemmDev& p, int m, int n, float a) {
  const size_t o = static_cast<size_t>(m) * p.N + n;
  if (p.epi == kEpiRawF32) {
    static_cast<float*>(p.y)[o] = a;
  } else if (p.epi == kEpiF32) {
    static_cast<float*>(p.y)[o] = __half2float(__float2half_rn(a));
  } else if (p.epi == kEpiRelu2) {
    const float t = fmaxf(__half2float(__float2half_rn(a)), 0.f);
    static_cast<half*>(p.y)[o] = __float2half_rn(t * t);
  } else if (p.epi == kEpiVres) {
    const float vv = __half2float(p.v[o]);
    const float gate = 1.0f / (1.0f + expf(-(__half2float(p.v0[n]) + a)));
    static_cast<half*>(p.y)[o] = __float2half_rn(vv + (__half2float(p.v_first[o]) - vv) * gate);
  } else {
    static_cast<half*>(p.y)[o] = __float2half_rn(a);
  }
}

__global__ void __launch_bounds__(kThreads) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                           const __grid_constant__ CUtensorMap map_x, const GemmDev p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[8], empty_bar[8], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kBM, m0 = blockIdx.y * p.Nt;
  const int kb_total = (p.K + kBK - 1) / kBK;
  const int kb_begin = blockIdx.z * p.kb_per_split;
  const int kblocks = min(kb_total - kb_begin, p.kb_per_split);  // >= 1 by construction of the grid
  const uint32_t stage_bytes = kBM * 128 + p.Nt * 128;
  // the dynamic window is 1024-byte aligned by the launch (required by the 128-byte swizzle)
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(p.Nt)) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&acc_bar), 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_slot;

  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ---- TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % p.stages;
        if (kb >= p.stages && !mbar_wait(smem_u32(&empty_bar[s]), ((kb / p.stages) - 1) & 1)) { failed = 1; break; }
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t a = smem_base + s * stage_bytes;
        mbar_expect_tx(bar, stage_bytes);
        tma_load_2d(a, &map_w, bar, (kb_begin + kb) * kBK, n0);
        tma_load_2d(a + kBM * 128, &map_x, bar, (kb_begin + kb) * kBK, m0);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(p.Nt >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < kblocks && ok; ++kb) {
        const int s = kb % p.stages;
        ok = mbar_wait(smem_u32(&full_bar[s]), (kb / p.stages) & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_base + s * stage_bytes;
        const uint64_t da = smem_desc(a), db = smem_desc(a + kBM * 128);
#pragma unroll
        for (int k4 = 0; k4 < kBK / 16; ++k4)  // 32 bytes further along the swizzled row per K=16 step
          mma_f16(tmem_acc, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
        mma_commit(smem_u32(&empty_bar[s]));
      }
      if (ok) mma_commit(smem_u32(&acc_bar));
      else failed = 1;
    }
  } else {
    // ---- epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 = output channels n0 + that
    const bool ok = mbar_wait(smem_u32(&acc_bar), 0);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      // Phase A: TMEM -> registers -> an fp32 tile [Nt][128 (+4 pad)] in the (now idle) stage memory, so that
      // phase B can write y with 8- or 16-byte stores along the channel dimension.
      const int q = warp & 3;
      float* tile = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)));
      constexpr int kLd = kBM + 4;
      const int m_valid = min(p.Nt, p.M - m0);
      for (int c0 = 0; c0 < m_valid; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_acc + (static_cast<uint32_t>(q * 32) << 16) + c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) tile[(c0 + j) * kLd + q * 32 + lane] = __uint_as_float(r[j]);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // Phase B: thread t owns 4 consecutive channels of rows t/32, t/32 + 4, ...
      const int t = threadIdx.x - 64;
      const int c4 = (t & 31) * 4, n = n0 + c4;
      if (n < p.N) {
        float sc[4] = {1.f, 1.f, 1.f, 1.f};
        if (p.scale) {
#pragma unroll
          for (int i = 0; i < 4; ++i) sc[i] = __half2float(p.scale[n + i]);
        }
        for (int ml = t >> 5; ml < m_valid; ml += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(tile + ml * kLd + c4);
          const float a[4] = {a4.x * sc[0], a4.y * sc[1], a4.z * sc[2], a4.w * sc[3]};
          const size_t o = static_cast<size_t>(m0 + ml) * p.N + n;
          if (p.splits > 1) {
            *reinterpret_cast<float4*>(p.partial + static_cast<size_t>(blockIdx.z) * p.M * p.N + o) = a4;
          } else if (p.epi == kEpiRawF32) {
            *reinterpret_cast<float4*>(static_cast<float*>(p.y) + o) = make_float4(a[0], a[1], a[2], a[3]);
          } else if (p.epi == kEpiF32) {
            float4 o4;
            o4.x = __half2float(__float2half_rn(a[0])); o4.y = __half2float(__float2half_rn(a[1]));
            o4.z = __half2float(__float2half_rn(a[2])); o4.w = __half2float(__float2half_rn(a[3]));
            *reinterpret_cast<float4*>(static_cast<float*>(p.y) + o) = o4;
          } else {
            float e[4];
            if (p.epi == kEpiRelu2) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float u = fmaxf(__half2float(__float2half_rn(a[i])), 0.f);
                e[i] = u * u;
              }
            } else if (p.epi == kEpiVres) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float vv = __half2float(p.v[o + i]);
                const float gate = 1.0f / (1.0f + expf(-(__half2float(p.v0[n + i]) + a[i])));
                e[i] = vv + (__half2float(p.v_first[o + i]) - vv) * gate;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) e[i] = a[i];
            }
            const __half2 lo = __floats2half2_rn(e[0], e[1]), hi = __floats2half2_rn(e[2], e[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(static_cast<half*>(p.y) + o) = pk;
          }
        }
      }
    } else if (lane == 0) {
      failed = 1;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && failed) atomicExch(&g_gemm_timeout, 1);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(tmem_cols) : "memory");
  }
}

// Second pass of a split-K GEMM: adds the fp32 partial sums in split order (the result does not
// depend on which CTA finished first) and applies the epilogue.  One thread per four output channels.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmDev p) {
  pdl_wait();
  pdl_trigger();
  const int n4 = p.N >> 2;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(p.M) * n4) return;
  const int m = static_cast<int>(i / n4), n = static_cast<int>(i - static_cast<long long>(m) * n4) * 4;
  const size_t plane = static_cast<size_t>(p.M) * p.N;
  const float* src = p.partial + static_cast<size_t>(m) * p.N + n;
  float4 acc = __ldcg(reinterpret_cast<const float4*>(src));
  for (int z = 1; z < p.splits; ++z) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(src + z * plane));
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  const float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) emit(p, m, n + j, v[j] * (p.scale ? __half2float(p.scale[n + j]) : 1.0f));
}

}  // namespace

// ---------------------------------------------------------------------------------- host side
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return static_cast<EncodeFn>(nullptr);
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}

// 2-D fp16 tensor [rows, cols] with row stride ld (elements), boxes of 64 columns x box_rows rows,
// 128-byte swizzle, zero fill outside the tensor.
int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeFn fn = encode_fn();
  RK_REQUIRE(fn, kCuda, "gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RK_REQUIRE(r == CUDA_SUCCESS, kCuda, "gemm_tc: cuTensorMapEncodeTiled failed with %d (rows=%d cols=%d ld=%d)", static_cast<int>(r), rows, cols, ld);
  return kOk;
}

int pick_nt(int M) {
  if (M >= 256) return 256;
  return ((M + 15) / 16) * 16;
}

}  // namespace

bool gemm_tc_supported(const LinearArgs& a) {
  const int ldx = a.ldx ? a.ldx : a.K;
  return a.fmt == 0 && a.in_act == kActNone && a.K % 8 == 0 && ldx % 8 == 0 && a.M > 4 && a.N % 4 == 0 &&
         (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0;
}

int gemm_tc(cudaStream_t stream, const LinearArgs& a) {
  RK_REQUIRE(gemm_tc_supported(a), kShape, "gemm_tc: unsupported problem");
  const int ldx = a.ldx ? a.ldx : a.K;
  GemmDev p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.epi = a.epi; p.y = a.y; p.scale = a.out_scale;
  p.v = a.ea.v; p.v_first = a.ea.v_first; p.v0 = a.ea.v0;
  p.Nt = pick_nt(a.M);
  const size_t stage_bytes = static_cast<size_t>(kBM) * 128 + static_cast<size_t>(p.Nt) * 128;
  p.stages = static_cast<int>(std::min<size_t>(8, (200 * 1024) / stage_bytes));
  const size_t smem = stage_bytes * p.stages + 1024;
  CUtensorMap map_w, map_x;
  int s = make_map(&map_w, a.w, a.N, a.K, a.K, kBM);
  if (s != kOk) return s;
  s = make_map(&map_x, a.x, a.M, a.K, ldx, p.Nt);
  if (s != kOk) return s;
  RK_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 201 * 1024 + 1024));
  // Split K over grid.z until the grid covers the SMs: a tile of 128 output channels per CTA alone
  // leaves most of them idle for the narrow layers (C x C projections, LoRA).  Needs scratch for the
  // fp32 partial sums (a second small kernel adds them in split order); without it the kernel runs unsplit.
  const int tiles = ((a.N + kBM - 1) / kBM) * ((a.M + p.Nt - 1) / p.Nt);
  const int kb_total = (a.K + kBK - 1) / kBK;
  int splits = 1;
  if (a.scratch && tiles < 120 && a.N % 4 == 0) {
    splits = std::min({(148 + tiles - 1) / tiles, std::max(1, kb_total / 2), 32});
    const size_t per_split = static_cast<size_t>(a.M) * a.N * sizeof(float);
    splits = static_cast<int>(std::min<size_t>(splits, a.scratch_bytes / per_split));
    splits = std::max(splits, 1);
  }
  p.kb_per_split = (kb_total + splits - 1) / splits;
  p.splits = (kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  p.partial = a.scratch;
  const dim3 grid((a.N + kBM - 1) / kBM, (a.M + p.Nt - 1) / p.Nt, p.splits), block(kThreads);
  RK_CUDA(launch_pdl(gemm_tc_kernel, grid, block, smem, stream, map_w, map_x, p));
  RK_LAUNCH_CHECK("gemm_tc launch");
  if (p.splits > 1) {
    const long long work = static_cast<long long>(a.M) * (a.N / 4);
    RK_CUDA(launch_pdl(splitk_reduce_kernel, dim3(static_cast<unsigned>((work + 255) / 256)), dim3(256), 0, stream, p));
    RK_LAUNCH_CHECK("splitk_reduce launch");
  }
  return kOk;
}

// ---------------------------------------------------------------------------------------------
// Split-K GEMM for callers that must not allocate: the fp32 partial sums go to a fixed device array
// that is part of the loaded library image (every GPU that loads the library holds these 16 MiB
// until the process exits).
constexpr size_t kStaticScratchFloats = static_cast<size_t>(4) << 20;  // 16 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

int gemm_tc_static_scratch(cudaStream_t stream, const LinearArgs& a) {
  RK_REQUIRE(gemm_tc_supported(a), kShape, "linear (static scratch): needs more than 4 rows, fp16 weights, K %% 8 == 0");
  RK_REQUIRE(a.N % 4 == 0, kShape, "linear (static scratch): N must be a multiple of 4");
  // at least two K splits must fit: 2 * M * N floats
  RK_REQUIRE(static_cast<size_t>(a.M) * a.N * 2 <= kStaticScratchFloats, kShape,
             "linear (static scratch): M*N = %lld exceeds the built-in scratch (max %lld elements)",
             static_cast<long long>(a.M) * a.N, static_cast<long long>(kStaticScratchFloats / 2));
  // In host code the array's name is only a stand-in; the device address is looked up once per device
  // (with that device current, as it is here) and cached.
  static float* dev_ptr[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  RK_CUDA(cudaGetDevice(&dev));
  RK_REQUIRE(dev >= 0 && dev < 64, kBadArg, "linear (static scratch): device ordinal out of range");
  float* ptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!dev_ptr[dev]) {
      void* p = nullptr;
      RK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
      dev_ptr[dev] = static_cast<float*>(p);
    }
    ptr = dev_ptr[dev];
  }
  LinearArgs b = a;
  b.scratch = ptr;
  b.scratch_bytes = kStaticScratchFloats * sizeof(float);
  return gemm_tc(stream, b);
}

int gemm_timeout_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_timeout, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace rk
