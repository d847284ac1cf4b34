// Tensor-core GEMM for row counts above the weight-streaming GEMV range (batched decode, prefill
// chunks): y[M,N] = epi(x[M,K] W[N,K]^T), fp16 operands, fp32 accumulation in tensor memory.  Up to
// eight such products that share M run as ONE persistent launch (a layer's r/k/v projections and
// LoRA down-projections, or its four LoRA up-projections).
//
// sm_100a design: the weight matrix takes the MMA's M side ("swap AB"), so a work unit is 128 output
// channels (weight rows) x a tile of Nt <= 256 activation rows x a range of K.  One CTA per SM walks
// the unit list with a stride of the grid size.  Tiles of 128x64 (weights) and Nt x 64 (activations)
// are brought into 128-byte-swizzled shared memory by TMA (cp.async.bulk.tensor) through one ring of
// stages that keeps running across units; one elected thread issues tcgen05.mma (cta_group::1,
// kind::f16, M=128, N=Nt, K=16) into one of two TMEM accumulators; tcgen05.commit releases the stage;
// eight epilogue warps read the finished accumulator back with tcgen05.ld, apply the epilogue and store
// y (one rounding to half, the reference's rounding point for its cuBLAS calls,
// cuda/rwkv7_v3a_ops.cu:2235-2302) while the next unit's MMAs fill the other accumulator.
// Replaces rwkv7_v3a_linear_f16_orig_launch / _lt_cfg_launch / linear_orig_rows_* for rows > 4.
//
// Narrow products are split along K so that every SM has work; the fp32 partial sums go to scratch and
// a second small kernel adds them in split order (the result does not depend on timing).
//
// W8A16 / W4A16 weights (kQuant instantiation): TMA brings the PACKED tile (128 rows x 64 int8, or x 32 bytes of
// nibbles) into a raw staging area of the stage; four more warps -- one thread per weight row -- expand it in
// registers to the fp16 values the format defines (W8A16: the integer code, the channel scale goes on the
// accumulator in the epilogue; W4A16: half((q - zero) * scale) with the group's scale and zero) and write the
// 128-byte-swizzled tile the MMA reads; a second barrier per stage tells the MMA issuer that the tile is ready.
// HBM traffic is the packed bytes; no fp16 copy of a quantised matrix exists anywhere.
//
// Every mbarrier wait is bounded; on a time-out the kernel records it in a device flag, every role
// leaves its loop, the CTA reaches its final barrier, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "tensormap.h"

namespace rk {
namespace {

constexpr int kBM = 128;  // weight rows (output channels) per unit = MMA M
constexpr int kBK = 64;   // halves per K block = one 128-byte swizzle row
constexpr int kEpiThreads = 256;  // eight epilogue warps: two per scheduler, each pair shares a TMEM lane quadrant
constexpr int kCtrlThreads = 64;   // TMA producer and MMA issuer (one lane of a warp each)
constexpr int kThreads = kCtrlThreads + kEpiThreads;
constexpr int kDequantThreads = 256;  // quantised weights only: two groups of 128 (one thread per weight row of a tile)
                                      // that take alternate stages, so two tiles are being expanded at any time
constexpr int kRawBytes = kBM * kBK;  // raw staging area of a stage: a packed int8 tile (an int4 tile takes half)
constexpr int kMaxProb = 8;
constexpr int kEpiRows = 32;             // activation rows transposed through shared memory at a time
constexpr int kEpiLd = kBM + 4;          // padded row of the transposition tile (floats)
constexpr int kEpiBytes = kEpiRows * kEpiLd * 4;
constexpr int kMaxStages = 8;

struct Prob {
  int M, N, K, epi;
  int tiles_n;               // ceil(N / 128)
  int splits, kb_per_split;  // K blocks per unit
  int unit_begin;            // index of this product's first work unit
  int red_begin;             // first 256-thread block of the reduction kernel that belongs to this product
  float* partial;            // [splits, M, N] fp32 partial sums, when splits > 1
  void* y;
  const half* scale;         // optional per-output-channel factor applied to the accumulator
  int fmt;                   // weight format of this product (0 fp16, 1 W8A16, 2 W4A16)
  const half* qscale;        // W4A16: [N, K/128] group scales and zeros
  const half* qzero;
  const half* v;             // kEpiVres
  const half* v_first;
  const half* v0;
};

struct GroupDev {
  int n_prob, total_units, Nt, stages, tiles_m, red_blocks;
  int bm;         // output channels per work unit: 128, or 256 for the CTA-pair kernel
  int w_dynamic;  // the weights may have been written by the previous kernel: wait for it before reading them
  int* timeout;   // the device's failure word: a bounded wait that runs out ORs kTimeoutGemm into it
  Prob prob[kMaxProb];
};

struct MapPack {
  CUtensorMap w[kMaxProb];
  CUtensorMap x[kMaxProb];
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// First expired wait of the device since the record was last cleared: who waited, and on what (status.cu).
__device__ __forceinline__ void note_timeout(int* word, int role, int unit, int it, int stages, int total, int prob, int M, int N,
                                             int K, int fmt, int Nt, int splits) {
  if (!word || atomicCAS(word + 1, 0, 1) != 0) return;
  const int v[13] = {role, static_cast<int>(blockIdx.x), unit, it, stages, total, prob, M, N, K, fmt, Nt, splits};
  for (int i = 0; i < 13; ++i) word[2 + i] = v[i];
}

// ---- CTA-pair (cta_group::2) forms: two CTAs of a cluster work on one 256-channel tile.  Each loads its own 128
// weight rows and HALF of the activation tile; the leader (cluster rank 0) issues the MMAs for both.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in the CTA of the given cluster rank.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The destination is this CTA's shared memory; the barrier (a shared::cluster address) is the leader's.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both)
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

// What the epilogue needs of one product, copied into registers once per unit (reading the kernel parameter
// block through a run-time index inside the store loop costs a dependent constant load per row).
struct EpiCtx {
  int M, N, epi, splits;
  float* partial;
  void* y;
  const half *scale, *v, *v_first, *v0;
};
__device__ __forceinline__ EpiCtx make_ctx(const Prob& p) {
  EpiCtx c;
  c.M = p.M; c.N = p.N; c.epi = p.epi; c.splits = p.splits; c.partial = p.partial; c.y = p.y;
  c.scale = p.scale; c.v = p.v; c.v_first = p.v_first; c.v0 = p.v0;
  return c;
}

// The epilogue of one fp32 result (already scaled): the layer's single rounding to half follows in store4.
__device__ __forceinline__ float epi_value(const EpiCtx& p, size_t o, int n, float a) {
  if (p.epi == kEpiRelu2) {
    const float u = fmaxf(__half2float(__float2half_rn(a)), 0.f);
    return u * u;
  }
  if (p.epi == kEpiVres) {
    const float vv = __half2float(p.v[o]);
    const float gate = 1.0f / (1.0f + expf(-(__half2float(p.v0[n]) + a)));
    return vv + (__half2float(p.v_first[o]) - vv) * gate;
  }
  if (p.epi == kEpiTanhH) return apply_in_act(__half2float(__float2half_rn(a)), kActTanh);
  if (p.epi == kEpiSigmoidH) return apply_in_act(__half2float(__float2half_rn(a)), kActSigmoid);
  return a;
}

__device__ __forceinline__ void store_half4(half* y, size_t o, float e0, float e1, float e2, float e3) {
  const __half2 lo = __floats2half2_rn(e0, e1), hi = __floats2half2_rn(e2, e3);
  uint2 pk;
  pk.x = *reinterpret_cast<const uint32_t*>(&lo);
  pk.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(y + o) = pk;
}

// Stores four consecutive output channels of one row.
__device__ __forceinline__ void store4(const EpiCtx& p, int m, int n, const float (&a)[4]) {
  const size_t o = static_cast<size_t>(m) * p.N + n;
  if (p.epi == kEpiNone) {
    store_half4(static_cast<half*>(p.y), o, a[0], a[1], a[2], a[3]);
  } else if (p.epi == kEpiRawF32) {
    *reinterpret_cast<float4*>(static_cast<float*>(p.y) + o) = make_float4(a[0], a[1], a[2], a[3]);
  } else if (p.epi == kEpiF32) {
    float4 o4;
    o4.x = __half2float(__float2half_rn(a[0])); o4.y = __half2float(__float2half_rn(a[1]));
    o4.z = __half2float(__float2half_rn(a[2])); o4.w = __half2float(__float2half_rn(a[3]));
    *reinterpret_cast<float4*>(static_cast<float*>(p.y) + o) = o4;
  } else {
    float e[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) e[i] = epi_value(p, o + i, n + i, a[i]);
    store_half4(static_cast<half*>(p.y), o, e[0], e[1], e[2], e[3]);
  }
}

// Barrier over the 256 epilogue threads that also ANDs a predicate.
__device__ __forceinline__ bool epi_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 256, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(ok))
      : "memory");
  return r != 0;
}

struct Unit {
  int prob, n0, m0, kb_begin, kblocks, split;
};

__device__ __forceinline__ Unit decode_unit(const GroupDev& g, int u) {
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kMaxProb; ++i)
    if (i < g.n_prob && u >= g.prob[i].unit_begin) pi = i;
  const Prob& p = g.prob[pi];
  int local = u - p.unit_begin;
  // consecutive units are the row tiles of one weight tile: they run at the same time on neighbouring
  // CTAs, so the weight tile comes from DRAM once and from L2 afterwards
  const int mt = local % g.tiles_m;
  local /= g.tiles_m;
  const int nt = local % p.tiles_n, split = local / p.tiles_n;
  Unit r;
  r.prob = pi;
  r.n0 = nt * g.bm;
  r.m0 = mt * g.Nt;
  r.split = split;
  r.kb_begin = split * p.kb_per_split;
  const int kb_total = (p.K + kBK - 1) / kBK;
  r.kblocks = min(kb_total - r.kb_begin, p.kb_per_split);  // >= 1 by construction of the unit list
  return r;
}

template <bool kPair, bool kQuant>
__global__ void __launch_bounds__(kThreads + (kQuant ? kDequantThreads : 0), 1)
    gemm_group_kernel(const __grid_constant__ MapPack maps, const GroupDev g) {
  static_assert(!(kPair && kQuant), "the CTA-pair variant takes fp16 weights only");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], ready_bar[kMaxStages];
  __shared__ __align__(8) uint64_t acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kWBytes = kBM * 128;
  // CTA pair: cluster rank 0 leads; every CTA stages its own 128 weight rows and half of the activation rows
  const uint32_t rank = kPair ? cluster_rank() : 0u;
  const int first_unit = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int unit_stride = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int x_rows = kPair ? g.Nt / 2 : g.Nt;
  const uint32_t x_bytes = x_rows * 128;
  // the dynamic window is 1024-byte aligned here (required by the 128-byte swizzle): weight ring, activation ring,
  // epilogue tile
  const uint32_t stage_bytes = kWBytes + x_bytes + (kQuant ? kRawBytes : 0);  // [fp16 weights][activations][packed weights]
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  float* const epi_tile = reinterpret_cast<float*>(smem_raw + (ring - smem_u32(smem_raw)) + g.stages * stage_bytes);
  constexpr uint32_t kTmemCols = 512;  // two accumulators of up to 256 columns; one CTA per SM

  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&ready_bar[s]), kDequantThreads / 2);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), kPair ? 2 : 1);  // one arrival per CTA whose epilogue drains the accumulator
    }
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  __syncwarp();
  if (kPair) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---- TMA producer: one ring of stages, each a weight tile followed by an activation tile.  Weights that were
    // written long before this launch do not depend on the previous kernel, so the first ring fill's weight tiles
    // are requested before the dependency wait; the activation tiles follow after it.
    if (lane == 0) {
      auto load_w = [&](const Unit& u, int kb, int s) {
        const uint32_t bar = smem_u32(&full_bar[s]);
        if (kPair) {  // both CTAs' tiles complete the leader's barrier
          if (rank == 0) mbar_expect_tx(bar, 2 * stage_bytes);
          tma_load_2d_pair(ring + s * stage_bytes, &maps.w[u.prob], map_to_rank(bar, 0), (u.kb_begin + kb) * kBK,
                           u.n0 + static_cast<int>(rank) * kBM);
        } else if (kQuant && g.prob[u.prob].fmt != 0) {  // packed tile into the raw area: 64 or 32 bytes per row
          const int row_bytes = g.prob[u.prob].fmt == 1 ? kBK : kBK / 2;
          mbar_expect_tx(bar, static_cast<uint32_t>(kBM * row_bytes) + x_bytes);
          tma_load_2d(ring + s * stage_bytes + kWBytes + x_bytes, &maps.w[u.prob], bar, (u.kb_begin + kb) * row_bytes, u.n0);
        } else {
          mbar_expect_tx(bar, kWBytes + x_bytes);
          tma_load_2d(ring + s * stage_bytes, &maps.w[u.prob], bar, (u.kb_begin + kb) * kBK, u.n0);
        }
      };
      auto load_x = [&](const Unit& u, int kb, int s) {
        const uint32_t bar = smem_u32(&full_bar[s]);
        if (kPair)
          tma_load_2d_pair(ring + s * stage_bytes + kWBytes, &maps.x[u.prob], map_to_rank(bar, 0), (u.kb_begin + kb) * kBK,
                           u.m0 + static_cast<int>(rank) * x_rows);
        else
          tma_load_2d(ring + s * stage_bytes + kWBytes, &maps.x[u.prob], bar, (u.kb_begin + kb) * kBK, u.m0);
      };
      int pre = 0;
      if (!g.w_dynamic && first_unit < g.total_units) {
        const Unit u = decode_unit(g, first_unit);
        pre = min(u.kblocks, g.stages);
        for (int kb = 0; kb < pre; ++kb) load_w(u, kb, kb);
      }
      pdl_wait();
      pdl_trigger();
      bool ok = true;
      int it = 0;
      for (int ui = first_unit; ui < g.total_units && ok && !failed; ui += unit_stride) {
        const Unit u = decode_unit(g, ui);
        for (int kb = 0; kb < u.kblocks; ++kb, ++it) {
          const int s = it % g.stages;
          if (it >= pre) {
            if (it >= g.stages && !mbar_wait(smem_u32(&empty_bar[s]), ((it / g.stages) - 1) & 1)) {
              note_timeout(g.timeout, 1, ui, it, g.stages, g.total_units, u.prob, g.prob[u.prob].M, g.prob[u.prob].N, g.prob[u.prob].K, g.prob[u.prob].fmt, g.Nt, g.prob[u.prob].splits);
              ok = false;
              break;
            }
            load_w(u, kb, s);
          }
          load_x(u, kb, s);
        }
      }
      if (!ok) failed = 1;
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0 && rank == 0) {
      // fp32 accumulate, fp16 operands, both K-major; N = row-tile width, M = 128 per CTA
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(g.Nt >> 3) << 17) |
                             (static_cast<uint32_t>((kPair ? 2 * kBM : kBM) >> 4) << 24);
      bool ok = true;
      int it = 0, n_unit = 0;
      for (int ui = first_unit; ui < g.total_units && ok && !failed; ui += unit_stride, ++n_unit) {
        const Unit u = decode_unit(g, ui);
        const int acc = n_unit & 1;
        if (n_unit >= 2) {  // the epilogue of the unit that used this accumulator two units ago has drained it
          ok = mbar_wait(smem_u32(&acc_empty[acc]), ((n_unit >> 1) - 1) & 1);
          if (!ok) {
            note_timeout(g.timeout, 20, ui, it, g.stages, g.total_units, u.prob, g.prob[u.prob].M, g.prob[u.prob].N, g.prob[u.prob].K, g.prob[u.prob].fmt, g.Nt, g.prob[u.prob].splits);
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * g.Nt);
        for (int kb = 0; kb < u.kblocks; ++kb, ++it) {
          const int s = it % g.stages;
          ok = mbar_wait(smem_u32(&full_bar[s]), (it / g.stages) & 1);
          if (!ok) note_timeout(g.timeout, 21, ui, it, g.stages, g.total_units, u.prob, g.prob[u.prob].M, g.prob[u.prob].N, g.prob[u.prob].K, g.prob[u.prob].fmt, g.Nt, g.prob[u.prob].splits);
          if (kQuant && ok) {
            ok = mbar_wait(smem_u32(&ready_bar[s]), (it / g.stages) & 1);  // the expanded tile is written
            if (!ok) note_timeout(g.timeout, 22, ui, it, g.stages, g.total_units, u.prob, g.prob[u.prob].M, g.prob[u.prob].N, g.prob[u.prob].K, g.prob[u.prob].fmt, g.Nt, g.prob[u.prob].splits);
          }
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da = smem_desc(ring + s * stage_bytes), db = smem_desc(ring + s * stage_bytes + kWBytes);
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4) {  // 32 bytes further along the swizzled row per K=16 step
            if (kPair) mma_f16_pair(tmem_acc, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
            else mma_f16(tmem_acc, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
          }
          if (kPair) {
            mma_commit_pair(smem_u32(&empty_bar[s]));
          } else {
            mma_commit(smem_u32(&empty_bar[s]));
          }
        }
        if (ok) {
          if (kPair) mma_commit_pair(smem_u32(&acc_full[acc]));
          else mma_commit(smem_u32(&acc_full[acc]));
        }
      }
      if (!ok) failed = 1;
    }
  } else if (kQuant && threadIdx.x >= kThreads) {
    // ---- dequantisation: thread r expands weight row r of every stage's packed tile into the swizzled fp16 tile.
    // Row r of the tile is 128 bytes at r * 128; its 16-byte chunk c lives at chunk position c ^ (r & 7).
    const int r = (static_cast<int>(threadIdx.x) - kThreads) & 127;
    const int my_parity = (static_cast<int>(threadIdx.x) - kThreads) >> 7;  // this group's stages: it % 2 == my_parity
    unsigned char* const ring_g = smem_raw + (ring - smem_u32(smem_raw));
    bool ok = true;
    int it = 0;
    for (int ui = first_unit; ui < g.total_units && ok && !failed; ui += unit_stride) {
      const Unit u = decode_unit(g, ui);
      const Prob& p = g.prob[u.prob];
      const int fmt = p.fmt, row = u.n0 + r, groups = p.K >> 7;
      for (int kb = 0; kb < u.kblocks; ++kb, ++it) {
        const int s = it % g.stages;
        const bool mine = (it & 1) == my_parity;
        __half2 sc2 = __floats2half2_rn(0.f, 0.f), add2 = sc2;
        if (mine && fmt == 2 && row < p.N) {  // this K block's group parameters, requested before the wait for the tile
          const size_t gi = static_cast<size_t>(row) * groups + (((u.kb_begin + kb) * kBK) >> 7);
          const half sc = p.qscale[gi];
          const float z = __half2float(p.qzero[gi]);
          sc2 = __half2half2(sc);
          // low nibble: (1024 + q) - (1024 + z); high nibble arrives as 1024 + 16 q: / 16 - (64 + z)
          add2 = __halves2half2(__hneg(__float2half_rn(1024.f + z)), __hneg(__float2half_rn(64.f + z)));
        }
        ok = mbar_wait(smem_u32(&full_bar[s]), (it / g.stages) & 1);
        // Every thread watches EVERY fill of every stage, also those the other group expands: a waiter that skipped a
        // phase of a barrier would find the parity of the phase after it "already complete" while the one in between
        // is still pending (the parity test cannot tell phase n + 2 from phase n), and expand a tile that has not
        // landed -- seen as expired waits on launches where a later stage's tile arrived before an earlier one's.
        if (ok && !mine) continue;
        if (!ok) {
          if (r == 0) note_timeout(g.timeout, 3, ui, it, g.stages, g.total_units, u.prob, g.prob[u.prob].M, g.prob[u.prob].N, g.prob[u.prob].K, g.prob[u.prob].fmt, g.Nt, g.prob[u.prob].splits);
          break;
        }
        if (fmt != 0) {
          unsigned char* stage = ring_g + static_cast<size_t>(s) * stage_bytes;
          uint4* dst = reinterpret_cast<uint4*>(stage + r * 128);
          if (fmt == 1) {
            const uint4* src = reinterpret_cast<const uint4*>(stage + kWBytes + x_bytes + r * kBK);
            const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // 16 codes -> two chunks of 8 halves
              const uint4 q = src[c];
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
              uint32_t h[8];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t t = w[i] ^ 0x80808080u;
                uint32_t h01 = __byte_perm(t, 0x64646464u, 0x4140);
                uint32_t h23 = __byte_perm(t, 0x64646464u, 0x4342);
                const __half2 a = __hsub2(*reinterpret_cast<__half2*>(&h01), bias);
                const __half2 b = __hsub2(*reinterpret_cast<__half2*>(&h23), bias);
                h[2 * i] = *reinterpret_cast<const uint32_t*>(&a);
                h[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&b);
              }
              dst[(2 * c) ^ (r & 7)] = make_uint4(h[0], h[1], h[2], h[3]);
              dst[(2 * c + 1) ^ (r & 7)] = make_uint4(h[4], h[5], h[6], h[7]);
            }
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(stage + kWBytes + x_bytes + r * (kBK / 2));
            const __half2 mul = __floats2half2_rn(1.0f, 0.0625f);
#pragma unroll
            for (int c = 0; c < 2; ++c) {  // 32 codes -> four chunks
              const uint4 q = src[c];
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {  // a word = 8 codes = one chunk; byte b holds codes 2b (low nibble), 2b + 1
                uint32_t h[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const uint32_t both = __byte_perm(w[i], 0u, 0x4040u + 0x0101u * b);  // the byte in both halves
                  uint32_t pair = (both & 0x00f0000fu) | 0x64006400u;                  // (1024 + lo, 1024 + 16 hi)
                  const __half2 v = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&pair), mul, add2), sc2);
                  h[b] = *reinterpret_cast<const uint32_t*>(&v);
                }
                dst[(4 * c + i) ^ (r & 7)] = make_uint4(h[0], h[1], h[2], h[3]);
              }
            }
          }
          // the tile was written through the generic proxy; the tensor core reads it through the async proxy
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        mbar_arrive(smem_u32(&ready_bar[s]));
      }
    }
    if (!ok) failed = 1;
  } else {
    // ---- epilogue: warp w reads TMEM lanes 32*(w%4) .. +31 = output channels n0 + that
    pdl_wait();  // y and the partial sums may still be read by the previous kernel
    const int q = warp & 3;
    const int t = threadIdx.x - kCtrlThreads;
    const int c4 = (t & 31) * 4;
    int n_unit = 0;
    for (int ui = first_unit; ui < g.total_units; ui += unit_stride, ++n_unit) {
      Unit u = decode_unit(g, ui);
      u.n0 += static_cast<int>(rank) * kBM;  // this CTA's 128 channels of the tile
      const EpiCtx p = make_ctx(g.prob[u.prob]);
      const int acc = n_unit & 1;
      bool ok = !failed && mbar_wait(smem_u32(&acc_full[acc]), (n_unit >> 1) & 1);
      // the four warps must agree, or the named barriers below would not match up
      ok = epi_all(ok);
      if (!ok) {
        if (t == 0) {
          if (!failed) note_timeout(g.timeout, 4, ui, n_unit, g.stages, g.total_units, u.prob, g.prob[u.prob].M, g.prob[u.prob].N, g.prob[u.prob].K, g.prob[u.prob].fmt, g.Nt, g.prob[u.prob].splits);
          failed = 1;
        }
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * g.Nt) + (static_cast<uint32_t>(q * 32) << 16);
      const int m_valid = min(g.Nt, p.M - u.m0);
      const int n = u.n0 + c4;
      float sc[4] = {1.f, 1.f, 1.f, 1.f};
      if (p.scale && n < p.N) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[i] = __half2float(p.scale[n + i]);
      }
      for (int c0 = 0; c0 < m_valid; c0 += kEpiRows) {
        // phase A: TMEM -> registers -> fp32 tile [32 rows][128 channels (+4 pad)]; the two warps of a lane
        // quadrant take 16 rows each
        const int half_rows = (warp - kCtrlThreads / 32) >> 2;
        if (c0 + half_rows * 16 < g.Nt) {
          uint32_t r0[16];
          tmem_ld16(tmem_acc + c0 + half_rows * 16, r0);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) epi_tile[(half_rows * 16 + j) * kEpiLd + q * 32 + lane] = __uint_as_float(r0[j]);
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // phase B: thread t owns 4 consecutive channels of rows t/32, t/32 + 8, ... of this slab
        const int rows_here = min(kEpiRows, m_valid - c0);
        if (n < p.N) {
          constexpr int kIter = kEpiRows / (kEpiThreads / 32);
          float4 a4[kIter];
#pragma unroll
          for (int i = 0; i < kIter; ++i)  // all shared-memory reads first, then the stores
            a4[i] = *reinterpret_cast<const float4*>(epi_tile + ((t >> 5) + (kEpiThreads / 32) * i) * kEpiLd + c4);
          const int m_first = u.m0 + c0 + (t >> 5);
          const size_t o_first = static_cast<size_t>(m_first) * p.N + n;
#pragma unroll
          for (int i = 0; i < kIter; ++i) {
            const int ml = (t >> 5) + (kEpiThreads / 32) * i;
            if (ml >= rows_here) continue;
            const size_t o = o_first + static_cast<size_t>((kEpiThreads / 32) * i) * p.N;
            if (p.splits > 1) {
              *reinterpret_cast<float4*>(p.partial + static_cast<size_t>(u.split) * p.M * p.N + o) = a4[i];
            } else if (p.epi == kEpiNone && !p.scale) {
              store_half4(static_cast<half*>(p.y), o, a4[i].x, a4[i].y, a4[i].z, a4[i].w);
            } else {
              const float a[4] = {a4[i].x * sc[0], a4[i].y * sc[1], a4[i].z * sc[2], a4[i].w * sc[3]};
              store4(p, m_first + (kEpiThreads / 32) * i, n, a);
            }
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
      // every warp's TMEM reads are complete (wait::ld + the barrier above): hand the accumulator back
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (t == 0) {
        if (kPair) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty[acc]), 0));
        else mbar_arrive(smem_u32(&acc_empty[acc]));
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (threadIdx.x == 0 && failed && g.timeout) atomicOr(g.timeout, kTimeoutGemm);
  __syncwarp();
  if (kPair) cluster_sync_all();  // neither CTA leaves while its partner may still signal its barriers or read its tiles
  if (warp == 1) {
    if (kPair) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// Second pass of split-K products: adds the fp32 partial sums in split order (the result does not depend on which
// CTA finished first) and applies the epilogue.  One thread per four output channels; blocks are laid out product
// after product.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GroupDev g) {
  pdl_wait();
  pdl_trigger();
  int pi = 0;
#pragma unroll
  for (int i = 1; i < kMaxProb; ++i)
    if (i < g.n_prob && g.prob[i].splits > 1 && static_cast<int>(blockIdx.x) >= g.prob[i].red_begin) pi = i;
  const Prob& p = g.prob[pi];
  if (p.splits <= 1) return;  // only when product 0 is unsplit and owns no blocks
  const int n4 = p.N >> 2;
  const long long i = static_cast<long long>(static_cast<int>(blockIdx.x) - p.red_begin) * blockDim.x + threadIdx.x;
  if (i < 0 || i >= static_cast<long long>(p.M) * n4) return;
  const int m = static_cast<int>(i / n4), n = static_cast<int>(i - static_cast<long long>(m) * n4) * 4;
  const size_t plane = static_cast<size_t>(p.M) * p.N;
  const float* src = p.partial + static_cast<size_t>(m) * p.N + n;
  float4 acc = __ldcg(reinterpret_cast<const float4*>(src));
  for (int z = 1; z < p.splits; ++z) {
    const float4 t = __ldcg(reinterpret_cast<const float4*>(src + z * plane));
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  float a[4] = {acc.x, acc.y, acc.z, acc.w};
  if (p.scale) {
#pragma unroll
    for (int j = 0; j < 4; ++j) a[j] *= __half2float(p.scale[n + j]);
  }
  store4(make_ctx(p), m, n, a);
}

}  // namespace

// ---------------------------------------------------------------------------------- host side
namespace {

using EncodeFn = TensorMapEncodeFn;
inline EncodeFn encode_fn() { return tensor_map_encode_fn(); }

// 2-D fp16 tensor [rows, cols] with row stride ld (elements), boxes of 64 columns x box_rows rows,
// 128-byte swizzle, zero fill outside the tensor.  Encoded maps are kept: a model asks for the same few
// hundred (pointer, shape) combinations on every call.
struct MapKey {
  const void* base;
  int rows, cols, ld, box_rows;  // box_rows < 0: a packed (byte) matrix, box of -box_rows bytes x 128 rows
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    for (int v : {k.rows, k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ static_cast<size_t>(v);
    return h;
  }
};

int make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, cols, ld, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return kOk;
    }
  }
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
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *map);
  return kOk;
}

// Packed weights: 2-D byte tensor [rows, row_bytes], boxes of box_bytes x 128 rows, no swizzle, zero fill outside.
int make_map_packed(CUtensorMap* map, const void* base, int rows, int row_bytes, int box_bytes) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, row_bytes, row_bytes, -box_bytes};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return kOk;
    }
  }
  EncodeFn fn = encode_fn();
  RK_REQUIRE(fn, kCuda, "gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(kBM)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RK_REQUIRE(r == CUDA_SUCCESS, kCuda, "gemm_tc: cuTensorMapEncodeTiled (packed weights) failed with %d (rows=%d row_bytes=%d)",
             static_cast<int>(r), rows, row_bytes);
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *map);
  return kOk;
}

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

int round16(int m) { return ((m + 15) / 16) * 16; }

// Chooses the row-tile width and the K split of every product: the candidate with the smallest estimated
// makespan over the SMs (in units of one K block streamed by one CTA) wins.  Smaller row tiles and K splits
// both make more units; splitting K costs partial-sum traffic and the second kernel, narrower row tiles cost
// re-reads of the weight tile from L2.
struct Plan {
  int Nt = 0, tiles_m = 0, total_units = 0;
  int splits[kMaxProb] = {0}, kbps[kMaxProb] = {0};
  double cost = 1e30;
  bool any_split = false;
};

Plan make_plan_uncached(const LinearArgs* a, int n, size_t scratch_bytes, int sms, int bm);

// Plans depend only on the shapes; a model asks for the same few again and again.
// sms: CTAs (bm == 128) or CTA pairs (bm == 256) that walk the unit list.
Plan make_plan(const LinearArgs* a, int n, size_t scratch_bytes, int sms, int bm) {
  static std::mutex mu;
  static std::unordered_map<std::string, Plan> cache;
  std::string key;
  key.reserve(16 + 8 * static_cast<size_t>(n));
  auto put = [&key](long long v) { key.append(reinterpret_cast<const char*>(&v), sizeof(v)); };
  put(a[0].M); put(n); put(static_cast<long long>(scratch_bytes)); put(sms); put(bm);
  for (int i = 0; i < n; ++i) { put(a[i].N); put(a[i].K); }
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  const Plan p = make_plan_uncached(a, n, scratch_bytes, sms, bm);
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(std::move(key), p);
  return p;
}

Plan make_plan_uncached(const LinearArgs* a, int n, size_t scratch_bytes, int sms, int bm) {
  const int M = a[0].M;
  int nts[3], n_nt = 0;
  if (bm == 2 * kBM) {
    nts[n_nt++] = std::min(256, ((M + 31) / 32) * 32);  // each CTA of a pair stages half of the row tile
  } else {
    nts[n_nt++] = std::min(256, round16(M));
    if (M > 128) nts[n_nt++] = 128;
    if (M > 64) nts[n_nt++] = 64;
  }
  static const int targets[] = {1 << 30, 128, 96, 64, 48, 32, 24, 16, 12, 8, 6, 4};
  Plan best;
  std::vector<double> load(static_cast<size_t>(sms));
  for (int ni = 0; ni < n_nt; ++ni) {
    const int Nt = nts[ni], tiles_m = (M + Nt - 1) / Nt;
    for (int target : targets) {
      Plan p;
      p.Nt = Nt;
      p.tiles_m = tiles_m;
      size_t need = 0;
      for (int i = 0; i < n; ++i) {
        const int kb = (a[i].K + kBK - 1) / kBK;
        int s = std::max(1, std::min((kb + target - 1) / target, 32));
        if (a[i].N % 4 != 0) s = 1;
        p.kbps[i] = (kb + s - 1) / s;
        p.splits[i] = (kb + p.kbps[i] - 1) / p.kbps[i];  // no empty split
        if (p.splits[i] > 1) {
          p.any_split = true;
          need += static_cast<size_t>(p.splits[i]) * M * a[i].N * sizeof(float);
        }
      }
      if (need > scratch_bytes) continue;
      std::fill(load.begin(), load.end(), 0.0);
      int u = 0;
      for (int i = 0; i < n; ++i) {
        const int tiles_n = (a[i].N + bm - 1) / bm;
        const int units = tiles_n * tiles_m * p.splits[i];
        // weight tile from DRAM for the first row tile, from L2 for the others; epilogue cost grows with Nt
        const double epi = (p.splits[i] > 1 ? 2.0 : 1.0) * Nt / 128.0 + 1.5;
        for (int k = 0; k < units; ++k, ++u) {
          const bool first_row_tile = (k % tiles_m) == 0;
          load[static_cast<size_t>(u % sms)] += p.kbps[i] * (first_row_tile ? 1.0 : 0.6) + epi;
        }
      }
      p.total_units = u;
      p.cost = *std::max_element(load.begin(), load.end()) + (p.any_split ? 10.0 : 0.0);
      if (p.cost < best.cost) best = p;
    }
  }
  return best;
}

bool problem_ok(const LinearArgs& a) {
  const int ldx = a.ldx ? a.ldx : a.K;
  if (a.fmt == 1 && (a.K % 16 != 0 || !a.scale)) return false;             // packed rows must be 16-byte multiples
  if (a.fmt == 2 && (a.K % 128 != 0 || !a.scale || !a.zero)) return false;
  return a.fmt >= 0 && a.fmt <= 2 && a.in_act == kActNone && a.K % 8 == 0 && ldx % 8 == 0 && a.M >= 2 && a.N % 4 == 0 &&
         (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0;
}

}  // namespace

bool gemm_tc_supported(const LinearArgs& a) { return problem_ok(a); }

namespace {
thread_local int g_last_max_splits = 0;
}
// Largest K split of the products of this thread's most recent tensor-core launch (1 = no partial sums were used).
int gemm_last_max_splits() { return g_last_max_splits; }

// Up to eight products with the same row count in one launch (plus one reduction launch if any K is split).
// Split-K needs scratch (taken from the first product's args); without it every product runs unsplit.
int gemm_group(cudaStream_t stream, const LinearArgs* a, int n) {
  RK_REQUIRE(a && n >= 1 && n <= kMaxProb, kBadArg, "gemm_group: 1..%d products", kMaxProb);
  for (int i = 0; i < n; ++i) {
    RK_REQUIRE(problem_ok(a[i]), kShape, "gemm_group: unsupported product %d", i);
    RK_REQUIRE(a[i].M == a[0].M, kShape, "gemm_group: all products must share M");
    RK_REQUIRE(a[i].y, kBadArg, "gemm_group: null output");
  }
  const int sms = sm_count();
  // CTA pairs (cta_group::2: each CTA stages half of the activation tile) are opt-in: on the shapes of this model
  // they measured equal to single CTAs (M = 256 .. 2048), so the simpler kernel is the default.
  const int pair_mode = options().gemm_cta_pair;
  static std::mutex mu;
  static int pairs_dev[64] = {0};  // co-resident CTA pairs per device; -1 = cluster launch not available
  int dev = 0;
  RK_CUDA(cudaGetDevice(&dev));
  RK_REQUIRE(dev >= 0 && dev < 64, kBadArg, "gemm_group: device ordinal out of range");
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!pairs_dev[dev]) {
      RK_CUDA(cudaFuncSetAttribute(gemm_group_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024));
      RK_CUDA(cudaFuncSetAttribute(gemm_group_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024));
      RK_CUDA(cudaFuncSetAttribute(gemm_group_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024));
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(static_cast<unsigned>(sms & ~1));
      probe.blockDim = dim3(kThreads);
      probe.dynamicSmemBytes = 200 * 1024;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      probe.attrs = at;
      probe.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, gemm_group_kernel<true, false>, &probe) != cudaSuccess || clusters < 1) {
        cudaGetLastError();
        clusters = -1;
      }
      pairs_dev[dev] = clusters;
    }
  }
  bool quant = false;
  for (int i = 0; i < n; ++i) quant = quant || a[i].fmt != 0;
  const bool pair = pair_mode == 1 && pairs_dev[dev] > 0 && !quant;
  const int walkers = pair ? std::min(pairs_dev[dev], sms / 2) : sms;
  const int bm = pair ? 2 * kBM : kBM;
  const Plan plan = make_plan(a, n, a[0].scratch ? a[0].scratch_bytes : 0, walkers, bm);
  RK_REQUIRE(plan.Nt > 0 && plan.total_units > 0, kShape, "gemm_group: no launch plan");
  g_last_max_splits = *std::max_element(plan.splits, plan.splits + n);

  static MapPack maps;  // filled and consumed under the lock: kernel parameters are copied at launch
  GroupDev g = {};
  g.n_prob = n;
  g.bm = bm;
  g.Nt = plan.Nt;
  g.tiles_m = plan.tiles_m;
  g.total_units = plan.total_units;
  // shared memory: as many stages (weight tile + activation tile) as fit beside the epilogue tile.  (Separate rings
  // with their own barriers and producer threads measured slower: 0.53 instead of 0.38 us per K block at 128 rows.)
  const int x_rows = pair ? g.Nt / 2 : g.Nt;
  const size_t x_bytes = static_cast<size_t>(x_rows) * 128, w_bytes = static_cast<size_t>(kBM) * 128;
  const size_t budget = 224 * 1024 - kEpiBytes;
  const size_t stage_bytes = x_bytes + w_bytes + (quant ? kRawBytes : 0);
  g.stages = static_cast<int>(std::min<size_t>(kMaxStages, budget / stage_bytes));
  const size_t smem = stage_bytes * g.stages + kEpiBytes + 1024;
  g.w_dynamic = 0;
  for (int i = 0; i < n; ++i) g.w_dynamic |= a[i].w_dynamic ? 1 : 0;
  g.timeout = timeout_word_or_null();

  std::lock_guard<std::mutex> lock(mu);
  float* scratch = a[0].scratch;
  int unit = 0, red = 0;
  for (int i = 0; i < n; ++i) {
    Prob& p = g.prob[i];
    p.M = a[i].M; p.N = a[i].N; p.K = a[i].K; p.epi = a[i].epi; p.y = a[i].y; p.scale = a[i].out_scale;
    p.fmt = a[i].fmt; p.qscale = a[i].scale; p.qzero = a[i].zero;
    if (a[i].fmt == 1 && !p.scale) p.scale = a[i].scale;  // W8A16: one scale per output channel, applied to the accumulator
    p.v = a[i].ea.v; p.v_first = a[i].ea.v_first; p.v0 = a[i].ea.v0;
    p.tiles_n = (a[i].N + bm - 1) / bm;
    p.splits = plan.splits[i];
    p.kb_per_split = plan.kbps[i];
    p.unit_begin = unit;
    unit += p.tiles_n * g.tiles_m * p.splits;
    p.red_begin = red;
    p.partial = nullptr;
    if (p.splits > 1) {
      p.partial = scratch;
      scratch += static_cast<size_t>(p.splits) * p.M * p.N;
      red += static_cast<int>((static_cast<long long>(p.M) * (p.N / 4) + 255) / 256);
    }
    int s;
    if (a[i].fmt == 0) s = make_map(&maps.w[i], a[i].w, a[i].N, a[i].K, a[i].K, kBM);
    else if (a[i].fmt == 1) s = make_map_packed(&maps.w[i], a[i].w, a[i].N, a[i].K, kBK);
    else s = make_map_packed(&maps.w[i], a[i].w, a[i].N, a[i].K / 2, kBK / 2);
    if (s != kOk) return s;
    s = make_map(&maps.x[i], a[i].x, a[i].M, a[i].K, a[i].ldx ? a[i].ldx : a[i].K, x_rows);
    if (s != kOk) return s;
  }
  for (int i = n; i < kMaxProb; ++i) {
    maps.w[i] = maps.w[0];
    maps.x[i] = maps.x[0];
  }
  g.red_blocks = red;
  if (pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * std::min(walkers, g.total_units)));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 2;
    RK_CUDA(cudaLaunchKernelEx(&cfg, gemm_group_kernel<true, false>, maps, g));
  } else if (quant) {
    const dim3 grid(static_cast<unsigned>(std::min(walkers, g.total_units))), block(kThreads + kDequantThreads);
    RK_CUDA(launch_pdl(gemm_group_kernel<false, true>, grid, block, smem, stream, maps, g));
  } else {
    const dim3 grid(static_cast<unsigned>(std::min(walkers, g.total_units))), block(kThreads);
    RK_CUDA(launch_pdl(gemm_group_kernel<false, false>, grid, block, smem, stream, maps, g));
  }
  RK_LAUNCH_CHECK("gemm_group launch");
  if (red > 0) {
    RK_CUDA(launch_pdl(splitk_reduce_kernel, dim3(static_cast<unsigned>(red)), dim3(256), 0, stream, g));
    RK_LAUNCH_CHECK("splitk_reduce launch");
  }
  return kOk;
}

int gemm_tc(cudaStream_t stream, const LinearArgs& a) { return gemm_group(stream, &a, 1); }

// ---------------------------------------------------------------------------------------------
// Split-K GEMM for callers that must not allocate: the fp32 partial sums go to a fixed device array
// that is part of the loaded library image (every GPU that loads the library holds these 16 MiB
// until the process exits).
constexpr size_t kStaticScratchFloats = static_cast<size_t>(4) << 20;  // 16 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

int gemm_tc_static_scratch(cudaStream_t stream, const LinearArgs& a) {
  RK_REQUIRE(a.M > 4 && gemm_tc_supported(a), kShape, "linear (static scratch): needs more than 4 rows, fp16 weights, K %% 8 == 0");
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

}  // namespace rk
