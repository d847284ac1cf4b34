// Scalar weight-streaming GEMV (M <= 4; fp16, W8A16 or W4A16 weights, dequantised in registers; since gemv_mma.cu the
// route of one-row launches that are small or whose shapes that kernel refuses -- linear.cu decides) with the
// weights staged through shared memory by the bulk-copy engine: every warp owns a ring of kSlots buffers, one lane requests the next piece of
// the warp's contiguous weight stream with cp.async.bulk (completion on an mbarrier), the warp
// consumes pieces in order with 128-bit shared-memory loads and re-arms the slot it has just read.
// Two 4 KiB slots per warp (128 KiB per CTA of 16 warps) are in flight without holding registers, which is
// what it takes to keep HBM3e busy from 148 SMs; the first kSlots pieces are requested before the
// programmatic-dependency wait, so a kernel's weight stream starts while its predecessor drains.
// Same arithmetic and rounding as the register-staged kernel in linear.cu.
#include <algorithm>

#include "gemv.h"
#include "kernels.h"

namespace rk {
namespace {

constexpr int kMaxWarps = 16;
constexpr int kMaxSlots = 6;
constexpr int kPieceCap = 4096;  // bytes

// One 16-byte weight chunk (8 halves) against 8 fp32 activations from shared memory.
__device__ __forceinline__ void fma_chunk(const uint4& q, const float* x, float& a0, float& a1) {
  const float4 xa = *reinterpret_cast<const float4*>(x);
  const float4 xb = *reinterpret_cast<const float4*>(x + 4);
  const float2 w0 = h2f2(q.x), w1 = h2f2(q.y), w2 = h2f2(q.z), w3 = h2f2(q.w);
  a0 = fmaf(xa.x, w0.x, a0); a1 = fmaf(xa.y, w0.y, a1);
  a0 = fmaf(xa.z, w1.x, a0); a1 = fmaf(xa.w, w1.y, a1);
  a0 = fmaf(xb.x, w2.x, a0); a1 = fmaf(xb.y, w2.y, a1);
  a0 = fmaf(xb.z, w3.x, a0); a1 = fmaf(xb.w, w3.y, a1);
}

// kQuant: some problem of the launch has int8 / int4 weights (the fp16-only instantiation carries no dequant code).
// One CTA per SM by design (the rings take most of the shared memory): saying so in the launch bounds lets the compiler
// spend registers on keeping more weight chunks in flight per lane (2.94 -> 2.86 ms per 7.2B decode step).
template <int kM, int kW, bool kQuant>
__global__ void __launch_bounds__(kW * 32, 1) gemv_tma_kernel(const GemvBatch p, int x_bytes, int n_slots, int slot_stride) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t bars[kW][kMaxSlots];
  __shared__ float red_scratch[kW];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSeg; ++i)
    if (i < p.n_seg && static_cast<int>(blockIdx.x) >= p.seg[i].cta_begin) s = i;
  const GemvSeg& sg = p.seg[s];
  const int row0 = (blockIdx.x - sg.cta_begin) * sg.rows_per_cta;
  const int rows_end = min(sg.N, row0 + sg.rows_per_cta);
  // the CTA's rows are shared out over its warps as evenly as they go (the first `rem` warps take one more)
  const int rows_here = max(rows_end - row0, 0);
  const int base = rows_here / kW, rem = rows_here - base * kW;
  const int r_begin = row0 + warp * base + min(warp, rem);
  const int r_end = r_begin + base + (warp < rem ? 1 : 0);
  const int parts = sg.parts, piece = sg.piece_bytes;
  const int total = r_end > r_begin ? (r_end - r_begin) * parts : 0;
  const int K = sg.K;
  const int fmt = kQuant ? sg.fmt : 0;
  const int elems = fmt == 0 ? 8 : fmt == 1 ? 16 : 32;  // weights per 16-byte chunk
  const char* stream = static_cast<const char*>(sg.w) + static_cast<size_t>(r_begin) * parts * piece;

  float* xs = reinterpret_cast<float*>(smem_raw);  // activations, fp32, input activation applied
  unsigned char* ring = smem_raw + x_bytes + static_cast<size_t>(warp) * n_slots * slot_stride;
  // pieces of a row are visited in a per-warp rotated order so that the warps' streams do not march
  // through the same low address bits (and hence the same memory channels) in lock step
  const int rot = (blockIdx.x * kW + warp) % parts;

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kMaxSlots; ++i) mbar_init(smem_u32(&bars[warp][i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // producer state (lane 0): next piece to request, as (row, rotated part, slot)
  int q_row = 0, q_pp = rot, q_slot = 0, q_left = total;
  auto issue = [&]() {
    if (lane == 0) {
      const uint32_t bar = smem_u32(&bars[warp][q_slot]);
      mbar_expect_tx(bar, piece);
      bulk_g2s(smem_u32(ring + q_slot * slot_stride), stream + (static_cast<size_t>(q_row) * parts + q_pp) * piece, piece, bar);
    }
    --q_left;
    if (++q_slot == n_slots) q_slot = 0;
    if (++q_pp == parts) q_pp = 0;
    if (q_pp == rot) ++q_row;
  };
  // weights do not depend on the previous kernel: fill the ring before waiting for it
  for (int i = 0; i < n_slots && q_left > 0; ++i) issue();

  LnPrefetch pf;
  if (sg.ln_w) ln_prefetch<kW * 32>(sg, pf);
  pdl_wait();
  pdl_trigger();  // after the wait: at most this kernel and its successor are ever in flight together
  const bool first_cta = static_cast<int>(blockIdx.x) == sg.cta_begin;
  if (first_cta && sg.copy_src)
    for (int i = threadIdx.x; i < (sg.copy_n >> 1); i += kW * 32)
      reinterpret_cast<__half2*>(sg.copy_dst)[i] = reinterpret_cast<const __half2*>(sg.copy_src)[i];
  if (sg.ln_w)
    stage_ln_mix<kM, kW * 32>(sg, [&](int m, int k, float2 v) { *reinterpret_cast<float2*>(xs + static_cast<size_t>(m) * K + k) = v; },
                              red_scratch, first_cta, pf);
  else stage_activations<kM, kW * 32>(sg, nullptr, xs);
  __syncthreads();

  const int chunks = piece >> 4;  // 16-byte chunks per piece
  float acc0[kM], acc1[kM];
#pragma unroll
  for (int m = 0; m < kM; ++m) acc0[m] = acc1[m] = 0.f;
  int slot = 0, phase = 0, pp = rot, part = 0, row = r_begin;
  // Quantisation parameters are requested ahead of their use (read where they are used they cost a cache-miss round
  // trip per piece): W8A16 -- the row's scale when the row begins; W4A16 -- lane g holds (scale, zero) of group g
  // (and g + 32) of a piece, loaded one piece ahead, and hands them out by shuffle.
  float row_scale = 1.f;
  uint32_t sz_cur[2] = {0u, 0u}, sz_next[2] = {0u, 0u};
  const int groups = kQuant && fmt == 2 ? piece >> 6 : 0;  // 128 weights = 64 bytes per group
  auto load_sz = [&](int r, int part_idx, uint32_t (&dst)[2]) {
    const size_t g0 = static_cast<size_t>(r) * (K >> 7) + static_cast<size_t>(part_idx) * groups;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int g = lane + 32 * i;
      if (g < groups) {
        const __half2 pk = __halves2half2(sg.scale[g0 + g], sg.zero[g0 + g]);
        dst[i] = *reinterpret_cast<const uint32_t*>(&pk);
      }
    }
  };
  if (kQuant && total > 0) {
    if (fmt == 1) row_scale = __half2float(sg.scale[row]);
    if (fmt == 2) load_sz(row, pp, sz_cur);
  }
  for (int pc = 0; pc < total; ++pc) {
    if (kQuant && fmt == 2 && pc + 1 < total) {  // the piece after this one: next part of the row, or the next row
      int npp = pp + 1 == parts ? 0 : pp + 1;
      load_sz(part + 1 == parts ? row + 1 : row, npp, sz_next);
    }
    const uint32_t bar = smem_u32(&bars[warp][slot]);
    if (!mbar_try_wait(bar, phase) && !mbar_wait(bar, phase)) {
      if (lane == 0 && p.timeout) atomicOr(p.timeout, kTimeoutGemv);
      return;
    }
    const uint4* wsm = reinterpret_cast<const uint4*>(ring + slot * slot_stride) + lane;
    if (!kQuant || fmt == 0) {
      const float* xk = xs + pp * (piece >> 1) + lane * 8;
      if (piece == kPieceCap) {
        uint4 q[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) q[it] = wsm[it * 32];
#pragma unroll
        for (int it = 0; it < 8; ++it)
#pragma unroll
          for (int m = 0; m < kM; ++m) fma_chunk(q[it], xk + m * K + it * 256, acc0[m], acc1[m]);
      } else {
        for (int c = lane; c < chunks; c += 32) {
          const uint4 q = wsm[c - lane];
#pragma unroll
          for (int m = 0; m < kM; ++m) fma_chunk(q, xk + m * K + (c - lane) * 8, acc0[m], acc1[m]);
        }
      }
    } else {
      // int8 / int4, dequantised in registers (exact integer-valued floats for W8A16, half((q - zero) * scale) for
      // W4A16) and multiplied with fp32 activations from shared memory.  A lane takes 4-byte words of the piece
      // (word = lane + 32 j), so that consecutive lanes read consecutive 16 / 32 bytes of activations: no bank
      // conflicts, which 16-byte weight chunks per lane would cause on the activation side.
      const uint32_t* wsm32 = reinterpret_cast<const uint32_t*>(ring + slot * slot_stride);
      const int words = piece >> 2;
      if (fmt == 1) {
        const int k_piece = pp * piece;  // one byte per weight
        const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll 4
        for (int wd = lane; wd < words; wd += 32) {
          const uint32_t t = wsm32[wd] ^ 0x80808080u;
          uint32_t h01 = __byte_perm(t, 0x64646464u, 0x4140);
          uint32_t h23 = __byte_perm(t, 0x64646464u, 0x4342);
          const float2 w01 = __half22float2(__hsub2(*reinterpret_cast<__half2*>(&h01), bias));
          const float2 w23 = __half22float2(__hsub2(*reinterpret_cast<__half2*>(&h23), bias));
#pragma unroll
          for (int m = 0; m < kM; ++m) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + m * K + k_piece + wd * 4);
            acc0[m] = fmaf(xv.x, w01.x, acc0[m]); acc1[m] = fmaf(xv.y, w01.y, acc1[m]);
            acc0[m] = fmaf(xv.z, w23.x, acc0[m]); acc1[m] = fmaf(xv.w, w23.y, acc1[m]);
          }
        }
      } else {
        const int k_piece = pp * piece * 2;  // two weights per byte
#pragma unroll 2
        for (int w0 = 0; w0 < words; w0 += 32) {  // uniform trip count: every lane takes part in the shuffle
          const int wd = w0 + lane;
          const int gi = wd >> 4;                  // 16 words = 128 weights = one group
          const uint32_t pk = __shfl_sync(0xffffffffu, (w0 >> 9) ? sz_cur[1] : sz_cur[0], gi & 31);
          if (wd >= words) continue;
          const __half2 sz = *reinterpret_cast<const __half2*>(&pk);
          const uint32_t u = wsm32[wd];
          const int k = k_piece + wd * 8;
          const __half2 zb = __float2half2_rn(1024.f + __high2float(sz));
          const __half2 s2 = __half2half2(__low2half(sz));
          float wf[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // nibble n of the word is element n: a shift and one mask give elements (j, j + 4)
            uint32_t pair = ((u >> (4 * j)) & 0x000f000fu) | 0x64006400u;  // 1024 + q in both halves
            const float2 f = __half22float2(__hmul2(__hsub2(*reinterpret_cast<__half2*>(&pair), zb), s2));
            wf[j] = f.x;
            wf[j + 4] = f.y;
          }
#pragma unroll
          for (int m = 0; m < kM; ++m) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + m * K + k);
            const float4 xb = *reinterpret_cast<const float4*>(xs + m * K + k + 4);
            acc0[m] = fmaf(xa.x, wf[0], acc0[m]); acc1[m] = fmaf(xa.y, wf[1], acc1[m]);
            acc0[m] = fmaf(xa.z, wf[2], acc0[m]); acc1[m] = fmaf(xa.w, wf[3], acc1[m]);
            acc0[m] = fmaf(xb.x, wf[4], acc0[m]); acc1[m] = fmaf(xb.y, wf[5], acc1[m]);
            acc0[m] = fmaf(xb.z, wf[6], acc0[m]); acc1[m] = fmaf(xb.w, wf[7], acc1[m]);
          }
        }
      }
    }
    __syncwarp();  // every lane has read the slot: it may be overwritten
    if (q_left > 0) issue();
    if (kQuant && fmt == 2) { sz_cur[0] = sz_next[0]; sz_cur[1] = sz_next[1]; }
    if (++slot == n_slots) { slot = 0; phase ^= 1; }
    if (++pp == parts) pp = 0;
    if (++part == parts) {
      part = 0;
#pragma unroll
      for (int m = 0; m < kM; ++m) {
        float a = warp_sum(acc0[m] + acc1[m]);
        if (kQuant && fmt == 1) a *= row_scale;  // W8A16: one scale per output channel
        if (lane == 0) store_result(sg, m, row, a);
        acc0[m] = acc1[m] = 0.f;
      }
      ++row;
      if (kQuant && fmt == 1 && pc + 1 < total) row_scale = __half2float(sg.scale[row]);
    }
  }
}

}  // namespace

// Fills cta_begin / rows_per_cta / parts / piece_bytes for the bulk-copy kernel.  Returns false when
// a problem does not fit it (non-fp16 weights, or a row that cannot be cut into 16-byte multiples).
bool gemv_tma_plan(GemvBatch& b, int M, size_t* smem_bytes, int* grid, int* n_slots, int* slot_stride, int* n_warps) {
  size_t x_bytes = 0;
  double total_bytes = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    GemvSeg& g = b.seg[i];
    if (g.fmt == 2 && g.K % 128 != 0) return false;
    const int row_bytes = g.fmt == 0 ? g.K * 2 : g.fmt == 1 ? g.K : g.K / 2;
    if (row_bytes % 16 != 0) return false;
    int parts = (row_bytes + kPieceCap - 1) / kPieceCap;
    const int unit = g.fmt == 2 ? 64 : 16;  // W4A16: a piece holds whole quantisation groups (64 bytes each)
    while (parts <= 64 && (row_bytes % (parts * unit) != 0)) ++parts;
    if (parts > 64) return false;
    g.parts = parts;
    g.piece_bytes = row_bytes / parts;
    x_bytes = std::max(x_bytes, static_cast<size_t>(M) * g.K * 4);
    total_bytes += static_cast<double>(g.N) * row_bytes;
  }
  x_bytes = (x_bytes + 127) & ~static_cast<size_t>(127);
  const int cap = kPieceCap;
  // measured best on B200: one CTA of 16 warps per SM, two 4 KiB slots per warp (128 KiB in flight)
  int slots = 2, kWarps = 16;
  if (x_bytes + static_cast<size_t>(kWarps) * slots * cap > 200 * 1024) {
    kWarps = 8;  // very large activation rows: fewer warps, whatever ring depth still fits
    slots = static_cast<int>((200 * 1024 - x_bytes) / (static_cast<size_t>(kWarps) * cap));
    slots = std::min(slots, kMaxSlots);
    if (slots < 2) return false;
  }
  for (int i = 0; i < b.n_seg; ++i) {
    GemvSeg& g = b.seg[i];
    const int row_bytes = g.fmt == 0 ? g.K * 2 : g.fmt == 1 ? g.K : g.K / 2;
    int parts = (row_bytes + cap - 1) / cap;
    const int unit = g.fmt == 2 ? 64 : 16;
    while (parts <= 256 && (row_bytes % (parts * unit) != 0)) ++parts;
    if (parts > 256) return false;
    g.parts = parts;
    g.piece_bytes = row_bytes / parts;
  }
  const size_t smem = x_bytes + static_cast<size_t>(kWarps) * slots * cap;
  // CTAs are shared out by weight bytes: every problem starts with its rounded-down share (at least one CTA), the
  // rest go one at a time to whichever problem has the most bytes per CTA, so that all SMs finish together.  (Rows
  // per CTA need not be a multiple of the warp count: 4096 rows on 148 SMs are 28 rows each, not 32 on 128 SMs.)
  const int budget = 148;
  int n_cta[kMaxSeg];
  int used = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    const GemvSeg& g = b.seg[i];
    const double share = static_cast<double>(g.N) * g.parts * g.piece_bytes / total_bytes;
    n_cta[i] = std::max(1, std::min(g.N, static_cast<int>(share * budget)));
    used += n_cta[i];
  }
  while (used < budget) {
    int best = -1;
    double worst = 0;
    for (int i = 0; i < b.n_seg; ++i) {
      const GemvSeg& g = b.seg[i];
      if (n_cta[i] >= g.N) continue;
      const double per = static_cast<double>((g.N + n_cta[i] - 1) / n_cta[i]) * g.parts * g.piece_bytes;
      if (per > worst) { worst = per; best = i; }
    }
    if (best < 0) break;
    ++n_cta[best];
    ++used;
  }
  // Small launches (a few MB: narrow models) are latency-bound, not bandwidth-bound: there fewer, fatter CTAs measured
  // faster, so every warp of a problem gets the same whole number of rows as if all CTAs were used.
  const bool small = total_bytes < 8.0 * 1024 * 1024;
  int cta = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    GemvSeg& g = b.seg[i];
    if (small) {
      const double share = static_cast<double>(g.N) * g.parts * g.piece_bytes / total_bytes;
      const int n = std::max(1, static_cast<int>(share * budget + 0.5));
      g.rows_per_cta = std::max(1, (g.N + n * kWarps - 1) / (n * kWarps)) * kWarps;
    } else {
      g.rows_per_cta = (g.N + n_cta[i] - 1) / n_cta[i];
    }
    g.cta_begin = cta;
    cta += (g.N + g.rows_per_cta - 1) / g.rows_per_cta;
  }
  *smem_bytes = smem;
  *grid = cta;
  *n_slots = slots;
  *slot_stride = cap;
  *n_warps = kWarps;
  return true;
}

// Whether M rows of K fp32 activations fit beside the smallest ring (8 warps, two 4 KiB slots) the planner accepts.
bool gemv_tma_fits(int M, int K) {
  const size_t x_bytes = (static_cast<size_t>(M) * K * 4 + 127) & ~static_cast<size_t>(127);
  return x_bytes + static_cast<size_t>(8) * 2 * kPieceCap <= 200 * 1024;
}

int gemv_tma_launch(cudaStream_t stream, const GemvBatch& b, int M, size_t smem_bytes, int grid, int n_slots, int slot_stride,
                    int kWarps) {
  const int x_bytes = static_cast<int>(smem_bytes - static_cast<size_t>(kWarps) * n_slots * slot_stride);
  auto launch = [&](auto kernel) -> int {
    RK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RK_CUDA(launch_pdl(kernel, dim3(grid), dim3(kWarps * 32), smem_bytes, stream, b, x_bytes, n_slots, slot_stride));
    return kOk;
  };
  bool quant = false;
  for (int i = 0; i < b.n_seg; ++i) quant = quant || b.seg[i].fmt != 0;
  int s;
  if (!quant) {
    if (kWarps == 16) {
      switch (M) {
        case 1: s = launch(gemv_tma_kernel<1, 16, false>); break;
        case 2: s = launch(gemv_tma_kernel<2, 16, false>); break;
        case 3: s = launch(gemv_tma_kernel<3, 16, false>); break;
        default: s = launch(gemv_tma_kernel<4, 16, false>); break;
      }
    } else {
      switch (M) {
        case 1: s = launch(gemv_tma_kernel<1, 8, false>); break;
        case 2: s = launch(gemv_tma_kernel<2, 8, false>); break;
        case 3: s = launch(gemv_tma_kernel<3, 8, false>); break;
        default: s = launch(gemv_tma_kernel<4, 8, false>); break;
      }
    }
  } else if (kWarps == 16) {
    switch (M) {
      case 1: s = launch(gemv_tma_kernel<1, 16, true>); break;
      case 2: s = launch(gemv_tma_kernel<2, 16, true>); break;
      case 3: s = launch(gemv_tma_kernel<3, 16, true>); break;
      default: s = launch(gemv_tma_kernel<4, 16, true>); break;
    }
  } else {
    switch (M) {
      case 1: s = launch(gemv_tma_kernel<1, 8, true>); break;
      case 2: s = launch(gemv_tma_kernel<2, 8, true>); break;
      case 3: s = launch(gemv_tma_kernel<3, 8, true>); break;
      default: s = launch(gemv_tma_kernel<4, 8, true>); break;
    }
  }
  if (s != kOk) return s;
  RK_LAUNCH_CHECK("gemv_tma launch");
  return kOk;
}

}  // namespace rk
