// Weight-streaming linear layers for 1..4 rows of activations on the warp-level tensor-core instruction
// (mma.sync m16n8k16, fp32 accumulation): 16 output channels of weights are the M side of the instruction, the rows
// of activations (at most 4 of its 8 columns are used) the N side.  This is the kernel of the decode step: every
// linear layer of a 7.2B step at 1..4 sequences runs here (fp16: 5.9 TB/s on a 134 MB matrix, 6.9 TB/s on the 537 MB
// lm-head at one row); linear.cu says which launches go to the scalar kernel of gemv_tma.cu instead (one row of
// fp16 / W8A16 in small launches).  What it buys over one fused multiply-add per weight and row: int8 / int4 weights
// are turned into halves with a few half2 operations per 32-bit word ONCE for all rows, the multiply-adds cost one
// instruction per 16 x 16 weights, the activations are halves (one 16-byte load per 16 bytes of fp16 weights), and the
// 16 warps of a CTA work on the same weight rows at the same time.  The arithmetic is exact in the same sense as the
// scalar kernels: products of halves accumulated in fp32, int8 as exact integers with the channel scale on the sum,
// int4 as half((q - zero) * scale).
//
// Data movement: one 16-warp CTA per SM owns a contiguous range of output channels (a multiple of 4) and walks it in
// tiles of 16 or 32 channels; the K extent of a tile is cut into boxes of 128 bytes, box b going to warp b mod 16.  A
// box (16 or 32 channels x 128 bytes, 2 or 4 KiB) is fetched by ONE 2-D tensor copy with the 128-byte swizzle into the
// warp's own ring (8 KiB per warp, 128 KiB per CTA in flight; completion on an mbarrier), so a lane's 16-byte reads of
// the rows g and g + 8 of the fragment layout are free of bank conflicts; a tile with fewer valid channels is fetched
// as boxes of 4 channels, so no byte of another CTA's range is read.  The activations are staged once per CTA as
// halves in the order the fragments want them (a lane's operands of one or two instructions are 16 contiguous bytes).
// At the end of a tile the warps leave their partial sums in shared memory and one warp adds them in warp order:
// results do not depend on timing.  W4A16: the scales and zeros of a box travel with it (4-byte asynchronous copies
// into the slot, counted by the same mbarrier).  The ring fill is issued before the programmatic-dependency wait.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "gemv.h"
#include "kernels.h"
#include "tensormap.h"

namespace rk {
namespace {

constexpr int kWarps = 16;
constexpr int kSlotBytes = 2048;  // 16 channels x 128 bytes
constexpr int kMaxSlots = 4;
constexpr int kPartBufs = 4;                              // tiles whose partial sums may be pending at a time
constexpr int kPartialBytes = kPartBufs * kWarps * 256;   // per buffer and warp: 16 channels x 4 rows of fp32
constexpr int kSzBytes = kWarps * kMaxSlots * 128;        // W4A16: per slot 16 channels x (2 scales, 2 zeros)
constexpr int kSmemLimit = 224 * 1024;

struct MmaMaps {
  CUtensorMap full[kMaxSeg];  // boxes of 16 channels
  CUtensorMap quad[kMaxSeg];  // boxes of 4 channels (ragged last tile of a CTA's range)
  CUtensorMap tall[kMaxSeg];  // boxes of 32 channels (tiles of two blocks)
};

__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// The same for the lanes with `on` set; the others keep what the registers held (columns of the instruction beyond
// the rows of activations may hold anything: their sums are never stored) and cost no shared-memory cycle.
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t addr, uint32_t on) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %5, 0;\n\t@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
               : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
               : "r"(addr), "r"(on));
}
// D += A B with A 16 x 16 (weights: channels x k), B 16 x 8 (activations: k x rows), fp32 accumulators.
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mbar_arrive_cta(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// (a & b) | c in one instruction.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// Where the 16-byte block j (activations 8j .. 8j+7 of a row) lives in shared memory, in 16-byte units.  A box of
// weights covers 8 << fmt blocks; lane t of a fragment row reads the weight chunks 2t and 2t+1 of the box, and for a
// fixed (chunk parity, block of the chunk) the four lanes t read four consecutive blocks.
__device__ __forceinline__ int act_pos(int fmt, int j) {
  const int r = j & ((8 << fmt) - 1);
  const int c = r >> fmt, s = r & ((1 << fmt) - 1);
  return (j - r) + ((((c & 1) << fmt) + s) << 2) + (c >> 1);
}
// W4A16: nibble n of a 32-bit word is element n and one mask yields the elements (n, n + 4) as a half2, so a block is
// stored as x0 x4 x1 x5 x2 x6 x3 x7.
__device__ __forceinline__ int act_slot(int fmt, int e) { return fmt == 2 ? ((e & 3) << 1) + (e >> 2) : e; }

// Bounded wait of a whole warp on an mbarrier phase.
__device__ __forceinline__ bool wait_phase(uint32_t bar, uint32_t parity) { return mbar_try_wait(bar, parity) || mbar_wait(bar, parity); }

// kBlk: 16-channel blocks per tile.  Two (tiles of 32 channels, 4 KiB ring slots) halve the per-box bookkeeping of the
// quantised formats, which are bound by instruction issue; the planner uses it where the activations leave room.
template <int kM, bool kQuant, int kBlk>
__global__ void __launch_bounds__(kWarps * 32, 1)
    gemv_mma_kernel(const __grid_constant__ MmaMaps maps, const GemvBatch p, int n_slots, int x_pitch) {
  constexpr int kTileRows = 16 * kBlk;
  constexpr int kSlot = kSlotBytes * kBlk;          // bytes of a ring slot
  constexpr int kSzSlot = 128 * kBlk;               // W4A16: per slot and channel 2 scales + 2 zeros
  constexpr int kPartWarp = 64 * kBlk;              // floats a warp leaves per tile: kTileRows channels x 4 rows
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t bars[kWarps][kMaxSlots];  // a box (and its quantisation parameters) has landed
  __shared__ __align__(8) uint64_t part_full[kPartBufs];     // all warps have left their partial sums of a tile
  __shared__ __align__(8) uint64_t part_free[kPartBufs];     // ... and the adding warp has read them
  __shared__ float red_scratch[kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSeg; ++i)
    if (i < p.n_seg && static_cast<int>(blockIdx.x) >= p.seg[i].cta_begin) s = i;
  const GemvSeg& sg = p.seg[s];
  const int row0 = (blockIdx.x - sg.cta_begin) * sg.rows_per_cta;
  const int rows_end = min(sg.N, row0 + sg.rows_per_cta);
  const int n_tiles = rows_end > row0 ? (rows_end - row0 + kTileRows - 1) / kTileRows : 0;
  const int K = sg.K;
  const int fmt = kQuant ? sg.fmt : 0;
  const int KB = (fmt == 0 ? K * 2 : fmt == 1 ? K : K >> 1) >> 7;  // 128-byte boxes along a weight row
  const bool w4 = kQuant && fmt == 2;

  const uint32_t dyn = smem_u32(smem_dyn);
  const uint32_t base = (dyn + 1023u) & ~1023u;  // the swizzle pattern is a function of the address: slots at 1 KiB
  const uint32_t ring = base + warp * n_slots * kSlot;
  const uint32_t part = base + kWarps * n_slots * kSlot;
  // (fp16-only launches meet at a CTA barrier per tile: two buffers of partial sums are enough, and there are no
  // quantisation parameters to stage -- the room goes to the activations, so that more shapes fit tiles of 32 channels)
  constexpr int kBufs = kQuant ? kPartBufs : 2;
  constexpr uint32_t kPartBytes = kBufs * kWarps * 256 * kBlk;
  const uint32_t szs = part + kPartBytes + warp * kMaxSlots * kSzSlot;
  const uint32_t xs = part + kPartBytes + (kQuant ? kSzBytes * kBlk : 0);
  unsigned char* xs_ptr = smem_dyn + (xs - dyn);

  if (lane == 0) {
    // W4A16: a slot is complete when the box has landed (one arrival with the byte count) and every lane's copies of
    // quantisation parameters have (32 arrivals)
#pragma unroll
    for (int i = 0; i < kMaxSlots; ++i) mbar_init(smem_u32(&bars[warp][i]), w4 ? 33 : 1);
    if (warp == 0) {
#pragma unroll
      for (int i = 0; i < kPartBufs; ++i) {
        mbar_init(smem_u32(&part_full[i]), kWarps);
        mbar_init(smem_u32(&part_free[i]), 1);
      }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // A warp's boxes in the order it visits them: box kb of tile t, kb = warp, warp + 16, ... over the flattened
  // (tile, box) sequence of the CTA.
  auto advance = [&](int& tile, int& kb) {
    kb += kWarps;
    while (kb >= KB && tile < n_tiles) { kb -= KB; ++tile; }
  };
  const int groups = K >> 7;
  int q_tile = 0, q_kb = warp - kWarps, q_slot = 0;
  advance(q_tile, q_kb);
  auto issue = [&]() {
    const int r = row0 + q_tile * kTileRows;
    const uint32_t bar = smem_u32(&bars[warp][q_slot]);
    if (lane == 0) {
      const int valid = min(kTileRows, rows_end - r);
      const uint32_t dst = ring + q_slot * kSlot;
      mbar_expect_tx(bar, valid << 7);
      if (valid == kTileRows) {
        tma_box(dst, kBlk == 2 ? &maps.tall[s] : &maps.full[s], bar, q_kb << 7, r);
      } else {
        for (int b = 0; b < (valid >> 2); ++b) tma_box(dst + (b << 9), &maps.quad[s], bar, q_kb << 7, r + (b << 2));
      }
    }
    if (w4) {  // lane = 2 * channel + (0: the scales, 1: the zeros) of the box's two groups, 4 bytes
#pragma unroll
      for (int b = 0; b < kBlk; ++b) {
        const int row = min(r + 16 * b + (lane >> 1), sg.N - 1);
        const half* src = ((lane & 1) ? sg.zero : sg.scale) + row * groups + (q_kb << 1);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(szs + q_slot * kSzSlot + (b << 7) + (lane << 2)), "l"(src) : "memory");
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
    }
    if (++q_slot == n_slots) q_slot = 0;
    advance(q_tile, q_kb);
  };
  // weights do not depend on the previous kernel: fill the ring before waiting for it
  for (int i = 0; i < n_slots && q_tile < n_tiles; ++i) issue();

  LnPrefetch pf;
  if (sg.ln_w) ln_prefetch<kWarps * 32>(sg, pf);
  pdl_wait();
  pdl_trigger();  // after the wait: at most this kernel and its successor are ever in flight together
  const bool first_cta = static_cast<int>(blockIdx.x) == sg.cta_begin;
  if (first_cta && sg.copy_src)
    for (int i = threadIdx.x; i < (sg.copy_n >> 1); i += kWarps * 32)
      reinterpret_cast<__half2*>(sg.copy_dst)[i] = reinterpret_cast<const __half2*>(sg.copy_src)[i];
  if (sg.ln_w) {
    stage_ln_mix<kM, kWarps * 32>(
        sg,
        [&](int m, int k, float2 v) {
          half* blk = reinterpret_cast<half*>(xs_ptr + m * x_pitch + (act_pos(fmt, k >> 3) << 4));
          blk[act_slot(fmt, k & 7)] = __float2half_rn(v.x);
          blk[act_slot(fmt, (k & 7) + 1)] = __float2half_rn(v.y);
        },
        red_scratch, first_cta, pf);
  } else {
    const int n_blk = K >> 3;
    for (int i = threadIdx.x; i < kM * n_blk; i += kWarps * 32) {
      const int m = i / n_blk, j = i - m * n_blk;
      uint4 q = *reinterpret_cast<const uint4*>(sg.x + static_cast<size_t>(m) * sg.ldx + j * 8);
      if (w4)
        q = make_uint4(__byte_perm(q.x, q.z, 0x5410), __byte_perm(q.x, q.z, 0x7632), __byte_perm(q.y, q.w, 0x5410),
                       __byte_perm(q.y, q.w, 0x7632));
      *reinterpret_cast<uint4*>(xs_ptr + m * x_pitch + (act_pos(fmt, j) << 4)) = q;
    }
  }
  __syncthreads();

  // Two accumulator sets per block of 16 channels, used alternately, so that consecutive instructions do not wait for
  // one another.
  float ca[kBlk][4], cb[kBlk][4];
#pragma unroll
  for (int b = 0; b < kBlk; ++b)
#pragma unroll
    for (int i = 0; i < 4; ++i) ca[b][i] = cb[b][i] = 0.f;
  int c_tile = 0, c_kb = warp - kWarps, slot = 0, phase = 0, cur_tile = 0;
  advance(c_tile, c_kb);
  bool dead = false;  // a wait ran out: stop waiting and computing, keep signalling the other warps
  auto give_up = [&]() {
    if (lane == 0 && p.timeout) atomicOr(p.timeout, kTimeoutGemv);
    dead = true;
  };
  // Only the lanes that hold one of the kM rows of activations load them (see lds128_if).
  const uint32_t x_lane = xs + min(g, kM - 1) * x_pitch + (tq << 4);
  const uint32_t x_on = g < kM ? 1u : 0u;
  uint4 xv = make_uint4(0u, 0u, 0u, 0u);
  const uint32_t w_lane = (g << 7);
  float* part_ptr = reinterpret_cast<float*>(smem_dyn + (part - dyn));

  // Adds the 16 warps' partial sums of a tile in warp order and stores the results.
  // kQuant: the warps run free of one another (mbarrier hand-over of the partial sums, the sums of tile t added while
  // tile t + 1 is under way) -- the dequantisation makes them issue-bound and a CTA-wide barrier per tile costs 10-20 %.
  // fp16 only: the warps meet at a CTA barrier per tile; they are bound by the weight stream, and warps that stay in
  // step ask for neighbouring 128-byte pieces of the same weight rows together, which the DRAM serves faster (5.2
  // instead of 4.2 TB/s on a 65536 x 4096 matrix).
  constexpr bool kLockstep = !kQuant;
  auto reduce_tile = [&](int t) {
    const int buf = t & (kBufs - 1);
    if (!kLockstep && !dead && !wait_phase(smem_u32(&part_full[buf]), (t / kPartBufs) & 1)) give_up();
    if (!dead && tq < 2) {
#pragma unroll
      for (int b = 0; b < kBlk; ++b) {
        const int ra = row0 + t * kTileRows + 16 * b + g, rb = ra + 8, m0 = tq << 1;
        if (ra >= rows_end) break;  // (rows g + 8 of a block are valid only when rows g are)
        const float* src = part_ptr + buf * kWarps * kPartWarp + b * 64 + ((g << 1) + tq) * 4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float4 v = *reinterpret_cast<const float4*>(src + w * kPartWarp);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        {
          const float sc = (kQuant && fmt == 1) ? __half2float(sg.scale[ra]) : 1.f;
          if (m0 < kM) store_result(sg, m0, ra, acc.x * sc);
          if (m0 + 1 < kM) store_result(sg, m0 + 1, ra, acc.y * sc);
        }
        if (rb < rows_end) {
          const float sc = (kQuant && fmt == 1) ? __half2float(sg.scale[rb]) : 1.f;
          if (m0 < kM) store_result(sg, m0, rb, acc.z * sc);
          if (m0 + 1 < kM) store_result(sg, m0 + 1, rb, acc.w * sc);
        }
      }
    }
    if (!kLockstep) {
      __syncwarp();
      if (lane == 0) mbar_arrive_cta(smem_u32(&part_free[buf]));
    }
  };

  for (;;) {
    // Tile boundaries.  Every warp passes every one of them, whether or not it had a box in the tile: it leaves its
    // partial sums and goes on; the warp whose turn it is adds the PREVIOUS tile's sums, which by then are complete
    // as a rule, so that no warp waits for the others at a boundary.
    for (const int upto = min(c_tile, n_tiles); cur_tile < upto; ++cur_tile) {
      const int buf = cur_tile & (kBufs - 1);
      if (!kLockstep && cur_tile >= kPartBufs && !dead && !wait_phase(smem_u32(&part_free[buf]), (cur_tile / kPartBufs - 1) & 1)) give_up();
#pragma unroll
      for (int b = 0; b < kBlk; ++b) {
        if (tq < 2)
          *reinterpret_cast<float4*>(part_ptr + (buf * kWarps + warp) * kPartWarp + b * 64 + ((g << 1) + tq) * 4) =
              make_float4(ca[b][0] + cb[b][0], ca[b][1] + cb[b][1], ca[b][2] + cb[b][2], ca[b][3] + cb[b][3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) ca[b][i] = cb[b][i] = 0.f;
      }
      if (kLockstep) {
        __syncthreads();
        if (warp == (cur_tile & (kWarps - 1))) reduce_tile(cur_tile);
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive_cta(smem_u32(&part_full[buf]));
        if (cur_tile >= 1 && warp == ((cur_tile - 1) & (kWarps - 1))) reduce_tile(cur_tile - 1);
      }
    }
    if (c_tile >= n_tiles) break;

    const uint32_t bar = smem_u32(&bars[warp][slot]);
    if (!dead && !wait_phase(bar, phase)) give_up();
    if (!dead) {
      const uint32_t wbase = ring + slot * kSlot + w_lane;
      // a ragged last tile may end before its second block of 16 channels
      const bool two = kBlk == 2 && rows_end - (row0 + c_tile * kTileRows) > 16;
      if (!kQuant || fmt == 0) {
        const uint32_t xa_addr = x_lane + (c_kb << 7);  // 8 blocks of 16 bytes per box
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t off = static_cast<uint32_t>(((tq << 1) + h) ^ g) << 4;
          lds128_if(xv, xa_addr + (h << 6), x_on);
#pragma unroll
          for (int b = 0; b < kBlk; ++b) {
            if (b == 1 && !two) break;
            const uint4 wa = lds128(wbase + b * kSlotBytes + off), wb = lds128(wbase + b * kSlotBytes + 1024 + off);
            mma16816(ca[b], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
            mma16816(cb[b], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
          }
        }
      } else if (fmt == 1) {
        const uint32_t xa_addr = x_lane + (c_kb << 8);  // 16 blocks per box
        const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t off = static_cast<uint32_t>(((tq << 1) + h) ^ g) << 4;
          uint32_t ua[kBlk][4], ub[kBlk][4];
#pragma unroll
          for (int b = 0; b < kBlk; ++b) {
            const uint4 wa = lds128(wbase + b * kSlotBytes + off), wb = lds128(wbase + b * kSlotBytes + 1024 + off);
            ua[b][0] = wa.x; ua[b][1] = wa.y; ua[b][2] = wa.z; ua[b][3] = wa.w;
            ub[b][0] = wb.x; ub[b][1] = wb.y; ub[b][2] = wb.z; ub[b][3] = wb.w;
          }
#pragma unroll
          for (int sb = 0; sb < 2; ++sb) {
            lds128_if(xv, xa_addr + (((h << 1) + sb) << 6), x_on);
#pragma unroll
            for (int b = 0; b < kBlk; ++b) {
              if (b == 1 && !two) break;
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const uint32_t wa = ua[b][2 * sb + i] ^ 0x80808080u, wb = ub[b][2 * sb + i] ^ 0x80808080u;
                const uint32_t a01 = h2u(__hsub2(u2h(__byte_perm(wa, 0x64646464u, 0x4140)), bias));
                const uint32_t a23 = h2u(__hsub2(u2h(__byte_perm(wa, 0x64646464u, 0x4342)), bias));
                const uint32_t b01 = h2u(__hsub2(u2h(__byte_perm(wb, 0x64646464u, 0x4140)), bias));
                const uint32_t b23 = h2u(__hsub2(u2h(__byte_perm(wb, 0x64646464u, 0x4342)), bias));
                if (i == 0) mma16816(ca[b], a01, b01, a23, b23, xv.x, xv.y);
                else mma16816(cb[b], a01, b01, a23, b23, xv.z, xv.w);
              }
            }
          }
        }
      } else {
        const uint32_t xa_addr = x_lane + (c_kb << 9);  // 32 blocks per box
        // (scale, zero) of this lane's group (two chunks of 16 bytes = one group of 128 weights) for rows g and g + 8
        const uint32_t sel = (tq >> 1) ? 0x3232u : 0x1010u;
        const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f);
        __half2 sa2[kBlk], sb2[kBlk], za_lo[kBlk], zb_lo[kBlk], za_hi[kBlk], zb_hi[kBlk];
#pragma unroll
        for (int b = 0; b < kBlk; ++b) {
          uint32_t pa_s, pa_z, pb_s, pb_z;
          const uint32_t sa = szs + slot * kSzSlot + (b << 7) + (g << 3);
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pa_s), "=r"(pa_z) : "r"(sa));
          asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(pb_s), "=r"(pb_z) : "r"(sa + 64));
          sa2[b] = u2h(__byte_perm(pa_s, 0u, sel));
          sb2[b] = u2h(__byte_perm(pb_s, 0u, sel));
          const __half2 za = u2h(__byte_perm(pa_z, 0u, sel)), zb = u2h(__byte_perm(pb_z, 0u, sel));
          za_lo[b] = __hadd2(za, __floats2half2_rn(1024.f, 1024.f));
          zb_lo[b] = __hadd2(zb, __floats2half2_rn(1024.f, 1024.f));
          za_hi[b] = __hneg2(__hadd2(za, __floats2half2_rn(64.f, 64.f)));
          zb_hi[b] = __hneg2(__hadd2(zb, __floats2half2_rn(64.f, 64.f)));
        }
        auto dq = [&](uint32_t u, const __half2 sc, const __half2 zlo, const __half2 zhi, uint32_t (&o)[4]) {
          const uint32_t v = u >> 8;
          o[0] = h2u(__hmul2(__hsub2(u2h(and_or(u, 0x000f000fu, 0x64006400u)), zlo), sc));
          o[1] = h2u(__hmul2(__hfma2(u2h(and_or(u, 0x00f000f0u, 0x64006400u)), sixteenth, zhi), sc));
          o[2] = h2u(__hmul2(__hsub2(u2h(and_or(v, 0x000f000fu, 0x64006400u)), zlo), sc));
          o[3] = h2u(__hmul2(__hfma2(u2h(and_or(v, 0x00f000f0u, 0x64006400u)), sixteenth, zhi), sc));
        };
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t off = static_cast<uint32_t>(((tq << 1) + h) ^ g) << 4;
          uint32_t ua[kBlk][4], ub[kBlk][4];
#pragma unroll
          for (int b = 0; b < kBlk; ++b) {
            const uint4 wa = lds128(wbase + b * kSlotBytes + off), wb = lds128(wbase + b * kSlotBytes + 1024 + off);
            ua[b][0] = wa.x; ua[b][1] = wa.y; ua[b][2] = wa.z; ua[b][3] = wa.w;
            ub[b][0] = wb.x; ub[b][1] = wb.y; ub[b][2] = wb.z; ub[b][3] = wb.w;
          }
#pragma unroll
          for (int wd = 0; wd < 4; ++wd) {
            lds128_if(xv, xa_addr + (((h << 2) + wd) << 6), x_on);
#pragma unroll
            for (int b = 0; b < kBlk; ++b) {
              if (b == 1 && !two) break;
              uint32_t pa[4], pb2[4];
              dq(ua[b][wd], sa2[b], za_lo[b], za_hi[b], pa);
              dq(ub[b][wd], sb2[b], zb_lo[b], zb_hi[b], pb2);
              mma16816(ca[b], pa[0], pb2[0], pa[1], pb2[1], xv.x, xv.y);
              mma16816(cb[b], pa[2], pb2[2], pa[3], pb2[3], xv.z, xv.w);
            }
          }
        }
      }
    }
    __syncwarp();  // every lane has read the slot: it may be overwritten
    if (!dead && q_tile < n_tiles) issue();
    if (++slot == n_slots) { slot = 0; phase ^= 1; }
    advance(c_tile, c_kb);
  }
  if (!kLockstep && n_tiles >= 1 && warp == ((n_tiles - 1) & (kWarps - 1))) reduce_tile(n_tiles - 1);
}

// ---------------------------------------------------------------------------------- host side
using EncodeFn = TensorMapEncodeFn;
inline EncodeFn encode_fn() { return tensor_map_encode_fn(); }

struct MapKey {
  const void* base;
  int rows, row_bytes, box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && row_bytes == o.row_bytes && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    for (int v : {k.rows, k.row_bytes, k.box_rows}) h = h * 1000003u ^ static_cast<size_t>(v);
    return h;
  }
};

// A weight matrix of any format as a 2-D byte tensor [rows, row_bytes]; boxes of 128 bytes x box_rows rows, 128-byte
// swizzle.  Encoded maps are kept: a model asks for the same few hundred matrices on every call.
int make_byte_map(CUtensorMap* map, const void* base, int rows, int row_bytes, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, rows, row_bytes, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return kOk;
    }
  }
  EncodeFn fn = encode_fn();
  RK_REQUIRE(fn, kCuda, "gemv_mma: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  RK_REQUIRE(r == CUDA_SUCCESS, kCuda, "gemv_mma: cuTensorMapEncodeTiled failed with %d (rows=%d row_bytes=%d)", static_cast<int>(r), rows, row_bytes);
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *map);
  return kOk;
}

int row_bytes_of(const GemvSeg& g) { return g.fmt == 0 ? g.K * 2 : g.fmt == 1 ? g.K : g.K / 2; }

}  // namespace

// Shares the CTAs out over the problems by weight bytes and picks the ring depth.  Returns false for what the kernel
// does not take: an input activation, weight rows that are not whole 128-byte boxes, channel counts that are not a
// multiple of 4, activations that leave no room for a ring.
bool gemv_mma_plan(GemvBatch& b, int M, GemvMmaPlan* plan) {
  if (M < 1 || M > 4) return false;
  int max_k = 0;
  double total_bytes = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    const GemvSeg& g = b.seg[i];
    if (g.in_act != kActNone || g.N % 4 != 0 || row_bytes_of(g) % 128 != 0) return false;
    if (g.fmt == 2 && g.K % 128 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(g.w) & 15u) != 0) return false;
    max_k = std::max(max_k, g.K);
    total_bytes += static_cast<double>(g.N) * row_bytes_of(g);
  }
  const int x_pitch = max_k * 2 + 64;  // rows 64 bytes apart modulo 128: two rows of activations share no bank
  bool quant = false;
  for (int i = 0; i < b.n_seg; ++i) quant = quant || b.seg[i].fmt != 0;
  // Tiles of 32 channels (two 4 KiB slots per warp) halve the per-box bookkeeping.  Measured per decode step of the 7.2B
  // model: fp16 2.85 -> 2.59 ms at one row, 3.43 -> 3.25 at two, 3.72 -> 3.65 at three, but 4.01 -> 4.21 at four;
  // W4A16 2.03 -> 1.90 ms at one row, but 2.29 -> 2.54 at two and 2.96 -> 3.39 at four (large single matrices gain at
  // any row count; which launch of the step loses was not isolated).  Hence, by default (gemv_mma_tall = 2): one row of
  // any format, and up to three rows of fp16.  1: one row of quantised weights only; 3: wherever they fit; 0: never.
  const int tall_mode = options().gemv_mma_tall;
  const bool want_tall = tall_mode >= 3 || (tall_mode == 2 && (M == 1 || (!quant && M <= 3))) || (tall_mode == 1 && quant && M == 1);
  int blk = 1, slots = kMaxSlots;
  auto fixed_bytes = [&](int blocks) {  // alignment slack + partial sums + quantisation parameters + activations
    const size_t part = static_cast<size_t>(quant ? kPartBufs : 2) * kWarps * 256 * blocks;
    return 1024 + part + (quant ? static_cast<size_t>(kSzBytes) * blocks : 0) + static_cast<size_t>(M) * x_pitch;
  };
  size_t fixed = fixed_bytes(1);
  const size_t fixed_tall = fixed_bytes(2);
  if (want_tall && fixed_tall + static_cast<size_t>(kWarps) * 2 * 2 * kSlotBytes <= static_cast<size_t>(kSmemLimit)) {
    blk = 2;
    slots = 2;
    fixed = fixed_tall;
  } else {
    while (slots >= 2 && fixed + static_cast<size_t>(kWarps) * slots * kSlotBytes > static_cast<size_t>(kSmemLimit)) --slots;
    if (slots < 2) return false;
  }
  const int budget = 148;
  int n_cta[kMaxSeg];
  int used = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    const GemvSeg& g = b.seg[i];
    const double share = static_cast<double>(g.N) * row_bytes_of(g) / total_bytes;
    n_cta[i] = std::max(1, std::min(g.N / 4, static_cast<int>(share * budget)));
    used += n_cta[i];
  }
  while (used < budget) {  // the rest go one at a time to whichever problem has the most bytes per CTA
    int best = -1;
    double worst = 0;
    for (int i = 0; i < b.n_seg; ++i) {
      const GemvSeg& g = b.seg[i];
      if (n_cta[i] >= g.N / 4) continue;
      const double per = static_cast<double>((g.N + n_cta[i] - 1) / n_cta[i]) * row_bytes_of(g);
      if (per > worst) { worst = per; best = i; }
    }
    if (best < 0) break;
    ++n_cta[best];
    ++used;
  }
  int cta = 0;
  for (int i = 0; i < b.n_seg; ++i) {
    GemvSeg& g = b.seg[i];
    g.rows_per_cta = ((g.N + n_cta[i] - 1) / n_cta[i] + 3) & ~3;
    g.cta_begin = cta;
    cta += (g.N + g.rows_per_cta - 1) / g.rows_per_cta;
  }
  plan->smem_bytes = fixed + static_cast<size_t>(kWarps) * slots * blk * kSlotBytes;
  plan->grid = cta;
  plan->n_slots = slots;
  plan->blocks = blk;
  plan->x_pitch = x_pitch;
  return true;
}

bool gemv_mma_fits(int M, int K) {  // (the quantised layout, which is the larger one)
  return M >= 1 && M <= 4 && 1024 + kPartialBytes + kSzBytes + static_cast<size_t>(M) * (K * 2 + 64) + static_cast<size_t>(kWarps) * 2 * kSlotBytes <=
                                 static_cast<size_t>(kSmemLimit);
}

int gemv_mma_launch(cudaStream_t stream, const GemvBatch& b, int M, const GemvMmaPlan& plan) {
  MmaMaps maps;
  bool quant = false;
  for (int i = 0; i < kMaxSeg; ++i) {
    const GemvSeg& g = b.seg[i < b.n_seg ? i : 0];
    if (i < b.n_seg) {
      quant = quant || g.fmt != 0;
      int s = make_byte_map(&maps.full[i], g.w, g.N, row_bytes_of(g), 16);
      if (s != kOk) return s;
      s = make_byte_map(&maps.quad[i], g.w, g.N, row_bytes_of(g), 4);
      if (s != kOk) return s;
      if (plan.blocks == 2) s = make_byte_map(&maps.tall[i], g.w, g.N, row_bytes_of(g), 32);
      else maps.tall[i] = maps.full[i];
      if (s != kOk) return s;
    } else {
      maps.full[i] = maps.full[0];
      maps.quad[i] = maps.quad[0];
      maps.tall[i] = maps.tall[0];
    }
  }
  auto launch = [&](auto kernel) -> int {
    RK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    RK_CUDA(launch_pdl(kernel, dim3(plan.grid), dim3(kWarps * 32), plan.smem_bytes, stream, maps, b, plan.n_slots, plan.x_pitch));
    return kOk;
  };
  int s;
  if (quant && plan.blocks == 2) {
    switch (M) {
      case 1: s = launch(gemv_mma_kernel<1, true, 2>); break;
      case 2: s = launch(gemv_mma_kernel<2, true, 2>); break;
      case 3: s = launch(gemv_mma_kernel<3, true, 2>); break;
      default: s = launch(gemv_mma_kernel<4, true, 2>); break;
    }
  } else if (quant) {
    switch (M) {
      case 1: s = launch(gemv_mma_kernel<1, true, 1>); break;
      case 2: s = launch(gemv_mma_kernel<2, true, 1>); break;
      case 3: s = launch(gemv_mma_kernel<3, true, 1>); break;
      default: s = launch(gemv_mma_kernel<4, true, 1>); break;
    }
  } else if (plan.blocks == 2) {
    switch (M) {
      case 1: s = launch(gemv_mma_kernel<1, false, 2>); break;
      case 2: s = launch(gemv_mma_kernel<2, false, 2>); break;
      case 3: s = launch(gemv_mma_kernel<3, false, 2>); break;
      default: s = launch(gemv_mma_kernel<4, false, 2>); break;
    }
  } else {
    switch (M) {
      case 1: s = launch(gemv_mma_kernel<1, false, 1>); break;
      case 2: s = launch(gemv_mma_kernel<2, false, 1>); break;
      case 3: s = launch(gemv_mma_kernel<3, false, 1>); break;
      default: s = launch(gemv_mma_kernel<4, false, 1>); break;
    }
  }
  if (s != kOk) return s;
  RK_LAUNCH_CHECK("gemv_mma launch");
  return kOk;
}

}  // namespace rk
