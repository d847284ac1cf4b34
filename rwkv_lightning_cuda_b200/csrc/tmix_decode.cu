// One-token time-mix core, one CTA per (sequence, head):
//   LoRA up-projections (decay w, in-context rate a, gate g, value residual v)
//   -> kk normalisation / a gate / key update -> WKV-7 state update -> GroupNorm + bonus + gate.
// Replaces, for decode steps of up to a few sequences, the chain
//   linear_wagv_rank_out_f16 (cuda/rwkv7_v3a_ops.cu:1027-1130) -> tmix_kk_a_gate (cuda/rwkv7_fast_ops_fp16.cu:129-172)
//   -> wkv_fp16_* / wkv_fp32_v2_* (cuda/rwkv7_wkv_fp16_v2.cu, cuda/rwkv7_wkv_fp32_v2.cu)
//   -> tmix_lnx_rkvres_xg (cuda/rwkv7_fast_ops_fp16.cu:174-237)
// of the reference with a single launch: the head's 64 rows of the four up-projection matrices and
// its 64x64 state tile are requested (cp.async into shared memory / registers) before the
// programmatic-dependency wait, so their HBM latency overlaps the tail of the previous kernel.
// Rounding points are the reference's: w12, a12, g, v, k', -kk, kk*a and y are each rounded to
// half once; the fp16-state update reproduces the reference's half2 FMA chains bit for bit.
#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

constexpr float kTwoNeg41 = 4.547473508864641e-13f;
constexpr float kNegExpHalfLog2e = -0.8750387749145276f;
constexpr float kNegLog2e = -1.4426950408889634f;

struct TmixDev {
  int C, H, layer0, round_act;
  int R[4];               // ranks of w, a, g, v
  const half* l1[4];      // [B, R] LoRA down outputs
  const half* up[4];      // [C, R] LoRA up matrices (row = output channel)
  const half *r, *k, *v, *v_first;
  const half *w0, *a0, *v0, *k_k, *k_a, *r_k, *lnx_w, *lnx_b;
  void* state;
  const int* elapsed;
  half* y2;
  const half* shift_src;  // optional [B,C] rows to move into the time-mix shift state (this head's 64 channels)
  half* shift_dst;
  int* timeout;           // the device's failure word: set when the bounded wait for the weight rows gives up
};

template <bool kWkv32>
__global__ void __launch_bounds__(256) tmix_decode_kernel(const TmixDev p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(16) float acts[4 * 512];
  __shared__ float res[4][kHead];
  __shared__ __align__(16) half hv[8][kHead];  // r, d, k', a, b, v, g, y
  __shared__ float red[4];
  __shared__ __align__(8) uint64_t wbar;

  const int bh = blockIdx.x;
  const int b_id = bh / p.H;
  const int h = bh - b_id * p.H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t tok = static_cast<size_t>(b_id) * p.C + static_cast<size_t>(h) * kHead;

  // ---- requests that do not depend on the previous kernel: up-projection rows and the state
  // Thread j owns up-projection row j (matrix j/64, channel j%64 of this head).  The rows are fetched
  // by the bulk-copy engine, one request per row, into rows padded by 16 bytes so that the 32 lanes
  // of a warp later read their own rows without bank conflicts.
  uint4* tile = reinterpret_cast<uint4*>(smem_raw);             // fp16 state tile, 8 KiB (unused for fp32)
  unsigned char* wsm = smem_raw + (kWkv32 ? 0 : 8192);
  const int my_seg = tid >> 6, my_ch = tid & 63;
  const bool has_row = !(p.layer0 && my_seg == 3);
  int my_off = 0, total_bytes = 0;
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    const int seg_bytes = (p.layer0 && s == 3) ? 0 : kHead * (p.R[s] * 2 + 16);
    if (s < my_seg) my_off += seg_bytes;
    if (!(p.layer0 && s == 3)) total_bytes += kHead * p.R[s] * 2;
  }
  const int my_R = p.R[my_seg];
  const unsigned char* my_row = wsm + my_off + my_ch * (my_R * 2 + 16);
  if (tid == 0) {
    mbar_init(smem_u32(&wbar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(smem_u32(&wbar), total_bytes);
  }
  __syncthreads();
  if (has_row)
    bulk_g2s(smem_u32(my_row), p.up[my_seg] + (static_cast<size_t>(h) * kHead + my_ch) * my_R, my_R * 2, smem_u32(&wbar));
  float4 S32[4];
  if (kWkv32) {
    const float4* sb = reinterpret_cast<const float4*>(static_cast<float*>(p.state) + static_cast<size_t>(bh) * (kHead * kHead));
#pragma unroll
    for (int q = 0; q < 4; ++q) S32[q] = sb[(q * 16 + (tid >> 4)) * 16 + (tid & 15)];
  } else {
    const half* sb = static_cast<const half*>(p.state) + static_cast<size_t>(bh) * (kHead * kHead);
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int q = it * 256 + tid;
      const int row = q >> 3, c = q & 7;
      cp_async16(&tile[row * 8 + (c ^ (row & 7))], sb + q * 8);
    }
  }
  cp_async_commit();
  // This head's per-channel parameters are static too: requested here, used far down the dependent chain (read where
  // they are used, each cost a DRAM round trip in the middle of it -- between two steps the 14 GB of weights pass
  // through L2, so none of them is still cached).
  half c_v0 = __float2half_rn(0.f), c_kk = c_v0, c_w0 = c_v0, c_a0 = c_v0, c_ka = c_v0, c_rk = c_v0, c_lw = c_v0, c_lb = c_v0;
  if (tid < kHead) {
    const int c = h * kHead + tid;
    if (!p.layer0) c_v0 = p.v0[c];
    c_kk = p.k_k[c]; c_w0 = p.w0[c]; c_a0 = p.a0[c]; c_ka = p.k_a[c]; c_rk = p.r_k[c]; c_lw = p.lnx_w[c]; c_lb = p.lnx_b[c];
  }

  pdl_wait();
  pdl_trigger();
  if (p.shift_src && tid < kHead / 2)
    reinterpret_cast<__half2*>(p.shift_dst + tok)[tid] = reinterpret_cast<const __half2*>(p.shift_src + tok)[tid];
  // ---- everything the previous kernel wrote is requested at once (ranks are at most 512: two values per thread and
  // matrix); taken one matrix after the other, each load would wait for the previous one's shared-memory store
  half raw[4][2];
#pragma unroll
  for (int s = 0; s < 4; ++s) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + 256 * j;
      raw[s][j] = __float2half_rn(0.f);
      if (!(p.layer0 && s == 3) && i < p.R[s]) raw[s][j] = p.l1[s][static_cast<size_t>(b_id) * p.R[s] + i];
    }
  }
  float kf = 0.f, vf = 0.f, vfirstf = 0.f;
  int elapsed_b = 0;
  half r_in = __float2half_rn(0.f);
  if (tid < kHead) {
    elapsed_b = p.elapsed[b_id];
    r_in = p.r[tok + tid];
    kf = __half2float(p.k[tok + tid]);
    vf = __half2float(p.v[tok + tid]);
    vfirstf = __half2float(p.v_first[tok + tid]);
  }
  // ---- LoRA inputs with their activations, kept in fp32
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (p.layer0 && s == 3) continue;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + 256 * j;
      if (i >= p.R[s]) continue;
      float x = __half2float(raw[s][j]);
      if (p.round_act) {  // what the separate activation kernels of the many-row path produce
        if (s == 0) x = __half2float(__float2half_rn(apply_in_act(x, kActTanh)));
        if (s == 2) x = __half2float(__float2half_rn(apply_in_act(x, kActSigmoid)));
      } else {
        if (s == 0) x = tanhf(x);
        if (s == 2) x = 1.0f / (1.0f + expf(-x));
      }
      acts[s * 512 + i] = x;
    }
  }
  if (tid < kHead) hv[0][tid] = r_in;
  cp_async_wait<0>();
  __syncthreads();
  if (!mbar_wait(smem_u32(&wbar), 0)) {  // uniform: every thread waits on the same barrier
    if (tid == 0 && p.timeout) atomicOr(p.timeout, kTimeoutTmix);
    return;
  }

  // ---- up-projections: thread j computes the dot product of its row with the activated LoRA input
  if (has_row) {
    const float* xa = acts + my_seg * 512;
    // four independent partial sums: one chain of up to 480 dependent FMAs would be a microsecond of latency
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int c = 0; c < my_R; c += 8) {
      const uint4 q = *reinterpret_cast<const uint4*>(my_row + c * 2);
      const float4 x0 = *reinterpret_cast<const float4*>(xa + c);
      const float4 x1 = *reinterpret_cast<const float4*>(xa + c + 4);
      const float2 f0 = h2f2(q.x), f1 = h2f2(q.y), f2 = h2f2(q.z), f3 = h2f2(q.w);
      a0 = fmaf(x0.x, f0.x, a0); a1 = fmaf(x0.y, f0.y, a1);
      a2 = fmaf(x0.z, f1.x, a2); a3 = fmaf(x0.w, f1.y, a3);
      a0 = fmaf(x1.x, f2.x, a0); a1 = fmaf(x1.y, f2.y, a1);
      a2 = fmaf(x1.z, f3.x, a2); a3 = fmaf(x1.w, f3.y, a3);
    }
    res[my_seg][my_ch] = (a0 + a1) + (a2 + a3);
  }
  __syncthreads();

  // ---- per-channel gates (threads 0..63 = the head's channels)
  float v_use = 0.f;
  if (tid < kHead) {
    const int c = h * kHead + tid;
    const half w12 = __float2half_rn(res[0][tid]);
    const half a12 = __float2half_rn(res[1][tid]);
    hv[6][tid] = __float2half_rn(res[2][tid]);
    if (p.layer0) {
      v_use = vf;
    } else {
      if (p.round_act) {
        const float gate = sigmoid_fast(__half2float(c_v0) + __half2float(__float2half_rn(res[3][tid])));
        v_use = __half2float(__float2half_rn(fmaf(vfirstf - vf, gate, vf)));
      } else {
        const float gate = 1.0f / (1.0f + expf(-(__half2float(c_v0) + res[3][tid])));
        v_use = __half2float(__float2half_rn(vf + (vfirstf - vf) * gate));
      }
    }
    hv[5][tid] = __float2half_rn(v_use);
    const float u = kf * __half2float(c_kk);
    const float ss = warp_sum(u * u);
    if (lane == 0) red[warp] = ss;
    // decay pre-activation
    float wf = __half2float(w12);
    const float w0f = __half2float(c_w0);
    float d;
    if (kWkv32) {
      wf = __half2float(__float2half_rn(wf + w0f));  // the reference pre-adds w0 and rounds for the fp32 state
      d = exp2f(kNegExpHalfLog2e / (1.0f + exp2f(kNegLog2e * wf)));
      acts[tid] = d;                                  // fp32 decay, reuses the activation buffer
    } else {
      wf += w0f;
      const int rot = static_cast<int>(2654435769u * static_cast<unsigned>(elapsed_b + c));
      d = exp2f(kNegExpHalfLog2e / (1.0f + exp2f(kNegLog2e * wf))) - 1.0f + kTwoNeg41 * static_cast<float>(rot);
      hv[1][tid] = __float2half_rn(d);
    }
    // kk / a / k' need the head-wide norm: finish after the barrier below
    acts[512 + tid] = u;
    acts[1024 + tid] = sigmoid_fast(__half2float(c_a0) + __half2float(a12));
  }
  __syncthreads();
  if (tid < kHead) {
    const int c = h * kHead + tid;
    const float inv_d = 1.0f / fmaxf(sqrtf(red[0] + red[1]), 1.0e-12f);
    const float kk = acts[512 + tid] * inv_d;
    const float av = acts[1024 + tid];
    const float ka = __half2float(c_ka);
    hv[2][tid] = __float2half_rn(kf * fmaf(av, ka, 1.0f - ka));
    hv[3][tid] = __float2half_rn(-kk);
    hv[4][tid] = __float2half_rn(kk * av);
  }
  __syncthreads();

  // ---- WKV-7 state update
  if (kWkv32) {
    const int c4 = tid & 15, rsub = tid >> 4;
    auto ld4 = [&](const half* src) {
      const uint2 u = *reinterpret_cast<const uint2*>(src + c4 * 4);
      const float2 lo = h2f2(u.x), hi = h2f2(u.y);
      return make_float4(lo.x, lo.y, hi.x, hi.y);
    };
    const float4 rr = ld4(hv[0]), kk4 = ld4(hv[2]), aa = ld4(hv[3]), bb = ld4(hv[4]);
    const float4 ww = *reinterpret_cast<const float4*>(acts + c4 * 4);
    float4* sb = reinterpret_cast<float4*>(static_cast<float*>(p.state) + static_cast<size_t>(bh) * (kHead * kHead));
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int row = q * 16 + rsub;
      float4 s = S32[q];
      float sa = s.x * aa.x + s.y * aa.y + s.z * aa.z + s.w * aa.w;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sa += __shfl_xor_sync(0xffffffffu, sa, o);
      const float vi = __half2float(hv[5][row]);
      s.x = s.x * ww.x + sa * bb.x + kk4.x * vi;
      s.y = s.y * ww.y + sa * bb.y + kk4.y * vi;
      s.z = s.z * ww.z + sa * bb.z + kk4.z * vi;
      s.w = s.w * ww.w + sa * bb.w + kk4.w * vi;
      float yy = s.x * rr.x + s.y * rr.y + s.z * rr.z + s.w * rr.w;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) yy += __shfl_xor_sync(0xffffffffu, yy, o);
      sb[row * 16 + c4] = s;
      if (c4 == 0) hv[7][row] = __float2half_rn(yy);
    }
  } else if (tid < kHead) {
    const int i = tid;
    __half2 S[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 q = tile[i * 8 + (c ^ (i & 7))];
      S[4 * c + 0] = *reinterpret_cast<const __half2*>(&q.x);
      S[4 * c + 1] = *reinterpret_cast<const __half2*>(&q.y);
      S[4 * c + 2] = *reinterpret_cast<const __half2*>(&q.z);
      S[4 * c + 3] = *reinterpret_cast<const __half2*>(&q.w);
    }
    const __half2* r2 = reinterpret_cast<const __half2*>(hv[0]);
    const __half2* d2 = reinterpret_cast<const __half2*>(hv[1]);
    const __half2* k2 = reinterpret_cast<const __half2*>(hv[2]);
    const __half2* a2 = reinterpret_cast<const __half2*>(hv[3]);
    const __half2* b2 = reinterpret_cast<const __half2*>(hv[4]);
    __half2 sa2 = __floats2half2_rn(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 32; ++j) sa2 = __hfma2(a2[j], S[j], sa2);
    const half sa = __hadd(__low2half(sa2), __high2half(sa2));
    sa2 = __half2half2(sa);
    const __half2 vv2 = __half2half2(hv[5][i]);
    __half2 y2 = __floats2half2_rn(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      __half2 s = S[j];
      s = __hfma2(s, d2[j], __hfma2(k2[j], vv2, __hfma2(sa2, b2[j], s)));
      S[j] = s;
      y2 = __hfma2(s, r2[j], y2);
    }
    hv[7][i] = __hadd(__low2half(y2), __high2half(y2));
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 q;
      q.x = *reinterpret_cast<const uint32_t*>(&S[4 * c + 0]);
      q.y = *reinterpret_cast<const uint32_t*>(&S[4 * c + 1]);
      q.z = *reinterpret_cast<const uint32_t*>(&S[4 * c + 2]);
      q.w = *reinterpret_cast<const uint32_t*>(&S[4 * c + 3]);
      tile[i * 8 + (c ^ (i & 7))] = q;
    }
  }
  __syncthreads();
  if (!kWkv32) {
    half* sb = static_cast<half*>(p.state) + static_cast<size_t>(bh) * (kHead * kHead);
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int q = it * 256 + tid;
      const int row = q >> 3, c = q & 7;
      reinterpret_cast<uint4*>(sb)[q] = tile[row * 8 + (c ^ (row & 7))];
    }
  }

  // ---- GroupNorm over the head + bonus + gate (two warps)
  float yv = 0.f, dmean = 0.f;
  if (tid < kHead) {
    yv = __half2float(hv[7][tid]);
    const float s = warp_sum(yv);
    if (lane == 0) red[warp] = s;
  }
  __syncthreads();
  if (tid < kHead) {
    const float mean = (red[0] + red[1]) * (1.0f / 64.0f);
    dmean = yv - mean;
    const float ss = warp_sum(dmean * dmean);
    const float dot = warp_sum(__half2float(hv[0][tid]) * __half2float(hv[2][tid]) * __half2float(c_rk));
    if (lane == 0) {
      red[2 + warp] = ss;
      acts[1536 + warp] = dot;
    }
  }
  __syncthreads();
  if (tid < kHead) {
    const int c = h * kHead + tid;
    const float rstd = rsqrtf((red[2] + red[3]) * (1.0f / 64.0f) + 64.0e-5f);
    const float rkv = acts[1536] + acts[1537];
    const float out = (dmean * rstd * __half2float(c_lw) + __half2float(c_lb) + rkv * v_use) * __half2float(hv[6][tid]);
    p.y2[tok + tid] = __float2half_rn(out);
  }
}

}  // namespace

bool tmix_decode_supported(const TmixDecodeArgs& a) {
  const int sum_r = a.R[0] + a.R[1] + a.R[2] + (a.layer0 ? 0 : a.R[3]);
  const size_t smem = static_cast<size_t>(kHead) * (sum_r * 2 + 64) + (a.wkv32 ? 0 : 8192);
  for (int s = 0; s < 4; ++s)
    if (a.R[s] > 512 || a.R[s] % 8 != 0) return false;
  return smem <= 200 * 1024;
}

int tmix_decode(cudaStream_t stream, const TmixDecodeArgs& a) {
  RK_REQUIRE(a.B > 0 && a.C > 0 && a.C % kHead == 0, kShape, "tmix_decode: C must be a multiple of 64");
  RK_REQUIRE(tmix_decode_supported(a), kShape, "tmix_decode: LoRA ranks too large for the shared-memory staging");
  RK_REQUIRE(a.state && a.elapsed && a.r && a.k && a.v && a.v_first && a.y2, kBadArg, "tmix_decode: null pointer");
  TmixDev p;
  p.C = a.C; p.H = a.C / kHead; p.layer0 = a.layer0 ? 1 : 0; p.round_act = a.round_act ? 1 : 0;
  for (int s = 0; s < 4; ++s) { p.R[s] = a.R[s]; p.l1[s] = a.l1[s]; p.up[s] = a.up[s]; }
  p.r = a.r; p.k = a.k; p.v = a.v; p.v_first = a.v_first;
  p.w0 = a.w0; p.a0 = a.a0; p.v0 = a.v0; p.k_k = a.k_k; p.k_a = a.k_a; p.r_k = a.r_k; p.lnx_w = a.lnx_w; p.lnx_b = a.lnx_b;
  p.state = a.state; p.elapsed = a.elapsed; p.y2 = a.y2; p.shift_src = a.shift_src; p.shift_dst = a.shift_dst;
  p.timeout = timeout_word_or_null();
  const int sum_r = a.R[0] + a.R[1] + a.R[2] + (a.layer0 ? 0 : a.R[3]);
  const size_t smem = static_cast<size_t>(kHead) * (sum_r * 2 + 64) + (a.wkv32 ? 0 : 8192);
  const dim3 grid(a.B * p.H), block(256);
  if (a.wkv32) {
    // always raised: the kernel's static shared memory counts against the default 48 KiB limit as well
    RK_CUDA(cudaFuncSetAttribute(tmix_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RK_CUDA(launch_pdl(tmix_decode_kernel<true>, grid, block, smem, stream, p));
  } else {
    RK_CUDA(cudaFuncSetAttribute(tmix_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RK_CUDA(launch_pdl(tmix_decode_kernel<false>, grid, block, smem, stream, p));
  }
  RK_LAUNCH_CHECK("tmix_decode launch");
  return kOk;
}

}  // namespace rk
