// WKV-7 recurrence for sm_100a: per head, S <- S diag(w) + (S a) b^T + v k^T, y = S r.
//
// State layout (shared with the reference engine and its state cache):
//   [B][H][64 (i: value index)][64 (j: key index)], half or float, updated in place.
// Token tensors r,w,k,v,a,b,y are [B][T][C] half with C = 64 H.
//
// Replaces rwkv7_wkv_fp16_seq_launch / rwkv7_wkv_fp16_seq_w0_launch
// (cuda/rwkv7_wkv_fp16_v2.cu:676-830) and rwkv7_wkv_fp32io16_launch
// (cuda/rwkv7_wkv_fp32_v2.cu:237-294) of the reference.
#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

constexpr float kTwoNeg41 = 4.547473508864641e-13f;
constexpr float kNegExpHalfLog2e = -0.8750387749145276f;  // -exp(-0.5) * log2(e)
constexpr float kNegLog2e = -1.4426950408889634f;

__device__ __forceinline__ float decay_f32(float w) {
  // exp(-exp(-0.5) * sigmoid(w)) in base 2
  return exp2f(kNegExpHalfLog2e / (1.0f + exp2f(kNegLog2e * w)));
}

// ---------------------------------------------------------------------------------------
// fp16 state.  The result is defined operation by operation: every state update is a half2
// fused multiply-add, the two reductions run as two sequential half chains (even and odd j)
// joined by one half add, and the decay carries an integer-hash dither.  One thread owns one
// state row so that those chains are reproduced bit for bit; the 8 KiB tile is staged through
// shared memory with a 16-byte XOR swizzle so that global traffic is fully coalesced and the
// row reads are bank-conflict free.
//
// kWMode: 0 = w holds the decay pre-activation; 1 = w + w0 added in fp32 (no intermediate
// rounding); 2 = half(w + w0) first (what a separate add kernel would produce).
template <int kWMode>
__global__ void __launch_bounds__(64) wkv7_fp16_kernel(
    int T, int C, int H, half* __restrict__ state, const half* __restrict__ r,
    const half* __restrict__ w, const half* __restrict__ w0, const half* __restrict__ k,
    const half* __restrict__ v, const half* __restrict__ a, const half* __restrict__ b,
    half* __restrict__ y, const int* __restrict__ elapsed, int channel0) {
  __shared__ __align__(128) uint4 tile[512];
  __shared__ __align__(16) half vec[2][6][kHead];  // r, w, k, a, b, v
  __shared__ __align__(16) half dvec[kHead];

  const int bh = blockIdx.x;
  const int b_id = bh / H;
  const int h = bh - b_id * H;
  const int i = threadIdx.x;
  half* sbase = state + static_cast<size_t>(bh) * (kHead * kHead);

#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int q = it * 64 + i;
    const int row = q >> 3, c = q & 7;
    cp_async16(&tile[row * 8 + (c ^ (row & 7))], sbase + q * 8);
  }

  const half* srcs[6] = {r, w, k, a, b, v};
  const int vi = i >> 3, chunk = i & 7;
  const half* my_src = nullptr;
#pragma unroll
  for (int s = 0; s < 6; ++s)
    if (vi == s) my_src = srcs[s];
  const size_t tok0 = (static_cast<size_t>(b_id) * T) * C + static_cast<size_t>(h) * kHead;
  if (i < 48) cp_async16(&vec[0][vi][chunk * 8], my_src + tok0 + chunk * 8);
  cp_async_commit();

  const int phase0 = elapsed[b_id] + channel0 + h * kHead + i;  // the dither counts channels of the whole model
  float w0f = 0.f;
  if (kWMode != 0) w0f = __half2float(w0[h * kHead + i]);

  __half2 S[32];
  for (int t = 0; t < T; ++t) {
    const int cur = t & 1;
    cp_async_wait<0>();
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 q = tile[i * 8 + (c ^ (i & 7))];
        S[4 * c + 0] = *reinterpret_cast<const __half2*>(&q.x);
        S[4 * c + 1] = *reinterpret_cast<const __half2*>(&q.y);
        S[4 * c + 2] = *reinterpret_cast<const __half2*>(&q.z);
        S[4 * c + 3] = *reinterpret_cast<const __half2*>(&q.w);
      }
    }
    if (t + 1 < T && i < 48)
      cp_async16(&vec[cur ^ 1][vi][chunk * 8], my_src + tok0 + static_cast<size_t>(t + 1) * C + chunk * 8);
    cp_async_commit();

    const __half2* r2 = reinterpret_cast<const __half2*>(vec[cur][0]);
    const __half2* k2 = reinterpret_cast<const __half2*>(vec[cur][2]);
    const __half2* a2 = reinterpret_cast<const __half2*>(vec[cur][3]);
    const __half2* b2 = reinterpret_cast<const __half2*>(vec[cur][4]);

    __half2 sa2 = __floats2half2_rn(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 32; ++j) sa2 = __hfma2(a2[j], S[j], sa2);
    const half sa = __hadd(__low2half(sa2), __high2half(sa2));
    sa2 = __half2half2(sa);

    {
      float wf = __half2float(vec[cur][1][i]);
      if (kWMode == 1) wf += w0f;
      if (kWMode == 2) wf = __half2float(__float2half_rn(wf + w0f));
      const int rot = static_cast<int>(2654435769u * static_cast<unsigned>(phase0 + t));
      const float d = exp2f(kNegExpHalfLog2e / (1.0f + exp2f(kNegLog2e * wf))) - 1.0f +
                      kTwoNeg41 * static_cast<float>(rot);
      dvec[i] = __float2half_rn(d);
    }
    __syncthreads();

    const __half2* d2 = reinterpret_cast<const __half2*>(dvec);
    const __half2 vv2 = __half2half2(vec[cur][5][i]);
    __half2 y2 = __floats2half2_rn(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      __half2 s = S[j];
      s = __hfma2(s, d2[j], __hfma2(k2[j], vv2, __hfma2(sa2, b2[j], s)));
      S[j] = s;
      y2 = __hfma2(s, r2[j], y2);
    }
    y[tok0 + static_cast<size_t>(t) * C + i] = __hadd(__low2half(y2), __high2half(y2));
  }

#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = *reinterpret_cast<const uint32_t*>(&S[4 * c + 0]);
    q.y = *reinterpret_cast<const uint32_t*>(&S[4 * c + 1]);
    q.z = *reinterpret_cast<const uint32_t*>(&S[4 * c + 2]);
    q.w = *reinterpret_cast<const uint32_t*>(&S[4 * c + 3]);
    tile[i * 8 + (c ^ (i & 7))] = q;
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int q = it * 64 + i;
    const int row = q >> 3, c = q & 7;
    reinterpret_cast<uint4*>(sbase)[q] = tile[row * 8 + (c ^ (row & 7))];
  }
}

// ---------------------------------------------------------------------------------------
// fp32 state, one token (decode).  HBM-bound: 32 KiB of state traffic per head and ~1 KiB of
// vectors.  16 lanes share one state row as float4s, so every load and store is a fully
// coalesced 512-byte warp transaction straight between HBM and registers; the two reductions
// are 4-step shuffles inside the 16-lane group.
// kAddW0: w0 is added to w and the sum rounded to half before the decay.
template <bool kAddW0>
__global__ void __launch_bounds__(256) wkv7_fp32_decode_kernel(
    int C, int H, float* __restrict__ state, const half* __restrict__ r, const half* __restrict__ w,
    const half* __restrict__ w0, const half* __restrict__ k, const half* __restrict__ v,
    const half* __restrict__ a, const half* __restrict__ b, half* __restrict__ y) {
  const int bh = blockIdx.x;
  const int b_id = bh / H;
  const int h = bh - b_id * H;
  const int tid = threadIdx.x;
  const int c4 = tid & 15;       // which float4 of the row
  const int rsub = tid >> 4;     // row within a pass of 16 rows
  float4* sbase = reinterpret_cast<float4*>(state + static_cast<size_t>(bh) * (kHead * kHead));
  const size_t tok = static_cast<size_t>(b_id) * C + static_cast<size_t>(h) * kHead;

  float4 S[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) S[p] = sbase[(p * 16 + rsub) * 16 + c4];

  auto ld4 = [&](const half* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p + tok + c4 * 4);
    const float2 lo = h2f2(u.x), hi = h2f2(u.y);
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  };
  const float4 rr = ld4(r), kk = ld4(k), aa = ld4(a), bb = ld4(b);
  float4 ww = ld4(w);
  if (kAddW0) {
    const uint2 u = *reinterpret_cast<const uint2*>(w0 + h * kHead + c4 * 4);
    const float2 lo = h2f2(u.x), hi = h2f2(u.y);
    ww.x = __half2float(__float2half_rn(ww.x + lo.x));
    ww.y = __half2float(__float2half_rn(ww.y + lo.y));
    ww.z = __half2float(__float2half_rn(ww.z + hi.x));
    ww.w = __half2float(__float2half_rn(ww.w + hi.y));
  }
  ww.x = decay_f32(ww.x); ww.y = decay_f32(ww.y); ww.z = decay_f32(ww.z); ww.w = decay_f32(ww.w);

#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int row = p * 16 + rsub;
    float4 s = S[p];
    float sa = s.x * aa.x + s.y * aa.y + s.z * aa.z + s.w * aa.w;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sa += __shfl_xor_sync(0xffffffffu, sa, o);
    const float vi = __half2float(v[tok + row]);
    s.x = s.x * ww.x + sa * bb.x + kk.x * vi;
    s.y = s.y * ww.y + sa * bb.y + kk.y * vi;
    s.z = s.z * ww.z + sa * bb.z + kk.z * vi;
    s.w = s.w * ww.w + sa * bb.w + kk.w * vi;
    float yy = s.x * rr.x + s.y * rr.y + s.z * rr.z + s.w * rr.w;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) yy += __shfl_xor_sync(0xffffffffu, yy, o);
    sbase[row * 16 + c4] = s;
    if (c4 == 0) y[tok + row] = __float2half_rn(yy);
  }
}

// ---------------------------------------------------------------------------------------
// fp32 state, T tokens (prefill chunks).  Sequential in t.  A thread owns two rows x 16 columns of the state in
// registers for the whole chunk; four lanes share a row pair, so each reduction is a 2-step shuffle.  (Every
// thread reads the 16 columns' worth of five token vectors from shared memory per step; with one row per thread
// that traffic, not the arithmetic, sets the step time -- two rows per thread halve it.)  A CTA covers kRows rows
// of one head: 64, or 32 when there are few heads, so that a head's two halves run on two SMs.
// Token vectors are staged eight tokens at a time: every thread fetches its share of the NEXT block into
// registers before it computes the current block (the global-memory latency hides behind eight recurrence
// steps), then converts it into a double-buffered fp32 block in shared memory (segments padded by 4 floats so
// the four lanes' float4 reads hit distinct banks).  One barrier per block; the steps inside a block only
// exchange data through shuffles.
template <bool kAddW0, int kRows>
__global__ void __launch_bounds__(kRows * 2) wkv7_fp32_scan_kernel(
    int T, int C, int H, float* __restrict__ state, const half* __restrict__ r,
    const half* __restrict__ w, const half* __restrict__ w0, const half* __restrict__ k,
    const half* __restrict__ v, const half* __restrict__ a, const half* __restrict__ b,
    half* __restrict__ y) {
  constexpr int kSeg = 20;   // 16 floats + 4 pad
  constexpr int kBlk = 8;    // tokens per staged block
  constexpr int kThreads = kRows * 2;
  constexpr int kSlots = kBlk * (kHead / 2) / kThreads;  // half2 slots of a block each thread stages (per vector)
  constexpr int kParts = kHead / kRows;                  // CTAs per head
  __shared__ __align__(16) float vecs[2][5][kBlk][4 * kSeg];  // r, decay, k, a, b
  __shared__ __align__(8) float vsm[2][kBlk][kHead];

  const int bh = blockIdx.x / kParts;
  const int part = blockIdx.x - bh * kParts;
  const int b_id = bh / H;
  const int h = bh - b_id * H;
  const int tid = threadIdx.x;
  const int row = part * kRows + (tid >> 2) * 2, q = tid & 3;   // rows row, row + 1
  float* srow = state + static_cast<size_t>(bh) * (kHead * kHead) + row * kHead + q * 16;
  const size_t tok0 = (static_cast<size_t>(b_id) * T) * C + static_cast<size_t>(h) * kHead;

  __half2 pre[kSlots][6];
  float2 w0f[kSlots];
#pragma unroll
  for (int i = 0; i < kSlots; ++i) {
    const int ch = ((tid + i * kThreads) & 31) * 2;
    w0f[i] = kAddW0 ? __half22float2(*reinterpret_cast<const __half2*>(w0 + h * kHead + ch)) : make_float2(0.f, 0.f);
  }
  auto fetch = [&](int t_first) {
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      const int slot = tid + i * kThreads;  // token slot / 32 of the block, channels 2 * (slot % 32) and + 1
      const int t = t_first + (slot >> 5);
      if (t < T) {
        const size_t idx = tok0 + static_cast<size_t>(t) * C + (slot & 31) * 2;
        pre[i][0] = *reinterpret_cast<const __half2*>(r + idx);
        pre[i][1] = *reinterpret_cast<const __half2*>(w + idx);
        pre[i][2] = *reinterpret_cast<const __half2*>(k + idx);
        pre[i][3] = *reinterpret_cast<const __half2*>(a + idx);
        pre[i][4] = *reinterpret_cast<const __half2*>(b + idx);
        pre[i][5] = *reinterpret_cast<const __half2*>(v + idx);
      }
    }
  };
  auto put = [&](int buf) {
#pragma unroll
    for (int i = 0; i < kSlots; ++i) {
      const int slot = tid + i * kThreads;
      const int tok = slot >> 5, ch = (slot & 31) * 2;
      const int pos = (ch >> 4) * kSeg + (ch & 15);
      float2 wf = __half22float2(pre[i][1]);
      if (kAddW0) {
        wf.x = __half2float(__float2half_rn(wf.x + w0f[i].x));
        wf.y = __half2float(__float2half_rn(wf.y + w0f[i].y));
      }
      *reinterpret_cast<float2*>(&vecs[buf][0][tok][pos]) = __half22float2(pre[i][0]);
      *reinterpret_cast<float2*>(&vecs[buf][1][tok][pos]) = make_float2(decay_f32(wf.x), decay_f32(wf.y));
      *reinterpret_cast<float2*>(&vecs[buf][2][tok][pos]) = __half22float2(pre[i][2]);
      *reinterpret_cast<float2*>(&vecs[buf][3][tok][pos]) = __half22float2(pre[i][3]);
      *reinterpret_cast<float2*>(&vecs[buf][4][tok][pos]) = __half22float2(pre[i][4]);
      *reinterpret_cast<float2*>(&vsm[buf][tok][ch]) = __half22float2(pre[i][5]);
    }
  };

  fetch(0);
  float S0[16], S1[16];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float4 t0 = reinterpret_cast<const float4*>(srow)[c];
    const float4 t1 = reinterpret_cast<const float4*>(srow + kHead)[c];
    S0[4 * c] = t0.x; S0[4 * c + 1] = t0.y; S0[4 * c + 2] = t0.z; S0[4 * c + 3] = t0.w;
    S1[4 * c] = t1.x; S1[4 * c + 1] = t1.y; S1[4 * c + 2] = t1.z; S1[4 * c + 3] = t1.w;
  }

  int buf = 0;
  for (int t0 = 0; t0 < T; t0 += kBlk, buf ^= 1) {
    put(buf);          // tokens t0 .. t0+7 (slots of tokens >= T hold stale values and are not used)
    __syncthreads();   // also: every warp has finished the block before last, which used this buffer
    if (t0 + kBlk < T) fetch(t0 + kBlk);
    const int n_here = min(kBlk, T - t0);
    for (int tl = 0; tl < n_here; ++tl) {  // (fully unrolling the block and splitting the sums measured slower)
      const float* rv = &vecs[buf][0][tl][q * kSeg];
      const float* wv = &vecs[buf][1][tl][q * kSeg];
      const float* kv = &vecs[buf][2][tl][q * kSeg];
      const float* av = &vecs[buf][3][tl][q * kSeg];
      const float* bv = &vecs[buf][4][tl][q * kSeg];
      float sa0 = 0.f, sa1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float aj = av[j];
        sa0 = fmaf(S0[j], aj, sa0);
        sa1 = fmaf(S1[j], aj, sa1);
      }
      sa0 += __shfl_xor_sync(0xffffffffu, sa0, 1);
      sa1 += __shfl_xor_sync(0xffffffffu, sa1, 1);
      sa0 += __shfl_xor_sync(0xffffffffu, sa0, 2);
      sa1 += __shfl_xor_sync(0xffffffffu, sa1, 2);
      const float2 vi = *reinterpret_cast<const float2*>(&vsm[buf][tl][row]);
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float wj = wv[j], bj = bv[j], kj = kv[j], rj = rv[j];
        const float s0 = S0[j] * wj + sa0 * bj + kj * vi.x;
        const float s1 = S1[j] * wj + sa1 * bj + kj * vi.y;
        S0[j] = s0;
        S1[j] = s1;
        y0 = fmaf(s0, rj, y0);
        y1 = fmaf(s1, rj, y1);
      }
      y0 += __shfl_xor_sync(0xffffffffu, y0, 1);
      y1 += __shfl_xor_sync(0xffffffffu, y1, 1);
      y0 += __shfl_xor_sync(0xffffffffu, y0, 2);
      y1 += __shfl_xor_sync(0xffffffffu, y1, 2);
      if (q == 0)
        *reinterpret_cast<__half2*>(y + tok0 + static_cast<size_t>(t0 + tl) * C + row) = __floats2half2_rn(y0, y1);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    reinterpret_cast<float4*>(srow)[c] = make_float4(S0[4 * c], S0[4 * c + 1], S0[4 * c + 2], S0[4 * c + 3]);
    reinterpret_cast<float4*>(srow + kHead)[c] = make_float4(S1[4 * c], S1[4 * c + 1], S1[4 * c + 2], S1[4 * c + 3]);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int wkv7_fp16(cudaStream_t stream, int B, int T, int C, int H, half* state, const half* r, const half* w,
              const half* w0, int w_mode, const half* k, const half* v, const half* a, const half* b,
              half* y, const int* elapsed, int channel0) {
  RK_REQUIRE(B > 0 && T > 0 && H > 0 && C == H * kHead, kShape, "wkv7_fp16: need B,T,H > 0 and C == 64*H");
  RK_REQUIRE(state && r && w && k && v && a && b && y && elapsed, kBadArg, "wkv7_fp16: null pointer");
  RK_REQUIRE(w_mode == 0 || w0, kBadArg, "wkv7_fp16: w0 required for w_mode %d", w_mode);
  RK_REQUIRE(aligned16(state) && aligned16(r) && aligned16(w) && aligned16(k) && aligned16(v) && aligned16(a) &&
                 aligned16(b), kBadArg, "wkv7_fp16: tensors must be 16-byte aligned");
  const dim3 grid(B * H), block(64);
  if (w_mode == 0) wkv7_fp16_kernel<0><<<grid, block, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y, elapsed, channel0);
  else if (w_mode == 1) wkv7_fp16_kernel<1><<<grid, block, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y, elapsed, channel0);
  else if (w_mode == 2) wkv7_fp16_kernel<2><<<grid, block, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y, elapsed, channel0);
  else RK_REQUIRE(false, kBadArg, "wkv7_fp16: w_mode must be 0, 1 or 2");
  RK_LAUNCH_CHECK("wkv7_fp16 launch");
  return kOk;
}

int wkv7_fp32(cudaStream_t stream, int B, int T, int C, int H, float* state, const half* r, const half* w,
              const half* w0, const half* k, const half* v, const half* a, const half* b, half* y) {
  RK_REQUIRE(B > 0 && T > 0 && H > 0 && C == H * kHead, kShape, "wkv7_fp32: need B,T,H > 0 and C == 64*H");
  RK_REQUIRE(state && r && w && k && v && a && b && y, kBadArg, "wkv7_fp32: null pointer");
  RK_REQUIRE(aligned16(state) && aligned16(r) && aligned16(w) && aligned16(k) && aligned16(a) && aligned16(b),
             kBadArg, "wkv7_fp32: tensors must be 16-byte aligned");
  if (wkv7_fp32_chunked_applies(T) && options().wkv_chunked) return wkv7_fp32_chunked(stream, B, T, C, H, state, r, w, w0, k, v, a, b, y);
  const dim3 grid(B * H), block(256);
  if (T == 1) {
    if (w0) wkv7_fp32_decode_kernel<true><<<grid, block, 0, stream>>>(C, H, state, r, w, w0, k, v, a, b, y);
    else wkv7_fp32_decode_kernel<false><<<grid, block, 0, stream>>>(C, H, state, r, w, w0, k, v, a, b, y);
  } else {
    // few heads: two CTAs per head, so that the sequential scan spreads over twice as many SMs
    if (B * H <= 160) {
      const dim3 g2(B * H * 2), b2(64);
      if (w0) wkv7_fp32_scan_kernel<true, 32><<<g2, b2, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y);
      else wkv7_fp32_scan_kernel<false, 32><<<g2, b2, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y);
    } else {
      const dim3 b1(128);
      if (w0) wkv7_fp32_scan_kernel<true, 64><<<grid, b1, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y);
      else wkv7_fp32_scan_kernel<false, 64><<<grid, b1, 0, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y);
    }
  }
  RK_LAUNCH_CHECK("wkv7_fp32 launch");
  return kOk;
}

}  // namespace rk
