// Row-wise fusions of the RWKV-7 forward: embedding gather, residual add, LayerNorm and the
// token-shift interpolations, plus the small per-head gates around the WKV recurrence.
//
// One kernel (row_op_kernel) covers what the reference spreads over
//   layer_norm_f16 / add_layer_norm_f16 / add_last_layer_norm_f16        cuda/rwkv7_v3a_ops.cu:1272-1351,1800-1931
//   add_layer_norm_cmix_mix_f16 / add_layer_norm_tmix_mix6_f16 (T=1)     cuda/rwkv7_v3a_ops.cu:1515-2060
//   tmix_mix6 / cmix_mix / update_shift_state_last                       cuda/rwkv7_fast_ops_fp16.cu:53-127,393-419
// for every T: a CTA normalises its own row and, when t > 0, re-normalises row t-1 as the
// "previous token" instead of waiting for another CTA; the CTAs of t = 0 alone read and then
// replace the shift state, so no second launch is needed.  Rows live in registers (no shared-memory
// staging) and a row may be split over several CTAs so that a decode step's single row does not
// serialise on one SM.
// Rounding points follow the reference: the sum x + residual and the LayerNorm output are each
// rounded to half once, the interpolation reads the rounded LayerNorm output.
#include "common.cuh"
#include <algorithm>
#include <cstdlib>

#include "kernels.h"

namespace rk {
namespace {

constexpr int kRowThreads = 256;

struct RowOpDev {
  int B, T, C, vocab, n_mix, last_only, identity, n_slices;
  float eps;
  const int64_t* tokens;
  const half* table;
  const half* x;
  const half* residual;
  const float* residual_f32;  // alternative residual: fp32 sums, rounded to half before they are added
  half* x_out;
  const half* ln_w;
  const half* ln_b;
  half* n_out;
  half* shift;
  const half* mix[6];
  half* mix_out[6];
  int* bad_token_flag;
};

// A thread owns the channel pairs q = tid + 256 i, i < kPairs, of a row, in registers.
// Loads row (b,t) as fp32 (x + residual, or the gathered embedding row).
template <int kPairs>
__device__ __forceinline__ void load_row(const RowOpDev& p, int b, int t, float2 (&v)[kPairs]) {
  const size_t row = static_cast<size_t>(b) * p.T + t;
  const int pairs = p.C >> 1;
  if (p.table) {
    long long tok = p.tokens[row];
    if (tok < 0 || tok >= p.vocab) {
      if (threadIdx.x == 0 && p.bad_token_flag) *p.bad_token_flag = 1;
      tok = 0;
    }
    const __half2* src = reinterpret_cast<const __half2*>(p.table + static_cast<size_t>(tok) * p.C);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const int q = threadIdx.x + kRowThreads * i;
      v[i] = q < pairs ? __half22float2(src[q]) : make_float2(0.f, 0.f);
    }
  } else {
    const __half2* xs = reinterpret_cast<const __half2*>(p.x + row * p.C);
    const __half2* rs = p.residual ? reinterpret_cast<const __half2*>(p.residual + row * p.C) : nullptr;
    const float2* rf = p.residual_f32 ? reinterpret_cast<const float2*>(p.residual_f32 + row * p.C) : nullptr;
    __half2 xv[kPairs], rv[kPairs];
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const int q = threadIdx.x + kRowThreads * i;
      xv[i] = q < pairs ? xs[q] : __floats2half2_rn(0.f, 0.f);
      rv[i] = (rs && q < pairs) ? rs[q] : __floats2half2_rn(0.f, 0.f);
      if (rf && q < pairs) {
        const float2 t = rf[q];
        rv[i] = __floats2half2_rn(t.x, t.y);
      }
    }
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const float2 a = __half22float2(xv[i]), r = __half22float2(rv[i]);
      v[i] = make_float2(a.x + r.x, a.y + r.y);
    }
  }
}

// In place: v <- float(half(LN(v))).  Two-pass statistics in fp32 over the whole row.
// Statistics cover the whole row; only the pairs i in [i_lo, i_hi) (whose weights lw/lb were
// prefetched) are normalised, the others are left as they are and not used afterwards.
template <int kPairs>
__device__ __forceinline__ void ln_row(const RowOpDev& p, float2 (&v)[kPairs], float* scratch,
                                       const __half2 (&lw)[kPairs], const __half2 (&lb)[kPairs], int i_lo, int i_hi) {
  if (p.identity) return;  // plain token shift: the row is used as it is
  const int pairs = p.C >> 1;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kPairs; ++i) s += v[i].x + v[i].y;  // absent pairs hold zeros
  const float inv_c = 1.0f / static_cast<float>(p.C);
  const float mean = block_sum<kRowThreads>(s, scratch) * inv_c;
  float sv = 0.f;
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    if (threadIdx.x + kRowThreads * i < pairs) {
      const float d0 = v[i].x - mean, d1 = v[i].y - mean;
      sv += d0 * d0 + d1 * d1;
    }
  }
  const float rstd = rsqrtf(block_sum<kRowThreads>(sv, scratch) * inv_c + p.eps);
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int q = threadIdx.x + kRowThreads * i;
    if (q < pairs && i >= i_lo && i < i_hi) {
      const float2 w = __half22float2(lw[i]);
      const float2 b = __half22float2(lb[i]);
      v[i] = __half22float2(__floats2half2_rn((v[i].x - mean) * rstd * w.x + b.x, (v[i].y - mean) * rstd * w.y + b.y));
    }
  }
}

// grid = (n_slices, rows).  Every CTA computes the statistics of its whole row; slice s writes the
// outputs of pairs i in [s*kPairs/n_slices, (s+1)*kPairs/n_slices) so that a single decode row is
// spread over several SMs.
template <int kPairs>
__device__ __forceinline__ void row_op_body(const RowOpDev& p) {
  __shared__ float scratch[kRowThreads / 32];
  int b, t;
  if (p.last_only) {
    b = blockIdx.y;
    t = p.T - 1;
  } else {
    b = blockIdx.y / p.T;
    t = blockIdx.y - b * p.T;
  }
  const size_t row = static_cast<size_t>(b) * p.T + t;
  const int pairs = p.C >> 1;
  const int per = kPairs / p.n_slices;
  const int i_lo = blockIdx.x * per, i_hi = i_lo + per;
  auto owned = [&](int i) { return i >= i_lo && i < i_hi && threadIdx.x + kRowThreads * i < pairs; };

  // Weights, and the shift row (last written one step ago), are requested before the dependency wait.
  __half2 lw[kPairs], lb[kPairs], mixv[kPairs][6];
  float2 prev[kPairs];
  __half2* shift2 = p.shift ? reinterpret_cast<__half2*>(p.shift + static_cast<size_t>(b) * p.C) : nullptr;
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int q = threadIdx.x + kRowThreads * i;
    prev[i] = make_float2(0.f, 0.f);
    if (!owned(i)) continue;
    if (p.ln_w) {
      lw[i] = reinterpret_cast<const __half2*>(p.ln_w)[q];
      lb[i] = reinterpret_cast<const __half2*>(p.ln_b)[q];
    }
#pragma unroll
    for (int m = 0; m < 6; ++m)
      if (m < p.n_mix) mixv[i][m] = reinterpret_cast<const __half2*>(p.mix[m])[q];
    if (p.n_mix && t == 0) prev[i] = __half22float2(shift2[q]);
  }
  pdl_wait();
  pdl_trigger();
  float2 cur[kPairs];
  load_row<kPairs>(p, b, t, cur);
  if (p.x_out) {
#pragma unroll
    for (int i = 0; i < kPairs; ++i)
      if (owned(i)) reinterpret_cast<__half2*>(p.x_out + row * p.C)[threadIdx.x + kRowThreads * i] = __floats2half2_rn(cur[i].x, cur[i].y);
  }
  if (!p.ln_w && !p.identity) return;
  ln_row<kPairs>(p, cur, scratch, lw, lb, i_lo, i_hi);
  if (p.n_out) {
    half* dst = p.n_out + (p.last_only ? static_cast<size_t>(b) : row) * p.C;
#pragma unroll
    for (int i = 0; i < kPairs; ++i)
      if (owned(i)) reinterpret_cast<__half2*>(dst)[threadIdx.x + kRowThreads * i] = __floats2half2_rn(cur[i].x, cur[i].y);
  }
  if (p.n_mix == 0) return;

  if (t != 0) {
    load_row<kPairs>(p, b, t - 1, prev);
    ln_row<kPairs>(p, prev, scratch, lw, lb, i_lo, i_hi);
  }
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    if (!owned(i)) continue;
    const float dx0 = prev[i].x - cur[i].x, dx1 = prev[i].y - cur[i].y;
#pragma unroll
    for (int m = 0; m < 6; ++m) {
      if (m < p.n_mix) {
        const float2 c = __half22float2(mixv[i][m]);
        reinterpret_cast<__half2*>(p.mix_out[m] + row * p.C)[threadIdx.x + kRowThreads * i] =
            __floats2half2_rn(cur[i].x + dx0 * c.x, cur[i].y + dx1 * c.y);
      }
    }
  }
  if (t == 0) {
    // only the CTAs of t == 0 touch shift[b]; each has consumed its old pairs above
    if (p.T > 1) {
      load_row<kPairs>(p, b, p.T - 1, cur);
      ln_row<kPairs>(p, cur, scratch, lw, lb, i_lo, i_hi);
    }
#pragma unroll
    for (int i = 0; i < kPairs; ++i)
      if (owned(i)) shift2[threadIdx.x + kRowThreads * i] = __floats2half2_rn(cur[i].x, cur[i].y);
  }
}

template <int kPairs>
__global__ void __launch_bounds__(kRowThreads) row_op_kernel(const RowOpDev p) {
  row_op_body<kPairs>(p);
}

// The same kernel compiled for at most 128 registers, so that two CTAs share an SM: for launches with more rows than
// SMs (batched decode), where one CTA per SM means a second wave.
template <int kPairs>
__global__ void __launch_bounds__(kRowThreads, 2) row_op_two_per_sm_kernel(const RowOpDev p) {
  row_op_body<kPairs>(p);
}

// ---- Chunks (T > 1) with many rows.  512 threads per row, so that a thread holds half as many pairs, and the
// second row a CTA needs -- the previous token (t > 0), or the chunk's last token, which the CTAs of t == 0 store as
// the new shift state -- is loaded together with its own row and normalised in the same chain of reductions.
constexpr int kChunkThreads = 512;

template <int kPairs>
__device__ __forceinline__ void load_row_chunk(const RowOpDev& p, int b, int t, float2 (&v)[kPairs]) {
  const size_t row = static_cast<size_t>(b) * p.T + t;
  const int pairs = p.C >> 1;
  const __half2* xs = reinterpret_cast<const __half2*>(p.x + row * p.C);
  const __half2* rs = p.residual ? reinterpret_cast<const __half2*>(p.residual + row * p.C) : nullptr;
  const float2* rf = p.residual_f32 ? reinterpret_cast<const float2*>(p.residual_f32 + row * p.C) : nullptr;
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int q = threadIdx.x + kChunkThreads * i;
    float2 a = make_float2(0.f, 0.f), r = make_float2(0.f, 0.f);
    if (q < pairs) {
      a = __half22float2(xs[q]);
      if (rs) r = __half22float2(rs[q]);
      if (rf) {
        const float2 t2 = rf[q];
        r = __half22float2(__floats2half2_rn(t2.x, t2.y));
      }
    }
    v[i] = make_float2(a.x + r.x, a.y + r.y);
  }
}

// Sums two values over the CTA with one pair of barriers; every thread receives both totals.
__device__ __forceinline__ float2 block_sum2_chunk(float a, float b, float* scratch /* 2 * kChunkThreads/32 floats */) {
  a = warp_sum(a);
  b = warp_sum(b);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) {
    scratch[warp] = a;
    scratch[kChunkThreads / 32 + warp] = b;
  }
  __syncthreads();
  float ta = 0.f, tb = 0.f;
#pragma unroll
  for (int w = 0; w < kChunkThreads / 32; ++w) {
    ta += scratch[w];
    tb += scratch[kChunkThreads / 32 + w];
  }
  return make_float2(ta, tb);
}

// grid = rows.  Needs x (not the embedding table), LayerNorm weights or identity, n_mix > 0, not last_only.
template <int kPairs>
__global__ void __launch_bounds__(kChunkThreads) row_op_chunk_kernel(const RowOpDev p) {
  __shared__ float scratch[2 * kChunkThreads / 32];
  const int b = blockIdx.x / p.T, t = blockIdx.x - b * p.T;
  const size_t row = static_cast<size_t>(b) * p.T + t;
  const int pairs = p.C >> 1;
  __half2 lw[kPairs], lb[kPairs], mixv[kPairs][6];
  float2 prev[kPairs];
  __half2* shift2 = reinterpret_cast<__half2*>(p.shift + static_cast<size_t>(b) * p.C);
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int q = threadIdx.x + kChunkThreads * i;
    prev[i] = make_float2(0.f, 0.f);
    if (q >= pairs) continue;
    if (p.ln_w) {
      lw[i] = reinterpret_cast<const __half2*>(p.ln_w)[q];
      lb[i] = reinterpret_cast<const __half2*>(p.ln_b)[q];
    }
#pragma unroll
    for (int m = 0; m < 6; ++m)
      if (m < p.n_mix) mixv[i][m] = reinterpret_cast<const __half2*>(p.mix[m])[q];
    if (t == 0) prev[i] = __half22float2(shift2[q]);  // last written one launch ago at the latest
  }
  pdl_wait();
  pdl_trigger();
  float2 cur[kPairs], oth[kPairs];
  load_row_chunk<kPairs>(p, b, t, cur);
  load_row_chunk<kPairs>(p, b, t != 0 ? t - 1 : p.T - 1, oth);
  if (p.x_out) {
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const int q = threadIdx.x + kChunkThreads * i;
      if (q < pairs) reinterpret_cast<__half2*>(p.x_out + row * p.C)[q] = __floats2half2_rn(cur[i].x, cur[i].y);
    }
  }
  if (!p.identity) {
    float s = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {  // absent pairs hold zeros
      s += cur[i].x + cur[i].y;
      s2 += oth[i].x + oth[i].y;
    }
    const float inv_c = 1.0f / static_cast<float>(p.C);
    float2 mean = block_sum2_chunk(s, s2, scratch);
    mean.x *= inv_c;
    mean.y *= inv_c;
    float sv = 0.f, sv2 = 0.f;
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      if (threadIdx.x + kChunkThreads * i < pairs) {
        const float d0 = cur[i].x - mean.x, d1 = cur[i].y - mean.x;
        sv += d0 * d0 + d1 * d1;
        const float e0 = oth[i].x - mean.y, e1 = oth[i].y - mean.y;
        sv2 += e0 * e0 + e1 * e1;
      }
    }
    const float2 var = block_sum2_chunk(sv, sv2, scratch);
    const float rstd = rsqrtf(var.x * inv_c + p.eps), rstd2 = rsqrtf(var.y * inv_c + p.eps);
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      if (threadIdx.x + kChunkThreads * i < pairs) {
        const float2 w = __half22float2(lw[i]);
        const float2 bb = __half22float2(lb[i]);
        cur[i] = __half22float2(__floats2half2_rn((cur[i].x - mean.x) * rstd * w.x + bb.x, (cur[i].y - mean.x) * rstd * w.y + bb.y));
        oth[i] = __half22float2(__floats2half2_rn((oth[i].x - mean.y) * rstd2 * w.x + bb.x, (oth[i].y - mean.y) * rstd2 * w.y + bb.y));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kPairs; ++i) {
    const int q = threadIdx.x + kChunkThreads * i;
    if (q >= pairs) continue;
    if (p.n_out) reinterpret_cast<__half2*>(p.n_out + row * p.C)[q] = __floats2half2_rn(cur[i].x, cur[i].y);
    const float2 pv = t != 0 ? oth[i] : prev[i];
    const float dx0 = pv.x - cur[i].x, dx1 = pv.y - cur[i].y;
#pragma unroll
    for (int m = 0; m < 6; ++m) {
      if (m < p.n_mix) {
        const float2 c = __half22float2(mixv[i][m]);
        reinterpret_cast<__half2*>(p.mix_out[m] + row * p.C)[q] = __floats2half2_rn(cur[i].x + dx0 * c.x, cur[i].y + dx1 * c.y);
      }
    }
    // only the CTAs of t == 0 touch shift[b]; each has consumed its old pairs above
    if (t == 0) shift2[q] = __floats2half2_rn(oth[i].x, oth[i].y);
  }
}

// kk = normalize(k * k_k) per head, a = sigmoid(a0 + a12), k' = k (1 + (a - 1) k_a);
// emits k', -kk and kk*a (the WKV "a" and "b" operands).  One warp per (row, head).
// Reference: tmix_kk_a_gate_kernel, cuda/rwkv7_fast_ops_fp16.cu:129-172.
__global__ void __launch_bounds__(128) kk_a_gate_kernel(
    int H, long long n_heads_total, const half* __restrict__ k, const half* __restrict__ k_k,
    const half* __restrict__ a0, const half* __restrict__ a12, const half* __restrict__ k_a,
    half* __restrict__ new_k, half* __restrict__ neg_kk, half* __restrict__ kka,
    // optional second job for the same channels: the value-residual gate (vres_gate_kernel's formula)
    const half* __restrict__ v, const half* __restrict__ v_first, const half* __restrict__ v0,
    const half* __restrict__ v12, half* __restrict__ v_out) {
  const long long bth = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (bth >= n_heads_total) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(bth % H);
  const long long idx = bth * kHead + lane * 2;
  const int c = h * kHead + lane * 2;
  if (v_out) {
    const float2 vv = __half22float2(*reinterpret_cast<const __half2*>(v + idx));
    const float2 vf = __half22float2(*reinterpret_cast<const __half2*>(v_first + idx));
    const float2 b0 = __half22float2(*reinterpret_cast<const __half2*>(v0 + c));
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(v12 + idx));
    const float g0 = sigmoid_fast(b0.x + lo.x), g1 = sigmoid_fast(b0.y + lo.y);
    *reinterpret_cast<__half2*>(v_out + idx) = __floats2half2_rn(fmaf(vf.x - vv.x, g0, vv.x), fmaf(vf.y - vv.y, g1, vv.y));
  }
  const float2 kv = __half22float2(*reinterpret_cast<const __half2*>(k + idx));
  const float2 ks = __half22float2(*reinterpret_cast<const __half2*>(k_k + c));
  const float u0 = kv.x * ks.x, u1 = kv.y * ks.y;
  const float total = warp_sum(u0 * u0 + u1 * u1);
  const float inv_d = 1.0f / fmaxf(sqrtf(total), 1.0e-12f);
  const float kk0 = u0 * inv_d, kk1 = u1 * inv_d;
  const float2 a0v = __half22float2(*reinterpret_cast<const __half2*>(a0 + c));
  const float2 a12v = __half22float2(*reinterpret_cast<const __half2*>(a12 + idx));
  const float av0 = sigmoid_fast(a0v.x + a12v.x), av1 = sigmoid_fast(a0v.y + a12v.y);
  const float2 ka = __half22float2(*reinterpret_cast<const __half2*>(k_a + c));
  *reinterpret_cast<__half2*>(new_k + idx) =
      __floats2half2_rn(kv.x * fmaf(av0, ka.x, 1.0f - ka.x), kv.y * fmaf(av1, ka.y, 1.0f - ka.y));
  *reinterpret_cast<__half2*>(neg_kk + idx) = __floats2half2_rn(-kk0, -kk1);
  *reinterpret_cast<__half2*>(kka + idx) = __floats2half2_rn(kk0 * av0, kk1 * av1);
}

// out = (GroupNorm_64(y; eps 64e-5) * w + b + (sum_j r k r_k) v) * g.  One warp per (row, head).
// Reference: tmix_lnx_rkvres_xg_kernel, cuda/rwkv7_fast_ops_fp16.cu:174-237.
__global__ void __launch_bounds__(128) lnx_rkvres_xg_kernel(
    int H, long long n_heads_total, const half* __restrict__ y, const half* __restrict__ r,
    const half* __restrict__ k, const half* __restrict__ v, const half* __restrict__ r_k,
    const half* __restrict__ w, const half* __restrict__ b, const half* __restrict__ g,
    half* __restrict__ out) {
  const long long bth = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (bth >= n_heads_total) return;
  const int lane = threadIdx.x & 31;
  const int h = static_cast<int>(bth % H);
  const long long idx = bth * kHead + lane * 2;
  const int c = h * kHead + lane * 2;
  const float2 yv = __half22float2(*reinterpret_cast<const __half2*>(y + idx));
  const float mean = warp_sum(yv.x + yv.y) * (1.0f / 64.0f);
  const float d0 = yv.x - mean, d1 = yv.y - mean;
  const float var = warp_sum(d0 * d0 + d1 * d1) * (1.0f / 64.0f);
  const float rstd = rsqrtf(var + 64.0e-5f);
  const float2 rv = __half22float2(*reinterpret_cast<const __half2*>(r + idx));
  const float2 kv = __half22float2(*reinterpret_cast<const __half2*>(k + idx));
  const float2 vv = __half22float2(*reinterpret_cast<const __half2*>(v + idx));
  const float2 rk = __half22float2(*reinterpret_cast<const __half2*>(r_k + c));
  const float rkv = warp_sum(rv.x * kv.x * rk.x + rv.y * kv.y * rk.y);
  const float2 wv = __half22float2(*reinterpret_cast<const __half2*>(w + c));
  const float2 bv = __half22float2(*reinterpret_cast<const __half2*>(b + c));
  const float2 gv = __half22float2(*reinterpret_cast<const __half2*>(g + idx));
  *reinterpret_cast<__half2*>(out + idx) = __floats2half2_rn(
      (d0 * rstd * wv.x + bv.x + rkv * vv.x) * gv.x, (d1 * rstd * wv.y + bv.y + rkv * vv.y) * gv.y);
}

// Reference: tmix_vres_gate_kernel, cuda/rwkv7_fast_ops_fp16.cu:239-255.
__global__ void vres_gate_kernel(int C, long long total, const half* __restrict__ v,
                                 const half* __restrict__ v_first, const half* __restrict__ v0,
                                 const half* __restrict__ v12, half* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % C);
  const float vv = __half2float(v[i]);
  const float gate = sigmoid_fast(__half2float(v0[c]) + __half2float(v12[i]));
  out[i] = __float2half_rn(fmaf(__half2float(v_first[i]) - vv, gate, vv));
}

__global__ void advance_i32_kernel(int* x, int amount, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += amount;
}

// out = half(act(x)): the rounded tanh / sigmoid of a LoRA intermediate that the reference materialises
// for more than four rows (act_tanh_kernel / act_sigmoid_kernel, cuda/rwkv7_fast_ops_fp16.cu:437-470).
__global__ void act_kernel(const half* __restrict__ x, half* __restrict__ out, long long n, int act) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2half_rn(apply_in_act(__half2float(x[i]), act));
}

__global__ void relu_square_kernel(const half* __restrict__ x, half* __restrict__ out, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float t = fmaxf(__half2float(x[i]), 0.f);
  out[i] = __float2half_rn(t * t);
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

// fp16 = round_to_nearest(float(bf16)): the canonical device value of a checkpoint weight
// (reference: bf16_to_f16_kernel, cuda/rwkv7_v3a_ops.cu:79-88).
__global__ void bf16_to_f16_kernel(const uint16_t* __restrict__ src, half* __restrict__ dst, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2half_rn(bf16_bits_to_float(src[i]));
}

__global__ void transpose_f16_kernel(const half* __restrict__ src, half* __restrict__ dst, int rows, int cols) {
  __shared__ half tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
    const int rr = r0 + dy, cc = c0 + threadIdx.x;
    if (rr < rows && cc < cols) tile[dy][threadIdx.x] = src[static_cast<size_t>(rr) * cols + cc];
  }
  __syncthreads();
  for (int dy = threadIdx.y; dy < 32; dy += blockDim.y) {
    const int cc = c0 + dy, rr = r0 + threadIdx.x;
    if (rr < rows && cc < cols) dst[static_cast<size_t>(cc) * rows + rr] = tile[threadIdx.x][dy];
  }
}

// Embedding table with LN0 folded in, from bf16 or fp16 checkpoint values, statistics in fp32
// (reference: emb_ln0_bf16_to_f16_kernel, cuda/rwkv7_v3a_ops.cu:153-187).
template <bool kBf16>
__global__ void __launch_bounds__(256) emb_ln0_kernel(int C, const uint16_t* __restrict__ emb,
                                                      const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                                                      half* __restrict__ out, float eps) {
  __shared__ float scratch[8];
  auto cvt = [](uint16_t bits) {
    return kBf16 ? bf16_bits_to_float(bits) : __half2float(__ushort_as_half(bits));
  };
  const uint16_t* er = emb + static_cast<size_t>(blockIdx.x) * C;
  float s = 0.f;
  for (int c = threadIdx.x; c < C; c += 256) s += cvt(er[c]);
  const float mean = block_sum<256>(s, scratch) / static_cast<float>(C);
  float sv = 0.f;
  for (int c = threadIdx.x; c < C; c += 256) {
    const float d = cvt(er[c]) - mean;
    sv += d * d;
  }
  const float rstd = rsqrtf(block_sum<256>(sv, scratch) / static_cast<float>(C) + eps);
  half* yr = out + static_cast<size_t>(blockIdx.x) * C;
  for (int c = threadIdx.x; c < C; c += 256) yr[c] = __float2half_rn((cvt(er[c]) - mean) * rstd * cvt(w[c]) + cvt(b[c]));
}

}  // namespace

int row_op(cudaStream_t stream, const RowOpArgs& a) {
  RK_REQUIRE(a.B > 0 && a.T > 0 && a.C > 0 && (a.C & 1) == 0, kShape, "row_op: need B,T > 0 and even C");
  RK_REQUIRE((a.table && a.tokens && a.vocab > 0) || a.x, kBadArg, "row_op: no source");
  RK_REQUIRE(a.n_mix == 0 || a.n_mix == 1 || a.n_mix == 6, kBadArg, "row_op: n_mix must be 0, 1 or 6");
  RK_REQUIRE(a.n_mix == 0 || (a.shift && (a.ln_w || a.identity_norm) && !a.last_only), kBadArg,
             "row_op: token shift needs shift state and LayerNorm weights");
  RK_REQUIRE(!a.ln_w || a.ln_b, kBadArg, "row_op: LayerNorm bias missing");
  RK_REQUIRE(!(a.ln_w && a.identity_norm), kBadArg, "row_op: identity_norm excludes LayerNorm weights");
  RowOpDev p;
  p.B = a.B; p.T = a.T; p.C = a.C; p.vocab = a.vocab; p.n_mix = a.n_mix; p.last_only = a.last_only ? 1 : 0; p.identity = a.identity_norm ? 1 : 0;
  p.eps = a.eps; p.tokens = a.tokens; p.table = a.table; p.x = a.x; p.residual = a.residual; p.residual_f32 = a.residual_f32; p.x_out = a.x_out;
  p.ln_w = a.ln_w; p.ln_b = a.ln_b; p.n_out = a.n_out; p.shift = a.shift; p.bad_token_flag = a.bad_token_flag;
  for (int m = 0; m < 6; ++m) {
    p.mix[m] = a.mix[m];
    p.mix_out[m] = a.mix_out[m];
    RK_REQUIRE(m >= a.n_mix || (a.mix[m] && a.mix_out[m]), kBadArg, "row_op: mix tensor %d missing", m);
  }
  const int rows = a.last_only ? a.B : a.B * a.T;
  if (a.T > 1 && rows > 32 && !a.last_only && a.n_mix > 0 && !a.table && a.C >= 1024 && a.C <= 8192) {
    const int need512 = (a.C / 2 + kChunkThreads - 1) / kChunkThreads;
    const dim3 grid(rows), block(kChunkThreads);
    cudaError_t e;
    if (need512 <= 2) e = launch_pdl(row_op_chunk_kernel<2>, grid, block, 0, stream, p);
    else if (need512 <= 4) e = launch_pdl(row_op_chunk_kernel<4>, grid, block, 0, stream, p);
    else e = launch_pdl(row_op_chunk_kernel<8>, grid, block, 0, stream, p);
    RK_CUDA(e);
    RK_LAUNCH_CHECK("row_op (chunk) launch");
    return kOk;
  }
  const int need = (a.C / 2 + kRowThreads - 1) / kRowThreads;  // pairs per thread
  RK_REQUIRE(need <= 16, kShape, "row_op: C=%d too large (max 8192)", a.C);
  const int kp = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : need <= 8 ? 8 : 16;
  p.n_slices = rows <= 32 ? kp : 1;  // spread few rows over more SMs
  const dim3 grid(p.n_slices, rows), block(kRowThreads);
  cudaError_t e;
  if (rows > 148 && kp == 8) {
    e = launch_pdl(row_op_two_per_sm_kernel<8>, grid, block, 0, stream, p);
    RK_CUDA(e);
    RK_LAUNCH_CHECK("row_op launch");
    return kOk;
  }
  switch (kp) {
    case 1: e = launch_pdl(row_op_kernel<1>, grid, block, 0, stream, p); break;
    case 2: e = launch_pdl(row_op_kernel<2>, grid, block, 0, stream, p); break;
    case 4: e = launch_pdl(row_op_kernel<4>, grid, block, 0, stream, p); break;
    case 8: e = launch_pdl(row_op_kernel<8>, grid, block, 0, stream, p); break;
    default: e = launch_pdl(row_op_kernel<16>, grid, block, 0, stream, p); break;
  }
  RK_CUDA(e);
  RK_LAUNCH_CHECK("row_op launch");
  return kOk;
}

int tmix_kk_a_gate(cudaStream_t stream, int rows, int C, const half* k, const half* k_k, const half* a0,
                   const half* a12, const half* k_a, half* new_k, half* neg_kk, half* kka) {
  RK_REQUIRE(rows > 0 && C > 0 && C % kHead == 0, kShape, "kk_a_gate: C must be a multiple of 64");
  RK_REQUIRE(k && k_k && a0 && a12 && k_a && new_k && neg_kk && kka, kBadArg, "kk_a_gate: null pointer");
  const int H = C / kHead;
  const long long total = static_cast<long long>(rows) * H;
  kk_a_gate_kernel<<<static_cast<unsigned>((total + 3) / 4), 128, 0, stream>>>(H, total, k, k_k, a0, a12, k_a, new_k, neg_kk, kka,
                                                                            nullptr, nullptr, nullptr, nullptr, nullptr);
  RK_LAUNCH_CHECK("kk_a_gate launch");
  return kOk;
}

int tmix_kk_a_vres_gate(cudaStream_t stream, int rows, int C, const half* k, const half* k_k, const half* a0, const half* a12,
                        const half* k_a, half* new_k, half* neg_kk, half* kka, const half* v, const half* v_first,
                        const half* v0, const half* v12, half* v_out) {
  RK_REQUIRE(rows > 0 && C > 0 && C % kHead == 0, kShape, "kk_a_vres_gate: C must be a multiple of 64");
  RK_REQUIRE(k && k_k && a0 && a12 && k_a && new_k && neg_kk && kka && v && v_first && v0 && v12 && v_out, kBadArg,
             "kk_a_vres_gate: null pointer");
  const int H = C / kHead;
  const long long total = static_cast<long long>(rows) * H;
  kk_a_gate_kernel<<<static_cast<unsigned>((total + 3) / 4), 128, 0, stream>>>(H, total, k, k_k, a0, a12, k_a, new_k, neg_kk, kka, v,
                                                                            v_first, v0, v12, v_out);
  RK_LAUNCH_CHECK("kk_a_vres_gate launch");
  return kOk;
}

int tmix_lnx_rkvres_xg(cudaStream_t stream, int rows, int C, const half* y, const half* r, const half* k,
                       const half* v, const half* r_k, const half* w, const half* b, const half* g, half* out) {
  RK_REQUIRE(rows > 0 && C > 0 && C % kHead == 0, kShape, "lnx_rkvres_xg: C must be a multiple of 64");
  RK_REQUIRE(y && r && k && v && r_k && w && b && g && out, kBadArg, "lnx_rkvres_xg: null pointer");
  const int H = C / kHead;
  const long long total = static_cast<long long>(rows) * H;
  lnx_rkvres_xg_kernel<<<static_cast<unsigned>((total + 3) / 4), 128, 0, stream>>>(H, total, y, r, k, v, r_k, w, b, g, out);
  RK_LAUNCH_CHECK("lnx_rkvres_xg launch");
  return kOk;
}

int tmix_vres_gate(cudaStream_t stream, int rows, int C, const half* v, const half* v_first, const half* v0,
                   const half* v12, half* out) {
  RK_REQUIRE(rows > 0 && C > 0, kShape, "vres_gate: empty");
  RK_REQUIRE(v && v_first && v0 && v12 && out, kBadArg, "vres_gate: null pointer");
  const long long total = static_cast<long long>(rows) * C;
  vres_gate_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(C, total, v, v_first, v0, v12, out);
  RK_LAUNCH_CHECK("vres_gate launch");
  return kOk;
}

__global__ void interleave_gathered_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int G, int B, int Vl4) {
  const long long n = static_cast<long long>(G) * B * Vl4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % Vl4);
    const int b = static_cast<int>((i / Vl4) % B);
    const int g = static_cast<int>(i / (static_cast<long long>(Vl4) * B));
    dst[(static_cast<long long>(b) * G + g) * Vl4 + v] = src[i];
  }
}

int interleave_gathered(cudaStream_t stream, const float* src, float* dst, int G, int B, int Vl) {
  RK_REQUIRE(src && dst && G > 0 && B > 0 && Vl > 0 && Vl % 4 == 0, kBadArg, "interleave_gathered: bad argument");
  const long long n = static_cast<long long>(G) * B * (Vl / 4);
  const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 148 * 8));
  interleave_gathered_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst), G, B, Vl / 4);
  RK_LAUNCH_CHECK("interleave_gathered launch");
  return kOk;
}

namespace {
// WKV state between its two precisions (a session paused under one setting of the reference's --wkv32 switch and
// resumed under the other): fp16 -> fp32 is exact, fp32 -> fp16 rounds to nearest even.
__global__ void wkv_state_convert_kernel(long long n8, const void* __restrict__ src, void* __restrict__ dst, int src_is_fp32) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  if (src_is_fp32) {
    const float4 a = reinterpret_cast<const float4*>(src)[2 * i], b = reinterpret_cast<const float4*>(src)[2 * i + 1];
    const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w), h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&h0); o.y = *reinterpret_cast<const uint32_t*>(&h1);
    o.z = *reinterpret_cast<const uint32_t*>(&h2); o.w = *reinterpret_cast<const uint32_t*>(&h3);
    reinterpret_cast<uint4*>(dst)[i] = o;
  } else {
    const uint4 q = reinterpret_cast<const uint4*>(src)[i];
    const float2 f0 = h2f2(q.x), f1 = h2f2(q.y), f2 = h2f2(q.z), f3 = h2f2(q.w);
    reinterpret_cast<float4*>(dst)[2 * i] = make_float4(f0.x, f0.y, f1.x, f1.y);
    reinterpret_cast<float4*>(dst)[2 * i + 1] = make_float4(f2.x, f2.y, f3.x, f3.y);
  }
}
}  // namespace

int wkv_state_convert(cudaStream_t stream, const void* src, void* dst, long long elems, int src_is_fp32) {
  RK_REQUIRE(src && dst && elems > 0 && elems % 8 == 0, kBadArg, "wkv_state_convert: need a positive multiple of 8 elements");
  RK_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0, kBadArg,
             "wkv_state_convert: buffers must be 16-byte aligned");
  const long long n8 = elems / 8;
  wkv_state_convert_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, stream>>>(n8, src, dst, src_is_fp32);
  RK_LAUNCH_CHECK("wkv_state_convert launch");
  return kOk;
}

int advance_i32(cudaStream_t stream, int* x, int amount, int n) {
  RK_REQUIRE(x && n > 0, kBadArg, "advance_i32: bad argument");
  advance_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(x, amount, n);
  RK_LAUNCH_CHECK("advance_i32 launch");
  return kOk;
}

int activate(cudaStream_t stream, const half* x, half* out, long long n, int act) {
  RK_REQUIRE(x && out && n > 0 && (act == kActTanh || act == kActSigmoid), kBadArg, "activate: bad argument");
  act_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(x, out, n, act);
  RK_LAUNCH_CHECK("activate launch");
  return kOk;
}

int relu_square(cudaStream_t stream, const half* x, half* out, long long n) {
  RK_REQUIRE(x && out && n > 0, kBadArg, "relu_square: bad argument");
  relu_square_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(x, out, n);
  RK_LAUNCH_CHECK("relu_square launch");
  return kOk;
}

int bf16_to_f16(cudaStream_t stream, const uint16_t* src, half* dst, long long n) {
  RK_REQUIRE(src && dst && n > 0, kBadArg, "bf16_to_f16: bad argument");
  bf16_to_f16_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(src, dst, n);
  RK_LAUNCH_CHECK("bf16_to_f16 launch");
  return kOk;
}

int transpose_f16(cudaStream_t stream, const half* src, half* dst, int rows, int cols) {
  RK_REQUIRE(src && dst && rows > 0 && cols > 0, kBadArg, "transpose_f16: bad argument");
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  transpose_f16_kernel<<<grid, block, 0, stream>>>(src, dst, rows, cols);
  RK_LAUNCH_CHECK("transpose_f16 launch");
  return kOk;
}

int emb_ln0(cudaStream_t stream, int V, int C, const void* emb, const void* w, const void* b, int src_is_bf16,
            half* out, float eps) {
  RK_REQUIRE(V > 0 && C > 0 && emb && w && b && out, kBadArg, "emb_ln0: bad argument");
  if (src_is_bf16)
    emb_ln0_kernel<true><<<V, 256, 0, stream>>>(C, static_cast<const uint16_t*>(emb), static_cast<const uint16_t*>(w),
                                               static_cast<const uint16_t*>(b), out, eps);
  else
    emb_ln0_kernel<false><<<V, 256, 0, stream>>>(C, static_cast<const uint16_t*>(emb), static_cast<const uint16_t*>(w),
                                                static_cast<const uint16_t*>(b), out, eps);
  RK_LAUNCH_CHECK("emb_ln0 launch");
  return kOk;
}

}  // namespace rk
