// Shared definitions of the weight-streaming GEMV kernels (linear.cu, gemv_tma.cu).
#pragma once

#include "common.cuh"

namespace rk {

constexpr int kMaxSeg = 8;

// One problem y = epi(act(x) W^T) of a batched launch.
struct GemvSeg {
  const half* x;
  const void* w;
  const half* scale;
  const half* zero;
  void* y;
  const half* v;
  const half* v_first;
  const half* v0;
  int ldx, N, K, fmt, in_act, epi;
  int cta_begin, rows_per_cta;  // CTAs [cta_begin, ...) own rows_per_cta consecutive output rows each
  int parts, piece_bytes;       // bulk-copy path: a weight row is fetched as `parts` pieces
  // Optional fused prologue for decode rows (one token per sequence, K == channels): the activations
  // are x' = half(n + (shift - n) * mix) with n = half(LayerNorm(x + res)), computed by every CTA from
  // the residual stream instead of being read from memory.  The first CTA of the problem also stores
  // half(x + res) to x_out and n to n_out (a later kernel moves n_out into the shift state, which all
  // CTAs of this kernel are still reading).
  const half* res;
  const half* ln_w;
  const half* ln_b;
  const half* shift;
  const half* mix;
  half* x_out;
  half* n_out;
  float eps;
  // Optional small copy done by the first CTA after the dependency wait (moves a previous kernel's
  // n_out into the shift state).
  const half* copy_src;
  half* copy_dst;
  int copy_n;
};

bool gemv_tma_fits(int M, int K);  // gemv_tma.cu

struct GemvBatch {
  int n_seg;
  GemvSeg seg[kMaxSeg];
  int* timeout;  // the device's failure word (kernels.h): a bounded wait that runs out ORs kTimeoutGemv into it
};

#ifdef __CUDACC__
// Rounds and stores one fp32 accumulator: the single rounding point of a linear layer.
__device__ __forceinline__ void store_result(const GemvSeg& sg, int m, int n, float a) {
  const size_t o = static_cast<size_t>(m) * sg.N + n;
  if (sg.epi == kEpiRawF32) {
    static_cast<float*>(sg.y)[o] = a;
  } else if (sg.epi == kEpiF32) {
    static_cast<float*>(sg.y)[o] = __half2float(__float2half_rn(a));
  } else if (sg.epi == kEpiRelu2) {
    const float t = fmaxf(__half2float(__float2half_rn(a)), 0.f);
    static_cast<half*>(sg.y)[o] = __float2half_rn(t * t);
  } else if (sg.epi == kEpiVres) {
    const float vv = __half2float(sg.v[o]);
    const float gate = 1.0f / (1.0f + expf(-(__half2float(sg.v0[n]) + a)));
    static_cast<half*>(sg.y)[o] = __float2half_rn(vv + (__half2float(sg.v_first[o]) - vv) * gate);
  } else {
    static_cast<half*>(sg.y)[o] = __float2half_rn(a);
  }
}

// Expands one 16-byte weight chunk to fp32.
template <int kFmt>
__device__ __forceinline__ void dequant_chunk(const uint4& q, float* out, float s, float z);

template <>
__device__ __forceinline__ void dequant_chunk<0>(const uint4& q, float* out, float, float) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = h2f2(u[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// int8 -> exact integer-valued float via the fp16 "1024 + n" encoding.
template <>
__device__ __forceinline__ void dequant_chunk<1>(const uint4& q, float* out, float, float) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t t = u[i] ^ 0x80808080u;
    uint32_t h01 = __byte_perm(t, 0x64646464u, 0x4140);
    uint32_t h23 = __byte_perm(t, 0x64646464u, 0x4342);
    const float2 a = __half22float2(__hsub2(*reinterpret_cast<__half2*>(&h01), bias));
    const float2 b = __half22float2(__hsub2(*reinterpret_cast<__half2*>(&h23), bias));
    out[4 * i] = a.x;
    out[4 * i + 1] = a.y;
    out[4 * i + 2] = b.x;
    out[4 * i + 3] = b.y;
  }
}

// int4 -> half((q - zero) * scale), the written definition of the W4A16 weight value.
template <>
__device__ __forceinline__ void dequant_chunk<2>(const uint4& q, float* out, float s, float z) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
  const __half2 zb = __float2half2_rn(1024.f + z);
  const __half2 s2 = __float2half2_rn(s);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // byte j of the word holds elements 2j (low nibble) and 2j+1 (high nibble)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = (u[i] >> (8 * j)) & 0xffu;
      uint32_t pair = (byte & 0xfu) | ((byte >> 4) << 16) | 0x64006400u;
      const __half2 w2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&pair), zb), s2);
      const float2 f = __half22float2(w2);
      out[8 * i + 2 * j] = f.x;
      out[8 * i + 2 * j + 1] = f.y;
    }
  }
}

// Stages the activations of a segment in shared memory: half as they are, or fp32 with the input
// activation applied once when there is one.
template <int kM, int kThreads>
__device__ __forceinline__ void stage_activations(const GemvSeg& sg, half* xs16, float* xs32) {
  const int n_vec = sg.K >> 3;
  for (int i = threadIdx.x; i < kM * n_vec; i += kThreads) {
    const int m = i / n_vec, kv = i - m * n_vec;
    const uint4 q = *reinterpret_cast<const uint4*>(sg.x + static_cast<size_t>(m) * sg.ldx + kv * 8);
    if (xs32) {
      const uint32_t u[4] = {q.x, q.y, q.z, q.w};
      float* dst = xs32 + static_cast<size_t>(m) * sg.K + kv * 8;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = h2f2(u[e]);
        dst[2 * e] = apply_in_act(f.x, sg.in_act);
        dst[2 * e + 1] = apply_in_act(f.y, sg.in_act);
      }
    } else {
      *reinterpret_cast<uint4*>(xs16 + static_cast<size_t>(m) * sg.K + kv * 8) = q;
    }
  }
}
// Fused prologue (see GemvSeg): residual add + LayerNorm + token shift for kM decode rows, result as
// fp32 in xs [kM, K].  Rounding points as in the separate row kernel: half(x + res), half(LN), half(mix).
// A thread owns the channel pairs q = tid + kThreads*i, i < kLnPairs (K <= 2*kThreads*kLnPairs); the
// LayerNorm weights, the mix coefficients and the first row's shift values are requested before the
// dependency wait (LnPrefetch), the row itself stays in registers between the passes.
constexpr int kLnPairs = 8;

struct LnPrefetch {
  __half2 w[kLnPairs], b[kLnPairs], mix[kLnPairs], shift0[kLnPairs];
};

template <int kThreads>
__device__ __forceinline__ void ln_prefetch(const GemvSeg& sg, LnPrefetch& pf) {
  const int pairs = sg.K >> 1;
#pragma unroll
  for (int i = 0; i < kLnPairs; ++i) {
    const int q = threadIdx.x + kThreads * i;
    if (q < pairs) {
      pf.w[i] = reinterpret_cast<const __half2*>(sg.ln_w)[q];
      pf.b[i] = reinterpret_cast<const __half2*>(sg.ln_b)[q];
      if (sg.mix) {
        pf.mix[i] = reinterpret_cast<const __half2*>(sg.mix)[q];
        pf.shift0[i] = reinterpret_cast<const __half2*>(sg.shift)[q];  // written one step ago
      }
    }
  }
}

// `put(m, k, v)` receives the two activations (k, k + 1) of row m; both are exact halves.
template <int kM, int kThreads, class Put>
__device__ __forceinline__ void stage_ln_mix(const GemvSeg& sg, Put put, float* scratch, bool writer, const LnPrefetch& pf) {
  const int K = sg.K, pairs = K >> 1;
#pragma unroll
  for (int m = 0; m < kM; ++m) {
    const __half2* xg = reinterpret_cast<const __half2*>(sg.x + static_cast<size_t>(m) * sg.ldx);
    const __half2* rg = sg.res ? reinterpret_cast<const __half2*>(sg.res + static_cast<size_t>(m) * K) : nullptr;
    __half2 xv[kLnPairs], rv[kLnPairs], sh[kLnPairs];
#pragma unroll
    for (int i = 0; i < kLnPairs; ++i) {
      const int q = threadIdx.x + kThreads * i;
      const bool ok = q < pairs;
      xv[i] = ok ? xg[q] : __floats2half2_rn(0.f, 0.f);
      rv[i] = (ok && rg) ? rg[q] : __floats2half2_rn(0.f, 0.f);
      if (sg.mix) sh[i] = (m == 0) ? pf.shift0[i] : (ok ? reinterpret_cast<const __half2*>(sg.shift + static_cast<size_t>(m) * K)[q] : pf.shift0[i]);
    }
    float2 v[kLnPairs];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kLnPairs; ++i) {
      const float2 a = __half22float2(xv[i]), r = __half22float2(rv[i]);
      v[i] = make_float2(a.x + r.x, a.y + r.y);
      s += v[i].x + v[i].y;
    }
    const float inv_k = 1.0f / static_cast<float>(K);
    const float mean = block_sum<kThreads>(s, scratch) * inv_k;
    float sv = 0.f;
#pragma unroll
    for (int i = 0; i < kLnPairs; ++i) {
      if (threadIdx.x + kThreads * i < pairs) {
        const float d0 = v[i].x - mean, d1 = v[i].y - mean;
        sv += d0 * d0 + d1 * d1;
      }
    }
    const float rstd = rsqrtf(block_sum<kThreads>(sv, scratch) * inv_k + sg.eps);
#pragma unroll
    for (int i = 0; i < kLnPairs; ++i) {
      const int q = threadIdx.x + kThreads * i;
      if (q >= pairs) continue;
      const float2 w = __half22float2(pf.w[i]), b = __half22float2(pf.b[i]);
      const __half2 nh = __floats2half2_rn((v[i].x - mean) * rstd * w.x + b.x, (v[i].y - mean) * rstd * w.y + b.y);
      if (writer) {
        if (sg.x_out) reinterpret_cast<__half2*>(sg.x_out + static_cast<size_t>(m) * K)[q] = __floats2half2_rn(v[i].x, v[i].y);
        if (sg.n_out) reinterpret_cast<__half2*>(sg.n_out + static_cast<size_t>(m) * K)[q] = nh;
      }
      float2 n = __half22float2(nh);
      if (sg.mix) {
        const float2 p = __half22float2(sh[i]), c = __half22float2(pf.mix[i]);
        n = __half22float2(__floats2half2_rn(n.x + (p.x - n.x) * c.x, n.y + (p.y - n.y) * c.y));
      }
      put(m, 2 * q, n);
    }
  }
}
#endif

// gemv_mma.cu: 2..4 rows of any format and one row of quantised weights: 16-row weight tiles (2-D TMA, 128-byte
// swizzle) against the activations on mma.sync, so that the weights are dequantised in half2 arithmetic once per
// tile instead of once per row of activations.  plan() returns false for shapes it does not take.
struct GemvMmaPlan {
  size_t smem_bytes;
  int grid, n_slots, x_pitch;  // x_pitch: bytes between rows of activations in shared memory
  int blocks;                  // 16-channel blocks per tile (1, or 2 for quantised weights where shared memory allows)
};
bool gemv_mma_plan(GemvBatch& b, int M, GemvMmaPlan* plan);
int gemv_mma_launch(cudaStream_t stream, const GemvBatch& b, int M, const GemvMmaPlan& plan);

// gemv_tma.cu: fp16 weights fetched with per-warp rings of bulk copies (cp.async.bulk + mbarrier).
bool gemv_tma_plan(GemvBatch& b, int M, size_t* smem_bytes, int* grid, int* n_slots, int* slot_stride, int* n_warps);
int gemv_tma_launch(cudaStream_t stream, const GemvBatch& b, int M, size_t smem_bytes, int grid, int n_slots, int slot_stride,
                    int n_warps);

}  // namespace rk
