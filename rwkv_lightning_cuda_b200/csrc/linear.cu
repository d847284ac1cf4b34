// Weight-streaming linear layers for decode-sized row counts: y = act(x) W^T, W [N,K] row-major
// in fp16, int8 (W8A16) or packed int4 (W4A16, group 128).  The weights are read exactly once
// with 128-bit non-allocating loads, dequantised in registers, accumulated in fp32 and reduced
// with warp shuffles; the result is rounded to half once (the reference's rounding point,
// cuda/rwkv7_v3a_ops.cu:464-509).  Replaces linear_orig_row{1,2}_exact*_f16_kernel and the
// linear_t*/LoRA kernels of cuda/rwkv7_v3a_ops.cu for rows <= 4; larger row counts go to the
// tensor-core GEMM.
#include "common.cuh"
#include "kernels.h"

namespace rk {

int gemm_tc(cudaStream_t stream, const LinearArgs& a);  // gemm_tcgen05.cu
bool gemm_tc_supported(const LinearArgs& a);

namespace {

struct LinearDev {
  int M, K, N, ldx, in_act, epi;
  const half* x;
  const void* w;
  const half* scale;
  const half* zero;
  const half* v;
  const half* v_first;
  const half* v0;
  void* y;
};

constexpr int kWarpsPerCta = 8;
constexpr int kOutPerWarp = 2;
constexpr int kUnroll = 4;

template <int kFmt>
struct Fmt;
template <>
struct Fmt<0> { static constexpr int kElems = 8; };   // 8 halves per 16-byte load
template <>
struct Fmt<1> { static constexpr int kElems = 16; };  // 16 int8
template <>
struct Fmt<2> { static constexpr int kElems = 32; };  // 32 int4

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

template <int kM, int kFmt>
__global__ void __launch_bounds__(kWarpsPerCta * 32) gemv_kernel(const LinearDev p) {
  constexpr int E = Fmt<kFmt>::kElems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * kWarpsPerCta + warp) * kOutPerWarp;
  if (n0 >= p.N) return;
  const int n_valid = min(kOutPerWarp, p.N - n0);
  const size_t row_bytes = static_cast<size_t>(p.K) * 16 / E;  // bytes per weight row
  const char* wbase = static_cast<const char*>(p.w) + static_cast<size_t>(n0) * row_bytes;
  const int groups = p.K >> 7;

  float acc[kM][kOutPerWarp];
#pragma unroll
  for (int m = 0; m < kM; ++m)
#pragma unroll
    for (int j = 0; j < kOutPerWarp; ++j) acc[m][j] = 0.f;

  const int step = 32 * E;
  for (int k0 = lane * E; k0 < p.K; k0 += step * kUnroll) {
    uint4 wq[kUnroll][kOutPerWarp];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = k0 + u * step;
#pragma unroll
      for (int j = 0; j < kOutPerWarp; ++j) {
        if (k < p.K && j < n_valid) wq[u][j] = ldg_stream(wbase + j * row_bytes + static_cast<size_t>(k) * 16 / E);
        else wq[u][j] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = k0 + u * step;
      if (k >= p.K) break;
      float wf[kOutPerWarp][E];
#pragma unroll
      for (int j = 0; j < kOutPerWarp; ++j) {
        float s = 0.f, z = 0.f;
        if (kFmt == 2) {
          const int nn = min(n0 + j, p.N - 1);
          s = __half2float(p.scale[static_cast<size_t>(nn) * groups + (k >> 7)]);
          z = __half2float(p.zero[static_cast<size_t>(nn) * groups + (k >> 7)]);
        }
        dequant_chunk<kFmt>(wq[u][j], wf[j], s, z);
      }
#pragma unroll
      for (int m = 0; m < kM; ++m) {
        const half* xr = p.x + static_cast<size_t>(m) * p.ldx + k;
#pragma unroll
        for (int c = 0; c < E / 8; ++c) {
          const uint4 xq = *reinterpret_cast<const uint4*>(xr + c * 8);
          const uint32_t xu[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 xf = h2f2(xu[i]);
            if (p.in_act != kActNone) {
              xf.x = apply_in_act(xf.x, p.in_act);
              xf.y = apply_in_act(xf.y, p.in_act);
            }
#pragma unroll
            for (int j = 0; j < kOutPerWarp; ++j) {
              acc[m][j] = fmaf(xf.x, wf[j][c * 8 + 2 * i], acc[m][j]);
              acc[m][j] = fmaf(xf.y, wf[j][c * 8 + 2 * i + 1], acc[m][j]);
            }
          }
        }
      }
    }
  }

#pragma unroll
  for (int m = 0; m < kM; ++m)
#pragma unroll
    for (int j = 0; j < kOutPerWarp; ++j) acc[m][j] = warp_sum(acc[m][j]);

  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < kOutPerWarp; ++j) {
      if (j >= n_valid) break;
      const int n = n0 + j;
      const float sc = (kFmt == 1) ? __half2float(p.scale[n]) : 1.0f;
#pragma unroll
      for (int m = 0; m < kM; ++m) {
        const float a = acc[m][j] * sc;
        const size_t o = static_cast<size_t>(m) * p.N + n;
        if (p.epi == kEpiF32) {
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
    }
  }
}

template <int kFmt>
int launch_gemv(cudaStream_t stream, const LinearDev& p) {
  const int warps = (p.N + kOutPerWarp - 1) / kOutPerWarp;
  const int grid = (warps + kWarpsPerCta - 1) / kWarpsPerCta;
  const int block = kWarpsPerCta * 32;
  switch (p.M) {
    case 1: gemv_kernel<1, kFmt><<<grid, block, 0, stream>>>(p); break;
    case 2: gemv_kernel<2, kFmt><<<grid, block, 0, stream>>>(p); break;
    case 3: gemv_kernel<3, kFmt><<<grid, block, 0, stream>>>(p); break;
    default: gemv_kernel<4, kFmt><<<grid, block, 0, stream>>>(p); break;
  }
  RK_LAUNCH_CHECK("gemv launch");
  return kOk;
}

}  // namespace

int linear(cudaStream_t stream, const LinearArgs& a) {
  RK_REQUIRE(a.M > 0 && a.K > 0 && a.N > 0, kShape, "linear: M, K, N must be positive");
  RK_REQUIRE(a.x && a.w && a.y, kBadArg, "linear: null pointer");
  RK_REQUIRE(a.fmt >= 0 && a.fmt <= 2, kBadArg, "linear: unknown weight format %d", a.fmt);
  const int elems = a.fmt == 0 ? 8 : (a.fmt == 1 ? 16 : 32);
  RK_REQUIRE(a.K % elems == 0, kShape, "linear: K=%d must be a multiple of %d for this weight format", a.K, elems);
  RK_REQUIRE(a.fmt != 1 || a.scale, kBadArg, "linear: W8A16 needs scales");
  RK_REQUIRE(a.fmt != 2 || (a.scale && a.zero && a.K % 128 == 0), kBadArg, "linear: W4A16 needs scales, zeros and K %% 128 == 0");
  RK_REQUIRE(a.epi != kEpiVres || (a.ea.v && a.ea.v_first && a.ea.v0), kBadArg, "linear: v-residual epilogue needs v, v_first, v0");
  const int ldx = a.ldx ? a.ldx : a.K;
  RK_REQUIRE(ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0,
             kBadArg, "linear: x and w must be 16-byte aligned");

  if (a.M > 4 && gemm_tc_supported(a)) return gemm_tc(stream, a);

  LinearDev p;
  p.K = a.K; p.N = a.N; p.ldx = ldx; p.in_act = a.in_act; p.epi = a.epi;
  p.w = a.w; p.scale = a.scale; p.zero = a.zero; p.v0 = a.ea.v0;
  const size_t out_elem = a.epi == kEpiF32 ? sizeof(float) : sizeof(half);
  for (int m0 = 0; m0 < a.M; m0 += 4) {
    p.M = a.M - m0 < 4 ? a.M - m0 : 4;
    p.x = a.x + static_cast<size_t>(m0) * ldx;
    p.y = static_cast<char*>(a.y) + static_cast<size_t>(m0) * a.N * out_elem;
    p.v = a.ea.v ? a.ea.v + static_cast<size_t>(m0) * a.N : nullptr;
    p.v_first = a.ea.v_first ? a.ea.v_first + static_cast<size_t>(m0) * a.N : nullptr;
    int s;
    if (a.fmt == 0) s = launch_gemv<0>(stream, p);
    else if (a.fmt == 1) s = launch_gemv<1>(stream, p);
    else s = launch_gemv<2>(stream, p);
    if (s != kOk) return s;
  }
  return kOk;
}

}  // namespace rk
