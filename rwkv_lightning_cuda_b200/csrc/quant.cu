// W8A16 / W4A16 weight formats: pack (quantise) and unpack (dequantise) on the device.
// The reference has no quantised path; the formats are defined here and restated by the
// CPU oracle, and the two must agree bit for bit.
//   W8A16: per output channel, symmetric.  scale[n] = half(max_k |W[n,k]| / 127),
//          q = clamp(rint(W / float(scale)), -127, 127), int8 row-major [N,K].
//   W4A16: groups of 128 along K, asymmetric, range widened to contain 0.
//          scale = half((max - min) / 15), zero = clamp(rint(-min / float(scale)), 0, 15) stored as
//          an integer-valued half, q = clamp(rint(W / float(scale)) + zero, 0, 15); byte j of a row
//          holds q[2j] (low nibble) and q[2j+1] (high nibble).
//          Dequantised weight = half((q - zero) * float(scale)).
// Divisions and roundings use the IEEE intrinsics so that fast-math compilation cannot change
// a quantised value.
#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

__global__ void __launch_bounds__(256) pack_w8_kernel(int K, const half* __restrict__ W, int8_t* __restrict__ q,
                                                      half* __restrict__ scale) {
  __shared__ float red[8];
  const half* wr = W + static_cast<size_t>(blockIdx.x) * K;
  float amax = 0.f;
  for (int k = threadIdx.x; k < K; k += 256) amax = fmaxf(amax, fabsf(__half2float(wr[k])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const half s = __float2half_rn(__fdiv_rn(amax, 127.0f));
  if (threadIdx.x == 0) scale[blockIdx.x] = s;
  const float sf = __half2float(s);
  for (int k = threadIdx.x; k < K; k += 256) {
    float v = sf > 0.f ? rintf(__fdiv_rn(__half2float(wr[k]), sf)) : 0.f;
    v = fminf(fmaxf(v, -127.f), 127.f);
    q[static_cast<size_t>(blockIdx.x) * K + k] = static_cast<int8_t>(v);
  }
}

__global__ void unpack_w8_kernel(int K, long long total, const int8_t* __restrict__ q, const half* __restrict__ scale,
                                 half* __restrict__ W) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  W[i] = __float2half_rn(__fmul_rn(static_cast<float>(q[i]), __half2float(scale[i / K])));
}

// One warp per (row, group of 128): lane handles 4 consecutive weights = 2 packed bytes.
__global__ void __launch_bounds__(128) pack_w4_kernel(int K, long long n_groups, const half* __restrict__ W,
                                                      uint8_t* __restrict__ q, half* __restrict__ scale,
                                                      half* __restrict__ zero) {
  const long long g = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (g >= n_groups) return;
  const int lane = threadIdx.x & 31;
  const half* w = W + g * 128 + lane * 4;
  float v[4];
  float mn = 0.f, mx = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = __half2float(w[i]);
    mn = fminf(mn, v[i]);
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  const half s = __float2half_rn(__fdiv_rn(__fsub_rn(mx, mn), 15.0f));
  const float sf = __half2float(s);
  float z = sf > 0.f ? rintf(__fdiv_rn(-mn, sf)) : 0.f;
  z = fminf(fmaxf(z, 0.f), 15.f);
  if (lane == 0) {
    scale[g] = s;
    zero[g] = __float2half_rn(z);
  }
  uint8_t nib[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float t = sf > 0.f ? __fadd_rn(rintf(__fdiv_rn(v[i], sf)), z) : 0.f;
    t = fminf(fmaxf(t, 0.f), 15.f);
    nib[i] = static_cast<uint8_t>(t);
  }
  uint8_t* qb = q + g * 64 + lane * 2;
  qb[0] = static_cast<uint8_t>(nib[0] | (nib[1] << 4));
  qb[1] = static_cast<uint8_t>(nib[2] | (nib[3] << 4));
}

__global__ void unpack_w4_kernel(long long total, const uint8_t* __restrict__ q, const half* __restrict__ scale,
                                 const half* __restrict__ zero, half* __restrict__ W) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const uint8_t byte = q[i >> 1];
  const int qq = (i & 1) ? (byte >> 4) : (byte & 15);
  const long long g = i >> 7;
  W[i] = __float2half_rn(__fmul_rn(__fsub_rn(static_cast<float>(qq), __half2float(zero[g])), __half2float(scale[g])));
}

}  // namespace

int quant_pack_w8(cudaStream_t stream, int N, int K, const half* W, int8_t* q, half* scale) {
  RK_REQUIRE(N > 0 && K > 0 && W && q && scale, kBadArg, "quant_pack_w8: bad argument");
  pack_w8_kernel<<<N, 256, 0, stream>>>(K, W, q, scale);
  RK_LAUNCH_CHECK("quant_pack_w8 launch");
  return kOk;
}

int quant_unpack_w8(cudaStream_t stream, int N, int K, const int8_t* q, const half* scale, half* W) {
  RK_REQUIRE(N > 0 && K > 0 && W && q && scale, kBadArg, "quant_unpack_w8: bad argument");
  const long long total = static_cast<long long>(N) * K;
  unpack_w8_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(K, total, q, scale, W);
  RK_LAUNCH_CHECK("quant_unpack_w8 launch");
  return kOk;
}

int quant_pack_w4(cudaStream_t stream, int N, int K, const half* W, uint8_t* q, half* scale, half* zero) {
  RK_REQUIRE(N > 0 && K > 0 && K % 128 == 0 && W && q && scale && zero, kBadArg, "quant_pack_w4: K must be a multiple of 128");
  const long long groups = static_cast<long long>(N) * (K / 128);
  pack_w4_kernel<<<static_cast<unsigned>((groups + 3) / 4), 128, 0, stream>>>(K, groups, W, q, scale, zero);
  RK_LAUNCH_CHECK("quant_pack_w4 launch");
  return kOk;
}

int quant_unpack_w4(cudaStream_t stream, int N, int K, const uint8_t* q, const half* scale, const half* zero, half* W) {
  RK_REQUIRE(N > 0 && K > 0 && K % 128 == 0 && W && q && scale && zero, kBadArg, "quant_unpack_w4: K must be a multiple of 128");
  const long long total = static_cast<long long>(N) * K;
  unpack_w4_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(total, q, scale, zero, W);
  RK_LAUNCH_CHECK("quant_unpack_w4 launch");
  return kOk;
}

}  // namespace rk
