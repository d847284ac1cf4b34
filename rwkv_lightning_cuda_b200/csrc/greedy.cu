// Greedy token choice on the device, the step that follows the lm-head in a decode loop.
//
// The reference widens the logits to fp32, runs its 1024-thread multi-pass sampler
// (batch_sampling_repetition_temperature_topk_topp_kernel, src/utils/sampling.cu:205-471), copies the token
// to the host and starts the next forward from there.  With top_p == 0 the sampler is greedy (top_k = 1,
// src/utils/sampling.cu:507-512): the token with the largest penalised logit wins, and the temperature, a
// positive factor, cannot change the winner.  This kernel keeps exactly that case: per sequence
//   value[i]  = finite(logit[i]) - penalty[i]          (:253; NaN counts as 0, +-inf as +-FLT_MAX, :139-142)
//   token     = argmax_i value[i]                      (lowest index among equal values; the reference draws among
//                                                       them at random, :388-458)
//   penalty[i] = penalty[i] * decay + (i == token ? (penalty[i] == 0 ? presence : repetition) : 0)     (:460-469)
// and writes the token where the next decode step's embedding gather reads it, so that a run of decode steps needs
// no host round trip.
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

constexpr int kPickThreads = 1024;

__device__ __forceinline__ float finite_or_clamped(float x) {
  const uint32_t u = __float_as_uint(x) & 0x7fffffffu;
  if (u > 0x7f800000u) return 0.f;                          // NaN
  if (u == 0x7f800000u) return copysignf(FLT_MAX, x);       // +-inf
  return x;
}

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__global__ void __launch_bounds__(kPickThreads) greedy_pick_kernel(int V, const float* __restrict__ logits, float* penalties,
                                                                   float presence, float repetition, float decay,
                                                                   int* __restrict__ out, int64_t* __restrict__ next_tokens) {
  __shared__ Best red[kPickThreads / 32];
  __shared__ int chosen;
  const int b = blockIdx.x, t = threadIdx.x;
  const float* lg = logits + static_cast<size_t>(b) * V;
  float* pen = penalties ? penalties + static_cast<size_t>(b) * V : nullptr;
  const int V4 = (V % 4 == 0) ? V / 4 : 0;  // rows of a vocabulary that is no multiple of four are not 16-byte aligned

  Best best{-INFINITY, 0x7fffffff};
  for (int i = t; i < V4; i += kPickThreads) {
    const float4 l4 = reinterpret_cast<const float4*>(lg)[i];
    float4 p4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pen) p4 = reinterpret_cast<const float4*>(pen)[i];
    const float l[4] = {l4.x, l4.y, l4.z, l4.w}, p[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) best = better(best, Best{finite_or_clamped(l[j]) - p[j], 4 * i + j});
  }
  for (int i = 4 * V4 + t; i < V; i += kPickThreads)
    best = better(best, Best{finite_or_clamped(lg[i]) - (pen ? pen[i] : 0.f), i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if ((t & 31) == 0) red[t >> 5] = best;
  __syncthreads();
  if (t < 32) {
    best = red[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (t == 0) {
      const int token = best.i < V ? best.i : 0;  // every value NaN (a NaN penalty): token 0, as the reference's out-of-range guard
      chosen = token;
      out[b] = token;
      if (next_tokens) next_tokens[b] = token;
    }
  }
  if (!pen) return;
  __syncthreads();
  const int token = chosen;
  for (int i = t; i < V4; i += kPickThreads) {
    float4 p4 = reinterpret_cast<float4*>(pen)[i];
    float* p = reinterpret_cast<float*>(&p4);
#pragma unroll
    for (int j = 0; j < 4; ++j) p[j] = __fmaf_rn(p[j], decay, (4 * i + j != token) ? 0.f : (p[j] == 0.f ? presence : repetition));
    reinterpret_cast<float4*>(pen)[i] = p4;
  }
  for (int i = 4 * V4 + t; i < V; i += kPickThreads) {
    const float p = pen[i];
    pen[i] = __fmaf_rn(p, decay, (i != token) ? 0.f : (p == 0.f ? presence : repetition));
  }
}

}  // namespace

int greedy_pick(cudaStream_t stream, int B, int V, const float* logits, float* penalties, float presence, float repetition,
                float decay, int* out, int64_t* next_tokens) {
  RK_REQUIRE(B > 0 && V > 0 && logits && out, kBadArg, "greedy_pick: bad argument");
  greedy_pick_kernel<<<B, kPickThreads, 0, stream>>>(V, logits, penalties, presence, repetition, decay, out, next_tokens);
  RK_LAUNCH_CHECK("greedy_pick launch");
  return kOk;
}

}  // namespace rk
