// Temperature / top-k / top-p sampling with repetition penalties on the device: the general case of the step that
// follows the lm-head (greedy.cu keeps the top_p == 0 case).
//
// Same rule as the reference's sampler (batch_sampling_repetition_temperature_topk_topp_kernel,
// src/utils/sampling.cu:205-471; argument normalisation :492-512), restated:
//   z[i] = clamp_finite((clamp_finite(logit[i]) - penalty[i]) * log2(e) / temperature)            (:253)
//   p[i] = 2^(z[i] - max z) / sum                                                                  (:262-291)
//   threshold = the smallest probability value t such that the tokens with p > t hold fewer than top_k tokens AND
//               less than top_p of the mass, i.e. the value at which a budget is reached going down the sorted
//               probabilities (found by bisection on the float bit pattern, :300-362)
//   tokens with p > t keep their probability; the n tokens with p == t share what is left of both budgets:
//               each keeps p * comp, comp = clamp(min((top_p - mass_above) / (t n), (top_k - count_above) / n), 0, 1)
//                                                                                                  (:364-399)
//   the token is drawn in proportion to what is kept                                               (:401-458)
//   penalty[i] = penalty[i] * decay + (i == token ? (penalty[i] == 0 ? presence : repetition) : 0) (:460-469)
// What differs, on purpose: the random numbers come from a counter-based generator (Philox-4x32-10 keyed by the
// caller's seed, counter = (offset, row)), so a draw is a pure function of (seed, offset, row, inputs) -- the reference
// keeps a cuRAND state per row seeded from the clock, so its draws cannot be reproduced; and the token is found with one
// uniform number and one ordered pass over the vocabulary instead of two numbers and a two-level search.
// One CTA of 1024 threads per row; `probs` is caller-provided scratch, fp32 [B, V] (it stays in L2 between the passes).
#include <cfloat>

#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ float clamp_finite(float x) {
  const uint32_t u = __float_as_uint(x) & 0x7fffffffu;
  if (u > 0x7f800000u) return 0.f;
  if (u == 0x7f800000u) return copysignf(FLT_MAX, x);
  return x;
}

// Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"); first output word.
__device__ __forceinline__ uint32_t philox_first(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0; c1 = lo1; c2 = hi0 ^ c3 ^ k1; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return c0;
}

template <typename T, typename Op>
__device__ __forceinline__ T block_all(T v, Op op, T* scratch /* 32 */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  T r = scratch[threadIdx.x & 31];  // kSampleThreads / 32 == 32 partial results
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = op(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(int V, const float* __restrict__ logits, float* penalties,
                                                                float* __restrict__ probs, float presence, float repetition,
                                                                float decay, float log2_inv_temp, int top_k, float top_p,
                                                                uint32_t seed_lo, uint32_t seed_hi, uint32_t off_lo, uint32_t off_hi,
                                                                int* __restrict__ out, int64_t* __restrict__ next_tokens) {
  __shared__ float fs[32];
  __shared__ unsigned us[32];
  __shared__ float scan[kSampleThreads / 32];
  __shared__ int chosen;
  const int b = blockIdx.x, t = threadIdx.x;
  const float* lg = logits + static_cast<size_t>(b) * V;
  float* pen = penalties ? penalties + static_cast<size_t>(b) * V : nullptr;
  float* pr = probs + static_cast<size_t>(b) * V;
  auto fmax_op = [](float a, float c) { return fmaxf(a, c); };
  auto fmin_op = [](float a, float c) { return fminf(a, c); };
  auto fadd_op = [](float a, float c) { return a + c; };
  auto uadd_op = [](unsigned a, unsigned c) { return a + c; };

  // 1-3: scaled logits, softmax in base 2
  float zmax = -INFINITY;
  for (int i = t; i < V; i += kSampleThreads) {
    const float z = clamp_finite((clamp_finite(lg[i]) - (pen ? pen[i] : 0.f)) * log2_inv_temp);
    pr[i] = z;
    zmax = fmaxf(zmax, z);
  }
  zmax = block_all(zmax, fmax_op, fs);
  float denom = 0.f;
  for (int i = t; i < V; i += kSampleThreads) denom += exp2f(pr[i] - zmax);
  denom = block_all(denom, fadd_op, fs);
  float pmax = 0.f, pmin = INFINITY;
  for (int i = t; i < V; i += kSampleThreads) {
    const float p = exp2f(pr[i] - zmax) / denom;
    pr[i] = p;
    pmax = fmaxf(pmax, p);
    pmin = fminf(pmin, p);
  }
  pmax = block_all(pmax, fmax_op, fs);
  pmin = block_all(pmin, fmin_op, fs);

  // 4: bisection on the bit pattern: at `left` a budget is still exceeded, at `right` both hold strictly
  unsigned left = __float_as_uint(pmin), right = __float_as_uint(pmax) + 1;
  unsigned cnt_left = static_cast<unsigned>(V);
  float mass_left = 1.f;
  while ((cnt_left > static_cast<unsigned>(top_k) || mass_left > top_p) && left + 1 < right) {
    const unsigned mid = left + (right - left) / 2;
    const float pivot = __uint_as_float(mid);
    unsigned c = 0;
    float m = 0.f;
    for (int i = t; i < V; i += kSampleThreads) {
      const float p = pr[i];
      if (p >= pivot) { ++c; m += p; }
    }
    c = block_all(c, uadd_op, us);
    m = block_all(m, fadd_op, fs);
    if (c < static_cast<unsigned>(top_k) && m < top_p) {
      right = mid;
    } else {
      left = mid;
      cnt_left = c;
      mass_left = m;
    }
  }
  const float thr = __uint_as_float(left);

  // 5: what lies strictly above the threshold, how many tokens sit on it, and their share
  unsigned gt_c = 0, eq_c = 0;
  float gt_m = 0.f;
  for (int i = t; i < V; i += kSampleThreads) {
    const float p = pr[i];
    if (p > thr) { ++gt_c; gt_m += p; }
    else if (p == thr) ++eq_c;
  }
  gt_c = block_all(gt_c, uadd_op, us);
  eq_c = block_all(eq_c, uadd_op, us);
  gt_m = block_all(gt_m, fadd_op, fs);
  float comp = 1.f;
  if (eq_c > 0) {
    comp = fminf(clamp_finite((top_p - gt_m) / (thr * static_cast<float>(eq_c))), comp);
    comp = fminf(clamp_finite(static_cast<float>(top_k - static_cast<int>(gt_c)) / static_cast<float>(eq_c)), comp);
    comp = fmaxf(comp, 0.f);
  }

  // 6: the draw.  Thread t owns the tokens [t * seg, (t + 1) * seg) in order; an inclusive scan over the threads' sums
  // finds the thread whose range holds the target, which then walks its range.
  const int seg = (V + kSampleThreads - 1) / kSampleThreads;
  const int i_begin = min(t * seg, V), i_end = min(i_begin + seg, V);
  float mine = 0.f;
  for (int i = i_begin; i < i_end; ++i) {
    const float p = pr[i];
    mine += p > thr ? p : (p == thr ? p * comp : 0.f);
  }
  // inclusive scan over 1024 partial sums: within warps by shuffles, across warps through shared memory
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if ((t & 31) >= o) incl += up;
  }
  __syncthreads();
  if ((t & 31) == 31) scan[t >> 5] = incl;
  __syncthreads();
  if (t < 32) {
    float w = scan[t];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, w, o);
      if (t >= o) w += up;
    }
    scan[t] = w;
  }
  if (t == 0) chosen = -1;
  __syncthreads();
  const float before_warp = (t >> 5) ? scan[(t >> 5) - 1] : 0.f;
  incl += before_warp;
  float excl = __shfl_up_sync(0xffffffffu, incl, 1);  // the previous thread's inclusive sum: exactly monotone
  if ((t & 31) == 0) excl = before_warp;
  const float total = scan[31];
  const uint32_t bits = philox_first(off_lo, off_hi, static_cast<uint32_t>(b), 0u, seed_lo, seed_hi);
  const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  const float target = u * total;
  // the first thread (lowest t) whose inclusive sum reaches the target owns the token
  const bool here = incl >= target && excl < target;
  if (here) {
    float run = excl;
    int pick = -1;
    for (int i = i_begin; i < i_end; ++i) {
      const float p = pr[i];
      const float w = p > thr ? p : (p == thr ? p * comp : 0.f);
      if (w > 0.f) {
        pick = i;  // (the last kept token of the range if rounding leaves the sum just short of the target)
        run += w;
        if (run >= target) break;
      }
    }
    if (pick >= 0) atomicMax(&chosen, pick);  // at most one thread gets here; atomicMax keeps it well defined anyway
  }
  __syncthreads();
  if (chosen < 0) {
    // rounding at the very end of the scan (target above every inclusive sum): the last kept token of the vocabulary
    int last = -1;
    for (int i = i_begin; i < i_end; ++i) {
      const float p = pr[i];
      if (p > thr || (p == thr && comp > 0.f)) last = i;
    }
    if (last >= 0) atomicMax(&chosen, last);
    __syncthreads();
  }
  const int token = chosen >= 0 ? chosen : 0;
  if (t == 0) {
    out[b] = token;
    if (next_tokens) next_tokens[b] = token;
  }
  // 7: penalties
  if (!pen) return;
  for (int i = t; i < V; i += kSampleThreads) {
    const float p = pen[i];
    pen[i] = __fmaf_rn(p, decay, (i != token) ? 0.f : (p == 0.f ? presence : repetition));
  }
}

}  // namespace

int sample_tokens(cudaStream_t stream, int B, int V, const float* logits, float* penalties, float* probs, float presence,
                  float repetition, float decay, float temperature, int top_k, float top_p, unsigned long long seed,
                  unsigned long long offset, int* out, int64_t* next_tokens) {
  RK_REQUIRE(B > 0 && V > 0 && logits && probs && out, kBadArg, "sample: bad argument");
  RK_REQUIRE(temperature >= 0.001f && temperature <= 1000.f, kBadArg, "sample: temperature outside [0.001, 1000]");
  // the reference's normalisation (src/utils/sampling.cu:504-512)
  if (top_k <= 0 || top_k > V) top_k = V;
  if (!(top_p >= 0.f && top_p <= 1.f)) top_p = 1.f;
  if (top_p == 0.f) { top_k = 1; top_p = 1.f; }
  const float log2_inv_temp = 1.4426950408889634f / temperature;
  sample_kernel<<<B, kSampleThreads, 0, stream>>>(V, logits, penalties, probs, presence, repetition, decay, log2_inv_temp, top_k, top_p,
                                                  static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32),
                                                  static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32), out, next_tokens);
  RK_LAUNCH_CHECK("sample launch");
  return kOk;
}

}  // namespace rk
