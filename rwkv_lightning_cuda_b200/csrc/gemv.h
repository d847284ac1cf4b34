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
};

struct GemvBatch {
  int n_seg;
  GemvSeg seg[kMaxSeg];
};

#ifdef __CUDACC__
// Rounds and stores one fp32 accumulator: the single rounding point of a linear layer.
__device__ __forceinline__ void store_result(const GemvSeg& sg, int m, int n, float a) {
  const size_t o = static_cast<size_t>(m) * sg.N + n;
  if (sg.epi == kEpiF32) {
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
#endif

// gemv_tma.cu: fp16 weights fetched with per-warp rings of bulk copies (cp.async.bulk + mbarrier).
bool gemv_tma_plan(GemvBatch& b, int M, size_t* smem_bytes, int* grid, int* n_slots, int* slot_stride);
int gemv_tma_launch(cudaStream_t stream, const GemvBatch& b, int M, size_t smem_bytes, int grid, int n_slots, int slot_stride);

}  // namespace rk
