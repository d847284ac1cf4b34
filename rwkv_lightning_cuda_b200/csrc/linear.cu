// Weight-streaming linear layers for decode-sized row counts (M <= 4): y = epi(act(x) W^T),
// W [N,K] row-major in fp16, int8 (W8A16) or packed int4 (W4A16, group 128).
//
// Memory-bound by construction: every weight byte is read exactly once with 128-bit
// non-allocating loads, two stages of eight loads per lane are kept in flight (register double
// buffering), the activations are staged once per CTA in shared memory, weights are dequantised
// in registers, accumulated in fp32 and reduced with warp shuffles; the result is rounded to half
// once (the reference's rounding point, cuda/rwkv7_v3a_ops.cu:464-509).  Several independent
// problems (e.g. the r/k/v projections and the LoRA down-projections of one layer) run as one
// launch.  The first weight stage is requested before the programmatic-dependency wait, so the
// HBM stream of one kernel starts while its predecessor drains.
//
// Replaces linear_orig_row{1,2}_exact*_f16_kernel, the linear_t*/LoRA kernels and the sparse
// FFN-down kernels (cuda/rwkv7_v3a_ops.cu:209-1270, cuda/rwkv7_fast_ops_fp16.cu:487-827) for
// rows <= 4; larger row counts go to the tensor-core GEMM.
#include <algorithm>
#include <type_traits>

#include "gemv.h"
#include "kernels.h"

namespace rk {

int gemm_tc(cudaStream_t stream, const LinearArgs& a);  // gemm_tcgen05.cu
int gemm_group(cudaStream_t stream, const LinearArgs* a, int n);
bool gemm_tc_supported(const LinearArgs& a);

namespace {

constexpr int kWarps = 8;       // warps per CTA
constexpr int kU = 4;           // 16-byte chunks per lane and weight row in one stage
constexpr int kRowsPerTile = 2 * kWarps;

template <int kFmt>
struct Fmt;
template <>
struct Fmt<0> { static constexpr int kElems = 8; };   // 8 halves per 16-byte load
template <>
struct Fmt<1> { static constexpr int kElems = 16; };  // 16 int8
template <>
struct Fmt<2> { static constexpr int kElems = 32; };  // 32 int4

template <int kFmt>
struct Stage {
  uint4 w[kU][2];
  __half2 sz[kU][2];  // W4A16: (scale, zero) of the chunk's group
};

template <int kM, int kFmt>
__device__ __forceinline__ void run_segment(const GemvSeg& sg, half* xs16, float* xs32, int row0, int rows_end) {
  constexpr int E = Fmt<kFmt>::kElems;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = sg.K;
  const size_t row_bytes = static_cast<size_t>(K) * 16 / E;
  const int groups = K >> 7;
  const int chunk_span = 32 * E;                              // elements covered by one warp-wide chunk
  const int n_stages = (K + chunk_span * kU - 1) / (chunk_span * kU);
  const int first = row0 + 2 * warp;
  const int n_pairs = first < rows_end ? (rows_end - first + kRowsPerTile - 1) / kRowsPerTile : 0;
  const int total = n_pairs * n_stages;
  const char* wbase = static_cast<const char*>(sg.w);

  auto issue = [&](int item, Stage<kFmt>& st) {
    const int pair = item / n_stages, stg = item - pair * n_stages;
    const int n = first + pair * kRowsPerTile;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int k = (stg * kU + u) * chunk_span + lane * E;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const bool ok = k < K && n + j < rows_end;
        st.w[u][j] = ok ? ldg_stream(wbase + static_cast<size_t>(n + j) * row_bytes + static_cast<size_t>(k) * 16 / E)
                        : make_uint4(0, 0, 0, 0);
        if (kFmt == 2) {
          const size_t gi = static_cast<size_t>(ok ? n + j : row0) * groups + (ok ? (k >> 7) : 0);
          st.sz[u][j] = __halves2half2(sg.scale[gi], sg.zero[gi]);
        }
      }
    }
  };

  float acc[kM][2];
  auto compute = [&](int item, const Stage<kFmt>& st) {
    const int pair = item / n_stages, stg = item - pair * n_stages;
    if (stg == 0) {
#pragma unroll
      for (int m = 0; m < kM; ++m) acc[m][0] = acc[m][1] = 0.f;
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int k = (stg * kU + u) * chunk_span + lane * E;
      if (k >= K) break;
      float wf[2][E];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float s = 0.f, z = 0.f;
        if (kFmt == 2) {
          s = __low2float(st.sz[u][j]);
          z = __high2float(st.sz[u][j]);
        }
        dequant_chunk<kFmt>(st.w[u][j], wf[j], s, z);
      }
#pragma unroll
      for (int m = 0; m < kM; ++m) {
#pragma unroll
        for (int c = 0; c < E / 8; ++c) {
          float xf[8];
          if (xs32) {
            const float4 a = *reinterpret_cast<const float4*>(xs32 + static_cast<size_t>(m) * K + k + c * 8);
            const float4 b = *reinterpret_cast<const float4*>(xs32 + static_cast<size_t>(m) * K + k + c * 8 + 4);
            xf[0] = a.x; xf[1] = a.y; xf[2] = a.z; xf[3] = a.w; xf[4] = b.x; xf[5] = b.y; xf[6] = b.z; xf[7] = b.w;
          } else {
            const uint4 xq = *reinterpret_cast<const uint4*>(xs16 + static_cast<size_t>(m) * K + k + c * 8);
            const uint32_t xu[4] = {xq.x, xq.y, xq.z, xq.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = h2f2(xu[i]);
              xf[2 * i] = f.x;
              xf[2 * i + 1] = f.y;
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            acc[m][0] = fmaf(xf[i], wf[0][c * 8 + i], acc[m][0]);
            acc[m][1] = fmaf(xf[i], wf[1][c * 8 + i], acc[m][1]);
          }
        }
      }
    }
    if (stg != n_stages - 1) return;
    const int n = first + pair * kRowsPerTile;
#pragma unroll
    for (int m = 0; m < kM; ++m) {
      acc[m][0] = warp_sum(acc[m][0]);
      acc[m][1] = warp_sum(acc[m][1]);
    }
    if (lane < 2 && n + lane < rows_end) {
      const int nn = n + lane;
      const float sc = (kFmt == 1) ? __half2float(sg.scale[nn]) : 1.0f;
#pragma unroll
      for (int m = 0; m < kM; ++m) {
        store_result(sg, m, nn, (lane == 0 ? acc[m][0] : acc[m][1]) * sc);
      }
    }
  };

  // Weights do not depend on the previous kernel: request the first stage before waiting for it.
  Stage<kFmt> sa, sb;
  if (total > 0) issue(0, sa);
  pdl_wait();
  pdl_trigger();
  stage_activations<kM, kWarps * 32>(sg, xs16, xs32);
  __syncthreads();
  for (int item = 0; item < total; item += 2) {
    if (item + 1 < total) issue(item + 1, sb);
    compute(item, sa);
    if (item + 1 < total) {
      if (item + 2 < total) issue(item + 2, sa);
      compute(item + 1, sb);
    }
  }
}

// kMaxFmt: highest weight format present in the batch; code for formats above it is not compiled
// in, which keeps the fp16-only kernel's register count (and so its occupancy) unaffected by int4.
template <int kM, int kMaxFmt>
__global__ void __launch_bounds__(kWarps * 32) gemv_multi_kernel(const GemvBatch p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int s = 0;
#pragma unroll
  for (int i = 1; i < kMaxSeg; ++i)
    if (i < p.n_seg && static_cast<int>(blockIdx.x) >= p.seg[i].cta_begin) s = i;
  const GemvSeg& sg = p.seg[s];
  const int row0 = (blockIdx.x - sg.cta_begin) * sg.rows_per_cta;
  const int rows_end = min(sg.N, row0 + sg.rows_per_cta);
  half* xs16 = sg.in_act == kActNone ? reinterpret_cast<half*>(smem_raw) : nullptr;
  float* xs32 = sg.in_act == kActNone ? nullptr : reinterpret_cast<float*>(smem_raw);
  if (kMaxFmt >= 2 && sg.fmt == 2) run_segment<kM, 2>(sg, xs16, xs32, row0, rows_end);
  else if (kMaxFmt >= 1 && sg.fmt == 1) run_segment<kM, 1>(sg, xs16, xs32, row0, rows_end);
  else run_segment<kM, 0>(sg, xs16, xs32, row0, rows_end);
}

int check_args(const LinearArgs& a) {
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
  return kOk;
}

}  // namespace

// Up to 8 independent problems with the same row count M <= 4 in one launch.
int linear_batch(cudaStream_t stream, const LinearArgs* args, int n) {
  RK_REQUIRE(args && n > 0 && n <= kMaxSeg, kBadArg, "linear_batch: 1..%d problems", kMaxSeg);
  const int M = args[0].M;
  RK_REQUIRE(M >= 1 && M <= 4, kShape, "linear_batch: M must be 1..4");
  GemvBatch b;
  b.n_seg = n;
  long long tiles = 0;
  size_t smem = 0;
  for (int i = 0; i < n; ++i) {
    int s = check_args(args[i]);
    if (s != kOk) return s;
    RK_REQUIRE(args[i].M == M, kShape, "linear_batch: all problems must share M");
    tiles += (args[i].N + kRowsPerTile - 1) / kRowsPerTile;
    smem = std::max(smem, static_cast<size_t>(M) * args[i].K * (args[i].in_act == kActNone ? 2 : 4));
  }
  int max_fmt = 0;
  bool fused = false;
  for (int i = 0; i < n; ++i) {
    const LinearArgs& a = args[i];
    GemvSeg& g = b.seg[i];
    g.x = a.x; g.w = a.w; g.scale = a.scale; g.zero = a.zero; g.y = a.y;
    g.v = a.ea.v; g.v_first = a.ea.v_first; g.v0 = a.ea.v0;
    g.ldx = a.ldx ? a.ldx : a.K; g.N = a.N; g.K = a.K; g.fmt = a.fmt; g.in_act = a.in_act; g.epi = a.epi;
    g.cta_begin = 0; g.rows_per_cta = 0; g.parts = 0; g.piece_bytes = 0;
    g.res = a.res; g.ln_w = a.ln_w; g.ln_b = a.ln_b; g.shift = a.shift; g.mix = a.mix; g.x_out = a.x_out; g.n_out = a.n_out;
    g.eps = a.eps; g.copy_src = a.copy_src; g.copy_dst = a.copy_dst; g.copy_n = a.copy_n;
    fused = fused || a.ln_w || a.copy_src;
    max_fmt = std::max(max_fmt, a.fmt);
  }
  for (int i = n; i < kMaxSeg; ++i) b.seg[i] = b.seg[0];
  b.timeout = timeout_word_or_null();

  // The kernel built on the warp-level tensor-core instruction (gemv_mma.cu) takes, by default (option gemv_mma = 3):
  // W4A16 at any row count; 2..4 rows of W8A16 and fp16; and ONE row of fp16 / W8A16 when the launch streams at least
  // 8 MB and every weight row gives each of the 16 warps of a CTA a box (fp16: rows of 2 KiB and more) or two (W8A16:
  // 4 KiB and more) -- there its 2-D tensor copies and warps working on the same rows stream faster than the per-warp
  // bulk-copy rings below (decode step of 7.2B fp16 2.85 -> 2.59 ms, 7.2B W8A16 2.12 -> 1.96 ms, 2.9B fp16 1.68 -> 1.54 ms,
  // 1.5B fp16 0.94 -> 0.91 ms), while smaller launches are latency-bound and stay on the scalar kernel (1.5B W8A16 0.81
  // against 0.84 ms, 0.1B 0.25 against 0.26 ms).
  const int mma_mode = options().gemv_mma;
  double launch_bytes = 0;
  int min_row_bytes = 1 << 30;
  for (int i = 0; i < n; ++i) {
    const int rb = args[i].fmt == 0 ? args[i].K * 2 : args[i].fmt == 1 ? args[i].K : args[i].K / 2;
    launch_bytes += static_cast<double>(args[i].N) * rb;
    min_row_bytes = std::min(min_row_bytes, rb);
  }
  const bool one_row_scalar = M == 1 && max_fmt <= 1;   // one row of fp16 / W8A16: the scalar kernel's home ground
  long long launch_rows = 0;
  for (int i = 0; i < n; ++i) launch_rows += args[i].N;
  // (W8A16 also wants about a 32-channel tile per CTA: the 2048 x 8192 ffn.value of the 1.5B model is faster on the scalar kernel)
  const bool large = launch_bytes >= 8e6 && min_row_bytes >= (max_fmt == 0 ? 2048 : 4096) && (max_fmt == 0 || launch_rows >= 4096);
  const bool use_mma = mma_mode >= 4 || (one_row_scalar ? (mma_mode >= 3 && large)
                                                        : ((mma_mode >= 1 && max_fmt > 0) || (mma_mode >= 2 && M >= 2)));
  if (use_mma) {
    GemvMmaPlan mp;
    if (gemv_mma_plan(b, M, &mp)) return gemv_mma_launch(stream, b, M, mp);
  }
  // bulk-copy kernel (shared-memory rings fed by the copy engine); the register-staged kernel below takes what it
  // cannot (row sizes that do not cut into 16-byte pieces, activations too large for shared memory)
  size_t tma_smem = 0;
  int tma_grid = 0, tma_slots = 0, tma_stride = 0, tma_warps = 0;
  if (gemv_tma_plan(b, M, &tma_smem, &tma_grid, &tma_slots, &tma_stride, &tma_warps))
    return gemv_tma_launch(stream, b, M, tma_smem, tma_grid, tma_slots, tma_stride, tma_warps);

  RK_REQUIRE(!fused, kShape, "linear_batch: the fused LayerNorm prologue needs fp16 weights and a row size the bulk-copy kernel accepts");
  RK_REQUIRE(smem <= 160 * 1024, kShape, "linear_batch: M*K too large for the activation staging buffer");
  const int tiles_per_cta = static_cast<int>(std::max<long long>(1, (tiles + 295) / 296));  // about two CTAs per SM
  int cta = 0;
  for (int i = 0; i < n; ++i) {
    GemvSeg& g = b.seg[i];
    g.cta_begin = cta;
    g.rows_per_cta = tiles_per_cta * kRowsPerTile;
    cta += (g.N + g.rows_per_cta - 1) / g.rows_per_cta;
  }
  for (int i = n; i < kMaxSeg; ++i) b.seg[i] = b.seg[0];
  const dim3 grid(cta), block(kWarps * 32);
  auto launch = [&](auto kernel) -> int {
    if (smem > 48 * 1024) RK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    RK_CUDA(launch_pdl(kernel, grid, block, smem, stream, b));
    return kOk;
  };
  auto by_m = [&](auto fmt_tag) -> int {
    constexpr int F = decltype(fmt_tag)::value;
    switch (M) {
      case 1: return launch(gemv_multi_kernel<1, F>);
      case 2: return launch(gemv_multi_kernel<2, F>);
      case 3: return launch(gemv_multi_kernel<3, F>);
      default: return launch(gemv_multi_kernel<4, F>);
    }
  };
  int s;
  if (max_fmt == 0) s = by_m(std::integral_constant<int, 0>{});
  else if (max_fmt == 1) s = by_m(std::integral_constant<int, 1>{});
  else s = by_m(std::integral_constant<int, 2>{});
  if (s != kOk) return s;
  RK_LAUNCH_CHECK("gemv launch");
  return kOk;
}

int linear(cudaStream_t stream, const LinearArgs& a) {
  int s = check_args(a);
  if (s != kOk) return s;
  if ((a.M > 4 || (a.prefer_tc && a.M >= 2)) && gemm_tc_supported(a)) return gemm_tc(stream, a);
  const int ldx = a.ldx ? a.ldx : a.K;
  const size_t out_elem = (a.epi == kEpiF32 || a.epi == kEpiRawF32) ? sizeof(float) : sizeof(half);
  for (int m0 = 0; m0 < a.M; m0 += 4) {
    LinearArgs c = a;
    c.M = a.M - m0 < 4 ? a.M - m0 : 4;
    c.ldx = ldx;
    c.x = a.x + static_cast<size_t>(m0) * ldx;
    c.y = static_cast<char*>(a.y) + static_cast<size_t>(m0) * a.N * out_elem;
    if (a.ea.v) c.ea.v = a.ea.v + static_cast<size_t>(m0) * a.N;
    if (a.ea.v_first) c.ea.v_first = a.ea.v_first + static_cast<size_t>(m0) * a.N;
    s = linear_batch(stream, &c, 1);
    if (s != kOk) return s;
  }
  return kOk;
}

bool linear_batch_fused_fits(int M, int K) { return M >= 1 && M <= 4 && gemv_tma_fits(M, K); }

int linear_group(cudaStream_t stream, const LinearArgs* args, int n) {
  RK_REQUIRE(args && n >= 1 && n <= 8, kBadArg, "linear_group: 1..8 products");
  bool together = true;
  for (int i = 0; i < n; ++i)
    together = together && (args[i].M > 4 || (args[i].prefer_tc && args[i].M >= 2)) && args[i].M == args[0].M && gemm_tc_supported(args[i]);
  if (together) return gemm_group(stream, args, n);
  for (int i = 0; i < n; ++i) {
    LinearArgs b = args[i];
    int act = kActNone;
    if (b.epi == kEpiTanhH) act = kActTanh;
    if (b.epi == kEpiSigmoidH) act = kActSigmoid;
    if (act != kActNone) b.epi = kEpiNone;
    if (!b.scratch) { b.scratch = args[0].scratch; b.scratch_bytes = args[0].scratch_bytes; }
    int s = linear(stream, b);
    if (s != kOk) return s;
    if (act != kActNone) {
      half* y = static_cast<half*>(b.y);
      s = activate(stream, y, y, static_cast<long long>(b.M) * b.N, act);
      if (s != kOk) return s;
    }
  }
  return kOk;
}

}  // namespace rk
