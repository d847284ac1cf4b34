// WKV-7 with fp32 state over a chunk of tokens in MATRIX form on the tensor cores (prefill), instead of one
// recurrence step per token.
//
// The recurrence of one head, S [64 value rows i] x [64 key columns j] (src/rwkv7_fast_v4.cu:1263-1271 ->
// cuda/rwkv7_wkv_fp32_v2.cu:66-132 of the reference):
//     u_t = S_{t-1} a_t ;  S_t = S_{t-1} diag(w_t) + u_t b_t^T + v_t k_t^T ;  y_t = S_t r_t
// Every value row evolves on its own under the same 64 x 64 transition, so rows split freely over warps.  For a
// sub-chunk of L = 16 tokens with P_t = w_1 * ... * w_t (per column, P_0 = 1) and the scaled vectors
//     A^_t = a_t * P_{t-1},  B^_t = b_t / P_t,  K^_t = k_t / P_t,  R^_t = r_t * P_t
// unrolling the recurrence gives, with U = [u_1 .. u_L] and V = [v_1 .. v_L] as (rows x L) matrices,
//     U  = (S_0 A^^T + V N_ka) (I - N_ab)^-1        N_ab = strict_upper(B^ A^^T),  N_ka = strict_upper(K^ A^^T)
//     Y  = S_0 R^^T + U M_br + V M_kr               M_br = upper(B^ R^^T),         M_kr = upper(K^ R^^T)
//     S_L = (S_0 + U B^ + V K^) diag(P_L)
// The L x L matrices depend on the token vectors only, so they are computed for all sub-chunks of a 64-token block at
// once; what stays sequential is three small products per sub-chunk instead of sixteen recurrence steps.  The
// decay per step is at least exp(-e^-0.5) = 0.545 by construction, so P_L >= 6e-5 over 16 tokens and the divisions
// are safe in fp32.
//
// All products run as mma.sync m16n8k8 on TF32 operands split in two (x = hi + lo, three MMAs per product: hi*hi +
// lo*hi + hi*lo), which keeps about 21 mantissa bits -- the state has to stay within 1e-4 of the sequential fp32
// recurrence.  (The warp-level MMA is used on purpose: a sub-chunk is a chain of 16-row products that each depend
// on the previous one; the asynchronous tcgen05 path adds a tensor-memory round trip per link of that chain.)
// One CTA of four warps per (sequence, head); warp w owns value rows 16 w .. 16 w + 15 and keeps its 16 x 64 slice of
// the state in accumulator registers for the whole call.
#include "common.cuh"
#include "kernels.h"

namespace rk {
namespace {

constexpr int kL = 16;        // tokens per sub-chunk
constexpr int kBlock = 64;    // tokens staged per block (four sub-chunks)
constexpr int kSub = kBlock / kL;
constexpr int kPitch = 68;    // floats per staged token row (64 + 4: conflict-free fragment loads)
constexpr int kMatPitch = 17;
constexpr int kThreadsChunk = 128;
constexpr int kPlaneTok = kBlock * kPitch;          // floats per plane of a token array
constexpr int kPlaneMat = kSub * kL * kMatPitch;    // floats per plane of a set of 16 x 16 matrices

__device__ __forceinline__ float decay_of(float w) {
  // exp(-exp(-0.5) * sigmoid(w)), as cuda/rwkv7_wkv_fp32_v2.cu:26-28 writes it
  return exp2f(-0.8750387749145276f / (1.0f + exp2f(-1.4426950408889634f * w)));
}

__device__ __forceinline__ uint32_t tf32_of(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = tf32_of(x);
  lo = tf32_of(x - __uint_as_float(hi));
}
// (not volatile: products into different accumulators are independent and the compiler may interleave them)
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// Operands live in shared memory already split: plane 0 holds hi = tf32(x) and plane 1 (kPlane floats further)
// lo = tf32(x - hi), so the inner loops convert nothing; the three MMAs of a product are hi*hi + lo*hi + hi*lo.
__device__ __forceinline__ void put_split(float* dst, int plane, float x) {
  uint32_t hi, lo;
  split_tf32(x, hi, lo);
  dst[0] = __uint_as_float(hi);
  dst[plane] = __uint_as_float(lo);
}

// Fragment conventions (lane = 4 g + t): an accumulator tile holds (g, 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1).
// An accumulator tile is fed back as the A operand of the next product by reading its columns in the order
// 2t, 2t+1 for the MMA's k = t, t+4; the B operand is then fetched with the same permutation of k.
// The cross terms go to their own accumulator (`lo`) so that consecutive MMAs do not wait for one another.

// acc[NT] += Acc[KS] * B, A taken from accumulator tiles; B(k, n) = bsrc[k * ldk + n * ldn] (+ plane for the low part).
template <int NT, int KS>
__device__ __forceinline__ void mm_acc_a(float (&acc)[NT][4], float (&lo)[NT][4], const float (&A)[KS][4], const float* bsrc,
                                         int plane, int ldk, int ldn, int g, int t) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const float a[4] = {A[ks][0], A[ks][2], A[ks][1], A[ks][3]};
    uint32_t ah[4], al[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) split_tf32(a[i], ah[i], al[i]);
    uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float* p = bsrc + (ks * 8 + 2 * t) * ldk + (nt * 8 + g) * ldn;
      bh[nt][0] = __float_as_uint(p[0]); bh[nt][1] = __float_as_uint(p[ldk]);
      bl[nt][0] = __float_as_uint(p[plane]); bl[nt][1] = __float_as_uint(p[plane + ldk]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(lo[nt], al, bh[nt]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(lo[nt], ah, bl[nt]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], ah, bh[nt]);
  }
}
// acc[NT] += A * B with A(row, k) = asrc[row * lda_r + k * lda_k] from shared memory (split planes unless kExactA:
// values that are fp16 numbers have no low part), natural k order.
template <int NT, int KS, bool kExactA>
__device__ __forceinline__ void mm_smem_a(float (&acc)[NT][4], float (&lo)[NT][4], const float* asrc, int aplane, int lda_r,
                                          int lda_k, const float* bsrc, int plane, int ldk, int ldn, int g, int t) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int k0 = ks * 8 + t;
    const float* pa[4] = {asrc + g * lda_r + k0 * lda_k, asrc + (g + 8) * lda_r + k0 * lda_k, asrc + g * lda_r + (k0 + 4) * lda_k,
                          asrc + (g + 8) * lda_r + (k0 + 4) * lda_k};
    uint32_t ah[4], al[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ah[i] = __float_as_uint(pa[i][0]);
      al[i] = kExactA ? 0u : __float_as_uint(pa[i][aplane]);
    }
    uint32_t bh[NT][2], bl[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float* p = bsrc + k0 * ldk + (nt * 8 + g) * ldn;
      bh[nt][0] = __float_as_uint(p[0]); bh[nt][1] = __float_as_uint(p[4 * ldk]);
      bl[nt][0] = __float_as_uint(p[plane]); bl[nt][1] = __float_as_uint(p[plane + 4 * ldk]);
    }
    if (!kExactA) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma_tf32(lo[nt], al, bh[nt]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(lo[nt], ah, bl[nt]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], ah, bh[nt]);
  }
}
template <int NT>
__device__ __forceinline__ void fold(float (&acc)[NT][4], float (&lo)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) { acc[nt][e] += lo[nt][e]; lo[nt][e] = 0.f; }
}


template <bool kAddW0>
__global__ void __launch_bounds__(kThreadsChunk) wkv7_fp32_chunk_kernel(
    int T, int C, int H, float* __restrict__ state, const half* __restrict__ r, const half* __restrict__ w,
    const half* __restrict__ w0, const half* __restrict__ k, const half* __restrict__ v, const half* __restrict__ a,
    const half* __restrict__ b, half* __restrict__ y) {
  extern __shared__ __align__(16) float sm[];
  // token vectors of the block, each as two planes (hi, lo) of [64][68]; v is exact in TF32 (it is an fp16 value)
  float* Ah = sm;                          // a * P_{t-1}   (plane 0 first holds P_{t-1})
  float* Bh = Ah + 2 * kPlaneTok;          // b / P_t
  float* Kh = Bh + 2 * kPlaneTok;          // k / P_t       (plane 0 first holds the decays, then P_t)
  float* Rh = Kh + 2 * kPlaneTok;          // r * P_t
  float* Vs = Rh + 2 * kPlaneTok;          // v, [t][i]
  float* Nka = Vs + kPlaneTok;             // the 16 x 16 matrices of the four sub-chunks, two planes of [4][16][17] each
  float* Tm = Nka + 2 * kPlaneMat;
  float* Mbr = Tm + 2 * kPlaneMat;
  float* Mkr = Mbr + 2 * kPlaneMat;
  float* PL = Mkr + 2 * kPlaneMat;         // [4][64]
  half* Ysm = reinterpret_cast<half*>(PL + kSub * kHead);  // [64][64 + 8]
  constexpr int kYPitch = kHead + 8;

  const int bh = blockIdx.x, b_id = bh / H, h = bh - b_id * H;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const size_t tok0 = (static_cast<size_t>(b_id) * T) * C + static_cast<size_t>(h) * kHead;
  const int i0 = warp * 16;  // this warp's value rows

  // the warp's 16 x 64 slice of the state, as eight accumulator tiles
  float S[8][4];
  float* sbase = state + static_cast<size_t>(bh) * (kHead * kHead);
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const float2 lo = *reinterpret_cast<const float2*>(sbase + (i0 + g) * kHead + nt * 8 + 2 * t4);
    const float2 hi = *reinterpret_cast<const float2*>(sbase + (i0 + g + 8) * kHead + nt * 8 + 2 * t4);
    S[nt][0] = lo.x; S[nt][1] = lo.y; S[nt][2] = hi.x; S[nt][3] = hi.y;
  }

  for (int tb = 0; tb < T; tb += kBlock) {
    const int n_tok = min(kBlock, T - tb);
    // the block's other token vectors are requested now (twenty 16-byte loads per thread) and used in step A3, after
    // the decays and their running products: their latency hides behind those two steps
    uint4 q[4][5];
    {
      const int j0 = (tid & 7) * 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tl = (tid + kThreadsChunk * i) >> 3;
        const size_t o = tok0 + static_cast<size_t>(tb + tl) * C + j0;
        const half* src[5] = {r, k, a, b, v};
#pragma unroll
        for (int x = 0; x < 5; ++x) q[i][x] = tl < n_tok ? *reinterpret_cast<const uint4*>(src[x] + o) : make_uint4(0, 0, 0, 0);
      }
    }
    // ---- A1: decays of the block's tokens (tokens past the end leave the state alone: decay 1, vectors 0).
    // A thread takes four 16-byte pieces (8 channels of one token each) per tensor and requests them all at once.
    {
      uint4 wq4[4];
      const int j0 = (tid & 7) * 8;  // the same 8 channels in all four pieces
      uint4 w0q = make_uint4(0, 0, 0, 0);
      if (kAddW0) w0q = *reinterpret_cast<const uint4*>(w0 + h * kHead + j0);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tl = (tid + kThreadsChunk * i) >> 3;
        wq4[i] = tl < n_tok ? *reinterpret_cast<const uint4*>(w + tok0 + static_cast<size_t>(tb + tl) * C + j0) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tl = (tid + kThreadsChunk * i) >> 3;
        const uint32_t wq[4] = {wq4[i].x, wq4[i].y, wq4[i].z, wq4[i].w}, w0w[4] = {w0q.x, w0q.y, w0q.z, w0q.w};
        float d[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 wf = h2f2(wq[e]);
          if (kAddW0) {
            const float2 w0f = h2f2(w0w[e]);
            wf.x = __half2float(__float2half_rn(wf.x + w0f.x));  // the reference pre-adds w0 and rounds to half
            wf.y = __half2float(__float2half_rn(wf.y + w0f.y));
          }
          d[2 * e] = tl < n_tok ? decay_of(wf.x) : 1.f;
          d[2 * e + 1] = tl < n_tok ? decay_of(wf.y) : 1.f;
        }
        *reinterpret_cast<float4*>(Kh + tl * kPitch + j0) = make_float4(d[0], d[1], d[2], d[3]);
        *reinterpret_cast<float4*>(Kh + tl * kPitch + j0 + 4) = make_float4(d[4], d[5], d[6], d[7]);
      }
    }
    __syncthreads();
    // ---- A2: running products per column inside every sub-chunk: Kh <- P_t, Ah <- P_{t-1}
    for (int idx = tid; idx < kSub * kHead; idx += kThreadsChunk) {
      const int c = idx >> 6, j = idx & 63;
      float p = 1.f;
#pragma unroll
      for (int tl = 0; tl < kL; ++tl) {
        const int row = (c * kL + tl) * kPitch + j;
        Ah[row] = p;
        p *= Kh[row];
        Kh[row] = p;
      }
      PL[c * kHead + j] = p;
    }
    __syncthreads();
    // ---- A3: the scaled token vectors
    {
      const int j0 = (tid & 7) * 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tl = (tid + kThreadsChunk * i) >> 3;
        const int row = tl * kPitch + j0;
        const uint32_t* rq = &q[i][0].x;
        const uint32_t* kq = &q[i][1].x;
        const uint32_t* aq = &q[i][2].x;
        const uint32_t* bq = &q[i][3].x;
        const uint32_t* vq = &q[i][4].x;
        // eight channels of one token: the products, split, then stored as 16-byte vectors per plane
        float pa[8], pb[8], pk[8], pr[8], pv[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 rv = h2f2(rq[e]), kv = h2f2(kq[e]), av = h2f2(aq[e]), bv = h2f2(bq[e]), vv = h2f2(vq[e]);
          const float2 P = *reinterpret_cast<const float2*>(Kh + row + 2 * e), Pp = *reinterpret_cast<const float2*>(Ah + row + 2 * e);
          const float2 iP = make_float2(1.0f / P.x, 1.0f / P.y);
          pa[2 * e] = av.x * Pp.x; pa[2 * e + 1] = av.y * Pp.y;
          pb[2 * e] = bv.x * iP.x; pb[2 * e + 1] = bv.y * iP.y;
          pk[2 * e] = kv.x * iP.x; pk[2 * e + 1] = kv.y * iP.y;
          pr[2 * e] = rv.x * P.x;  pr[2 * e + 1] = rv.y * P.y;
          pv[2 * e] = vv.x; pv[2 * e + 1] = vv.y;
        }
        auto store_split = [&](float* dst, const float (&x)[8]) {
          float hi[8], lo[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            uint32_t h32, l32;
            split_tf32(x[e], h32, l32);
            hi[e] = __uint_as_float(h32);
            lo[e] = __uint_as_float(l32);
          }
          *reinterpret_cast<float4*>(dst) = make_float4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(hi[4], hi[5], hi[6], hi[7]);
          *reinterpret_cast<float4*>(dst + kPlaneTok) = make_float4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<float4*>(dst + kPlaneTok + 4) = make_float4(lo[4], lo[5], lo[6], lo[7]);
        };
        store_split(Ah + row, pa);
        store_split(Bh + row, pb);
        store_split(Kh + row, pk);
        store_split(Rh + row, pr);
        *reinterpret_cast<float4*>(Vs + row) = make_float4(pv[0], pv[1], pv[2], pv[3]);
        *reinterpret_cast<float4*>(Vs + row + 4) = make_float4(pv[4], pv[5], pv[6], pv[7]);
      }
    }
    __syncthreads();
    // ---- B: the 16 x 16 matrices of sub-chunk `warp`: rows s (tokens of B^ / K^), columns t (tokens of A^ / R^)
    {
      const int c = warp;
      const float* Xb = Bh + c * kL * kPitch;
      const float* Xk = Kh + c * kL * kPitch;
      const float* Ya = Ah + c * kL * kPitch;
      const float* Yr = Rh + c * kL * kPitch;
      float nab[2][4] = {}, nka[2][4] = {}, mbr[2][4] = {}, mkr[2][4] = {}, lo[2][4] = {};
      // A(s, j) = X[s][j]; B(j, t) = Y[t][j]
      mm_smem_a<2, 8, false>(nab, lo, Xb, kPlaneTok, kPitch, 1, Ya, kPlaneTok, 1, kPitch, g, t4);
      fold(nab, lo);
      mm_smem_a<2, 8, false>(nka, lo, Xk, kPlaneTok, kPitch, 1, Ya, kPlaneTok, 1, kPitch, g, t4);
      fold(nka, lo);
      mm_smem_a<2, 8, false>(mbr, lo, Xb, kPlaneTok, kPitch, 1, Yr, kPlaneTok, 1, kPitch, g, t4);
      fold(mbr, lo);
      mm_smem_a<2, 8, false>(mkr, lo, Xk, kPlaneTok, kPitch, 1, Yr, kPlaneTok, 1, kPitch, g, t4);
      fold(mkr, lo);
      float* m_nab = Tm + c * kL * kMatPitch;
      float* m_nka = Nka + c * kL * kMatPitch;
      float* m_mbr = Mbr + c * kL * kMatPitch;
      float* m_mkr = Mkr + c * kL * kMatPitch;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int s = g + (e >> 1) * 8, tt = nt * 8 + 2 * t4 + (e & 1);
          m_nab[s * kMatPitch + tt] = s < tt ? nab[nt][e] : 0.f;   // plain fp32: inverted below, split afterwards
          put_split(m_nka + s * kMatPitch + tt, kPlaneMat, s < tt ? nka[nt][e] : 0.f);
          put_split(m_mbr + s * kMatPitch + tt, kPlaneMat, s <= tt ? mbr[nt][e] : 0.f);
          put_split(m_mkr + s * kMatPitch + tt, kPlaneMat, s <= tt ? mkr[nt][e] : 0.f);
        }
      }
      __syncwarp();
      // (I - N_ab)^-1, column by column: T[s][t] = [s == t] + sum_{m > s} N[s][m] T[m][t] (T is upper triangular, so the
      // terms with m > t vanish by themselves).  Lane t < 16 keeps column t in registers and walks s downwards; the
      // rows of N are read from shared memory (the same address for every lane).
      if (lane < kL) {
        float Tc[kL];
#pragma unroll
        for (int s = kL - 1; s >= 0; --s) {
          float val = s == lane ? 1.f : 0.f;
#pragma unroll
          for (int m = s + 1; m < kL; ++m) val = fmaf(m_nab[s * kMatPitch + m], Tc[m], val);
          Tc[s] = val;
        }
        __syncwarp(0x0000ffffu);  // every column has read N before it is overwritten
#pragma unroll
        for (int s = 0; s < kL; ++s) put_split(m_nab + s * kMatPitch + lane, kPlaneMat, Tc[s]);
      }
    }
    __syncthreads();
    // ---- C: the sequential part, sub-chunk after sub-chunk, every warp on its own 16 rows
    for (int c = 0; c < kSub; ++c) {
      const float* Ya = Ah + c * kL * kPitch;
      const float* Yr = Rh + c * kL * kPitch;
      const float* Xb = Bh + c * kL * kPitch;
      const float* Xk = Kh + c * kL * kPitch;
      const float* Vc = Vs + c * kL * kPitch + i0;  // A(i, s) = Vc[s * kPitch + i]
      const float* m_t = Tm + c * kL * kMatPitch;
      const float* m_nka = Nka + c * kL * kMatPitch;
      const float* m_mbr = Mbr + c * kL * kMatPitch;
      const float* m_mkr = Mkr + c * kL * kMatPitch;
      // X = S A^^T + V N_ka        B(j, t) = A^[t][j]; B(s, t) = N_ka[s][t]
      float X[2][4] = {}, lo[2][4] = {};
      mm_acc_a<2, 8>(X, lo, S, Ya, kPlaneTok, 1, kPitch, g, t4);
      mm_smem_a<2, 2, true>(X, lo, Vc, 0, 1, kPitch, m_nka, kPlaneMat, kMatPitch, 1, g, t4);
      fold(X, lo);
      // U = X (I - N_ab)^-1
      float U[2][4] = {};
      mm_acc_a<2, 2>(U, lo, X, m_t, kPlaneMat, kMatPitch, 1, g, t4);
      fold(U, lo);
      // Y = S R^^T + U M_br + V M_kr   (rows i, columns t)
      float Y[2][4] = {};
      mm_acc_a<2, 8>(Y, lo, S, Yr, kPlaneTok, 1, kPitch, g, t4);
      mm_acc_a<2, 2>(Y, lo, U, m_mbr, kPlaneMat, kMatPitch, 1, g, t4);
      mm_smem_a<2, 2, true>(Y, lo, Vc, 0, 1, kPitch, m_mkr, kPlaneMat, kMatPitch, 1, g, t4);
      fold(Y, lo);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + g + (e >> 1) * 8, tt = c * kL + nt * 8 + 2 * t4 + (e & 1);
          Ysm[tt * kYPitch + i] = __float2half_rn(Y[nt][e]);
        }
      }
      // S = (S + U B^ + V K^) diag(P_L)     B(s, j) = B^[s][j], K^[s][j]   (eight column tiles: the cross terms go
      // straight into S, consecutive MMAs already hit different tiles)
      mm_acc_a<8, 2>(S, S, U, Xb, kPlaneTok, kPitch, 1, g, t4);
      mm_smem_a<8, 2, true>(S, S, Vc, 0, 1, kPitch, Xk, kPlaneTok, kPitch, 1, g, t4);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float2 pl = *reinterpret_cast<const float2*>(PL + c * kHead + nt * 8 + 2 * t4);
        S[nt][0] *= pl.x; S[nt][1] *= pl.y; S[nt][2] *= pl.x; S[nt][3] *= pl.y;
      }
    }
    __syncthreads();
    // ---- D: this block's outputs, coalesced
    for (int idx = tid; idx < kBlock * 8; idx += kThreadsChunk) {
      const int tl = idx >> 3, c8 = (idx & 7) * 8;
      if (tl < n_tok)
        *reinterpret_cast<uint4*>(y + tok0 + static_cast<size_t>(tb + tl) * C + c8) = *reinterpret_cast<const uint4*>(Ysm + tl * kYPitch + c8);
    }
    __syncthreads();
  }
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    *reinterpret_cast<float2*>(sbase + (i0 + g) * kHead + nt * 8 + 2 * t4) = make_float2(S[nt][0], S[nt][1]);
    *reinterpret_cast<float2*>(sbase + (i0 + g + 8) * kHead + nt * 8 + 2 * t4) = make_float2(S[nt][2], S[nt][3]);
  }
}

constexpr size_t kChunkSmem = (9 * kPlaneTok + 8 * kPlaneMat + kSub * kHead) * sizeof(float) + kBlock * (kHead + 8) * sizeof(half);

}  // namespace


// Chunks of at least this many tokens take the matrix form (below it the per-token scan is faster: the matrix form
// stages and prepares a block of 64 tokens at a time).
bool wkv7_fp32_chunked_applies(int T) { return T >= 64; }

int wkv7_fp32_chunked(cudaStream_t stream, int B, int T, int C, int H, float* state, const half* r, const half* w,
                      const half* w0, const half* k, const half* v, const half* a, const half* b, half* y) {
  static bool attr_set[64] = {};
  int dev = 0;
  RK_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    RK_CUDA(cudaFuncSetAttribute(wkv7_fp32_chunk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kChunkSmem)));
    RK_CUDA(cudaFuncSetAttribute(wkv7_fp32_chunk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kChunkSmem)));
    attr_set[dev] = true;
  }
  const dim3 grid(B * H), block(kThreadsChunk);
  if (w0) wkv7_fp32_chunk_kernel<true><<<grid, block, kChunkSmem, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y);
  else wkv7_fp32_chunk_kernel<false><<<grid, block, kChunkSmem, stream>>>(T, C, H, state, r, w, w0, k, v, a, b, y);
  RK_LAUNCH_CHECK("wkv7_fp32_chunked launch");
  return kOk;
}

}  // namespace rk
