/*
 * CPU oracle of the RWKV-7 per-layer forward hot path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA kernels and the timed CPU baseline of the benchmark;
 * no product code path may call it.
 *
 * Every function restates, as scalar C, the arithmetic of one reference launcher
 * (paths are relative to the reference project root):
 *   orc_layer_norm ............ cuda/rwkv7_v3a_ops.cu:1272-1308
 *   orc_add_layer_norm ........ cuda/rwkv7_v3a_ops.cu:1310-1351
 *   orc_add_last_layer_norm ... cuda/rwkv7_v3a_ops.cu:1886-1931
 *   orc_emb_ln0 ............... cuda/rwkv7_v3a_ops.cu:153-187
 *   orc_tmix_mix6 ............. cuda/rwkv7_fast_ops_fp16.cu:53-127
 *   orc_cmix_mix .............. cuda/rwkv7_fast_ops_fp16.cu:393-419
 *   orc_kk_a_gate ............. cuda/rwkv7_fast_ops_fp16.cu:129-172
 *   orc_lnx_rkvres_xg ......... cuda/rwkv7_fast_ops_fp16.cu:174-237
 *   orc_vres_gate ............. cuda/rwkv7_fast_ops_fp16.cu:239-255
 *   orc_linear_orig ........... cuda/rwkv7_v3a_ops.cu:464-509 (y = x W^T, fp32 accumulate, one rounding)
 *   orc_linear_kn ............. cuda/rwkv7_v3a_ops.cu:209-241 (y = x W, W stored [K,N])
 *   orc_wkv_fp32 .............. cuda/rwkv7_wkv_fp32_v2.cu:26-28,66-132
 *   orc_wkv_fp16 .............. cuda/rwkv7_wkv_fp16_v2.cu:41-52,110-208
 *   orc_forward ............... src/rwkv7_fast_v4.cu:1046-1345
 * The W8A16 / W4A16 functions have no counterpart in the reference (it has no
 * quantisation); they are the written definition of those formats for this project
 * (parity unpinned for them).
 *
 * Pinned: every function above is checked on the CPU against outputs recorded from the
 * reference's own kernels and from its whole ModelBackend (ref_ops.npz and
 * ref_model_tiny.npz under tests/golden, made by make_golden.py there; checked by
 * tests/test_golden_cpu.py).
 *
 * Where the reference sums in an unspecified parallel order in fp32 (dot products,
 * LayerNorm statistics) the oracle sums in double: the result is the correctly rounded
 * value every fp32 summation order approximates.  Where the reference's order and
 * rounding are part of the result (the fp16-state WKV) they are reproduced exactly.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "softfp16.h"

#define HS 64 /* head size, fixed by the reference (include/rwkv7_fast_v4_common.hpp:286) */

typedef sh_t h16;

static inline float hf(h16 x) { return sh_to_f(x); }
static inline h16 fh(float x) { return sh_from_f(x); }

h16 orc_f2h(float x) { return fh(x); }
float orc_h2f(h16 x) { return hf(x); }
h16 orc_hfma(h16 a, h16 b, h16 c) { return sh_fma(a, b, c); }
h16 orc_hadd(h16 a, h16 b) { return sh_add(a, b); }

static inline float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

/* ------------------------------------------------------------------ LayerNorm family */

static void ln_stats(const float* v, int C, float eps, float* mean_out, float* rstd_out) {
  double sum = 0.0;
  for (int c = 0; c < C; ++c) sum += v[c];
  const float mean = (float)(sum / C);
  double sv = 0.0;
  for (int c = 0; c < C; ++c) {
    const float d = v[c] - mean;
    sv += (double)d * d;
  }
  *mean_out = mean;
  *rstd_out = 1.0f / sqrtf((float)(sv / C) + eps);
}

void orc_layer_norm(int rows, int C, const h16* x, const h16* w, const h16* b, h16* y, float eps) {
  float* v = (float*)malloc(sizeof(float) * C);
  for (int r = 0; r < rows; ++r) {
    for (int c = 0; c < C; ++c) v[c] = hf(x[(size_t)r * C + c]);
    float mean, rstd;
    ln_stats(v, C, eps, &mean, &rstd);
    for (int c = 0; c < C; ++c) y[(size_t)r * C + c] = fh((v[c] - mean) * rstd * hf(w[c]) + hf(b[c]));
  }
  free(v);
}

/* x_out = half(x + residual); y = half(LN(x + residual)) with statistics of the unrounded sum. */
void orc_add_layer_norm(int rows, int C, const h16* x, const h16* res, const h16* w, const h16* b,
                        h16* x_out, h16* y, float eps) {
  float* v = (float*)malloc(sizeof(float) * C);
  for (int r = 0; r < rows; ++r) {
    for (int c = 0; c < C; ++c) v[c] = hf(x[(size_t)r * C + c]) + hf(res[(size_t)r * C + c]);
    float mean, rstd;
    ln_stats(v, C, eps, &mean, &rstd);
    for (int c = 0; c < C; ++c) {
      if (x_out) x_out[(size_t)r * C + c] = fh(v[c]);
      y[(size_t)r * C + c] = fh((v[c] - mean) * rstd * hf(w[c]) + hf(b[c]));
    }
  }
  free(v);
}

/* y[b] = half(LN(x[b,T-1] + residual[b,T-1])) */
void orc_add_last_layer_norm(int B, int T, int C, const h16* x, const h16* res, const h16* w,
                             const h16* b, h16* y, float eps) {
  for (int bi = 0; bi < B; ++bi) {
    const size_t src = ((size_t)bi * T + (T - 1)) * C;
    orc_add_layer_norm(1, C, x + src, res + src, w, b, NULL, y + (size_t)bi * C, eps);
  }
}

/* Embedding table with LN0 folded in, computed in fp32 from the checkpoint values. */
void orc_emb_ln0(int V, int C, const float* emb, const float* w, const float* b, h16* out, float eps) {
  for (int t = 0; t < V; ++t) {
    float mean, rstd;
    ln_stats(emb + (size_t)t * C, C, eps, &mean, &rstd);
    for (int c = 0; c < C; ++c)
      out[(size_t)t * C + c] = fh((emb[(size_t)t * C + c] - mean) * rstd * w[c] + b[c]);
  }
}

/* ------------------------------------------------------------------ token shift */

void orc_tmix_mix6(int B, int T, int C, const h16* x, h16* shift, const h16* const mix[6], h16* const out[6]) {
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int c = 0; c < C; ++c) {
        const size_t idx = ((size_t)b * T + t) * C + c;
        const float cur = hf(x[idx]);
        const float prev = hf(t == 0 ? shift[(size_t)b * C + c] : x[idx - C]);
        const float dx = prev - cur;
        for (int m = 0; m < 6; ++m) out[m][idx] = fh(cur + dx * hf(mix[m][c]));
      }
  for (int b = 0; b < B; ++b)
    memcpy(shift + (size_t)b * C, x + ((size_t)b * T + (T - 1)) * C, sizeof(h16) * C);
}

void orc_cmix_mix(int B, int T, int C, const h16* x, h16* shift, const h16* x_k, h16* out) {
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int c = 0; c < C; ++c) {
        const size_t idx = ((size_t)b * T + t) * C + c;
        const float cur = hf(x[idx]);
        const float prev = hf(t == 0 ? shift[(size_t)b * C + c] : x[idx - C]);
        out[idx] = fh(cur + (prev - cur) * hf(x_k[c]));
      }
  for (int b = 0; b < B; ++b)
    memcpy(shift + (size_t)b * C, x + ((size_t)b * T + (T - 1)) * C, sizeof(h16) * C);
}

/* ------------------------------------------------------------------ per-head gates */

void orc_kk_a_gate(int rows, int C, const h16* k, const h16* k_k, const h16* a0, const h16* a12,
                   const h16* k_a, h16* new_k, h16* neg_kk, h16* kka) {
  const int H = C / HS;
  for (int r = 0; r < rows; ++r)
    for (int h = 0; h < H; ++h) {
      const size_t base = (size_t)r * C + (size_t)h * HS;
      float u[HS];
      double ss = 0.0;
      for (int j = 0; j < HS; ++j) {
        u[j] = hf(k[base + j]) * hf(k_k[h * HS + j]);
        ss += (double)u[j] * u[j];
      }
      const float inv = 1.0f / fmaxf(sqrtf((float)ss), 1.0e-12f);
      for (int j = 0; j < HS; ++j) {
        const int c = h * HS + j;
        const float kk = u[j] * inv;
        const float av = sigmoidf_(hf(a0[c]) + hf(a12[base + j]));
        const float ka = hf(k_a[c]);
        new_k[base + j] = fh(hf(k[base + j]) * fmaf(av, ka, 1.0f - ka));
        neg_kk[base + j] = fh(-kk);
        kka[base + j] = fh(kk * av);
      }
    }
}

void orc_vres_gate(int rows, int C, const h16* v, const h16* v_first, const h16* v0, const h16* v12, h16* out) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < C; ++c) {
      const size_t i = (size_t)r * C + c;
      const float vv = hf(v[i]);
      const float gate = sigmoidf_(hf(v0[c]) + hf(v12[i]));
      out[i] = fh(fmaf(hf(v_first[i]) - vv, gate, vv));
    }
}

/* GroupNorm over each head (eps 64e-5) * w + b, plus (sum_j r k r_k) v, times g. */
void orc_lnx_rkvres_xg(int rows, int C, const h16* y, const h16* r, const h16* k, const h16* v,
                       const h16* r_k, const h16* w, const h16* b, const h16* g, h16* out) {
  const int H = C / HS;
  for (int row = 0; row < rows; ++row)
    for (int h = 0; h < H; ++h) {
      const size_t base = (size_t)row * C + (size_t)h * HS;
      double s = 0.0;
      for (int j = 0; j < HS; ++j) s += hf(y[base + j]);
      const float mean = (float)(s * (1.0 / 64.0));
      double sv = 0.0, dot = 0.0;
      for (int j = 0; j < HS; ++j) {
        const float d = hf(y[base + j]) - mean;
        sv += (double)d * d;
        dot += (double)(hf(r[base + j]) * hf(k[base + j]) * hf(r_k[h * HS + j]));
      }
      const float rstd = 1.0f / sqrtf((float)(sv * (1.0 / 64.0)) + 64.0e-5f);
      const float rkv = (float)dot;
      for (int j = 0; j < HS; ++j) {
        const int c = h * HS + j;
        const float d = hf(y[base + j]) - mean;
        out[base + j] = fh((d * rstd * hf(w[c]) + hf(b[c]) + rkv * hf(v[base + j])) * hf(g[base + j]));
      }
    }
}

/* ------------------------------------------------------------------ linear layers */

/* in_act / epilogue codes shared with the CUDA library */
enum { ACT_NONE = 0, ACT_TANH = 1, ACT_SIGMOID = 2 };
enum { EPI_NONE = 0, EPI_RELU2 = 1 };

static inline float apply_in_act(float x, int act) {
  if (act == ACT_TANH) return tanhf(x);
  if (act == ACT_SIGMOID) return sigmoidf_(x);
  return x;
}

/* y[m,n] = half(sum_k act(x[m,k]) * W[n,k]); W in the checkpoint's [out,in] orientation. */
void orc_linear_orig(int M, int K, int N, const h16* x, const h16* W, h16* y, int in_act, int epi) {
  float* xa = (float*)malloc(sizeof(float) * (size_t)M * K);
  for (size_t i = 0; i < (size_t)M * K; ++i) xa[i] = apply_in_act(hf(x[i]), in_act);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const h16* wr = W + (size_t)n * K;
    for (int m = 0; m < M; ++m) {
      const float* xr = xa + (size_t)m * K;
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)(xr[k] * hf(wr[k]));
      h16 o = fh((float)acc);
      if (epi == EPI_RELU2) {
        const float t = fmaxf(hf(o), 0.0f);
        o = fh(t * t);
      }
      y[(size_t)m * N + n] = o;
    }
  }
  free(xa);
}

/* y[m,n] = half(sum_k act(x[m,k]) * W[k,n]); W stored [K,N] (LoRA matrices as in the
 * checkpoint, and the transposed ffn.value the reference keeps on the device). */
void orc_linear_kn(int M, int K, int N, const h16* x, const h16* W, h16* y, int in_act) {
  double* acc = (double*)malloc(sizeof(double) * N);
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) acc[n] = 0.0;
    for (int k = 0; k < K; ++k) {
      const float xv = apply_in_act(hf(x[(size_t)m * K + k]), in_act);
      if (xv == 0.0f) continue;
      const h16* wr = W + (size_t)k * N;
      for (int n = 0; n < N; ++n) acc[n] += (double)(xv * hf(wr[n]));
    }
    for (int n = 0; n < N; ++n) y[(size_t)m * N + n] = fh((float)acc[n]);
  }
  free(acc);
}

/* ------------------------------------------------------------------ quantised formats
 * W8A16: per-output-channel symmetric int8.  scale[n] = half(max_k|W[n,k]| / 127),
 *        q = clamp(rint(W / float(scale)), -127, 127), stored row-major int8 [N,K].
 *        y[m,n] = half(float(scale[n]) * sum_k x[m,k] * q[n,k]).
 * W4A16: groups of 128 along K, asymmetric, range widened to contain 0.
 *        scale = half((max - min) / 15), zero = clamp(rint(-min / float(scale)), 0, 15) kept
 *        as an integer-valued half, q = clamp(rint(W / float(scale)) + zero, 0, 15);
 *        byte j of a row holds q[2j] in the low nibble and q[2j+1] in the high nibble.
 *        Dequantised weight = half((q - zero) * float(scale)); y is then the ordinary
 *        fp16 linear layer on those weights.
 */

void orc_quant_pack_w8(int N, int K, const h16* W, int8_t* q, h16* scale) {
  for (int n = 0; n < N; ++n) {
    float amax = 0.0f;
    for (int k = 0; k < K; ++k) amax = fmaxf(amax, fabsf(hf(W[(size_t)n * K + k])));
    const h16 s = fh(amax / 127.0f);
    scale[n] = s;
    const float sf = hf(s);
    for (int k = 0; k < K; ++k) {
      float v = sf > 0.0f ? rintf(hf(W[(size_t)n * K + k]) / sf) : 0.0f;
      v = fminf(fmaxf(v, -127.0f), 127.0f);
      q[(size_t)n * K + k] = (int8_t)v;
    }
  }
}

void orc_quant_unpack_w8(int N, int K, const int8_t* q, const h16* scale, h16* W) {
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) W[(size_t)n * K + k] = fh((float)q[(size_t)n * K + k] * hf(scale[n]));
}

void orc_quant_pack_w4(int N, int K, const h16* W, uint8_t* q, h16* scale, h16* zero) {
  const int G = K / 128;
  for (int n = 0; n < N; ++n)
    for (int g = 0; g < G; ++g) {
      const h16* w = W + (size_t)n * K + (size_t)g * 128;
      float mn = 0.0f, mx = 0.0f;
      for (int k = 0; k < 128; ++k) {
        mn = fminf(mn, hf(w[k]));
        mx = fmaxf(mx, hf(w[k]));
      }
      const h16 s = fh((mx - mn) / 15.0f);
      const float sf = hf(s);
      float z = sf > 0.0f ? rintf(-mn / sf) : 0.0f;
      z = fminf(fmaxf(z, 0.0f), 15.0f);
      scale[(size_t)n * G + g] = s;
      zero[(size_t)n * G + g] = fh(z);
      uint8_t* qb = q + ((size_t)n * K + (size_t)g * 128) / 2;
      for (int k = 0; k < 128; k += 2) {
        uint8_t nib[2];
        for (int u = 0; u < 2; ++u) {
          float v = sf > 0.0f ? rintf(hf(w[k + u]) / sf) + z : 0.0f;
          v = fminf(fmaxf(v, 0.0f), 15.0f);
          nib[u] = (uint8_t)v;
        }
        qb[k / 2] = (uint8_t)(nib[0] | (nib[1] << 4));
      }
    }
}

void orc_quant_unpack_w4(int N, int K, const uint8_t* q, const h16* scale, const h16* zero, h16* W) {
  const int G = K / 128;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const size_t gi = (size_t)n * G + k / 128;
      const uint8_t byte = q[((size_t)n * K + k) / 2];
      const int qq = (k & 1) ? (byte >> 4) : (byte & 15);
      W[(size_t)n * K + k] = fh(((float)qq - hf(zero[gi])) * hf(scale[gi]));
    }
}

void orc_linear_w8a16(int M, int K, int N, const h16* x, const int8_t* q, const h16* scale, h16* y, int epi) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int m = 0; m < M; ++m) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)(hf(x[(size_t)m * K + k]) * (float)q[(size_t)n * K + k]);
      h16 o = fh((float)acc * hf(scale[n]));
      if (epi == EPI_RELU2) {
        const float t = fmaxf(hf(o), 0.0f);
        o = fh(t * t);
      }
      y[(size_t)m * N + n] = o;
    }
}

void orc_linear_w4a16(int M, int K, int N, const h16* x, const uint8_t* q, const h16* scale,
                      const h16* zero, h16* y, int epi) {
  h16* W = (h16*)malloc(sizeof(h16) * (size_t)N * K);
  orc_quant_unpack_w4(N, K, q, scale, zero, W);
  orc_linear_orig(M, K, N, x, W, y, ACT_NONE, epi);
  free(W);
}

/* ------------------------------------------------------------------ WKV-7 recurrence */

static inline float w_eff(float w) {
  /* exp(-exp(-0.5) * sigmoid(w)) written as the reference writes it */
  return exp2f(-0.8750387749145276f / (1.0f + exp2f(-1.4426950408889634f * w)));
}

/* fp32 state, fp16 in/out.  state [B,H,64(i: value),64(j: key)], tensors [B,T,C].
 * w is the raw decay pre-activation (w0 already added and rounded by the caller). */
void orc_wkv_fp32(int B, int T, int C, int H, float* state, const h16* r, const h16* w, const h16* k,
                  const h16* v, const h16* a, const h16* b, h16* y) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bi = 0; bi < B; ++bi)
    for (int h = 0; h < H; ++h) {
      float* S = state + ((size_t)bi * H + h) * HS * HS;
      for (int t = 0; t < T; ++t) {
        const size_t tok = ((size_t)bi * T + t) * C + (size_t)h * HS;
        float rr[HS], ww[HS], kk[HS], aa[HS], bb[HS];
        for (int j = 0; j < HS; ++j) {
          rr[j] = hf(r[tok + j]);
          ww[j] = w_eff(hf(w[tok + j]));
          kk[j] = hf(k[tok + j]);
          aa[j] = hf(a[tok + j]);
          bb[j] = hf(b[tok + j]);
        }
        for (int i = 0; i < HS; ++i) {
          float* s = S + (size_t)i * HS;
          float sa = 0.0f;
          for (int j = 0; j < HS; ++j) sa += s[j] * aa[j];
          const float vi = hf(v[tok + i]);
          float yy = 0.0f;
          for (int j = 0; j < HS; ++j) {
            const float sn = s[j] * ww[j] + sa * bb[j] + kk[j] * vi;
            yy += sn * rr[j];
            s[j] = sn;
          }
          y[tok + i] = fh(yy);
        }
      }
    }
}

/* fp16 state.  Every state operation is a half fused multiply-add, the two lane sums run
 * over even and odd key indices separately (the .x and .y lanes of a half2) and are joined
 * by one half add.  The decay is d = half(w_eff - 1 + dither) so that S*d + S == S*w_eff up
 * to the dither; dither = 2^-41 * float(int32(0x9E3779B9 * phase)) with 32-bit wrap-around,
 * phase = elapsed[b] + 64 h + j + t.  w0 may be NULL (then w already contains it). */
void orc_wkv_fp16(int B, int T, int C, int H, h16* state, const h16* r, const h16* w, const h16* w0,
                  const h16* k, const h16* v, const h16* a, const h16* b, h16* y, const int* elapsed) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int bi = 0; bi < B; ++bi)
    for (int h = 0; h < H; ++h) {
      h16* S = state + ((size_t)bi * H + h) * HS * HS;
      for (int t = 0; t < T; ++t) {
        const size_t tok = ((size_t)bi * T + t) * C + (size_t)h * HS;
        h16 d[HS];
        for (int j = 0; j < HS; ++j) {
          float wf = hf(w[tok + j]);
          if (w0) wf += hf(w0[h * HS + j]);
          const uint32_t phase = (uint32_t)(elapsed[bi] + h * HS + j + t);
          const int32_t rot = (int32_t)(2654435769u * phase);
          const float dd = exp2f(-0.8750387749145276f / (1.0f + exp2f(-1.4426950408889634f * wf))) - 1.0f +
                           4.547473508864641e-13f * (float)rot;
          d[j] = fh(dd);
        }
        for (int i = 0; i < HS; ++i) {
          h16* s = S + (size_t)i * HS;
          h16 sa0 = 0, sa1 = 0;
          for (int j = 0; j < HS; j += 2) {
            sa0 = sh_fma(a[tok + j], s[j], sa0);
            sa1 = sh_fma(a[tok + j + 1], s[j + 1], sa1);
          }
          const h16 sa = sh_add(sa0, sa1);
          const h16 vi = v[tok + i];
          h16 y0 = 0, y1 = 0;
          for (int j = 0; j < HS; j += 2) {
            h16 s0 = sh_fma(s[j], d[j], sh_fma(k[tok + j], vi, sh_fma(sa, b[tok + j], s[j])));
            h16 s1 = sh_fma(s[j + 1], d[j + 1], sh_fma(k[tok + j + 1], vi, sh_fma(sa, b[tok + j + 1], s[j + 1])));
            s[j] = s0;
            s[j + 1] = s1;
            y0 = sh_fma(s0, r[tok + j], y0);
            y1 = sh_fma(s1, r[tok + j + 1], y1);
          }
          y[tok + i] = sh_add(y0, y1);
        }
      }
    }
}

/* ------------------------------------------------------------------ whole model */

enum { FMT_F16 = 0, FMT_W8A16 = 1, FMT_W4A16 = 2 };

typedef struct {
  int rows, cols;       /* [N,K] */
  int fmt;
  h16* w;               /* FMT_F16 */
  int8_t* q8;           /* FMT_W8A16 */
  uint8_t* q4;          /* FMT_W4A16 */
  h16 *scale, *zero;
} orc_matrix;

typedef struct {
  h16 *ln1_w, *ln1_b, *ln2_w, *ln2_b;
  h16 *x_r, *x_w, *x_k, *x_v, *x_a, *x_g;
  orc_matrix Wr, Wk, Wv, Wo;
  h16 *w0, *w1, *w2, *a0, *a1, *a2, *g1, *g2, *v0, *v1, *v2; /* LoRA as stored: w1 [C,R], w2 [R,C] */
  h16 *k_k, *k_a, *r_k, *lnx_w, *lnx_b;
  h16* ffn_x_k;
  orc_matrix Wkey;  /* [F,C] */
  orc_matrix Wval;  /* [C,F] as in the checkpoint */
} orc_layer;

typedef struct {
  int L, C, H, F, V, Rw, Ra, Rv, Rg;
  int fmt;
  h16* emb_ln0; /* [V,C] */
  h16 *ln_out_w, *ln_out_b;
  orc_matrix head; /* [V,C] */
  orc_layer* layers;
} orc_model;

orc_model* orc_model_create(int L, int C, int F, int V, int Rw, int Ra, int Rv, int Rg, int fmt) {
  orc_model* m = (orc_model*)calloc(1, sizeof(orc_model));
  m->L = L; m->C = C; m->H = C / HS; m->F = F; m->V = V;
  m->Rw = Rw; m->Ra = Ra; m->Rv = Rv; m->Rg = Rg; m->fmt = fmt;
  m->layers = (orc_layer*)calloc((size_t)L, sizeof(orc_layer));
  return m;
}

static h16* dup16(const h16* src, size_t n) {
  h16* p = (h16*)malloc(sizeof(h16) * n);
  memcpy(p, src, sizeof(h16) * n);
  return p;
}

static void set_matrix(orc_matrix* mat, const h16* w, int N, int K, int fmt) {
  mat->rows = N; mat->cols = K; mat->fmt = fmt;
  if (fmt == FMT_F16) {
    mat->w = dup16(w, (size_t)N * K);
  } else if (fmt == FMT_W8A16) {
    mat->q8 = (int8_t*)malloc((size_t)N * K);
    mat->scale = (h16*)malloc(sizeof(h16) * N);
    orc_quant_pack_w8(N, K, w, mat->q8, mat->scale);
  } else {
    mat->q4 = (uint8_t*)malloc((size_t)N * K / 2);
    mat->scale = (h16*)malloc(sizeof(h16) * (size_t)N * (K / 128));
    mat->zero = (h16*)malloc(sizeof(h16) * (size_t)N * (K / 128));
    orc_quant_pack_w4(N, K, w, mat->q4, mat->scale, mat->zero);
  }
}

/* Tensors are addressed by their checkpoint names (src/rwkv7_fast_v4.cu:574-596); data are
 * fp16 bits, i.e. half_rn(float(bf16)) of the checkpoint values (cuda/rwkv7_v3a_ops.cu:70-88).
 * "emb_ln0" is the [V,C] table produced by orc_emb_ln0.  Returns 0 if the name is unknown. */
int orc_model_set(orc_model* m, const char* name, const h16* data, long long n) {
  const int C = m->C, F = m->F, V = m->V;
  if (!strcmp(name, "emb_ln0")) { m->emb_ln0 = dup16(data, n); return n == (long long)V * C; }
  if (!strcmp(name, "ln_out.weight")) { m->ln_out_w = dup16(data, n); return n == C; }
  if (!strcmp(name, "ln_out.bias")) { m->ln_out_b = dup16(data, n); return n == C; }
  if (!strcmp(name, "head.weight")) { set_matrix(&m->head, data, V, C, m->fmt); return n == (long long)V * C; }
  int layer = -1, off = 0;
  if (sscanf(name, "blocks.%d.%n", &layer, &off) < 1 || layer < 0 || layer >= m->L) return 0;
  const char* s = name + off;
  orc_layer* l = &m->layers[layer];
#define VEC(key, field) if (!strcmp(s, key)) { l->field = dup16(data, n); return 1; }
  VEC("ln1.weight", ln1_w) VEC("ln1.bias", ln1_b) VEC("ln2.weight", ln2_w) VEC("ln2.bias", ln2_b)
  VEC("att.x_r", x_r) VEC("att.x_w", x_w) VEC("att.x_k", x_k) VEC("att.x_v", x_v) VEC("att.x_a", x_a) VEC("att.x_g", x_g)
  VEC("att.w0", w0) VEC("att.w1", w1) VEC("att.w2", w2) VEC("att.a0", a0) VEC("att.a1", a1) VEC("att.a2", a2)
  VEC("att.g1", g1) VEC("att.g2", g2) VEC("att.v0", v0) VEC("att.v1", v1) VEC("att.v2", v2)
  VEC("att.k_k", k_k) VEC("att.k_a", k_a) VEC("att.r_k", r_k) VEC("att.ln_x.weight", lnx_w) VEC("att.ln_x.bias", lnx_b)
  VEC("ffn.x_k", ffn_x_k)
#undef VEC
  if (!strcmp(s, "att.receptance.weight")) { set_matrix(&l->Wr, data, C, C, m->fmt); return 1; }
  if (!strcmp(s, "att.key.weight")) { set_matrix(&l->Wk, data, C, C, m->fmt); return 1; }
  if (!strcmp(s, "att.value.weight")) { set_matrix(&l->Wv, data, C, C, m->fmt); return 1; }
  if (!strcmp(s, "att.output.weight")) { set_matrix(&l->Wo, data, C, C, m->fmt); return 1; }
  if (!strcmp(s, "ffn.key.weight")) { set_matrix(&l->Wkey, data, F, C, m->fmt); return 1; }
  if (!strcmp(s, "ffn.value.weight")) { set_matrix(&l->Wval, data, C, F, m->fmt); return 1; }
  if (!strcmp(s, "ln0.weight") || !strcmp(s, "ln0.bias")) return 1; /* folded into emb_ln0 */
  return 0;
}

static void free_matrix(orc_matrix* a) { free(a->w); free(a->q8); free(a->q4); free(a->scale); free(a->zero); }

void orc_model_destroy(orc_model* m) {
  if (!m) return;
  for (int i = 0; i < m->L; ++i) {
    orc_layer* l = &m->layers[i];
    h16* vecs[] = {l->ln1_w, l->ln1_b, l->ln2_w, l->ln2_b, l->x_r, l->x_w, l->x_k, l->x_v, l->x_a, l->x_g,
                   l->w0, l->w1, l->w2, l->a0, l->a1, l->a2, l->g1, l->g2, l->v0, l->v1, l->v2,
                   l->k_k, l->k_a, l->r_k, l->lnx_w, l->lnx_b, l->ffn_x_k};
    for (size_t j = 0; j < sizeof(vecs) / sizeof(vecs[0]); ++j) free(vecs[j]);
    free_matrix(&l->Wr); free_matrix(&l->Wk); free_matrix(&l->Wv); free_matrix(&l->Wo);
    free_matrix(&l->Wkey); free_matrix(&l->Wval);
  }
  free(m->layers); free(m->emb_ln0); free(m->ln_out_w); free(m->ln_out_b); free_matrix(&m->head);
  free(m);
}

static void linear_any(int M, const orc_matrix* W, const h16* x, h16* y, int epi) {
  if (W->fmt == FMT_F16) orc_linear_orig(M, W->cols, W->rows, x, W->w, y, ACT_NONE, epi);
  else if (W->fmt == FMT_W8A16) orc_linear_w8a16(M, W->cols, W->rows, x, W->q8, W->scale, y, epi);
  else orc_linear_w4a16(M, W->cols, W->rows, x, W->q4, W->scale, W->zero, y, epi);
}

/* Forward of tokens[B][T] (row-major), updating the recurrent state in place and writing
 * fp32 logits [B,V] of the last token of every sequence.  State layouts are the reference's
 * (src/rwkv7_fast_v4.cu:1177-1185): shift half [L][2][B][C], wkv [L][B][H][64][64] (half or
 * float), elapsed int [B].
 * lora_round_act = 0 reproduces the reference's fused LoRA path (rows<=4 and C>=1024:
 * tanh/sigmoid of the rank-R intermediate and the v LoRA output stay in fp32);
 * lora_round_act = 1 reproduces its unfused path (those are rounded to fp16 first).
 * Returns 0 on success, -1 on a bad token id. */
int orc_forward(const orc_model* m, const long long* tokens, int B, int T, int wkv32, int lora_round_act,
                h16* shift, void* wkv, int* elapsed, float* logits) {
  const int C = m->C, H = m->H, F = m->F, V = m->V, L = m->L;
  const int rows = B * T;
  const size_t RC = (size_t)rows * C;
  const float eps = 1e-5f;
  for (int i = 0; i < rows; ++i)
    if (tokens[i] < 0 || tokens[i] >= V) return -1;

  h16* buf = (h16*)malloc(sizeof(h16) * (RC * 24 + (size_t)rows * F * 2 + (size_t)rows * 2048 + (size_t)B * C));
  h16* p = buf;
#define TAKE(name, n) h16* name = p; p += (n);
  TAKE(x, RC) TAKE(xx, RC) TAKE(xr, RC) TAKE(xw, RC) TAKE(xk, RC) TAKE(xv, RC) TAKE(xa, RC) TAKE(xg, RC)
  TAKE(r, RC) TAKE(k, RC) TAKE(v, RC) TAKE(vfirst, RC) TAKE(w12, RC) TAKE(a12, RC) TAKE(g, RC) TAKE(tmp, RC)
  TAKE(k2, RC) TAKE(nkk, RC) TAKE(kka, RC) TAKE(win, RC) TAKE(y, RC) TAKE(y2, RC) TAKE(att, RC) TAKE(n2, RC)
  TAKE(hid, (size_t)rows * F) TAKE(act, (size_t)rows * F)
  TAKE(w1, (size_t)rows * 512) TAKE(a1, (size_t)rows * 512) TAKE(g1, (size_t)rows * 512) TAKE(v1, (size_t)rows * 512)
  TAKE(xf, (size_t)B * C)
#undef TAKE
  h16* mixed = xr; /* reuse after the time-mix block */
  h16* ffn = xw;

  for (int i = 0; i < rows; ++i) memcpy(x + (size_t)i * C, m->emb_ln0 + (size_t)tokens[i] * C, sizeof(h16) * C);
  orc_layer_norm(rows, C, x, m->layers[0].ln1_w, m->layers[0].ln1_b, xx, eps);

  for (int li = 0; li < L; ++li) {
    const orc_layer* l = &m->layers[li];
    h16* shift0 = shift + (size_t)li * 2 * B * C;
    h16* shift1 = shift0 + (size_t)B * C;
    const h16* mix[6] = {l->x_r, l->x_w, l->x_k, l->x_v, l->x_a, l->x_g};
    h16* outs[6] = {xr, xw, xk, xv, xa, xg};
    orc_tmix_mix6(B, T, C, xx, shift0, mix, outs);

    linear_any(rows, &l->Wr, xr, r, EPI_NONE);
    linear_any(rows, &l->Wk, xk, k, EPI_NONE);
    linear_any(rows, &l->Wv, xv, v, EPI_NONE);

    orc_linear_kn(rows, C, m->Rw, xw, l->w1, w1, ACT_NONE);
    orc_linear_kn(rows, C, m->Ra, xa, l->a1, a1, ACT_NONE);
    orc_linear_kn(rows, C, m->Rg, xg, l->g1, g1, ACT_NONE);
    if (lora_round_act) {
      for (size_t i = 0; i < (size_t)rows * m->Rw; ++i) w1[i] = fh(tanhf(hf(w1[i])));
      for (size_t i = 0; i < (size_t)rows * m->Rg; ++i) g1[i] = fh(sigmoidf_(hf(g1[i])));
      orc_linear_kn(rows, m->Rw, C, w1, l->w2, w12, ACT_NONE);
      orc_linear_kn(rows, m->Rg, C, g1, l->g2, g, ACT_NONE);
    } else {
      orc_linear_kn(rows, m->Rw, C, w1, l->w2, w12, ACT_TANH);
      orc_linear_kn(rows, m->Rg, C, g1, l->g2, g, ACT_SIGMOID);
    }
    orc_linear_kn(rows, m->Ra, C, a1, l->a2, a12, ACT_NONE);

    const h16* v_use = v;
    if (li == 0) {
      memcpy(vfirst, v, sizeof(h16) * RC);
    } else {
      orc_linear_kn(rows, C, m->Rv, xv, l->v1, v1, ACT_NONE);
      if (lora_round_act) {
        orc_linear_kn(rows, m->Rv, C, v1, l->v2, tmp, ACT_NONE);
        orc_vres_gate(rows, C, v, vfirst, l->v0, tmp, tmp);
      } else {
        /* gate from the unrounded LoRA output */
        for (int rr = 0; rr < rows; ++rr)
          for (int c = 0; c < C; ++c) {
            double acc = 0.0;
            for (int q = 0; q < m->Rv; ++q) acc += (double)(hf(v1[(size_t)rr * m->Rv + q]) * hf(l->v2[(size_t)q * C + c]));
            const size_t i = (size_t)rr * C + c;
            const float vv = hf(v[i]);
            const float gate = sigmoidf_(hf(l->v0[c]) + (float)acc);
            tmp[i] = fh(vv + (hf(vfirst[i]) - vv) * gate);
          }
      }
      v_use = tmp;
    }

    orc_kk_a_gate(rows, C, k, l->k_k, l->a0, a12, l->k_a, k2, nkk, kka);

    if (wkv32) {
      for (size_t i = 0; i < RC; ++i) win[i] = fh(hf(w12[i]) + hf(l->w0[i % C]));
      orc_wkv_fp32(B, T, C, H, (float*)wkv + (size_t)li * B * H * HS * HS, r, win, k2, v_use, nkk, kka, y);
    } else if (T <= 16) {
      orc_wkv_fp16(B, T, C, H, (h16*)wkv + (size_t)li * B * H * HS * HS, r, w12, l->w0, k2, v_use, nkk, kka, y, elapsed);
    } else {
      for (size_t i = 0; i < RC; ++i) win[i] = fh(hf(w12[i]) + hf(l->w0[i % C]));
      orc_wkv_fp16(B, T, C, H, (h16*)wkv + (size_t)li * B * H * HS * HS, r, win, NULL, k2, v_use, nkk, kka, y, elapsed);
    }

    orc_lnx_rkvres_xg(rows, C, y, r, k2, v_use, l->r_k, l->lnx_w, l->lnx_b, g, y2);
    linear_any(rows, &l->Wo, y2, att, EPI_NONE);
    /* x <- x + att ; n2 = LN2(x + att) ; channel-mix token shift */
    orc_add_layer_norm(rows, C, x, att, l->ln2_w, l->ln2_b, x, n2, eps);
    orc_cmix_mix(B, T, C, n2, shift1, l->ffn_x_k, mixed);
    linear_any(rows, &l->Wkey, mixed, hid, EPI_RELU2);
    memcpy(act, hid, sizeof(h16) * (size_t)rows * F);
    linear_any(rows, &l->Wval, act, ffn, EPI_NONE);
    if (li + 1 < L) {
      orc_add_layer_norm(rows, C, x, ffn, m->layers[li + 1].ln1_w, m->layers[li + 1].ln1_b, x, xx, eps);
    } else {
      orc_add_last_layer_norm(B, T, C, x, ffn, m->ln_out_w, m->ln_out_b, xf, eps);
    }
  }
  for (int b = 0; b < B; ++b) elapsed[b] += T;

  h16* lg = (h16*)malloc(sizeof(h16) * (size_t)B * V);
  linear_any(B, &m->head, xf, lg, EPI_NONE);
  for (size_t i = 0; i < (size_t)B * V; ++i) logits[i] = hf(lg[i]);
  free(lg);
  free(buf);
  return 0;
}
