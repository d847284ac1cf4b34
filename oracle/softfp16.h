/*
 * Software IEEE binary16 for the CPU oracle (test infrastructure, not product code).
 *
 * The reference's fp16-state WKV kernel (cuda/rwkv7_wkv_fp16_v2.cu:150-190) does every
 * state operation as a half2 fused multiply-add and every lane reduction as a half add.
 * Those are single-rounding operations; this header reproduces them exactly on a CPU:
 *   sh_fma(a,b,c) = RNE_half(a*b + c)   one rounding, subnormals kept
 *   sh_add(a,b)   = RNE_half(a + b)
 * The product of two halves is exact in a double; the sum with the addend may need more
 * than 53 bits, so the double sum is corrected to round-to-odd with the TwoSum error term
 * before the final rounding to 11 significant bits (double rounding is then harmless).
 */
#ifndef ORACLE_SOFTFP16_H
#define ORACLE_SOFTFP16_H

#include <math.h>
#include <stdint.h>
#include <string.h>

typedef uint16_t sh_t; /* raw binary16 bits */

static inline float sh_to_f(sh_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  const uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      /* subnormal: value = man * 2^-24, exact in float */
      float f = (float)man * 5.9604644775390625e-8f;
      memcpy(&bits, &f, 4);
      bits |= sign;
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float out;
  memcpy(&out, &bits, 4);
  return out;
}

/* Round a double to binary16, round-to-nearest-even (the rounding of __float2half_rn,
 * __hfma, __hadd). */
static inline sh_t sh_from_d(double x) {
  uint64_t xb;
  memcpy(&xb, &x, 8);
  const sh_t sign = (sh_t)((xb >> 48) & 0x8000u);
  if (x != x) return (sh_t)(sign | 0x7fffu); /* canonical NaN like the GPU */
  double ax = fabs(x);
  if (ax >= 65520.0) return (sh_t)(sign | 0x7c00u); /* overflow to inf (65520 = max + ulp/2) */
  if (ax < 6.103515625e-05) {                       /* below 2^-14: subnormal grid 2^-24 */
    double q = rint(ax * 16777216.0);               /* RNE in the default rounding mode */
    return (sh_t)(sign | (uint16_t)q);              /* 1024 encodes the smallest normal */
  }
  int e = ilogb(ax);                                /* 2^e <= ax < 2^(e+1) */
  double q = rint(scalbn(ax, 10 - e));              /* in [1024, 2048] */
  if (q >= 2048.0) {
    q = 1024.0;
    e += 1;
  }
  if (e > 15) return (sh_t)(sign | 0x7c00u);
  return (sh_t)(sign | (uint16_t)((e + 15) << 10) | ((uint16_t)q - 1024u));
}

static inline sh_t sh_from_f(float f) { return sh_from_d((double)f); }

static inline sh_t sh_add(sh_t a, sh_t b) {
  /* two halves span < 53 bits together, the double sum is exact */
  return sh_from_d((double)sh_to_f(a) + (double)sh_to_f(b));
}

static inline sh_t sh_fma(sh_t a, sh_t b, sh_t c) {
  const double p = (double)sh_to_f(a) * (double)sh_to_f(b); /* exact: 22 significant bits */
  const double cc = (double)sh_to_f(c);
  double s = p + cc;
  const double bb = s - p;
  const double err = (p - (s - bb)) + (cc - bb); /* TwoSum: s + err == p + cc exactly */
  if (err != 0.0 && s == s && fabs(s) < 1e300) {
    uint64_t sb;
    memcpy(&sb, &s, 8);
    const int same_dir = (err > 0.0) == (s > 0.0);
    if (!same_dir) sb -= 1; /* truncate toward zero */
    sb |= 1;                /* sticky bit: round to odd */
    memcpy(&s, &sb, 8);
  }
  return sh_from_d(s);
}

static inline sh_t sh_mul(sh_t a, sh_t b) {
  return sh_from_d((double)sh_to_f(a) * (double)sh_to_f(b));
}

#endif
