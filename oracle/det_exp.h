/* TEST INFRASTRUCTURE - not part of the product.
 *
 * exp() and sigmoid() made only of IEEE-754 correctly rounded single-precision
 * operations, written out independently of the CUDA kernels but with the same
 * operation sequence, so the router's weights can be checked bit for bit.
 * Compile without floating-point contraction (-ffp-contract=off). */
#ifndef ORACLE_DET_EXP_H_
#define ORACLE_DET_EXP_H_
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float orc_pow2i(int e) {
  uint32_t bits = (uint32_t)(e + 127) << 23;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static inline float orc_expf(float x) {
  if (x != x) return x;
  if (x > 88.75f) return INFINITY;
  if (x < -104.0f) return 0.0f;
  volatile float t = x * 1.44269504088896341f;
  float n = rintf(t);
  float r = fmaf(n, -0.693359375f, x);
  r = fmaf(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  volatile float r2 = r * r;
  p = fmaf(p, r2, r);
  volatile float q = p + 1.0f;
  int ni = (int)n;
  int n1 = ni / 2, n2 = ni - n1;
  volatile float s1 = q * orc_pow2i(n1);
  volatile float s2 = s1 * orc_pow2i(n2);
  return s2;
}

static inline float orc_sigmoidf(float x) {
  volatile float e = orc_expf(-x);
  volatile float d = 1.0f + e;
  volatile float r = 1.0f / d;
  return r;
}
#endif
