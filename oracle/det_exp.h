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

/* log(x), positive normal x: the Cephes logf scheme with every operation rounded once. */
static inline float orc_logf(float x) {
  if (!(x < INFINITY)) return x; /* NaN and +inf pass through */
  uint32_t bits;
  memcpy(&bits, &x, 4);
  int e = (int)(bits >> 23) - 126;
  uint32_t mb = (bits & 0x007fffffu) | 0x3f000000u;
  float m;
  memcpy(&m, &mb, 4);
  if (m < 0.70710678118654752f) {
    e -= 1;
    volatile float m2 = m + m;
    volatile float m3 = m2 + -1.0f;
    m = m3;
  } else {
    volatile float m3 = m + -1.0f;
    m = m3;
  }
  volatile float z = m * m;
  float p = 7.0376836292e-2f;
  p = fmaf(p, m, -1.1514610310e-1f);
  p = fmaf(p, m, 1.1676998740e-1f);
  p = fmaf(p, m, -1.2420140846e-1f);
  p = fmaf(p, m, 1.4249322787e-1f);
  p = fmaf(p, m, -1.6668057665e-1f);
  p = fmaf(p, m, 2.0000714765e-1f);
  p = fmaf(p, m, -2.4999993993e-1f);
  p = fmaf(p, m, 3.3333331174e-1f);
  volatile float pm = p * m;
  volatile float y0 = pm * z;
  float fe = (float)e;
  float y = fmaf(-2.12194440e-4f, fe, y0);
  y = fmaf(-0.5f, z, y);
  volatile float r0 = m + y;
  return fmaf(0.693359375f, fe, r0);
}

/* sqrt(softplus(x)), softplus(x) = x above 20 (topk_softplus_sqrt_kernels.cpp:233-261). */
static inline float orc_softplus_sqrtf(float x) {
  if (x > 20.0f) return sqrtf(x);
  volatile float one_plus = 1.0f + orc_expf(x);
  return sqrtf(orc_logf(one_plus));
}

#endif
