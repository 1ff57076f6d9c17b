// Deterministic single-precision exp / sigmoid built only from IEEE-754
// correctly rounded operations (mul, add, fma, div, round-to-nearest-even), so
// that a host compiler and nvcc produce the same bits for the same input.
// Routing weights computed with these functions can therefore be compared
// bit-for-bit between the CUDA kernels and a CPU restatement that performs the
// same sequence of operations.
#pragma once

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDA_ARCH__)
#define DM_HD __host__ __device__ __forceinline__
#define DM_MUL(a, b) __fmul_rn((a), (b))
#define DM_ADD(a, b) __fadd_rn((a), (b))
#define DM_FMA(a, b, c) __fmaf_rn((a), (b), (c))
#define DM_DIV(a, b) __fdiv_rn((a), (b))
#elif defined(__CUDACC__)
#define DM_HD __host__ __device__ __forceinline__
#define DM_MUL(a, b) ((a) * (b))
#define DM_ADD(a, b) ((a) + (b))
#define DM_FMA(a, b, c) fmaf((a), (b), (c))
#define DM_DIV(a, b) ((a) / (b))
#else
#define DM_HD static inline
#define DM_MUL(a, b) ((a) * (b))
#define DM_ADD(a, b) ((a) + (b))
#define DM_FMA(a, b, c) fmaf((a), (b), (c))
#define DM_DIV(a, b) ((a) / (b))
#endif

DM_HD float dm_pow2i(int e) {  // 2^e for e in [-126, 127]
  uint32_t bits = (uint32_t)(e + 127) << 23;
  float f;
#if defined(__CUDA_ARCH__)
  f = __uint_as_float(bits);
#else
  memcpy(&f, &bits, sizeof(f));
#endif
  return f;
}

// exp(x): range reduction x = n*ln2 + r, |r| <= ln2/2, degree-6 polynomial,
// result scaled by 2^n in two exact steps (so that results in the subnormal
// range are rounded once).  Max error about 1 ulp.
DM_HD float dm_expf(float x) {
  if (x != x) return x;
  if (x > 88.75f) return INFINITY;
  if (x < -104.0f) return 0.0f;
  float t = DM_MUL(x, 1.44269504088896341f);
  float n = rintf(t);
  float r = DM_FMA(n, -0.693359375f, x);
  r = DM_FMA(n, 2.12194440e-4f, r);
  float p = 1.9875691500e-4f;
  p = DM_FMA(p, r, 1.3981999507e-3f);
  p = DM_FMA(p, r, 8.3334519073e-3f);
  p = DM_FMA(p, r, 4.1665795894e-2f);
  p = DM_FMA(p, r, 1.6666665459e-1f);
  p = DM_FMA(p, r, 5.0000001201e-1f);
  float r2 = DM_MUL(r, r);
  p = DM_FMA(p, r2, r);
  p = DM_ADD(p, 1.0f);
  int ni = (int)n;
  int n1 = ni / 2;
  int n2 = ni - n1;
  p = DM_MUL(p, dm_pow2i(n1));
  p = DM_MUL(p, dm_pow2i(n2));
  return p;
}

DM_HD float dm_sigmoidf(float x) {
  float e = dm_expf(-x);
  return DM_DIV(1.0f, DM_ADD(1.0f, e));
}

// log(x) for positive normal x: x = m * 2^e with m in [sqrt(1/2), sqrt(2)),
// degree-9 polynomial in m - 1 (the Cephes logf scheme), every step a
// correctly rounded IEEE operation.  About 1 ulp.  NaN and +inf are returned as is.
DM_HD float dm_logf(float x) {
  if (!(x < INFINITY)) return x;   // NaN and +inf pass through
  uint32_t bits;
#if defined(__CUDA_ARCH__)
  bits = __float_as_uint(x);
#else
  memcpy(&bits, &x, sizeof(bits));
#endif
  int e = (int)(bits >> 23) - 126;
  const uint32_t mb = (bits & 0x007fffffu) | 0x3f000000u;   // m in [0.5, 1)
  float m;
#if defined(__CUDA_ARCH__)
  m = __uint_as_float(mb);
#else
  memcpy(&m, &mb, sizeof(m));
#endif
  if (m < 0.70710678118654752f) {
    e -= 1;
    m = DM_ADD(DM_ADD(m, m), -1.0f);
  } else {
    m = DM_ADD(m, -1.0f);
  }
  const float z = DM_MUL(m, m);
  float p = 7.0376836292e-2f;
  p = DM_FMA(p, m, -1.1514610310e-1f);
  p = DM_FMA(p, m, 1.1676998740e-1f);
  p = DM_FMA(p, m, -1.2420140846e-1f);
  p = DM_FMA(p, m, 1.4249322787e-1f);
  p = DM_FMA(p, m, -1.6668057665e-1f);
  p = DM_FMA(p, m, 2.0000714765e-1f);
  p = DM_FMA(p, m, -2.4999993993e-1f);
  p = DM_FMA(p, m, 3.3333331174e-1f);
  float y = DM_MUL(DM_MUL(p, m), z);
  const float fe = (float)e;
  y = DM_FMA(-2.12194440e-4f, fe, y);
  y = DM_FMA(-0.5f, z, y);
  float r = DM_ADD(m, y);
  r = DM_FMA(0.693359375f, fe, r);
  return r;
}

// sqrt(softplus(x)) with softplus(x) = x for x > 20, else log(1 + exp(x))
// (csrc/moe/topk_softplus_sqrt_kernels.cpp:233-261, 303-309 of vllm-xpu-kernels).
DM_HD float dm_softplus_sqrtf(float x) {
  const float sp = (x > 20.0f) ? x : dm_logf(DM_ADD(1.0f, dm_expf(x)));
#if defined(__CUDA_ARCH__)
  return __fsqrt_rn(sp);
#else
  return sqrtf(sp);
#endif
}
