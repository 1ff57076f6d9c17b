// Shared helpers for the sm_100a MoE kernels: error plumbing for the C ABI,
// element-type traits and 128-bit vector access.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/b200moe.h"

namespace b200moe {

// Records a message for b200moe_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

#define B200_CHECK_ARG(cond, ...)                                   \
  do {                                                              \
    if (!(cond)) return ::b200moe::fail(B200MOE_E_BADARG, __VA_ARGS__); \
  } while (0)

#define B200_CUDA_OK(expr)                                                     \
  do {                                                                         \
    cudaError_t e__ = (expr);                                                  \
    if (e__ != cudaSuccess)                                                    \
      return ::b200moe::fail(B200MOE_E_CUDA, "%s failed: %s", #expr,          \
                             cudaGetErrorString(e__));                         \
  } while (0)

#define B200_LAUNCH_OK(name)                                                   \
  do {                                                                         \
    cudaError_t e__ = cudaGetLastError();                                      \
    if (e__ != cudaSuccess)                                                    \
      return ::b200moe::fail(B200MOE_E_CUDA, "launch of %s failed: %s", name, \
                             cudaGetErrorString(e__));                         \
  } while (0)

inline cudaStream_t as_stream(b200moe_stream s) { return (cudaStream_t)s; }

inline int dtype_bytes(b200moe_dtype t) {
  switch (t) {
    case B200MOE_F32: case B200MOE_I32: case B200MOE_U32: return 4;
    case B200MOE_F16: case B200MOE_BF16: return 2;
    case B200MOE_I64: return 8;
    default: return 1;
  }
}

// ---- scalar conversions --------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// e4m3fn round-to-nearest-even with saturation to +-448 (NaN stays NaN).
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// e5m2 is the upper byte of an IEEE half.
__device__ __forceinline__ float e5m2_to_f32(uint8_t v) {
  __half_raw h;
  h.x = (unsigned short)((unsigned short)v << 8);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// e2m1 code (4 bits) -> float: {0,.5,1,1.5,2,3,4,6} with sign bit 3.
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float m = mag[code & 7];
  return (code & 8) ? -m : m;
}
// e8m0 byte -> 2^(b-127) (b = 0 gives 2^-127, a subnormal float; 255 = NaN).
__device__ __forceinline__ float e8m0_to_f32(uint32_t b) {
  if (b == 255) return __uint_as_float(0x7fc00000u);
  if (b == 0) return __uint_as_float(0x00400000u);
  return __uint_as_float(b << 23);
}

// ---- 16-byte vector load/store ---------------------------------------------
struct alignas(16) vec16 { uint32_t w[4]; };

__device__ __forceinline__ vec16 ld16(const void* p) {
  return *reinterpret_cast<const vec16*>(p);
}
__device__ __forceinline__ void st16(void* p, const vec16& v) {
  *reinterpret_cast<vec16*>(p) = v;
}

// Dispatch a lambda-like macro body on a 16/32-bit float element type.
#define B200_DISPATCH_FLOAT(DTYPE, NAME, ...)                                  \
  switch (DTYPE) {                                                             \
    case B200MOE_F32: { using scalar_t = float; __VA_ARGS__; break; }          \
    case B200MOE_F16: { using scalar_t = __half; __VA_ARGS__; break; }         \
    case B200MOE_BF16: { using scalar_t = __nv_bfloat16; __VA_ARGS__; break; } \
    default:                                                                   \
      return ::b200moe::fail(B200MOE_E_BADARG,                                 \
                             "%s: only float32, float16 and bfloat16 are "     \
                             "supported", NAME);                               \
  }

}  // namespace b200moe
