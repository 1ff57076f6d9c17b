// HBM-bound elementwise stages of the MoE layer: gated activations, dynamic
// per-token-group fp8 quantisation, and the top-k reductions (moe_gather,
// moe_sum).  All of them move 16 bytes per thread per access and use one
// thread block per row (or per row slice) so that every global access of a
// warp is one contiguous 512-byte run.
//
// Math follows csrc/activation.cpp:16-20, 81-87, 277-295,
// csrc/quantization/fp8/fp8_quant.cpp:335-387, csrc/moe/moe_gather.cpp:46-87
// and csrc/moe/moe_align_sum_kernels.cpp:629-663 of vllm-xpu-kernels.
#include "common.cuh"

namespace b200moe {
namespace {

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// out[r, i] = T(silu(in[r, i])) * in[r, d + i], product rounded once to T.
template <typename T>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(T* __restrict__ out, const T* __restrict__ in, int d, bool vec_ok) {
  constexpr int N = Vec<T>::N;
  const int64_t r = blockIdx.x;
  const T* g = in + r * 2 * (int64_t)d;
  const T* u = g + d;
  T* o = out + r * (int64_t)d;
  if (vec_ok) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d / N; j += gridDim.y * blockDim.x) {
      const vec16 gv = ld16(g + (int64_t)j * N);
      const vec16 uv = ld16(u + (int64_t)j * N);
      vec16 ov;
      const T* ge = reinterpret_cast<const T*>(&gv);
      const T* ue = reinterpret_cast<const T*>(&uv);
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const T s = from_f32<T>(silu_f32(to_f32<T>(ge[i])));
        oe[i] = from_f32<T>(to_f32<T>(s) * to_f32<T>(ue[i]));
      }
      st16(o + (int64_t)j * N, ov);
    }
  } else {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d; j += gridDim.y * blockDim.x) {
      const T s = from_f32<T>(silu_f32(to_f32<T>(g[j])));
      o[j] = from_f32<T>(to_f32<T>(s) * to_f32<T>(u[j]));
    }
  }
}

// Other gated activations of the layer (csrc/activation.cpp:45-75, 299-312 of the
// reference).  kKind 1: gelu (erf), 2: gelu (tanh form): out = T(act(x)) *_T y as
// in silu_and_mul; 3: swiglustep: out = T(min(silu(g), limit) * clamp(u, +-limit))
// in fp32; 4: relu2_no_mul: out = T(max(x, 0)^2), no second half.
template <typename T, int kKind>
__device__ __forceinline__ T gated_act(T gv, T uv, float limit) {
  const float f = to_f32<T>(gv);
  if (kKind == 1) {
    const T a = from_f32<T>(f * 0.5f * (1.0f + erff(f * 0.70710678118654752440f)));
    return from_f32<T>(to_f32<T>(a) * to_f32<T>(uv));
  } else if (kKind == 2) {
    const float inner = 0.79788456080286535588f * (f + 0.044715f * (f * f * f));
    const T a = from_f32<T>(0.5f * f * (1.0f + tanhf(inner)));
    return from_f32<T>(to_f32<T>(a) * to_f32<T>(uv));
  } else if (kKind == 3) {
    const float sg = fminf(silu_f32(f), limit);
    const float u = fminf(fmaxf(to_f32<T>(uv), -limit), limit);
    return from_f32<T>(sg * u);
  } else {
    const float r = fmaxf(f, 0.0f);
    return from_f32<T>(r * r);
  }
}

// Rows of [x(d) | y(d)] -> d outputs (kKind 4: rows of d inputs -> d outputs).
template <typename T, int kKind>
__global__ void __launch_bounds__(256)
gated_act_kernel(T* __restrict__ out, const T* __restrict__ in, int d, float limit, bool vec_ok) {
  constexpr int N = Vec<T>::N;
  constexpr bool kGated = kKind != 4;
  const int64_t r = blockIdx.x;
  const T* g = in + r * (kGated ? 2 : 1) * (int64_t)d;
  const T* u = kGated ? g + d : g;
  T* o = out + r * (int64_t)d;
  if (vec_ok) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d / N; j += gridDim.y * blockDim.x) {
      const vec16 gv = ld16(g + (int64_t)j * N);
      const vec16 uv = kGated ? ld16(u + (int64_t)j * N) : gv;
      const T* ge = reinterpret_cast<const T*>(&gv);
      const T* ue = reinterpret_cast<const T*>(&uv);
      vec16 ov;
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = gated_act<T, kKind>(ge[i], ue[i], limit);
      st16(o + (int64_t)j * N, ov);
    }
  } else {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d; j += gridDim.y * blockDim.x)
      o[j] = gated_act<T, kKind>(g[j], u[j], limit);
  }
}

__device__ __forceinline__ float swigluoai_f32(float g, float u, float alpha, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  const float sig = 1.0f / (1.0f + expf(-g * alpha));
  return (u + 1.0f) * g * sig;
}

// gate = even columns, up = odd columns of in[r, 0:2d].
template <typename T>
__global__ void __launch_bounds__(256)
swigluoai_and_mul_kernel(T* __restrict__ out, const T* __restrict__ in, int d, float alpha,
                         float limit, bool vec_ok) {
  constexpr int N = Vec<T>::N;  // inputs per 16-byte load; N/2 outputs
  const int64_t r = blockIdx.x;
  const T* x = in + r * 2 * (int64_t)d;
  T* o = out + r * (int64_t)d;
  if (vec_ok) {
    // two loads -> N outputs -> one 16-byte store
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d / N; j += gridDim.y * blockDim.x) {
      const vec16 a = ld16(x + (int64_t)j * 2 * N);
      const vec16 b = ld16(x + (int64_t)j * 2 * N + N);
      vec16 ov;
      const T* ae = reinterpret_cast<const T*>(&a);
      const T* be = reinterpret_cast<const T*>(&b);
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        oe[i] = from_f32<T>(swigluoai_f32(to_f32<T>(ae[2 * i]), to_f32<T>(ae[2 * i + 1]), alpha, limit));
        oe[N / 2 + i] = from_f32<T>(swigluoai_f32(to_f32<T>(be[2 * i]), to_f32<T>(be[2 * i + 1]), alpha, limit));
      }
      st16(o + (int64_t)j * N, ov);
    }
  } else {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < d; j += gridDim.y * blockDim.x)
      o[j] = from_f32<T>(swigluoai_f32(to_f32<T>(x[2 * j]), to_f32<T>(x[2 * j + 1]), alpha, limit));
  }
}

// Rounds a positive scale up to the next power of two (exact version of
// exp2(ceil(log2(s)))).
__device__ __forceinline__ float ceil_pow2(float s) {
  s = fmaxf(fabsf(s), 1e-10f);
  uint32_t b = __float_as_uint(s);
  if (b & 0x007fffffu) b = (b & 0xff800000u) + 0x00800000u;
  return __uint_as_float(b);
}

// One block per row.  A thread owns 16 bytes of input; `lanes_per_group`
// adjacent lanes (a power of two <= 32) share one scale.
template <typename T>
__global__ void __launch_bounds__(1024)
group_quant_fp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ s,
                       int cols, int group, float eps, bool ue8m0, int64_t s_stride_row,
                       int64_t s_stride_col) {
  constexpr int N = Vec<T>::N;
  const int64_t r = blockIdx.x;
  const int lanes_per_group = group / N;
  const int nvec = cols / N;
  const T* xr = x + r * (int64_t)cols;
  uint8_t* qr = q + r * (int64_t)cols;
  for (int j0 = (threadIdx.x & ~31); j0 < nvec; j0 += blockDim.x) {
    const int j = j0 + (threadIdx.x & 31);
    const bool active = j < nvec;
    float v[N];
    float amax = active ? eps : 0.f;
    if (active) {
      const vec16 in = ld16(xr + (int64_t)j * N);
      const T* e = reinterpret_cast<const T*>(&in);
#pragma unroll
      for (int i = 0; i < N; ++i) { v[i] = to_f32<T>(e[i]); amax = fmaxf(amax, fabsf(v[i])); }
    }
    for (int off = 1; off < lanes_per_group; off <<= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float ys = fmaxf(__fdiv_rn(amax, 448.f), 1.0f / (448.f * 512.f));
    if (ue8m0) ys = ceil_pow2(ys);
    if (active) {
      if ((j % lanes_per_group) == 0)
        s[r * s_stride_row + (int64_t)(j / lanes_per_group) * s_stride_col] = ys;
      const float inv = __fdiv_rn(1.0f, ys);
      alignas(8) uint8_t o[N];
#pragma unroll
      for (int i = 0; i < N; ++i)
        o[i] = f32_to_e4m3(fminf(fmaxf(__fmul_rn(v[i], inv), -448.f), 448.f));
      if (N == 8) {
        *reinterpret_cast<uint2*>(qr + (int64_t)j * 8) = *reinterpret_cast<uint2*>(o);
      } else {
        *reinterpret_cast<uint32_t*>(qr + (int64_t)j * 4) = *reinterpret_cast<uint32_t*>(o);
      }
    }
  }
}

// Scalar fallback: one warp per group, any group size.
template <typename T>
__global__ void __launch_bounds__(256)
group_quant_fp8_scalar_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                              float* __restrict__ s, int64_t n_groups, int groups_per_row,
                              int group, float eps, bool ue8m0, int64_t s_stride_row,
                              int64_t s_stride_col) {
  const int lane = threadIdx.x & 31;
  const int64_t g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= n_groups) return;
  const T* xg = x + g * group;
  float amax = eps;
  for (int i = lane; i < group; i += 32) amax = fmaxf(amax, fabsf(to_f32<T>(xg[i])));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  float ys = fmaxf(__fdiv_rn(amax, 448.f), 1.0f / (448.f * 512.f));
  if (ue8m0) ys = ceil_pow2(ys);
  if (lane == 0) s[(g / groups_per_row) * s_stride_row + (g % groups_per_row) * s_stride_col] = ys;
  const float inv = __fdiv_rn(1.0f, ys);
  for (int i = lane; i < group; i += 32)
    q[g * group + i] = f32_to_e4m3(fminf(fmaxf(__fmul_rn(to_f32<T>(xg[i]), inv), -448.f), 448.f));
}

// MX-format activation quantisation: per 32 consecutive values one power-of-two
// scale 2^(b-127) (stored as the e8m0 byte b, the smallest power of two with
// amax / scale <= 448) and e4m3 codes of x / scale.  With terms == 2 a second
// plane holds the residual x - code * scale quantised the same way, so that the
// two planes together carry about 8 significant bits.
// Layouts: codes [terms][rows][cols]; scales as 32-bit words [terms][ceil(cols/128)]
// [rows], byte (g & 3) of word [g >> 2][row] for group g (so the GEMM reads one
// coalesced word per row and 128-wide K block); bytes of groups past the row end
// are 0x7f (2^0).  A lane owns 8 values, four lanes one group; one block per row.
template <typename T>
__global__ void __launch_bounds__(256)
quant_mxfp8_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ s,
                   int64_t rows, int cols, int terms) {
  const int64_t r = blockIdx.x;
  const T* xr = x + r * (int64_t)cols;
  const int nvec = cols / 8;
  const int num_kb = (cols + 127) / 128;
  const int64_t q_plane = rows * (int64_t)cols;
  const int64_t s_plane = (int64_t)num_kb * rows * 4;
  for (int j0 = (threadIdx.x & ~31); j0 < nvec; j0 += blockDim.x) {
    const int j = j0 + (threadIdx.x & 31);
    const bool active = j < nvec;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (active) {
      const vec16 in = ld16(xr + (int64_t)j * 8);
      const T* e = reinterpret_cast<const T*>(&in);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = to_f32<T>(e[i]);
    }
    const int64_t s_off = (((int64_t)(j >> 4)) * rows + r) * 4 + ((j >> 2) & 3);
    for (int term = 0; term < terms; ++term) {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // smallest power of two >= amax / 448 (floor 1e-10)
      const float sc = ceil_pow2(__fdiv_rn(amax, 448.f));
      const uint32_t sbyte = (__float_as_uint(sc) >> 23) & 0xffu;
      if (active) {
        if ((j & 3) == 0) s[term * s_plane + s_off] = (uint8_t)sbyte;
        const float inv = __fdiv_rn(1.0f, sc);
        alignas(8) uint8_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          o[i] = f32_to_e4m3(fminf(fmaxf(__fmul_rn(v[i], inv), -448.f), 448.f));
          v[i] = __fsub_rn(v[i], __fmul_rn(e4m3_to_f32(o[i]), sc));  // residual for the next plane
        }
        *reinterpret_cast<uint2*>(q + term * q_plane + r * (int64_t)cols + (int64_t)j * 8) =
            *reinterpret_cast<uint2*>(o);
      }
    }
  }
  const int pad = 4 * num_kb - cols / 32;
  if ((int)threadIdx.x < pad * terms) {
    const int term = threadIdx.x / pad, g = cols / 32 + threadIdx.x % pad;
    s[term * s_plane + (((int64_t)(g >> 2)) * rows + r) * 4 + (g & 3)] = 0x7f;
  }
}

// out[t, :] = sum_k w[t,k] * moe_out[row_map[t,k], :], fp32, k ascending.
// kWeighted = false is moe_sum: slot (t,k) reads row t*K+k of src and is skipped
// when its id is negative or maps to a negative entry of `map`.
template <typename T, bool kWeighted>
__global__ void __launch_bounds__(256)
topk_reduce_kernel(T* __restrict__ out, const T* __restrict__ src, const float* __restrict__ w,
                   const int32_t* __restrict__ row_map, const void* __restrict__ ids,
                   b200moe_dtype ids_dtype, const int32_t* __restrict__ map, int H, int K,
                   bool vec_ok) {
  constexpr int N = Vec<T>::N;
  const int64_t t = blockIdx.x;
  __shared__ int rows[64];
  __shared__ float wk[64];
  if (threadIdx.x < K) {
    const int64_t slot = t * K + threadIdx.x;
    if (kWeighted) {
      rows[threadIdx.x] = row_map[slot];
      wk[threadIdx.x] = w[slot];
    } else {
      bool skip = false;
      if (ids != nullptr) {
        const int64_t e = (ids_dtype == B200MOE_I64)
                              ? reinterpret_cast<const int64_t*>(ids)[slot]
                              : (int64_t) reinterpret_cast<const int32_t*>(ids)[slot];
        skip = (e < 0) || (map != nullptr && map[e] < 0);
      }
      rows[threadIdx.x] = skip ? -1 : (int)slot;
      wk[threadIdx.x] = 1.0f;
    }
  }
  __syncthreads();
  if (vec_ok) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < H / N; j += gridDim.y * blockDim.x) {
      float acc[N];
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int r = rows[k];
        if (r < 0) continue;
        const vec16 v = ld16(src + (int64_t)r * H + (int64_t)j * N);
        const T* e = reinterpret_cast<const T*>(&v);
        const float wv = wk[k];
#pragma unroll
        for (int i = 0; i < N; ++i)
          acc[i] = kWeighted ? fmaf(to_f32<T>(e[i]), wv, acc[i]) : acc[i] + to_f32<T>(e[i]);
      }
      vec16 ov;
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = from_f32<T>(acc[i]);
      st16(out + t * (int64_t)H + (int64_t)j * N, ov);
    }
  } else {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < H; j += gridDim.y * blockDim.x) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        const int r = rows[k];
        if (r < 0) continue;
        const float x = to_f32<T>(src[(int64_t)r * H + j]);
        acc = kWeighted ? fmaf(x, wk[k], acc) : acc + x;
      }
      out[t * (int64_t)H + j] = from_f32<T>(acc);
    }
  }
}

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

inline dim3 row_grid(int64_t rows, int work_items) {
  // Split long rows across blockIdx.y when there are few rows, so that small
  // token counts still fill the 148 SMs.
  int y = 1;
  if (rows < 296) {
    const int per_block = 256;
    const int max_y = (work_items + per_block - 1) / per_block;
    y = (int)((296 + rows - 1) / (rows > 0 ? rows : 1));
    if (y > max_y) y = max_y;
    if (y < 1) y = 1;
  }
  return dim3((unsigned)rows, (unsigned)y, 1);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_silu_and_mul(void* out, const void* in, b200moe_dtype dtype, int64_t rows,
                                    int d, b200moe_stream stream) {
  B200_CHECK_ARG(rows >= 0 && d >= 0, "silu_and_mul: negative size");
  if (rows == 0 || d == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && in, "silu_and_mul: null pointer");
  B200_DISPATCH_FLOAT(dtype, "silu_and_mul", {
    constexpr int N = 16 / sizeof(scalar_t);
    const bool vec_ok = (d % N == 0) && aligned16(out) && aligned16(in);
    silu_and_mul_kernel<scalar_t><<<row_grid(rows, vec_ok ? d / N : d), 256, 0, as_stream(stream)>>>(
        (scalar_t*)out, (const scalar_t*)in, d, vec_ok);
  });
  B200_LAUNCH_OK("silu_and_mul_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_swigluoai_and_mul(void* out, const void* in, b200moe_dtype dtype,
                                         int64_t rows, int d, float alpha, float limit,
                                         b200moe_stream stream) {
  B200_CHECK_ARG(rows >= 0 && d >= 0, "swigluoai_and_mul: negative size");
  if (rows == 0 || d == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && in, "swigluoai_and_mul: null pointer");
  B200_DISPATCH_FLOAT(dtype, "swigluoai_and_mul", {
    constexpr int N = 16 / sizeof(scalar_t);
    const bool vec_ok = (d % N == 0) && aligned16(out) && aligned16(in);
    swigluoai_and_mul_kernel<scalar_t>
        <<<row_grid(rows, vec_ok ? d / N : d), 256, 0, as_stream(stream)>>>(
            (scalar_t*)out, (const scalar_t*)in, d, alpha, limit, vec_ok);
  });
  B200_LAUNCH_OK("swigluoai_and_mul_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_per_token_group_fp8_quant(const void* x, b200moe_dtype dtype, void* q,
                                                 float* s, int64_t rows, int cols, int group_size,
                                                 float eps, int scale_ue8m0, int64_t s_stride_row,
                                                 int64_t s_stride_col, b200moe_stream stream) {
  B200_CHECK_ARG(rows >= 0 && cols >= 0, "per_token_group_fp8_quant: negative size");
  B200_CHECK_ARG(group_size >= 1 && cols % group_size == 0,
                 "per_token_group_fp8_quant: the row length must be a multiple of group_size");
  if (rows == 0 || cols == 0) return B200MOE_OK;
  B200_CHECK_ARG(x && q && s, "per_token_group_fp8_quant: null pointer");
  cudaStream_t st = as_stream(stream);
  B200_DISPATCH_FLOAT(dtype, "per_token_group_fp8_quant", {
    constexpr int N = 16 / sizeof(scalar_t);
    const int lpg = group_size / N;
    const bool vec_ok = (group_size % N == 0) && lpg <= 32 && (lpg & (lpg - 1)) == 0 &&
                        aligned16(x) && (((uintptr_t)q & 7) == 0);
    if (vec_ok) {
      int threads = ((cols / N + 31) / 32) * 32;
      if (threads > 1024) threads = 1024;
      group_quant_fp8_kernel<scalar_t><<<(unsigned)rows, threads, 0, st>>>(
          (const scalar_t*)x, (uint8_t*)q, s, cols, group_size, eps, scale_ue8m0 != 0,
          s_stride_row, s_stride_col);
    } else {
      const int64_t n_groups = rows * (cols / group_size);
      group_quant_fp8_scalar_kernel<scalar_t><<<(unsigned)((n_groups + 7) / 8), 256, 0, st>>>(
          (const scalar_t*)x, (uint8_t*)q, s, n_groups, cols / group_size, group_size, eps,
          scale_ue8m0 != 0, s_stride_row, s_stride_col);
    }
  });
  B200_LAUNCH_OK("group_quant_fp8_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_moe_gather(void* out, const void* moe_out, const float* topk_weights,
                                  const int32_t* row_map, b200moe_dtype dtype, int64_t num_tokens,
                                  int hidden, int topk, b200moe_stream stream) {
  B200_CHECK_ARG(topk >= 1 && topk <= 64, "error: not support TOPK=%d", topk);
  B200_CHECK_ARG(num_tokens >= 0 && hidden >= 0, "moe_gather: negative size");
  if (num_tokens == 0 || hidden == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && moe_out && topk_weights && row_map, "moe_gather: null pointer");
  B200_DISPATCH_FLOAT(dtype, "moe_gather", {
    constexpr int N = 16 / sizeof(scalar_t);
    const bool vec_ok = (hidden % N == 0) && aligned16(out) && aligned16(moe_out);
    topk_reduce_kernel<scalar_t, true>
        <<<row_grid(num_tokens, vec_ok ? hidden / N : hidden), 256, 0, as_stream(stream)>>>(
            (scalar_t*)out, (const scalar_t*)moe_out, topk_weights, row_map, nullptr, B200MOE_I32,
            nullptr, hidden, topk, vec_ok);
  });
  B200_LAUNCH_OK("topk_reduce_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_moe_sum(void* out, const void* in, b200moe_dtype dtype, int64_t num_tokens,
                               int topk, int hidden, const void* topk_ids, b200moe_dtype ids_dtype,
                               const int32_t* expert_map, b200moe_stream stream) {
  B200_CHECK_ARG(topk >= 1, "moe_sum: topk must be positive");
  B200_CHECK_ARG(expert_map == nullptr || topk_ids != nullptr,
                 "expert_map requires topk_ids to be provided");
  B200_CHECK_ARG(topk_ids == nullptr || ids_dtype == B200MOE_I32 || ids_dtype == B200MOE_I64,
                 "moe_sum: topk_ids must be int32 or int64");
  if (num_tokens == 0 || hidden == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && in, "moe_sum: null pointer");
  B200_CHECK_ARG(topk <= 64, "moe_sum: topk larger than 64 is not supported");
  B200_DISPATCH_FLOAT(dtype, "moe_sum", {
    constexpr int N = 16 / sizeof(scalar_t);
    const bool vec_ok = (hidden % N == 0) && aligned16(out) && aligned16(in);
    topk_reduce_kernel<scalar_t, false>
        <<<row_grid(num_tokens, vec_ok ? hidden / N : hidden), 256, 0, as_stream(stream)>>>(
            (scalar_t*)out, (const scalar_t*)in, nullptr, nullptr, topk_ids, ids_dtype,
            expert_map, hidden, topk, vec_ok);
  });
  B200_LAUNCH_OK("topk_reduce_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_quant_mxfp8(const void* x, b200moe_dtype dtype, void* q, void* s, int64_t rows,
                                   int cols, int terms, b200moe_stream stream) {
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "quant_mxfp8: input must be bfloat16 or float16");
  B200_CHECK_ARG(rows >= 0 && cols >= 0 && cols % 32 == 0, "quant_mxfp8: the row length must be a multiple of 32");
  B200_CHECK_ARG(terms == 1 || terms == 2, "quant_mxfp8: terms must be 1 or 2");
  if (rows == 0 || cols == 0) return B200MOE_OK;
  B200_CHECK_ARG(x && q && s, "quant_mxfp8: null pointer");
  B200_CHECK_ARG(aligned16(x) && (((uintptr_t)q & 7) == 0), "quant_mxfp8: buffers must be 16-byte aligned");
  if (dtype == B200MOE_BF16)
    quant_mxfp8_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, as_stream(stream)>>>(
        (const __nv_bfloat16*)x, (uint8_t*)q, (uint8_t*)s, rows, cols, terms);
  else
    quant_mxfp8_kernel<__half><<<(unsigned)rows, 256, 0, as_stream(stream)>>>(
        (const __half*)x, (uint8_t*)q, (uint8_t*)s, rows, cols, terms);
  B200_LAUNCH_OK("quant_mxfp8_kernel");
  return B200MOE_OK;
}

namespace {
template <int kKind>
int launch_gated_act(void* out, const void* in, b200moe_dtype dtype, int64_t rows, int d, float limit,
                     b200moe_stream stream, const char* name) {
  B200_CHECK_ARG(rows >= 0 && d >= 0, "%s: negative size", name);
  if (rows == 0 || d == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && in, "%s: null pointer", name);
  B200_DISPATCH_FLOAT(dtype, name, {
    constexpr int N = 16 / sizeof(scalar_t);
    const bool vec_ok = (d % N == 0) && aligned16(out) && aligned16(in);
    gated_act_kernel<scalar_t, kKind><<<row_grid(rows, vec_ok ? d / N : d), 256, 0, as_stream(stream)>>>(
        (scalar_t*)out, (const scalar_t*)in, d, limit, vec_ok);
  });
  B200_LAUNCH_OK(name);
  return B200MOE_OK;
}
}  // namespace

extern "C" int b200moe_gelu_and_mul(void* out, const void* in, b200moe_dtype dtype, int64_t rows, int d,
                                    b200moe_stream stream) {
  return launch_gated_act<1>(out, in, dtype, rows, d, 0.f, stream, "gelu_and_mul");
}
extern "C" int b200moe_gelu_tanh_and_mul(void* out, const void* in, b200moe_dtype dtype, int64_t rows, int d,
                                         b200moe_stream stream) {
  return launch_gated_act<2>(out, in, dtype, rows, d, 0.f, stream, "gelu_tanh_and_mul");
}
extern "C" int b200moe_swiglustep_and_mul(void* out, const void* in, b200moe_dtype dtype, int64_t rows, int d,
                                          float limit, b200moe_stream stream) {
  return launch_gated_act<3>(out, in, dtype, rows, d, limit, stream, "swiglustep_and_mul");
}
extern "C" int b200moe_relu2_no_mul(void* out, const void* in, b200moe_dtype dtype, int64_t rows, int d,
                                    b200moe_stream stream) {
  return launch_gated_act<4>(out, in, dtype, rows, d, 0.f, stream, "relu2_no_mul");
}
