// Activation + quantisation ops that vLLM calls next to the fused-MoE layer
// (dense MLP, shared experts):
//   silu_and_mul_per_block_quant  csrc/quantization/fused_kernels/fused_silu_mul_block_quant.cpp:14-239
//   silu_and_mul_mxfp4_quant      csrc/quantization/fused_kernels/fused_silu_mul_mxfp4_quant.cpp:19-210
//   per_token_group_quant_mxfp4   csrc/quantization/fp4/mxfp4_quant.h:17-245, mxfp4_quant.cpp:24-126
//   silu_and_mul_quant            csrc/activation.cpp:191-234, 552-566
// of vllm-xpu-kernels.  One block per row; a thread owns 16 bytes of input (8
// sixteen-bit or 4 fp32 values), the lanes of a quantisation group are
// neighbours in a warp and combine their maxima with xor shuffles, exactly the
// work split of the reference kernels, so the operation order per value is
// theirs: fp32 silu(g) * u, group maximum, scale, divide (or multiply by the
// reciprocal where the reference does), clamp, round.  Scales use IEEE
// division; the per-value exp and divisions use the fast hardware forms (a
// couple of ulp), which can move a value across a rounding boundary about once
// in a million: the ops are arithmetic-bound, not HBM-bound, with the IEEE forms.
#include "common.cuh"

namespace b200moe {
namespace {

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// exp2(ceil(log2(max(|s|, eps)))) without the rounding of log2 / exp2.
__device__ __forceinline__ float ceil_pow2_eps(float s, float eps) {
  s = fmaxf(fabsf(s), eps);
  uint32_t b = __float_as_uint(s);
  if (b & 0x007fffffu) b = (b & 0xff800000u) + 0x00800000u;
  return __uint_as_float(b);
}

// e2m1 code of x (|x| <= 6): number of midpoints strictly below |x|, sign bit 3
// (csrc/quantization/fp4/mxfp4_quant.h:17-30 of the reference: ties go down).
__device__ __forceinline__ uint32_t f32_to_e2m1(float x) {
  const float a = fabsf(x);
  const uint32_t code = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) +
                        (a > 3.5f) + (a > 5.0f);
  return code | (x < 0.0f ? 8u : 0u);
}

__device__ __forceinline__ int8_t f32_to_i8_rn(float x) {
  return (int8_t)fminf(fmaxf(rintf(x), -128.0f), 127.0f);
}

enum OutFmt { kOutE4m3 = 0, kOutI8 = 1, kOutE2m1 = 2 };

struct GroupQuantArgs {
  const void* in;
  void* out;
  float* scales;
  const float* scale_ub;
  int hidden;           // values per output row
  int group;            // values per scale
  int64_t s_stride_row, s_stride_group;
  float eps;
  int ue8m0;
  // optional: only the first sum(rows_per_segment[0..num_segments)) rows are in use (row
  // buffers sized for a worst case); blocks past them return at once
  const int32_t* rows_per_segment = nullptr;
  int num_segments = 0;
};

// kGated: input rows are [gate(hidden) | up(hidden)] and the quantised value is
// silu(gate) * up in fp32; else the input row itself.  A block works on kRows
// consecutive rows at a time and issues all their loads before the arithmetic,
// so that enough bytes are in flight per SM to reach the HBM rate.
constexpr int kRows = 4;

template <typename T, bool kGated, int kFmt>
__global__ void __launch_bounds__(1024)
group_quant_kernel(const GroupQuantArgs a, int64_t rows) {
  constexpr int N = Vec16<T>::N;
  const int64_t r0 = (int64_t)blockIdx.x * kRows;
  if (a.rows_per_segment != nullptr) {
    __shared__ int64_t in_use;
    if (threadIdx.x < 32) {
      int64_t sum = 0;
      for (int e = threadIdx.x; e < a.num_segments; e += 32) sum += max(a.rows_per_segment[e], 0);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (threadIdx.x == 0) in_use = sum;
    }
    __syncthreads();
    if (in_use < rows) rows = in_use;
    if (r0 >= rows) return;
  }
  const int lanes_per_group = a.group / N;
  const int nvec = a.hidden / N;
  const int64_t in_pitch = (int64_t)a.hidden * (kGated ? 2 : 1);
  const T* in0 = reinterpret_cast<const T*>(a.in);
  const int lane = threadIdx.x & 31;
  for (int base = 0; base < nvec; base += blockDim.x) {
    const int c = base + threadIdx.x;
    vec16 gq[kRows], uq[kRows];
#pragma unroll
    for (int k = 0; k < kRows; ++k) {
      if (c < nvec && r0 + k < rows) {
        const T* in = in0 + (r0 + k) * in_pitch;
        gq[k] = ld16(in + (int64_t)c * N);
        if (kGated) uq[k] = ld16(in + a.hidden + (int64_t)c * N);
      }
    }
#pragma unroll
    for (int k = 0; k < kRows; ++k) {
      const int64_t r = r0 + k;
      const bool active = c < nvec && r < rows;
      float v[N];
      float amax = 0.f;
      if (active) {
        const T* ge = reinterpret_cast<const T*>(&gq[k]);
        if (kGated) {
          const T* ue = reinterpret_cast<const T*>(&uq[k]);
#pragma unroll
          for (int i = 0; i < N; ++i) {
            const float gf = to_f32<T>(ge[i]);
            v[i] = __fmul_rn(__fdividef(gf, 1.0f + __expf(-gf)), to_f32<T>(ue[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < N; ++i) v[i] = to_f32<T>(ge[i]);
        }
#pragma unroll
        for (int i = 0; i < N; ++i) amax = fmaxf(amax, fabsf(v[i]));
      }
      for (int off = 1; off < lanes_per_group; off <<= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));

      float scale;
      if (kFmt == kOutI8) {
        scale = fmaxf(__fdiv_rn(amax, 127.0f), 1.1920928955078125e-07f);
      } else if (kFmt == kOutE4m3) {
        const float floor_s = 1.0f / (448.0f * 512.0f);
        scale = fmaxf(__fdiv_rn(amax, 448.0f), floor_s);
        if (a.scale_ub != nullptr) scale = fmaxf(fminf(scale, *a.scale_ub), floor_s);
        if (a.ue8m0) scale = ceil_pow2_eps(scale, 1e-10f);
      } else {
        scale = ceil_pow2_eps(__fdiv_rn(amax, 6.0f), a.eps);
      }
      if (active && (lane % lanes_per_group) == 0)
        a.scales[r * a.s_stride_row + (int64_t)(c / lanes_per_group) * a.s_stride_group] = scale;

      if (active) {
        if (kFmt == kOutE2m1) {
          const float inv = __fdiv_rn(1.0f, scale);
          alignas(4) uint8_t o[N / 2];
#pragma unroll
          for (int i = 0; i < N; i += 2) {
            const uint32_t n0 = f32_to_e2m1(fmaxf(-6.0f, fminf(__fmul_rn(v[i], inv), 6.0f)));
            const uint32_t n1 = f32_to_e2m1(fmaxf(-6.0f, fminf(__fmul_rn(v[i + 1], inv), 6.0f)));
            o[i / 2] = (uint8_t)((n1 << 4) | n0);
          }
          uint8_t* dst = reinterpret_cast<uint8_t*>(a.out) + r * (int64_t)(a.hidden / 2) + (int64_t)c * (N / 2);
          if (N == 8) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(o);
          else *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(o);
        } else {
          alignas(8) uint8_t o[N];
#pragma unroll
          for (int i = 0; i < N; ++i) {
            const float q = __fdividef(v[i], scale);
            if (kFmt == kOutI8) o[i] = (uint8_t)f32_to_i8_rn(q);
            else o[i] = f32_to_e4m3(fmaxf(-448.0f, fminf(q, 448.0f)));
          }
          uint8_t* dst = reinterpret_cast<uint8_t*>(a.out) + r * (int64_t)a.hidden + (int64_t)c * N;
          if (N == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
          else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(o);
        }
      }
    }
  }
}

int threads_for(int nvec) {
  int t = ((nvec + 31) / 32) * 32;
  if (t > 1024) t = 1024;
  if (t < 32) t = 32;
  return t;
}

// out[r, i] = e4m3(clamp(float(T(silu(x[r,i])) * x[r,d+i]) / scale)): the product is
// rounded to T before the division, as the reference's scalar_t arithmetic does.
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_static_quant_kernel(uint8_t* __restrict__ out, const T* __restrict__ in,
                             const float* __restrict__ scale, int d, bool vec_ok) {
  constexpr int N = Vec16<T>::N;
  const int64_t r = blockIdx.x;
  const T* g = in + r * 2 * (int64_t)d;
  const T* u = g + d;
  uint8_t* o = out + r * (int64_t)d;
  const float inv = __fdiv_rn(1.0f, *scale);
  auto one = [&](T gv, T uv) {
    const float gf = to_f32<T>(gv);
    const T s = from_f32<T>(__fdividef(gf, 1.0f + __expf(-gf)));
    const T prod = from_f32<T>(to_f32<T>(s) * to_f32<T>(uv));
    return f32_to_e4m3(fmaxf(-448.0f, fminf(__fmul_rn(to_f32<T>(prod), inv), 448.0f)));
  };
  if (vec_ok) {
    for (int j = threadIdx.x; j < d / N; j += blockDim.x) {
      const vec16 gv = ld16(g + (int64_t)j * N), uv = ld16(u + (int64_t)j * N);
      const T* ge = reinterpret_cast<const T*>(&gv);
      const T* ue = reinterpret_cast<const T*>(&uv);
      alignas(8) uint8_t q[N];
#pragma unroll
      for (int i = 0; i < N; ++i) q[i] = one(ge[i], ue[i]);
      *reinterpret_cast<uint2*>(o + (int64_t)j * N) = *reinterpret_cast<const uint2*>(q);
    }
  } else {
    for (int j = threadIdx.x; j < d; j += blockDim.x) o[j] = one(g[j], u[j]);
  }
}

template <bool kGated, int kFmt>
int launch_group_quant(b200moe_dtype dtype, const GroupQuantArgs& a, int64_t rows, cudaStream_t st,
                       const char* name) {
  if (dtype == B200MOE_BF16) {
    group_quant_kernel<__nv_bfloat16, kGated, kFmt><<<(unsigned)((rows + kRows - 1) / kRows), threads_for(a.hidden / 8), 0, st>>>(a, rows);
  } else if (dtype == B200MOE_F16) {
    group_quant_kernel<__half, kGated, kFmt><<<(unsigned)((rows + kRows - 1) / kRows), threads_for(a.hidden / 8), 0, st>>>(a, rows);
  } else {
    group_quant_kernel<float, kGated, kFmt><<<(unsigned)((rows + kRows - 1) / kRows), threads_for(a.hidden / 4), 0, st>>>(a, rows);
  }
  B200_LAUNCH_OK(name);
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_silu_and_mul_per_block_quant(void* out, b200moe_dtype out_dtype, float* scales,
                                                    const void* in, b200moe_dtype dtype, int64_t rows,
                                                    int hidden, int group_size, const float* scale_ub,
                                                    int64_t s_stride_row, int64_t s_stride_group,
                                                    int scale_ue8m0, b200moe_stream stream) {
  B200_CHECK_ARG(out_dtype == B200MOE_FP8_E4M3 || out_dtype == B200MOE_I8,
                 "out must be float8_e4m3fn or int8 (float8_e5m2 is not built)");
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "input must be float16 or bfloat16");
  B200_CHECK_ARG(group_size == 32 || group_size == 64 || group_size == 128,
                 "group_size must be 32, 64, or 128, got %d", group_size);
  B200_CHECK_ARG(scale_ub == nullptr || out_dtype == B200MOE_FP8_E4M3, "scale_ub is only supported for FP8 output");
  B200_CHECK_ARG(rows >= 0 && hidden >= 0 && hidden % group_size == 0,
                 "hidden_size must be divisible by group_size");
  if (rows == 0 || hidden == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && scales && in, "silu_and_mul_per_block_quant: null pointer");
  B200_CHECK_ARG(aligned16(in) && (((uintptr_t)out & 7) == 0), "silu_and_mul_per_block_quant: misaligned buffer");
  GroupQuantArgs a = {in, out, scales, scale_ub, hidden, group_size, s_stride_row, s_stride_group, 0.f, scale_ue8m0};
  if (out_dtype == B200MOE_I8)
    return launch_group_quant<true, kOutI8>(dtype, a, rows, as_stream(stream), "silu_and_mul_per_block_quant");
  return launch_group_quant<true, kOutE4m3>(dtype, a, rows, as_stream(stream), "silu_and_mul_per_block_quant");
}

extern "C" int b200moe_silu_and_mul_per_block_quant_ragged(void* out, float* scales, const void* in,
                                                           b200moe_dtype dtype, int64_t rows, int hidden,
                                                           const int32_t* rows_per_segment, int num_segments,
                                                           b200moe_stream stream) {
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "input must be float16 or bfloat16");
  B200_CHECK_ARG(rows >= 0 && hidden >= 0 && hidden % 128 == 0, "hidden_size must be divisible by group_size");
  B200_CHECK_ARG(rows_per_segment != nullptr && num_segments >= 1, "silu_and_mul_per_block_quant_ragged: no row counts");
  if (rows == 0 || hidden == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && scales && in, "silu_and_mul_per_block_quant: null pointer");
  B200_CHECK_ARG(aligned16(in) && (((uintptr_t)out & 7) == 0), "silu_and_mul_per_block_quant: misaligned buffer");
  GroupQuantArgs a = {in, out, scales, nullptr, hidden, 128, hidden / 128, 1, 0.f, 0, rows_per_segment, num_segments};
  return launch_group_quant<true, kOutE4m3>(dtype, a, rows, as_stream(stream), "silu_and_mul_per_block_quant");
}

extern "C" int b200moe_silu_and_mul_mxfp4_quant(void* out, float* scales, const void* in, b200moe_dtype dtype,
                                                int64_t rows, int hidden, float eps, int64_t s_stride_row,
                                                int64_t s_stride_group, b200moe_stream stream) {
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "input must be float16 or bfloat16");
  B200_CHECK_ARG(rows >= 0 && hidden >= 0 && hidden % 32 == 0, "hidden_size must be divisible by group_size");
  if (rows == 0 || hidden == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && scales && in, "silu_and_mul_mxfp4_quant: null pointer");
  B200_CHECK_ARG(aligned16(in) && (((uintptr_t)out & 3) == 0), "silu_and_mul_mxfp4_quant: misaligned buffer");
  GroupQuantArgs a = {in, out, scales, nullptr, hidden, 32, s_stride_row, s_stride_group, eps, 0};
  return launch_group_quant<true, kOutE2m1>(dtype, a, rows, as_stream(stream), "silu_and_mul_mxfp4_quant");
}

extern "C" int b200moe_per_token_group_quant_mxfp4(const void* in, b200moe_dtype dtype, void* out_q, float* out_s,
                                                   int64_t rows, int hidden, float eps, int64_t s_stride_row,
                                                   int64_t s_stride_group, b200moe_stream stream) {
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16 || dtype == B200MOE_F32,
                 "per_token_group_quant_mxfp4: input must be float32, float16 or bfloat16");
  B200_CHECK_ARG(rows >= 0 && hidden >= 0 && hidden % 32 == 0,
                 "per_token_group_quant_mxfp4: the row length must be a multiple of 32");
  if (rows == 0 || hidden == 0) return B200MOE_OK;
  B200_CHECK_ARG(in && out_q && out_s, "per_token_group_quant_mxfp4: null pointer");
  B200_CHECK_ARG(aligned16(in) && (((uintptr_t)out_q & 3) == 0), "per_token_group_quant_mxfp4: misaligned buffer");
  GroupQuantArgs a = {in, out_q, out_s, nullptr, hidden, 32, s_stride_row, s_stride_group, eps, 0};
  return launch_group_quant<false, kOutE2m1>(dtype, a, rows, as_stream(stream), "per_token_group_quant_mxfp4");
}

extern "C" int b200moe_silu_and_mul_quant(void* out, const void* in, b200moe_dtype dtype, const float* scale,
                                          int64_t rows, int d, b200moe_stream stream) {
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "silu_and_mul_quant: input must be float16 or bfloat16");
  B200_CHECK_ARG(rows >= 0 && d >= 0, "silu_and_mul_quant: bad sizes");
  if (rows == 0 || d == 0) return B200MOE_OK;
  B200_CHECK_ARG(out && in && scale, "silu_and_mul_quant: null pointer");
  const bool vec_ok = d % 8 == 0 && aligned16(in) && (((uintptr_t)out & 7) == 0);
  if (dtype == B200MOE_BF16)
    silu_mul_static_quant_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, as_stream(stream)>>>(
        (uint8_t*)out, (const __nv_bfloat16*)in, scale, d, vec_ok);
  else
    silu_mul_static_quant_kernel<__half><<<(unsigned)rows, 256, 0, as_stream(stream)>>>(
        (uint8_t*)out, (const __half*)in, scale, d, vec_ok);
  B200_LAUNCH_OK("silu_and_mul_quant");
  return B200MOE_OK;
}
