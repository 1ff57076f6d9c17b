// Plain-CUDA grouped GEMM over ragged expert segments: the checking kernel.
//
// It covers every weight format and epilogue of b200moe_grouped_gemm with the
// simplest possible schedule (64x64 tile per block, fp32 FMAs on dequantised
// operands) so that the tensor-core kernels can be compared against it on the
// GPU, and so that formats the tensor-core path does not yet take still run
// on the device.  It is not a performance path.
//
// Numerics follow csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:192-230, 394-419,
// 455-488 of vllm-xpu-kernels: weights are dequantised to the activation type
// (fp8 block: fp8 * scale rounded to that type; mxfp4: LUT * 2^(b-127)), fp32
// accumulate, per-tensor fp8 scale applied to the accumulator, bias added in
// fp32.  With fp8 activations the block-scaled sum
//   sum_kb (sum_{k in kb} a_q * w_q) * a_s[m,kb] * w_s[n/128,kb]
// is formed instead.
#include "common.cuh"

namespace b200moe {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

struct CheckArgs {
  const void* a; const float* a_scale; const void* w; const void* w_scale;
  const void* bias; void* d; const int32_t* rows_per_expert;
  int64_t m; int n, k, num_experts;
  int fmt, epi; float alpha, limit, clamp_limit;
  int w_experts;   // >0: segment s uses weight set s % w_experts
  int n_out;  // columns of D
  int group;  // INT4: K elements per scale
};

template <typename T>
__device__ __forceinline__ float round_to(float x) { return to_f32<T>(from_f32<T>(x)); }

// Dequantised weight element W_e[n, k] as the activation type would hold it.
template <typename T>
__device__ __forceinline__ float load_w(const CheckArgs& g, int e, int n, int k) {
  const int64_t N = g.n, K = g.k;
  switch (g.fmt) {
    case B200MOE_W_BF16_KN:
      return to_f32<T>(reinterpret_cast<const T*>(g.w)[((int64_t)e * K + k) * N + n]);
    case B200MOE_W_BF16_NK:
      return to_f32<T>(reinterpret_cast<const T*>(g.w)[((int64_t)e * N + n) * K + k]);
    case B200MOE_W_FP8_TENSOR_KN:
      return round_to<T>(e4m3_to_f32(reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * K + k) * N + n]));
    case B200MOE_W_FP8E5M2_TENSOR_KN:
      return round_to<T>(e5m2_to_f32(reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * K + k) * N + n]));
    case B200MOE_W_MXFP8_KN: {
      const uint8_t q = reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * K + k) * N + n];
      const uint8_t sb = reinterpret_cast<const uint8_t*>(g.w_scale)[((int64_t)e * (K / 32) + k / 32) * N + n];
      return round_to<T>(e4m3_to_f32(q) * e8m0_to_f32(sb));
    }
    case B200MOE_W_FP8_BLOCK_NK:
    case B200MOE_W_FP8_BLOCK_KN: {
      const uint8_t q = (g.fmt == B200MOE_W_FP8_BLOCK_NK)
                            ? reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * N + n) * K + k]
                            : reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * K + k) * N + n];
      if (g.a_scale != nullptr) return e4m3_to_f32(q);  // scales applied per block
      const float s = reinterpret_cast<const float*>(g.w_scale)[((int64_t)e * (N / 128) + n / 128) * (K / 128) + k / 128];
      return round_to<T>(e4m3_to_f32(q) * s);
    }
    case B200MOE_W_INT4_NK: {
      // two's-complement nibble times the group's scale, rounded to the activation type
      // (csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:400-410, 455-471 of the reference)
      const uint8_t b = reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * N + n) * (K / 2) + k / 2];
      const int q = (int)(((k & 1) ? (b >> 4) : (b & 15)) ^ 8) - 8;
      const float sc = to_f32<T>(reinterpret_cast<const T*>(g.w_scale)[((int64_t)e * N + n) * (K / g.group) + k / g.group]);
      return round_to<T>((float)q * sc);
    }
    case B200MOE_W_MXFP4_NK: {
      const uint8_t b = reinterpret_cast<const uint8_t*>(g.w)[((int64_t)e * N + n) * (K / 2) + k / 2];
      const uint32_t code = (k & 1) ? (b >> 4) : (b & 15);
      const uint8_t sb = reinterpret_cast<const uint8_t*>(g.w_scale)[((int64_t)e * N + n) * (K / 32) + k / 32];
      return round_to<T>(e2m1_to_f32(code) * e8m0_to_f32(sb));
    }
  }
  return 0.f;
}

template <typename T>
__device__ __forceinline__ float load_a(const CheckArgs& g, int64_t r, int k, bool a_fp8) {
  if (a_fp8) return e4m3_to_f32(reinterpret_cast<const uint8_t*>(g.a)[r * g.k + k]);
  return to_f32<T>(reinterpret_cast<const T*>(g.a)[r * g.k + k]);
}

// kPlanes = 2 for gated epilogues: plane 0 = gate rows of W, plane 1 = up rows.
template <typename T, int kPlanes>
__global__ void __launch_bounds__(256)
gemm_check_kernel(CheckArgs g, bool a_fp8) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Ws[kPlanes][TK][TN + 1];
  __shared__ int s_expert, s_row0, s_rows;

  // Find the expert segment and the row tile of this block.
  if (threadIdx.x == 0) {
    int tile = blockIdx.y, row0 = 0, found = -1, rows = 0;
    for (int e = 0; e < g.num_experts; ++e) {
      const int r = g.rows_per_expert[e];
      const int tiles = (r + TM - 1) / TM;
      if (tile < tiles) { found = e; row0 = row0 + tile * TM; rows = r - tile * TM; break; }
      tile -= tiles;
      row0 += r;
    }
    // from here on the index only selects weights, scales and bias
    s_expert = (found >= 0 && g.w_experts > 0) ? found % g.w_experts : found;
    s_row0 = row0; s_rows = rows < TM ? rows : TM;
  }
  __syncthreads();
  const int e = s_expert;
  if (e < 0) return;
  const int row0 = s_row0, rows = s_rows;
  const int n0 = blockIdx.x * TN;     // output column base (in units of D columns)
  const int n_out = g.n_out;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const bool block_scaled = a_fp8;
  const int I = g.n / 2;

  float acc[kPlanes][4][4];
  float part[kPlanes][4][4];
#pragma unroll
  for (int p = 0; p < kPlanes; ++p)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[p][i][j] = 0.f; part[p][i][j] = 0.f; }

  // W row that feeds output column c of plane p.
  auto w_row = [&](int c, int p) -> int {
    if (kPlanes == 1) return c;
    if (g.epi == B200MOE_EPI_SILU_MUL) return p == 0 ? c : I + c;
    return 2 * c + p;  // SwigluOAI: interleaved gate / up
  };

  for (int k0 = 0; k0 < g.k; k0 += TK) {
    for (int idx = threadIdx.x; idx < TM * TK; idx += 256) {
      const int kk = idx % TK, mm = idx / TK;
      float v = 0.f;
      if (mm < rows && k0 + kk < g.k) v = load_a<T>(g, row0 + mm, k0 + kk, a_fp8);
      As[kk][mm] = v;
    }
#pragma unroll
    for (int p = 0; p < kPlanes; ++p) {
      for (int idx = threadIdx.x; idx < TN * TK; idx += 256) {
        int kk, nn;
        if (g.fmt == B200MOE_W_BF16_KN || g.fmt == B200MOE_W_FP8_TENSOR_KN || g.fmt == B200MOE_W_FP8E5M2_TENSOR_KN ||
            g.fmt == B200MOE_W_FP8_BLOCK_KN || g.fmt == B200MOE_W_MXFP8_KN) {
          nn = idx % TN; kk = idx / TN;
        } else {
          kk = idx % TK; nn = idx / TK;
        }
        float v = 0.f;
        if (n0 + nn < n_out && k0 + kk < g.k) v = load_w<T>(g, e, w_row(n0 + nn, p), k0 + kk);
        Ws[p][kk][nn] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float av[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int p = 0; p < kPlanes; ++p) {
        float wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] = Ws[p][kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) part[p][i][j] = fmaf(av[i], wv[j], part[p][i][j]);
      }
    }
    __syncthreads();
    // Close a 128-wide K block: apply the block scales (fp8 x fp8) or just
    // move the partial sum over.
    if (((k0 + TK) % 128) == 0 || k0 + TK >= g.k) {
      const int kb = k0 / 128;
#pragma unroll
      for (int p = 0; p < kPlanes; ++p)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float s = 1.f;
            if (block_scaled) {
              const int mm = ty * 4 + i, c = n0 + tx * 4 + j;
              if (mm < rows && c < n_out) {
                const int wr = w_row(c, p);
                s = g.a_scale[(int64_t)(row0 + mm) * (g.k / 128) + kb] *
                    reinterpret_cast<const float*>(g.w_scale)[((int64_t)e * (g.n / 128) + wr / 128) * (g.k / 128) + kb];
              }
            }
            acc[p][i][j] = fmaf(part[p][i][j], s, acc[p][i][j]);
            part[p][i][j] = 0.f;
          }
    }
  }

  T* D = reinterpret_cast<T*>(g.d);
  const T* bias = reinterpret_cast<const T*>(g.bias);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int mm = ty * 4 + i;
    if (mm >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c >= n_out) continue;
      float v[kPlanes];
#pragma unroll
      for (int p = 0; p < kPlanes; ++p) {
        v[p] = acc[p][i][j];
        const int wr = w_row(c, p);
        if (g.fmt == B200MOE_W_FP8_TENSOR_KN || g.fmt == B200MOE_W_FP8E5M2_TENSOR_KN)
          v[p] *= reinterpret_cast<const float*>(g.w_scale)[e];
        if (bias != nullptr) v[p] += to_f32<T>(bias[(int64_t)e * g.n + wr]);
      }
      float out;
      if (kPlanes == 1) {
        out = v[0];
      } else {
        float gate = v[0], up = v[kPlanes - 1];
        if (g.clamp_limit > 0.f) {
          gate = fminf(gate, g.clamp_limit);
          up = fminf(fmaxf(up, -g.clamp_limit), g.clamp_limit);
        }
        if (g.epi == B200MOE_EPI_SILU_MUL) {
          out = gate / (1.0f + expf(-gate)) * up;
        } else {
          gate = fminf(gate, g.limit);
          up = fminf(fmaxf(up, -g.limit), g.limit);
          out = (up + 1.0f) * gate * (1.0f / (1.0f + expf(-gate * g.alpha)));
        }
      }
      D[(int64_t)(row0 + mm) * n_out + c] = from_f32<T>(out);
    }
  }
}

}  // namespace

int grouped_gemm_check(const b200moe_gemm_args* a, cudaStream_t st) {
  CheckArgs g;
  g.a = a->a; g.a_scale = reinterpret_cast<const float*>(a->a_scale); g.w = a->w; g.w_scale = a->w_scale; g.bias = a->bias;
  g.d = a->d; g.rows_per_expert = a->rows_per_expert; g.m = a->m; g.n = a->n; g.k = a->k;
  g.num_experts = a->num_experts; g.fmt = a->w_format; g.epi = a->epilogue;
  g.alpha = a->act_alpha; g.limit = a->act_limit; g.clamp_limit = a->clamp_limit;
  g.group = a->group_size > 0 ? a->group_size : 32;
  g.w_experts = (a->w_experts > 0 && a->w_experts != a->num_experts) ? a->w_experts : 0;
  const bool gated = a->epilogue != B200MOE_EPI_NONE;
  g.n_out = gated ? a->n / 2 : a->n;
  const bool a_fp8 = a->a_dtype == B200MOE_FP8_E4M3;
  const int64_t max_tiles = (a->m + TM - 1) / TM + a->num_experts;
  dim3 grid((g.n_out + TN - 1) / TN, (unsigned)max_tiles, 1);
  if (grid.y > 65535) return fail(B200MOE_E_UNSUPPORTED, "grouped_gemm (check kernel): too many rows");
  if (a->d_dtype == B200MOE_BF16) {
    if (gated) gemm_check_kernel<__nv_bfloat16, 2><<<grid, 256, 0, st>>>(g, a_fp8);
    else gemm_check_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(g, a_fp8);
  } else {
    if (gated) gemm_check_kernel<__half, 2><<<grid, 256, 0, st>>>(g, a_fp8);
    else gemm_check_kernel<__half, 1><<<grid, 256, 0, st>>>(g, a_fp8);
  }
  B200_LAUNCH_OK("gemm_check_kernel");
  return B200MOE_OK;
}

}  // namespace b200moe
