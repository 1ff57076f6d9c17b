// Router kernels: softmax / sigmoid / sqrt(softplus) top-k gating and group-limited top-k.
//
// One row (token) is handled by a power-of-two group of R <= 32 lanes; lane j
// owns the expert columns j, j+R, j+2R, ... so that global loads coalesce.  All
// reductions are xor-butterflies over the group, which makes every lane end up
// with the same value and fixes the floating-point summation order:
// per-lane partial sums in ascending column order, then masks R/2, R/4, .., 1.
// exp() and sigmoid() come from det_math.h, so the weights can be reproduced
// bit-for-bit on a CPU.
//
// Behaviour follows csrc/moe/topk.cpp:395-583 (gating),
// csrc/moe/topk_softplus_sqrt_kernels.cpp:205-400 (sqrt-softplus gating) and
// csrc/moe/grouped_topk.cpp:404-447, 525-678 (grouped) of vllm-xpu-kernels.
#include "common.cuh"
#include "det_math.h"

namespace b200moe {
namespace {

constexpr int kWarpsPerBlock = 4;

__device__ __forceinline__ void store_index(void* base, b200moe_dtype dt,
                                            int64_t pos, int value) {
  if (dt == B200MOE_I64) {
    reinterpret_cast<int64_t*>(base)[pos] = value;
  } else {  // I32 and U32 share the bit pattern for non-negative ids
    reinterpret_cast<int32_t*>(base)[pos] = value;
  }
}

// R lanes per row, VPT columns per lane.  E <= R * VPT.
// kMode 0: softmax, 1: sigmoid, 2: sqrt(softplus) (its weight is the biased
// score minus the bias again, as the reference computes it).
template <typename T, int R, int VPT, int kMode>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
topk_gating_kernel(const T* __restrict__ gating, float* __restrict__ out_w,
                   void* __restrict__ out_idx, b200moe_dtype idx_dtype,
                   int32_t* __restrict__ out_src, const float* __restrict__ bias,
                   int64_t num_rows, int E, int K, bool renorm, float rsf) {
  constexpr int kRowsPerWarp = 32 / R;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane % R;
  const int64_t row = ((int64_t)blockIdx.x * kWarpsPerBlock + warp) * kRowsPerWarp + lane / R;
  // Rows past the end still run the shuffles (with dummy data) so that every
  // lane of the warp takes part in them.
  const bool live = row < num_rows;
  const T* src = gating + (live ? row : 0) * (int64_t)E;

  float p[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = sub + i * R;
    p[i] = (c < E) ? to_f32<T>(src[c]) : -INFINITY;
  }

  if (kMode == 0) {
    float m = p[0];
#pragma unroll
    for (int i = 1; i < VPT; ++i) m = fmaxf(m, p[i]);
#pragma unroll
    for (int mask = R / 2; mask > 0; mask >>= 1)
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, mask));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = sub + i * R;
      p[i] = (c < E) ? dm_expf(__fsub_rn(p[i], m)) : 0.f;
      s = __fadd_rn(s, p[i]);
    }
#pragma unroll
    for (int mask = R / 2; mask > 0; mask >>= 1)
      s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, mask));
    const float rs = __fdiv_rn(1.f, s);
#pragma unroll
    for (int i = 0; i < VPT; ++i) p[i] = __fmul_rn(p[i], rs);
  } else if (kMode == 1) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = sub + i * R;
      // The sigmoid is rounded through the input type, as the reference does.
      p[i] = (c < E) ? to_f32<T>(from_f32<T>(dm_sigmoidf(p[i]))) : 0.f;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = sub + i * R;
      p[i] = (c < E) ? dm_softplus_sqrtf(p[i]) : 0.f;
    }
  }

  float v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = sub + i * R;
    if (c < E) {
      v[i] = (bias != nullptr) ? __fadd_rn(p[i], bias[c]) : p[i];
    } else {
      v[i] = -INFINITY;
    }
  }

  float sum_val = 0.f;
  for (int k = 0; k < K; ++k) {
    float best_v = v[0];
    float best_p = p[0];
    int best_i = 0;
#pragma unroll
    for (int i = 1; i < VPT; ++i) {
      if (v[i] > best_v) { best_v = v[i]; best_p = p[i]; best_i = i; }
    }
    const int local_e = sub + best_i * R;
    int e = local_e;
#pragma unroll
    for (int mask = R / 2; mask > 0; mask >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, mask);
      const float op = __shfl_xor_sync(0xffffffffu, best_p, mask);
      const int oe = __shfl_xor_sync(0xffffffffu, e, mask);
      if (ov > best_v || (ov == best_v && oe < e)) { best_v = ov; best_p = op; e = oe; }
    }
    if (kMode == 2 && bias != nullptr) best_p = __fsub_rn(best_v, bias[e]);
    sum_val = __fadd_rn(sum_val, best_p);
    if (live && sub == 0) {
      const int64_t pos = row * K + k;
      store_index(out_idx, idx_dtype, pos, e);
      out_src[pos] = (int32_t)((int64_t)k * num_rows + row);
      out_w[pos] = best_p;  // rescaled below
    }
    if (e == local_e) {
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        if (i == best_i) v[i] = -10000.f;
    }
  }
  if (live && sub == 0) {
    float scale = rsf;
    if (renorm) scale = __fdiv_rn(scale, sum_val > 0.f ? sum_val : 1.f);
    for (int k = 0; k < K; ++k) {
      const int64_t pos = row * K + k;
      out_w[pos] = __fmul_rn(out_w[pos], scale);
    }
  }
}

template <typename T, int kMode>
int launch_gating(const T* gating, float* w, void* idx, b200moe_dtype idx_dtype,
                  int32_t* src, const float* bias, int64_t T_, int E, int K,
                  bool renorm, float rsf, cudaStream_t st) {
#define B200_GATING_CASE(R_, VPT_)                                              \
  {                                                                             \
    constexpr int rows_per_block = kWarpsPerBlock * (32 / R_);                  \
    const unsigned grid = (unsigned)((T_ + rows_per_block - 1) / rows_per_block); \
    topk_gating_kernel<T, R_, VPT_, kMode>                                      \
        <<<grid, kWarpsPerBlock * 32, 0, st>>>(gating, w, idx, idx_dtype, src,  \
                                               bias, T_, E, K, renorm, rsf);    \
  }
  if (E <= 1) B200_GATING_CASE(1, 1)
  else if (E <= 2) B200_GATING_CASE(2, 1)
  else if (E <= 4) B200_GATING_CASE(4, 1)
  else if (E <= 8) B200_GATING_CASE(8, 1)
  else if (E <= 16) B200_GATING_CASE(16, 1)
  else if (E <= 32) B200_GATING_CASE(32, 1)
  else if (E <= 64) B200_GATING_CASE(32, 2)
  else if (E <= 128) B200_GATING_CASE(32, 4)
  else if (E <= 256) B200_GATING_CASE(32, 8)
  else if (E <= 512) B200_GATING_CASE(32, 16)
  else B200_GATING_CASE(32, 32)
#undef B200_GATING_CASE
  B200_LAUNCH_OK("topk_gating_kernel");
  return B200MOE_OK;
}

int gating_entry(int mode, float* topk_weights, void* topk_indices,
                 b200moe_dtype index_dtype, int32_t* token_expert_indices,
                 const void* gating, b200moe_dtype gating_dtype,
                 int64_t num_tokens, int num_experts, int topk, int renormalize,
                 const float* bias, double rsf, b200moe_stream stream) {
  const char* name = mode == 0 ? "topk_softmax" : (mode == 1 ? "topk_sigmoid" : "topk_softplus_sqrt");
  B200_CHECK_ARG(index_dtype == B200MOE_I32 || index_dtype == B200MOE_U32 ||
                     index_dtype == B200MOE_I64,
                 "%s: topk_indices must be int32, uint32 or int64", name);
  B200_CHECK_ARG(num_experts >= 1 && num_experts <= 1024,
                 "%s: num_experts must be in [1, 1024], got %d", name, num_experts);
  B200_CHECK_ARG(topk >= 1 && topk <= num_experts,
                 "%s: topk must be in [1, num_experts], got %d", name, topk);
  B200_CHECK_ARG(num_tokens >= 0, "%s: negative num_tokens", name);
  if (num_tokens == 0) return B200MOE_OK;
  B200_CHECK_ARG(topk_weights && topk_indices && token_expert_indices && gating,
                 "%s: null pointer", name);
  cudaStream_t st = as_stream(stream);
  B200_DISPATCH_FLOAT(gating_dtype, name, {
    if (mode == 0)
      return launch_gating<scalar_t, 0>(
          (const scalar_t*)gating, topk_weights, topk_indices, index_dtype,
          token_expert_indices, bias, num_tokens, num_experts, topk,
          renormalize != 0, (float)rsf, st);
    if (mode == 2)
      return launch_gating<scalar_t, 2>(
          (const scalar_t*)gating, topk_weights, topk_indices, index_dtype,
          token_expert_indices, bias, num_tokens, num_experts, topk,
          renormalize != 0, (float)rsf, st);
    return launch_gating<scalar_t, 1>(
        (const scalar_t*)gating, topk_weights, topk_indices, index_dtype,
        token_expert_indices, bias, num_tokens, num_experts, topk,
        renormalize != 0, (float)rsf, st);
  });
  return B200MOE_OK;
}

// ---------------------------------------------------------------------------
// Group-limited top-k: one warp per token, all columns in registers.
// ---------------------------------------------------------------------------
template <typename T, int VPT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
grouped_topk_kernel(const T* __restrict__ scores, const T* __restrict__ swb,
                    T* __restrict__ out_val, int32_t* __restrict__ out_idx,
                    int64_t num_tokens, int E, int n_group, int topk_group, int K,
                    bool renorm, double rsf) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (tok >= num_tokens) return;  // whole warp leaves together
  const int G = E / n_group;
  const T* sb = swb + tok * (int64_t)E;
  const T* sc = scores + tok * (int64_t)E;

  float v[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    v[i] = (c < E) ? to_f32<T>(sb[c]) : -INFINITY;
  }

  // Score of group g = sum of its two largest biased scores, kept by lane g,
  // rounded through T as the reference stores it in that type.
  float my_gs = -INFINITY;
  for (int g = 0; g < n_group; ++g) {
    float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < E && c / G == g) {
        const float x = v[i];
        if (x > m1) { m2 = m1; m1 = x; }
        else if (x > m2) { m2 = x; }
      }
    }
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, m1, mask);
      const float o2 = __shfl_xor_sync(0xffffffffu, m2, mask);
      const float n1 = fmaxf(m1, o1);
      const float n2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
      m1 = n1; m2 = n2;
    }
    const float gs = to_f32<T>(from_f32<T>(__fadd_rn(m1, m2)));
    if (lane == g) my_gs = gs;
  }

  // Threshold search: knock out the current maximum (all lanes equal to it)
  // until at least topk_group groups are gone.  Lanes >= n_group count as
  // already knocked out.
  float value = (lane < n_group && isfinite(my_gs)) ? my_gs : -INFINITY;
  const int target = 32 - n_group + topk_group;
  int count = 32 - n_group;
  int pre_count = 0;
  float thr = -INFINITY;
  for (int it = 0; it < 32 && count < target; ++it) {
    float mx = value;
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1)
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, mask));
    thr = mx;
    if (value == mx) value = -INFINITY;
    pre_count = count;
    count = __popc(__ballot_sync(0xffffffffu, value == -INFINITY));
  }
  const int num_equal_allowed = target - pre_count;
  const bool proceed = (thr != -INFINITY);

  if (!proceed) {
    for (int i = lane; i < K; i += 32) {
      out_idx[tok * K + i] = i;
      out_val[tok * K + i] = from_f32<T>(1.0f / (float)K);
    }
    return;
  }

  // Which groups survive: score > thr, or == thr for the first
  // num_equal_allowed such groups in index order.
  uint32_t keep_mask = 0;
  {
    const uint32_t gt = __ballot_sync(0xffffffffu, lane < n_group && my_gs > thr);
    const uint32_t eq = __ballot_sync(0xffffffffu, lane < n_group && my_gs == thr);
    keep_mask = gt;
    int taken = 0;
    for (int g = 0; g < n_group; ++g) {
      if ((eq >> g) & 1u) {
        if (taken < num_equal_allowed) keep_mask |= (1u << g);
        ++taken;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    const bool ok = (c < E) && ((keep_mask >> (c / G)) & 1u) && isfinite(v[i]);
    if (!ok) v[i] = -INFINITY;
  }

  // K rounds of arg-max; ties go to the lower expert id.
  uint32_t taken_bits = 0;
  int my_id = 0;  // lane k keeps the k-th id
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
    int bi = -1;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < E && !((taken_bits >> i) & 1u)) {
        if (bi < 0 || v[i] > bv) { bv = v[i]; be = c; bi = i; }
      }
    }
    const int local_e = be;
#pragma unroll
    for (int mask = 16; mask > 0; mask >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, mask);
      const int oe = __shfl_xor_sync(0xffffffffu, be, mask);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
    }
    if (be == local_e && bi >= 0) taken_bits |= (1u << bi);
    if (lane == k) my_id = be;
  }

  float w = 0.f;
  if (lane < K) w = to_f32<T>(sc[my_id]);
  float s = w;
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1)
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, mask));
  const float topk_sum = __fadd_rn(1e-20f, s);
  if (lane < K) {
    float r;
    if (renorm) r = (float)((double)__fdiv_rn(w, topk_sum) * rsf);
    else r = (float)((double)w * rsf);
    out_idx[tok * K + lane] = my_id;
    out_val[tok * K + lane] = from_f32<T>(r);
  }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_topk_softmax(float* topk_weights, void* topk_indices,
                                    b200moe_dtype index_dtype,
                                    int32_t* token_expert_indices,
                                    const void* gating,
                                    b200moe_dtype gating_dtype,
                                    int64_t num_tokens, int num_experts, int topk,
                                    int renormalize, const float* bias,
                                    b200moe_stream stream) {
  return gating_entry(0, topk_weights, topk_indices, index_dtype,
                      token_expert_indices, gating, gating_dtype, num_tokens,
                      num_experts, topk, renormalize, bias, 1.0, stream);
}

extern "C" int b200moe_topk_sigmoid(float* topk_weights, void* topk_indices,
                                    b200moe_dtype index_dtype,
                                    int32_t* token_expert_indices,
                                    const void* gating,
                                    b200moe_dtype gating_dtype,
                                    int64_t num_tokens, int num_experts, int topk,
                                    int renormalize, const float* bias,
                                    double routed_scaling_factor,
                                    b200moe_stream stream) {
  return gating_entry(1, topk_weights, topk_indices, index_dtype,
                      token_expert_indices, gating, gating_dtype, num_tokens,
                      num_experts, topk, renormalize, bias,
                      routed_scaling_factor, stream);
}

extern "C" int b200moe_grouped_topk(void* topk_values, int32_t* topk_indices,
                                    const void* scores,
                                    const void* scores_with_bias,
                                    b200moe_dtype dtype, int64_t num_tokens,
                                    int num_experts, int n_group, int topk_group,
                                    int topk, int renormalize,
                                    double routed_scaling_factor,
                                    b200moe_stream stream) {
  B200_CHECK_ARG(n_group >= 1 && num_experts % n_group == 0,
                 "num_experts should be divisible by n_group");
  B200_CHECK_ARG(n_group <= 32,
                 "n_group should be smaller than or equal to 32 for now");
  B200_CHECK_ARG(topk >= 1 && topk <= 32,
                 "topk should be smaller than or equal to 32 for now");
  B200_CHECK_ARG(topk_group >= 1 && topk_group <= n_group,
                 "grouped_topk: topk_group must be in [1, n_group]");
  B200_CHECK_ARG(num_experts >= 1 && num_experts <= 1024,
                 "grouped_topk: num_experts must be in [1, 1024]");
  B200_CHECK_ARG(topk <= num_experts, "grouped_topk: topk exceeds num_experts");
  if (num_tokens == 0) return B200MOE_OK;
  B200_CHECK_ARG(topk_values && topk_indices && scores && scores_with_bias,
                 "grouped_topk: null pointer");
  cudaStream_t st = as_stream(stream);
  const unsigned grid = (unsigned)((num_tokens + kWarpsPerBlock - 1) / kWarpsPerBlock);
#define B200_GT_CASE(VPT_)                                                     \
  grouped_topk_kernel<scalar_t, VPT_><<<grid, kWarpsPerBlock * 32, 0, st>>>(   \
      (const scalar_t*)scores, (const scalar_t*)scores_with_bias,              \
      (scalar_t*)topk_values, topk_indices, num_tokens, num_experts, n_group,  \
      topk_group, topk, renormalize != 0, routed_scaling_factor)
  switch (dtype) {
    case B200MOE_F32: case B200MOE_F16: case B200MOE_BF16: break;
    default:
      return fail(B200MOE_E_BADARG,
                  "Invalid dtype, only supports float16, float32, and bfloat16");
  }
  B200_DISPATCH_FLOAT(dtype, "grouped_topk", {
    if (num_experts <= 32) B200_GT_CASE(1);
    else if (num_experts <= 64) B200_GT_CASE(2);
    else if (num_experts <= 128) B200_GT_CASE(4);
    else if (num_experts <= 256) B200_GT_CASE(8);
    else if (num_experts <= 512) B200_GT_CASE(16);
    else B200_GT_CASE(32);
  });
#undef B200_GT_CASE
  B200_LAUNCH_OK("grouped_topk_kernel");
  return B200MOE_OK;
}

namespace b200moe {
namespace {
__device__ __forceinline__ int64_t load_index(const void* base, b200moe_dtype dt, int64_t pos) {
  if (dt == B200MOE_I64) return reinterpret_cast<const int64_t*>(base)[pos];
  if (dt == B200MOE_U32) return reinterpret_cast<const uint32_t*>(base)[pos];
  return reinterpret_cast<const int32_t*>(base)[pos];
}

// Hash routing (csrc/moe/topk_softplus_sqrt_kernels.cpp:238-301): the expert ids of
// a token come from row input_ids[t] of the table tid2eid [vocab, K]; weights
// are sqrt(softplus(logit)) of those experts (non-finite -> 0), renormalised
// in k order.  One thread per token.
template <typename T>
__global__ void __launch_bounds__(128)
softplus_sqrt_hash_kernel(const T* __restrict__ gating, float* __restrict__ out_w,
                          void* __restrict__ out_idx, b200moe_dtype idx_dtype,
                          int32_t* __restrict__ out_src, const void* __restrict__ input_ids,
                          const void* __restrict__ tid2eid, int64_t num_rows, int E, int K,
                          bool renorm, float rsf) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= num_rows) return;
  const int64_t tok = load_index(input_ids, idx_dtype, row);
  float sum = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = (int)load_index(tid2eid, idx_dtype, tok * K + k);
    float w = 0.f;
    if (e >= 0 && e < E) {
      w = dm_softplus_sqrtf(to_f32<T>(gating[row * (int64_t)E + e]));
      if (!isfinite(w)) w = 0.f;
    }
    const int64_t pos = row * K + k;
    out_w[pos] = w;
    store_index(out_idx, idx_dtype, pos, (e >= 0 && e < E) ? e : E);
    out_src[pos] = (int32_t)((int64_t)k * num_rows + row);
    if (renorm) sum = __fadd_rn(sum, w);
  }
  float scale = rsf;
  if (renorm) scale = __fdiv_rn(scale, sum > 0.f ? sum : 1.f);
  for (int k = 0; k < K; ++k) out_w[row * K + k] = __fmul_rn(out_w[row * K + k], scale);
}
}  // namespace
}  // namespace b200moe

extern "C" int b200moe_topk_softplus_sqrt(float* topk_weights, void* topk_indices,
                                          b200moe_dtype index_dtype, int32_t* token_expert_indices,
                                          const void* gating, b200moe_dtype gating_dtype,
                                          int64_t num_tokens, int num_experts, int topk, int renormalize,
                                          double routed_scaling_factor, const float* correction_bias,
                                          const void* input_ids, const void* tid2eid,
                                          b200moe_stream stream) {
  if (tid2eid == nullptr)
    return gating_entry(2, topk_weights, topk_indices, index_dtype, token_expert_indices, gating,
                        gating_dtype, num_tokens, num_experts, topk, renormalize, correction_bias,
                        routed_scaling_factor, stream);
  B200_CHECK_ARG(input_ids != nullptr, "input_ids is required for hash MoE");
  B200_CHECK_ARG(index_dtype == B200MOE_I32 || index_dtype == B200MOE_U32 || index_dtype == B200MOE_I64,
                 "topk_softplus_sqrt: topk_indices must be int32, uint32 or int64");
  B200_CHECK_ARG(num_experts >= 1 && topk >= 1 && num_tokens >= 0, "topk_softplus_sqrt: bad sizes");
  if (num_tokens == 0) return B200MOE_OK;
  B200_CHECK_ARG(topk_weights && topk_indices && token_expert_indices && gating, "topk_softplus_sqrt: null pointer");
  const unsigned grid = (unsigned)((num_tokens + 127) / 128);
  B200_DISPATCH_FLOAT(gating_dtype, "topk_softplus_sqrt", {
    b200moe::softplus_sqrt_hash_kernel<scalar_t><<<grid, 128, 0, b200moe::as_stream(stream)>>>(
        (const scalar_t*)gating, topk_weights, topk_indices, index_dtype, token_expert_indices, input_ids,
        tid2eid, num_tokens, num_experts, topk, renormalize != 0, (float)routed_scaling_factor);
  });
  B200_LAUNCH_OK("softplus_sqrt_hash_kernel");
  return B200MOE_OK;
}
