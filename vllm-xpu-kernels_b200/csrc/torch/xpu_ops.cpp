// torch.ops._xpu_C.cutlass_grouped_gemm_interface (schema of
// csrc/xpu/torch_bindings.cpp:46-53 in vllm-xpu-kernels) and the extended
// form the Python layer uses (explicit weight layout, fused gated epilogue).
// Weight format detection and the argument checks follow
// csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:174-243, 267-287,
// 322-383, 397-398.
#include "shim.h"

#include <mutex>

using namespace b200shim;

namespace {

// One status word per device, in pinned host memory that the device can write and the host
// can read without a synchronisation.  A grouped GEMM whose bounded wait ran out sets it to 1
// (b200moe_gemm_args.status); the next grouped-GEMM call on that device, or an explicit
// b200_check_status, raises and clears it.  Allocated on first use, kept for the process.
constexpr int kMaxStatusDevices = 64;
std::mutex g_status_mutex;
at::Tensor g_status[kMaxStatusDevices];

int32_t* device_status_word(int device) {
  TORCH_CHECK(device >= 0 && device < kMaxStatusDevices, "device index out of range");
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status[device].defined()) {
    g_status[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCPU).pinned_memory(true));
  }
  return g_status[device].data_ptr<int32_t>();
}

void raise_if_timed_out(int32_t* word) {
  volatile int32_t* w = word;
  if (*w != 0) {
    *w = 0;
    check_status(b200moe_status_to_code(1));
  }
}

// layout: 0 = as the reference infers it from shapes, 1 = [E,N,K], 2 = [E,K,N]
at::Tensor grouped_gemm_impl(at::Tensor& ptr_A, const std::optional<at::Tensor>& ptr_A_scale,
                             at::Tensor& ptr_B, const std::optional<at::Tensor>& ptr_B_scale,
                             const std::optional<at::Tensor>& ptr_bias, at::Tensor& ptr_D,
                             at::Tensor& rows_per_expert, int64_t N, int64_t K, int64_t num_experts,
                             int64_t layout, int64_t epilogue, double alpha, double limit,
                             double clamp_limit, int64_t impl, int64_t max_ctas, bool allow_segments,
                             int64_t rows_hint = 0, const std::optional<at::Tensor>& ptr_D_scale = std::nullopt,
                             bool mid_f16 = false) {
  check_cuda(ptr_A, "ptr_A");
  const auto A_dtype = ptr_A.scalar_type();
  const auto B_dtype = ptr_B.scalar_type();
  const bool is_weight_fp8 = (B_dtype == at::kFloat8_e4m3fn) || (B_dtype == at::kFloat8_e5m2);
  const bool is_B_mxfp4 = (B_dtype == at::kFloat4_e2m1fn_x2) && ptr_B_scale.has_value();
  const bool is_B_int4 = (B_dtype == at::kChar) && ptr_B_scale.has_value();
  // fp8 weights with one-byte (e8m0) scales: the "mxfp8" recipe of
  // vllm_xpu_kernels/fused_moe_interface.py:47-61, weights [E,K,N], scales [E,K/32,N]
  const bool is_B_mxfp8 = is_weight_fp8 && ptr_B_scale.has_value() && ptr_B_scale->element_size() == 1;
  const bool is_B_fp8_block = is_weight_fp8 && !is_B_mxfp8 && ptr_B_scale.has_value() && ptr_B_scale->dim() == 3;

  TORCH_CHECK(N % 8 == 0, "N must be divisible by 8");
  TORCH_CHECK(ptr_A.dim() == 2, "ptr_A must be 2D [Total_M, K]");
  TORCH_CHECK(ptr_B.dim() == 3, "ptr_B must be 3D");
  TORCH_CHECK(ptr_D.dim() == 2, "ptr_D must be 2D [Total_M, N]");
  if (ptr_bias.has_value()) TORCH_CHECK(ptr_bias->dim() == 2, "ptr_bias must be 2D [num_experts, N]");
  TORCH_CHECK(ptr_A.is_contiguous(), "ptr_A must be contiguous");
  TORCH_CHECK(ptr_B.is_contiguous(), "ptr_B must be contiguous");
  TORCH_CHECK(ptr_D.is_contiguous(), "ptr_D must be contiguous");
  if (ptr_bias.has_value()) TORCH_CHECK(ptr_bias->is_contiguous(), "ptr_bias must be contiguous");

  const int64_t A_total_M = ptr_A.size(0), A_K = ptr_A.size(1);
  const int64_t B_E = ptr_B.size(0);
  int64_t B_K = ptr_B.size(1), B_N = ptr_B.size(2);
  b200moe_weight_format fmt;
  if (is_B_int4) {
    B_K = ptr_B.size(2) * 2; B_N = ptr_B.size(1);
    fmt = B200MOE_W_INT4_NK;
  } else if (is_B_mxfp4) {
    B_K = ptr_B.size(2) * 2; B_N = ptr_B.size(1);
    fmt = B200MOE_W_MXFP4_NK;
  } else if (is_B_mxfp8) {
    fmt = B200MOE_W_MXFP8_KN;
  } else if (is_B_fp8_block) {
    const bool nk = ptr_B.size(1) == N && ptr_B.size(2) == K;
    const bool kn = N != K && ptr_B.size(1) == K && ptr_B.size(2) == N;
    TORCH_CHECK(nk || kn, "block FP8 ptr_B must be [num_experts, N, K] or [num_experts, K, N] (N=", N,
                ", K=", K, "), got ", ptr_B.sizes());
    B_K = K; B_N = N;
    fmt = kn ? B200MOE_W_FP8_BLOCK_KN : B200MOE_W_FP8_BLOCK_NK;
    if (layout == 1) fmt = B200MOE_W_FP8_BLOCK_NK;
    if (layout == 2) fmt = B200MOE_W_FP8_BLOCK_KN;
  } else if (is_weight_fp8) {
    fmt = B_dtype == at::kFloat8_e5m2 ? B200MOE_W_FP8E5M2_TENSOR_KN : B200MOE_W_FP8_TENSOR_KN;
  } else {
    fmt = B200MOE_W_BF16_KN;
    if (layout == 1) { fmt = B200MOE_W_BF16_NK; B_K = ptr_B.size(2); B_N = ptr_B.size(1); }
  }
  const int64_t D_total_M = ptr_D.size(0), D_N = ptr_D.size(1);
  const int64_t n_out = epilogue ? N / 2 : N;
  TORCH_CHECK(B_E == num_experts, "ptr_B.size(0) must match num_experts");
  // Extended op only: rows_per_expert may hold a multiple of num_experts segments; segment s
  // then multiplies with weight set s % num_experts (b200moe_gemm_args.w_experts).
  const int64_t segments = rows_per_expert.numel();
  TORCH_CHECK(rows_per_expert.scalar_type() == at::kInt && rows_per_expert.is_contiguous() &&
              (segments == num_experts || (allow_segments && segments > 0 && segments % num_experts == 0)),
              "rows_per_expert must be int32 [num_experts]");
  TORCH_CHECK(A_total_M == D_total_M || ((is_B_mxfp4 || (is_weight_fp8 && !is_B_fp8_block)) && A_dtype == at::kFloat8_e4m3fn && A_total_M == 2 * D_total_M),
              "ptr_A.size(0) must match ptr_D.size(0)");
  TORCH_CHECK(A_K == B_K && B_K == K, "ptr_A K dimension must match ptr_B logical K dimension and K");
  TORCH_CHECK(B_N == N && D_N == n_out, "ptr_B logical N dimension must match ptr_D N dimension and N");
  if (ptr_bias.has_value()) {
    TORCH_CHECK(ptr_bias->size(0) == num_experts, "ptr_bias.size(0) must match num_experts");
    TORCH_CHECK(ptr_bias->size(1) == N, "ptr_bias.size(1) must match N");
    TORCH_CHECK(ptr_bias->scalar_type() == ptr_D.scalar_type() ||
                    (ptr_D.scalar_type() == at::kFloat8_e4m3fn &&
                     ptr_bias->scalar_type() == (mid_f16 ? at::kHalf : at::kBFloat16)),
                "ptr_bias must have ptr_D's dtype");
  }
  int64_t group_size = 0;
  if (is_B_int4) {
    TORCH_CHECK(ptr_B_scale->is_contiguous(), "ptr_scales must be contiguous");
    TORCH_CHECK(ptr_B_scale->dim() == 3, "ptr_scales of int4 must be 3D [num_experts, group_num, N]");
    TORCH_CHECK(ptr_B_scale->size(0) == num_experts, "ptr_scales.size(0) of int4 must match num_experts");
    TORCH_CHECK(K % ptr_B_scale->size(2) == 0, "ptr_scales.size(2) of int4 must be divisible by K");
    TORCH_CHECK(ptr_B_scale->size(1) == N, "ptr_scales.size(1) of int4 must match N");
    group_size = K / ptr_B_scale->size(2);
    TORCH_CHECK(group_size == 32 || group_size == 64 || group_size == 128 || group_size == 256,
                "group_size must be 32, 64, 128 or 256");
    TORCH_CHECK(ptr_B_scale->scalar_type() == A_dtype, "int4 scales must have the activation dtype");
  } else if (is_B_mxfp4) {
    TORCH_CHECK(ptr_B_scale->is_contiguous(), "ptr_scales must be contiguous");
    TORCH_CHECK(ptr_B_scale->dim() == 3, "ptr_scales of int4 must be 3D [num_experts, group_num, N]");
    TORCH_CHECK(ptr_B_scale->size(0) == num_experts, "ptr_scales.size(0) of int4 must match num_experts");
    TORCH_CHECK(ptr_B_scale->size(1) == N, "ptr_scales.size(1) of int4 must match N");
    TORCH_CHECK(ptr_B_scale->size(2) * 32 == K, "group_size must be 32, 64, 128 or 256");
    TORCH_CHECK(ptr_B_scale->element_size() == 1, "mxfp4 scales must be e8m0 bytes");
  } else if (is_B_mxfp8) {
    TORCH_CHECK(B_dtype == at::kFloat8_e4m3fn, "mxfp8 grouped GEMM only supports float8_e4m3fn weights");
    TORCH_CHECK(ptr_B_scale->is_contiguous(), "ptr_scales must be contiguous");
    TORCH_CHECK(K % 32 == 0 && ptr_B_scale->dim() == 3 && ptr_B_scale->size(0) == num_experts &&
                ptr_B_scale->size(1) == K / 32 && ptr_B_scale->size(2) == N,
                "mxfp8 scales must have shape [num_experts, K / 32, N]");
  } else if (is_weight_fp8) {
    TORCH_CHECK(ptr_B_scale.has_value(), "w8a16 grouped gemm must have scales");
    TORCH_CHECK(ptr_B_scale->is_contiguous(), "ptr_scales must be contiguous");
    TORCH_CHECK(ptr_B_scale->scalar_type() == at::kFloat, "ptr_scales must be float");
    if (is_B_fp8_block) {
      TORCH_CHECK(B_dtype == at::kFloat8_e4m3fn, "block-scaled grouped GEMM only supports float8_e4m3fn weights");
      TORCH_CHECK(N % 128 == 0 && K % 128 == 0, "block-scaled grouped GEMM requires N and K divisible by 128");
      TORCH_CHECK(ptr_B_scale->size(0) == num_experts && ptr_B_scale->size(1) == N / 128 &&
                  ptr_B_scale->size(2) == K / 128,
                  "block scales must have shape [num_experts, N / 128, K / 128]");
    } else {
      TORCH_CHECK(ptr_B_scale->dim() == 1, "ptr_scales of fp8 must be 1D [num_experts]");
      TORCH_CHECK(ptr_B_scale->size(0) == num_experts, "ptr_scales.size(0) of fp8 must match num_experts");
    }
  } else {
    TORCH_CHECK(!ptr_B_scale.has_value(), "w16a16 grouped gemm must not have scales");
    TORCH_CHECK(B_dtype == A_dtype, "w16a16 grouped gemm needs weights of the activation dtype");
  }

  b200moe_gemm_args g = {};
  g.a = ptr_A.data_ptr();
  if (A_dtype == at::kFloat8_e4m3fn) {
    TORCH_CHECK((is_weight_fp8 || is_B_mxfp4) && ptr_A_scale.has_value(),
                "fp8 activations need fp8 or mxfp4 weights and ptr_A_scale");
    g.a_dtype = B200MOE_FP8_E4M3;
    if (is_B_mxfp4 || !is_B_fp8_block) {
      // ptr_A [planes * Total_M, K] (planes = 1 or 2, the second the residual), scales
      // int32 [planes, ceil(K / 128), Total_M]: the outputs of _C::b200_quant_mxfp8.
      const int64_t planes = A_total_M / D_total_M;
      TORCH_CHECK((planes == 1 || planes == 2) && planes * D_total_M == A_total_M,
                  "ptr_A must hold one or two planes of ptr_D.size(0) rows");
      TORCH_CHECK(ptr_A_scale->scalar_type() == at::kInt && ptr_A_scale->is_contiguous() &&
                  ptr_A_scale->dim() == 3 && ptr_A_scale->size(0) == planes &&
                  ptr_A_scale->size(1) == (K + 127) / 128 && ptr_A_scale->size(2) == D_total_M,
                  "ptr_A_scale must be int32 [planes, ceil(K / 128), Total_M]");
      if (planes == 2) g.a_dtype = B200MOE_FP8_E4M3_X2;
    } else {
      TORCH_CHECK(ptr_A_scale->scalar_type() == at::kFloat && ptr_A_scale->is_contiguous() &&
                  ptr_A_scale->dim() == 2 && ptr_A_scale->size(0) == A_total_M &&
                  ptr_A_scale->size(1) == K / 128, "ptr_A_scale must be float32 [Total_M, K / 128]");
    }
    g.a_scale = ptr_A_scale->data_ptr();
  } else {
    TORCH_CHECK(A_dtype == at::kBFloat16 || A_dtype == at::kHalf, "ptr_A must be bfloat16, float16 or float8_e4m3fn");
    TORCH_CHECK(A_dtype == ptr_D.scalar_type(), "ptr_A and ptr_D must have the same dtype");
    g.a_dtype = A_dtype == at::kBFloat16 ? B200MOE_BF16 : B200MOE_F16;
  }
  const bool d_quant = ptr_D.scalar_type() == at::kFloat8_e4m3fn;
  TORCH_CHECK(ptr_D.scalar_type() == at::kBFloat16 || ptr_D.scalar_type() == at::kHalf || d_quant,
              "ptr_D must be bfloat16 or float16");
  if (d_quant) {
    // extended op only: quantised output of the fused SiLU epilogue, scales [Total_M, N / 256]
    TORCH_CHECK(allow_segments && epilogue == 1 && ptr_D_scale.has_value() && is_B_fp8_block &&
                A_dtype == at::kFloat8_e4m3fn, "float8_e4m3fn ptr_D needs the SiLU epilogue, ptr_D_scale, fp8 "
                "activations and block-scaled fp8 weights");
    TORCH_CHECK(N % 256 == 0 && ptr_D_scale->scalar_type() == at::kFloat && ptr_D_scale->is_contiguous() &&
                ptr_D_scale->numel() == D_total_M * (N / 256), "ptr_D_scale must be float32 [Total_M, N / 256]");
  }
  g.w = ptr_B.data_ptr();
  g.w_format = fmt;
  g.w_scale = ptr_B_scale.has_value() ? ptr_B_scale->data_ptr() : nullptr;
  g.bias = ptr_bias.has_value() ? ptr_bias->data_ptr() : nullptr;
  g.d = ptr_D.data_ptr();
  g.d_dtype = d_quant ? B200MOE_FP8_E4M3 : (ptr_D.scalar_type() == at::kBFloat16 ? B200MOE_BF16 : B200MOE_F16);
  g.d_scale = d_quant ? ptr_D_scale->data_ptr() : nullptr;
  g.mid_dtype = mid_f16 ? B200MOE_F16 : B200MOE_BF16;
  g.rows_per_expert = rows_per_expert.data_ptr<int32_t>();
  g.m = D_total_M; g.n = (int)N; g.k = (int)K; g.num_experts = (int)segments;
  g.w_experts = segments != num_experts ? (int)num_experts : 0;
  g.epilogue = (b200moe_epilogue)epilogue;
  g.act_alpha = (float)alpha; g.act_limit = (float)limit; g.clamp_limit = (float)clamp_limit;
  int32_t* status_word = device_status_word(ptr_A.get_device());
  raise_if_timed_out(status_word);   // an earlier call on this device gave up a wait
  g.status = status_word;
  g.impl = (int)impl;
  g.max_ctas = (int)max_ctas;
  g.group_size = (int)group_size;
  g.rows_hint = rows_hint;
  const c10::cuda::CUDAGuard guard(ptr_A.device());
  check_status(b200moe_grouped_gemm(&g, current_stream()));
  return ptr_D;
}

at::Tensor cutlass_grouped_gemm_interface(at::Tensor ptr_A, const std::optional<at::Tensor>& ptr_A_scale,
                                          at::Tensor ptr_B, const std::optional<at::Tensor>& ptr_B_scale,
                                          const std::optional<at::Tensor>& ptr_bias, at::Tensor ptr_D,
                                          at::Tensor rows_per_expert, int64_t N, int64_t K,
                                          int64_t num_experts) {
  // The reference accepts ptr_A_scale and ignores it for 16-bit activations.
  return grouped_gemm_impl(ptr_A, ptr_A_scale, ptr_B, ptr_B_scale, ptr_bias, ptr_D, rows_per_expert, N,
                           K, num_experts, 0, 0, 1.702, 7.0, 0.0, 0, 0, false);
}

at::Tensor b200_grouped_gemm(at::Tensor ptr_A, const std::optional<at::Tensor>& ptr_A_scale,
                             at::Tensor ptr_B, const std::optional<at::Tensor>& ptr_B_scale,
                             const std::optional<at::Tensor>& ptr_bias, at::Tensor ptr_D,
                             at::Tensor rows_per_expert, int64_t N, int64_t K, int64_t num_experts,
                             int64_t layout, int64_t epilogue, double alpha, double limit,
                             double clamp_limit, int64_t impl, int64_t max_ctas, int64_t rows_hint,
                             const std::optional<at::Tensor>& ptr_D_scale, bool mid_f16) {
  return grouped_gemm_impl(ptr_A, ptr_A_scale, ptr_B, ptr_B_scale, ptr_bias, ptr_D, rows_per_expert, N,
                           K, num_experts, layout, epilogue, alpha, limit, clamp_limit, impl, max_ctas, true,
                           rows_hint, ptr_D_scale, mid_f16);
}

// Raises if a grouped GEMM on `like`'s device has given up a bounded wait since the last
// check; with `synchronize` the device is synchronised first, so every call made so far is
// covered.  Returns 0 otherwise.
int64_t b200_check_status(const at::Tensor& like, bool synchronize) {
  check_cuda(like, "like");
  const c10::cuda::CUDAGuard guard(like.device());
  if (synchronize) C10_CUDA_CHECK(cudaDeviceSynchronize());
  raise_if_timed_out(device_status_word(like.get_device()));
  return 0;
}

// Launches the bounded-wait self test (b200moe_selftest_bounded_wait) against this device's
// status word: after it has run, b200_check_status raises exactly as it would after a
// grouped GEMM that gave up.
void b200_selftest_bounded_wait(const at::Tensor& like, int64_t budget_cycles) {
  check_cuda(like, "like");
  const c10::cuda::CUDAGuard guard(like.device());
  check_status(b200moe_selftest_bounded_wait(device_status_word(like.get_device()), budget_cycles, current_stream()));
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(_xpu_C, m) {
  m.def(
      "cutlass_grouped_gemm_interface(Tensor ptr_A, Tensor? ptr_A_scale, Tensor ptr_B, Tensor? "
      "ptr_B_scale, Tensor? ptr_bias, Tensor ptr_D, Tensor rows_per_expert, int N, int K, int "
      "num_experts) -> Tensor");
  m.def(
      "b200_grouped_gemm(Tensor ptr_A, Tensor? ptr_A_scale, Tensor ptr_B, Tensor? ptr_B_scale, "
      "Tensor? ptr_bias, Tensor(a!) ptr_D, Tensor rows_per_expert, int N, int K, int num_experts, "
      "int layout=0, int epilogue=0, float alpha=1.702, float limit=7.0, float clamp_limit=0.0, "
      "int impl=0, int max_ctas=0, int rows_hint=0, Tensor(b!)? ptr_D_scale=None, bool mid_f16=False) -> Tensor(a!)");
  m.def("b200_check_status(Tensor like, bool synchronize=True) -> int");
  m.def("b200_selftest_bounded_wait(Tensor like, int budget_cycles) -> ()");
}

TORCH_LIBRARY_IMPL(_xpu_C, CUDA, m) {
  m.impl("cutlass_grouped_gemm_interface", &cutlass_grouped_gemm_interface);
  m.impl("b200_grouped_gemm", &b200_grouped_gemm);
  m.impl("b200_check_status", &b200_check_status);
  m.impl("b200_selftest_bounded_wait", &b200_selftest_bounded_wait);
}

B200_REGISTER_EXTENSION(_xpu_C)
