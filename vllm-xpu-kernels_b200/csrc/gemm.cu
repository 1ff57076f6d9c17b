// b200moe_grouped_gemm: argument checks (messages follow
// csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:184-243, 267-287,
// 322-383 of vllm-xpu-kernels) and the choice between the tensor-core kernel
// and the plain-CUDA checking kernel.
#include <atomic>

#include "common.cuh"

namespace b200moe {
int grouped_gemm_tc(const b200moe_gemm_args* a, cudaStream_t st);
int grouped_gemm_tc_fp8t(const b200moe_gemm_args* a, cudaStream_t st);
int grouped_gemm_tc_dq(const b200moe_gemm_args* a, cudaStream_t st);
int grouped_gemm_tc_mx(const b200moe_gemm_args* a, cudaStream_t st);
int grouped_gemm_check(const b200moe_gemm_args* a, cudaStream_t st);
}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_grouped_gemm(const b200moe_gemm_args* a, b200moe_stream stream) {
  B200_CHECK_ARG(a != nullptr, "grouped_gemm: null argument struct");
  B200_CHECK_ARG(a->n % 8 == 0, "N must be divisible by 8");
  B200_CHECK_ARG(a->m >= 0 && a->n >= 0 && a->k > 0 && a->num_experts >= 1,
                 "grouped_gemm: bad sizes (m=%lld n=%d k=%d experts=%d)", (long long)a->m, a->n,
                 a->k, a->num_experts);
  const bool d_quant = a->d_dtype == B200MOE_FP8_E4M3;
  B200_CHECK_ARG(a->d_dtype == B200MOE_BF16 || a->d_dtype == B200MOE_F16 || d_quant,
                 "grouped_gemm: ptr_D must be bfloat16 or float16");
  B200_CHECK_ARG(!d_quant || (a->epilogue == B200MOE_EPI_SILU_MUL && a->d_scale != nullptr &&
                              a->a_dtype == B200MOE_FP8_E4M3 &&
                              (a->w_format == B200MOE_W_FP8_BLOCK_NK || a->w_format == B200MOE_W_FP8_BLOCK_KN) &&
                              (a->mid_dtype == B200MOE_BF16 || a->mid_dtype == B200MOE_F16)),
                 "grouped_gemm: e4m3 output needs the SiLU epilogue, d_scale, a 16-bit mid_dtype, fp8 "
                 "activations and block-scaled fp8 weights");
  const bool a_x2 = a->a_dtype == B200MOE_FP8_E4M3_X2;
  const bool a_fp8 = a->a_dtype == B200MOE_FP8_E4M3 || a_x2;
  B200_CHECK_ARG(a_fp8 || a->a_dtype == a->d_dtype,
                 "grouped_gemm: ptr_A must be fp8 (with scales) or have ptr_D's dtype");
  switch (a->w_format) {
    case B200MOE_W_BF16_KN:
    case B200MOE_W_BF16_NK:
      B200_CHECK_ARG(a->w_scale == nullptr, "w16a16 grouped gemm must not have scales");
      B200_CHECK_ARG(!a_fp8, "grouped_gemm: fp8 activations need block-scaled fp8 weights");
      break;
    case B200MOE_W_FP8_TENSOR_KN:
    case B200MOE_W_FP8E5M2_TENSOR_KN:
      B200_CHECK_ARG(a->w_scale != nullptr, "w8a16 grouped gemm must have scales");
      B200_CHECK_ARG(!a_fp8 || a->a_scale != nullptr,
                     "grouped_gemm: fp8 activations with per-tensor fp8 weights need the e8m0 scale words "
                     "[planes][ceil(K / 128)][M] of b200moe_quant_mxfp8");
      break;
    case B200MOE_W_FP8_BLOCK_NK:
    case B200MOE_W_FP8_BLOCK_KN:
      B200_CHECK_ARG(a->w_scale != nullptr, "w8a16 grouped gemm must have scales");
      B200_CHECK_ARG(a->n % 128 == 0 && a->k % 128 == 0,
                     "block-scaled grouped GEMM requires N and K divisible by 128");
      B200_CHECK_ARG(!a_fp8 || a->a_scale != nullptr,
                     "grouped_gemm: fp8 activations need ptr_A_scale [M, K / 128]");
      break;
    case B200MOE_W_MXFP4_NK:
      B200_CHECK_ARG(a->w_scale != nullptr, "w8a16 grouped gemm must have scales");
      B200_CHECK_ARG(a->k % 32 == 0, "group_size must be 32, 64, 128 or 256");
      B200_CHECK_ARG(!a_fp8 || a->a_scale != nullptr,
                     "grouped_gemm: fp8 activations with MXFP4 weights need the e8m0 scale words "
                     "[planes][ceil(K / 128)][M] of b200moe_quant_mxfp8");
      break;
    case B200MOE_W_MXFP8_KN:
      B200_CHECK_ARG(a->w_scale != nullptr, "w8a16 grouped gemm must have scales");
      B200_CHECK_ARG(a->k % 32 == 0, "mxfp8 grouped gemm requires K divisible by 32");
      B200_CHECK_ARG(!a_fp8 || a->a_scale != nullptr,
                     "grouped_gemm: fp8 activations with MXFP8 weights need the e8m0 scale words "
                     "[planes][ceil(K / 128)][M] of b200moe_quant_mxfp8");
      break;
    case B200MOE_W_INT4_NK:
      B200_CHECK_ARG(a->w_scale != nullptr, "w8a16 grouped gemm must have scales");
      B200_CHECK_ARG(a->group_size == 32 || a->group_size == 64 || a->group_size == 128 || a->group_size == 256,
                     "group_size must be 32, 64, 128 or 256");
      B200_CHECK_ARG(a->k % a->group_size == 0, "ptr_scales.size(2) of int4 must be divisible by K");
      B200_CHECK_ARG(!a_fp8, "grouped_gemm: int4 weights take 16-bit activations");
      break;
    default:
      return fail(B200MOE_E_BADARG, "grouped_gemm: unknown weight format %d", (int)a->w_format);
  }
  const bool w_tensor8 = a->w_format == B200MOE_W_FP8_TENSOR_KN || a->w_format == B200MOE_W_FP8E5M2_TENSOR_KN ||
                         a->w_format == B200MOE_W_MXFP8_KN;
  B200_CHECK_ARG(!a_x2 || a->w_format == B200MOE_W_MXFP4_NK || w_tensor8,
                 "grouped_gemm: two-plane fp8 activations need MXFP4, MXFP8 or per-tensor fp8 weights");
  const bool segmented = a->w_experts > 0 && a->w_experts != a->num_experts;
  B200_CHECK_ARG(a->w_experts >= 0 && (!segmented || a->num_experts % a->w_experts == 0),
                 "grouped_gemm: w_experts must divide num_experts");
  B200_CHECK_ARG(!segmented || a->w_format == B200MOE_W_BF16_KN || a->w_format == B200MOE_W_BF16_NK ||
                     a->w_format == B200MOE_W_FP8_BLOCK_NK || a->w_format == B200MOE_W_FP8_BLOCK_KN,
                 "grouped_gemm: row segments that share weight sets need 16-bit or block-scaled fp8 weights");
  B200_CHECK_ARG(a->epilogue == B200MOE_EPI_NONE || a->n % 2 == 0,
                 "grouped_gemm: a gated epilogue needs an even N");
  if (a->m == 0 || a->n == 0) return B200MOE_OK;
  B200_CHECK_ARG(a->a && a->w && a->d && a->rows_per_expert, "grouped_gemm: null pointer");
  cudaStream_t st = as_stream(stream);
  // MXFP8 activations exist on the block-scaled tensor-core path only.
  if ((a->w_format == B200MOE_W_MXFP4_NK || w_tensor8) && a_fp8) return grouped_gemm_tc_mx(a, st);
  if (d_quant) {
    B200_CHECK_ARG(a->impl != 2, "grouped_gemm: the checking kernel has no quantised output");
    return grouped_gemm_tc_fp8t(a, st);
  }
  if (a->impl == 2 || a->w_format == B200MOE_W_MXFP8_KN) return grouped_gemm_check(a, st);   // 16-bit activations
  int rc = (a->w_format == B200MOE_W_MXFP4_NK || a->w_format == B200MOE_W_INT4_NK) ? grouped_gemm_tc_dq(a, st)
                                                                                    : grouped_gemm_tc(a, st);
  if (rc == B200MOE_E_UNSUPPORTED && a->impl == 0) {
    // A request no tensor-core kernel covers (16-bit activations against fp8 weights, a gated
    // epilogue whose output width is not a multiple of 16, a row pitch that is not a multiple of
    // 16 bytes) still gets its
    // result from the plain-CUDA checking kernel, which is correct and one to two orders of
    // magnitude slower: say so once per process instead of degrading silently.
    static std::atomic<bool> warned{false};
    if (!warned.exchange(true))
      fprintf(stderr, "b200moe: grouped GEMM request outside the tensor-core kernels (%s); running the slow "
                      "checking kernel for it (reported once)\n", b200moe_last_error());
    return grouped_gemm_check(a, st);
  }
  return rc;
}
