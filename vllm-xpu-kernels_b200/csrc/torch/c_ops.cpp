// torch.ops._C.*: gated activations and the dynamic per-token-group fp8
// quantisation.  Schemas are the ones of csrc/torch_bindings.cpp:80-81,
// 170-177, 187-191 in vllm-xpu-kernels.
#include "shim.h"

using namespace b200shim;

namespace {

void silu_and_mul(at::Tensor& out, at::Tensor& input) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == input.scalar_type(), "silu_and_mul: dtype mismatch");
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), "silu_and_mul expects contiguous tensors");
  const int d = input.size(-1) / 2;
  const int64_t rows = d ? input.numel() / input.size(-1) : 0;
  TORCH_CHECK(out.numel() == rows * d, "silu_and_mul: out must be [..., d]");
  if (input.numel() == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_silu_and_mul(out.data_ptr(), input.data_ptr(), float_dtype(input, "silu_and_mul"),
                                    rows, d, current_stream()));
}

void swigluoai_and_mul(at::Tensor& out, at::Tensor& input, double alpha, double limit) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == input.scalar_type(), "swigluoai_and_mul: dtype mismatch");
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), "swigluoai_and_mul expects contiguous tensors");
  const int d = input.size(-1) / 2;
  const int64_t rows = d ? input.numel() / input.size(-1) : 0;
  TORCH_CHECK(out.numel() == rows * d, "swigluoai_and_mul: out must be [..., d]");
  if (input.numel() == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_swigluoai_and_mul(out.data_ptr(), input.data_ptr(),
                                         float_dtype(input, "swigluoai_and_mul"), rows, d,
                                         (float)alpha, (float)limit, current_stream()));
}

void per_token_group_fp8_quant(const at::Tensor& input, at::Tensor& output_q, at::Tensor& output_s,
                               int64_t group_size, double eps, double fp8_min, double fp8_max,
                               bool scale_ue8m0, bool dummy_is_scale_transposed,
                               bool dummy_is_tma_aligned) {
  (void)fp8_min; (void)fp8_max; (void)dummy_is_scale_transposed; (void)dummy_is_tma_aligned;
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous());
  TORCH_CHECK(output_q.is_contiguous());
  TORCH_CHECK(group_size > 0 && input.numel() % group_size == 0);
  TORCH_CHECK(output_s.dim() == 2);
  TORCH_CHECK(output_q.scalar_type() == at::kFloat8_e4m3fn,
              "per_token_group_fp8_quant: output_q must be float8_e4m3fn");
  TORCH_CHECK(output_s.scalar_type() == at::kFloat, "per_token_group_fp8_quant: output_s must be float32");
  const int64_t rows = output_s.size(0);
  if (input.numel() == 0) return;
  const int cols = (int)(input.numel() / rows);
  TORCH_CHECK(cols % group_size == 0 && output_s.size(1) == cols / group_size,
              "per_token_group_fp8_quant: output_s must be [rows, cols / group_size]");
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_per_token_group_fp8_quant(
      input.data_ptr(), float_dtype(input, "per_token_group_fp8_quant"), output_q.data_ptr(),
      output_s.data_ptr<float>(), rows, cols, (int)group_size, (float)eps, scale_ue8m0,
      output_s.stride(0), output_s.stride(1), current_stream()));
}

// x [rows, cols] bf16/f16 -> q e4m3 [planes * rows, cols], s int32 [planes, ceil(cols/128), rows]
// (four e8m0 bytes per word); planes = 1, or 2 with the residual plane.
void b200_quant_mxfp8(const at::Tensor& input, at::Tensor& output_q, at::Tensor& output_s) {
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous() && output_q.is_contiguous() && output_s.is_contiguous());
  TORCH_CHECK(input.dim() == 2 && output_q.dim() == 2 && output_s.dim() == 3);
  const int64_t rows = input.size(0), cols = input.size(1), planes = output_s.size(0);
  TORCH_CHECK(planes == 1 || planes == 2, "b200_quant_mxfp8: one or two planes");
  TORCH_CHECK(output_q.scalar_type() == at::kFloat8_e4m3fn && output_q.size(0) == planes * rows &&
              output_q.size(1) == cols, "b200_quant_mxfp8: output_q must be float8_e4m3fn [planes * rows, cols]");
  TORCH_CHECK(output_s.scalar_type() == at::kInt && output_s.size(1) == (cols + 127) / 128 &&
              output_s.size(2) == rows, "b200_quant_mxfp8: output_s must be int32 [planes, ceil(cols / 128), rows]");
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_quant_mxfp8(input.data_ptr(), float_dtype(input, "b200_quant_mxfp8"),
                                   output_q.data_ptr(), output_s.data_ptr(), rows, (int)cols, (int)planes,
                                   current_stream()));
}

// gelu_and_mul / gelu_tanh_and_mul / swiglustep_and_mul: [..., 2d] -> [..., d]
// (csrc/activation.cpp:576-592, 711-716 of the reference).
template <typename F>
void gated_act_op(at::Tensor& out, at::Tensor& input, const char* name, F call) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == input.scalar_type(), name, ": dtype mismatch");
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), name, " expects contiguous tensors");
  const int d = input.size(-1) / 2;
  const int64_t rows = d ? input.numel() / input.size(-1) : 0;
  TORCH_CHECK(out.numel() == rows * d, name, ": out must be [..., d]");
  if (input.numel() == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(call(out.data_ptr(), input.data_ptr(), float_dtype(input, name), rows, d, current_stream()));
}
void gelu_and_mul(at::Tensor& out, at::Tensor& input) {
  gated_act_op(out, input, "gelu_and_mul", b200moe_gelu_and_mul);
}
void gelu_tanh_and_mul(at::Tensor& out, at::Tensor& input) {
  gated_act_op(out, input, "gelu_tanh_and_mul", b200moe_gelu_tanh_and_mul);
}
void swiglustep_and_mul(at::Tensor& out, at::Tensor& input, double limit) {
  gated_act_op(out, input, "swiglustep_and_mul",
               [limit](void* o, const void* i, b200moe_dtype dt, int64_t rows, int d, b200moe_stream st) {
                 return b200moe_swiglustep_and_mul(o, i, dt, rows, d, (float)limit, st);
               });
}
// relu2_no_mul: out and input have the same shape (csrc/activation.cpp:674-681).
void relu2_no_mul(at::Tensor& out, at::Tensor& input) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == input.scalar_type(), "relu2_no_mul: dtype mismatch");
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous(), "relu2_no_mul expects contiguous tensors");
  TORCH_CHECK(out.numel() == input.numel(), "relu2_no_mul: out must have the input's shape");
  if (input.numel() == 0) return;
  const int d = input.size(-1);
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_relu2_no_mul(out.data_ptr(), input.data_ptr(), float_dtype(input, "relu2_no_mul"),
                                    input.numel() / d, d, current_stream()));
}

// csrc/quantization/fused_kernels/fused_silu_mul_block_quant.cpp:141-195 of the reference.
void silu_and_mul_per_block_quant(at::Tensor& out, const at::Tensor& input, at::Tensor& scales,
                                  int64_t group_size, const std::optional<at::Tensor>& scale_ub,
                                  bool is_scale_transposed, bool scale_ue8m0) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kFloat8_e4m3fn || out.scalar_type() == at::kFloat8_e5m2 ||
                  out.scalar_type() == at::kChar,
              "out must be float8_e4m3fn, float8_e5m2, or int8");
  TORCH_CHECK(out.scalar_type() != at::kFloat8_e5m2, "float8_e5m2 output is not available in this build");
  TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16,
              "input must be float16 or bfloat16");
  TORCH_CHECK(out.is_contiguous(), "out must be contiguous");
  TORCH_CHECK(input.is_contiguous(), "input must be contiguous");
  TORCH_CHECK(scales.scalar_type() == at::kFloat, "scales must be float32");
  TORCH_CHECK(group_size == 32 || group_size == 64 || group_size == 128,
              "group_size must be 32, 64, or 128, got ", group_size);
  if (scale_ub.has_value())
    TORCH_CHECK(out.scalar_type() == at::kFloat8_e4m3fn, "scale_ub is only supported for FP8 output");
  TORCH_CHECK(input.dim() == 2, "input must be 2-dimensional");
  TORCH_CHECK(out.dim() == 2, "out must be 2-dimensional");
  const int64_t num_tokens = input.size(0), hidden = out.size(-1);
  TORCH_CHECK(input.size(-1) == hidden * 2, "input last dim must be 2 * hidden_size");
  TORCH_CHECK(hidden % group_size == 0, "hidden_size must be divisible by group_size");
  TORCH_CHECK(out.size(0) == num_tokens, "out.size(0) must equal num_tokens (input.size(0))");
  const int64_t num_groups = hidden / group_size;
  TORCH_CHECK(scales.size(0) == num_tokens && scales.size(1) == num_groups,
              "scales must have logical shape [num_tokens, num_groups]");
  if (num_tokens == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_silu_and_mul_per_block_quant(
      out.data_ptr(), out.scalar_type() == at::kChar ? B200MOE_I8 : B200MOE_FP8_E4M3, scales.data_ptr<float>(),
      input.data_ptr(), float_dtype(input, "silu_and_mul_per_block_quant"), num_tokens, (int)hidden,
      (int)group_size, scale_ub.has_value() ? scale_ub->data_ptr<float>() : nullptr,
      is_scale_transposed ? 1 : num_groups, is_scale_transposed ? num_tokens : 1, scale_ue8m0, current_stream()));
}

// The layer's form: e4m3, group 128, and only the rows the grouped GEMM's segments use.
void b200_silu_and_mul_block_quant_rows(at::Tensor& out, const at::Tensor& input, at::Tensor& scales,
                                        const at::Tensor& rows_per_segment) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kFloat8_e4m3fn && scales.scalar_type() == at::kFloat, "out must be float8_e4m3fn, scales float32");
  TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16, "input must be float16 or bfloat16");
  TORCH_CHECK(out.is_contiguous() && input.is_contiguous() && scales.is_contiguous() && input.dim() == 2 && out.dim() == 2,
              "out, input and scales must be contiguous 2-D tensors");
  const int64_t rows = input.size(0), hidden = out.size(1);
  TORCH_CHECK(input.size(1) == 2 * hidden && out.size(0) == rows && hidden % 128 == 0 && scales.numel() == rows * (hidden / 128),
              "shapes: input [rows, 2 * hidden], out [rows, hidden], scales [rows, hidden / 128]");
  TORCH_CHECK(rows_per_segment.scalar_type() == at::kInt && rows_per_segment.is_contiguous(), "rows_per_segment must be int32");
  if (rows == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_silu_and_mul_per_block_quant_ragged(
      out.data_ptr(), scales.data_ptr<float>(), input.data_ptr(), float_dtype(input, "silu_and_mul_per_block_quant"), rows,
      (int)hidden, rows_per_segment.data_ptr<int32_t>(), (int)rows_per_segment.numel(), current_stream()));
}

// csrc/quantization/fused_kernels/fused_silu_mul_mxfp4_quant.cpp:134-185 of the reference.
void silu_and_mul_mxfp4_quant(at::Tensor& out, const at::Tensor& input, at::Tensor& scales, int64_t group_size,
                              double eps) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kByte, "out must be uint8");
  TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16,
              "input must be float16 or bfloat16");
  TORCH_CHECK(out.is_contiguous() && input.is_contiguous(), "out and input must be contiguous");
  TORCH_CHECK(scales.scalar_type() == at::kFloat, "scales must be float32");
  TORCH_CHECK(group_size == 32, "MXFP4 requires group_size == 32, got ", group_size);
  TORCH_CHECK(input.dim() == 2 && out.dim() == 2 && scales.dim() == 2, "input, out and scales must be 2-dimensional");
  const int64_t num_tokens = input.size(0), hidden = input.size(-1) / 2;
  TORCH_CHECK(input.size(-1) % 2 == 0 && hidden % group_size == 0, "hidden_size must be divisible by group_size");
  TORCH_CHECK(out.size(0) == num_tokens && out.size(1) == hidden / 2, "out must be [num_tokens, hidden_size / 2]");
  TORCH_CHECK(scales.size(0) == num_tokens && scales.size(1) == hidden / group_size,
              "scales must have logical shape [num_tokens, num_groups]");
  if (num_tokens == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_silu_and_mul_mxfp4_quant(out.data_ptr(), scales.data_ptr<float>(), input.data_ptr(),
                                                float_dtype(input, "silu_and_mul_mxfp4_quant"), num_tokens,
                                                (int)hidden, (float)eps, scales.stride(0), scales.stride(1),
                                                current_stream()));
}

// csrc/quantization/fp4/mxfp4_quant.cpp:24-86 of the reference.
void per_token_group_quant_mxfp4(const at::Tensor& input, at::Tensor& output_q, at::Tensor& output_s,
                                 int64_t group_size, double eps) {
  check_cuda(input, "input");
  TORCH_CHECK(input.is_contiguous(), "input must be contiguous");
  TORCH_CHECK(output_q.is_contiguous(), "output_q must be contiguous");
  TORCH_CHECK(group_size == 32, "MXFP4 requires group_size == 32, got ", group_size);
  TORCH_CHECK(input.numel() % group_size == 0, "input numel must be divisible by group_size");
  TORCH_CHECK(output_s.dim() == 2, "output_s must be 2-D");
  TORCH_CHECK(output_q.scalar_type() == at::kByte, "output_q must be uint8");
  TORCH_CHECK(output_s.scalar_type() == at::kFloat, "output_s must be float32");
  if (input.numel() == 0) {
    TORCH_CHECK(output_q.numel() == 0, "output_q must be empty when input is empty");
    TORCH_CHECK(output_s.numel() == 0, "output_s must be empty when input is empty");
    return;
  }
  const int64_t hidden = input.size(-1), rows = input.numel() / hidden;
  TORCH_CHECK(hidden % group_size == 0,
              "per_token_group_quant_mxfp4: rows that are not a multiple of 32 long are not available in this build");
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_per_token_group_quant_mxfp4(input.data_ptr(), float_dtype(input, "per_token_group_quant_mxfp4"),
                                                   output_q.data_ptr(), output_s.data_ptr<float>(), rows, (int)hidden,
                                                   (float)eps, output_s.stride(0), output_s.stride(1),
                                                   current_stream()));
}

// csrc/activation.cpp:552-566 of the reference.
void silu_and_mul_quant(at::Tensor& out, at::Tensor& input, at::Tensor& scale) {
  check_cuda(input, "input");
  TORCH_CHECK(out.scalar_type() == at::kFloat8_e4m3fn || out.scalar_type() == at::kFloat8_e5m2);
  TORCH_CHECK(out.scalar_type() == at::kFloat8_e4m3fn, "float8_e5m2 output is not available in this build");
  TORCH_CHECK(input.scalar_type() == at::kHalf || input.scalar_type() == at::kBFloat16);
  TORCH_CHECK(input.size(-1) % 2 == 0);
  TORCH_CHECK(input.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(scale.scalar_type() == at::kFloat && scale.numel() >= 1);
  const int64_t d = input.size(-1) / 2;
  const int64_t rows = input.numel() / input.size(-1);
  if (rows == 0) return;
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_silu_and_mul_quant(out.data_ptr(), input.data_ptr(), float_dtype(input, "silu_and_mul_quant"),
                                          scale.data_ptr<float>(), rows, (int)d, current_stream()));
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(_C, m) {
  m.def("gelu_and_mul(Tensor! out, Tensor input) -> ()");
  m.def("gelu_tanh_and_mul(Tensor! out, Tensor input) -> ()");
  m.def("relu2_no_mul(Tensor! out, Tensor! input) -> ()");
  m.def(
      "swiglustep_and_mul(Tensor! out, Tensor input, float limit=7.0) "
      "-> ()");
  m.def("silu_and_mul_quant(Tensor! result, Tensor input, Tensor scale) -> ()");
  m.def(
      "silu_and_mul_per_block_quant("
      "Tensor! out, "
      "Tensor input, "
      "Tensor! scales, "
      "int group_size, "
      "Tensor? scale_ub=None, "
      "bool is_scale_transposed=False, "
      "bool scale_ue8m0=False) -> ()");
  m.def("b200_silu_and_mul_block_quant_rows(Tensor! out, Tensor input, Tensor! scales, Tensor rows_per_segment) -> ()");
  m.def(
      "silu_and_mul_mxfp4_quant("
      "Tensor! out, Tensor input, Tensor! scales, "
      "int group_size, float eps=1e-10) -> ()");
  m.def(
      "per_token_group_quant_mxfp4(Tensor input, Tensor! output_q, Tensor! "
      "output_s, int group_size, float eps) -> ()");
  m.def("b200_quant_mxfp8(Tensor input, Tensor! output_q, Tensor! output_s) -> ()");
  m.def("silu_and_mul(Tensor! result, Tensor input) -> ()");
  m.def("swigluoai_and_mul(Tensor! out, Tensor input, float alpha=1.702, float limit=7.0) -> ()");
  m.def(
      "per_token_group_fp8_quant(Tensor input, Tensor! output_q, Tensor! "
      "output_s, "
      "int group_size, float eps, float fp8_min, float fp8_max, bool "
      "scale_ue8m0, bool dummy_is_scale_transposed, bool dummy_is_tma_aligned "
      ") -> ()");
}

TORCH_LIBRARY_IMPL(_C, CUDA, m) {
  m.impl("silu_and_mul", &silu_and_mul);
  m.impl("swigluoai_and_mul", &swigluoai_and_mul);
  m.impl("per_token_group_fp8_quant", &per_token_group_fp8_quant);
  m.impl("b200_quant_mxfp8", &b200_quant_mxfp8);
  m.impl("gelu_and_mul", &gelu_and_mul);
  m.impl("gelu_tanh_and_mul", &gelu_tanh_and_mul);
  m.impl("relu2_no_mul", &relu2_no_mul);
  m.impl("swiglustep_and_mul", &swiglustep_and_mul);
  m.impl("silu_and_mul_quant", &silu_and_mul_quant);
  m.impl("silu_and_mul_per_block_quant", &silu_and_mul_per_block_quant);
  m.impl("b200_silu_and_mul_block_quant_rows", &b200_silu_and_mul_block_quant_rows);
  m.impl("silu_and_mul_mxfp4_quant", &silu_and_mul_mxfp4_quant);
  m.impl("per_token_group_quant_mxfp4", &per_token_group_quant_mxfp4);
}

B200_REGISTER_EXTENSION(_C)
