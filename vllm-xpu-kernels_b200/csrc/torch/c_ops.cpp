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

}  // namespace

TORCH_LIBRARY_FRAGMENT(_C, m) {
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
}

B200_REGISTER_EXTENSION(_C)
