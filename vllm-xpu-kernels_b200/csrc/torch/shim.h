// Helpers shared by the three op-registration libraries (_C, _moe_C, _xpu_C).
// They translate torch tensors into the plain pointers of the C ABI
// (include/b200moe.h), pick the current CUDA stream and turn a non-zero status
// into the RuntimeError a TORCH_CHECK raises.  No kernel lives here.
#pragma once

#include <Python.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <optional>

#include "../../../include/b200moe.h"

#define B200_REGISTER_EXTENSION(NAME)                                        \
  PyMODINIT_FUNC PyInit_##NAME() {                                           \
    static struct PyModuleDef module = {PyModuleDef_HEAD_INIT, #NAME,       \
                                        nullptr, 0, nullptr, nullptr,       \
                                        nullptr, nullptr, nullptr};         \
    return PyModule_Create(&module);                                         \
  }

namespace b200shim {

inline b200moe_stream current_stream() {
  return (b200moe_stream)at::cuda::getCurrentCUDAStream().stream();
}

inline void check_status(int rc) {
  TORCH_CHECK(rc == B200MOE_OK, b200moe_last_error(), " [", b200moe_status_string(rc), "]");
}

inline b200moe_dtype float_dtype(const at::Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kFloat: return B200MOE_F32;
    case at::kHalf: return B200MOE_F16;
    case at::kBFloat16: return B200MOE_BF16;
    default: TORCH_CHECK(false, what, ": only float32, float16 and bfloat16 are supported");
  }
  return B200MOE_F32;
}

inline b200moe_dtype index_dtype(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kInt: return B200MOE_I32;
    case at::kUInt32: return B200MOE_U32;
    case at::kLong: return B200MOE_I64;
    default: return B200MOE_U8;  // rejected by the callee
  }
}

inline void check_cuda(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}

// Scratch for the multi-block sort path; empty when the single-block path runs.
inline at::Tensor sort_workspace(const at::Tensor& like, int64_t numel, int64_t buckets) {
  const size_t bytes = b200moe_sort_workspace_bytes(numel, (int)buckets);
  return at::empty({(int64_t)bytes}, like.options().dtype(at::kByte));
}

}  // namespace b200shim
