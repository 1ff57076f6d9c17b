// torch.ops._moe_C.*: routing, alignment, permutation and top-k reductions.
// Schemas are the ones of csrc/moe/torch_bindings.cpp in vllm-xpu-kernels
// (registered there for the XPU dispatch key; here for CUDA).
#include "shim.h"

using namespace b200shim;

namespace {

void topk_softmax(at::Tensor& topk_weights, at::Tensor& topk_indices,
                  at::Tensor& token_expert_indices, at::Tensor& gating_output,
                  bool renormalize, std::optional<at::Tensor> bias) {
  check_cuda(gating_output, "gating_output");
  const int num_experts = gating_output.size(-1);
  const int64_t num_tokens = num_experts ? gating_output.numel() / num_experts : 0;
  const int topk = topk_weights.size(-1);
  TORCH_CHECK(topk_indices.scalar_type() == at::kInt || topk_indices.scalar_type() == at::kUInt32 ||
              topk_indices.scalar_type() == at::kLong,
              "topk_indices must be int32, uint32 or int64");
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, "topk_weights must be float32");
  TORCH_CHECK(gating_output.is_contiguous() && topk_weights.is_contiguous() &&
              topk_indices.is_contiguous() && token_expert_indices.is_contiguous(),
              "topk_softmax expects contiguous tensors");
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous(), "bias must be contiguous float32");
  const c10::cuda::CUDAGuard guard(gating_output.device());
  check_status(b200moe_topk_softmax(
      topk_weights.data_ptr<float>(), topk_indices.data_ptr(), index_dtype(topk_indices),
      token_expert_indices.data_ptr<int32_t>(), gating_output.data_ptr(),
      float_dtype(gating_output, "topk_softmax"), num_tokens, num_experts, topk, renormalize,
      bias.has_value() ? bias->data_ptr<float>() : nullptr, current_stream()));
}

void topk_sigmoid(at::Tensor& topk_weights, at::Tensor& topk_indices,
                  at::Tensor& token_expert_indices, at::Tensor& gating_output,
                  bool renormalize, std::optional<at::Tensor> bias,
                  double routed_scaling_factor) {
  check_cuda(gating_output, "gating_output");
  const int num_experts = gating_output.size(-1);
  const int64_t num_tokens = num_experts ? gating_output.numel() / num_experts : 0;
  const int topk = topk_weights.size(-1);
  TORCH_CHECK(topk_indices.scalar_type() == at::kInt || topk_indices.scalar_type() == at::kUInt32 ||
              topk_indices.scalar_type() == at::kLong,
              "topk_indices must be int32, uint32 or int64");
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, "topk_weights must be float32");
  TORCH_CHECK(gating_output.is_contiguous() && topk_weights.is_contiguous() &&
              topk_indices.is_contiguous() && token_expert_indices.is_contiguous(),
              "topk_sigmoid expects contiguous tensors");
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous(), "bias must be contiguous float32");
  const c10::cuda::CUDAGuard guard(gating_output.device());
  check_status(b200moe_topk_sigmoid(
      topk_weights.data_ptr<float>(), topk_indices.data_ptr(), index_dtype(topk_indices),
      token_expert_indices.data_ptr<int32_t>(), gating_output.data_ptr(),
      float_dtype(gating_output, "topk_sigmoid"), num_tokens, num_experts, topk, renormalize,
      bias.has_value() ? bias->data_ptr<float>() : nullptr, routed_scaling_factor,
      current_stream()));
}

// csrc/moe/moe_align_sum_kernels.cpp:1183-1222 of the reference.
void batched_moe_align_block_size(int64_t max_tokens_per_batch, int64_t block_size,
                                  const at::Tensor& batch_num_tokens, at::Tensor sorted_ids,
                                  at::Tensor batch_ids, at::Tensor num_tokens_post_pad) {
  check_cuda(batch_num_tokens, "expert_num_tokens");
  const int64_t B = batch_num_tokens.size(0);
  const int64_t sorted_size = (max_tokens_per_batch + block_size - 1) / block_size * block_size * B;
  TORCH_CHECK(sorted_ids.size(0) == sorted_size);
  TORCH_CHECK(batch_ids.size(0) == sorted_size / block_size);
  TORCH_CHECK(num_tokens_post_pad.size(0) == 1);
  TORCH_CHECK(B <= 1024);
  TORCH_CHECK(batch_num_tokens.scalar_type() == at::kInt && sorted_ids.scalar_type() == at::kInt &&
              batch_ids.scalar_type() == at::kInt && num_tokens_post_pad.scalar_type() == at::kInt,
              "batched_moe_align_block_size expects int32 tensors");
  TORCH_CHECK(batch_num_tokens.is_contiguous() && sorted_ids.is_contiguous() && batch_ids.is_contiguous());
  if (B == 0) return;
  const c10::cuda::CUDAGuard guard(batch_num_tokens.device());
  check_status(b200moe_batched_moe_align_block_size(
      (int)max_tokens_per_batch, (int)block_size, batch_num_tokens.data_ptr<int32_t>(), (int)B,
      sorted_ids.data_ptr<int32_t>(), batch_ids.data_ptr<int32_t>(), num_tokens_post_pad.data_ptr<int32_t>(),
      current_stream()));
}

// csrc/moe/fused_moe_prologue.cpp:170-216 of the reference.  Rows and scales are moved
// as opaque storage elements, so every dtype the reference dispatches on (bf16, fp16,
// fp8 e4m3 with f32 or e8m0 scales, packed fp4 with e8m0 scales) is covered by its
// element size.
void fused_moe_prologue(at::Tensor input, const std::optional<at::Tensor>& input_scales,
                        at::Tensor token_selected_experts, at::Tensor token_final_scales,
                        at::Tensor workspace, int64_t hidden_size, int64_t inter_size, int64_t block_k,
                        int64_t ep_rank, int64_t ep_size, int64_t num_experts_on_rank) {
  (void)inter_size;
  check_cuda(input, "input");
  check_cuda(workspace, "workspace");
  TORCH_CHECK(token_selected_experts.scalar_type() == at::kLong, "token_selected_experts must be int64");
  TORCH_CHECK(token_final_scales.scalar_type() == at::kFloat, "token_final_scales must be float32");
  TORCH_CHECK(input.dim() == 2 && input.is_contiguous() && token_selected_experts.dim() == 2 &&
              token_selected_experts.is_contiguous() && token_final_scales.is_contiguous() &&
              workspace.is_contiguous(),
              "fused_moe_prologue expects contiguous tensors");
  TORCH_CHECK(input.size(1) == hidden_size, "hidden_size does not match the input rows");
  TORCH_CHECK(ep_rank >= 0 && ep_rank < ep_size, "ep_rank out of range");
  const int64_t num_rows = input.size(0);
  const int topk = (int)token_selected_experts.size(1);
  TORCH_CHECK(token_selected_experts.size(0) == num_rows && token_final_scales.numel() == num_rows * topk,
              "routing tensors do not match the input rows");
  int scale_bytes = 0;
  const void* scales = nullptr;
  if (input_scales.has_value()) {
    TORCH_CHECK(input_scales->is_contiguous() && input_scales->is_cuda(), "input_scales must be contiguous CUDA");
    TORCH_CHECK(input_scales->numel() == num_rows * (hidden_size / block_k),
                "input_scales must hold hidden_size / block_k entries per row");
    scale_bytes = (int)input_scales->element_size();
    scales = input_scales->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(input.device());
  const size_t scratch_bytes =
      b200moe_fused_moe_prologue_scratch_bytes(num_rows, topk, (int)num_experts_on_rank);
  at::Tensor scratch = at::empty({(int64_t)scratch_bytes}, input.options().dtype(at::kByte));
  check_status(b200moe_fused_moe_prologue(
      input.data_ptr(), (int)input.element_size(), scales, scale_bytes,
      token_selected_experts.data_ptr<int64_t>(), token_final_scales.data_ptr<float>(),
      workspace.data_ptr(), (size_t)workspace.nbytes(), num_rows, hidden_size, (int)block_k, topk,
      (int)ep_rank, (int)ep_size, (int)num_experts_on_rank, scratch.data_ptr(), scratch_bytes,
      current_stream()));
}

// csrc/moe/moe_align_sum_kernels.cpp:1374-1549 of the reference.
void moe_lora_align_block_size(at::Tensor topk_ids, at::Tensor token_lora_mapping, int64_t num_experts,
                               int64_t block_size, int64_t max_loras, int64_t max_num_tokens_padded,
                               int64_t max_num_m_blocks, at::Tensor sorted_token_ids,
                               at::Tensor expert_ids, at::Tensor num_tokens_post_pad,
                               at::Tensor adapter_enabled, at::Tensor lora_ids,
                               std::optional<at::Tensor> maybe_expert_map) {
  check_cuda(topk_ids, "topk_ids");
  TORCH_CHECK(block_size > 0, "block_size should be greater than 0. ");
  TORCH_CHECK((num_experts + 31) / 32 * 32 < 1024, "padded_num_experts must be less than 1024");
  TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.is_contiguous(), "topk_ids must be a contiguous [tokens, topk] tensor");
  for (const at::Tensor* t : {&token_lora_mapping, &sorted_token_ids, &expert_ids, &num_tokens_post_pad,
                              &adapter_enabled, &lora_ids})
    TORCH_CHECK(t->scalar_type() == at::kInt && t->is_contiguous() && t->is_cuda(),
                "moe_lora_align_block_size expects contiguous int32 CUDA tensors");
  TORCH_CHECK(token_lora_mapping.numel() >= topk_ids.size(0), "token_lora_mapping is shorter than the token count");
  TORCH_CHECK(sorted_token_ids.numel() >= max_loras * max_num_tokens_padded, "sorted_token_ids is too small");
  TORCH_CHECK(expert_ids.numel() >= max_loras * max_num_m_blocks, "experts_ids is too small");
  TORCH_CHECK(num_tokens_post_pad.numel() >= max_loras, "num_tokens_post_pad is too small");
  TORCH_CHECK(lora_ids.numel() >= max_loras + 1 && adapter_enabled.numel() >= max_loras,
              "lora_ids needs max_loras + 1 entries and adapter_enabled max_loras");
  const int32_t* map = nullptr;
  if (maybe_expert_map.has_value()) {
    TORCH_CHECK(maybe_expert_map->scalar_type() == at::kInt && maybe_expert_map->is_contiguous(),
                "expert_map must be contiguous int32");
    map = maybe_expert_map->data_ptr<int32_t>();
  }
  const c10::cuda::CUDAGuard guard(topk_ids.device());
  check_status(b200moe_moe_lora_align_block_size(
      topk_ids.data_ptr(), index_dtype(topk_ids), topk_ids.numel(), (int)topk_ids.size(1),
      token_lora_mapping.data_ptr<int32_t>(), (int)num_experts, (int)block_size, (int)max_loras,
      (int)max_num_tokens_padded, (int)max_num_m_blocks, sorted_token_ids.data_ptr<int32_t>(),
      expert_ids.data_ptr<int32_t>(), num_tokens_post_pad.data_ptr<int32_t>(),
      adapter_enabled.data_ptr<int32_t>(), lora_ids.data_ptr<int32_t>(), map, current_stream()));
}

// csrc/moe/topk_softplus_sqrt_kernels.cpp:596-772 of the reference.
void topk_softplus_sqrt(at::Tensor& topk_weights, at::Tensor& topk_indices,
                        at::Tensor& token_expert_indices, at::Tensor& gating_output, bool renormalize,
                        double routed_scaling_factor, const std::optional<at::Tensor>& correction_bias,
                        const std::optional<at::Tensor>& input_ids, const std::optional<at::Tensor>& tid2eid) {
  check_cuda(gating_output, "gating_output");
  const int num_experts = gating_output.size(-1);
  const int64_t num_tokens = num_experts ? gating_output.numel() / num_experts : 0;
  const int topk = topk_weights.size(-1);
  TORCH_CHECK(topk_indices.scalar_type() == at::kInt || topk_indices.scalar_type() == at::kUInt32 ||
              topk_indices.scalar_type() == at::kLong,
              "topk_indices must be int32, uint32 or int64");
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, "topk_weights must be float32");
  TORCH_CHECK(gating_output.scalar_type() == at::kFloat || gating_output.scalar_type() == at::kHalf ||
              gating_output.scalar_type() == at::kBFloat16,
              "Unsupported gating_output data type: ", gating_output.scalar_type());
  TORCH_CHECK(gating_output.is_contiguous() && topk_weights.is_contiguous() &&
              topk_indices.is_contiguous() && token_expert_indices.is_contiguous(),
              "topk_softplus_sqrt expects contiguous tensors");
  if (correction_bias.has_value())
    TORCH_CHECK(correction_bias->scalar_type() == at::kFloat && correction_bias->is_contiguous(),
                "correction_bias must be contiguous float32");
  const void* ids_ptr = nullptr;
  const void* table_ptr = nullptr;
  if (tid2eid.has_value()) {
    TORCH_CHECK(input_ids.has_value(), "input_ids is required for hash MoE");
    TORCH_CHECK(input_ids->scalar_type() == topk_indices.scalar_type(),
                "input_ids dtype must match topk_indices dtype");
    TORCH_CHECK(tid2eid->scalar_type() == topk_indices.scalar_type(),
                "tid2eid dtype must match topk_indices dtype");
    TORCH_CHECK(input_ids->is_contiguous() && tid2eid->is_contiguous() && input_ids->numel() == num_tokens &&
                tid2eid->size(-1) == topk, "input_ids must be [num_tokens] and tid2eid [vocab, topk]");
    ids_ptr = input_ids->data_ptr();
    table_ptr = tid2eid->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(gating_output.device());
  check_status(b200moe_topk_softplus_sqrt(
      topk_weights.data_ptr<float>(), topk_indices.data_ptr(), index_dtype(topk_indices),
      token_expert_indices.data_ptr<int32_t>(), gating_output.data_ptr(),
      float_dtype(gating_output, "topk_softplus_sqrt"), num_tokens, num_experts, topk, renormalize,
      routed_scaling_factor, correction_bias.has_value() ? correction_bias->data_ptr<float>() : nullptr, ids_ptr,
      table_ptr, current_stream()));
}

std::tuple<at::Tensor, at::Tensor> grouped_topk(const at::Tensor& scores,
                                                const at::Tensor& scores_with_bias,
                                                int64_t n_group, int64_t topk_group, int64_t topk,
                                                bool renormalize, double routed_scaling_factor) {
  check_cuda(scores, "scores");
  TORCH_CHECK(scores_with_bias.dim() == 2, "scores_with_bias must be a 2D Tensor");
  TORCH_CHECK(scores.sizes() == scores_with_bias.sizes() &&
              scores.scalar_type() == scores_with_bias.scalar_type(),
              "scores and scores_with_bias must have the same shape and dtype");
  const int64_t num_tokens = scores_with_bias.size(0);
  const int64_t num_experts = scores_with_bias.size(1);
  TORCH_CHECK(n_group > 0 && num_experts % n_group == 0, "num_experts should be divisible by n_group");
  TORCH_CHECK(n_group <= 32, "n_group should be smaller than or equal to 32 for now");
  TORCH_CHECK(topk <= 32, "topk should be smaller than or equal to 32 for now");
  if (scores.scalar_type() != at::kFloat && scores.scalar_type() != at::kHalf &&
      scores.scalar_type() != at::kBFloat16)
    throw std::invalid_argument("Invalid dtype, only supports float16, float32, and bfloat16");
  const c10::cuda::CUDAGuard guard(scores.device());
  at::Tensor s = scores.contiguous(), sb = scores_with_bias.contiguous();
  at::Tensor values = at::empty({num_tokens, topk}, s.options());
  at::Tensor indices = at::empty({num_tokens, topk}, s.options().dtype(at::kInt));
  check_status(b200moe_grouped_topk(values.data_ptr(), indices.data_ptr<int32_t>(), s.data_ptr(),
                                    sb.data_ptr(), float_dtype(s, "grouped_topk"), num_tokens,
                                    (int)num_experts, (int)n_group, (int)topk_group, (int)topk,
                                    renormalize, routed_scaling_factor, current_stream()));
  return {values, indices};
}

void moe_align_block_size(at::Tensor topk_ids, int64_t num_experts, int64_t block_size,
                          at::Tensor sorted_token_ids, at::Tensor experts_ids,
                          at::Tensor num_tokens_post_pad,
                          std::optional<at::Tensor> maybe_expert_map) {
  check_cuda(topk_ids, "topk_ids");
  TORCH_CHECK(((num_experts + 31) / 32) * 32 < 1024, "padded_num_experts must be less than 1024");
  TORCH_CHECK(sorted_token_ids.scalar_type() == at::kInt && experts_ids.scalar_type() == at::kInt &&
              num_tokens_post_pad.scalar_type() == at::kInt,
              "moe_align_block_size outputs must be int32");
  TORCH_CHECK(topk_ids.is_contiguous() && sorted_token_ids.is_contiguous() &&
              experts_ids.is_contiguous(), "moe_align_block_size expects contiguous tensors");
  if (maybe_expert_map.has_value())
    TORCH_CHECK(maybe_expert_map->scalar_type() == at::kInt && maybe_expert_map->is_contiguous(),
                "expert_map must be int32");
  const c10::cuda::CUDAGuard guard(topk_ids.device());
  at::Tensor ws = sort_workspace(topk_ids, topk_ids.numel(), num_experts);
  check_status(b200moe_moe_align_block_size(
      topk_ids.data_ptr(), index_dtype(topk_ids), topk_ids.numel(), (int)num_experts,
      (int)block_size, sorted_token_ids.data_ptr<int32_t>(), sorted_token_ids.numel(),
      experts_ids.data_ptr<int32_t>(), experts_ids.numel(), num_tokens_post_pad.data_ptr<int32_t>(),
      maybe_expert_map.has_value() ? maybe_expert_map->data_ptr<int32_t>() : nullptr,
      ws.numel() ? ws.data_ptr() : nullptr, (size_t)ws.numel(), current_stream()));
}

void moe_sum(at::Tensor& input, at::Tensor& output, const std::optional<at::Tensor>& topk_ids,
             const std::optional<at::Tensor>& expert_map) {
  check_cuda(input, "input");
  const int hidden_size = input.size(-1);
  const int64_t num_tokens = hidden_size ? output.numel() / hidden_size : 0;
  const int topk = input.size(1);
  TORCH_CHECK(input.scalar_type() == output.scalar_type(),
              "moe_sum: input and output must have the same dtype");
  TORCH_CHECK(input.device() == output.device(),
              "moe_sum: input and output must be on the same device");
  TORCH_CHECK(input.is_contiguous() && output.is_contiguous(),
              "moe_sum expects contiguous input and output");
  TORCH_CHECK(input.numel() == output.numel() * topk,
              "moe_sum: input shape must be [num_tokens, topk, hidden] matching output "
              "[num_tokens, hidden]");
  TORCH_CHECK(!(expert_map.has_value() && !topk_ids.has_value()),
              "moe_sum: expert_map requires topk_ids to be provided");
  if (topk_ids.has_value()) {
    const auto& tk = topk_ids.value();
    TORCH_CHECK(tk.is_contiguous(), "moe_sum: topk_ids must be contiguous");
    TORCH_CHECK(tk.device() == input.device(), "moe_sum: topk_ids must be on the same device as input");
    TORCH_CHECK(tk.dim() == 2 && tk.size(0) == num_tokens && tk.size(1) == topk,
                "moe_sum: topk_ids must have shape [num_tokens, topk]");
    TORCH_CHECK(tk.scalar_type() == at::kInt || tk.scalar_type() == at::kLong,
                "moe_sum: topk_ids must be int32 or int64");
    if (expert_map.has_value()) {
      const auto& em = expert_map.value();
      TORCH_CHECK(em.scalar_type() == at::kInt, "moe_sum: expert_map must be int32");
      TORCH_CHECK(em.is_contiguous(), "moe_sum: expert_map must be contiguous");
      TORCH_CHECK(em.device() == input.device(), "moe_sum: expert_map must be on the same device as input");
    }
  }
  const c10::cuda::CUDAGuard guard(input.device());
  check_status(b200moe_moe_sum(
      output.data_ptr(), input.data_ptr(), float_dtype(input, "moe_sum"), num_tokens, topk,
      hidden_size, topk_ids.has_value() ? topk_ids->data_ptr() : nullptr,
      topk_ids.has_value() ? index_dtype(*topk_ids) : B200MOE_I32,
      expert_map.has_value() ? expert_map->data_ptr<int32_t>() : nullptr, current_stream()));
}

void moe_gather(at::Tensor& output, const at::Tensor& moe_output, const at::Tensor& topk_weights,
                const at::Tensor& unpermuted_row_to_permuted_row, int64_t num_experts) {
  check_cuda(output, "output");
  const int64_t num_tokens = topk_weights.size(0);
  const int topk = topk_weights.size(1);
  const int hidden_size = output.size(1);
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat, "topk_weights must be float32");
  if (output.scalar_type() != at::kHalf && output.scalar_type() != at::kBFloat16 &&
      output.scalar_type() != at::kFloat)
    throw std::runtime_error("Unsupported data type in moe_gather");
  TORCH_CHECK(moe_output.scalar_type() == output.scalar_type(),
              "moe_gather: moe_output and output must have the same dtype");
  TORCH_CHECK(unpermuted_row_to_permuted_row.scalar_type() == at::kInt,
              "moe_gather: unpermuted_row_to_permuted_row must be int32");
  TORCH_CHECK(output.is_contiguous() && moe_output.is_contiguous() && topk_weights.is_contiguous() &&
              unpermuted_row_to_permuted_row.is_contiguous(), "moe_gather expects contiguous tensors");
  const c10::cuda::CUDAGuard guard(output.device());
  check_status(b200moe_moe_gather(output.data_ptr(), moe_output.data_ptr(),
                                  topk_weights.data_ptr<float>(),
                                  unpermuted_row_to_permuted_row.data_ptr<int32_t>(),
                                  float_dtype(output, "moe_gather"), num_tokens, hidden_size, topk,
                                  current_stream()));
}

void init_expert_map(at::Tensor& expert_map, int64_t num_experts, int64_t ep_rank, int64_t ep_size) {
  check_cuda(expert_map, "expert_map");
  TORCH_CHECK(expert_map.scalar_type() == at::kInt, "expert_map must be int32");
  TORCH_CHECK(expert_map.numel() == num_experts * ep_size, "expert_map must be [num_experts * ep_size]");
  const c10::cuda::CUDAGuard guard(expert_map.device());
  check_status(b200moe_init_expert_map(expert_map.data_ptr<int32_t>(), (int)num_experts,
                                       (int)ep_rank, (int)ep_size, current_stream()));
}

struct RemapChecked {
  int64_t num_rows; int hidden, topk;
};

RemapChecked check_remap(const at::Tensor& hidden_states, const at::Tensor& remapped,
                         const std::optional<at::Tensor>& expert_map, const at::Tensor& rows_per_expert,
                         const at::Tensor& row_map, const at::Tensor& topk_ids,
                         int64_t total_experts_num, int64_t local_experts_num) {
  if (expert_map.has_value())
    TORCH_CHECK(expert_map->scalar_type() == at::kInt, "expert_map must be int32");
  TORCH_CHECK(rows_per_expert.scalar_type() == at::kInt, "rows_per_expert must be int32");
  TORCH_CHECK(topk_ids.scalar_type() == at::kLong || topk_ids.scalar_type() == at::kInt,
              "topk_ids must be int64 or int32");
  TORCH_CHECK(row_map.scalar_type() == at::kInt, "unpermuted_row_to_permuted_row must be int32");
  RemapChecked r;
  r.num_rows = hidden_states.size(0);
  r.hidden = hidden_states.size(1);
  r.topk = topk_ids.size(1);
  TORCH_CHECK(remapped.size(0) == r.num_rows * r.topk && hidden_states.size(1) == remapped.size(1),
              "remapped_hidden_states must be [num_rows * TopK, hidden_size]");
  if (expert_map.has_value())
    TORCH_CHECK(expert_map->size(0) == total_experts_num, "expert_map must be [total_experts_num]");
  TORCH_CHECK(rows_per_expert.size(0) == local_experts_num, "rows_per_expert must be [local_experts_num]");
  TORCH_CHECK(topk_ids.size(0) == r.num_rows && topk_ids.size(1) == r.topk,
              "topk_ids must be [num_rows, TopK]");
  TORCH_CHECK(hidden_states.is_contiguous() && remapped.is_contiguous() && topk_ids.is_contiguous() &&
              rows_per_expert.is_contiguous() && row_map.is_contiguous(),
              "remap_hidden_states expects contiguous tensors");
  if (local_experts_num > 1024)
    throw std::runtime_error("local_experts_num exceeds the maximum supported number");
  return r;
}

void remap_hidden_states(at::Tensor& hidden_states, const std::optional<at::Tensor>& hidden_states_scales,
                         at::Tensor& remapped_hidden_states,
                         const std::optional<at::Tensor>& remapped_hidden_states_scales,
                         const std::optional<at::Tensor>& expert_map, at::Tensor& rows_per_expert,
                         at::Tensor& unpermuted_row_to_permuted_row, at::Tensor& topk_ids,
                         int64_t total_experts_num, int64_t local_experts_num) {
  check_cuda(hidden_states, "hidden_states");
  TORCH_CHECK(hidden_states.scalar_type() == remapped_hidden_states.scalar_type(),
              "hidden_states and remapped_hidden_states must have save dtype");
  if (hidden_states_scales.has_value()) {
    TORCH_CHECK(remapped_hidden_states_scales.has_value(),
                "if hidden_states_scales is provided, remapped_hidden_states_scales "
                "must also be provided");
    TORCH_CHECK(hidden_states_scales->scalar_type() == remapped_hidden_states_scales->scalar_type(),
                "hidden_states_scales and remapped_hidden_states_scales must have save dtype");
  }
  RemapChecked r = check_remap(hidden_states, remapped_hidden_states, expert_map, rows_per_expert,
                               unpermuted_row_to_permuted_row, topk_ids, total_experts_num,
                               local_experts_num);
  int scale_cols = 0, scale_bytes = 0;
  if (hidden_states_scales.has_value()) {
    TORCH_CHECK(remapped_hidden_states_scales->size(0) == r.num_rows * r.topk &&
                hidden_states_scales->size(1) == remapped_hidden_states_scales->size(1),
                "remapped_hidden_states_scales must be [num_rows * TopK, hidden_size // block_k]");
    TORCH_CHECK(hidden_states_scales->is_contiguous() && remapped_hidden_states_scales->is_contiguous(),
                "remap_hidden_states expects contiguous scales");
    scale_cols = hidden_states_scales->size(1);
    scale_bytes = hidden_states_scales->element_size();
  }
  const int elem = hidden_states.element_size();
  if (elem != 1 && elem != 2 && elem != 4) throw std::runtime_error("Unsupported data type in hidden_states");
  const c10::cuda::CUDAGuard guard(hidden_states.device());
  at::Tensor ws = sort_workspace(hidden_states, r.num_rows * r.topk, local_experts_num);
  check_status(b200moe_remap_hidden_states(
      hidden_states.data_ptr(), hidden_states_scales.has_value() ? hidden_states_scales->data_ptr() : nullptr,
      remapped_hidden_states.data_ptr(),
      remapped_hidden_states_scales.has_value() ? remapped_hidden_states_scales->data_ptr() : nullptr,
      expert_map.has_value() ? expert_map->data_ptr<int32_t>() : nullptr,
      rows_per_expert.data_ptr<int32_t>(), unpermuted_row_to_permuted_row.data_ptr<int32_t>(),
      topk_ids.data_ptr(), index_dtype(topk_ids), r.num_rows, r.hidden, elem, scale_cols, scale_bytes,
      r.topk, (int)total_experts_num, (int)local_experts_num, ws.numel() ? ws.data_ptr() : nullptr,
      (size_t)ws.numel(), current_stream()));
}

// Not in the reference: permute fused with the dynamic 1x128 e4m3 quantisation.
void b200_remap_quant_fp8(at::Tensor& hidden_states, at::Tensor& remapped_q, at::Tensor& remapped_scales,
                          const std::optional<at::Tensor>& expert_map, at::Tensor& rows_per_expert,
                          at::Tensor& unpermuted_row_to_permuted_row, at::Tensor& topk_ids,
                          int64_t total_experts_num, int64_t local_experts_num) {
  check_cuda(hidden_states, "hidden_states");
  TORCH_CHECK(remapped_q.scalar_type() == at::kFloat8_e4m3fn, "remapped_q must be float8_e4m3fn");
  TORCH_CHECK(remapped_scales.scalar_type() == at::kFloat && remapped_scales.is_contiguous(),
              "remapped_scales must be contiguous float32");
  RemapChecked r = check_remap(hidden_states, remapped_q, expert_map, rows_per_expert,
                               unpermuted_row_to_permuted_row, topk_ids, total_experts_num,
                               local_experts_num);
  TORCH_CHECK(r.hidden % 128 == 0 && remapped_scales.size(0) == r.num_rows * r.topk &&
              remapped_scales.size(1) == r.hidden / 128,
              "remapped_scales must be [num_rows * TopK, hidden_size / 128]");
  const c10::cuda::CUDAGuard guard(hidden_states.device());
  at::Tensor ws = sort_workspace(hidden_states, r.num_rows * r.topk, local_experts_num);
  check_status(b200moe_remap_quant_fp8(
      hidden_states.data_ptr(), float_dtype(hidden_states, "b200_remap_quant_fp8"), remapped_q.data_ptr(),
      remapped_scales.data_ptr<float>(), expert_map.has_value() ? expert_map->data_ptr<int32_t>() : nullptr,
      rows_per_expert.data_ptr<int32_t>(), unpermuted_row_to_permuted_row.data_ptr<int32_t>(),
      topk_ids.data_ptr(), index_dtype(topk_ids), r.num_rows, r.hidden, r.topk, (int)total_experts_num,
      (int)local_experts_num, ws.numel() ? ws.data_ptr() : nullptr, (size_t)ws.numel(), current_stream()));
}


// ---- expert parallelism over peer memory (no counterpart in the reference) ----------
// `tables` is an int64 CPU tensor [6, ep]: for every rank the addresses, as this process
// sees them, of recv_rows, recv_scales, recv_ids, recv_weights, recv_counts, comb_rows.
b200moe_ep_peers make_peers(const at::Tensor& tables, int64_t ep_rank, int64_t num_local_experts,
                            int64_t topk, int64_t hidden, int64_t capacity, bool quantized) {
  TORCH_CHECK(tables.device().is_cpu() && tables.scalar_type() == at::kLong && tables.dim() == 2 &&
              tables.size(0) == 6 && tables.is_contiguous(), "tables must be an int64 CPU tensor [6, ep]");
  const int64_t ep = tables.size(1);
  TORCH_CHECK(ep >= 1 && ep <= B200MOE_MAX_EP, "at most ", B200MOE_MAX_EP, " expert-parallel ranks");
  b200moe_ep_peers pe = {};
  pe.ep_size = (int)ep; pe.ep_rank = (int)ep_rank; pe.num_local_experts = (int)num_local_experts;
  pe.topk = (int)topk; pe.hidden = (int)hidden; pe.quantized = quantized ? 1 : 0; pe.capacity = capacity;
  const int64_t* t = tables.data_ptr<int64_t>();
  for (int64_t d = 0; d < ep; ++d) {
    pe.recv_rows[d] = reinterpret_cast<void*>(t[0 * ep + d]);
    pe.recv_scales[d] = reinterpret_cast<float*>(t[1 * ep + d]);
    pe.recv_ids[d] = reinterpret_cast<int32_t*>(t[2 * ep + d]);
    pe.recv_weights[d] = reinterpret_cast<float*>(t[3 * ep + d]);
    pe.recv_counts[d] = reinterpret_cast<int32_t*>(t[4 * ep + d]);
    pe.comb_rows[d] = reinterpret_cast<void*>(t[5 * ep + d]);
  }
  return pe;
}

void b200_ep_dispatch(const at::Tensor& hidden_states, const at::Tensor& topk_ids, const at::Tensor& topk_weights,
                      at::Tensor& send_counts, at::Tensor& send_pos, at::Tensor& workspace,
                      const at::Tensor& tables, int64_t ep_rank, int64_t num_local_experts, int64_t capacity,
                      bool quantized, const std::optional<at::Tensor>& expert_slot) {
  check_cuda(hidden_states, "hidden_states");
  TORCH_CHECK(hidden_states.dim() == 2 && hidden_states.is_contiguous(), "hidden_states must be contiguous [T, H]");
  const int64_t T = hidden_states.size(0), H = hidden_states.size(1);
  TORCH_CHECK(topk_ids.dim() == 2 && topk_ids.size(0) == T && topk_ids.is_contiguous(), "topk_ids must be [T, K]");
  const int64_t K = topk_ids.size(1), ep = tables.size(1);
  TORCH_CHECK(topk_weights.scalar_type() == at::kFloat && topk_weights.is_contiguous() &&
              topk_weights.numel() == T * K, "topk_weights must be float32 [T, K]");
  TORCH_CHECK(send_counts.scalar_type() == at::kInt && send_counts.numel() == ep && send_counts.is_contiguous(),
              "send_counts must be int32 [ep]");
  TORCH_CHECK(send_pos.scalar_type() == at::kInt && send_pos.numel() == T * ep && send_pos.is_contiguous(),
              "send_pos must be int32 [T, ep]");
  b200moe_ep_peers pe = make_peers(tables, ep_rank, num_local_experts, K, H, capacity, quantized);
  if (expert_slot.has_value()) {
    check_cuda(*expert_slot, "expert_slot");
    TORCH_CHECK(expert_slot->scalar_type() == at::kInt && expert_slot->is_contiguous() &&
                expert_slot->numel() == ep * num_local_experts && expert_slot->device() == hidden_states.device(),
                "expert_slot must be int32 [ep * num_local_experts] on the device of hidden_states");
    pe.expert_slot = expert_slot->data_ptr<int32_t>();
  }
  const size_t need = b200moe_ep_dispatch_workspace_bytes(T, (int)ep);
  TORCH_CHECK((size_t)workspace.numel() * workspace.element_size() >= need, "workspace of ", need, " bytes needed");
  const c10::cuda::CUDAGuard guard(hidden_states.device());
  check_status(b200moe_ep_dispatch(&pe, hidden_states.data_ptr(), float_dtype(hidden_states, "b200_ep_dispatch"),
                                   topk_ids.data_ptr(), index_dtype(topk_ids), topk_weights.data_ptr<float>(), T,
                                   send_counts.data_ptr<int32_t>(), send_pos.data_ptr<int32_t>(),
                                   need ? workspace.data_ptr() : nullptr, need, current_stream()));
}

void b200_ep_mask_unused(const at::Tensor& anchor, const at::Tensor& tables, int64_t ep_rank,
                         int64_t num_local_experts, int64_t topk, int64_t hidden, int64_t capacity, bool quantized) {
  check_cuda(anchor, "anchor");
  const b200moe_ep_peers pe = make_peers(tables, ep_rank, num_local_experts, topk, hidden, capacity, quantized);
  const c10::cuda::CUDAGuard guard(anchor.device());
  check_status(b200moe_ep_mask_unused(&pe, current_stream()));
}

void b200_ep_combine(const at::Tensor& moe_output, const at::Tensor& row_map, const at::Tensor& tables,
                     int64_t ep_rank, int64_t num_local_experts, int64_t capacity, bool quantized) {
  check_cuda(moe_output, "moe_output");
  TORCH_CHECK(moe_output.dim() == 2 && moe_output.is_contiguous(), "moe_output must be contiguous [M, H]");
  const int64_t ep = tables.size(1);
  TORCH_CHECK(row_map.scalar_type() == at::kInt && row_map.is_contiguous() && row_map.dim() == 2 &&
              row_map.size(0) == ep * capacity, "row_map must be int32 [ep * capacity, K]");
  const b200moe_ep_peers pe = make_peers(tables, ep_rank, num_local_experts, row_map.size(1), moe_output.size(1),
                                         capacity, quantized);
  const c10::cuda::CUDAGuard guard(moe_output.device());
  check_status(b200moe_ep_combine(&pe, moe_output.data_ptr(), row_map.data_ptr<int32_t>(),
                                  float_dtype(moe_output, "b200_ep_combine"), current_stream()));
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(_moe_C, m) {
  m.def("moe_sum(Tensor input, Tensor! output, Tensor? topk_ids, Tensor? expert_map) -> ()");
  m.def(
      "moe_align_block_size(Tensor topk_ids, int num_experts,"
      "                     int block_size, Tensor! sorted_token_ids,"
      "                     Tensor! experts_ids,"
      "                     Tensor! num_tokens_post_pad,"
      "                     Tensor? maybe_expert_map) -> ()");
  m.def(
      "grouped_topk(Tensor scores, Tensor scores_with_bias, int n_group, int "
      "topk_group, int topk, bool renormalize, float "
      "routed_scaling_factor) -> (Tensor, Tensor)");
  m.def(
      "topk_softmax(Tensor! topk_weights, Tensor! topk_indices, Tensor! "
      "token_expert_indices, Tensor gating_output, bool renormalize, Tensor? "
      "bias) -> ()");
  m.def(
      "topk_sigmoid(Tensor! topk_weights, Tensor! topk_indices, Tensor! "
      "token_expert_indices, Tensor gating_output, bool renormalize, Tensor? "
      "bias, float routed_scaling_factor) -> ()");
  m.def(
      "batched_moe_align_block_size(int max_tokens_per_batch,"
      "                     int block_size, Tensor expert_num_tokens,"
      "                     Tensor! sorted_token_ids,"
      "                     Tensor! experts_ids,"
      "                     Tensor! num_tokens_post_pad) -> ()");
  m.def(
      "moe_lora_align_block_size(Tensor topk_ids,"
      "                     Tensor token_lora_mapping,"
      "                     int num_experts,"
      "                     int block_size, int max_loras, "
      "                     int max_num_tokens_padded, "
      "                     int max_num_m_blocks, "
      "                     Tensor! sorted_token_ids,"
      "                     Tensor! experts_ids,"
      "                     Tensor! num_tokens_post_pad,"
      "                     Tensor! adapter_enabled,"
      "                     Tensor! lora_ids,"
      "                     Tensor? maybe_expert_map) -> () ");
  m.def(
      "topk_softplus_sqrt(Tensor! topk_weights, Tensor! topk_indices, "
      "Tensor! token_expert_indices, Tensor gating_output, bool renormalize, "
      "float routed_scaling_factor, Tensor? correction_bias=None, Tensor? "
      "input_ids=None, Tensor? tid2eid=None) -> ()");
  m.def(
      "moe_gather(Tensor! output, Tensor moe_output, Tensor topk_weights, "
      "Tensor unpermuted_row_to_permuted_row, int num_experts) -> ()");
  m.def(
      "fused_moe_prologue(Tensor input, Tensor? input_scales, Tensor "
      "token_selected_experts, "
      "Tensor "
      "token_final_scales, Tensor workspace, int hidden_size, int inter_size, "
      "int block_k, "
      "int ep_rank, int ep_size,"
      "int num_experts_on_rank) -> "
      "()");
  m.def("init_expert_map(Tensor expert_map, int num_experts, int ep_rank, int ep_size) -> ()");
  m.def(
      "b200_ep_dispatch(Tensor hidden_states, Tensor topk_ids, Tensor topk_weights, Tensor(a!) send_counts, "
      "Tensor(b!) send_pos, Tensor(c!) workspace, Tensor tables, int ep_rank, int num_local_experts, "
      "int capacity, bool quantized, Tensor? expert_slot=None) -> ()");
  m.def(
      "b200_ep_mask_unused(Tensor anchor, Tensor tables, int ep_rank, int num_local_experts, int topk, "
      "int hidden, int capacity, bool quantized) -> ()");
  m.def(
      "b200_ep_combine(Tensor moe_output, Tensor row_map, Tensor tables, int ep_rank, int num_local_experts, "
      "int capacity, bool quantized) -> ()");
  m.def(
      "remap_hidden_states(Tensor hidden_states, Tensor? hidden_states_scales, "
      "Tensor remapped_hidden_states,"
      "Tensor? remapped_hidden_states_scales,"
      "Tensor? expert_map, Tensor rows_per_expert,"
      "Tensor unpermuted_row_to_permuted_row, Tensor topk_ids,"
      "int total_experts_num, int "
      "local_experts_num) -> "
      "()");
  m.def(
      "b200_remap_quant_fp8(Tensor hidden_states, Tensor! remapped_q, Tensor! remapped_scales, "
      "Tensor? expert_map, Tensor! rows_per_expert, Tensor! unpermuted_row_to_permuted_row, "
      "Tensor topk_ids, int total_experts_num, int local_experts_num) -> ()");
}

TORCH_LIBRARY_IMPL(_moe_C, CUDA, m) {
  m.impl("moe_sum", &moe_sum);
  m.impl("moe_align_block_size", &moe_align_block_size);
  m.impl("grouped_topk", &grouped_topk);
  m.impl("topk_softplus_sqrt", &topk_softplus_sqrt);
  m.impl("batched_moe_align_block_size", &batched_moe_align_block_size);
  m.impl("moe_lora_align_block_size", &moe_lora_align_block_size);
  m.impl("fused_moe_prologue", &fused_moe_prologue);
  m.impl("topk_softmax", &topk_softmax);
  m.impl("topk_sigmoid", &topk_sigmoid);
  m.impl("moe_gather", &moe_gather);
  m.impl("init_expert_map", &init_expert_map);
  m.impl("b200_ep_dispatch", &b200_ep_dispatch);
  m.impl("b200_ep_mask_unused", &b200_ep_mask_unused);
  m.impl("b200_ep_combine", &b200_ep_combine);
  m.impl("remap_hidden_states", &remap_hidden_states);
  m.impl("b200_remap_quant_fp8", &b200_remap_quant_fp8);
}

B200_REGISTER_EXTENSION(_moe_C)
