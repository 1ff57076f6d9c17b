/*
 * b200moe.h — C ABI of the B200 (sm_100a) fused Mixture-of-Experts kernels.
 *
 * Every entry point is `extern "C"`, takes plain device pointers, sizes and
 * small enums, enqueues its kernels on the CUDA stream it is given and returns
 * before they finish.  None of them synchronises.  None of them allocates
 * device memory: where a kernel needs scratch the caller passes it (see the
 * *_workspace_bytes helpers).  Return value: 0 on success, a negative
 * B200MOE_E_* code otherwise (b200moe_status_string() names it and
 * b200moe_last_error() holds a message for the calling thread).
 *
 * Each declaration names the reference interface it replaces, by the file's
 * path inside the vllm-xpu-kernels project.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element types of buffers crossing the boundary. */
typedef enum {
  B200MOE_F32 = 0,
  B200MOE_F16 = 1,
  B200MOE_BF16 = 2,
  B200MOE_FP8_E4M3 = 3, /* float8_e4m3fn                                  */
  B200MOE_U8 = 4,       /* raw bytes: e8m0 scales, packed e2m1 pairs      */
  B200MOE_I32 = 5,
  B200MOE_I64 = 6,
  B200MOE_U32 = 7,
  B200MOE_FP4X2 = 8, /* float4_e2m1fn_x2: two e2m1 codes per byte, low nibble first */
  B200MOE_FP8_E4M3_X2 = 9, /* two float8_e4m3fn planes [2][rows][cols]: value =
                              plane 0 + plane 1 (MXFP8 activations + residual) */
  B200MOE_I8 = 10 /* int8 */
} b200moe_dtype;

/* Status codes. */
enum {
  B200MOE_OK = 0,
  B200MOE_E_BADARG = -1,      /* shape / dtype / alignment rejected before launch */
  B200MOE_E_UNSUPPORTED = -2, /* valid request this build has no kernel for       */
  B200MOE_E_CUDA = -3,        /* a CUDA runtime / driver call failed              */
  B200MOE_E_WORKSPACE = -4,   /* workspace missing or too small                   */
  B200MOE_E_DEVICE_TIMEOUT = -5 /* a bounded device-side wait gave up             */
};

typedef void* b200moe_stream; /* a cudaStream_t */

const char* b200moe_status_string(int status);
/* Message of the last failing call made by this thread ("" if none). */
const char* b200moe_last_error(void);
/* ABI version: bumped when a signature changes. */
int b200moe_abi_version(void);

/* Status words.  The tensor-core kernels bound every wait on an mbarrier; a CTA
 * whose wait runs out raises a flag, all its warps leave, tensor memory is
 * freed and the caller's status word (b200moe_gemm_args.status) is set to 1 with
 * a plain store - the word may live in device memory or in mapped (pinned) host
 * memory, which a host can poll without synchronising.
 * b200moe_status_to_code turns the value read from such a word into B200MOE_OK or
 * B200MOE_E_DEVICE_TIMEOUT (with a message for b200moe_last_error).
 * b200moe_selftest_bounded_wait launches one small CTA that waits, with the
 * same wait routine and teardown as the GEMM kernels but a budget of
 * `budget_cycles` SM clock cycles (at most 2e8, about 0.1 s), on an mbarrier
 * nobody arrives at; it gives up, returns and sets *status = 1.  Hosts use it
 * to check that the failure path reaches them.  Neither function has a
 * counterpart in the reference (its kernels have no bounded waits). */
int b200moe_status_to_code(int32_t status_word);
int b200moe_selftest_bounded_wait(int32_t* status, int64_t budget_cycles,
                                  b200moe_stream stream);

/* ------------------------------------------------------------------------- */
/* Routing                                                                    */
/* ------------------------------------------------------------------------- */

/* Softmax top-k gating.  Replaces `topk_softmax` (csrc/moe/topk.cpp:848-898,
 * kernel :281-599; schema csrc/moe/torch_bindings.cpp:59-63).
 * gating [T,E] (f32/f16/bf16) -> topk_weights [T,K] f32, topk_indices [T,K]
 * (i32/u32/i64), token_expert_indices [T,K] i32 (= k*T + t).
 * bias (fp32 [E], may be NULL) is added for selection only. */
int b200moe_topk_softmax(float* topk_weights, void* topk_indices,
                         b200moe_dtype index_dtype,
                         int32_t* token_expert_indices, const void* gating,
                         b200moe_dtype gating_dtype, int64_t num_tokens,
                         int num_experts, int topk, int renormalize,
                         const float* bias, b200moe_stream stream);

/* Sigmoid top-k gating.  Replaces `topk_sigmoid` (csrc/moe/topk.cpp:900-952;
 * schema csrc/moe/torch_bindings.cpp:65-69). */
int b200moe_topk_sigmoid(float* topk_weights, void* topk_indices,
                         b200moe_dtype index_dtype,
                         int32_t* token_expert_indices, const void* gating,
                         b200moe_dtype gating_dtype, int64_t num_tokens,
                         int num_experts, int topk, int renormalize,
                         const float* bias, double routed_scaling_factor,
                         b200moe_stream stream);

/* sqrt(softplus) top-k gating (DeepSeek-V4 style).  Replaces `topk_softplus_sqrt`
 * (csrc/moe/topk_softplus_sqrt_kernels.cpp:701-772, kernel :205-400; schema
 * csrc/moe/torch_bindings.cpp:70-76).  score = sqrt(softplus(x)) (softplus(x) = x
 * above 20); selection on score + correction_bias, ties to the lower index;
 * weight = (score + bias) - bias; with `renormalize` divided by their sum (if
 * positive), times routed_scaling_factor.  With `tid2eid` ([vocab, topk], same
 * integer type as topk_indices) the ids of token t are row input_ids[t] of the
 * table and the weights their scores (non-finite -> 0). */
int b200moe_topk_softplus_sqrt(float* topk_weights, void* topk_indices,
                               b200moe_dtype index_dtype,
                               int32_t* token_expert_indices, const void* gating,
                               b200moe_dtype gating_dtype, int64_t num_tokens,
                               int num_experts, int topk, int renormalize,
                               double routed_scaling_factor,
                               const float* correction_bias,
                               const void* input_ids, const void* tid2eid,
                               b200moe_stream stream);

/* Group-limited top-k on already activated scores.  Replaces `grouped_topk`
 * (csrc/moe/grouped_topk.cpp:782-876, kernels :404-695; schema
 * csrc/moe/torch_bindings.cpp:53-57).
 * scores, scores_with_bias [T,E] (same dtype) -> topk_values [T,K] (same
 * dtype), topk_indices [T,K] i32. */
int b200moe_grouped_topk(void* topk_values, int32_t* topk_indices,
                         const void* scores, const void* scores_with_bias,
                         b200moe_dtype dtype, int64_t num_tokens,
                         int num_experts, int n_group, int topk_group,
                         int topk, int renormalize,
                         double routed_scaling_factor, b200moe_stream stream);

/* ------------------------------------------------------------------------- */
/* Alignment / permutation                                                    */
/* ------------------------------------------------------------------------- */

/* Scratch needed by b200moe_moe_align_block_size and
 * b200moe_remap_hidden_states for `numel` (= T*K) routed slots over
 * `num_experts` buckets.  0 when the single-block path is taken. */
size_t b200moe_sort_workspace_bytes(int64_t numel, int num_experts);

/* Replaces `moe_align_block_size` (csrc/moe/moe_align_sum_kernels.cpp:1034-1181;
 * schema csrc/moe/torch_bindings.cpp:14-20).
 * topk_ids [numel] (i32/i64/u32...) -> sorted_token_ids [sorted_len] i32 (slot
 * indices grouped by expert, each expert padded to block_size with `numel`),
 * expert_ids [expert_ids_len] i32, num_tokens_post_pad [1] i32.
 * Within one expert the slots appear in ascending order (the reference leaves
 * that order unspecified). */
int b200moe_moe_align_block_size(const void* topk_ids, b200moe_dtype ids_dtype,
                                 int64_t numel, int num_experts,
                                 int block_size, int32_t* sorted_token_ids,
                                 int64_t sorted_len, int32_t* expert_ids,
                                 int64_t expert_ids_len,
                                 int32_t* num_tokens_post_pad,
                                 const int32_t* expert_map, void* workspace,
                                 size_t workspace_bytes,
                                 b200moe_stream stream);

/* Same result as b200moe_moe_align_block_size, for callers that cannot supply
 * scratch memory: foreign-function hosts (cgo, JNI, ctypes) that are handed
 * only input and output buffers and own no device allocator, and serving
 * loops that must keep cudaMalloc - which serialises the device and can fail
 * once a framework's pool holds all memory - off their hot path.  The
 * scratch is a fixed 1 MiB array inside the library (held by every GPU that
 * loads it until the process ends; b200moe_noalloc_scratch_capacity() returns
 * its size); the call allocates nothing, neither directly nor through a
 * library.  Requests whose scratch need (b200moe_sort_workspace_bytes)
 * exceeds the array are refused with B200MOE_E_WORKSPACE before any launch.
 * The first call on each device looks up the array's device address, so make
 * that first call before any stream capture begins.  All calls on a device
 * share the one array: two calls whose kernels overlap on the GPU (different
 * streams, no ordering between them) race on it - serialise them.  The array
 * keeps whatever the previous call left; the kernels rewrite every cell they
 * read, so nothing needs clearing.
 * The device that is current at the call must be the one that owns `stream`
 * and the buffers (the array that is used is the current device's).  The
 * looked-up address is remembered per device ordinal for the life of the
 * process: after cudaDeviceReset on that device it is stale and the entry
 * point must not be used again in that process.
 * This entry point has no counterpart in the reference. */
int b200moe_moe_align_block_size_noalloc(const void* topk_ids,
                                         b200moe_dtype ids_dtype,
                                         int64_t numel, int num_experts,
                                         int block_size,
                                         int32_t* sorted_token_ids,
                                         int64_t sorted_len,
                                         int32_t* expert_ids,
                                         int64_t expert_ids_len,
                                         int32_t* num_tokens_post_pad,
                                         const int32_t* expert_map,
                                         b200moe_stream stream);
size_t b200moe_noalloc_scratch_capacity(void);

/* Replaces `batched_moe_align_block_size` (csrc/moe/moe_align_sum_kernels.cpp:1183-1222,
 * kernel :25-133; schema csrc/moe/torch_bindings.cpp:24-33).  Batch b owns token
 * slots [b*max_tokens, (b+1)*max_tokens) and has batch_num_tokens[b] of them in
 * use; sorted_ids [B * ceil(max_tokens/block) * block] lists them batch by batch,
 * each batch padded to whole blocks with the sentinel B*max_tokens; batch_ids holds
 * the batch of every block (-1 for unused blocks). */
int b200moe_batched_moe_align_block_size(int max_tokens_per_batch, int block_size,
                                         const int32_t* batch_num_tokens,
                                         int num_batches, int32_t* sorted_ids,
                                         int32_t* batch_ids,
                                         int32_t* num_tokens_post_pad,
                                         b200moe_stream stream);

/* Replaces `moe_lora_align_block_size` (csrc/moe/moe_align_sum_kernels.cpp:1374-1549,
 * kernels :732-1027; schema csrc/moe/torch_bindings.cpp:36-50).  For every entry
 * l = lora_ids[i], i in [0, max_loras], that is a valid enabled adapter
 * (0 <= l < max_loras, adapter_enabled[l] != 0) the slots whose token has
 * token_lora_mapping[token] == l are aligned like moe_align_block_size into
 * segment l of the outputs: sorted_token_ids[l*max_num_tokens_padded ...] (padding
 * = numel), expert_ids[l*max_num_m_blocks ...] (unused blocks = -1) and
 * num_tokens_post_pad[l].  Segments of other adapters are not written.  Slots of
 * one expert appear in ascending order (the reference leaves it unspecified). */
int b200moe_moe_lora_align_block_size(const void* topk_ids, b200moe_dtype ids_dtype,
                                      int64_t numel, int topk,
                                      const int32_t* token_lora_mapping,
                                      int num_experts, int block_size, int max_loras,
                                      int max_num_tokens_padded, int max_num_m_blocks,
                                      int32_t* sorted_token_ids, int32_t* expert_ids,
                                      int32_t* num_tokens_post_pad,
                                      const int32_t* adapter_enabled,
                                      const int32_t* lora_ids,
                                      const int32_t* expert_map, b200moe_stream stream);

/* Replaces `fused_moe_prologue` (csrc/moe/fused_moe_prologue.cpp:5-216, kernels
 * csrc/moe/fused_moe_prologue.hpp:153-709; schema csrc/moe/torch_bindings.cpp:83-92):
 * the routed rows that belong to this rank's experts
 * [ep_rank*num_experts_on_rank, (ep_rank+1)*num_experts_on_rank) are sorted by expert,
 * ascending token inside an expert, and written into the packed workspace whose ten
 * 256-byte aligned regions b200moe_fused_moe_prologue_layout returns, in this order:
 *   0 permuted_row_to_unpermuted_row i32 [T*K]  (unpermuted row = k*T + token)
 *   1 permuted_token_selected_experts i32 [T*K] (local expert id)
 *   2 unpermuted_row_to_permuted_row i32 [T*K]  (only cells of rows kept are written)
 *   3,4,5 scratch of the reference's three-step sort (sized as there, not written here)
 *   6 expert_first_token_offset i64 [E_local+1]
 *   7 permuted_token_final_scales f32 [T*K]
 *   8 permuted rows [T*K, hidden_size] of elem_bytes each
 *   9 permuted scale rows [T*K, hidden_size/block_k] of scale_elem_bytes each.
 * Rows and scales are moved as opaque bytes (bf16/fp16 2, fp8 and packed fp4 1; scales
 * f32 4 or e8m0 1; hidden_size counts storage elements).  `scratch` is caller memory of
 * b200moe_fused_moe_prologue_scratch_bytes bytes that the call may overwrite. */
int b200moe_fused_moe_prologue_layout(int64_t num_rows, int topk, int num_experts_on_rank,
                                      int64_t hidden_size, int block_k, int elem_bytes,
                                      int scale_elem_bytes, size_t offsets[10],
                                      size_t* total_bytes);
size_t b200moe_fused_moe_prologue_scratch_bytes(int64_t num_rows, int topk,
                                                int num_experts_on_rank);
int b200moe_fused_moe_prologue(const void* input, int elem_bytes, const void* input_scales,
                               int scale_elem_bytes, const int64_t* token_selected_experts,
                               const float* token_final_scales, void* workspace,
                               size_t workspace_bytes, int64_t num_rows, int64_t hidden_size,
                               int block_k, int topk, int ep_rank, int ep_size,
                               int num_experts_on_rank, void* scratch, size_t scratch_bytes,
                               b200moe_stream stream);

/* Replaces `init_expert_map` (csrc/moe/init_expert_map.cpp:78-95; schema
 * csrc/moe/torch_bindings.cpp:93-98). expert_map has num_local*ep_size ints. */
int b200moe_init_expert_map(int32_t* expert_map, int num_local_experts,
                            int ep_rank, int ep_size, b200moe_stream stream);

/* Replaces `remap_hidden_states` (csrc/moe/remap_hidden_states.cpp:418-568;
 * schema csrc/moe/torch_bindings.cpp:99-108).
 * hidden [T,H] (elem_bytes per element: 1, 2 or 4), optional scales
 * [T,scale_cols] (scale_elem_bytes each) -> remapped [T*K,H] expert-major,
 * remapped_scales, rows_per_expert [E_local] i32,
 * row_map (= unpermuted_row_to_permuted_row) [T,K] i32 (-1 = not local).
 * Rows of one expert keep ascending (t,k) order. */
int b200moe_remap_hidden_states(const void* hidden, const void* scales,
                                void* remapped, void* remapped_scales,
                                const int32_t* expert_map,
                                int32_t* rows_per_expert, int32_t* row_map,
                                const void* topk_ids, b200moe_dtype ids_dtype,
                                int64_t num_rows, int hidden_size,
                                int elem_bytes, int scale_cols,
                                int scale_elem_bytes, int topk,
                                int total_experts, int local_experts,
                                void* workspace, size_t workspace_bytes,
                                b200moe_stream stream);

/* Fused permute + dynamic per-1x128 fp8 (e4m3) quantisation of bf16/f16
 * activations: same bookkeeping as b200moe_remap_hidden_states, but the
 * remapped rows are written as fp8 [T*K,H] with fp32 scales [T*K,H/128]
 * (the math of b200moe_per_token_group_fp8_quant with group 128, eps 1e-10).
 * No counterpart op in the reference: it runs `quant_fp8_block_act`
 * (vllm_xpu_kernels/moe_utils.py:150-166) and `remap_hidden_states` as two
 * steps. */
int b200moe_remap_quant_fp8(const void* hidden, b200moe_dtype dtype,
                            void* remapped_q, float* remapped_scales,
                            const int32_t* expert_map,
                            int32_t* rows_per_expert, int32_t* row_map,
                            const void* topk_ids, b200moe_dtype ids_dtype,
                            int64_t num_rows, int hidden_size, int topk,
                            int total_experts, int local_experts,
                            void* workspace, size_t workspace_bytes,
                            b200moe_stream stream);

/* ------------------------------------------------------------------------- */
/* Grouped GEMM                                                               */
/* ------------------------------------------------------------------------- */

typedef enum {
  B200MOE_W_BF16_KN = 0,  /* 16-bit weights [E,K,N] (dtype = activation dtype)      */
  B200MOE_W_BF16_NK = 1,  /* 16-bit weights [E,N,K]                                 */
  B200MOE_W_FP8_TENSOR_KN = 2, /* fp8 e4m3 [E,K,N] + fp32 scale [E]                 */
  B200MOE_W_FP8_BLOCK_NK = 3,  /* fp8 e4m3 [E,N,K] + fp32 scales [E,N/128,K/128]    */
  B200MOE_W_FP8_BLOCK_KN = 4,  /* fp8 e4m3 [E,K,N] + same scales                    */
  B200MOE_W_MXFP4_NK = 5, /* e2m1 pairs [E,N,K/2] + e8m0 bytes [E,N,K/32]           */
  B200MOE_W_FP8E5M2_TENSOR_KN = 6, /* fp8 e5m2 [E,K,N] + fp32 scale [E]               */
  B200MOE_W_INT4_NK = 7,  /* two's-complement 4-bit pairs [E,N,K/2] (low nibble = even k)
                             + scales [E,N,K/group_size] in the activation dtype   */
  B200MOE_W_MXFP8_KN = 8  /* fp8 e4m3 [E,K,N] + e8m0 bytes [E,K/32,N] (one per 32 K rows) */
} b200moe_weight_format;

typedef enum {
  B200MOE_EPI_NONE = 0,      /* D = acc (+bias)                                     */
  B200MOE_EPI_SILU_MUL = 1,  /* D[m,i] = silu(acc[m,i]) * acc[m,I+i], D is [M,N/2]  */
  B200MOE_EPI_SWIGLUOAI = 2  /* D[m,i] from acc[m,2i], acc[m,2i+1], D is [M,N/2]    */
} b200moe_epilogue;

/* Arguments of the grouped GEMM.  Replaces `cutlass_grouped_gemm_interface`
 * (csrc/xpu/grouped_gemm/grouped_gemm_interface.cpp:12-60 ->
 * xe_2/grouped_gemm_xe2_interface.hpp:162-431; schema
 * csrc/xpu/torch_bindings.cpp:46-53).
 * For each expert e with rows_e = rows_per_expert[e] > 0 and r0 = sum of the
 * earlier experts' rows:  D[r0:r0+rows_e, :] = A[r0:r0+rows_e, :] * W_e^T
 * (+ bias_e), fp32 accumulation, result cast to d_dtype. */
typedef struct {
  const void* a;          /* [M,K] a_dtype, row-major, 16-byte aligned            */
  b200moe_dtype a_dtype;  /* BF16, F16, or FP8_E4M3 (with a_scale)                */
  const void* a_scale;    /* fp8 activations: block-fp8 weights: fp32 [M,K/128];
                             MXFP4 weights (MXFP8 activations, a_dtype FP8_E4M3
                             or FP8_E4M3_X2): e8m0 bytes as 32-bit words
                             [planes][ceil(K/128)][M], the output of
                             b200moe_quant_mxfp8; else NULL                  */
  const void* w;          /* weights, layout per w_format                         */
  b200moe_weight_format w_format;
  const void* w_scale;    /* per w_format, else NULL                              */
  const void* bias;       /* [E,N] in d_dtype, or NULL                            */
  void* d;                /* [M,N] (or [M,N/2] with a gated epilogue) d_dtype     */
  b200moe_dtype d_dtype;  /* BF16 or F16; FP8_E4M3 with EPI_SILU_MUL on fp8 x
                             block-scaled fp8: the activated values leave the
                             kernel quantised per token and 128 features, as
                             b200moe_silu_and_mul_per_block_quant would quantise
                             the unfused output (same values)                     */
  const int32_t* rows_per_expert; /* [E] device                                   */
  int64_t m;              /* rows of A and D (upper bound of the rows in use)     */
  int n, k, num_experts;
  b200moe_epilogue epilogue;
  float act_alpha, act_limit; /* SwigluOAI parameters                             */
  float clamp_limit;      /* >0: gate=min(gate,L), up=clamp(up,-L,L) before the
                             gated epilogue (only with a gated epilogue)          */
  int32_t* status;        /* int the device can write (device memory or mapped host
                             memory): set to 1 if a bounded wait gave up; may be
                             NULL                                                 */
  int impl;               /* 0 = auto, 1 = tensor-core kernel, 2 = plain-CUDA
                             checking kernel, 3 = tensor-core kernel without the
                             CTA-pair forms (16-bit prefill tiles then run one CTA
                             per tile; same results), 4 = tensor-core kernel with
                             the CTA-pair form wherever one exists                */
  int max_ctas;           /* >0: the persistent tensor-core kernel uses at most this
                             many CTAs (leaves SMs to a concurrent collective);
                             0 = one per SM                                       */
  int group_size;         /* INT4 weights: K elements per scale (32, 64, 128 or 256);
                             ignored otherwise                                    */
  int w_experts;          /* 0 or num_experts: one weight set per row segment.  Else
                             (a divisor of num_experts) rows_per_expert has
                             num_experts segments and segment s multiplies with weight
                             set s % w_experts: the rows of an expert-parallel
                             exchange as they arrive, grouped by source rank and by
                             local expert inside a source, need no second
                             permutation.  16-bit and block-scaled fp8 weights.     */
  void* d_scale;          /* FP8_E4M3 output: fp32 scales [M, N/256]; else NULL     */
  b200moe_dtype mid_dtype;/* FP8_E4M3 output: BF16 or F16, the type the
                             pre-activation values (and the bias) have: they are
                             rounded to it before the activation, as the unfused
                             GEMM's output would be                                */
  int64_t rows_hint;      /* 0, or the number of rows expected to be in use when `m`
                             is only a loose upper bound (buffers sized for the worst
                             case): tile sizes are picked for rows_hint / num_experts
                             rows per expert.  Never changes the result.            */
} b200moe_gemm_args;

int b200moe_grouped_gemm(const b200moe_gemm_args* args, b200moe_stream stream);

/* ------------------------------------------------------------------------- */
/* Activations, quantisation, reductions                                      */
/* ------------------------------------------------------------------------- */

/* Replaces `silu_and_mul` (csrc/activation.cpp:492-499, kernel :146-184;
 * schema csrc/torch_bindings.cpp:80-81). in [rows,2d] -> out [rows,d]. */
int b200moe_silu_and_mul(void* out, const void* in, b200moe_dtype dtype,
                         int64_t rows, int d, b200moe_stream stream);

/* Replaces `swigluoai_and_mul` (csrc/activation.cpp:683-689, kernel :313-346;
 * schema csrc/torch_bindings.cpp:187-191). Interleaved gate/up. */
int b200moe_swigluoai_and_mul(void* out, const void* in, b200moe_dtype dtype,
                              int64_t rows, int d, float alpha, float limit,
                              b200moe_stream stream);

/* Replace `gelu_and_mul`, `gelu_tanh_and_mul` (csrc/activation.cpp:53-75, 576-592;
 * schema csrc/torch_bindings.cpp:112-116): in [rows,2d] -> out [rows,d] =
 * T(gelu(x)) *_T y, erf form / tanh form. */
int b200moe_gelu_and_mul(void* out, const void* in, b200moe_dtype dtype,
                         int64_t rows, int d, b200moe_stream stream);
int b200moe_gelu_tanh_and_mul(void* out, const void* in, b200moe_dtype dtype,
                              int64_t rows, int d, b200moe_stream stream);

/* Replaces `swiglustep_and_mul` (csrc/activation.cpp:299-312, 351-378, 711-716;
 * schema csrc/torch_bindings.cpp:197-201): gate = first half, up = second;
 * out = T(min(silu(gate), limit) * clamp(up, -limit, limit)) in fp32. */
int b200moe_swiglustep_and_mul(void* out, const void* in, b200moe_dtype dtype,
                               int64_t rows, int d, float limit,
                               b200moe_stream stream);

/* Replaces `relu2_no_mul` (csrc/activation.cpp:45-50, 674-681; schema
 * csrc/torch_bindings.cpp:193-195): out [rows,d] = T(max(x,0)^2), no gating. */
int b200moe_relu2_no_mul(void* out, const void* in, b200moe_dtype dtype,
                         int64_t rows, int d, b200moe_stream stream);

/* Replaces `per_token_group_fp8_quant` (csrc/quantization/fp8/fp8_quant.cpp:724-840,
 * kernel :278-390; schema csrc/torch_bindings.cpp:170-177).
 * x [rows,cols] -> q [rows,cols] e4m3, s [rows,cols/group] fp32 with element
 * strides (s_stride_row, s_stride_col). */
int b200moe_per_token_group_fp8_quant(const void* x, b200moe_dtype dtype,
                                      void* q, float* s, int64_t rows,
                                      int cols, int group_size, float eps,
                                      int scale_ue8m0, int64_t s_stride_row,
                                      int64_t s_stride_col,
                                      b200moe_stream stream);

/* Replaces `silu_and_mul_per_block_quant`
 * (csrc/quantization/fused_kernels/fused_silu_mul_block_quant.cpp:141-239, kernel
 * :14-128; schema csrc/torch_bindings.cpp:89-101).  in [rows, 2*hidden] (gate |
 * up) -> out [rows, hidden] e4m3 or int8 of silu(gate)*up (fp32) divided by a
 * per-group scale = max(amax/448, 1/(448*512)) (int8: max(amax/127, FLT_EPSILON)),
 * optionally capped by *scale_ub and rounded up to a power of two; scales
 * fp32 at [row*s_stride_row + group*s_stride_group]. */
int b200moe_silu_and_mul_per_block_quant(void* out, b200moe_dtype out_dtype,
                                         float* scales, const void* in,
                                         b200moe_dtype dtype, int64_t rows,
                                         int hidden, int group_size,
                                         const float* scale_ub,
                                         int64_t s_stride_row,
                                         int64_t s_stride_group,
                                         int scale_ue8m0, b200moe_stream stream);

/* The same with e4m3 output, group 128 and dense scales [rows, hidden/128], for row buffers
 * that are sized for a worst case: only the first sum(rows_per_segment[0..num_segments))
 * rows are in use (the expert-major rows of a grouped GEMM and its device-side row counts)
 * and only those are read and written.  No counterpart op in the reference, whose layer
 * sizes its buffers exactly (vllm_xpu_kernels/fused_moe_interface.py:336-396). */
int b200moe_silu_and_mul_per_block_quant_ragged(void* out, float* scales, const void* in,
                                                b200moe_dtype dtype, int64_t rows,
                                                int hidden,
                                                const int32_t* rows_per_segment,
                                                int num_segments,
                                                b200moe_stream stream);

/* Replaces `silu_and_mul_mxfp4_quant`
 * (csrc/quantization/fused_kernels/fused_silu_mul_mxfp4_quant.cpp:134-210, kernel
 * :19-131; schema csrc/torch_bindings.cpp:103-107).  in [rows, 2*hidden] ->
 * out [rows, hidden/2] packed e2m1 (low nibble = even element) of
 * silu(gate)*up, scales fp32 powers of two = ceil_pow2(max(amax/6, eps)) per 32. */
int b200moe_silu_and_mul_mxfp4_quant(void* out, float* scales, const void* in,
                                     b200moe_dtype dtype, int64_t rows,
                                     int hidden, float eps,
                                     int64_t s_stride_row,
                                     int64_t s_stride_group,
                                     b200moe_stream stream);

/* Replaces `per_token_group_quant_mxfp4` (csrc/quantization/fp4/mxfp4_quant.cpp:24-126,
 * kernel mxfp4_quant.h:133-245; schema csrc/torch_bindings.cpp:180-184).
 * in [rows, hidden] f32/f16/bf16 -> out_q [rows, hidden/2], out_s as above.
 * Rows must be a multiple of 32 values long (the reference's scalar path for
 * groups that straddle rows is not built). */
int b200moe_per_token_group_quant_mxfp4(const void* in, b200moe_dtype dtype,
                                        void* out_q, float* out_s, int64_t rows,
                                        int hidden, float eps,
                                        int64_t s_stride_row,
                                        int64_t s_stride_group,
                                        b200moe_stream stream);

/* Replaces `silu_and_mul_quant` (csrc/activation.cpp:552-566, kernel :191-234;
 * schema csrc/torch_bindings.cpp:84-86): out [rows,d] e4m3 =
 * clamp(float(T(silu(x)) *_T y) * (1 / *scale)), static per-tensor scale. */
int b200moe_silu_and_mul_quant(void* out, const void* in, b200moe_dtype dtype,
                               const float* scale, int64_t rows, int d,
                               b200moe_stream stream);

/* MX-format activation quantisation for the block-scaled MXFP4 GEMM: per 32
 * consecutive values of a row one e8m0 scale byte b (2^(b-127) is the smallest
 * power of two with amax / scale <= 448, floor 1e-10) and e4m3 codes of
 * x / scale.  With terms == 2 a second plane holds the residual
 * x - code * scale quantised the same way (activation = plane 0 + plane 1).
 * x [rows,cols] bf16/f16 -> q [terms][rows,cols] e4m3, s: 32-bit words
 * [terms][ceil(cols/128)][rows]; byte (g & 3) of word [g >> 2][row] is the
 * scale of group g, bytes of groups past the row end are 0x7f.
 * No reference counterpart as an op: the reference's device kernel for MXFP4
 * keeps 16-bit activations (csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:411-471);
 * the one-plane math is `per_token_group_fp8_quant` with group 32 and
 * scale_ue8m0 (csrc/quantization/fp8/fp8_quant.cpp:340-387). */
int b200moe_quant_mxfp8(const void* x, b200moe_dtype dtype, void* q, void* s,
                        int64_t rows, int cols, int terms,
                        b200moe_stream stream);

/* Replaces `moe_gather` (csrc/moe/moe_gather.cpp:161-204; schema
 * csrc/moe/torch_bindings.cpp:78-82).
 * out[t,:] = sum_k w[t,k] * moe_out[row_map[t,k],:] (fp32), skipping -1. */
int b200moe_moe_gather(void* out, const void* moe_out,
                       const float* topk_weights, const int32_t* row_map,
                       b200moe_dtype dtype, int64_t num_tokens, int hidden,
                       int topk, b200moe_stream stream);

/* Replaces `moe_sum` (csrc/moe/moe_align_sum_kernels.cpp:1224-1372; schema
 * csrc/moe/torch_bindings.cpp:7-10).
 * out[t,:] = sum_k in[t,k,:] (fp32); with topk_ids a slot is skipped when its
 * id < 0 or expert_map[id] < 0. */
int b200moe_moe_sum(void* out, const void* in, b200moe_dtype dtype,
                    int64_t num_tokens, int topk, int hidden,
                    const void* topk_ids, b200moe_dtype ids_dtype,
                    const int32_t* expert_map, b200moe_stream stream);

/* ------------------------------------------------------------------------- */
/* Expert parallelism over peer memory                                        */
/* ------------------------------------------------------------------------- */

/* The reference has no communication layer: its expert parallelism is the
 * per-rank mask of `init_expert_map` (csrc/moe/init_expert_map.cpp:33-53,
 * vllm_xpu_kernels/fused_moe_interface.py:256-271), which leaves every rank with
 * all tokens.  These three entry points add token dispatch and combine for one
 * process per GPU: every rank keeps receive buffers that its peers can address
 * (symmetric memory or IPC mappings; over NVLink), and the kernels below store
 * straight into them with ordinary global stores - no staging copy, no host
 * read of any count.  Every rank holds num_local_experts experts: expert g sits in
 * slot expert_slot[g] (slot g without a table), on rank slot / num_local_experts as
 * its local expert slot % num_local_experts.  The table lets a deployment place
 * experts by load instead of contiguously.
 *
 * Buffers of rank d, each in `ep_size` regions of `capacity` rows, region s
 * written by source rank s (capacity >= the tokens any rank dispatches per call):
 *   recv_rows    [ep][capacity][row_bytes]   the token's row: e4m3 (hidden bytes,
 *                                            with recv_scales) or 16-bit
 *   recv_scales  [ep][capacity][hidden/128]  fp32, only with quantised rows
 *   recv_ids     [ep][capacity][topk] i32    the token's expert ids local to rank d
 *                                            (-1 for experts of other ranks)
 *   recv_weights [ep][capacity][topk] f32    routing weights (0 for those slots)
 *   recv_counts  [ep] i32                    rows received from each source
 *   comb_rows    [ep][capacity][hidden]      16-bit partial sums coming back:
 *                                            region d holds what rank d computed
 * The tables below hold, for every rank, the address of that rank's buffer as
 * this process sees it.
 *
 * One layer call is: b200moe_ep_dispatch on every rank; a barrier between the
 * ranks (any mechanism that orders the peers' kernels, e.g. a small NCCL
 * all-reduce on the same stream); b200moe_ep_mask_unused, the local experts on
 * the [ep*capacity] received rows as a top-k layer, b200moe_ep_combine; a second
 * barrier; b200moe_moe_gather over comb_rows with send_pos as the row map and
 * unit weights.  No kernel here waits for another rank: ordering comes from the
 * barriers between the launches. */
#define B200MOE_MAX_EP 16
typedef struct {
  int ep_size, ep_rank;
  int num_local_experts;
  int topk;
  int hidden;
  int quantized;          /* 1: rows travel as e4m3 + 1x128 fp32 scales, 0: 16-bit */
  int64_t capacity;
  void* recv_rows[B200MOE_MAX_EP];
  float* recv_scales[B200MOE_MAX_EP];
  int32_t* recv_ids[B200MOE_MAX_EP];
  float* recv_weights[B200MOE_MAX_EP];
  int32_t* recv_counts[B200MOE_MAX_EP];
  void* comb_rows[B200MOE_MAX_EP];
  const int32_t* expert_slot; /* device, [ep_size * num_local_experts]: a permutation
                                 of the slots, the same on every rank; NULL = identity */
} b200moe_ep_peers;

/* Scratch of b200moe_ep_dispatch for `num_tokens` tokens. */
size_t b200moe_ep_dispatch_workspace_bytes(int64_t num_tokens, int ep_size);

/* Sends every token once to every rank that owns at least one of its experts.
 * hidden [T,H] bf16/f16 (quantised on the way to e4m3 with dynamic 1x128 scales
 * when peers->quantized, the math of b200moe_per_token_group_fp8_quant), topk_ids
 * [T,K] global expert ids, topk_weights [T,K].  Outputs on this rank:
 * send_counts [ep] (rows sent to each rank) and send_pos [T,ep] = d * capacity +
 * the row's index among this rank's rows for rank d (ascending token order), -1
 * where the token does not go to d.  The same index addresses the row in region
 * `ep_rank` of rank d's receive buffers and, later, the partial sum in region d
 * of this rank's comb_rows. */
int b200moe_ep_dispatch(const b200moe_ep_peers* peers, const void* hidden,
                        b200moe_dtype dtype, const void* topk_ids,
                        b200moe_dtype ids_dtype, const float* topk_weights,
                        int64_t num_tokens, int32_t* send_counts,
                        int32_t* send_pos, void* workspace,
                        size_t workspace_bytes, b200moe_stream stream);

/* After the barrier: marks the rows of this rank's recv_ids that no source
 * filled in this call (index >= recv_counts[s] in region s) with -1, so the local
 * top-k layer skips them. */
int b200moe_ep_mask_unused(const b200moe_ep_peers* peers, b200moe_stream stream);

/* The weighted top-k reduction of the local experts' output, stored straight
 * into the source ranks' comb_rows: for received row i of region s
 *   comb_rows[s][ep_rank][i][:] = sum_k recv_weights[s][i][k] * moe_out[row_map[s*capacity+i][k]][:]
 * (fp32, k ascending, row_map -1 skipped; the math of b200moe_moe_gather).
 * moe_out [M,H] and the result are `dtype` (bf16/f16); row_map [ep*capacity, topk]. */
int b200moe_ep_combine(const b200moe_ep_peers* peers, const void* moe_out,
                       const int32_t* row_map, b200moe_dtype dtype,
                       b200moe_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
