// Token -> expert bookkeeping: moe_align_block_size, remap_hidden_states,
// init_expert_map and the fused permute + fp8 group quantisation.
//
// Both ops are a stable counting sort of the T*K routed slots by (mapped)
// expert id.  The slots are cut into chunks of 256 handled by one warp each:
//   1. count : every warp builds a histogram of its chunk,
//   2. scan  : per expert an exclusive scan over the chunks, then a scan over
//              the experts (padded to block_size for the align op),
//   3. rank  : every warp walks its chunk 32 slots at a time; the rank of a
//              slot among equal ids in the same step comes from
//              __match_any_sync, so slots of one expert keep ascending order.
// Up to 2048 slots all three steps run in one block without any scratch;
// beyond that they are three launches that exchange the histograms through a
// caller-provided workspace.  The result is deterministic: no atomics decide
// an order.
//
// Semantics follow csrc/moe/moe_align_sum_kernels.cpp:135-273, 1034-1181 and
// csrc/moe/remap_hidden_states.cpp:42-116, 181-330 of vllm-xpu-kernels, which
// leave the order inside an expert unspecified.
#include <atomic>

#include "common.cuh"
#include "sort.cuh"

namespace b200moe {
namespace {

// ------------------------- row copy ------------------------------------------
// One block per token: the row is read once and written to its K destinations.
__global__ void __launch_bounds__(256)
remap_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                  const uint8_t* __restrict__ src_s, uint8_t* __restrict__ dst_s,
                  const int32_t* __restrict__ row_map, int row_bytes,
                  int scale_row_bytes, int K) {
  const int64_t tok = blockIdx.x;
  __shared__ int dest[32];
  if (threadIdx.x < K) dest[threadIdx.x] = row_map[tok * K + threadIdx.x];
  __syncthreads();
  const uint8_t* s = src + tok * (int64_t)row_bytes;
  const int nvec = row_bytes >> 4;
  for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
    const vec16 v = ld16(s + (int64_t)j * 16);
    for (int k = 0; k < K; ++k) {
      const int r = dest[k];
      if (r >= 0) st16(dst + (int64_t)r * row_bytes + (int64_t)j * 16, v);
    }
  }
  if (src_s != nullptr) {
    const uint8_t* ss = src_s + tok * (int64_t)scale_row_bytes;
    if ((scale_row_bytes & 3) == 0) {
      for (int j = threadIdx.x; j < (scale_row_bytes >> 2); j += blockDim.x) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(ss)[j];
        for (int k = 0; k < K; ++k) {
          const int r = dest[k];
          if (r >= 0) reinterpret_cast<uint32_t*>(dst_s + (int64_t)r * scale_row_bytes)[j] = v;
        }
      }
    } else {
      for (int j = threadIdx.x; j < scale_row_bytes; j += blockDim.x) {
        const uint8_t v = ss[j];
        for (int k = 0; k < K; ++k) {
          const int r = dest[k];
          if (r >= 0) dst_s[(int64_t)r * scale_row_bytes + j] = v;
        }
      }
    }
  }
}

// Row copy fused with the per-1x128 dynamic e4m3 quantisation.  A lane holds 8
// consecutive elements, 16 lanes cover one 128-wide group.
template <typename T>
__global__ void __launch_bounds__(256)
remap_quant_kernel(const T* __restrict__ src, uint8_t* __restrict__ dst_q,
                   float* __restrict__ dst_s, const int32_t* __restrict__ row_map,
                   int H, int K) {
  const int64_t tok = blockIdx.x;
  __shared__ int dest[32];
  if (threadIdx.x < K) dest[threadIdx.x] = row_map[tok * K + threadIdx.x];
  __syncthreads();
  const T* s = src + tok * (int64_t)H;
  const int groups = H / 128;
  const int nvec = H / 8;
  // Full warps iterate together so the 16-lane shuffles stay converged.
  for (int j0 = (threadIdx.x & ~31); j0 < nvec; j0 += blockDim.x) {
    const int j = j0 + (threadIdx.x & 31);
    float x[8];
    float amax = 0.f;
    if (j < nvec) {
      const vec16 v = ld16(s + (int64_t)j * 8);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) { x[i] = to_f32<T>(e[i]); amax = fmaxf(amax, fabsf(x[i])); }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
#pragma unroll
    for (int mask = 8; mask > 0; mask >>= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
    amax = fmaxf(amax, 1e-10f);
    const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1.0f / (448.f * 512.f));
    const float inv = __fdiv_rn(1.0f, scale);
    if (j < nvec) {
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float q = fminf(fmaxf(__fmul_rn(x[i], inv), -448.f), 448.f);
        lo |= (uint32_t)f32_to_e4m3(q) << (8 * i);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float q = fminf(fmaxf(__fmul_rn(x[4 + i], inv), -448.f), 448.f);
        hi |= (uint32_t)f32_to_e4m3(q) << (8 * i);
      }
      const int g = j / 16;
      for (int k = 0; k < K; ++k) {
        const int r = dest[k];
        if (r >= 0) {
          *reinterpret_cast<uint2*>(dst_q + (int64_t)r * H + (int64_t)j * 8) = make_uint2(lo, hi);
          if ((j & 15) == 0) dst_s[(int64_t)r * groups + g] = scale;
        }
      }
    }
  }
}

__global__ void init_expert_map_kernel(int32_t* map, int n_local, int ep_rank, int total) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g < total) {
    const int lo = ep_rank * n_local;
    map[g] = (g >= lo && g < lo + n_local) ? g - lo : -1;
  }
}

int check_ids_dtype(b200moe_dtype t, const char* name) {
  if (t == B200MOE_I32 || t == B200MOE_I64 || t == B200MOE_U32) return 0;
  return fail(B200MOE_E_BADARG, "%s: topk_ids must be int64 or int32", name);
}

int remap_bookkeeping(const int32_t* expert_map, int32_t* rows_per_expert,
                      int32_t* row_map, const void* topk_ids, b200moe_dtype ids_dtype,
                      int64_t num_rows, int topk, int total_experts, int local_experts,
                      void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (check_ids_dtype(ids_dtype, "remap_hidden_states")) return B200MOE_E_BADARG;
  B200_CHECK_ARG(topk >= 1 && topk <= 32, "Unsupported TopK value");
  B200_CHECK_ARG(local_experts >= 1 && local_experts <= kMaxBuckets,
                 "local_experts_num exceeds the maximum supported number");
  B200_CHECK_ARG(rows_per_expert && row_map && topk_ids, "remap_hidden_states: null pointer");
  SortParams p;
  p.ids = topk_ids; p.ids_dtype = ids_dtype; p.map = expert_map;
  p.numel = num_rows * topk;
  p.id_limit = expert_map ? total_experts : local_experts;
  p.n_buckets = local_experts;
  p.block_size = 1;
  AlignOut ao = {};
  RemapOut ro = {rows_per_expert, row_map};
  return run_sort<1>(p, ao, ro, workspace, workspace_bytes, st);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_sort_workspace_bytes(int64_t numel, int num_experts) {
  if (numel <= kBlockSlots) return 0;
  const int64_t n_chunks = (numel + kChunk - 1) / kChunk;
  const size_t ints = (size_t)num_experts * n_chunks + num_experts + 1;
  return (ints * sizeof(int) + 255) & ~(size_t)255;
}

extern "C" int b200moe_moe_align_block_size(
    const void* topk_ids, b200moe_dtype ids_dtype, int64_t numel, int num_experts,
    int block_size, int32_t* sorted_token_ids, int64_t sorted_len, int32_t* expert_ids,
    int64_t expert_ids_len, int32_t* num_tokens_post_pad, const int32_t* expert_map,
    void* workspace, size_t workspace_bytes, b200moe_stream stream) {
  B200_CHECK_ARG(ids_dtype == B200MOE_I32 || ids_dtype == B200MOE_I64 || ids_dtype == B200MOE_U32,
                 "moe_align_block_size: topk_ids must be an integer tensor");
  B200_CHECK_ARG(num_experts >= 1 && ((num_experts + 31) / 32) * 32 < 1024,
                 "padded_num_experts must be less than 1024");
  B200_CHECK_ARG(block_size >= 1, "moe_align_block_size: block_size must be positive");
  B200_CHECK_ARG(numel >= 0 && sorted_len >= 0 && expert_ids_len >= 0,
                 "moe_align_block_size: negative size");
  B200_CHECK_ARG((sorted_len == 0 || sorted_token_ids) && (expert_ids_len == 0 || expert_ids) &&
                     num_tokens_post_pad,
                 "moe_align_block_size: null output");
  B200_CHECK_ARG(numel == 0 || topk_ids, "moe_align_block_size: null topk_ids");
  SortParams p;
  p.ids = topk_ids; p.ids_dtype = ids_dtype; p.map = expert_map;
  p.numel = numel; p.id_limit = num_experts; p.n_buckets = num_experts;
  p.block_size = block_size;
  AlignOut ao = {sorted_token_ids, sorted_len, expert_ids, expert_ids_len, num_tokens_post_pad};
  RemapOut ro = {};
  return run_sort<0>(p, ao, ro, workspace, workspace_bytes, as_stream(stream));
}

// ------------------------- legacy prologue ------------------------------------
namespace b200moe {
namespace {

// Tokens per block of the reference's three-step sort; it only enters the size
// of two scratch regions of the packed workspace
// (csrc/moe/fused_moe_prologue.hpp:43-60 of the reference).
int64_t prologue_tokens_per_block(int64_t num_tokens, int64_t experts) {
  for (int64_t n = 32; n <= 1024; n *= 2)
    if ((num_tokens + n - 1) / n * experts <= n) return n;
  return 1024;
}

struct PrologueArgs {
  const unsigned char* input;  unsigned char* permuted;  int64_t row_bytes;
  const unsigned char* scales; unsigned char* permuted_scales; int64_t scale_row_bytes;
  const float* final_scales;   float* permuted_final_scales;
  const int32_t* rows_per_expert;  // [experts]
  const int32_t* row_map;          // [tokens * topk], -1 = not on this rank
  const void* ids; int id_offset;
  int32_t* permuted_to_unpermuted; int32_t* permuted_experts; int32_t* unpermuted_to_permuted;
  int64_t* first_token_offset;     // [experts + 1]
  int64_t num_tokens; int topk; int experts;
};

__device__ __forceinline__ void copy_bytes(unsigned char* dst, const unsigned char* src, int64_t n) {
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | (uintptr_t)n) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (int64_t i = threadIdx.x; i < n / 16; i += blockDim.x) d4[i] = __ldg(s4 + i);
  } else {
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
  }
}

// One block per routed slot (grid-stride): copies the token's row, its scale row
// and its routing weight to the slot's permuted position and writes the three
// index maps.  Block 0 first turns the per-expert counts into the int64 offsets.
__global__ void __launch_bounds__(kBlockThreads)
prologue_expand_kernel(PrologueArgs a) {
  __shared__ int scan[kMaxBuckets + 1];
  __shared__ int warp_tot[kWarps];
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < a.experts; e += kBlockThreads) scan[e] = a.rows_per_expert[e];
    __syncthreads();
    block_exclusive_scan(scan, a.experts, warp_tot);
    for (int e = threadIdx.x; e <= a.experts; e += kBlockThreads) a.first_token_offset[e] = scan[e];
  }
  const int64_t n = a.num_tokens * a.topk;
  for (int64_t i = blockIdx.x; i < n; i += gridDim.x) {
    const int pos = a.row_map[i];
    if (pos < 0) continue;
    const int64_t token = i / a.topk;
    const int k = (int)(i - token * a.topk);
    if (threadIdx.x == 0) {
      const int32_t u = (int32_t)(k * a.num_tokens + token);
      a.permuted_to_unpermuted[pos] = u;
      a.unpermuted_to_permuted[u] = pos;
      a.permuted_experts[pos] = (int32_t)(reinterpret_cast<const int64_t*>(a.ids)[i] - a.id_offset);
      a.permuted_final_scales[pos] = a.final_scales ? a.final_scales[i] : 1.0f;
    }
    copy_bytes(a.permuted + (int64_t)pos * a.row_bytes, a.input + token * a.row_bytes, a.row_bytes);
    if (a.scales != nullptr)
      copy_bytes(a.permuted_scales + (int64_t)pos * a.scale_row_bytes,
                 a.scales + token * a.scale_row_bytes, a.scale_row_bytes);
  }
}

}  // namespace
}  // namespace b200moe

extern "C" int b200moe_fused_moe_prologue_layout(int64_t num_rows, int topk, int num_experts_on_rank,
                                                 int64_t hidden_size, int block_k, int elem_bytes,
                                                 int scale_elem_bytes, size_t offsets[10],
                                                 size_t* total_bytes) {
  B200_CHECK_ARG(num_rows >= 0 && topk >= 1 && num_experts_on_rank >= 1 && hidden_size >= 0 &&
                     block_k >= 1 && elem_bytes >= 1 && scale_elem_bytes >= 0 && offsets && total_bytes,
                 "fused_moe_prologue_layout: bad arguments");
  const size_t n = (size_t)num_rows * topk;
  const int64_t tpb = prologue_tokens_per_block(num_rows, num_experts_on_rank);
  const size_t blocks_per_seq = (size_t)((num_rows + tpb - 1) / tpb);
  const size_t counts = (size_t)num_experts_on_rank * blocks_per_seq * sizeof(int);
  const size_t sizes[10] = {
      n * sizeof(int),                                     // permuted_row_to_unpermuted_row
      n * sizeof(int),                                     // permuted_token_selected_experts
      n * sizeof(int),                                     // unpermuted_row_to_permuted_row
      counts,                                              // blocked_expert_counts (scratch)
      counts,                                              // blocked_expert_counts_cumsum (scratch)
      (size_t)num_experts_on_rank * num_rows * sizeof(int),  // blocked_row_to_unpermuted_row (scratch)
      (size_t)(num_experts_on_rank + 1) * sizeof(int64_t), // expert_first_token_offset
      n * sizeof(float),                                   // permuted_token_final_scales
      n * (size_t)hidden_size * elem_bytes,                // permuted rows
      n * (size_t)hidden_size / block_k * scale_elem_bytes // permuted scale rows
  };
  size_t off = 0;
  for (int i = 0; i < 10; ++i) {
    offsets[i] = off;
    off += (sizes[i] + 255) & ~(size_t)255;
  }
  *total_bytes = off;
  return B200MOE_OK;
}

extern "C" size_t b200moe_fused_moe_prologue_scratch_bytes(int64_t num_rows, int topk,
                                                           int num_experts_on_rank) {
  const size_t n = (size_t)num_rows * topk;
  const size_t maps = ((n + num_experts_on_rank) * sizeof(int32_t) + 255) & ~(size_t)255;
  return maps + b200moe_sort_workspace_bytes((int64_t)n, num_experts_on_rank);
}

extern "C" int b200moe_fused_moe_prologue(
    const void* input, int elem_bytes, const void* input_scales, int scale_elem_bytes,
    const int64_t* token_selected_experts, const float* token_final_scales, void* workspace,
    size_t workspace_bytes, int64_t num_rows, int64_t hidden_size, int block_k, int topk,
    int ep_rank, int ep_size, int num_experts_on_rank, void* scratch, size_t scratch_bytes,
    b200moe_stream stream) {
  B200_CHECK_ARG(ep_size >= 1 && ep_rank >= 0 && ep_rank < ep_size, "fused_moe_prologue: bad ep_rank/ep_size");
  B200_CHECK_ARG(num_experts_on_rank >= 1 && num_experts_on_rank <= kMaxBuckets,
                 "fused_moe_prologue: at most 1024 experts per rank");
  B200_CHECK_ARG(topk >= 1 && topk <= 32 && num_rows >= 0 && hidden_size >= 1 && block_k >= 1,
                 "fused_moe_prologue: bad sizes");
  B200_CHECK_ARG((int64_t)num_rows * topk < (int64_t)1 << 31, "fused_moe_prologue: too many routed rows");
  B200_CHECK_ARG(workspace && (num_rows == 0 || (input && token_selected_experts)),
                 "fused_moe_prologue: null pointer");
  B200_CHECK_ARG(input_scales == nullptr || scale_elem_bytes >= 1, "fused_moe_prologue: scale element size");
  size_t off[10], total = 0;
  if (int rc = b200moe_fused_moe_prologue_layout(num_rows, topk, num_experts_on_rank, hidden_size, block_k,
                                                 elem_bytes, input_scales ? scale_elem_bytes : 0, off, &total))
    return rc;
  if (workspace_bytes < total)
    return fail(B200MOE_E_WORKSPACE, "fused_moe_prologue: workspace of %zu bytes needed, got %zu", total,
                workspace_bytes);
  const size_t need = b200moe_fused_moe_prologue_scratch_bytes(num_rows, topk, num_experts_on_rank);
  if (scratch == nullptr || scratch_bytes < need)
    return fail(B200MOE_E_WORKSPACE, "fused_moe_prologue: scratch of %zu bytes needed, got %zu", need,
                scratch_bytes);
  const size_t n = (size_t)num_rows * topk;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  int32_t* rows = reinterpret_cast<int32_t*>(scratch);
  int32_t* row_map = rows + num_experts_on_rank;
  const size_t maps = ((n + num_experts_on_rank) * sizeof(int32_t) + 255) & ~(size_t)255;
  cudaStream_t st = as_stream(stream);

  SortParams p;
  p.ids = token_selected_experts; p.ids_dtype = B200MOE_I64; p.map = nullptr;
  p.numel = (int64_t)n; p.id_limit = num_experts_on_rank; p.n_buckets = num_experts_on_rank;
  p.block_size = 1; p.topk = topk;
  p.id_offset = num_experts_on_rank * ep_rank; p.first_match_only = true;
  AlignOut ao = {};
  RemapOut ro = {rows, row_map};
  if (int rc = run_sort<1>(p, ao, ro, reinterpret_cast<unsigned char*>(scratch) + maps, scratch_bytes - maps, st))
    return rc;

  PrologueArgs a;
  a.input = reinterpret_cast<const unsigned char*>(input);
  a.permuted = ws + off[8];
  a.row_bytes = hidden_size * elem_bytes;
  a.scales = reinterpret_cast<const unsigned char*>(input_scales);
  a.permuted_scales = ws + off[9];
  a.scale_row_bytes = input_scales ? (hidden_size / block_k) * scale_elem_bytes : 0;
  a.final_scales = token_final_scales;
  a.permuted_final_scales = reinterpret_cast<float*>(ws + off[7]);
  a.rows_per_expert = rows; a.row_map = row_map;
  a.ids = token_selected_experts; a.id_offset = p.id_offset;
  a.permuted_to_unpermuted = reinterpret_cast<int32_t*>(ws + off[0]);
  a.permuted_experts = reinterpret_cast<int32_t*>(ws + off[1]);
  a.unpermuted_to_permuted = reinterpret_cast<int32_t*>(ws + off[2]);
  a.first_token_offset = reinterpret_cast<int64_t*>(ws + off[6]);
  a.num_tokens = num_rows; a.topk = topk; a.experts = num_experts_on_rank;
  const int64_t want = (int64_t)n < 1 ? 1 : (int64_t)n;
  const int grid = (int)(want < 148 * 8 ? want : 148 * 8);
  prologue_expand_kernel<<<grid, kBlockThreads, 0, st>>>(a);
  B200_LAUNCH_OK("prologue_expand_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_moe_lora_align_block_size(
    const void* topk_ids, b200moe_dtype ids_dtype, int64_t numel, int topk,
    const int32_t* token_lora_mapping, int num_experts, int block_size, int max_loras,
    int max_num_tokens_padded, int max_num_m_blocks, int32_t* sorted_token_ids,
    int32_t* expert_ids, int32_t* num_tokens_post_pad, const int32_t* adapter_enabled,
    const int32_t* lora_ids, const int32_t* expert_map, b200moe_stream stream) {
  B200_CHECK_ARG(ids_dtype == B200MOE_I32 || ids_dtype == B200MOE_I64 || ids_dtype == B200MOE_U32,
                 "moe_lora_align_block_size: topk_ids must be an integer tensor");
  B200_CHECK_ARG(block_size > 0, "block_size should be greater than 0. ");
  B200_CHECK_ARG(num_experts >= 1 && ((num_experts + 31) / 32) * 32 < 1024,
                 "padded_num_experts must be less than 1024");
  B200_CHECK_ARG(topk >= 1 && numel >= 0 && numel % topk == 0 && max_loras >= 0 &&
                     max_num_tokens_padded >= 0 && max_num_m_blocks >= 0,
                 "moe_lora_align_block_size: bad sizes");
  B200_CHECK_ARG(token_lora_mapping && sorted_token_ids && expert_ids && num_tokens_post_pad &&
                     adapter_enabled && lora_ids && (numel == 0 || topk_ids),
                 "moe_lora_align_block_size: null pointer");
  SortParams p;
  p.ids = topk_ids; p.ids_dtype = ids_dtype; p.map = expert_map;
  p.numel = numel; p.id_limit = num_experts; p.n_buckets = num_experts;
  p.block_size = block_size;
  p.token_lora = token_lora_mapping; p.topk = topk;
  LoraAlignArgs a = {adapter_enabled, lora_ids, max_loras, max_num_tokens_padded, max_num_m_blocks,
                     sorted_token_ids, expert_ids, num_tokens_post_pad};
  const size_t smem = (size_t)(kWarps * num_experts + num_experts + 1 + kWarps) * sizeof(int);
  // lora_ids has max_loras + 1 entries: every adapter slot plus a possible -1
  lora_align_kernel<<<max_loras + 1, kBlockThreads, smem, as_stream(stream)>>>(p, a);
  B200_LAUNCH_OK("lora_align_kernel");
  return B200MOE_OK;
}

namespace b200moe {
namespace {
// One block; thread b owns batch b (csrc/moe/moe_align_sum_kernels.cpp:61-130 of the
// reference): exclusive scan of the block-padded counts, then each thread
// writes its batch's token slots and block ids.
__global__ void __launch_bounds__(1024)
batched_align_kernel(const int32_t* __restrict__ counts, int B, int max_tokens, int block,
                     int32_t* __restrict__ sorted_ids, int32_t* __restrict__ block_ids,
                     int32_t* __restrict__ num_post_pad) {
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int blocks_per_batch = (max_tokens + block - 1) / block;
  const int n_sorted = blocks_per_batch * B * block;
  for (int i = tid; i < n_sorted; i += blockDim.x) sorted_ids[i] = B * max_tokens;
  for (int i = tid; i < n_sorted / block; i += blockDim.x) block_ids[i] = -1;
  const int n = tid < B ? counts[tid] : 0;
  const int ceil_n = (n + block - 1) / block * block;
  int incl = ceil_n;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();   // also orders the fills above before the writes below
  if (warp == 0) {
    int w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += o;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int start = incl - ceil_n + (warp > 0 ? warp_sums[warp - 1] : 0);
  if (tid == B - 1) *num_post_pad = start + ceil_n;
  if (tid < B) {
    for (int i = 0; i < n; ++i) sorted_ids[start + i] = tid * max_tokens + i;
    for (int i = 0; i < ceil_n / block; ++i) block_ids[start / block + i] = tid;
  }
}
}  // namespace
}  // namespace b200moe

extern "C" int b200moe_batched_moe_align_block_size(int max_tokens_per_batch, int block_size,
                                                    const int32_t* batch_num_tokens, int num_batches,
                                                    int32_t* sorted_ids, int32_t* batch_ids,
                                                    int32_t* num_tokens_post_pad, b200moe_stream stream) {
  B200_CHECK_ARG(num_batches >= 1 && num_batches <= 1024, "batched_moe_align_block_size: at most 1024 batches");
  B200_CHECK_ARG(block_size >= 1 && max_tokens_per_batch >= 0, "batched_moe_align_block_size: bad sizes");
  B200_CHECK_ARG(batch_num_tokens && sorted_ids && batch_ids && num_tokens_post_pad,
                 "batched_moe_align_block_size: null pointer");
  batched_align_kernel<<<1, 1024, 0, as_stream(stream)>>>(batch_num_tokens, num_batches, max_tokens_per_batch,
                                                          block_size, sorted_ids, batch_ids, num_tokens_post_pad);
  B200_LAUNCH_OK("batched_align_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_init_expert_map(int32_t* expert_map, int num_local_experts,
                                       int ep_rank, int ep_size, b200moe_stream stream) {
  B200_CHECK_ARG(expert_map, "init_expert_map: null pointer");
  B200_CHECK_ARG(num_local_experts >= 1 && ep_size >= 1 && ep_rank >= 0 && ep_rank < ep_size,
                 "init_expert_map: bad ep_rank/ep_size");
  const int total = num_local_experts * ep_size;
  init_expert_map_kernel<<<(total + 255) / 256, 256, 0, as_stream(stream)>>>(
      expert_map, num_local_experts, ep_rank, total);
  B200_LAUNCH_OK("init_expert_map_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_remap_hidden_states(
    const void* hidden, const void* scales, void* remapped, void* remapped_scales,
    const int32_t* expert_map, int32_t* rows_per_expert, int32_t* row_map,
    const void* topk_ids, b200moe_dtype ids_dtype, int64_t num_rows, int hidden_size,
    int elem_bytes, int scale_cols, int scale_elem_bytes, int topk, int total_experts,
    int local_experts, void* workspace, size_t workspace_bytes, b200moe_stream stream) {
  B200_CHECK_ARG(elem_bytes == 1 || elem_bytes == 2 || elem_bytes == 4,
                 "Unsupported data type in hidden_states");
  B200_CHECK_ARG((scales == nullptr) == (remapped_scales == nullptr),
                 "if hidden_states_scales is provided, remapped_hidden_states_scales "
                 "must also be provided");
  B200_CHECK_ARG(((int64_t)hidden_size * elem_bytes) % 16 == 0,
                 "hidden_size must be divisible by ElemsPerItem");
  B200_CHECK_ARG(num_rows >= 0, "remap_hidden_states: negative num_rows");
  cudaStream_t st = as_stream(stream);
  int rc = remap_bookkeeping(expert_map, rows_per_expert, row_map, topk_ids, ids_dtype,
                             num_rows, topk, total_experts, local_experts, workspace,
                             workspace_bytes, st);
  if (rc != B200MOE_OK || num_rows == 0) return rc;
  B200_CHECK_ARG(hidden && remapped, "remap_hidden_states: null pointer");
  B200_CHECK_ARG(((uintptr_t)hidden & 15) == 0 && ((uintptr_t)remapped & 15) == 0,
                 "remap_hidden_states: buffers must be 16-byte aligned");
  remap_copy_kernel<<<(unsigned)num_rows, 256, 0, st>>>(
      (const uint8_t*)hidden, (uint8_t*)remapped, (const uint8_t*)scales,
      (uint8_t*)remapped_scales, row_map, hidden_size * elem_bytes,
      scale_cols * scale_elem_bytes, topk);
  B200_LAUNCH_OK("remap_copy_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_remap_quant_fp8(
    const void* hidden, b200moe_dtype dtype, void* remapped_q, float* remapped_scales,
    const int32_t* expert_map, int32_t* rows_per_expert, int32_t* row_map,
    const void* topk_ids, b200moe_dtype ids_dtype, int64_t num_rows, int hidden_size,
    int topk, int total_experts, int local_experts, void* workspace,
    size_t workspace_bytes, b200moe_stream stream) {
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16,
                 "remap_quant_fp8: activations must be bfloat16 or float16");
  B200_CHECK_ARG(hidden_size % 128 == 0, "remap_quant_fp8: hidden_size must be a multiple of 128");
  cudaStream_t st = as_stream(stream);
  int rc = remap_bookkeeping(expert_map, rows_per_expert, row_map, topk_ids, ids_dtype,
                             num_rows, topk, total_experts, local_experts, workspace,
                             workspace_bytes, st);
  if (rc != B200MOE_OK || num_rows == 0) return rc;
  B200_CHECK_ARG(hidden && remapped_q && remapped_scales, "remap_quant_fp8: null pointer");
  B200_CHECK_ARG(((uintptr_t)hidden & 15) == 0 && ((uintptr_t)remapped_q & 7) == 0,
                 "remap_quant_fp8: buffers must be 16-byte aligned");
  if (dtype == B200MOE_BF16)
    remap_quant_kernel<__nv_bfloat16><<<(unsigned)num_rows, 256, 0, st>>>(
        (const __nv_bfloat16*)hidden, (uint8_t*)remapped_q, remapped_scales, row_map,
        hidden_size, topk);
  else
    remap_quant_kernel<__half><<<(unsigned)num_rows, 256, 0, st>>>(
        (const __half*)hidden, (uint8_t*)remapped_q, remapped_scales, row_map, hidden_size,
        topk);
  B200_LAUNCH_OK("remap_quant_kernel");
  return B200MOE_OK;
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the align op.
//
// Some hosts of this library cannot hand over scratch memory: a cgo / JNI /
// ctypes binding usually receives only the input and output buffers that its
// serving framework allocated and owns no device allocator of its own, and a
// latency-critical serving loop must not call cudaMalloc on its hot path
// (the call serialises the whole device and fails once the framework's pool
// has claimed all memory).  For them the histogram exchange buffer of the
// multi-block sort lives in a fixed array inside the library image.  Every GPU
// that loads the library holds these kNoAllocScratchBytes until the process
// exits.
// ---------------------------------------------------------------------------
namespace b200moe {
namespace {
constexpr size_t kNoAllocScratchBytes = 1u << 20;  // 1 MiB
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
// device address of the array per device ordinal; written once, read by any thread
std::atomic<void*> g_noalloc_ptr[kMaxDevices];
}  // namespace
}  // namespace b200moe

extern "C" size_t b200moe_noalloc_scratch_capacity(void) { return b200moe::kNoAllocScratchBytes; }

extern "C" int b200moe_moe_align_block_size_noalloc(
    const void* topk_ids, b200moe_dtype ids_dtype, int64_t numel, int num_experts, int block_size,
    int32_t* sorted_token_ids, int64_t sorted_len, int32_t* expert_ids, int64_t expert_ids_len,
    int32_t* num_tokens_post_pad, const int32_t* expert_map, b200moe_stream stream) {
  B200_CHECK_ARG(num_experts >= 1 && numel >= 0, "moe_align_block_size_noalloc: bad sizes");
  const size_t need = b200moe_sort_workspace_bytes(numel, num_experts);
  if (need > kNoAllocScratchBytes)
    return fail(B200MOE_E_WORKSPACE,
                "moe_align_block_size_noalloc: %lld slots over %d experts need %zu bytes of scratch, "
                "the built-in buffer holds %zu; use b200moe_moe_align_block_size with a workspace",
                (long long)numel, num_experts, need, (size_t)kNoAllocScratchBytes);
  int dev = -1;
  B200_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(B200MOE_E_UNSUPPORTED, "moe_align_block_size_noalloc: device ordinal %d out of range", dev);
  void* scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // In host code `g_noalloc_scratch` is only a handle for the symbol, not a
    // device address: resolve it once per device, with that device current.
    // (Two threads that race here both look up the same address.)
    B200_CUDA_OK(cudaGetSymbolAddress(&scratch, g_noalloc_scratch));
    if (scratch == nullptr) return fail(B200MOE_E_CUDA, "cudaGetSymbolAddress returned a null address");
    g_noalloc_ptr[dev].store(scratch, std::memory_order_release);
  }
  // Nothing in the buffer has to start at zero: the count pass overwrites every
  // histogram cell it later reads and the scan pass writes the prefix array.
  return b200moe_moe_align_block_size(topk_ids, ids_dtype, numel, num_experts, block_size,
                                      sorted_token_ids, sorted_len, expert_ids, expert_ids_len,
                                      num_tokens_post_pad, expert_map, scratch,
                                      kNoAllocScratchBytes, stream);
}
