// Stable counting sort of routed slots by (mapped) bucket id: the machinery behind
// moe_align_block_size, remap_hidden_states, the legacy prologue and the expert-parallel
// dispatch.
//
// The slots are cut into chunks of 256 handled by one warp each:
//   1. count : every warp builds a histogram of its chunk,
//   2. scan  : per bucket an exclusive scan over the chunks, then a scan over
//              the buckets (padded to block_size for the align op),
//   3. rank  : every warp walks its chunk 32 slots at a time; the rank of a
//              slot among equal ids in the same step comes from
//              __match_any_sync, so slots of one bucket keep ascending order.
// Up to 2048 slots all three steps run in one block without any scratch;
// beyond that they are three launches that exchange the histograms through a
// caller-provided workspace.  The result is deterministic: no atomics decide
// an order.
#pragma once

#include "common.cuh"

namespace b200moe {
namespace {

constexpr int kChunk = 256;          // slots per warp
constexpr int kBlockThreads = 256;   // 8 warps
constexpr int kWarps = kBlockThreads / 32;
constexpr int kBlockSlots = kChunk * kWarps;  // 2048
constexpr int kMaxBuckets = 1024;

struct SortParams {
  const void* ids;
  b200moe_dtype ids_dtype;
  const int32_t* map;  // optional id -> bucket map
  int64_t numel;
  int id_limit;        // ids >= id_limit (or < 0) are dropped
  int n_buckets;
  int block_size;      // align: pad every bucket to a multiple of this; remap: 1
  // LoRA variant: a slot counts only if its token is mapped to `lora_id`
  const int32_t* token_lora = nullptr;  // [numel / topk] or null
  int lora_id = 0;
  int topk = 1;
  // prologue variant: ids are global expert ids, bucket = id - id_offset; a
  // token that names the same expert twice keeps only the first slot
  int id_offset = 0;
  bool first_match_only = false;
  // expert-parallel dispatch: `ids` is [numel / ep_size, topk] global expert ids and slot
  // i = (token, rank d) belongs to bucket d when one of the token's experts lives on rank d
  // (expert g on rank slot(g) / ep_local_experts, slot(g) = ep_slot[g] or g), else to none
  int ep_size = 0;
  int ep_local_experts = 0;
  const int32_t* ep_slot = nullptr;
  // > 0: bucket b's rows are numbered from b * bucket_stride (fixed-capacity regions)
  // instead of from the end of bucket b - 1
  int64_t bucket_stride = 0;
};

__device__ __forceinline__ int64_t raw_id(const SortParams& p, int64_t i) {
  switch (p.ids_dtype) {
    case B200MOE_I64: return reinterpret_cast<const int64_t*>(p.ids)[i];
    case B200MOE_U32: return reinterpret_cast<const uint32_t*>(p.ids)[i];
    default: return reinterpret_cast<const int32_t*>(p.ids)[i];
  }
}

__device__ __forceinline__ int bucket_of(const SortParams& p, int64_t i) {
  if (p.ep_size > 0) {
    const int64_t tok = i / p.ep_size;
    const int d = (int)(i - tok * p.ep_size);
    for (int k = 0; k < p.topk; ++k) {
      int64_t g = raw_id(p, tok * p.topk + k);
      if (g < 0 || g >= (int64_t)p.ep_size * p.ep_local_experts) continue;
      if (p.ep_slot != nullptr) g = p.ep_slot[g];
      if (g / p.ep_local_experts == d) return d;
    }
    return -1;
  }
  const int64_t raw = raw_id(p, i);
  const int64_t e = raw - p.id_offset;
  if (e < 0 || e >= p.id_limit) return -1;
  if (p.first_match_only) {
    for (int64_t j = i - i % p.topk; j < i; ++j)
      if (raw_id(p, j) == raw) return -1;
  }
  if (p.token_lora != nullptr && p.token_lora[i / p.topk] != p.lora_id) return -1;
  int b = (int)e;
  if (p.map != nullptr) b = p.map[b];
  if (b < 0 || b >= p.n_buckets) return -1;
  return b;
}

// In-place exclusive scan of data[0..n) (n <= 1024, shared memory) by a block
// of kBlockThreads threads; data[n] receives the total.  `warp_tot` is scratch
// for kWarps ints.
__device__ void block_exclusive_scan(int* data, int n, int* warp_tot) {
  const int t = threadIdx.x;
  const int lane = t & 31, warp = t >> 5;
  int x[4];
  int local = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int idx = 4 * t + j;
    x[j] = (idx < n) ? data[idx] : 0;
    local += x[j];
  }
  int incl = local;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int base = 0;
  for (int w = 0; w < warp; ++w) base += warp_tot[w];
  int run = base + incl - local;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int idx = 4 * t + j;
    if (idx < n) data[idx] = run;
    run += x[j];
  }
  if (t == kBlockThreads - 1) data[n] = run;
  __syncthreads();
}

// Walks one warp's chunk and calls emit(slot, bucket, position) for every
// slot; `run` (shared, per warp, n_buckets ints) holds the next free position
// of each bucket for this warp and is advanced as the walk proceeds.
template <typename Emit>
__device__ __forceinline__ void rank_walk(const SortParams& p, int64_t chunk_begin,
                                          int* run, Emit emit) {
  const int lane = threadIdx.x & 31;
  const uint32_t lt = (1u << lane) - 1u;
  for (int step = 0; step < kChunk / 32; ++step) {
    const int64_t i = chunk_begin + step * 32 + lane;
    const bool in = i < p.numel;
    const int b = in ? bucket_of(p, i) : -1;
    // Lanes without a bucket use distinct keys so they never match a real one.
    const int key = (b >= 0) ? b : (kMaxBuckets + lane);
    const uint32_t peers = __match_any_sync(0xffffffffu, key);
    int pos = -1;
    if (b >= 0) pos = run[b] + __popc(peers & lt);
    __syncwarp();
    if (b >= 0 && (peers & lt) == 0) run[b] += __popc(peers);
    __syncwarp();
    if (in) emit(i, b, pos);
  }
}

// ------------------------- single-block path --------------------------------
// mode 0: align (sorted ids, expert ids, post-pad count);
// mode 1: remap (rows_per_expert, row map).
struct AlignOut {
  int32_t* sorted; int64_t sorted_len;
  int32_t* expert_ids; int64_t expert_ids_len;
  int32_t* post_pad;
};
struct RemapOut {
  int32_t* rows_per_expert;
  int32_t* row_map;
};

template <int kMode>
__global__ void __launch_bounds__(kBlockThreads)
sort_single_block_kernel(SortParams p, AlignOut ao, RemapOut ro) {
  extern __shared__ int smem[];
  int* hist = smem;                              // [kWarps][n_buckets]
  int* base = hist + kWarps * p.n_buckets;       // [n_buckets + 1]
  int* warp_tot = base + p.n_buckets + 1;        // [kWarps]
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nb = p.n_buckets;

  for (int i = t; i < kWarps * nb; i += kBlockThreads) hist[i] = 0;
  if (kMode == 0) {
    for (int64_t i = t; i < ao.sorted_len; i += kBlockThreads) ao.sorted[i] = (int32_t)p.numel;
  }
  __syncthreads();
  {
    const int64_t begin = (int64_t)warp * kChunk;
    for (int s = 0; s < kChunk / 32; ++s) {
      const int64_t i = begin + s * 32 + lane;
      if (i < p.numel) {
        const int b = bucket_of(p, i);
        if (b >= 0) atomicAdd(&hist[warp * nb + b], 1);
      }
    }
  }
  __syncthreads();
  for (int e = t; e < nb; e += kBlockThreads) {
    int run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const int c = hist[w * nb + e];
      hist[w * nb + e] = run;
      run += c;
    }
    if (kMode == 1) ro.rows_per_expert[e] = run;
    base[e] = (kMode == 0) ? ((run + p.block_size - 1) / p.block_size) * p.block_size : run;
  }
  __syncthreads();
  int padded[4];  // align: remember the padded sizes for expert_ids
#pragma unroll
  for (int j = 0; j < 4; ++j) padded[j] = (4 * t + j < nb) ? base[4 * t + j] : 0;
  block_exclusive_scan(base, nb, warp_tot);
  if (kMode == 0) {
    const int total = base[nb];
    if (t == 0) ao.post_pad[0] = total;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = 4 * t + j;
      if (e < nb) {
        for (int o = 0; o < padded[j]; o += p.block_size) {
          const int64_t blk = (base[e] + o) / p.block_size;
          if (blk < ao.expert_ids_len) ao.expert_ids[blk] = e;
        }
      }
    }
    for (int64_t blk = total / p.block_size + t; blk < ao.expert_ids_len; blk += kBlockThreads)
      ao.expert_ids[blk] = 0;
  }
  // hist[w][e] += base[e]  -> absolute next-free position per warp and bucket
  for (int i = t; i < kWarps * nb; i += kBlockThreads)
    hist[i] += p.bucket_stride > 0 ? (int)((i % nb) * p.bucket_stride) : base[i % nb];
  __syncthreads();
  rank_walk(p, (int64_t)warp * kChunk, hist + warp * nb,
            [&](int64_t i, int b, int pos) {
              if (kMode == 0) {
                if (b >= 0 && pos < ao.sorted_len) ao.sorted[pos] = (int32_t)i;
              } else {
                ro.row_map[i] = pos;  // -1 when the slot has no local expert
              }
            });
}

// ------------------------- LoRA variant ---------------------------------------
// One block per entry of lora_ids (csrc/moe/moe_align_sum_kernels.cpp:732-847,
// 926-1027 of the reference): the block aligns the slots whose token is mapped
// to its adapter into that adapter's segment of the outputs.  Entries that are
// -1, out of range or disabled return without writing anything.  The slots are
// walked in rounds of kBlockSlots with the same stable ranking as above, so the
// order inside an expert is ascending slot index.
struct LoraAlignArgs {
  const int32_t* adapter_enabled;
  const int32_t* lora_ids;
  int max_loras;
  int max_num_tokens_padded;
  int max_num_m_blocks;
  int32_t* sorted;
  int32_t* expert_ids;
  int32_t* post_pad;
};

__global__ void __launch_bounds__(kBlockThreads)
lora_align_kernel(SortParams p, LoraAlignArgs a) {
  extern __shared__ int smem[];
  const int nb = p.n_buckets;
  int* hist = smem;                        // [kWarps][nb]
  int* base = hist + kWarps * nb;          // [nb + 1]
  int* warp_tot = base + nb + 1;           // [kWarps]
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int lora_id = a.lora_ids[blockIdx.x];
  if (lora_id < 0 || lora_id >= a.max_loras || a.adapter_enabled[lora_id] == 0) return;
  p.lora_id = lora_id;
  int32_t* sorted = a.sorted + (int64_t)lora_id * a.max_num_tokens_padded;
  int32_t* eids = a.expert_ids + (int64_t)lora_id * a.max_num_m_blocks;

  for (int e = t; e <= nb; e += kBlockThreads) base[e] = 0;
  for (int i = t; i < a.max_num_tokens_padded; i += kBlockThreads) sorted[i] = (int32_t)p.numel;
  __syncthreads();
  for (int64_t i = t; i < p.numel; i += kBlockThreads) {
    const int b = bucket_of(p, i);
    if (b >= 0) atomicAdd(&base[b], 1);
  }
  __syncthreads();
  int padded[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = 4 * t + j;
    padded[j] = (e < nb) ? ((base[e] + p.block_size - 1) / p.block_size) * p.block_size : 0;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (4 * t + j < nb) base[4 * t + j] = padded[j];
  __syncthreads();
  block_exclusive_scan(base, nb, warp_tot);
  const int total = base[nb];
  if (t == 0) a.post_pad[lora_id] = total;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = 4 * t + j;
    if (e < nb) {
      for (int o = 0; o < padded[j]; o += p.block_size) {
        const int blk = (base[e] + o) / p.block_size;
        if (blk < a.max_num_m_blocks) eids[blk] = e;
      }
    }
  }
  for (int blk = total / p.block_size + t; blk < a.max_num_m_blocks; blk += kBlockThreads) eids[blk] = -1;

  // base[e] is from here on the next free position of expert e
  for (int64_t r0 = 0; r0 < p.numel; r0 += kBlockSlots) {
    for (int i = t; i < kWarps * nb; i += kBlockThreads) hist[i] = 0;
    __syncthreads();
    const int64_t begin = r0 + (int64_t)warp * kChunk;
    for (int s = 0; s < kChunk / 32; ++s) {
      const int64_t i = begin + s * 32 + lane;
      if (i < p.numel) {
        const int b = bucket_of(p, i);
        if (b >= 0) atomicAdd(&hist[warp * nb + b], 1);
      }
    }
    __syncthreads();
    for (int e = t; e < nb; e += kBlockThreads) {
      int run = base[e];
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const int c = hist[w * nb + e];
        hist[w * nb + e] = run;
        run += c;
      }
      base[e] = run;
    }
    __syncthreads();
    rank_walk(p, begin, hist + warp * nb, [&](int64_t i, int b, int pos) {
      if (b >= 0 && pos < a.max_num_tokens_padded) sorted[pos] = (int32_t)i;
    });
    __syncthreads();
  }
}

// ------------------------- multi-block path ---------------------------------
// workspace: counts[n_buckets][n_chunks] ints, then base[n_buckets + 1] ints.
__global__ void __launch_bounds__(kBlockThreads)
sort_count_kernel(SortParams p, int n_chunks, int* counts, int32_t* fill,
                  int64_t fill_len) {
  extern __shared__ int smem[];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nb = p.n_buckets;
  int* hist = smem + warp * nb;
  for (int i = t; i < kWarps * nb; i += kBlockThreads) smem[i] = 0;
  if (fill != nullptr) {
    for (int64_t i = (int64_t)blockIdx.x * kBlockThreads + t; i < fill_len;
         i += (int64_t)gridDim.x * kBlockThreads)
      fill[i] = (int32_t)p.numel;
  }
  __syncthreads();
  const int chunk = blockIdx.x * kWarps + warp;
  const int64_t begin = (int64_t)chunk * kChunk;
  for (int s = 0; s < kChunk / 32; ++s) {
    const int64_t i = begin + s * 32 + lane;
    if (i < p.numel) {
      const int b = bucket_of(p, i);
      if (b >= 0) atomicAdd(&hist[b], 1);
    }
  }
  __syncwarp();
  if (chunk < n_chunks) {
    for (int e = lane; e < nb; e += 32) counts[(int64_t)e * n_chunks + chunk] = hist[e];
  }
}

template <int kMode>
__global__ void __launch_bounds__(1024)
sort_scan_kernel(SortParams p, int n_chunks, int* counts, int* base_out,
                 AlignOut ao, RemapOut ro) {
  __shared__ int base[kMaxBuckets + 1];
  __shared__ int sizes[kMaxBuckets];
  __shared__ int warp_tot[32];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nb = p.n_buckets;
  // One warp per expert: exclusive scan over the chunks, 32 at a time.
  for (int e = warp; e < nb; e += 32) {
    int* row = counts + (int64_t)e * n_chunks;
    int carry = 0;
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
      const int c = c0 + lane;
      const int x = (c < n_chunks) ? row[c] : 0;
      int incl = x;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      if (c < n_chunks) row[c] = carry + incl - x;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      if (kMode == 1) ro.rows_per_expert[e] = carry;
      sizes[e] = (kMode == 0) ? ((carry + p.block_size - 1) / p.block_size) * p.block_size : carry;
    }
  }
  __syncthreads();
  // Exclusive scan over the experts (1024 threads, one value each).
  {
    const int x = (t < nb) ? sizes[t] : 0;
    int incl = x;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int b0 = 0;
    for (int w = 0; w < warp; ++w) b0 += warp_tot[w];
    if (t < nb) base[t] = b0 + incl - x;
    if (t == 1023) base[nb] = b0 + incl;
    __syncthreads();
  }
  for (int e = t; e <= nb; e += 1024) base_out[e] = base[e];
  if (kMode == 0) {
    const int total = base[nb];
    if (t == 0) ao.post_pad[0] = total;
    for (int e = t; e < nb; e += 1024) {
      for (int o = 0; o < sizes[e]; o += p.block_size) {
        const int64_t blk = (base[e] + o) / p.block_size;
        if (blk < ao.expert_ids_len) ao.expert_ids[blk] = e;
      }
    }
    for (int64_t blk = total / p.block_size + t; blk < ao.expert_ids_len; blk += 1024)
      ao.expert_ids[blk] = 0;
  }
}

template <int kMode>
__global__ void __launch_bounds__(kBlockThreads)
sort_rank_kernel(SortParams p, int n_chunks, const int* counts, const int* base,
                 AlignOut ao, RemapOut ro) {
  extern __shared__ int smem[];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int nb = p.n_buckets;
  int* run = smem + warp * nb;
  const int chunk = blockIdx.x * kWarps + warp;
  if (chunk < n_chunks) {
    for (int e = lane; e < nb; e += 32)
      run[e] = (p.bucket_stride > 0 ? (int)(e * p.bucket_stride) : base[e]) + counts[(int64_t)e * n_chunks + chunk];
  }
  __syncwarp();
  if (chunk >= n_chunks) return;
  rank_walk(p, (int64_t)chunk * kChunk, run, [&](int64_t i, int b, int pos) {
    if (kMode == 0) {
      if (b >= 0 && pos < ao.sorted_len) ao.sorted[pos] = (int32_t)i;
    } else {
      ro.row_map[i] = pos;
    }
  });
}

template <int kMode>
int run_sort(const SortParams& p, const AlignOut& ao, const RemapOut& ro,
             void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const int nb = p.n_buckets;
  if (p.numel <= kBlockSlots) {
    const size_t smem = (size_t)(kWarps * nb + nb + 1 + kWarps) * sizeof(int);
    sort_single_block_kernel<kMode><<<1, kBlockThreads, smem, st>>>(p, ao, ro);
    B200_LAUNCH_OK("sort_single_block_kernel");
    return B200MOE_OK;
  }
  const size_t need = b200moe_sort_workspace_bytes(p.numel, nb);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(B200MOE_E_WORKSPACE, "workspace of %zu bytes needed, got %zu", need,
                workspace_bytes);
  const int n_chunks = (int)((p.numel + kChunk - 1) / kChunk);
  const int n_blocks = (n_chunks + kWarps - 1) / kWarps;
  int* counts = reinterpret_cast<int*>(workspace);
  int* base = counts + (size_t)nb * n_chunks;
  const size_t smem = (size_t)kWarps * nb * sizeof(int);
  sort_count_kernel<<<n_blocks, kBlockThreads, smem, st>>>(
      p, n_chunks, counts, kMode == 0 ? ao.sorted : nullptr, kMode == 0 ? ao.sorted_len : 0);
  B200_LAUNCH_OK("sort_count_kernel");
  sort_scan_kernel<kMode><<<1, 1024, 0, st>>>(p, n_chunks, counts, base, ao, ro);
  B200_LAUNCH_OK("sort_scan_kernel");
  sort_rank_kernel<kMode><<<n_blocks, kBlockThreads, smem, st>>>(p, n_chunks, counts, base, ao, ro);
  B200_LAUNCH_OK("sort_rank_kernel");
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe
