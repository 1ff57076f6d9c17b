// Expert-parallel token dispatch and combine over peer memory (NVLink): the kernels
// store rows straight into the receive buffers of the ranks that own a token's experts
// and the partial sums straight back into the source's buffers, with ordinary global
// stores.  No kernel waits for another rank; the caller orders the phases with barriers
// between the launches.  The reference has no counterpart: its expert parallelism is the
// init_expert_map mask (csrc/moe/init_expert_map.cpp:33-53 of vllm-xpu-kernels).
#include "common.cuh"
#include "sort.cuh"

namespace b200moe {
namespace {

struct EpTables {
  uint8_t* rows[B200MOE_MAX_EP];
  float* scales[B200MOE_MAX_EP];
  int32_t* ids[B200MOE_MAX_EP];
  float* weights[B200MOE_MAX_EP];
  int32_t* counts[B200MOE_MAX_EP];
};

struct EpDispatchParams {
  EpTables peer;
  const void* ids;            // [T, K] global expert ids
  b200moe_dtype ids_dtype;
  const float* weights;       // [T, K]
  const int32_t* send_counts; // [ep]
  const int32_t* send_pos;    // [T, ep]
  const int32_t* slot;        // [ep * e_local] expert -> slot, or null (identity)
  int64_t num_tokens, capacity;
  int ep, rank, e_local, H, K;
};

__device__ __forceinline__ int64_t ep_raw_id(const void* ids, b200moe_dtype t, int64_t i) {
  switch (t) {
    case B200MOE_I64: return reinterpret_cast<const int64_t*>(ids)[i];
    case B200MOE_U32: return reinterpret_cast<const uint32_t*>(ids)[i];
    default: return reinterpret_cast<const int32_t*>(ids)[i];
  }
}

// Every rank walks its peers starting with its right-hand neighbour and ends with itself, so
// that at any moment the ranks store into different peers.  (With all ranks walking 0, 1, 2, ..
// they all store into the same peer at the same time, whose NVLink ingress then bounds all of
// them: measured on 8 GPUs, dispatch + combine took 1.4 ms on rank 0 and 3.1 ms on rank 6.)
__device__ __forceinline__ int dest_order(int rank, int i, int ep) {
  const int d = rank + 1 + i;
  return d >= ep ? d - ep : d;
}

// One block per token.  The row is read (and, kQuant, quantised per 1x128 group) once and
// stored to every destination rank; the token's expert ids local to that rank and its
// routing weights follow.  Block 0 also tells every rank how many rows this rank sent it.
template <typename T, bool kQuant>
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const T* __restrict__ src, const __grid_constant__ EpDispatchParams p) {
  const int64_t tok = blockIdx.x;
  __shared__ int dest[B200MOE_MAX_EP];   // row index inside region `rank` of the destination, or -1
  if (blockIdx.x == 0 && threadIdx.x < p.ep)
    p.peer.counts[threadIdx.x][p.rank] = p.send_counts[threadIdx.x];
  if (tok >= p.num_tokens) return;
  if (threadIdx.x < p.ep) {
    const int pos = p.send_pos[tok * p.ep + threadIdx.x];
    dest[threadIdx.x] = pos < 0 ? -1 : pos - threadIdx.x * (int)p.capacity;
  }
  __syncthreads();
  const int H = p.H;
  const T* s = src + tok * (int64_t)H;
  const int64_t region = (int64_t)p.rank * p.capacity;
  if (kQuant) {
    const int groups = H / 128;
    const int nvec = H / 8;
    for (int j0 = (threadIdx.x & ~31); j0 < nvec; j0 += blockDim.x) {   // whole warps: 16-lane shuffles
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
      for (int mask = 8; mask > 0; mask >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask));
      amax = fmaxf(amax, 1e-10f);
      const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1.0f / (448.f * 512.f));
      const float inv = __fdiv_rn(1.0f, scale);
      if (j < nvec) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          lo |= (uint32_t)f32_to_e4m3(fminf(fmaxf(__fmul_rn(x[i], inv), -448.f), 448.f)) << (8 * i);
          hi |= (uint32_t)f32_to_e4m3(fminf(fmaxf(__fmul_rn(x[4 + i], inv), -448.f), 448.f)) << (8 * i);
        }
        for (int dd = 0; dd < p.ep; ++dd) {
          const int d = dest_order(p.rank, dd, p.ep);
          const int r = dest[d];
          if (r < 0) continue;
          const int64_t row = region + r;
          *reinterpret_cast<uint2*>(p.peer.rows[d] + row * H + (int64_t)j * 8) = make_uint2(lo, hi);
          if ((j & 15) == 0) p.peer.scales[d][row * groups + (j >> 4)] = scale;
        }
      }
    }
  } else {
    const int nvec = (H * (int)sizeof(T)) >> 4;
    const int64_t row_bytes = (int64_t)H * sizeof(T);
    for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
      const vec16 v = ld16(reinterpret_cast<const uint8_t*>(s) + (int64_t)j * 16);
      for (int dd = 0; dd < p.ep; ++dd) {
        const int d = dest_order(p.rank, dd, p.ep);
        const int r = dest[d];
        if (r >= 0) st16(p.peer.rows[d] + (region + r) * row_bytes + (int64_t)j * 16, v);
      }
    }
  }
  // expert ids local to the destination and routing weights: thread (d, k)
  for (int u = threadIdx.x; u < p.ep * p.K; u += blockDim.x) {
    const int d = u / p.K, k = u - d * p.K;
    const int r = dest[d];
    if (r < 0) continue;
    int64_t g = ep_raw_id(p.ids, p.ids_dtype, tok * p.K + k);
    if (g >= (int64_t)p.ep * p.e_local) g = -1;
    if (g >= 0 && p.slot != nullptr) g = p.slot[g];
    const bool mine = g >= 0 && g / p.e_local == d;
    const int64_t cell = (region + r) * p.K + k;
    p.peer.ids[d][cell] = mine ? (int32_t)(g - (int64_t)d * p.e_local) : -1;
    p.peer.weights[d][cell] = mine ? p.weights[tok * p.K + k] : 0.f;
  }
  __threadfence_system();
}

__global__ void __launch_bounds__(256)
ep_mask_unused_kernel(int32_t* ids, const int32_t* counts, int64_t capacity, int K) {
  const int s = blockIdx.y;
  const int64_t first = (int64_t)min((int64_t)max(counts[s], 0), capacity) * K;
  const int64_t cells = capacity * K;
  int32_t* base = ids + (int64_t)s * cells;
  for (int64_t i = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < cells;
       i += (int64_t)gridDim.x * blockDim.x)
    base[i] = -1;
}

struct EpCombineParams {
  uint8_t* comb[B200MOE_MAX_EP];
  const float* weights;       // this rank's recv_weights [ep*capacity, K]
  const int32_t* counts;      // this rank's recv_counts [ep]
  const int32_t* row_map;     // [ep*capacity, K]
  int64_t capacity;
  int ep, rank, H, K;
};

// One block per received row: the top-k reduction of moe_gather, stored into region `rank`
// of the source rank's comb_rows.
template <typename T>
__global__ void __launch_bounds__(256)
ep_combine_kernel(const T* __restrict__ src, const __grid_constant__ EpCombineParams p) {
  constexpr int N = 16 / sizeof(T);
  const int s = dest_order(p.rank, (int)blockIdx.y, p.ep);   // blocks are scheduled y-major: peer by peer
  const int64_t i = blockIdx.x;
  if (i >= p.counts[s]) return;
  __shared__ int rows[64];
  __shared__ float wk[64];
  const int64_t g = (int64_t)s * p.capacity + i;
  if (threadIdx.x < p.K) {
    rows[threadIdx.x] = p.row_map[g * p.K + threadIdx.x];
    wk[threadIdx.x] = p.weights[g * p.K + threadIdx.x];
  }
  __syncthreads();
  T* out = reinterpret_cast<T*>(p.comb[s]) + ((int64_t)p.rank * p.capacity + i) * p.H;
  for (int j = threadIdx.x; j < p.H / N; j += blockDim.x) {
    float acc[N];
#pragma unroll
    for (int u = 0; u < N; ++u) acc[u] = 0.f;
    for (int k = 0; k < p.K; ++k) {
      const int r = rows[k];
      if (r < 0) continue;
      const vec16 v = ld16(src + (int64_t)r * p.H + (int64_t)j * N);
      const T* e = reinterpret_cast<const T*>(&v);
      const float wv = wk[k];
#pragma unroll
      for (int u = 0; u < N; ++u) acc[u] = fmaf(to_f32<T>(e[u]), wv, acc[u]);
    }
    vec16 ov;
    T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int u = 0; u < N; ++u) oe[u] = from_f32<T>(acc[u]);
    st16(out + (int64_t)j * N, ov);
  }
  __threadfence_system();
}

int check_peers(const b200moe_ep_peers* pe, const char* who) {
  B200_CHECK_ARG(pe != nullptr, "%s: null peer table", who);
  B200_CHECK_ARG(pe->ep_size >= 1 && pe->ep_size <= B200MOE_MAX_EP, "%s: ep_size must be 1..%d", who, B200MOE_MAX_EP);
  B200_CHECK_ARG(pe->ep_rank >= 0 && pe->ep_rank < pe->ep_size, "%s: ep_rank out of range", who);
  B200_CHECK_ARG(pe->num_local_experts >= 1 && pe->topk >= 1 && pe->topk <= 32, "%s: bad expert counts", who);
  B200_CHECK_ARG(pe->capacity >= 1 && pe->capacity * pe->ep_size < (1ll << 30), "%s: bad capacity", who);
  B200_CHECK_ARG(pe->hidden >= 8 && pe->hidden % 8 == 0, "%s: hidden must be a multiple of 8", who);
  B200_CHECK_ARG(!pe->quantized || pe->hidden % 128 == 0, "%s: quantised rows need hidden divisible by 128", who);
  for (int d = 0; d < pe->ep_size; ++d) {
    B200_CHECK_ARG(pe->recv_rows[d] && pe->recv_ids[d] && pe->recv_weights[d] && pe->recv_counts[d] &&
                       pe->comb_rows[d] && (!pe->quantized || pe->recv_scales[d]),
                   "%s: null buffer of rank %d", who, d);
    B200_CHECK_ARG((((uintptr_t)pe->recv_rows[d] | (uintptr_t)pe->comb_rows[d]) & 15) == 0,
                   "%s: row buffers must be 16-byte aligned", who);
  }
  return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" size_t b200moe_ep_dispatch_workspace_bytes(int64_t num_tokens, int ep_size) {
  return b200moe_sort_workspace_bytes(num_tokens * ep_size, ep_size);
}

extern "C" int b200moe_ep_dispatch(const b200moe_ep_peers* pe, const void* hidden, b200moe_dtype dtype,
                                   const void* topk_ids, b200moe_dtype ids_dtype, const float* topk_weights,
                                   int64_t num_tokens, int32_t* send_counts, int32_t* send_pos,
                                   void* workspace, size_t workspace_bytes, b200moe_stream stream) {
  if (int rc = check_peers(pe, "ep_dispatch")) return rc;
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "ep_dispatch: hidden must be bfloat16 or float16");
  B200_CHECK_ARG(ids_dtype == B200MOE_I32 || ids_dtype == B200MOE_I64 || ids_dtype == B200MOE_U32,
                 "ep_dispatch: topk_ids must be int64 or int32");
  B200_CHECK_ARG(num_tokens >= 0 && num_tokens <= pe->capacity,
                 "ep_dispatch: %lld tokens exceed the capacity %lld of the receive regions", (long long)num_tokens,
                 (long long)pe->capacity);
  B200_CHECK_ARG(send_counts && send_pos, "ep_dispatch: null output");
  B200_CHECK_ARG(num_tokens == 0 || (hidden && topk_ids && topk_weights), "ep_dispatch: null input");
  B200_CHECK_ARG(((uintptr_t)hidden & 15) == 0, "ep_dispatch: hidden must be 16-byte aligned");
  cudaStream_t st = as_stream(stream);
  const int ep = pe->ep_size;

  // 1. (token, rank) slots sorted by rank: counts and positions inside the fixed regions
  SortParams sp;
  sp.ids = topk_ids; sp.ids_dtype = ids_dtype; sp.map = nullptr;
  sp.numel = num_tokens * ep;
  sp.id_limit = ep; sp.n_buckets = ep; sp.block_size = 1;
  sp.topk = pe->topk; sp.ep_size = ep; sp.ep_local_experts = pe->num_local_experts;
  sp.ep_slot = pe->expert_slot;
  sp.bucket_stride = pe->capacity;
  AlignOut ao = {};
  RemapOut ro = {send_counts, send_pos};
  if (int rc = run_sort<1>(sp, ao, ro, workspace, workspace_bytes, st)) return rc;

  // 2. rows, scales, ids, weights and counts to their owners
  EpDispatchParams p;
  for (int d = 0; d < ep; ++d) {
    p.peer.rows[d] = reinterpret_cast<uint8_t*>(pe->recv_rows[d]);
    p.peer.scales[d] = pe->recv_scales[d];
    p.peer.ids[d] = pe->recv_ids[d];
    p.peer.weights[d] = pe->recv_weights[d];
    p.peer.counts[d] = pe->recv_counts[d];
  }
  p.ids = topk_ids; p.ids_dtype = ids_dtype; p.weights = topk_weights;
  p.send_counts = send_counts; p.send_pos = send_pos; p.slot = pe->expert_slot;
  p.num_tokens = num_tokens; p.capacity = pe->capacity;
  p.ep = ep; p.rank = pe->ep_rank; p.e_local = pe->num_local_experts; p.H = pe->hidden; p.K = pe->topk;
  const unsigned grid = (unsigned)(num_tokens > 0 ? num_tokens : 1);
  if (dtype == B200MOE_BF16) {
    if (pe->quantized) ep_dispatch_kernel<__nv_bfloat16, true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)hidden, p);
    else ep_dispatch_kernel<__nv_bfloat16, false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)hidden, p);
  } else {
    if (pe->quantized) ep_dispatch_kernel<__half, true><<<grid, 256, 0, st>>>((const __half*)hidden, p);
    else ep_dispatch_kernel<__half, false><<<grid, 256, 0, st>>>((const __half*)hidden, p);
  }
  B200_LAUNCH_OK("ep_dispatch_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_mask_unused(const b200moe_ep_peers* pe, b200moe_stream stream) {
  if (int rc = check_peers(pe, "ep_mask_unused")) return rc;
  const int64_t cells = pe->capacity * pe->topk;
  int gx = (int)((cells + 255) / 256);
  if (gx > 64) gx = 64;
  ep_mask_unused_kernel<<<dim3(gx, pe->ep_size), 256, 0, as_stream(stream)>>>(
      pe->recv_ids[pe->ep_rank], pe->recv_counts[pe->ep_rank], pe->capacity, pe->topk);
  B200_LAUNCH_OK("ep_mask_unused_kernel");
  return B200MOE_OK;
}

extern "C" int b200moe_ep_combine(const b200moe_ep_peers* pe, const void* moe_out, const int32_t* row_map,
                                  b200moe_dtype dtype, b200moe_stream stream) {
  if (int rc = check_peers(pe, "ep_combine")) return rc;
  B200_CHECK_ARG(dtype == B200MOE_BF16 || dtype == B200MOE_F16, "ep_combine: rows must be bfloat16 or float16");
  B200_CHECK_ARG(moe_out && row_map, "ep_combine: null pointer");
  B200_CHECK_ARG(((uintptr_t)moe_out & 15) == 0, "ep_combine: moe_out must be 16-byte aligned");
  B200_CHECK_ARG(pe->topk <= 64, "ep_combine: topk larger than 64 is not supported");
  EpCombineParams p;
  for (int d = 0; d < pe->ep_size; ++d) p.comb[d] = reinterpret_cast<uint8_t*>(pe->comb_rows[d]);
  p.weights = pe->recv_weights[pe->ep_rank];
  p.counts = pe->recv_counts[pe->ep_rank];
  p.row_map = row_map;
  p.capacity = pe->capacity; p.ep = pe->ep_size; p.rank = pe->ep_rank; p.H = pe->hidden; p.K = pe->topk;
  const dim3 grid((unsigned)pe->capacity, (unsigned)pe->ep_size);
  if (dtype == B200MOE_BF16) ep_combine_kernel<__nv_bfloat16><<<grid, 256, 0, as_stream(stream)>>>((const __nv_bfloat16*)moe_out, p);
  else ep_combine_kernel<__half><<<grid, 256, 0, as_stream(stream)>>>((const __half*)moe_out, p);
  B200_LAUNCH_OK("ep_combine_kernel");
  return B200MOE_OK;
}
