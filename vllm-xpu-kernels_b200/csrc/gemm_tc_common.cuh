// Pieces shared by the tensor-core grouped GEMM kernels: the tile walk over
// ragged expert segments, output conversion, and host-side tensor-map encoding.
#pragma once

#include <atomic>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace b200moe {
namespace {

constexpr int kFeat = 128;          // features per tile (UMMA M)
constexpr int kMaxExperts = 1024;

struct TileInfo {
  int e, n_tile, m_tile, row0, valid;   // e: index of the weights the tile multiplies with
};

// Tiles of one expert are numbered feature-tile-major with the token tiles
// adjacent, so CTAs that run at the same time share a weight tile in L2.
// With w_experts > 0 the row segments outnumber the weight sets: segment s multiplies with
// weights s % w_experts (the segments are the (source rank, local expert) pairs of an
// expert-parallel exchange, source-major).
template <int BT>
__device__ __forceinline__ void locate_tile(const int* tile_start, const int* row_start, int t,
                                            int& cursor, TileInfo& ti, int w_experts = 0) {
  while (t >= tile_start[cursor + 1]) ++cursor;
  const int local = t - tile_start[cursor];
  const int rows = row_start[cursor + 1] - row_start[cursor];
  const int m_tiles = (rows + BT - 1) / BT;
  ti.e = w_experts > 0 ? cursor % w_experts : cursor;
  ti.n_tile = local / m_tiles;
  ti.m_tile = local - ti.n_tile * m_tiles;
  ti.row0 = row_start[cursor] + ti.m_tile * BT;
  const int left = rows - ti.m_tile * BT;
  ti.valid = left < BT ? left : BT;
}

__device__ __forceinline__ void store_out(void* d, int out_f16, int64_t idx, float v) {
  if (out_f16) reinterpret_cast<__half*>(d)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(d)[idx] = __float2bfloat16_rn(v);
}
// A bounded wait gave up: tell the caller through its status word.  A plain store, so the
// word may live in device memory or in mapped host memory that the host polls without a
// synchronisation.
__device__ __forceinline__ void report_timeout(int32_t* status) {
  if (status != nullptr) {
    *reinterpret_cast<volatile int32_t*>(status) = 1;
    __threadfence_system();
  }
}
__device__ __forceinline__ float load_bias(const void* b, int out_f16, int64_t idx) {
  if (out_f16) return __half2float(reinterpret_cast<const __half*>(b)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(b)[idx]);
}


// Output path of the epilogue warps.  A warp holds a block of the result as
// vals[i] = D(token i, feature lane) (one TMEM lane per thread), but D is
// row-major over features, so a direct store would write 2 bytes per lane into
// 32 different 64-byte pieces.  The block is transposed through a per-warp
// shared-memory tile ([token][feature], 16-bit) and written as 16-byte vectors:
// kFeat/8 lanes cover one token row, 256/kFeat rows per store instruction.
// kFeat = 32 (one value per lane) or 16 (values on the even lanes only).
template <int kTok, int kFeatW>
__device__ __forceinline__ void store_block_transposed(uint16_t* xp, const float (&vals)[kTok],
                                                       void* d, int out_f16, int64_t row0,
                                                       int tok_valid, int64_t m_limit, int n_out,
                                                       int feat0, int lane) {
  const int col = (kFeatW == 32) ? lane : (lane >> 1);
  const bool writer = (kFeatW == 32) || !(lane & 1);
  const uint32_t xp_s = ptx::smem_u32(xp);
#pragma unroll
  for (int i = 0; i < kTok; ++i) {
    uint16_t bits;
    if (out_f16) { const __half h = __float2half_rn(vals[i]); bits = *reinterpret_cast<const uint16_t*>(&h); }
    else { const __nv_bfloat16 h = __float2bfloat16_rn(vals[i]); bits = *reinterpret_cast<const uint16_t*>(&h); }
    if (writer) ptx::sts16(xp_s + (i * kFeatW + col) * 2, bits);
  }
  __syncwarp();
  constexpr int kLanesPerRow = kFeatW / 8;          // 16-byte pieces per token row
  constexpr int kRowsPerIter = 32 / kLanesPerRow;
  const int piece = lane % kLanesPerRow;
  const int f = feat0 + piece * 8;
#pragma unroll
  for (int it = 0; it < kTok / kRowsPerIter; ++it) {
    const int tok = lane / kLanesPerRow + it * kRowsPerIter;
    if (tok < tok_valid && row0 + tok < m_limit && f < n_out) {
      const uint4 q = ptx::lds128(xp_s + (tok * kFeatW + piece * 8) * 2);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(d) + (row0 + tok) * (int64_t)n_out + f) = q;
    }
  }
  __syncwarp();
}

// Warp-cooperative prefix sums over the experts: row_start[e], tile_start[e]
// (tiles of expert e = ceil(rows_e / BT) * n_tiles).  Called by one full warp.
template <int BT>
__device__ __forceinline__ void build_tile_prefix(const int32_t* rows_per_expert, int num_experts,
                                                  int n_tiles, int* row_start, int* tile_start) {
  const int lane = threadIdx.x & 31;
  int carry_r = 0, carry_t = 0;
  if (lane == 0) { row_start[0] = 0; tile_start[0] = 0; }
  for (int base = 0; base < num_experts; base += 32) {
    const int e = base + lane;
    int r = (e < num_experts) ? rows_per_expert[e] : 0;
    if (r < 0) r = 0;
    int tl = ((r + BT - 1) / BT) * n_tiles;
    int ir = r, it = tl;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o_r = __shfl_up_sync(0xffffffffu, ir, d);
      const int o_t = __shfl_up_sync(0xffffffffu, it, d);
      if (lane >= d) { ir += o_r; it += o_t; }
    }
    if (e < num_experts) {
      row_start[e + 1] = carry_r + ir;
      tile_start[e + 1] = carry_t + it;
    }
    carry_r += __shfl_sync(0xffffffffu, ir, 31);
    carry_t += __shfl_sync(0xffffffffu, it, 31);
  }
}

// ------------------------------ host side ------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int encode_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
               const cuuint64_t* dims, const cuuint64_t* strides_bytes, const cuuint32_t* box,
               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return fail(B200MOE_E_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), dims, strides_bytes, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(B200MOE_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return B200MOE_OK;
}

constexpr int kMaxDevices = 64;

inline int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

// SM count of the current device (cached per device: a process may drive several).
int sm_count() {
  static std::atomic<int> n[kMaxDevices];
  const int dev = current_device();
  int v = n[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    if (v <= 0) v = 148;
    n[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (kernel, device) pair: the
// largest size set so far is remembered per device, so a process that drives several GPUs
// configures the kernel on each of them.  One static instance per kernel instantiation.
struct SmemConfig {
  std::atomic<size_t> bytes[kMaxDevices];
  template <typename Kern>
  int ensure(Kern kern, size_t need) {
    const int dev = current_device();
    if (bytes[dev].load(std::memory_order_acquire) < need) {
      B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need));
      bytes[dev].store(need, std::memory_order_release);
    }
    return B200MOE_OK;
  }
};


}  // namespace
}  // namespace b200moe
