// Tensor-core grouped GEMM for weights that are dequantised on the way in:
// MXFP4 (two e2m1 codes per byte, [E,N,K/2], one e8m0 scale per 32 elements,
// [E,N,K/32]) or INT4 (two's-complement nibbles, [E,N,K/2], one 16-bit scale per
// group of 32..256 elements, [E,N,K/group]) times 16-bit activations.
//
// Same orientation, tile walk and epilogue as grouped_gemm_tc_kernel (weights'
// output features on the 128-row M side of tcgen05.mma, tokens on the N side),
// with one more role between the TMA producer and the MMA issuer:
//   warp 0   : TMA producer: per 64-wide K block a packed weight tile (128 rows x
//              32 bytes, no swizzle) and an activation tile (BT rows x 128 bytes,
//              128B swizzle); small token tiles move two K blocks per stage
//   warps 2-9: converters: two threads per row, each expands 32 of the row's 64
//              16-bit values per K block and writes them in the 128-byte-swizzled
//              K-major layout the MMA reads; generic-proxy writes are fenced
//              before the hand-over.  The tile's scales (one contiguous piece of
//              the scale tensor) are copied to shared memory with cp.async one
//              tile ahead, so the conversion loop has one path and no global loads
//   warp 1   : MMA issuer (kind::f16), owns tensor memory
//   warps 10-13: epilogue
// HBM sees only the 4-bit weights (0.53 bytes per element with scales).
//
// Numerics follow csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:400-419, 455-471 of
// vllm-xpu-kernels: LUT[code] * 2^(byte-127) (INT4: nibble * scale) rounded to
// the activation type before the multiply, fp32 accumulation, bias added in fp32.
#include <cuda_fp4.h>
#include "common.cuh"
#include "gemm_tc_common.cuh"
#include "sm100_ptx.cuh"

namespace b200moe {
namespace {

constexpr int kOpBytes = 16384;   // 128 rows x 64 sixteen-bit values
constexpr int kRawBytes = 4096;   // 128 rows x 32 packed bytes
constexpr int kDqConvWarps = 8;    // two threads per weight row
constexpr int kDqThreads = 64 + 32 * kDqConvWarps + 128;
constexpr int kDqMaxStages = 8;
constexpr int kDqSfwCap = 24576;   // largest scale piece of a tile staged in shared memory

struct DqParams {
  const uint8_t* w_scale;  // MXFP4: [E, N, K/32] e8m0; INT4: [E, N, K/group] 16-bit values
  int group;               // INT4: K elements per scale
  int scale_row_bytes;     // bytes of one weight row's scales
  int sfw_bytes;           // bytes of one staging buffer
  const void* bias;
  void* d;
  const int32_t* rows_per_expert;
  int32_t* status;
  int64_t m;
  int n, k, num_experts;
  int n_tiles, num_kb;     // num_kb: 64-wide K blocks
  int stages, stage_bytes;
  uint32_t idesc;
  int out_f16;
  int swiglu;      // 1: D[m, f/2] = swigluoai(acc[m,f], acc[m,f+1]) for even f
  float alpha, limit, clamp_limit;
};

template <int BT>
struct DqCtrl {
  uint64_t full_raw[kDqMaxStages];
  uint64_t full_op[kDqMaxStages];
  uint64_t empty[kDqMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sfw_full[2];
  uint64_t sfw_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int tile_start[kMaxExperts + 1];
  int row_start[kMaxExperts + 1];
  alignas(16) uint16_t xpose[4][32 * 32];  // per epilogue warp: output transpose tile
};

template <int BT>
__host__ __device__ constexpr uint32_t dq_tmem_cols() { return 2 * BT < 32 ? 32u : (uint32_t)(2 * BT); }

// Two e2m1 codes (low nibble = even k) -> two fp32 values.
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
  const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)byte, __NV_E2M1);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int out_f16) {
  if (out_f16) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// MXFP4 through fp32: fp16 activations, and bf16 with scales above 2^1 (the
// integer path's multiplier 2^(scale-1) would leave the bf16 range).  Kept out
// of line so that the common conversion loop stays small.
__device__ __noinline__ void convert_mxfp4_general(uint32_t orow, const uint4 q0, uint32_t sbyte, int half, int r,
                                                   int out_f16) {
  const uint32_t words[4] = {q0.x, q0.y, q0.z, q0.w};
  const float sc = e8m0_to_f32(sbyte);
#pragma unroll
  for (int c = 0; c < 4; ++c) {  // 8 values = one 16-byte chunk of the row
    const uint32_t w = words[c];
    uint32_t o[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const float2 f = e2m1x2_to_float2((w >> (8 * b)) & 0xffu);
      o[b] = pack16(f.x * sc, f.y * sc, out_f16);
    }
    ptx::sts128(orow + (((4 * half + c) ^ (r & 7)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
  }
}

// 32 packed values of row r (16 bytes) -> 32 sixteen-bit values in the swizzled row.
// scale: MXFP4 the e8m0 byte, INT4 the 16-bit scale duplicated in both halves.
template <bool kInt4, bool kF16>
__device__ __forceinline__ void convert_row_half(uint32_t orow, const uint4 q0, uint32_t scale, int half, int r) {
  const uint32_t words[4] = {q0.x, q0.y, q0.z, q0.w};
  if (kInt4) {
    // nibble n (two's complement) -> 128 + (n ^ 8) (bf16 0x4300 | .; fp16: 1024 +,
    // 0x6400 | .) exactly, minus 136 (1032) = n as a signed value, times the scale:
    // one rounding, as the reference's product in the activation type.
    constexpr uint32_t magic = kF16 ? 0x64006400u : 0x43004300u;
    constexpr uint32_t offs = kF16 ? 0x64086408u : 0x43084308u;   // 1032.0 / 136.0
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t w = words[c];
      const uint32_t xe = (w & 0x0F0F0F0Fu) ^ 0x08080808u;
      const uint32_t xo = ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t q = __byte_perm(xe, xo, (uint32_t)(j | (4 << 4) | ((4 + j) << 8) | (4 << 12))) & 0x00ff00ffu;
        const uint32_t bits = magic | q;
        if (kF16) {
          const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&bits),
                                            *reinterpret_cast<const __half2*>(&offs)),
                                    *reinterpret_cast<const __half2*>(&scale));
          o[j] = *reinterpret_cast<const uint32_t*>(&v);
        } else {
          const __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&bits),
                                                   *reinterpret_cast<const __nv_bfloat162*>(&offs)),
                                           *reinterpret_cast<const __nv_bfloat162*>(&scale));
          o[j] = *reinterpret_cast<const uint32_t*>(&v);
        }
      }
      ptx::sts128(orow + (((4 * half + c) ^ (r & 7)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
  } else if (kF16 || scale > 128u) {
    convert_mxfp4_general(orow, q0, scale, half, r, kF16 ? 1 : 0);
  } else {
    // Integer path for bf16.  Put the code's exponent and mantissa bits where bf16
    // keeps them ((c & 7) << 6, sign to bit 15): read as bf16 that is the code's
    // value times 2^-126, subnormal codes included, so one exact multiply by
    // 2^(scale - 1) yields code * 2^(scale - 127).
    const uint32_t m0 = (scale + 126u) << 7;
    const uint32_t mm = m0 | (m0 << 16);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t w = words[c];
      const uint32_t xe = w & 0x0F0F0F0Fu;          // codes of even k in bytes 0..3
      const uint32_t xo = (w >> 4) & 0x0F0F0F0Fu;   // codes of odd k
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t q = __byte_perm(xe, xo, (uint32_t)(j | (j << 4) | ((4 + j) << 8) | ((4 + j) << 12)));
        const uint32_t bits = ((q << 6) & 0x01C001C0u) | ((q << 12) & 0x80008000u);
        const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&bits),
                                            *reinterpret_cast<const __nv_bfloat162*>(&mm));
        o[j] = *reinterpret_cast<const uint32_t*>(&prod);
      }
      ptx::sts128(orow + (((4 * half + c) ^ (r & 7)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
    }
  }
}

// BT tokens per tile; kSub 64-wide K blocks per pipeline stage.
template <int BT, bool kInt4, bool kF16, int kSub>
__global__ void __launch_bounds__(kDqThreads, 1)
grouped_gemm_dq_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_w, const DqParams p) {
  constexpr int kChunk = BT >= 32 ? 32 : 16;
  constexpr int kABytes = BT * 128;
  constexpr int kAOff = kSub * kOpBytes;                       // stage: [operands][activations][packed]
  constexpr int kRawOff = kSub * (kOpBytes + kABytes);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages;
  const int stage_bytes = p.stage_bytes;
  DqCtrl<BT>* ctrl = reinterpret_cast<DqCtrl<BT>*>(smem + stages * stage_bytes);
  uint8_t* sfw = smem + stages * stage_bytes + ((sizeof(DqCtrl<BT>) + 15) & ~(size_t)15);
  volatile int* abort_flag = &ctrl->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {
    build_tile_prefix<BT>(p.rows_per_expert, p.num_experts, p.n_tiles, ctrl->row_start,
                          ctrl->tile_start);
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_w);
    }
  } else if (warp == 1) {
    ptx::tmem_alloc(&ctrl->tmem_base, dq_tmem_cols<BT>());
    ptx::tmem_relinquish();
  } else if (warp == 2 && lane == 0) {
    for (int s = 0; s < kDqMaxStages; ++s) {
      ptx::mbar_init(&ctrl->full_raw[s], 1);
      ptx::mbar_init(&ctrl->full_op[s], kDqConvWarps);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], 4);
      ptx::mbar_init(&ctrl->sfw_full[a], 32 * kDqConvWarps);
      ptx::mbar_init(&ctrl->sfw_empty[a], kDqConvWarps);
    }
    ctrl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->tile_start[p.num_experts];
  const int* tile_start = ctrl->tile_start;
  const int* row_start = ctrl->row_start;
  const int num_st = (p.num_kb + kSub - 1) / kSub;   // stages per tile

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti);
        const int n0 = ti.n_tile * kFeat;
        for (int si = 0; si < num_st; ++si) {
          if (!ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* st = smem + s * stage_bytes;
          const int kb0 = si * kSub;
          const int nsub = (p.num_kb - kb0) < kSub ? (p.num_kb - kb0) : kSub;
          ptx::mbar_expect_tx(&ctrl->full_raw[s], nsub * (kRawBytes + kABytes));
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            if (sub < nsub) {
              ptx::tma_load_3d(st + kRawOff + sub * kRawBytes, &tmap_w, &ctrl->full_raw[s], (kb0 + sub) * 32, n0, ti.e);
              ptx::tma_load_2d(st + kAOff + sub * kABytes, &tmap_a, &ctrl->full_raw[s], (kb0 + sub) * 64, ti.row0);
            }
          }
          if (++s == (uint32_t)stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // (the whole warp runs the loop with the same values; one elected lane issues)
    {
      uint32_t s = 0, ph = 0, acc_it = 0;
      int cursor = 0;
      bool ok = true;
      const uint32_t smem_base = ptx::smem_u32(smem);
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti);
        const uint32_t a = acc_it & 1;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_empty[a], ((acc_it >> 1) & 1) ^ 1, abort_flag))) break;
        ptx::tc_fence_after();
        // a partly filled token tile multiplies only its valid columns (UMMA N in steps of 16)
        const uint32_t idesc = (p.idesc & ~(0x3fu << 17)) | ((uint32_t)(((ti.valid + 15) & ~15) >> 3) << 17);
        for (int si = 0; si < num_st; ++si) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->full_op[s], ph, abort_flag))) { ok = false; break; }
          ptx::tc_fence_after();
          // every operand descriptor of the stage = the first one + a compile-time offset
          const uint64_t desc0 = ptx::make_smem_desc(smem_base + s * stage_bytes, 16, 1024);
          const int kb0 = si * kSub;
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            if (kb0 + sub < p.num_kb) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint64_t wdesc = desc0 + (uint64_t)((sub * kOpBytes + j * 32) >> 4);
                const uint64_t adesc = desc0 + (uint64_t)((kAOff + sub * kABytes + j * 32) >> 4);
                ptx::umma_elect<false>(tmem_base + a * BT, wdesc, adesc, idesc, (kb0 + sub > 0 || j > 0) ? 1u : 0u);
              }
            }
          }
          ptx::umma_commit_elect(&ctrl->empty[s]);
          if (++s == (uint32_t)stages) { s = 0; ph ^= 1; }
        }
        if (ok) { ptx::umma_commit_elect(&ctrl->acc_full[a]); ++acc_it; }
      }
    }
  } else if (warp < 2 + kDqConvWarps) {
    // ------------------------------ converters --------------------------------
    const int ct = (warp - 2) * 32 + lane;   // 0..255
    const int r = ct & 127;                  // row of the tile
    const int half = ct >> 7;                // which 32 of a K block's 64 values
    const bool staged = p.sfw_bytes > 0;
    uint32_t s = 0, ph = 0, tile_seq = 0;
    int cursor = 0, cursor_next = 0;
    bool ok = true;
    // The scales of a tile's 128 rows are one contiguous piece of the scale tensor:
    // copy it to staging buffer (seq & 1) asynchronously, one tile ahead.
    auto stage_scales = [&](const TileInfo& tt, uint32_t seq) -> bool {
      const uint32_t b = seq & 1;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->sfw_empty[b], ((seq >> 1) & 1) ^ 1, abort_flag))) return false;
      const int n0 = tt.n_tile * kFeat;
      const int rows_here = (p.n - n0) < kFeat ? (p.n - n0) : kFeat;
      const int len = rows_here * p.scale_row_bytes;
      const uint8_t* src = p.w_scale + ((int64_t)tt.e * p.n + n0) * p.scale_row_bytes;
      const uint32_t dst = ptx::smem_u32(sfw + b * p.sfw_bytes);
      for (int off = ct * 16; off < len; off += 256 * 16)
        ptx::cp_async_16(dst + off, src + off, (len - off) < 16 ? (len - off) : 16);
      ptx::cp_async_mbar_arrive(&ctrl->sfw_full[b]);
      return true;
    };
    TileInfo ti, ti_next;
    if (staged && (int)blockIdx.x < total_tiles) {
      locate_tile<BT>(tile_start, row_start, blockIdx.x, cursor_next, ti_next);
      if (!stage_scales(ti_next, 0u)) { *abort_flag = 1; ok = false; }
    }
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_seq) {
      locate_tile<BT>(tile_start, row_start, t, cursor, ti);
      const int t_next = t + gridDim.x;
      if (staged && t_next < total_tiles) {
        locate_tile<BT>(tile_start, row_start, t_next, cursor_next, ti_next);
        if (!stage_scales(ti_next, tile_seq + 1)) { *abort_flag = 1; ok = false; break; }
      }
      const uint32_t b = tile_seq & 1;
      if (staged && !__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->sfw_full[b], (tile_seq >> 1) & 1, abort_flag))) {
        *abort_flag = 1; ok = false; break;
      }
      const int feat = ti.n_tile * kFeat + r;
      const bool feat_ok = feat < p.n;
      const uint32_t srow_s = ptx::smem_u32(sfw + b * p.sfw_bytes) + r * p.scale_row_bytes;
      const uint8_t* srow_g = p.w_scale + ((int64_t)ti.e * p.n + (feat_ok ? feat : 0)) * p.scale_row_bytes;
      for (int si = 0; si < num_st && ok; ++si) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->full_raw[s], ph, abort_flag))) {
          *abort_flag = 1; ok = false; break;
        }
        const uint32_t st = ptx::smem_u32(smem + s * stage_bytes);
#pragma unroll
        for (int sub = 0; sub < kSub; ++sub) {
          const int kb = si * kSub + sub;
          if (kb < p.num_kb) {
            // this thread's 32 values share one scale
            uint32_t scale;
            if (kInt4) {
              const int idx = (kb * 64 + half * 32) / p.group;
              const uint32_t v = !feat_ok ? 0u
                                 : (staged ? ptx::lds16(srow_s + 2 * idx)
                                           : (uint32_t)reinterpret_cast<const uint16_t*>(srow_g)[idx]);
              scale = v | (v << 16);
            } else {
              const int idx = 2 * kb + half;
              scale = !feat_ok ? 127u : (staged ? ptx::lds8(srow_s + idx) : (uint32_t)srow_g[idx]);
            }
            const uint4 q0 = ptx::lds128(st + kRawOff + sub * kRawBytes + r * 32 + half * 16);
            const uint32_t orow = st + sub * kOpBytes + (r >> 3) * 1024 + (r & 7) * 128;
            convert_row_half<kInt4, kF16>(orow, q0, scale, half, r);
          }
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctrl->full_op[s]);
        if (++s == (uint32_t)stages) { s = 0; ph ^= 1; }
      }
      if (staged && ok) {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctrl->sfw_empty[b]);
      }
    }
    ptx::cp_async_wait_all();
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;
    const int et = q * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    const int n_out = p.swiglu ? p.n / 2 : p.n;
    uint32_t acc_it = 0;
    int cursor = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      TileInfo ti;
      locate_tile<BT>(tile_start, row_start, t, cursor, ti);
      const int feat = ti.n_tile * kFeat + et;
      const bool feat_ok = feat < p.n;
      float bias_v = 0.f;
      if (p.bias != nullptr && feat_ok) bias_v = load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + feat);
      const uint32_t a = acc_it & 1;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_full[a], (acc_it >> 1) & 1, abort_flag))) {
        *abort_flag = 1; ok = false; break;
      }
      ptx::tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < BT; c0 += kChunk) {
        if (c0 < ti.valid) {
          uint32_t v[kChunk];
          if (kChunk == 32) ptx::tmem_ld_32x32(tmem_base + a * BT + c0 + lane_sel, reinterpret_cast<uint32_t(&)[32]>(v));
          else ptx::tmem_ld_32x16(tmem_base + a * BT + c0 + lane_sel, reinterpret_cast<uint32_t(&)[16]>(v));
          ptx::tmem_wait_ld();
          float vals[kChunk];
#pragma unroll
          for (int i = 0; i < kChunk; ++i) vals[i] = __uint_as_float(v[i]) + bias_v;
          if (p.swiglu) {
            // One branch around the whole block: the unrolled body stays straight-line code, so
            // the shuffle / exp / divide chains of the columns overlap.
            const float c_lim = p.clamp_limit > 0.f ? p.clamp_limit : INFINITY;
#pragma unroll
            for (int i = 0; i < kChunk; ++i) {
              // gate sits on even features, up on the next odd one: neighbours in the warp
              const float x = vals[i];
              const float other = __shfl_xor_sync(0xffffffffu, x, 1);
              float gate = (lane & 1) ? other : x;
              float up = (lane & 1) ? x : other;
              gate = fminf(gate, c_lim);
              up = fminf(fmaxf(up, -c_lim), c_lim);
              gate = fminf(gate, p.limit);
              up = fminf(fmaxf(up, -p.limit), p.limit);
              vals[i] = (up + 1.0f) * gate * __fdividef(1.0f, 1.0f + __expf(-gate * p.alpha));
            }
          }
          if (p.swiglu)
            store_block_transposed<kChunk, 16>(ctrl->xpose[warp - 2 - kDqConvWarps], vals, p.d, p.out_f16,
                                               (int64_t)ti.row0 + c0, ti.valid - c0, p.m, n_out,
                                               (ti.n_tile * kFeat + q * 32) >> 1, lane);
          else
            store_block_transposed<kChunk, 32>(ctrl->xpose[warp - 2 - kDqConvWarps], vals, p.d, p.out_f16,
                                               (int64_t)ti.row0 + c0, ti.valid - c0, p.m, n_out,
                                               ti.n_tile * kFeat + q * 32, lane);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[a]);
      ++acc_it;
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    if (*abort_flag != 0) __nanosleep(20000);
    ptx::tmem_dealloc(tmem_base, dq_tmem_cols<BT>());
  }
  if (tid == 0 && *abort_flag != 0) report_timeout(p.status);
}

template <int BT, bool kInt4, bool kF16, int kSub>
int launch_dq(const CUtensorMap& ta, const CUtensorMap& tw, DqParams& p, int grid, cudaStream_t st) {
  auto kern = grouped_gemm_dq_kernel<BT, kInt4, kF16, kSub>;
  p.stage_bytes = kSub * (kOpBytes + BT * 128 + kRawBytes);
  const int fixed = 1024 + (int)((sizeof(DqCtrl<BT>) + 15) & ~(size_t)15) + 2 * p.sfw_bytes;
  p.stages = (227 * 1024 - fixed) / p.stage_bytes;
  if (p.stages > kDqMaxStages) p.stages = kDqMaxStages;
  if (p.stages < 2) return fail(B200MOE_E_UNSUPPORTED, "dequantising tensor-core GEMM: tile does not fit shared memory");
  const size_t smem = (size_t)fixed + (size_t)p.stages * p.stage_bytes;
  static SmemConfig configured;
  if (int rc = configured.ensure(kern, smem)) return rc;
  kern<<<grid, kDqThreads, smem, st>>>(ta, tw, p);
  B200_LAUNCH_OK("grouped_gemm_dq_kernel");
  return B200MOE_OK;
}

}  // namespace

// MXFP4 or INT4 weights x 16-bit activations on the tensor cores.  Returns
// B200MOE_E_UNSUPPORTED (no launch) for anything else.
int grouped_gemm_tc_dq(const b200moe_gemm_args* a, cudaStream_t st) {
  const bool int4 = a->w_format == B200MOE_W_INT4_NK;
  if (!(a->w_format == B200MOE_W_MXFP4_NK || int4) || a->a_dtype == B200MOE_FP8_E4M3)
    return fail(B200MOE_E_UNSUPPORTED, "dequantising tensor-core GEMM takes MXFP4 or INT4 weights only");
  if (int4 && ((uintptr_t)a->w_scale & 1))
    return fail(B200MOE_E_BADARG, "grouped GEMM: INT4 scales must be 2-byte aligned");
  if (a->epilogue == B200MOE_EPI_SILU_MUL)
    return fail(B200MOE_E_UNSUPPORTED, "dequantising tensor-core GEMM: SiLU epilogue not available");
  if (a->num_experts > kMaxExperts || a->k % 64 != 0 || (a->k / 2) % 16 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "dequantising tensor-core GEMM: K must be a multiple of 64");
  if (((uintptr_t)a->a & 15) || ((uintptr_t)a->w & 15) || ((uintptr_t)a->d & 15))
    return fail(B200MOE_E_BADARG, "grouped GEMM: A, W and D must be 16-byte aligned");
  if (a->epilogue == B200MOE_EPI_SWIGLUOAI && (a->n / 2) % 8 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "dequantising tensor-core GEMM: gated output width must be a multiple of 8");
  if (a->m == 0 || a->n == 0) return B200MOE_OK;

  DqParams p;
  p.w_scale = reinterpret_cast<const uint8_t*>(a->w_scale);
  p.group = int4 ? a->group_size : 32;
  p.scale_row_bytes = int4 ? (a->k / a->group_size) * 2 : a->k / 32;
  // Scales go through shared memory when every tile's piece starts on a 16-byte
  // boundary and two pieces fit; else the converters read them in place.
  const int piece = ((128 * p.scale_row_bytes + 15) & ~15) + 16;
  p.sfw_bytes = (((uintptr_t)a->w_scale & 15) == 0 && ((int64_t)a->n * p.scale_row_bytes) % 16 == 0 &&
                 piece <= kDqSfwCap) ? piece : 0;
  p.bias = a->bias; p.d = a->d; p.rows_per_expert = a->rows_per_expert; p.status = a->status;
  p.m = a->m; p.n = a->n; p.k = a->k; p.num_experts = a->num_experts;
  p.n_tiles = (a->n + kFeat - 1) / kFeat;
  p.num_kb = a->k / 64;
  p.out_f16 = a->d_dtype == B200MOE_F16;
  p.swiglu = a->epilogue == B200MOE_EPI_SWIGLUOAI;
  p.alpha = a->act_alpha; p.limit = a->act_limit; p.clamp_limit = a->clamp_limit;

  const int64_t rows_in_use = (a->rows_hint > 0 && a->rows_hint < a->m) ? a->rows_hint : a->m;
  const int64_t avg = (rows_in_use + a->num_experts - 1) / a->num_experts;
  int bt = avg <= 8 ? 16 : (avg <= 40 ? 64 : 128);
  const bool f16 = a->a_dtype == B200MOE_F16;
  const uint32_t fmt = f16 ? 0u : 1u;
  p.idesc = ptx::make_idesc(fmt, fmt, 0u, 0u, kFeat, (uint32_t)bt);

  CUtensorMap ta, tw;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a->k, (cuuint64_t)a->m};
    cuuint64_t strides[1] = {(cuuint64_t)a->k * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)bt};
    int rc = encode_map(&ta, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        a->a, dims, strides, box);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)(a->k / 2), (cuuint64_t)a->n, (cuuint64_t)a->num_experts};
    cuuint64_t strides[2] = {(cuuint64_t)(a->k / 2), (cuuint64_t)(a->k / 2) * a->n};
    cuuint32_t box[3] = {32, (cuuint32_t)kFeat, 1};
    int rc = encode_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->w, dims, strides, box,
                        CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  const int64_t tile_bound = ((a->m + bt - 1) / bt + a->num_experts) * (int64_t)p.n_tiles;
  int grid = sm_count();
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if (tile_bound < grid) grid = (int)tile_bound;
  if (grid < 1) grid = 1;
  // small token tiles move two K blocks per pipeline stage
#define B200_DQ_CASES(I4, F16)                                                   \
  if (bt == 16) return launch_dq<16, I4, F16, 2>(ta, tw, p, grid, st);           \
  if (bt == 64) return launch_dq<64, I4, F16, 2>(ta, tw, p, grid, st);           \
  return launch_dq<128, I4, F16, 1>(ta, tw, p, grid, st);
  if (int4 && f16) { B200_DQ_CASES(true, true) }
  if (int4) { B200_DQ_CASES(true, false) }
  if (f16) { B200_DQ_CASES(false, true) }
  B200_DQ_CASES(false, false)
#undef B200_DQ_CASES
}

}  // namespace b200moe
