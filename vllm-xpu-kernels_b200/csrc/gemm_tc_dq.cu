// Tensor-core grouped GEMM for weights that are dequantised on the way in:
// MXFP4 (two e2m1 codes per byte, [E,N,K/2], one e8m0 scale per 32 elements,
// [E,N,K/32]) or INT4 (two's-complement nibbles, [E,N,K/2], one 16-bit scale per
// group of 32..256 elements, [E,N,K/group]) times 16-bit activations.
//
// Same orientation, tile walk and epilogue as grouped_gemm_tc_kernel (weights'
// output features on the 128-row M side of tcgen05.mma, tokens on the N side),
// with one more role between the TMA producer and the MMA issuer:
//   warp 0   : TMA producer: packed weight tile (128 rows x 32 bytes, no
//              swizzle) and activation tile (BT rows x 128 bytes, 128B swizzle)
//   warps 2-9: converters: two threads per row, each expands 32 of the row's 64
//              16-bit values (code * 2^(scale-127), exact in bf16/fp16 range)
//              and writes them in the 128-byte-swizzled K-major layout the MMA
//              reads; generic-proxy writes are fenced before the hand-over
//   warp 1   : MMA issuer (kind::f16), owns tensor memory
//   warps 10-13: epilogue
// HBM sees only the 4-bit weights (0.53 bytes per element with scales).
//
// Numerics follow csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:400-419, 455-471 of
// vllm-xpu-kernels: LUT[code] * 2^(byte-127) (INT4: nibble * scale) rounded to
// the activation type before the multiply, fp32 accumulation, bias added in fp32.
#include <cuda_fp4.h>
#include <stdlib.h>

#include "common.cuh"
#include "gemm_tc_common.cuh"
#include "sm100_ptx.cuh"

namespace b200moe {
namespace {

constexpr int kOpBytes = 16384;   // 128 rows x 64 sixteen-bit values
constexpr int kRawBytes = 4096;   // 128 rows x 32 packed bytes
constexpr int kDqConvWarps = 8;    // two per weight row half
constexpr int kDqThreads = 64 + 32 * kDqConvWarps + 128;
constexpr int kDqMaxStages = 8;
constexpr int kDqGroup = 8;      // K blocks per scale prefetch

struct DqParams {
  const uint8_t* w_scale;  // [E, N, K/32] e8m0; INT4: [E, N, K/group] 16-bit values
  int group;               // INT4: K elements per scale
  const void* bias;
  void* d;
  const int32_t* rows_per_expert;
  int32_t* status;
  int64_t m;
  int n, k, num_experts;
  int n_tiles, num_kb;
  uint32_t idesc;
  int out_f16;
  int swiglu;      // 1: D[m, f/2] = swigluoai(acc[m,f], acc[m,f+1]) for even f
  float alpha, limit, clamp_limit;
  int debug;  // experiment switches (B200MOE_DEBUG), 0 in normal use
};

template <int BT>
struct DqCtrl {
  uint64_t full_raw[kDqMaxStages];
  uint64_t full_op[kDqMaxStages];
  uint64_t empty[kDqMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int tile_start[kMaxExperts + 1];
  int row_start[kMaxExperts + 1];
  alignas(16) uint16_t xpose[4][32 * 32];  // per epilogue warp: output transpose tile
};

template <int BT>
__host__ __device__ constexpr int dq_stage_bytes() { return kOpBytes + BT * 128 + kRawBytes; }
template <int BT>
__host__ __device__ constexpr int dq_stages() {
  return (196 * 1024) / dq_stage_bytes<BT>() > kDqMaxStages ? kDqMaxStages
                                                            : (196 * 1024) / dq_stage_bytes<BT>();
}
template <int BT>
__host__ __device__ constexpr size_t dq_smem_bytes() {
  return 1024 + (size_t)dq_stages<BT>() * dq_stage_bytes<BT>() + sizeof(DqCtrl<BT>);
}
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

template <int BT, bool kInt4>
__global__ void __launch_bounds__(kDqThreads, 1)
grouped_gemm_dq_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_w, const DqParams p) {
  constexpr int kStages = dq_stages<BT>();
  constexpr int kStageBytes = dq_stage_bytes<BT>();
  constexpr int kChunk = BT >= 32 ? 32 : 16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  DqCtrl<BT>* ctrl = reinterpret_cast<DqCtrl<BT>*>(smem + kStages * kStageBytes);
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
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&ctrl->full_raw[s], 1);
      ptx::mbar_init(&ctrl->full_op[s], kDqConvWarps);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], 4);
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

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti);
        const int n0 = ti.n_tile * kFeat;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* st = smem + s * kStageBytes;
          ptx::mbar_expect_tx(&ctrl->full_raw[s], ((p.debug & 2) ? 0 : kRawBytes) + BT * 128);
          if (!(p.debug & 2)) ptx::tma_load_3d(st + kOpBytes + BT * 128, &tmap_w, &ctrl->full_raw[s], kb * 32, n0, ti.e);
          ptx::tma_load_2d(st + kOpBytes, &tmap_a, &ctrl->full_raw[s], kb * 64, ti.row0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      uint32_t it = 0, acc_it = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti);
        const uint32_t a = acc_it & 1;
        if (!ptx::mbar_wait(&ctrl->acc_empty[a], ((acc_it >> 1) & 1) ^ 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1;
          if (!ptx::mbar_wait(&ctrl->full_op[s], ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t wbase = ptx::smem_u32(smem + s * kStageBytes);
          const uint32_t abase = wbase + kOpBytes;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t wdesc = ptx::make_smem_desc(wbase + j * 32, 16, 1024);
            const uint64_t adesc = ptx::make_smem_desc(abase + j * 32, 16, 1024);
            ptx::umma<false>(tmem_base + a * BT, wdesc, adesc, p.idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          ptx::umma_commit(&ctrl->empty[s]);
        }
        if (ok) { ptx::umma_commit(&ctrl->acc_full[a]); ++acc_it; }
      }
    }
  } else if (warp < 2 + kDqConvWarps) {
    // ------------------------------ converters --------------------------------
    const int ct = (warp - 2) * 32 + lane;
    const int r = ct & 127;                // row of the tile
    const int half = ct >> 7;              // which 32 of the row's 64 values
    const int kgroups = p.k / 32;           // scale bytes per weight row
    const bool pair_aligned = (kgroups % 2 == 0) && ((reinterpret_cast<uintptr_t>(p.w_scale) & 1) == 0);
    uint32_t it = 0;
    int cursor = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      TileInfo ti;
      locate_tile<BT>(tile_start, row_start, t, cursor, ti);
      const int feat = ti.n_tile * kFeat + r;
      const bool feat_ok = feat < p.n;
      const uint8_t* srow = p.w_scale + ((int64_t)ti.e * p.n + (feat_ok ? feat : 0)) * kgroups;
      // Scale bytes of this thread's row, kDqGroup K blocks (two bytes each) at a
      // time and one group ahead of their use, so the loads never stall a stage.
      auto fetch = [&](int g, uint32_t (&dst)[kDqGroup]) {
#pragma unroll
        for (int u = 0; u < kDqGroup; ++u) {
          const int kb = g * kDqGroup + u;
          if (kInt4) {
            // the 16-bit scale of this thread's 32 values, duplicated into both halves
            uint32_t v = 0;
            if (feat_ok && kb < p.num_kb) {
              const uint16_t* s16 = reinterpret_cast<const uint16_t*>(p.w_scale) +
                                    ((int64_t)ti.e * p.n + feat) * (p.k / p.group);
              v = s16[(kb * 64 + half * 32) / p.group];
            }
            dst[u] = v | (v << 16);
            continue;
          }
          uint32_t v = 0x7f7fu;  // 2^0 twice
          if (feat_ok && 2 * kb + 1 < kgroups) {
            if (pair_aligned) v = *reinterpret_cast<const uint16_t*>(srow + 2 * kb);
            else v = (uint32_t)srow[2 * kb] | ((uint32_t)srow[2 * kb + 1] << 8);
          } else if (feat_ok && 2 * kb < kgroups) {
            v = (uint32_t)srow[2 * kb] | 0x7f00u;
          }
          dst[u] = v;
        }
      };
      uint32_t cur_s[kDqGroup], nxt_s[kDqGroup];
      fetch(0, cur_s);
      const int n_groups = (p.num_kb + kDqGroup - 1) / kDqGroup;
      for (int g = 0; g < n_groups && ok; ++g) {
       if (g + 1 < n_groups) fetch(g + 1, nxt_s);
#pragma unroll
       for (int u = 0; u < kDqGroup; ++u) {
        const int kb = g * kDqGroup + u;
        if (kb < p.num_kb && ok) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1;
        const uint32_t c0s = cur_s[u] & 0xffu, c1s = cur_s[u] >> 8;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->full_raw[s], ph, abort_flag))) {
          *abort_flag = 1; ok = false;
        }
        if (ok && (p.debug & 1)) {
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&ctrl->full_op[s]);
        }
        if (ok && !(p.debug & 1)) {
        const uint32_t st = ptx::smem_u32(smem + s * kStageBytes);
        const uint4 q0 = ptx::lds128(st + kOpBytes + BT * 128 + r * 32 + half * 16);
        const uint32_t words[4] = {q0.x, q0.y, q0.z, q0.w};
        const uint32_t sbyte = half ? c1s : c0s;
        const uint32_t orow = st + (r >> 3) * 1024 + (r & 7) * 128;
        if (kInt4) {
          // nibble n (two's complement) -> 128 + (n ^ 8) (bf16 0x4300 | .; fp16: 1024 +,
          // 0x6400 | .) exactly, minus 136 (1032) = n as a signed value, times the scale:
          // one rounding, as the reference's product in the activation type.
          const uint32_t magic = p.out_f16 ? 0x64006400u : 0x43004300u;
          const uint32_t offs = p.out_f16 ? 0x64086408u : 0x43084308u;   // 1032.0 / 136.0
          const uint32_t sc2 = cur_s[u];
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
              if (p.out_f16) {
                const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&bits),
                                                  *reinterpret_cast<const __half2*>(&offs)),
                                          *reinterpret_cast<const __half2*>(&sc2));
                o[j] = *reinterpret_cast<const uint32_t*>(&v);
              } else {
                const __nv_bfloat162 v = __hmul2(__hsub2(*reinterpret_cast<const __nv_bfloat162*>(&bits),
                                                         *reinterpret_cast<const __nv_bfloat162*>(&offs)),
                                                 *reinterpret_cast<const __nv_bfloat162*>(&sc2));
                o[j] = *reinterpret_cast<const uint32_t*>(&v);
              }
            }
            ptx::sts128(orow + (((4 * half + c) ^ (r & 7)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
          }
        } else if (!p.out_f16 && sbyte <= 128u) {
          // Integer path for bf16.  Put the code's exponent and mantissa bits
          // where bf16 keeps them ((c & 7) << 6, sign to bit 15): read as bf16
          // that is the code's value times 2^-126, subnormal codes included, so
          // one exact multiply by 2^(scale - 1) yields code * 2^(scale - 127).
          const uint32_t m0 = (sbyte + 126u) << 7;
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
        } else {
          const float sc = e8m0_to_f32(sbyte);
#pragma unroll
          for (int c = 0; c < 4; ++c) {  // 8 values = one 16-byte chunk of the row
            const uint32_t w = words[c];
            uint32_t o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const float2 f = e2m1x2_to_float2((w >> (8 * b)) & 0xffu);
              o[b] = pack16(f.x * sc, f.y * sc, p.out_f16);
            }
            ptx::sts128(orow + (((4 * half + c) ^ (r & 7)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
          }
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctrl->full_op[s]);
        }
        ++it;
        }
       }
#pragma unroll
       for (int u = 0; u < kDqGroup; ++u) cur_s[u] = nxt_s[u];
      }
    }
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
          for (int i = 0; i < kChunk; ++i) {
            float x = __uint_as_float(v[i]) + bias_v;
            if (p.swiglu) {
              // gate sits on even features, up on the next odd one: neighbours in the warp
              const float other = __shfl_xor_sync(0xffffffffu, x, 1);
              float gate = (lane & 1) ? other : x;
              float up = (lane & 1) ? x : other;
              if (p.clamp_limit > 0.f) {
                gate = fminf(gate, p.clamp_limit);
                up = fminf(fmaxf(up, -p.clamp_limit), p.clamp_limit);
              }
              gate = fminf(gate, p.limit);
              up = fminf(fmaxf(up, -p.limit), p.limit);
              x = (up + 1.0f) * gate * (1.0f / (1.0f + __expf(-gate * p.alpha)));
            }
            vals[i] = x;
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
  if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicExch(p.status, 1);
}

template <int BT, bool kInt4>
int launch_dq(const CUtensorMap& ta, const CUtensorMap& tw, const DqParams& p, int grid,
              cudaStream_t st) {
  auto kern = grouped_gemm_dq_kernel<BT, kInt4>;
  static bool configured = false;
  if (!configured) {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)dq_smem_bytes<BT>()));
    configured = true;
  }
  kern<<<grid, kDqThreads, dq_smem_bytes<BT>(), st>>>(ta, tw, p);
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
  p.bias = a->bias; p.d = a->d; p.rows_per_expert = a->rows_per_expert; p.status = a->status;
  p.m = a->m; p.n = a->n; p.k = a->k; p.num_experts = a->num_experts;
  p.n_tiles = (a->n + kFeat - 1) / kFeat;
  p.num_kb = a->k / 64;
  p.out_f16 = a->d_dtype == B200MOE_F16;
  p.swiglu = a->epilogue == B200MOE_EPI_SWIGLUOAI;
  p.alpha = a->act_alpha; p.limit = a->act_limit; p.clamp_limit = a->clamp_limit;
  {
    static int dbg = -1;
    if (dbg < 0) { const char* e = getenv("B200MOE_DEBUG"); dbg = e ? atoi(e) : 0; }
    p.debug = dbg;
  }

  const int64_t avg = (a->m + a->num_experts - 1) / a->num_experts;
  const int bt = avg <= 8 ? 16 : (avg <= 40 ? 64 : 128);
  const uint32_t fmt = a->a_dtype == B200MOE_BF16 ? 1u : 0u;
  p.idesc = ptx::make_idesc(fmt, fmt, 0u, 0u, kFeat, (uint32_t)bt);

  CUtensorMap ta, tw;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a->k, (cuuint64_t)a->m};
    cuuint64_t strides[1] = {(cuuint64_t)a->k * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)bt};
    int rc = encode_map(&ta, fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
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
  if (int4) {
    if (bt == 16) return launch_dq<16, true>(ta, tw, p, grid, st);
    if (bt == 64) return launch_dq<64, true>(ta, tw, p, grid, st);
    return launch_dq<128, true>(ta, tw, p, grid, st);
  }
  if (bt == 16) return launch_dq<16, false>(ta, tw, p, grid, st);
  if (bt == 64) return launch_dq<64, false>(ta, tw, p, grid, st);
  return launch_dq<128, false>(ta, tw, p, grid, st);
}

}  // namespace b200moe
