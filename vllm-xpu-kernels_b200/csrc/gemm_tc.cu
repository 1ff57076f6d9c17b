// Grouped GEMM over ragged expert segments on the sm_100a tensor cores.
//
//   D[r0:r0+rows_e, :] = A[r0:r0+rows_e, :] * W_e^T (+ bias_e)      per expert e
//
// Orientation: the weight's output features are the 128-row M side of
// tcgen05.mma and the tokens are its N side (16..256 wide), so a decode-sized
// expert segment of a few rows costs a 16-column MMA instead of a 128-row one
// while the weights stream through shared memory exactly once.  The fp32
// accumulator therefore sits in tensor memory as [128 features (lanes)] x
// [BT tokens (columns)].
//
// One persistent CTA per SM walks the tile list (expert, feature tile, token
// tile) derived from rows_per_expert on the device — the host never reads it:
//   warp 0  : TMA producer  (weights through a 3-D map [E, N, K], activations
//             through a 2-D map [M, K]; 128-byte swizzle; ring of kStages)
//   warp 1  : MMA issuer    (one lane), owns the tensor-memory allocation
//   warps 2-5 : epilogue (tcgen05.ld -> registers -> global)
// 16-bit inputs use kind::f16 with the whole K loop accumulated in tensor
// memory (two accumulator stages, so the epilogue of one tile overlaps the
// MMAs of the next).  fp8 inputs use kind::f8f6f4 per 128-wide K block; the
// epilogue warps promote each block's partial sum into fp32 registers with
// a_scale[row, kb] * w_scale[e, n/128, kb], as the block-scaled recipe needs.
// (fp8 segments of 12 rows per expert or more go to the token-major kernels of
// gemm_tc_fp8t.cu, where that scale is one register per thread.)
//
// Every wait on an mbarrier is bounded (see sm100_ptx.cuh): on expiry the CTA
// raises an abort flag, all roles leave their loops, tensor memory is freed and
// *status is set to 1.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "gemm_tc_common.cuh"


namespace b200moe {
int grouped_gemm_tc_fp8t(const b200moe_gemm_args* a, cudaStream_t st);
namespace {

constexpr int kWTileBytes = 16384;  // 128 rows x 128 bytes, or the same area K-by-N
constexpr int kMaxAccStages = 8;
constexpr int kMaxStages = 8;

struct TcParams {
  const float* a_scale;
  const float* w_scale;
  const void* bias;
  void* d;
  const int32_t* rows_per_expert;
  int32_t* status;
  int64_t m;
  int n, k, num_experts;
  int w_experts;  // >0: segment s uses weight set s % w_experts
  int n_tiles;  // ceil(n / 128)
  int num_kb;   // K blocks of 128 bytes
  uint32_t idesc;
  int out_f16;  // 1: D and bias are float16, 0: bfloat16
  float clamp;  // gated epilogue: >0 clamps gate from above and up to +-clamp first
  int swiglu;   // 1: gate on even, up on odd features; D = (up + 1) * gate * sigmoid(alpha * gate), n / 2 wide
  float alpha, limit;
};

template <int BT, bool kFp8>
struct Ctrl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[kMaxAccStages];
  uint64_t acc_empty[kMaxAccStages];
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) float sc[kFp8 ? 4 : 1][2][kFp8 ? BT : 4];  // per epilogue warp, double buffered
  alignas(16) uint16_t xpose[4][32 * 32];  // per epilogue warp: output transpose tile
  int tile_start[kMaxExperts + 1];
  int row_start[kMaxExperts + 1];
};

// kGated (16-bit inputs, token tiles up to 128): a tile pairs the 128 gate features j0.. with the
// 128 up features n/2 + j0.. (the SiLU-and-mul layout, csrc/activation.cpp:131-133 of the
// reference); a stage carries both weight tiles, the MMAs fill two accumulators and the epilogue
// writes silu(gate) * up as [M, n/2].
template <int BT, bool kGated = false>
__host__ __device__ constexpr int stage_bytes() { return (kGated ? 2 : 1) * kWTileBytes + BT * 128; }
template <int BT, bool kGated = false>
__host__ __device__ constexpr int num_stages() {
  return (200 * 1024) / stage_bytes<BT, kGated>() > kMaxStages ? kMaxStages
                                                                : (200 * 1024) / stage_bytes<BT, kGated>();
}
template <int BT, bool kFp8, bool kGated = false>
__host__ __device__ constexpr size_t smem_bytes() {
  return 1024 + (size_t)num_stages<BT, kGated>() * stage_bytes<BT, kGated>() + sizeof(Ctrl<BT, kFp8>);
}
// Accumulator stages in tensor memory.  16-bit inputs hand over one whole tile
// per stage (two are enough); fp8 hands over every 128-wide K block, so more
// stages let the MMA issuer run ahead of the promoting epilogue warps.
template <int BT, bool kFp8>
__host__ __device__ constexpr int acc_stages() {
  return !kFp8 ? 2 : (512 / BT > kMaxAccStages ? kMaxAccStages : 512 / BT);
}
template <int BT, bool kFp8, bool kGated = false>
__host__ __device__ constexpr uint32_t tmem_cols() {
  const int c = acc_stages<BT, kFp8>() * BT * (kGated ? 2 : 1);
  return c <= 32 ? 32u : c <= 64 ? 64u : c <= 128 ? 128u : c <= 256 ? 256u : 512u;
}
// Four epilogue warps cover the 128 TMEM lanes.
constexpr int kEpiWarps = 4;
constexpr int kTcThreads = 64 + 32 * kEpiWarps;

template <int BT, bool kFp8, bool kWKn, bool kGated = false>
__global__ void __launch_bounds__(kTcThreads, 1)
grouped_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_w, const TcParams p) {
  static_assert(!kFp8 || BT <= 64, "fp8 promotion keeps BT accumulators per thread");
  static_assert(!kGated || (!kFp8 && BT <= 128), "gated epilogue: 16-bit inputs, two accumulators of BT columns per stage");
  constexpr int kStages = num_stages<BT, kGated>();
  constexpr int kStageBytes = stage_bytes<BT, kGated>();
  constexpr int kAOff = (kGated ? 2 : 1) * kWTileBytes;   // activations follow the weight tile(s) in a stage
  constexpr int kAccCols = BT * (kGated ? 2 : 1);         // tensor-memory columns of one accumulator stage
  constexpr int kElemsPerKb = kFp8 ? 128 : 64;  // K elements per 128-byte row
  constexpr int kAccStages = acc_stages<BT, kFp8>();
  constexpr int kCols = BT;                      // token columns one epilogue warp owns
  constexpr int kChunk = kCols >= 32 ? 32 : 16;  // columns per tcgen05.ld

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Ctrl<BT, kFp8>* ctrl = reinterpret_cast<Ctrl<BT, kFp8>*>(smem + kStages * kStageBytes);
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
    ptx::tmem_alloc(&ctrl->tmem_base, tmem_cols<BT, kFp8, kGated>());
    ptx::tmem_relinquish();
  } else if (warp == 2 && lane == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&ctrl->full[s], 1);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], kEpiWarps);
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
      uint32_t it = 0, s = 0, ph = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti, p.w_experts);
        const int n0 = ti.n_tile * kFeat;
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          if (!ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* wdst = smem + s * kStageBytes;
          uint8_t* adst = wdst + kAOff;
          ptx::mbar_expect_tx(&ctrl->full[s], kStageBytes);
          const int k0 = kb * kElemsPerKb;
#pragma unroll
          for (int half = 0; half < (kGated ? 2 : 1); ++half) {   // gate tile, then (gated) the up tile
            uint8_t* wd = wdst + half * kWTileBytes;
            const int nn = n0 + half * (p.n >> 1);
            if (!kWKn) {
              ptx::tma_load_3d(wd, &tmap_w, &ctrl->full[s], k0, nn, ti.e);
            } else if (kFp8) {
              ptx::tma_load_3d(wd, &tmap_w, &ctrl->full[s], nn, k0, ti.e);
            } else {
              ptx::tma_load_3d(wd, &tmap_w, &ctrl->full[s], nn, k0, ti.e);
              ptx::tma_load_3d(wd + kWTileBytes / 2, &tmap_w, &ctrl->full[s], nn + 64, k0, ti.e);
            }
          }
          ptx::tma_load_2d(adst, &tmap_a, &ctrl->full[s], k0, ti.row0);
          if (++s == (uint32_t)kStages) { s = 0; ph ^= 1; }
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
      // leading-dimension byte offset of the weight operand: K-major 16, MN-major 8192 (16-bit) / 16384 (fp8)
      constexpr uint32_t kWLbo = !kWKn ? 16u : (kFp8 ? 16384u : 8192u);
      constexpr uint32_t kWStep = !kWKn ? 32u : (kFp8 ? 4096u : 2048u);   // bytes per 32-byte K step
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti, p.w_experts);
        uint32_t a = acc_it % kAccStages;
        // A partly filled token tile multiplies only its valid columns (UMMA N in steps of 16).
        const uint32_t n_eff = (uint32_t)((ti.valid + 15) & ~15);
        const uint32_t idesc = (p.idesc & ~(0x3fu << 17)) | ((n_eff >> 3) << 17);
        constexpr bool per_block = kFp8;
        if (!per_block) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_empty[a], ((acc_it / kAccStages) & 1) ^ 1, abort_flag))) break;
          ptx::tc_fence_after();
        }
        for (int kb = 0; kb < p.num_kb; ++kb) {
          bool go = true;
          if (per_block) {
            a = acc_it % kAccStages;
            go = ptx::mbar_wait(&ctrl->acc_empty[a], ((acc_it / kAccStages) & 1) ^ 1, abort_flag);
          }
          if (go) go = ptx::mbar_wait(&ctrl->full[s], ph, abort_flag);
          if (!__all_sync(0xffffffffu, go)) { ok = false; break; }
          ptx::tc_fence_after();
          // every operand descriptor of the stage = one base descriptor + a compile-time
          // offset (the address field counts 16-byte units), so the issue loop is adds only
          const uint32_t st_addr = smem_base + s * kStageBytes;
          const uint64_t wdesc0 = ptx::make_smem_desc(st_addr, kWLbo, 1024);
          const uint64_t adesc0 = ptx::make_smem_desc(st_addr + kAOff, 16, 1024);
          const uint32_t d_tmem = tmem_base + a * kAccCols;
#pragma unroll
          for (int half = 0; half < (kGated ? 2 : 1); ++half) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t accumulate = per_block ? (j > 0) : (kb > 0 || j > 0);
              ptx::umma_elect<kFp8>(d_tmem + half * BT, wdesc0 + (uint64_t)((half * kWTileBytes + j * kWStep) >> 4),
                                    adesc0 + (uint64_t)((j * 32) >> 4), idesc, accumulate);
            }
          }
          ptx::umma_commit_elect(&ctrl->empty[s]);
          if (per_block) { ptx::umma_commit_elect(&ctrl->acc_full[a]); ++acc_it; }
          if (++s == (uint32_t)kStages) { s = 0; ph ^= 1; }
        }
        if (!per_block && ok) { ptx::umma_commit_elect(&ctrl->acc_full[a]); ++acc_it; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int et = q * 32 + lane;           // feature row inside the tile
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    constexpr int col0 = 0;                 // first token column of this warp
    // fp8 block-scale prefetch state (see the promotion loop below)
    constexpr int kGroup = 4;
    constexpr int kPerLane = (kCols + 31) / 32;
    struct ScaleRegs { float a[kPerLane][kGroup]; float w[kGroup]; };
    ScaleRegs cur, pre;
    bool pre_valid = false;
    const int kbs = p.k / 128;  // scale blocks along K
    const bool vec4_ok = kFp8 && (kbs % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.a_scale) & 15) == 0);
    auto fetch_group = [&](const TileInfo& tt, int g, ScaleRegs& r) {
      const int kb0 = g * kGroup;
      const int64_t wsb = ((int64_t)tt.e * (p.n / 128) + tt.n_tile) * kbs + kb0;
#pragma unroll
      for (int jb = 0; jb < kGroup; ++jb) r.w[jb] = (kb0 + jb < kbs) ? p.w_scale[wsb + jb] : 0.f;
#pragma unroll
      for (int u = 0; u < kPerLane; ++u) {
        const int c = col0 + lane + 32 * u;
        const int row = tt.row0 + c;
        const bool live = (lane + 32 * u < kCols) && (c < tt.valid) && (row < p.m);
        const float* src = p.a_scale + (int64_t)row * kbs + kb0;
        if (live && vec4_ok && kGroup == 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(src);
          r.a[u][0] = q4.x; r.a[u][1] = q4.y; r.a[u][2 % kGroup] = q4.z; r.a[u][3 % kGroup] = q4.w;
        } else if (live && vec4_ok && kGroup == 2) {   // kbs % 4 == 0 and a 16-byte base: 8-byte aligned pairs
          const float2 q2 = *reinterpret_cast<const float2*>(src);
          r.a[u][0] = q2.x; r.a[u][1] = q2.y;
        } else {
#pragma unroll
          for (int jb = 0; jb < kGroup; ++jb) r.a[u][jb] = (live && kb0 + jb < kbs) ? src[jb] : 0.f;
        }
      }
    };
    uint32_t acc_it = 0;
    int cursor = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      TileInfo ti;
      locate_tile<BT>(tile_start, row_start, t, cursor, ti, p.w_experts);
      const int feat = ti.n_tile * kFeat + et;
      const int n_out = kGated ? (p.n >> 1) : p.n;
      const bool feat_ok = feat < n_out;
      float bias_v = 0.f, bias_up = 0.f;
      if (p.bias != nullptr && feat_ok) {
        bias_v = load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + feat);
        if (kGated) bias_up = load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + (p.n >> 1) + feat);
      }

      if (!kFp8) {
        const uint32_t a = acc_it % kAccStages;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_full[a], (acc_it / kAccStages) & 1, abort_flag))) {
          *abort_flag = 1; ok = false; break;
        }
        ptx::tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < BT; c0 += kChunk) {
          if (c0 < ti.valid) {
            uint32_t v[kChunk], vu[kGated ? kChunk : 1];
            const uint32_t col = tmem_base + a * kAccCols + c0 + lane_sel;
            if (kChunk == 32) ptx::tmem_ld_32x32(col, reinterpret_cast<uint32_t(&)[32]>(v));
            else ptx::tmem_ld_32x16(col, reinterpret_cast<uint32_t(&)[16]>(v));
            if (kGated) {
              if (kChunk == 32) ptx::tmem_ld_32x32(col + BT, reinterpret_cast<uint32_t(&)[32]>(vu));
              else ptx::tmem_ld_32x16(col + BT, reinterpret_cast<uint32_t(&)[16]>(vu));
            }
            ptx::tmem_wait_ld();
            float vals[kChunk];
#pragma unroll
            for (int i = 0; i < kChunk; ++i) {
              vals[i] = __uint_as_float(v[i]) + bias_v;
              if (kGated) {
                float g = vals[i], u = __uint_as_float(vu[kGated ? i : 0]) + bias_up;
                if (p.clamp > 0.f) { g = fminf(g, p.clamp); u = fminf(fmaxf(u, -p.clamp), p.clamp); }
                vals[i] = g * __fdividef(1.0f, 1.0f + __expf(-g)) * u;
              }
            }
            if (!kGated && p.swiglu) {
              // gate and up of one output feature sit on neighbouring lanes
              const float c_lim = p.clamp > 0.f ? p.clamp : INFINITY;
#pragma unroll
              for (int i = 0; i < kChunk; ++i) {
                const float x = vals[i];
                const float other = __shfl_xor_sync(0xffffffffu, x, 1);
                float gate = (lane & 1) ? other : x;
                float up = (lane & 1) ? x : other;
                gate = fminf(fminf(gate, c_lim), p.limit);
                up = fminf(fmaxf(up, -c_lim), c_lim);
                up = fminf(fmaxf(up, -p.limit), p.limit);
                vals[i] = (up + 1.0f) * gate * __fdividef(1.0f, 1.0f + __expf(-gate * p.alpha));
              }
              store_block_transposed<kChunk, 16>(ctrl->xpose[warp - 2], vals, p.d, p.out_f16,
                                                 (int64_t)ti.row0 + c0, ti.valid - c0, p.m, p.n >> 1,
                                                 (ti.n_tile * kFeat + q * 32) >> 1, lane);
            } else {
              store_block_transposed<kChunk, 32>(ctrl->xpose[warp - 2], vals, p.d, p.out_f16,
                                                 (int64_t)ti.row0 + c0, ti.valid - c0, p.m, n_out,
                                                 ti.n_tile * kFeat + q * 32, lane);
            }
          }
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[a]);
        ++acc_it;
      } else {
        float acc[kCols];
#pragma unroll
        for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
        // Scales are fetched kGroup K blocks at a time, one group ahead of their
        // use (the first group of the next tile during the last group of this
        // one), so the strided a_scale loads are off the critical path.  Each
        // warp stages its own copy of the combined scales of its columns in
        // shared memory (lane l owns columns l, l+32, ..): no barrier couples
        // the warps.
        if (!pre_valid) fetch_group(ti, 0, cur);
        else cur = pre;
        pre_valid = false;
        const int n_groups = (p.num_kb + kGroup - 1) / kGroup;
        for (int g = 0; g < n_groups && ok; ++g) {
          if (g + 1 < n_groups) {
            fetch_group(ti, g + 1, pre);
          } else if (t + (int)gridDim.x < total_tiles) {
            int cursor2 = cursor;
            TileInfo tn;
            locate_tile<BT>(tile_start, row_start, t + gridDim.x, cursor2, tn, p.w_experts);
            fetch_group(tn, 0, pre);
            pre_valid = true;
          }
#pragma unroll
          for (int jb = 0; jb < kGroup; ++jb) {
            const int kb = g * kGroup + jb;
            if (kb >= p.num_kb) break;
            const uint32_t sc = ptx::smem_u32(ctrl->sc[warp - 2][kb & 1]);
#pragma unroll
            for (int u = 0; u < kPerLane; ++u)
              if (lane + 32 * u < kCols) ptx::sts32f(sc + (lane + 32 * u) * 4, cur.a[u][jb] * cur.w[jb]);
            __syncwarp();
            const uint32_t a = acc_it % kAccStages;
            if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_full[a], (acc_it / kAccStages) & 1, abort_flag))) {
              *abort_flag = 1; ok = false; break;
            }
            ptx::tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < kCols; c0 += kChunk) {
              const bool last_chunk = (c0 + kChunk >= kCols);
              uint32_t v[kChunk];
              if (col0 + c0 < ti.valid) {
                if (kChunk == 32) ptx::tmem_ld_32x32(tmem_base + a * BT + col0 + c0 + lane_sel, reinterpret_cast<uint32_t(&)[32]>(v));
                else ptx::tmem_ld_32x16(tmem_base + a * BT + col0 + c0 + lane_sel, reinterpret_cast<uint32_t(&)[16]>(v));
                ptx::tmem_wait_ld();
              }
              if (last_chunk) {  // the stage is free as soon as its last column is in registers
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[a]);
              }
              if (col0 + c0 < ti.valid) {
#pragma unroll
                for (int i = 0; i < kChunk; i += 4) {
                  const float4 s4 = ptx::lds128f(sc + (c0 + i) * 4);
                  acc[c0 + i + 0] = fmaf(__uint_as_float(v[i + 0]), s4.x, acc[c0 + i + 0]);
                  acc[c0 + i + 1] = fmaf(__uint_as_float(v[i + 1]), s4.y, acc[c0 + i + 1]);
                  acc[c0 + i + 2] = fmaf(__uint_as_float(v[i + 2]), s4.z, acc[c0 + i + 2]);
                  acc[c0 + i + 3] = fmaf(__uint_as_float(v[i + 3]), s4.w, acc[c0 + i + 3]);
                }
              }
            }
            ++acc_it;
          }
          if (g + 1 < n_groups) cur = pre;
        }
        if (ok) {
#pragma unroll
          for (int c0 = 0; c0 < kCols; c0 += kChunk) {
            if (col0 + c0 < ti.valid) {
              float vals[kChunk];
#pragma unroll
              for (int i = 0; i < kChunk; ++i) vals[i] = acc[c0 + i] + bias_v;
              store_block_transposed<kChunk, 32>(ctrl->xpose[warp - 2], vals, p.d, p.out_f16,
                                                 (int64_t)ti.row0 + col0 + c0, ti.valid - col0 - c0, p.m,
                                                 p.n, ti.n_tile * kFeat + q * 32, lane);
            }
          }
        }
      }
    }
  }

  // Teardown: everyone meets here, also after an aborted wait.
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    if (*abort_flag != 0) __nanosleep(20000);  // let copies still in flight land
    ptx::tmem_dealloc(tmem_base, tmem_cols<BT, kFp8, kGated>());
  }
  if (tid == 0 && *abort_flag != 0) report_timeout(p.status);
}

template <int BT, bool kFp8, bool kWKn, bool kGated = false>
int launch_tc(const CUtensorMap& ta, const CUtensorMap& tw, const TcParams& p, int grid,
              cudaStream_t st) {
  auto kern = grouped_gemm_tc_kernel<BT, kFp8, kWKn, kGated>;
  static SmemConfig configured;
  if (int rc = configured.ensure(kern, smem_bytes<BT, kFp8, kGated>())) return rc;
  kern<<<grid, kTcThreads, smem_bytes<BT, kFp8, kGated>(), st>>>(ta, tw, p);
  B200_LAUNCH_OK("grouped_gemm_tc_kernel");
  return B200MOE_OK;
}


// ---------------------------------------------------------------------------------
// 16-bit prefill on CTA pairs.  The 256-token tile above is bound by what a CTA brings into
// shared memory per K block (16 KB of weights + 32 KB of tokens for 4.2 MFLOP).  Here a
// cluster of two CTAs shares the 256 tokens of a tile and covers 256 features: each CTA loads
// its own 128 features' weights and one half of the tokens (32 KB per CTA and K block), the
// even CTA issues tcgen05.mma with cta_group::2 (M = 256: 128 weight rows from each CTA, N = 256:
// 128 token rows from each CTA) for both, and each CTA's tensor memory receives the 128 x 256
// accumulator of its own features, which its epilogue warps store as above.  A 16-bit GEMM
// hands its accumulator over once per tile, so the longer way a hand-over takes between two
// SMs does not matter here (it does in the fp8 kernel, which hands over every K block).
// Barriers: `full` and `acc_empty` of the even CTA collect both CTAs' loads and arrivals;
// `empty` and `acc_full` are signalled in both CTAs by a multicast tcgen05.commit.
constexpr int kPairTok = 256;
constexpr int kPairStageBytes = kWTileBytes + 128 * 128;   // this CTA's weights + its half of the tokens
constexpr int kPairStages = 6;
constexpr size_t kPairSmem = 1024 + (size_t)kPairStages * kPairStageBytes + sizeof(Ctrl<kPairTok, false>);
// kGated (SiLU-and-mul): the even CTA takes the 128 gate features j0.., the odd one the up features
// n/2 + j0.. of the same tokens.  The odd CTA's epilogue warps send their accumulator chunks
// (bias added, fp32) into the even CTA's shared memory, whose warps apply silu(gate) * up and
// store [M, n/2]: one stage of the ring makes room for the exchange buffers (per epilogue warp two
// buffers of 32 features x 32 tokens fp32) and their barriers.
constexpr int kPairGatedStages = 5;
constexpr int kPairXBuf = 32 * 32 * 4;
struct PairXchg {
  uint64_t full[kEpiWarps][2];    // in the even CTA: a chunk has arrived
  uint64_t empty[kEpiWarps][2];   // in the odd CTA: the even CTA has read the chunk
};
constexpr size_t kPairGatedSmem = 1024 + (size_t)kPairGatedStages * kPairStageBytes + kEpiWarps * 2 * kPairXBuf +
                                  sizeof(PairXchg) + sizeof(Ctrl<kPairTok, false>);

template <bool kWKn, bool kGated>
__global__ void __launch_bounds__(kTcThreads, 1)
grouped_gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                            const __grid_constant__ CUtensorMap tmap_w, const TcParams p) {
  constexpr int kChunk = 32;
  constexpr int kStagesP = kGated ? kPairGatedStages : kPairStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* xbuf = smem + kStagesP * kPairStageBytes;                               // kGated only
  PairXchg* xc = reinterpret_cast<PairXchg*>(xbuf + kEpiWarps * 2 * kPairXBuf);   // kGated only
  Ctrl<kPairTok, false>* ctrl = reinterpret_cast<Ctrl<kPairTok, false>*>(
      smem + kStagesP * kPairStageBytes + (kGated ? kEpiWarps * 2 * kPairXBuf + sizeof(PairXchg) : 0));
  volatile int* abort_flag = &ctrl->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t cta = ptx::cluster_ctarank();
  const int walker = (int)ptx::cluster_id_x(), walkers = (int)ptx::cluster_count_x();
  // plain: feature tiles of 2 x 128; gated: one pair tile per 128 gate features (p.n_tiles counts those)
  const int pair_tiles = kGated ? p.n_tiles : (p.n_tiles + 1) / 2;

  if (warp == 0) {
    build_tile_prefix<kPairTok>(p.rows_per_expert, p.num_experts, pair_tiles, ctrl->row_start, ctrl->tile_start);
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_w);
    }
  } else if (warp == 1) {
    ptx::tmem_alloc_pair(&ctrl->tmem_base, 512);
    ptx::tmem_relinquish_pair();
  } else if (warp == 2 && lane == 0) {
    for (int s = 0; s < kStagesP; ++s) {
      ptx::mbar_init(&ctrl->full[s], 1);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], 2 * kEpiWarps);   // the epilogue warps of both CTAs
    }
    if (kGated) {
      for (int w = 0; w < kEpiWarps; ++w)
        for (int b = 0; b < 2; ++b) {
          ptx::mbar_init(&xc->full[w][b], 1);
          ptx::mbar_init(&xc->empty[w][b], 1);
        }
    }
    ctrl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();   // both CTAs' barriers and tensor memory exist before either signals the other
  ptx::tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  const int total_tiles = ctrl->tile_start[p.num_experts];
  const int* tile_start = ctrl->tile_start;
  const int* row_start = ctrl->row_start;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = walker; t < total_tiles && ok; t += walkers) {
        TileInfo ti;
        locate_tile<kPairTok>(tile_start, row_start, t, cursor, ti, p.w_experts);
        // past N: the load is zero-filled
        const int n0 = kGated ? (cta == 0 ? 0 : (p.n >> 1)) + ti.n_tile * kFeat : (ti.n_tile * 2 + (int)cta) * kFeat;
        const int row = ti.row0 + (int)cta * 128;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* wdst = smem + s * kPairStageBytes;
          // the even CTA's barrier counts the bytes of both CTAs
          if (cta == 0) ptx::mbar_expect_tx(&ctrl->full[s], 2 * kPairStageBytes);
          const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&ctrl->full[s]), 0);
          const int k0 = kb * 64;
          if (!kWKn) {
            ptx::tma_load_3d_pair(wdst, &tmap_w, bar, k0, n0, ti.e);
          } else {
            ptx::tma_load_3d_pair(wdst, &tmap_w, bar, n0, k0, ti.e);
            ptx::tma_load_3d_pair(wdst + kWTileBytes / 2, &tmap_w, bar, n0 + 64, k0, ti.e);
          }
          ptx::tma_load_2d_pair(wdst + kWTileBytes, &tmap_a, bar, k0, row);
          if (++s == (uint32_t)kStagesP) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA) -----------------------
    if (cta == 0) {
      uint32_t s = 0, ph = 0, acc_it = 0;
      bool ok = true;
      const uint32_t smem_base = ptx::smem_u32(smem);
      constexpr uint32_t kWLbo = !kWKn ? 16u : 8192u;
      constexpr uint32_t kWStep = !kWKn ? 32u : 2048u;
      const uint32_t idesc = (p.idesc & ~((0x3fu << 17) | (0x1fu << 24))) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
      for (int t = walker; t < total_tiles && ok; t += walkers) {
        const uint32_t a = acc_it & 1;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_empty[a], ((acc_it >> 1) & 1) ^ 1, abort_flag))) break;
        ptx::tc_fence_after();
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->full[s], ph, abort_flag))) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t st_addr = smem_base + s * kPairStageBytes;
          const uint64_t wdesc0 = ptx::make_smem_desc(st_addr, kWLbo, 1024);
          const uint64_t adesc0 = ptx::make_smem_desc(st_addr + kWTileBytes, 16, 1024);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            ptx::umma_f16_pair_elect(tmem_base + a * kPairTok, wdesc0 + (uint64_t)((j * kWStep) >> 4),
                                     adesc0 + (uint64_t)((j * 32) >> 4), idesc, (kb > 0 || j > 0) ? 1u : 0u);
          ptx::umma_commit_pair_elect(&ctrl->empty[s]);
          if (++s == (uint32_t)kStagesP) { s = 0; ph ^= 1; }
        }
        if (ok) { ptx::umma_commit_pair_elect(&ctrl->acc_full[a]); ++acc_it; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    const uint32_t acc_empty0 = ptx::map_to_cta(ptx::smem_u32(&ctrl->acc_empty[0]), 0);
    uint32_t acc_it = 0;
    int cursor = 0;
    // gated: this warp's exchange buffers in the even CTA, the barriers on both sides, and how
    // many chunks have gone through them
    const int ew = warp - 2;
    const uint32_t xbuf0 = ptx::map_to_cta(ptx::smem_u32(xbuf + ew * 2 * kPairXBuf), 0);
    const uint32_t xfull0 = ptx::map_to_cta(ptx::smem_u32(&xc->full[ew][0]), 0);
    const uint32_t xempty1 = ptx::map_to_cta(ptx::smem_u32(&xc->empty[ew][0]), 1);
    uint32_t xit = 0;
    bool ok = true;
    for (int t = walker; t < total_tiles && ok; t += walkers) {
      TileInfo ti;
      locate_tile<kPairTok>(tile_start, row_start, t, cursor, ti, p.w_experts);
      const int n_tile = kGated ? ti.n_tile : ti.n_tile * 2 + (int)cta;
      // the feature (row of W and of the bias) this thread's accumulator lane belongs to
      const int feat = (kGated && cta == 1 ? (p.n >> 1) : 0) + n_tile * kFeat + q * 32 + lane;
      const float bias_v = (p.bias != nullptr && feat < p.n) ? load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + feat) : 0.f;
      const uint32_t a = acc_it & 1;
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_full[a], (acc_it >> 1) & 1, abort_flag))) {
        *abort_flag = 1; break;
      }
      ptx::tc_fence_after();
#pragma unroll(kGated ? 1 : kPairTok / kChunk)
      for (int c0 = 0; c0 < kPairTok; c0 += kChunk) {
        if (c0 < ti.valid) {
          uint32_t v[kChunk];
          ptx::tmem_ld_32x32(tmem_base + a * kPairTok + c0 + lane_sel, v);
          ptx::tmem_wait_ld();
          float vals[kChunk];
#pragma unroll
          for (int i = 0; i < kChunk; ++i) vals[i] = __uint_as_float(v[i]) + bias_v;
          if (kGated) {
            const uint32_t b = xit & 1, par = (xit >> 1) & 1;
            if (cta == 1) {
              // up: wait until the even CTA has read this buffer's previous chunk, then send
              if (!__all_sync(0xffffffffu, ptx::mbar_wait_cluster(&xc->empty[ew][b], par ^ 1, abort_flag))) {
                *abort_flag = 1; ok = false; break;
              }
              if (p.clamp > 0.f) {
#pragma unroll
                for (int i = 0; i < kChunk; ++i) vals[i] = fminf(fmaxf(vals[i], -p.clamp), p.clamp);
              }
              const uint32_t dst = xbuf0 + b * kPairXBuf + lane * 16;     // [token quad][lane] 16-byte cells
#pragma unroll
              for (int i = 0; i < kChunk; i += 4)
                ptx::st_cluster_v4(dst + (i >> 2) * 512, vals[i], vals[i + 1], vals[i + 2], vals[i + 3]);
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive_cluster_release(xfull0 + b * 8);
            } else {
              // gate: take the up chunk of the same features and tokens, activate, store
              if (!__all_sync(0xffffffffu, ptx::mbar_wait_cluster(&xc->full[ew][b], par, abort_flag))) {
                *abort_flag = 1; ok = false; break;
              }
              const uint32_t src = ptx::smem_u32(xbuf + ew * 2 * kPairXBuf) + b * kPairXBuf + lane * 16;
#pragma unroll
              for (int i = 0; i < kChunk; i += 4) {
                const float4 u4 = ptx::lds128f(src + (i >> 2) * 512);
                const float uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  float g = vals[i + k];
                  if (p.clamp > 0.f) g = fminf(g, p.clamp);
                  vals[i + k] = g * __fdividef(1.0f, 1.0f + __expf(-g)) * uu[k];
                }
              }
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive_cluster_release(xempty1 + b * 8);
              store_block_transposed<kChunk, 32>(ctrl->xpose[warp - 2], vals, p.d, p.out_f16,
                                                 (int64_t)ti.row0 + c0, ti.valid - c0, p.m, p.n >> 1,
                                                 n_tile * kFeat + q * 32, lane);
            }
            ++xit;
          } else if (p.swiglu) {
            const float c_lim = p.clamp > 0.f ? p.clamp : INFINITY;
#pragma unroll
            for (int i = 0; i < kChunk; ++i) {
              const float x = vals[i];
              const float other = __shfl_xor_sync(0xffffffffu, x, 1);
              float gate = (lane & 1) ? other : x;
              float up = (lane & 1) ? x : other;
              gate = fminf(fminf(gate, c_lim), p.limit);
              up = fminf(fmaxf(up, -c_lim), c_lim);
              up = fminf(fmaxf(up, -p.limit), p.limit);
              vals[i] = (up + 1.0f) * gate * __fdividef(1.0f, 1.0f + __expf(-gate * p.alpha));
            }
            store_block_transposed<kChunk, 16>(ctrl->xpose[warp - 2], vals, p.d, p.out_f16,
                                               (int64_t)ti.row0 + c0, ti.valid - c0, p.m, p.n >> 1,
                                               (n_tile * kFeat + q * 32) >> 1, lane);
          } else {
            store_block_transposed<kChunk, 32>(ctrl->xpose[warp - 2], vals, p.d, p.out_f16,
                                               (int64_t)ti.row0 + c0, ti.valid - c0, p.m, p.n,
                                               n_tile * kFeat + q * 32, lane);
          }
        }
      }
      if (!ok) break;
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(acc_empty0 + a * 8);
      ++acc_it;
    }
  }

  // Teardown: neither CTA frees tensor memory or leaves while the other may still use its
  // shared memory, its barriers or MMAs in flight (every thread of both CTAs gets here after
  // bounded waits).
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after();
    if (*abort_flag != 0) __nanosleep(20000);
    ptx::tmem_dealloc_pair(tmem_base, 512);
  }
  if (tid == 0 && *abort_flag != 0) report_timeout(p.status);
}

// Clusters of two CTAs, as many as the device runs at once (at most `max_pairs`).
template <bool kWKn, bool kGated>
int launch_tc_pair(const CUtensorMap& ta, const CUtensorMap& tw, const TcParams& p, int max_pairs, cudaStream_t st) {
  auto kern = grouped_gemm_tc_pair_kernel<kWKn, kGated>;
  constexpr size_t kSmem = kGated ? kPairGatedSmem : kPairSmem;
  static SmemConfig configured;
  if (int rc = configured.ensure(kern, kSmem)) return rc;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kTcThreads); cfg.dynamicSmemBytes = kSmem; cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = 1;
  static std::atomic<int> resident[kMaxDevices];
  const int dev = current_device();
  int pairs = resident[dev].load(std::memory_order_relaxed);
  if (pairs == 0) {
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    if (cudaOccupancyMaxActiveClusters(&pairs, kern, &cfg) != cudaSuccess || pairs < 1) {
      (void)cudaGetLastError();
      pairs = -1;   // this device (a partition with too few SMs per GPC, say) runs no such cluster
    }
    resident[dev].store(pairs, std::memory_order_relaxed);
  }
  if (pairs < 0) return B200MOE_E_UNSUPPORTED;   // the caller takes the single-CTA kernel
  if (pairs > max_pairs) pairs = max_pairs;
  cfg.gridDim = dim3(2 * pairs);
  B200_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ta, tw, p));
  return B200MOE_OK;
}

}  // namespace

// Returns B200MOE_E_UNSUPPORTED (without a launch) for requests the
// tensor-core kernel does not cover; the caller decides what to do then.
int grouped_gemm_tc(const b200moe_gemm_args* a, cudaStream_t st) {
  const bool a_fp8 = a->a_dtype == B200MOE_FP8_E4M3;
  const bool w16 = a->w_format == B200MOE_W_BF16_KN || a->w_format == B200MOE_W_BF16_NK;
  const bool w8b = a->w_format == B200MOE_W_FP8_BLOCK_NK || a->w_format == B200MOE_W_FP8_BLOCK_KN;
  const bool gated = a->epilogue == B200MOE_EPI_SILU_MUL;
  const bool swiglu = a->epilogue == B200MOE_EPI_SWIGLUOAI;
  if (a->epilogue != B200MOE_EPI_NONE && !((gated || swiglu) && w16 && !a_fp8 && (a->n / 2) % 16 == 0))
    return fail(B200MOE_E_UNSUPPORTED, "tensor-core grouped GEMM: fused gated activations only on 16-bit weights");
  if (!((w16 && !a_fp8) || (w8b && a_fp8)))
    return fail(B200MOE_E_UNSUPPORTED,
                "tensor-core grouped GEMM takes 16-bit x 16-bit or fp8 x block-scaled fp8");
  if (a->num_experts > kMaxExperts)
    return fail(B200MOE_E_UNSUPPORTED, "tensor-core grouped GEMM: more than %d experts", kMaxExperts);
  const bool kn = a->w_format == B200MOE_W_BF16_KN || a->w_format == B200MOE_W_FP8_BLOCK_KN;
  const int es = a_fp8 ? 1 : 2;
  if (((int64_t)a->k * es) % 16 != 0 || ((int64_t)a->n * es) % 16 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "tensor-core grouped GEMM: row pitch must be a multiple of 16 bytes");
  if (((uintptr_t)a->a & 15) || ((uintptr_t)a->w & 15) || ((uintptr_t)a->d & 15))
    return fail(B200MOE_E_BADARG, "grouped GEMM: A, W and D must be 16-byte aligned");
  if (a->m == 0 || a->n == 0) return B200MOE_OK;

  const int kpb = a_fp8 ? 128 : 64;
  TcParams p;
  p.a_scale = reinterpret_cast<const float*>(a->a_scale); p.w_scale = reinterpret_cast<const float*>(a->w_scale);
  p.bias = a->bias; p.d = a->d; p.rows_per_expert = a->rows_per_expert; p.status = a->status;
  p.m = a->m; p.n = a->n; p.k = a->k; p.num_experts = a->num_experts;
  const int w_sets = (a->w_experts > 0 && a->w_experts != a->num_experts) ? a->w_experts : a->num_experts;
  p.w_experts = w_sets != a->num_experts ? w_sets : 0;
  p.n_tiles = ((gated ? a->n / 2 : a->n) + kFeat - 1) / kFeat;
  p.clamp = a->clamp_limit;
  p.swiglu = swiglu ? 1 : 0; p.alpha = a->act_alpha; p.limit = a->act_limit;
  p.num_kb = (a->k + kpb - 1) / kpb;
  p.out_f16 = a->d_dtype == B200MOE_F16;

  const int64_t rows_in_use = (a->rows_hint > 0 && a->rows_hint < a->m) ? a->rows_hint : a->m;
  const int64_t avg = (rows_in_use + a->num_experts - 1) / a->num_experts;
  // Token-tile width from the mean rows per expert (routing is never perfectly
  // even, so leave headroom before a second token tile re-reads the weights).
  int bt;
  if (a_fp8) {
    // fp8 pays a hand-over per 128-wide K block, so wider tiles win earlier (measured on the
    // DeepSeek and Qwen3 shapes: 8 rows per expert 0.72 / 0.88 / 0.84 of the copy rate at
    // 16 / 64 / 128 tokens, 32 rows 0.32 / 0.69 / 0.82)
    bt = avg <= 4 ? 16 : (avg < 12 ? 64 : 128);
  } else if (avg <= 8) bt = 16;
  else if (avg <= 40) bt = 64;
  else if (avg <= 96) bt = 128;   // measured on skewed routing: 128 rows per expert are 13 % faster at 256
  else bt = 256;
  // two accumulators per stage: tensor memory holds the gated form up to 128-token tiles; beyond,
  // a CTA pair splits gate and up between its two CTAs (whole 128-feature tiles only)
  // (whole 128-feature tiles only).  The pair's epilogue passes the up half through the other
  // CTA's shared memory chunk by chunk, which a tile's MMAs hide from K = 4096 on; with 256-token
  // tiles it also wants segments that fill them.  Measured, gemm1 of the Mixtral shape: 1024 rows
  // per expert 1.33 ms against 1.59 (single-CTA gated tile) and 1.42 (plain pair + silu_and_mul),
  // 128 rows per expert 0.39 against 0.31; N=2816, K=2048, 1024 rows: 0.120 against 0.096.
  // (impl 4 forces the pair form, impl 3 the single-CTA forms.)
  const bool gated_pair = gated && !a_fp8 && a->impl != 3 && (a->n / 2) % kFeat == 0 &&
                          (a->impl == 4 || (avg > 192 && a->k >= 4096));
  if (gated_pair || (a->impl == 4 && !a_fp8 && !gated)) bt = 256;
  else if (gated && bt > 128) bt = 128;

  // prefill-sized fp8 segments: the token-major kernels (one scale register per thread and K block)
  if (a_fp8 && bt >= 128) return grouped_gemm_tc_fp8t(a, st);

  const uint32_t fmt = a_fp8 ? 0u : (a->a_dtype == B200MOE_BF16 ? 1u : 0u);
  p.idesc = ptx::make_idesc(fmt, fmt, kn ? 1u : 0u, 0u, kFeat, (uint32_t)bt);

  const CUtensorMapDataType dt = a_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                       : (a->a_dtype == B200MOE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUtensorMap ta, tw;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a->k, (cuuint64_t)a->m};
    cuuint64_t strides[1] = {(cuuint64_t)a->k * es};
    cuuint32_t box[2] = {(cuuint32_t)kpb, (cuuint32_t)bt};
    int rc = encode_map(&ta, dt, 2, a->a, dims, strides, box);
    if (rc) return rc;
  }
  if (!kn) {
    cuuint64_t dims[3] = {(cuuint64_t)a->k, (cuuint64_t)a->n, (cuuint64_t)w_sets};
    cuuint64_t strides[2] = {(cuuint64_t)a->k * es, (cuuint64_t)a->k * a->n * es};
    cuuint32_t box[3] = {(cuuint32_t)kpb, (cuuint32_t)kFeat, 1};
    int rc = encode_map(&tw, dt, 3, a->w, dims, strides, box);
    if (rc) return rc;
  } else {
    cuuint64_t dims[3] = {(cuuint64_t)a->n, (cuuint64_t)a->k, (cuuint64_t)w_sets};
    cuuint64_t strides[2] = {(cuuint64_t)a->n * es, (cuuint64_t)a->k * a->n * es};
    cuuint32_t box[3] = {(cuuint32_t)(a_fp8 ? 128 : 64), (cuuint32_t)kpb, 1};
    int rc = encode_map(&tw, dt, 3, a->w, dims, strides, box);
    if (rc) return rc;
  }

  const int64_t tile_bound = ((a->m + bt - 1) / bt + a->num_experts) * (int64_t)p.n_tiles;
  int grid = sm_count();
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;

  // 16-bit prefill: the CTA-pair kernel (impl 3 / 4 force the single-CTA / the pair form)
  if (!a_fp8 && bt == 256 && a->impl != 3 && (gated ? gated_pair : p.n_tiles >= 2)) {
    CUtensorMap ta_half;
    cuuint64_t dims[2] = {(cuuint64_t)a->k, (cuuint64_t)a->m};
    cuuint64_t strides[1] = {(cuuint64_t)a->k * es};
    cuuint32_t box[2] = {(cuuint32_t)kpb, 128};
    if (int rc = encode_map(&ta_half, dt, 2, a->a, dims, strides, box)) return rc;
    const int64_t pair_bound = ((a->m + 255) / 256 + a->num_experts) * (int64_t)(gated ? p.n_tiles : (p.n_tiles + 1) / 2);
    int max_pairs = grid / 2 < 1 ? 1 : grid / 2;
    if (pair_bound < max_pairs) max_pairs = (int)pair_bound;
    const int rc = gated ? (kn ? launch_tc_pair<true, true>(ta_half, tw, p, max_pairs, st)
                               : launch_tc_pair<false, true>(ta_half, tw, p, max_pairs, st))
                         : (kn ? launch_tc_pair<true, false>(ta_half, tw, p, max_pairs, st)
                               : launch_tc_pair<false, false>(ta_half, tw, p, max_pairs, st));
    if (rc != B200MOE_E_UNSUPPORTED) return rc;
    if (gated) bt = 128;   // no clusters on this device: the single-CTA gated tile
  }

  if (tile_bound < grid) grid = (int)tile_bound;
  if (grid < 1) grid = 1;

#define B200_TC_CASE(BT_)                                                         \
  if (bt == BT_) {                                                                \
    if (a_fp8) {                                                                  \
      if (kn) return launch_tc<(BT_ > 64 ? 64 : BT_), true, true>(ta, tw, p, grid, st);  \
      return launch_tc<(BT_ > 64 ? 64 : BT_), true, false>(ta, tw, p, grid, st);         \
    }                                                                             \
    if (kn) return launch_tc<BT_, false, true>(ta, tw, p, grid, st);              \
    return launch_tc<BT_, false, false>(ta, tw, p, grid, st);                     \
  }
  if (gated) {
#define B200_TC_GATED(BT_)                                                          \
    if (bt == BT_) {                                                                \
      if (kn) return launch_tc<BT_, false, true, true>(ta, tw, p, grid, st);        \
      return launch_tc<BT_, false, false, true>(ta, tw, p, grid, st);               \
    }
    B200_TC_GATED(16)
    B200_TC_GATED(64)
    B200_TC_GATED(128)
#undef B200_TC_GATED
  }
  B200_TC_CASE(16)
  B200_TC_CASE(64)
  B200_TC_CASE(128)
  B200_TC_CASE(256)
#undef B200_TC_CASE
  return fail(B200MOE_E_UNSUPPORTED, "tensor-core grouped GEMM: no tile for %d", bt);
}

}  // namespace b200moe
