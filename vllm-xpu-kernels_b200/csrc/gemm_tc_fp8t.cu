// fp8 x block-scaled fp8 grouped GEMM for prefill-sized expert segments, tokens on the
// 128-row M side of tcgen05.mma and the weight's output features on its N side.
//
//   D[r0:r0+rows_e, :] = sum_kb a_scale[row, kb] * w_scale[e, n/128, kb] * (A_kb * W_e,kb^T)
//
// The block-scaled recipe (csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:361-383
// of vllm-xpu-kernels: e4m3 activations with one fp32 scale per 1x128 group, e4m3 weights with
// one per 128x128 block) needs every 128-wide K block's partial sum multiplied by its own
// scale before it is added up.  With tokens on the tensor-memory lanes an epilogue thread
// owns one token row, and the 128 features of the tile share one weight block: the scale of
// a K block is a single register per thread.  The promotion then is one fused
// multiply-add per accumulator, and the finished row goes to global memory as
// consecutive 16-byte stores.  (The feature-major kernel of gemm_tc.cu, which serves the
// smaller token tiles, has a different scale in every accumulator column and has to stage
// them through shared memory.)
//
// Two kernels: 128 x 128 tiles (below, used when N is a single 128-feature block) and
// 128 x 256 tiles (further down, the one prefill shapes run).
//
// Roles of the 128 x 128 kernel (320 threads, one persistent CTA per SM):
//   warp 0    : TMA producer, ring of 6 stages of [weights 128x128 B | tokens 128x128 B]
//   warp 1    : MMA issuer (one lane), kind::f8f6f4, one accumulator stage (128 columns of
//               tensor memory, four stages) per K block
//   warps 2-9 : promotion + epilogue; warp w reads lane quarter w & 3, columns
//               64 * ((w - 2) / 4) .. + 63: 64 accumulators per thread
// Every mbarrier wait is bounded; on expiry the CTA raises its abort flag, all roles leave
// their loops, tensor memory is freed and *status is set to 1.
#include "common.cuh"
#include "gemm_tc_common.cuh"
#include "sm100_ptx.cuh"


namespace b200moe {
namespace {

constexpr int kTTok = 128;            // tokens per tile (UMMA M)
constexpr int kTStages = 6;
constexpr int kTStageBytes = 32768;   // weights 16 KB, tokens 16 KB
constexpr int kTAcc = 4;              // accumulator stages
constexpr int kTThreads = 320;
constexpr int kTCols = 64;            // accumulator columns per epilogue thread
constexpr int kTGroup = 4;            // K blocks per scale prefetch group

struct TParams {
  const float* a_scale;   // [M, K/128]
  const float* w_scale;   // [E, N/128, K/128]
  const void* bias;
  void* d;
  const int32_t* rows_per_expert;
  int32_t* status;
  int64_t m;
  int n, k, num_experts;
  int w_experts;          // >0: segment s uses weight set s % w_experts
  int n_tiles, num_kb;
  uint32_t idesc;
  int out_f16;
  // gated epilogue of the 128 x 256 kernel (kGated): D is [M, n/2] e4m3 with one fp32 scale per
  // token and 128 features in d_scale [M, n/256]
  float* d_scale;
  float clamp;            // >0: gate = min(gate, clamp), up = clamp(up, -clamp, clamp)
  // 128 x 256 kernel: 4 stages and rows stored straight from the registers (few rows per expert:
  // HBM-bound, bytes in flight matter, few rows to store), or 3 stages and the rows transposed
  // through shared memory into whole 256-byte segments (many rows per expert: the store of a
  // tile, which the promotion warps cannot overlap with anything, is 4 us as scattered 16-byte
  // pieces and under 1 us as rows)
  int stages;
};

struct TCtrl {
  uint64_t full[kTStages];
  uint64_t empty[kTStages];
  uint64_t acc_full[kTAcc];
  uint64_t acc_empty[kTAcc];
  uint32_t tmem_base;
  int abort_flag;
  int tile_start[kMaxExperts + 1];
  int row_start[kMaxExperts + 1];
};

constexpr size_t kTSmem = 1024 + (size_t)kTStages * kTStageBytes + sizeof(TCtrl);

template <bool kWKn>
__global__ void __launch_bounds__(kTThreads, 1)
grouped_gemm_fp8t_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_w, const TParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  TCtrl* ctrl = reinterpret_cast<TCtrl*>(smem + kTStages * kTStageBytes);
  volatile int* abort_flag = &ctrl->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {
    build_tile_prefix<kTTok>(p.rows_per_expert, p.num_experts, p.n_tiles, ctrl->row_start, ctrl->tile_start);
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_w);
    }
  } else if (warp == 1) {
    ptx::tmem_alloc(&ctrl->tmem_base, 512);
    ptx::tmem_relinquish();
  } else if (warp == 2 && lane == 0) {
    for (int s = 0; s < kTStages; ++s) {
      ptx::mbar_init(&ctrl->full[s], 1);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < kTAcc; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], 8);
    }
    ctrl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  const int* tile_start = ctrl->tile_start;
  const int* row_start = ctrl->row_start;
  const int total_tiles = tile_start[p.num_experts];

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<kTTok>(tile_start, row_start, t, cursor, ti, p.w_experts);
        const int n0 = ti.n_tile * kFeat;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* wdst = smem + s * kTStageBytes;
          ptx::mbar_expect_tx(&ctrl->full[s], kTStageBytes);
          if (!kWKn) ptx::tma_load_3d(wdst, &tmap_w, &ctrl->full[s], kb * 128, n0, ti.e);
          else ptx::tma_load_3d(wdst, &tmap_w, &ctrl->full[s], n0, kb * 128, ti.e);
          ptx::tma_load_2d(wdst + 16384, &tmap_a, &ctrl->full[s], kb * 128, ti.row0);
          if (++s == (uint32_t)kTStages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // (the whole warp runs the loop with the same values; one elected lane issues)
    {
      uint32_t s = 0, ph = 0, a = 0, aph = 0;
      bool ok = true;
      const uint32_t smem_base = ptx::smem_u32(smem);
      // weights: K-major rows of 128 bytes, or (kWKn) the [K, N] tile read as an MN-major operand
      constexpr uint32_t kWLbo = !kWKn ? 16u : 16384u;
      constexpr uint32_t kWStep = !kWKn ? 32u : 4096u;   // bytes per 32-wide K step
      int my_tiles = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) ++my_tiles;
      const int64_t blocks = (int64_t)my_tiles * p.num_kb;   // every tile: same K loop, no tile state needed
      for (int64_t i = 0; i < blocks && ok; ++i) {
        bool go = ptx::mbar_wait(&ctrl->acc_empty[a], aph ^ 1, abort_flag);
        if (go) go = ptx::mbar_wait(&ctrl->full[s], ph, abort_flag);
        if (!__all_sync(0xffffffffu, go)) break;
        ptx::tc_fence_after();
        const uint32_t st_addr = smem_base + s * kTStageBytes;
        const uint64_t wdesc0 = ptx::make_smem_desc(st_addr, kWLbo, 1024);
        const uint64_t adesc0 = ptx::make_smem_desc(st_addr + 16384, 16, 1024);
        const uint32_t d_tmem = tmem_base + a * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ptx::umma_elect<true>(d_tmem, adesc0 + (uint64_t)((j * 32) >> 4), wdesc0 + (uint64_t)((j * kWStep) >> 4),
                                p.idesc, j > 0 ? 1u : 0u);
        ptx::umma_commit_elect(&ctrl->empty[s]);
        ptx::umma_commit_elect(&ctrl->acc_full[a]);
        if (++s == (uint32_t)kTStages) { s = 0; ph ^= 1; }
        if (++a == (uint32_t)kTAcc) { a = 0; aph ^= 1; }
      }
    }
  } else {
    // ------------------------ promotion and epilogue --------------------------
    const int q = warp & 3;
    const int r = q * 32 + lane;                       // token row inside the tile
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    const int col0 = ((warp - 2) >> 2) * kTCols;       // first feature column of this warp
    const int kbs = p.num_kb;
    const bool vec4_ok = (kbs % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.a_scale) & 15) == 0);
    struct ScaleRegs { float a[kTGroup]; float w[kTGroup]; };
    ScaleRegs cur, pre;
    bool pre_valid = false;
    auto fetch_group = [&](const TileInfo& tt, int g, ScaleRegs& sr) {
      const int kb0 = g * kTGroup;
      const int64_t wsb = ((int64_t)tt.e * p.n_tiles + tt.n_tile) * kbs + kb0;
#pragma unroll
      for (int jb = 0; jb < kTGroup; ++jb) sr.w[jb] = (kb0 + jb < kbs) ? p.w_scale[wsb + jb] : 0.f;
      const bool live = r < tt.valid;
      const float* src = p.a_scale + (int64_t)(tt.row0 + r) * kbs + kb0;
      if (live && vec4_ok) {
        const float4 q4 = *reinterpret_cast<const float4*>(src);
        sr.a[0] = q4.x; sr.a[1] = q4.y; sr.a[2] = q4.z; sr.a[3] = q4.w;
      } else {
#pragma unroll
        for (int jb = 0; jb < kTGroup; ++jb) sr.a[jb] = (live && kb0 + jb < kbs) ? src[jb] : 0.f;
      }
    };
    uint32_t a = 0, aph = 0;
    int cursor = 0;
    bool ok = true;
    const int n_groups = (p.num_kb + kTGroup - 1) / kTGroup;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      TileInfo ti;
      locate_tile<kTTok>(tile_start, row_start, t, cursor, ti, p.w_experts);
      float acc[kTCols];
#pragma unroll
      for (int i = 0; i < kTCols; ++i) acc[i] = 0.f;
      uint32_t va[32], vb[32];
      // scales are read one group of K blocks ahead of their use (the next tile's first group
      // during this tile's last)
      if (!pre_valid) fetch_group(ti, 0, cur);
      else cur = pre;
      pre_valid = false;
      for (int g = 0; g < n_groups && ok; ++g) {
        if (g + 1 < n_groups) {
          fetch_group(ti, g + 1, pre);
        } else if (t + (int)gridDim.x < total_tiles) {
          int cursor2 = cursor;
          TileInfo tn;
          locate_tile<kTTok>(tile_start, row_start, t + gridDim.x, cursor2, tn, p.w_experts);
          fetch_group(tn, 0, pre);
          pre_valid = true;
        }
#pragma unroll
        for (int jb = 0; jb < kTGroup; ++jb) {
          if (g * kTGroup + jb >= p.num_kb) break;
          const float sc = cur.a[jb] * cur.w[jb];
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_full[a], aph, abort_flag))) {
            *abort_flag = 1; ok = false; break;
          }
          ptx::tc_fence_after();
          // both halves in flight together, one wait: tcgen05.wait::ld covers every load before it
          ptx::tmem_ld_32x32(tmem_base + a * 128 + col0 + lane_sel, va);
          ptx::tmem_ld_32x32(tmem_base + a * 128 + col0 + 32 + lane_sel, vb);
          ptx::tmem_wait_ld_tied(va, vb);
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[a]);   // the stage is in registers
          if (++a == (uint32_t)kTAcc) { a = 0; aph ^= 1; }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            acc[i] = fmaf(__uint_as_float(va[i]), sc, acc[i]);
            acc[32 + i] = fmaf(__uint_as_float(vb[i]), sc, acc[32 + i]);
          }
        }
        if (g + 1 < n_groups) cur = pre;
      }
      if (ok && r < ti.valid) {
        const int f0 = ti.n_tile * kFeat + col0;
        uint16_t* drow = reinterpret_cast<uint16_t*>(p.d) + (int64_t)(ti.row0 + r) * p.n + f0;
#pragma unroll
        for (int c = 0; c < kTCols; c += 8) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            float x0 = acc[c + i], x1 = acc[c + i + 1];
            if (p.bias != nullptr) {
              x0 += load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + f0 + c + i);
              x1 += load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + f0 + c + i + 1);
            }
            if (p.out_f16) {
              const __half2 h = __floats2half2_rn(x0, x1);
              w[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
              const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
              w[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
          *reinterpret_cast<uint4*>(drow + c) = make_uint4(w[0], w[1], w[2], w[3]);
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
    ptx::tmem_dealloc(tmem_base, 512);
  }
  if (tid == 0 && *abort_flag != 0) report_timeout(p.status);
}

// ---------------------------------------------------------------------------------
// Wide variant: 128 tokens x 256 features per tile, so that every tcgen05.mma carries
// twice the work (the issuing thread, not the tensor pipe, bounds the 128-feature tile).
// A thread then owns 128 accumulators, more than the even register split of 384 threads
// allows: the warps are laid out in warpgroups and re-balance registers with setmaxnreg
//   warps 0-3  : producer (warp 0), MMA issuer (warp 1), two idle warps; 40 registers
//   warps 4-11 : promotion + epilogue, 232 registers; warp w reads lane quarter w & 3 and
//                the 128 columns of feature block (w - 4) / 4, in two passes of 64
// Tensor memory holds two accumulator stages of 256 columns.
constexpr int kT2Threads = 384;
// setmaxnreg.inc waits - without any limit - until the CTA's register pool holds what it asks
// for, so the re-balanced total must fit what the CTA got at launch (threads x launch registers)
constexpr int kT2LaunchRegs = 168, kT2LowRegs = 40, kT2HighRegs = 232;
static_assert(128 * kT2LowRegs + 256 * kT2HighRegs <= kT2Threads * kT2LaunchRegs, "setmaxnreg budget");
constexpr int kT2Stages = 4;          // ring of up to 4 stages (192 KB in flight per SM) ...
constexpr int kT2StagesStaged = 3;    // ... or 3 with the fourth stage's room given to the store tiles
constexpr int kT2RowPitch = 272;      // bytes per staged output row: 128 16-bit values + 16 (conflict-free 16-byte accesses)
constexpr int kT2StageBytes = 49152;   // weights 2 x 16 KB, tokens 16 KB
constexpr int kT2Acc = 2;

struct T2Ctrl {
  uint64_t full[kT2Stages];
  uint64_t empty[kT2Stages];
  uint64_t acc_full[kT2Acc];
  uint64_t acc_empty[kT2Acc];
  uint32_t tmem_base;
  int abort_flag;
  float xchg[2][2][128];   // gated epilogue: group maxima exchanged between the two warps of a token row
  uint64_t xbar[4];        // ... and the barrier of each such pair of warps (one per lane quarter)
  int tile_start[kMaxExperts + 1];
  int row_start[kMaxExperts + 1];
};
// store tiles (3-stage form): per epilogue warp its 32 token rows x 128 features in 16 bits
constexpr size_t kT2XposeBytes = 8 * 32 * kT2RowPitch;
constexpr size_t kT2Ring = (size_t)kT2Stages * kT2StageBytes;      // the ring's room either way
constexpr size_t kT2Smem = 1024 + kT2Ring + ((sizeof(T2Ctrl) + 15) & ~(size_t)15);
static_assert(kT2XposeBytes <= kT2StageBytes + 24 * 1024, "store tiles must fit the fourth stage's room");
constexpr size_t kT2SmemStaged = 1024 + (size_t)kT2StagesStaged * kT2StageBytes + kT2XposeBytes +
                                 ((sizeof(T2Ctrl) + 15) & ~(size_t)15);

//
// kGated (the first grouped GEMM of a SiLU layer with block-scaled fp8 experts): a tile pairs the
// 128 gate features j0.. with the 128 up features n/2 + j0.. of the same tokens; warp w reads
// lane quarter w & 3 and, of both blocks, the 64 columns of half (w - 4) / 4, so a thread holds
// gate and up of the same 64 features of its token.  The epilogue rounds both to the 16-bit
// type an unfused GEMM would have stored, applies silu(gate) * up, finds the maximum of the
// token's 128-feature group together with the partner warp (shared memory, a named barrier of
// the two warps) and stores e4m3 codes and the group's fp32 scale: the arithmetic of
// silu_and_mul_per_block_quant on the unfused output, value for value, without the [M, n]
// round trip through HBM.
template <bool kWKn, bool kGated>
__global__ void __launch_bounds__(kT2Threads, 1)
grouped_gemm_fp8t256_kernel(const __grid_constant__ CUtensorMap tmap_a,
                            const __grid_constant__ CUtensorMap tmap_w, const TParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t stages = (uint32_t)p.stages;
  uint8_t* xpose_base = smem + stages * kT2StageBytes;     // used by the 3-stage form only
  T2Ctrl* ctrl = reinterpret_cast<T2Ctrl*>(xpose_base + (stages == (uint32_t)kT2Stages ? 0 : kT2XposeBytes));
  volatile int* abort_flag = &ctrl->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // 256-feature tiles; gated: one tile per 128 gate features (p.n_tiles counts 128-feature blocks of n)
  const int n_tiles2 = kGated ? p.n_tiles / 2 : (p.n_tiles + 1) / 2;
  const int up_block0 = p.n_tiles / 2;        // gated: first 128-feature block of the up half

  if (warp == 0) {
    build_tile_prefix<kTTok>(p.rows_per_expert, p.num_experts, n_tiles2, ctrl->row_start, ctrl->tile_start);
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_w);
    }
  } else if (warp == 1) {
    ptx::tmem_alloc(&ctrl->tmem_base, 512);
    ptx::tmem_relinquish();
  } else if (warp == 2 && lane == 0) {
    for (int s = 0; s < kT2Stages; ++s) {
      ptx::mbar_init(&ctrl->full[s], 1);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < kT2Acc; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], 8);
    }
    for (int x = 0; x < 4; ++x) ptx::mbar_init(&ctrl->xbar[x], 2);
    ctrl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  const int* tile_start = ctrl->tile_start;
  const int* row_start = ctrl->row_start;
  const int total_tiles = tile_start[p.num_experts];

  if (warp < 4) {
    ptx::setmaxnreg_dec<kT2LowRegs>();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------------
      uint32_t s = 0, ph = 0;
      int cursor = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<kTTok>(tile_start, row_start, t, cursor, ti, p.w_experts);
        const int n0 = kGated ? ti.n_tile * 128 : ti.n_tile * 256;
        const int n1 = kGated ? (up_block0 + ti.n_tile) * 128 : n0 + 128;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag, true)) { ok = false; break; }
          uint8_t* wdst = smem + s * kT2StageBytes;
          ptx::mbar_expect_tx(&ctrl->full[s], kT2StageBytes);
          // two 128-feature blocks (the second one is zero-filled past N)
          if (!kWKn) {
            ptx::tma_load_3d(wdst, &tmap_w, &ctrl->full[s], kb * 128, n0, ti.e);
            ptx::tma_load_3d(wdst + 16384, &tmap_w, &ctrl->full[s], kb * 128, n1, ti.e);
          } else {
            ptx::tma_load_3d(wdst, &tmap_w, &ctrl->full[s], n0, kb * 128, ti.e);
            ptx::tma_load_3d(wdst + 16384, &tmap_w, &ctrl->full[s], n1, kb * 128, ti.e);
          }
          ptx::tma_load_2d(wdst + 32768, &tmap_a, &ctrl->full[s], kb * 128, ti.row0);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer --------------------------------
      // (the whole warp runs the loop with the same values; one elected lane issues)
      uint32_t s = 0, ph = 0, a = 0, aph = 0;
      const uint32_t smem_base = ptx::smem_u32(smem);
      constexpr uint32_t kWLbo = !kWKn ? 16u : 16384u;
      constexpr uint32_t kWStep = !kWKn ? 32u : 4096u;
      int my_tiles = 0;
      for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) ++my_tiles;
      const int64_t blocks = (int64_t)my_tiles * p.num_kb;
      const uint32_t idesc = (p.idesc & ~(0x3fu << 17)) | ((256u >> 3) << 17);
      auto mma = [&](uint32_t d, uint64_t ad, uint64_t wd, uint32_t accumulate) {
        ptx::umma_elect<true>(d, ad, wd, idesc, accumulate);
      };
      // The barriers of the next block are polled between this block's MMA issues, where
      // the thread would otherwise only wait for room in the tensor pipe's queue.
      bool full_ready = false, acc_ready = false;
      for (int64_t i = 0; i < blocks; ++i) {
        // (spinning waits here and in the promotion warps: the hand-over of an accumulator stage
        // is the kernel's critical loop, and a suspended try_wait wakes up late)
        bool go = true;
        if (!acc_ready) go = ptx::mbar_wait(&ctrl->acc_empty[a], aph ^ 1, abort_flag, true);
        if (go && !full_ready) go = ptx::mbar_wait(&ctrl->full[s], ph, abort_flag, true);
        if (!__all_sync(0xffffffffu, go)) break;
        ptx::tc_fence_after();
        const uint32_t st_addr = smem_base + s * kT2StageBytes;
        const uint64_t wdesc0 = ptx::make_smem_desc(st_addr, kWLbo, 1024);
        const uint64_t adesc0 = ptx::make_smem_desc(st_addr + 32768, 16, 1024);
        const uint32_t d_tmem = tmem_base + a * 256;
        const uint32_t s1 = (s + 1 == stages) ? 0u : s + 1, ph1 = (s1 == 0u) ? ph ^ 1u : ph;
        const uint32_t a1 = (a + 1 == (uint32_t)kT2Acc) ? 0u : a + 1, aph1 = (a1 == 0u) ? aph ^ 1u : aph;
        const bool more = i + 1 < blocks;
        mma(d_tmem, adesc0, wdesc0, 0u);
        mma(d_tmem, adesc0 + (uint64_t)(32 >> 4), wdesc0 + (uint64_t)(kWStep >> 4), 1u);
        full_ready = __all_sync(0xffffffffu, more && ptx::mbar_test_wait(&ctrl->full[s1], ph1));
        mma(d_tmem, adesc0 + (uint64_t)(64 >> 4), wdesc0 + (uint64_t)((2 * kWStep) >> 4), 1u);
        mma(d_tmem, adesc0 + (uint64_t)(96 >> 4), wdesc0 + (uint64_t)((3 * kWStep) >> 4), 1u);
        ptx::umma_commit_elect(&ctrl->empty[s]);
        ptx::umma_commit_elect(&ctrl->acc_full[a]);
        acc_ready = __all_sync(0xffffffffu, more && ptx::mbar_test_wait(&ctrl->acc_empty[a1], aph1 ^ 1u));
        s = s1; ph = ph1; a = a1; aph = aph1;
      }
    }
  } else {
    // ------------------------ promotion and epilogue --------------------------
    ptx::setmaxnreg_inc<kT2HighRegs>();
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    const int half = (warp - 4) >> 2;                  // which 128-feature block of the tile (gated: which 64 features of both)
    const int kbs = p.num_kb;
    const bool vec4_ok = (kbs % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.a_scale) & 15) == 0);
    // combined scales a_scale[row, kb] * w_scale[block, kb] of a group of K blocks: s0 for this warp's
    // (first) feature block, s1 (gated) for the up block
    struct ScaleRegs { float s0[kTGroup]; float s1[kGated ? kTGroup : 1]; };
    ScaleRegs cur, pre;
    bool pre_valid = false;
    auto fetch_group = [&](const TileInfo& tt, int g, ScaleRegs& sr) {
      const int kb0 = g * kTGroup;
      const int nb = kGated ? tt.n_tile : tt.n_tile * 2 + half;
      const int64_t wsb = ((int64_t)tt.e * p.n_tiles + nb) * kbs + kb0;
      float av[kTGroup];
      const bool live = r < tt.valid;
      const float* src = p.a_scale + (int64_t)(tt.row0 + r) * kbs + kb0;
      if (live && vec4_ok) {
        const float4 q4 = *reinterpret_cast<const float4*>(src);
        av[0] = q4.x; av[1] = q4.y; av[2] = q4.z; av[3] = q4.w;
      } else {
#pragma unroll
        for (int jb = 0; jb < kTGroup; ++jb) av[jb] = (live && kb0 + jb < kbs) ? src[jb] : 0.f;
      }
#pragma unroll
      for (int jb = 0; jb < kTGroup; ++jb)
        sr.s0[jb] = av[jb] * ((nb < p.n_tiles && kb0 + jb < kbs) ? p.w_scale[wsb + jb] : 0.f);
      if (kGated) {
        const int64_t wsb2 = ((int64_t)tt.e * p.n_tiles + up_block0 + tt.n_tile) * kbs + kb0;
#pragma unroll
        for (int jb = 0; jb < kTGroup; ++jb)
          sr.s1[kGated ? jb : 0] = av[jb] * ((kb0 + jb < kbs) ? p.w_scale[wsb2 + jb] : 0.f);
      }
    };
    uint32_t a = 0, aph = 0, xpar = 0;
    int cursor = 0;
    bool ok = true;
    const int n_groups = (p.num_kb + kTGroup - 1) / kTGroup;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      TileInfo ti;
      locate_tile<kTTok>(tile_start, row_start, t, cursor, ti, p.w_experts);
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      uint32_t va[32], vb[32];
      if (!pre_valid) fetch_group(ti, 0, cur);
      else cur = pre;
      pre_valid = false;
      for (int g = 0; g < n_groups && ok; ++g) {
        if (g + 1 < n_groups) {
          fetch_group(ti, g + 1, pre);
        } else if (t + (int)gridDim.x < total_tiles) {
          int cursor2 = cursor;
          TileInfo tn;
          locate_tile<kTTok>(tile_start, row_start, t + gridDim.x, cursor2, tn, p.w_experts);
          fetch_group(tn, 0, pre);
          pre_valid = true;
        }
#pragma unroll
        for (int jb = 0; jb < kTGroup; ++jb) {
          if (g * kTGroup + jb >= p.num_kb) break;
          const float sc0 = cur.s0[jb];
          const float sc1 = kGated ? cur.s1[kGated ? jb : 0] : sc0;
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_full[a], aph, abort_flag, true))) {
            *abort_flag = 1; ok = false; break;
          }
          ptx::tc_fence_after();
          // plain: the 128 columns of this warp's block in two passes; gated: 64 gate columns, then
          // the 64 up columns of the same features
          const uint32_t col = tmem_base + a * 256 + (kGated ? half * 64 : half * 128) + lane_sel;
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            const float sc = pass == 0 ? sc0 : sc1;
            ptx::tmem_ld_32x32(col + pass * (kGated ? 128 : 64), va);
            ptx::tmem_ld_32x32(col + pass * (kGated ? 128 : 64) + 32, vb);
            ptx::tmem_wait_ld_tied(va, vb);
            if (pass == 1) {   // the whole stage is in registers
              ptx::tc_fence_before();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(&ctrl->acc_empty[a]);
              if (++a == (uint32_t)kT2Acc) { a = 0; aph ^= 1; }
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              acc[pass * 64 + i] = fmaf(__uint_as_float(va[i]), sc, acc[pass * 64 + i]);
              acc[pass * 64 + 32 + i] = fmaf(__uint_as_float(vb[i]), sc, acc[pass * 64 + 32 + i]);
            }
          }
        }
        if (g + 1 < n_groups) cur = pre;
      }
      if (kGated) {
        // acc[0..64) = gate, acc[64..128) = up of features j0 + half * 64 ..
        const int half_n = p.n >> 1;
        const int j0 = ti.n_tile * 128 + half * 64;
        float amax = 0.f;
        // acc[i] becomes the activated value of feature j0 + i (the up half is consumed)
        auto activate = [&](auto round16) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            float g = acc[i], u = acc[64 + i];
            if (p.bias != nullptr) {
              g += load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + j0 + i);
              u += load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + half_n + j0 + i);
            }
            // what the unfused GEMM would have stored, then (optionally) the clamp on those values
            g = round16(g);
            u = round16(u);
            if (p.clamp > 0.f) {
              g = round16(fminf(g, p.clamp));
              u = round16(fminf(fmaxf(u, -p.clamp), p.clamp));
            }
            acc[i] = __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), u);
            amax = fmaxf(amax, fabsf(acc[i]));
          }
        };
        if (p.out_f16) activate([](float x) { return __half2float(__float2half_rn(x)); });
        else activate([](float x) { return __bfloat162float(__float2bfloat16_rn(x)); });
        // the other 64 features of the token's 128-feature group are with the partner warp
        // (two buffers by tile parity: the partner has read the previous value of a buffer before
        // it arrived at the barrier of the tile in between)
        ctrl->xchg[xpar][half][r] = amax;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctrl->xbar[q]);
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->xbar[q], xpar, abort_flag))) { *abort_flag = 1; ok = false; }
        amax = fmaxf(amax, ctrl->xchg[xpar][half ^ 1][r]);
        xpar ^= 1u;
        if (ok && r < ti.valid) {
          const float scale = fmaxf(__fdiv_rn(amax, 448.0f), 1.0f / (448.0f * 512.0f));
          // 64 codes of this thread's row into the warp's staging tile (rows of 64 + 16 bytes)
          const uint32_t my_row = ptx::smem_u32(xpose_base + (warp - 4) * 32 * kT2RowPitch) + lane * 80;
#pragma unroll
          for (int c = 0; c < 64; c += 16) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              uint32_t x = 0;
#pragma unroll
              for (int b = 0; b < 4; ++b)
                x |= (uint32_t)f32_to_e4m3(fmaxf(-448.0f, fminf(__fdividef(acc[c + i + b], scale), 448.0f))) << (8 * b);
              w[i >> 2] = x;
            }
            ptx::sts128(my_row + c, make_uint4(w[0], w[1], w[2], w[3]));
          }
          if (half == 0) p.d_scale[(int64_t)(ti.row0 + r) * (half_n >> 7) + ti.n_tile] = scale;
        }
        __syncwarp();
        if (ok) {
          // eight rows per store: four lanes cover the 64 bytes of a row
          const uint32_t xp = ptx::smem_u32(xpose_base + (warp - 4) * 32 * kT2RowPitch);
          const int piece = lane & 3;
          uint8_t* dbase = reinterpret_cast<uint8_t*>(p.d) + (int64_t)(ti.row0 + q * 32) * half_n + j0 + piece * 16;
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 8 + (lane >> 2);
            if (q * 32 + rr < ti.valid)
              *reinterpret_cast<uint4*>(dbase + (int64_t)rr * half_n) = ptx::lds128(xp + rr * 80 + piece * 16);
          }
        }
        __syncwarp();
        continue;
      }
      const int f0 = ti.n_tile * 256 + half * 128;
      if (ok && f0 < p.n) {
        // the 128 finished values of this thread's row, bias added and rounded, as 16 x 16 bytes
        auto packed = [&](int c, uint32_t (&w)[4]) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            float x0 = acc[c + i], x1 = acc[c + i + 1];
            if (p.bias != nullptr) {
              x0 += load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + f0 + c + i);
              x1 += load_bias(p.bias, p.out_f16, (int64_t)ti.e * p.n + f0 + c + i + 1);
            }
            if (p.out_f16) {
              const __half2 h = __floats2half2_rn(x0, x1);
              w[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
              const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
              w[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
        };
        if (stages == (uint32_t)kT2Stages) {
          if (r < ti.valid) {
            uint16_t* drow = reinterpret_cast<uint16_t*>(p.d) + (int64_t)(ti.row0 + r) * p.n + f0;
#pragma unroll
            for (int c = 0; c < 128; c += 8) {
              uint32_t w[4];
              packed(c, w);
              *reinterpret_cast<uint4*>(drow + c) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        } else {
          // into the warp's staging tile ...
          const uint32_t xp = ptx::smem_u32(xpose_base + (warp - 4) * 32 * kT2RowPitch);
          const uint32_t my_row = xp + lane * kT2RowPitch;
#pragma unroll
          for (int c = 0; c < 128; c += 8) {
            uint32_t w[4];
            packed(c, w);
            ptx::sts128(my_row + c * 2, make_uint4(w[0], w[1], w[2], w[3]));
          }
          __syncwarp();
          // ... and out again two whole rows per store: 16 lanes cover the 256 bytes of a row
          const int piece = lane & 15;
          uint16_t* dbase = reinterpret_cast<uint16_t*>(p.d) + (int64_t)(ti.row0 + q * 32) * p.n + f0 + piece * 8;
#pragma unroll
          for (int it = 0; it < 16; ++it) {
            const int rr = it * 2 + (lane >> 4);
            if (q * 32 + rr < ti.valid)
              *reinterpret_cast<uint4*>(dbase + (int64_t)rr * p.n) = ptx::lds128(xp + rr * kT2RowPitch + piece * 16);
          }
          __syncwarp();
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    if (*abort_flag != 0) __nanosleep(20000);
    ptx::tmem_dealloc(tmem_base, 512);
  }
  if (tid == 0 && *abort_flag != 0) report_timeout(p.status);
}

template <bool kWKn, bool kGated>
int launch_fp8t256(const CUtensorMap& ta, const CUtensorMap& tw, const TParams& p, int grid, cudaStream_t st) {
  auto kern = grouped_gemm_fp8t256_kernel<kWKn, kGated>;
  static SmemConfig configured;
  const size_t smem = p.stages == kT2Stages ? kT2Smem : kT2SmemStaged;
  if (int rc = configured.ensure(kern, kT2SmemStaged > kT2Smem ? kT2SmemStaged : kT2Smem)) return rc;
  kern<<<grid, kT2Threads, smem, st>>>(ta, tw, p);
  B200_LAUNCH_OK("grouped_gemm_fp8t256_kernel");
  return B200MOE_OK;
}

template <bool kWKn>
int launch_fp8t(const CUtensorMap& ta, const CUtensorMap& tw, const TParams& p, int grid, cudaStream_t st) {
  auto kern = grouped_gemm_fp8t_kernel<kWKn>;
  static SmemConfig configured;
  if (int rc = configured.ensure(kern, kTSmem)) return rc;
  kern<<<grid, kTThreads, kTSmem, st>>>(ta, tw, p);
  B200_LAUNCH_OK("grouped_gemm_fp8t_kernel");
  return B200MOE_OK;
}

}  // namespace

// fp8 activations [M,K] (+ fp32 scales [M,K/128]) times block-scaled fp8 weights ([E,N,K] or
// [E,K,N], scales [E,N/128,K/128]); N and K multiples of 128.  Returns
// B200MOE_E_UNSUPPORTED (no launch) for anything else.
int grouped_gemm_tc_fp8t(const b200moe_gemm_args* a, cudaStream_t st) {
  const bool w8b = a->w_format == B200MOE_W_FP8_BLOCK_NK || a->w_format == B200MOE_W_FP8_BLOCK_KN;
  const bool gated = a->epilogue == B200MOE_EPI_SILU_MUL;
  if (!w8b || a->a_dtype != B200MOE_FP8_E4M3 || a->a_scale == nullptr || a->w_scale == nullptr ||
      (a->epilogue != B200MOE_EPI_NONE && !gated))
    return fail(B200MOE_E_UNSUPPORTED, "token-major fp8 grouped GEMM takes fp8 x block-scaled fp8; fused epilogue: SiLU-and-mul");
  if (gated && (a->d_dtype != B200MOE_FP8_E4M3 || a->d_scale == nullptr || a->n % 256 != 0))
    return fail(B200MOE_E_UNSUPPORTED, "token-major fp8 grouped GEMM: the fused SiLU epilogue writes e4m3 + 1x128 scales "
                                       "(d_dtype FP8_E4M3, d_scale) and needs N / 2 divisible by 128");
  if (!gated && a->d_dtype == B200MOE_FP8_E4M3)
    return fail(B200MOE_E_UNSUPPORTED, "token-major fp8 grouped GEMM: e4m3 output only with the fused SiLU epilogue");
  if (a->num_experts > kMaxExperts || a->n % 128 != 0 || a->k % 128 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "token-major fp8 grouped GEMM: N and K must be multiples of 128");
  if (((uintptr_t)a->a & 15) || ((uintptr_t)a->w & 15) || ((uintptr_t)a->d & 15))
    return fail(B200MOE_E_BADARG, "grouped GEMM: A, W and D must be 16-byte aligned");
  if (a->m == 0 || a->n == 0) return B200MOE_OK;
  const bool kn = a->w_format == B200MOE_W_FP8_BLOCK_KN;

  TParams p;
  p.a_scale = reinterpret_cast<const float*>(a->a_scale);
  p.w_scale = reinterpret_cast<const float*>(a->w_scale);
  p.bias = a->bias; p.d = a->d; p.rows_per_expert = a->rows_per_expert; p.status = a->status;
  p.m = a->m; p.n = a->n; p.k = a->k; p.num_experts = a->num_experts;
  const int w_sets = (a->w_experts > 0 && a->w_experts != a->num_experts) ? a->w_experts : a->num_experts;
  p.w_experts = w_sets != a->num_experts ? w_sets : 0;
  p.n_tiles = a->n / kFeat;
  p.num_kb = a->k / 128;
  p.out_f16 = gated ? (a->mid_dtype == B200MOE_F16) : (a->d_dtype == B200MOE_F16);
  p.d_scale = reinterpret_cast<float*>(a->d_scale);
  p.clamp = a->clamp_limit;
  {
    const int64_t in_use = (a->rows_hint > 0 && a->rows_hint < a->m) ? a->rows_hint : a->m;
    p.stages = (gated || in_use / a->num_experts >= 128) ? kT2StagesStaged : kT2Stages;
  }
  // A operand = tokens (K-major), B operand = weights (K-major, or MN-major for [E,K,N])
  p.idesc = ptx::make_idesc(0u, 0u, 0u, kn ? 1u : 0u, kTTok, kFeat);

  CUtensorMap ta, tw;
  {
    cuuint64_t dims[2] = {(cuuint64_t)a->k, (cuuint64_t)a->m};
    cuuint64_t strides[1] = {(cuuint64_t)a->k};
    cuuint32_t box[2] = {128, (cuuint32_t)kTTok};
    int rc = encode_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->a, dims, strides, box);
    if (rc) return rc;
  }
  if (!kn) {
    cuuint64_t dims[3] = {(cuuint64_t)a->k, (cuuint64_t)a->n, (cuuint64_t)w_sets};
    cuuint64_t strides[2] = {(cuuint64_t)a->k, (cuuint64_t)a->k * a->n};
    cuuint32_t box[3] = {128, (cuuint32_t)kFeat, 1};
    int rc = encode_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->w, dims, strides, box);
    if (rc) return rc;
  } else {
    cuuint64_t dims[3] = {(cuuint64_t)a->n, (cuuint64_t)a->k, (cuuint64_t)w_sets};
    cuuint64_t strides[2] = {(cuuint64_t)a->n, (cuuint64_t)a->k * a->n};
    cuuint32_t box[3] = {128, 128, 1};
    int rc = encode_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->w, dims, strides, box);
    if (rc) return rc;
  }
  int grid = sm_count();
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  const bool wide = a->n >= 256;   // 256-feature tiles; a single 128-feature block takes the narrow kernel
  const int64_t tile_bound = ((a->m + kTTok - 1) / kTTok + a->num_experts) * (int64_t)(wide ? (p.n_tiles + 1) / 2 : p.n_tiles);
  if (tile_bound < grid) grid = (int)tile_bound;
  if (grid < 1) grid = 1;
  if (gated) return kn ? launch_fp8t256<true, true>(ta, tw, p, grid, st) : launch_fp8t256<false, true>(ta, tw, p, grid, st);
  if (wide) return kn ? launch_fp8t256<true, false>(ta, tw, p, grid, st) : launch_fp8t256<false, false>(ta, tw, p, grid, st);
  return kn ? launch_fp8t<true>(ta, tw, p, grid, st) : launch_fp8t<false>(ta, tw, p, grid, st);
}

}  // namespace b200moe
