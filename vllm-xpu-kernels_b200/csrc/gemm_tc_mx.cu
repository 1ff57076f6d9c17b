// Block-scaled tensor-core grouped GEMM: MXFP4 weights (two e2m1 codes per byte,
// [E,N,K/2], one e8m0 scale per 32 elements, [E,N,K/32]) times MXFP8 activations
// (e4m3 codes [terms][M,K], one e8m0 scale per 32 elements as 32-bit words
// [terms][K/128][M]).  With terms == 2 the second plane is the residual of the
// first (activation = plane0 + plane1): each weight tile is multiplied with
// both planes, which gives 16-bit-like activation accuracy at fp8 MMA speed.
//
// tcgen05.mma kind::mxf8f6f4.block_scale multiplies both operands by their
// power-of-two scales inside the tensor core, so nothing is dequantised by CUDA
// cores: HBM and shared memory see 4-bit weights and 8-bit activations only.
//
// Same orientation, tile walk and epilogue as the other tensor-core kernels
// (weights' output features on the 128-row M side, tokens on the N side).  Roles:
//   warp 0    : TMA producer.  Weight tile of 128 rows x 128 codes, fetched with
//               the 16U4_ALIGN16B tensor-map type, which spreads every 8 packed
//               bytes into a 16-byte slot (the operand format the MMA reads),
//               128-byte swizzle; activation tile BT rows x 128 bytes.
//   warp 1    : MMA issuer, owns tensor memory
//   warps 2-5 : scale feeders: bring the e8m0 bytes of the tile's 128 weight rows
//               (one contiguous piece of the scale tensor) into shared memory
//               with cp.async one tile ahead, read the tokens' scale words (one
//               coalesced 32-bit word per token and K block) a few K blocks
//               ahead, and write both to tensor memory (tcgen05.st), one copy
//               per lane quarter as the MMA wants.
//               When K is not a multiple of 128 (that tensor-map type needs it)
//               they also spread the last, partial block, which then arrives
//               through a plain byte tensor map.
//   warps 6-9 : epilogue
//
// The same kernel (kW8) multiplies per-tensor-scaled fp8 weights ([E,K,N], e4m3 or
// e5m2, one fp32 scale per expert: the reference's w8a16 recipe,
// csrc/xpu/grouped_gemm/xe_2/grouped_gemm_xe2_interface.hpp:322-360) with the same
// two-plane activations: the weight tile then is a plain byte tile read as an
// MN-major operand, its scale factors are 2^0, and the expert's scale
// multiplies the accumulator in the epilogue.  MXFP8 weights ([E,K,N] e4m3 with one
// e8m0 scale per 32 K rows, [E,K/32,N]: the reference's "mxfp8" recipe,
// vllm_xpu_kernels/moe_utils.py:76-78, 236-403) take the same path with their real
// scale factors, staged from the transposed scale tensor.
//
// Numerics: products of e2m1 and e4m3 codes are exact, scaling by powers of two is
// exact, accumulation is fp32; the difference from the reference's w4a16 path
// (csrc/xpu/grouped_gemm/xe_2/gemm_xe2.hpp:411-471 of vllm-xpu-kernels) is the
// rounding of the activations to MXFP8 only.
#include "common.cuh"
#include "gemm_tc_common.cuh"
#include "sm100_ptx.cuh"


namespace b200moe {
namespace {

constexpr int kMxWBytes = 16384;    // 128 rows x 128 codes in 16-byte slots of 16
constexpr int kMxRawBytes = 8192;   // 128 rows x 64 packed bytes
constexpr int kMxWTx = 8192;        // the spreading load reports the packed bytes it read to its barrier
constexpr int kMxThreads = 320;
constexpr int kMxMaxStages = 8;
constexpr int kMxGroup = 2;         // K blocks per token-scale prefetch group (read two groups ahead)
constexpr int kMxSfwCap = 24576 + 16;    // largest weight-scale piece (128 rows x K/32 bytes) staged in shared memory

struct MxParams {
  const uint8_t* w_scale;   // [E, N, K/32] e8m0; kW8 with w8_block: [E, K/32, N]; else unused
  const float* w_tensor_scale;  // kW8 without w8_block: [E] fp32, multiplies the result
  int w8_block;             // kW8: 1 = MXFP8 weights (scales per 32 K rows), 0 = one scale per expert
  const uint32_t* a_scale;  // [terms][num_kb][M] words of four e8m0 bytes
  const void* bias;
  void* d;
  const int32_t* rows_per_expert;
  int32_t* status;
  int64_t m;
  int n, k, num_experts;
  int n_tiles, num_kb;
  int terms;       // activation planes (1 or 2)
  int tail;        // 1: the last K block is partial and comes through the byte map
  int stages, stage_bytes;
  int sfw_bytes;   // bytes of one staged weight-scale buffer
  int raw_shared;  // 1: one buffer for the partial K block after the staging buffers, 0: one per stage
  uint32_t tmem_cols;
  uint32_t idesc;
  int out_f16;
  int swiglu;      // 1: D[m, f/2] = swigluoai(acc[m,f], acc[m,f+1]) for even f
  float alpha, limit, clamp_limit;
};

struct MxCtrl {
  uint64_t full[kMxMaxStages];
  uint64_t sf_full[kMxMaxStages];
  uint64_t empty[kMxMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sfw_full[2];
  uint64_t sfw_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) uint16_t xpose[4][32 * 32];
};
// Shared memory after the pipeline stages: one buffer for the partial K block
// (when the stages do not carry their own), MxCtrl, the tile walk's prefix arrays
// (2 x (experts + 1) ints) and two weight-scale staging buffers.
__host__ __device__ inline int mx_prefix_bytes(int num_experts) { return ((num_experts + 1) * 4 + 15) & ~15; }

// Weight scales of a tile's rows: one contiguous piece of the scale tensor,
// copied to staging buffer (seq & 1) asynchronously by the 128 feeder threads
// (`ft` = index among them); every thread arrives on sfw_full when its part has
// landed.  Returns false when the wait for the buffer gave up.
__device__ __forceinline__ bool stage_w_scales(const MxParams& p, MxCtrl* ctrl, uint8_t* sfw,
                                               const TileInfo& ti, uint32_t seq, int ft, int kgroups,
                                               volatile int* abort_flag) {
  const uint32_t b = seq & 1;
  if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->sfw_empty[b], ((seq >> 1) & 1) ^ 1, abort_flag)))
    return false;
  const int n0 = ti.n_tile * kFeat;
  const int rows_here = (p.n - n0) < kFeat ? (p.n - n0) : kFeat;
  const int len = rows_here * kgroups;
  const uint8_t* src = p.w_scale + ((int64_t)ti.e * p.n + n0) * kgroups;
  const uint32_t dst = ptx::smem_u32(sfw + b * p.sfw_bytes);
  for (int off = ft * 16; off < len; off += 128 * 16)
    ptx::cp_async_16(dst + off, src + off, (len - off) < 16 ? (len - off) : 16);
  ptx::cp_async_mbar_arrive(&ctrl->sfw_full[b]);
  return true;
}

// The same for MXFP8 weights, whose scales are [E, K/32, N]: for every K group the
// 128 bytes of the tile's features, stored as [group][128] in the staging buffer.
// N is a multiple of 16, so a tile's valid bytes per group are whole 16-byte chunks;
// chunks past N are zero-filled (their rows get 2^0 when the scales are packed).
__device__ __forceinline__ bool stage_w_scales_kn(const MxParams& p, MxCtrl* ctrl, uint8_t* sfw,
                                                  const TileInfo& ti, uint32_t seq, int ft, int kgroups,
                                                  volatile int* abort_flag) {
  const uint32_t b = seq & 1;
  if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->sfw_empty[b], ((seq >> 1) & 1) ^ 1, abort_flag)))
    return false;
  const int n0 = ti.n_tile * kFeat;
  const int valid = (p.n - n0) < kFeat ? (p.n - n0) : kFeat;
  const uint8_t* src = p.w_scale + (int64_t)ti.e * kgroups * p.n + n0;
  const uint32_t dst = ptx::smem_u32(sfw + b * p.sfw_bytes);
  for (int c = ft; c < kgroups * 8; c += 128) {
    const int g = c >> 3, part = c & 7;
    const int bytes = valid - part * 16 >= 16 ? 16 : 0;
    ptx::cp_async_16(dst + c * 16, src + (int64_t)g * p.n + (bytes ? part * 16 : 0), bytes);
  }
  ptx::cp_async_mbar_arrive(&ctrl->sfw_full[b]);
  return true;
}

// BT tokens per tile, kTerms activation planes, kSub 128-wide K blocks per
// pipeline stage (one barrier hand-over per stage: with small token tiles the
// roles' fixed cost per hand-over, not the data, bounds the rate).
template <int BT, int kTerms, int kSub, bool kW8>
__global__ void __launch_bounds__(kMxThreads, 1)
grouped_gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_w,
                       const __grid_constant__ CUtensorMap tmap_raw, const MxParams p) {
  static_assert(kSub == 1 || kSub == kMxGroup, "a stage holds one K block or one prefetch group");
  constexpr int kChunk = BT >= 32 ? 32 : 16;
  constexpr int kNT = kTerms * BT;                  // UMMA N: the planes side by side
  constexpr int kW = kNT >= 32 ? kNT / 32 : 1;       // token-scale columns (words per lane and K block)
  constexpr uint32_t kSfBase = 2 * kNT;
  // scale columns per K block: the weight rows' four, then the tokens' kW; the region of a K
  // block starts on a multiple of 8 columns
  constexpr int kSfPer = kW <= 4 ? 8 : 16;
  constexpr int kSfCols = kSfPer * kSub;            // scale columns of one stage
  constexpr int kABytes = kNT * 128;                // activation bytes of one K block (all planes)
  constexpr int kAOff = kSub * kMxWBytes;           // stage: [W blocks][A blocks][raw tail]
  constexpr int kRawOff = kSub * (kMxWBytes + kABytes);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = p.stages;
  const int stage_bytes = p.stage_bytes;
  uint8_t* raw_one = smem + stages * stage_bytes;   // used when p.raw_shared (1024-byte aligned)
  uint8_t* ctrl_at = raw_one + (p.raw_shared ? kMxRawBytes : 0);
  MxCtrl* ctrl = reinterpret_cast<MxCtrl*>(ctrl_at);
  uint8_t* after = ctrl_at + ((sizeof(MxCtrl) + 15) & ~(size_t)15);
  int* tile_start_w = reinterpret_cast<int*>(after);
  int* row_start_w = reinterpret_cast<int*>(after + mx_prefix_bytes(p.num_experts));
  uint8_t* sfw = after + 2 * mx_prefix_bytes(p.num_experts);
  volatile int* abort_flag = &ctrl->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {
    build_tile_prefix<BT>(p.rows_per_expert, p.num_experts, p.n_tiles, row_start_w, tile_start_w);
    if (lane == 0) {
      ptx::prefetch_tensormap(&tmap_a);
      ptx::prefetch_tensormap(&tmap_w);
      ptx::prefetch_tensormap(&tmap_raw);
    }
  } else if (warp == 1) {
    ptx::tmem_alloc(&ctrl->tmem_base, p.tmem_cols);
    ptx::tmem_relinquish();
  } else if (warp == 2 && lane == 0) {
    for (int s = 0; s < kMxMaxStages; ++s) {
      ptx::mbar_init(&ctrl->full[s], 1);
      ptx::mbar_init(&ctrl->sf_full[s], 4);
      ptx::mbar_init(&ctrl->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&ctrl->acc_full[a], 1);
      ptx::mbar_init(&ctrl->acc_empty[a], 4);
      ptx::mbar_init(&ctrl->sfw_full[a], 128);
      ptx::mbar_init(&ctrl->sfw_empty[a], 4);
    }
    ctrl->abort_flag = 0;
    ptx::fence_barrier_init();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  const int* tile_start = tile_start_w;
  const int* row_start = row_start_w;
  const int total_tiles = tile_start[p.num_experts];
  const int tail_kb = (!kW8 && p.tail) ? p.num_kb - 1 : -1;
  constexpr int kWTx = kW8 ? kMxWBytes : kMxWTx;   // bytes a weight-tile load reports
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
          ptx::mbar_expect_tx(&ctrl->full[s], nsub * (kWTx + kABytes));
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            const int kb = kb0 + sub;
            if (sub < nsub) {
              if (kW8)   // 128 K rows x 128 features, one byte each; rows past K are zero-filled
                ptx::tma_load_3d(st + sub * kMxWBytes, &tmap_w, &ctrl->full[s], n0, kb * 128, ti.e);
              else if (kb == tail_kb)
                ptx::tma_load_3d(p.raw_shared ? raw_one : st + kRawOff, &tmap_raw, &ctrl->full[s], kb * 64, n0, ti.e);
              else
                ptx::tma_load_3d(st + sub * kMxWBytes, &tmap_w, &ctrl->full[s], kb * 128, n0, ti.e);
#pragma unroll
              for (int term = 0; term < kTerms; ++term)
                ptx::tma_load_3d(st + kAOff + sub * kABytes + term * (BT * 128), &tmap_a, &ctrl->full[s],
                                 kb * 128, ti.row0, term);
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
      uint32_t idesc_j[4];
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) idesc_j[j] = (p.idesc & ~(0x3fu << 17)) | (j << 29) | (j << 4);
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        TileInfo ti;
        locate_tile<BT>(tile_start, row_start, t, cursor, ti);
        const uint32_t a = acc_it & 1;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->acc_empty[a], ((acc_it >> 1) & 1) ^ 1, abort_flag))) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * kNT;
        // A partly filled token tile multiplies only up to its last valid column (UMMA N in
        // steps of 16; with two planes the second one's columns follow the first one's BT).
        const uint32_t n_eff = (uint32_t)((kTerms - 1) * BT + ((ti.valid + 15) & ~15));
        const uint32_t n_bits = (n_eff >> 3) << 17;
        for (int si = 0; si < num_st; ++si) {
          bool go = ptx::mbar_wait(&ctrl->full[s], ph, abort_flag);
          if (go) go = ptx::mbar_wait(&ctrl->sf_full[s], ph, abort_flag);
          if (!__all_sync(0xffffffffu, go)) { ok = false; break; }
          ptx::tc_fence_after();
          // Every operand descriptor of the stage is the first weight block's plus a
          // compile-time offset (the address field counts 16-byte units).
          const uint64_t desc0 = ptx::make_smem_desc(smem_base + s * stage_bytes, 16, 1024);
          const uint64_t desc0w = kW8 ? ptx::make_smem_desc(smem_base + s * stage_bytes, 16384, 1024) : desc0;
          const uint32_t sf0 = tmem_base + kSfBase + s * kSfCols;
          const int kb0 = si * kSub;
#pragma unroll
          for (int sub = 0; sub < kSub; ++sub) {
            if (kb0 + sub < p.num_kb) {
              // The planes' activation tiles are adjacent in the stage: one K-major
              // operand of kNT rows; their results land in adjacent column blocks.
              const uint32_t sfa = sf0 + kSfPer * sub;
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j) {
                // K-major e2m1 tile: 32 codes further is 32 bytes; MN-major byte tile: 32 K rows
                const uint64_t wdesc = desc0w + (uint64_t)((sub * kMxWBytes + j * (kW8 ? 4096 : 32)) >> 4);
                const uint64_t adesc = desc0 + (uint64_t)((kAOff + sub * kABytes + j * 32) >> 4);
                ptx::umma_mx_elect(d_tmem, wdesc, adesc, idesc_j[j] | n_bits, (kb0 + sub > 0 || j > 0) ? 1u : 0u, sfa, sfa + 4);
              }
            }
          }
          ptx::umma_commit_elect(&ctrl->empty[s]);
          if (++s == (uint32_t)stages) { s = 0; ph ^= 1; }
        }
        if (ok) { ptx::umma_commit_elect(&ctrl->acc_full[a]); ++acc_it; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------ scale feeders ------------------------------
    const int q = warp & 3;                       // lane quarter this warp may write
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    const int ft = (warp - 2) * 32 + lane;         // 0..127: tile row spread by this thread (tail
                                                   // block), index in the cooperative copies
    const int kgroups = p.k / 32;
    const int n_groups = (p.num_kb + kMxGroup - 1) / kMxGroup;
    const int64_t plane_words = (int64_t)p.num_kb * p.m;
    uint32_t s = 0, ph = 0;
    int cursor = 0, cursor_next = 0, cursor_la = 0;
    bool ok = true;

    // Token scales of kMxGroup K blocks: word [plane][kb][row], coalesced over the
    // lanes.  They are read two groups ahead of their use (cur <- nxt <- nx2), by a
    // look-ahead position (la_*) that runs over the same (tile, group) sequence.
    uint32_t cur_b[kMxGroup][kW], nxt_b[kMxGroup][kW], nx2_b[kMxGroup][kW];
    auto fetch_b = [&](const TileInfo& ti, int g, uint32_t (&db)[kMxGroup][kW]) {
#pragma unroll
      for (int u = 0; u < kMxGroup; ++u) {
        const int kb = g * kMxGroup + u;
#pragma unroll
        for (int j = 0; j < kW; ++j) {
          const int n = lane + 32 * j;              // row of the side-by-side token operand
          const int term = n / BT, tok = n % BT;
          uint32_t v = 0x7f7f7f7fu;
          if (kb < p.num_kb && term < kTerms && tok < ti.valid)
            v = p.a_scale[term * plane_words + (int64_t)kb * p.m + ti.row0 + tok];
          db[u][j] = v;
        }
      }
    };
    int la_t = blockIdx.x, la_g = 0;
    TileInfo la_ti;
    bool la_valid = la_t < total_tiles;
    if (la_valid) locate_tile<BT>(tile_start, row_start, la_t, cursor_la, la_ti);
#define B200_MX_LA_ADVANCE()                                                              \
  do {                                                                                    \
    if (++la_g == n_groups) {                                                             \
      la_g = 0;                                                                           \
      la_t += gridDim.x;                                                                  \
      la_valid = la_t < total_tiles;                                                      \
      if (la_valid) locate_tile<BT>(tile_start, row_start, la_t, cursor_la, la_ti);       \
    }                                                                                     \
  } while (0)
    if (la_valid) { fetch_b(la_ti, la_g, cur_b); B200_MX_LA_ADVANCE(); }
    if (la_valid) { fetch_b(la_ti, la_g, nxt_b); B200_MX_LA_ADVANCE(); }

    uint32_t tile_seq = 0;
    TileInfo ti, ti_next;
    const bool staged = !kW8 || p.w8_block != 0;   // weight scales come through shared memory
    auto stage = [&](const TileInfo& tn, uint32_t seq) {
      return kW8 ? stage_w_scales_kn(p, ctrl, sfw, tn, seq, ft, kgroups, abort_flag)
                 : stage_w_scales(p, ctrl, sfw, tn, seq, ft, kgroups, abort_flag);
    };
    if (staged && (int)blockIdx.x < total_tiles) {
      locate_tile<BT>(tile_start, row_start, blockIdx.x, cursor_next, ti_next);
      if (!stage(ti_next, 0u)) { *abort_flag = 1; ok = false; }
    }
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_seq) {
      locate_tile<BT>(tile_start, row_start, t, cursor, ti);
      const int t_next = t + gridDim.x;
      if (staged && t_next < total_tiles) {
        locate_tile<BT>(tile_start, row_start, t_next, cursor_next, ti_next);
        if (!stage(ti_next, tile_seq + 1)) {
          *abort_flag = 1; ok = false; break;
        }
      }
      const uint32_t b = tile_seq & 1;
      if (staged && !__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->sfw_full[b], (tile_seq >> 1) & 1, abort_flag))) {
        *abort_flag = 1; ok = false; break;
      }
      const uint32_t sfw_s = ptx::smem_u32(sfw + b * p.sfw_bytes);
      const int n0 = ti.n_tile * kFeat;
      for (int g = 0; g < n_groups && ok; ++g) {
        if (la_valid) { fetch_b(la_ti, la_g, nx2_b); B200_MX_LA_ADVANCE(); }
#pragma unroll
        for (int u = 0; u < kMxGroup; ++u) {
          const int kb = g * kMxGroup + u;
          const int sub = u % kSub;                  // position of this K block in its stage
          if (kb < p.num_kb && ok) {
            // Four scale bytes per row from the staged piece: two aligned words and a
            // funnel shift (rows are K/32 bytes apart, any alignment); bytes of groups
            // past the row end become 0x7f.
            uint32_t wa[4];
            const int left = kgroups - 4 * kb;
            const uint32_t keep = left >= 4 ? 0xffffffffu : ((1u << (8 * left)) - 1u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int row = lane + 32 * j;
              if (!kW8) {
                const uint32_t addr = sfw_s + row * kgroups + 4 * kb;
                const uint32_t lo = ptx::lds32(addr & ~3u), hi = ptx::lds32((addr & ~3u) + 4);
                const uint32_t v = __funnelshift_r(lo, hi, (addr & 3u) * 8);
                wa[j] = (n0 + row < p.n) ? ((v & keep) | (0x7f7f7f7fu & ~keep)) : 0x7f7f7f7fu;
              } else if (p.w8_block) {
                // staged as [group][128 features]: one byte per group of this K block
                uint32_t v = 0;
#pragma unroll
                for (int gq = 0; gq < 4; ++gq)
                  if (gq < left) v |= ptx::lds8(sfw_s + (4 * kb + gq) * 128 + row) << (8 * gq);
                wa[j] = (n0 + row < p.n) ? (v | (0x7f7f7f7fu & ~keep)) : 0x7f7f7f7fu;
              } else {
                wa[j] = 0x7f7f7f7fu;   // per-tensor scale: applied in the epilogue
              }
            }
            if (sub == 0) {   // the stage's scale columns and weight buffer are free again
              if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->empty[s], ph ^ 1, abort_flag))) {
                *abort_flag = 1; ok = false;
              }
              ptx::tc_fence_after();
            }
            if (ok) {
              const uint32_t col = tmem_base + kSfBase + s * kSfCols + kSfPer * sub + lane_sel;
              {
                // eight columns at once: the weight rows' four, then the tokens' (unused ones 2^0)
                uint32_t r8[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) { r8[j] = wa[j]; r8[4 + j] = j < kW ? cur_b[u][j < kW ? j : 0] : 0x7f7f7f7fu; }
                ptx::tmem_st_32x8(col, r8);
                if (kW > 4)   // token tiles wider than 128 columns: their remaining scale columns
                  ptx::tmem_st_32x4(col + 8, cur_b[u][4 < kW ? 4 : 0], 5 < kW ? cur_b[u][5 < kW ? 5 : 0] : 0x7f7f7f7fu,
                                    0x7f7f7f7fu, 0x7f7f7f7fu);
              }
              if (kb == tail_kb) {
                // Spread the partial block: row ft, 64 packed bytes -> eight 16-byte
                // slots (8 data bytes each), slot index xor-ed with (ft & 7).
                if (!__all_sync(0xffffffffu, ptx::mbar_wait(&ctrl->full[s], ph, abort_flag))) {
                  *abort_flag = 1; ok = false;
                } else {
                  const uint32_t st = ptx::smem_u32(smem + s * stage_bytes);
                  const uint32_t src = (p.raw_shared ? ptx::smem_u32(raw_one) : st + kRawOff) + ft * 64;
                  const uint32_t dst = st + sub * kMxWBytes + (ft >> 3) * 1024 + (ft & 7) * 128;
#pragma unroll
                  for (int c = 0; c < 4; ++c) {
                    const uint4 v = ptx::lds128(src + c * 16);
                    ptx::sts64(dst + (((2 * c) ^ (ft & 7)) << 4), v.x, v.y);
                    ptx::sts64(dst + (((2 * c + 1) ^ (ft & 7)) << 4), v.z, v.w);
                  }
                  ptx::fence_proxy_async();
                }
              }
              if (sub == kSub - 1 || kb == p.num_kb - 1) {   // last K block of the stage
                ptx::tmem_wait_st();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ctrl->sf_full[s]);
                if (++s == (uint32_t)stages) { s = 0; ph ^= 1; }
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kMxGroup; ++u)
#pragma unroll
          for (int j = 0; j < kW; ++j) { cur_b[u][j] = nxt_b[u][j]; nxt_b[u][j] = nx2_b[u][j]; }
      }
      if (staged) {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&ctrl->sfw_empty[b]);
      }
    }
#undef B200_MX_LA_ADVANCE
    if (warp == 2 && lane == 0)
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
      const float w_mul = (kW8 && !p.w8_block) ? p.w_tensor_scale[ti.e] : 1.0f;
      const uint32_t a = acc_it & 1;
      // a whole tile's MMAs away: poll from one lane, sleeping in between, so that the
      // wait does not take issue slots from the feeder warp on the same scheduler
      if (!ptx::mbar_wait_warp(&ctrl->acc_full[a], (acc_it >> 1) & 1, abort_flag, 128)) { ok = false; break; }
      ptx::tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < BT; c0 += kChunk) {
        if (c0 < ti.valid) {
          uint32_t v[kChunk];
          float acc[kChunk];
#pragma unroll
          for (int i = 0; i < kChunk; ++i) acc[i] = 0.f;
#pragma unroll
          for (int term = 0; term < kTerms; ++term) {   // the planes' partial results add up
            const uint32_t col = tmem_base + a * kNT + term * BT + c0 + lane_sel;
            if (kChunk == 32) ptx::tmem_ld_32x32(col, reinterpret_cast<uint32_t(&)[32]>(v));
            else ptx::tmem_ld_32x16(col, reinterpret_cast<uint32_t(&)[16]>(v));
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < kChunk; ++i) acc[i] += __uint_as_float(v[i]);
          }
          float vals[kChunk];
#pragma unroll
          for (int i = 0; i < kChunk; ++i) vals[i] = kW8 ? fmaf(acc[i], w_mul, bias_v) : acc[i] + bias_v;
          if (p.swiglu) {
            // One branch around the whole block: the unrolled body stays straight-line code, so
            // the 32 shuffle / exp / divide chains overlap instead of running one after another.
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
            store_block_transposed<kChunk, 16>(ctrl->xpose[warp - 6], vals, p.d, p.out_f16,
                                               (int64_t)ti.row0 + c0, ti.valid - c0, p.m, n_out,
                                               (ti.n_tile * kFeat + q * 32) >> 1, lane);
          else
            store_block_transposed<kChunk, 32>(ctrl->xpose[warp - 6], vals, p.d, p.out_f16,
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
    ptx::tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (tid == 0 && *abort_flag != 0) report_timeout(p.status);
}

template <int BT, int kTerms, int kSub, bool kW8>
int launch_mx(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& traw, MxParams& p,
              int grid, cudaStream_t st) {
  auto kern = grouped_gemm_mx_kernel<BT, kTerms, kSub, kW8>;
  const uint32_t need = 2 * kTerms * BT + kMxMaxStages * (kTerms * BT > 128 ? 16 : 8) * kSub;
  p.tmem_cols = need <= 128 ? 128u : (need <= 256 ? 256u : 512u);
  // The partial K block's packed bytes get one buffer for the whole CTA when a tile
  // has at least as many stages as the pipeline (its next use then comes after
  // the previous one was consumed), else one per stage.
  const int body = kSub * (kMxWBytes + kTerms * BT * 128);
  const int fixed = 1024 + (int)((sizeof(MxCtrl) + 15) & ~(size_t)15) + 2 * mx_prefix_bytes(p.num_experts) +
                    2 * p.sfw_bytes;
  const int budget = 227 * 1024 - fixed;
  const int num_st = (p.num_kb + kSub - 1) / kSub;
  p.raw_shared = 0;
  p.stage_bytes = body + (p.tail ? kMxRawBytes : 0);
  p.stages = budget / p.stage_bytes;
  if (p.tail) {
    int st_shared = (budget - kMxRawBytes) / body;
    if (st_shared > kMxMaxStages) st_shared = kMxMaxStages;
    if (st_shared > p.stages && num_st >= st_shared) { p.raw_shared = 1; p.stage_bytes = body; p.stages = st_shared; }
  }
  if (p.stages > kMxMaxStages) p.stages = kMxMaxStages;
  if (p.stages < 2) return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: tile does not fit shared memory");
  const size_t smem = (size_t)fixed + (size_t)p.stages * p.stage_bytes + (p.raw_shared ? kMxRawBytes : 0);
  static SmemConfig configured;
  if (int rc = configured.ensure(kern, smem)) return rc;
  kern<<<grid, kMxThreads, smem, st>>>(ta, tw, traw, p);
  B200_LAUNCH_OK("grouped_gemm_mx_kernel");
  return B200MOE_OK;
}

}  // namespace

// MXFP4 weights x MXFP8 activations (one plane, or two with the residual) on the
// block-scaled tensor-core path.  a: codes [terms][M,K]; a_scale: 32-bit words
// [terms][ceil(K/128)][M] of four e8m0 bytes (what b200moe_quant_mxfp8 writes).
// Returns B200MOE_E_UNSUPPORTED (no launch) for anything else.
int grouped_gemm_tc_mx(const b200moe_gemm_args* a, cudaStream_t st) {
  const bool x2 = a->a_dtype == B200MOE_FP8_E4M3_X2;
  const bool w4 = a->w_format == B200MOE_W_MXFP4_NK;
  const bool w8mx = a->w_format == B200MOE_W_MXFP8_KN;
  const bool w8 = a->w_format == B200MOE_W_FP8_TENSOR_KN || a->w_format == B200MOE_W_FP8E5M2_TENSOR_KN || w8mx;
  if (!(w4 || w8) || !(a->a_dtype == B200MOE_FP8_E4M3 || x2) || a->a_scale == nullptr)
    return fail(B200MOE_E_UNSUPPORTED,
                "block-scaled GEMM takes MXFP4, MXFP8 or per-tensor fp8 weights and MXFP8 activations");
  if (a->epilogue == B200MOE_EPI_SILU_MUL)
    return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: SiLU epilogue not available");
  if (a->num_experts > kMaxExperts || a->k % 32 != 0 || a->k < 128 || (w4 && a->k % 64 != 0))
    return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: K must be a multiple of 64 (fp8 weights: 32), at least 128");
  if (w8 && a->n % 16 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: N must be a multiple of 16 for [E,K,N] fp8 weights");
  if (((uintptr_t)a->a & 15) || ((uintptr_t)a->w & 31) || ((uintptr_t)a->d & 15) || ((uintptr_t)a->a_scale & 3))
    return fail(B200MOE_E_BADARG, "block-scaled GEMM: A and D must be 16-byte, W 32-byte, A scales 4-byte aligned");
  if (a->epilogue == B200MOE_EPI_SWIGLUOAI && (a->n / 2) % 8 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: gated output width must be a multiple of 8");
  if (x2 && (a->m * (int64_t)a->k) % 16 != 0)
    return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: the second activation plane must be 16-byte aligned");
  if (a->m == 0 || a->n == 0) return B200MOE_OK;

  MxParams p;
  p.w_scale = reinterpret_cast<const uint8_t*>(a->w_scale);
  p.w_tensor_scale = reinterpret_cast<const float*>(a->w_scale);
  p.a_scale = reinterpret_cast<const uint32_t*>(a->a_scale);
  p.bias = a->bias; p.d = a->d; p.rows_per_expert = a->rows_per_expert; p.status = a->status;
  p.m = a->m; p.n = a->n; p.k = a->k; p.num_experts = a->num_experts;
  p.n_tiles = (a->n + kFeat - 1) / kFeat;
  p.num_kb = (a->k + 127) / 128;
  p.terms = x2 ? 2 : 1;
  p.tail = w4 && (a->k % 128) != 0;
  p.sfw_bytes = 0;
  p.w8_block = w8mx ? 1 : 0;
  if (w8mx) {
    // per K group the tile's 128 scale bytes: whole 16-byte chunks from a 16-byte aligned tensor
    const int piece = 128 * (a->k / 32);
    if (((uintptr_t)a->w_scale & 15) != 0 || piece > kMxSfwCap)
      return fail(B200MOE_E_UNSUPPORTED, "block-scaled GEMM: K at most 6144, scales 16-byte aligned");
    p.sfw_bytes = piece;
  }
  if (w4) {
    // The weight scales of a tile (128 rows x K/32 bytes, contiguous in the scale
    // tensor) are staged in shared memory: every tile's piece must start on a
    // 16-byte boundary and two pieces must fit.
    const int kgroups = a->k / 32;
    const int piece = ((128 * kgroups + 15) & ~15) + 16;
    if (((uintptr_t)a->w_scale & 15) != 0 || ((int64_t)a->n * kgroups) % 16 != 0 || piece > kMxSfwCap)
      return fail(B200MOE_E_UNSUPPORTED,
                  "block-scaled GEMM: N * K / 32 must be a multiple of 16, K at most 6144, scales 16-byte aligned");
    p.sfw_bytes = piece;
  }
  p.out_f16 = a->d_dtype == B200MOE_F16;
  p.swiglu = a->epilogue == B200MOE_EPI_SWIGLUOAI;
  p.alpha = a->act_alpha; p.limit = a->act_limit; p.clamp_limit = a->clamp_limit;

  const int64_t rows_in_use = (a->rows_hint > 0 && a->rows_hint < a->m) ? a->rows_hint : a->m;
  const int64_t avg = (rows_in_use + a->num_experts - 1) / a->num_experts;
  int bt = avg <= 8 ? 16 : (avg <= 40 ? 64 : 128);
  // both planes' accumulators share tensor memory: two planes of 96 tokens are one MMA of
  // N = 192 (enough work per instruction to keep the tensor pipe busy), two stages of them
  // and the scale columns fill the 512 columns
  if (x2 && bt > 64) bt = avg > 48 ? 96 : 64;   // measured: 64 rows per expert -22 %, 32 rows +8 %
  if (!x2 && avg > 128) bt = 192;               // one plane: the same N = 192 instruction
  // weights: e2m1 K-major, or e4m3 / e5m2 MN-major; activations e4m3 K-major
  const uint32_t a_fmt = w4 ? 5u : (a->w_format == B200MOE_W_FP8E5M2_TENSOR_KN ? 1u : 0u);
  p.idesc = ptx::make_idesc_mx(a_fmt, 0u, kFeat, (uint32_t)(bt * p.terms)) | (w8 ? (1u << 15) : 0u);

  CUtensorMap ta, tw, traw;
  {
    cuuint64_t dims[3] = {(cuuint64_t)a->k, (cuuint64_t)a->m, (cuuint64_t)p.terms};
    cuuint64_t strides[2] = {(cuuint64_t)a->k, (cuuint64_t)a->k * (cuuint64_t)a->m};
    cuuint32_t box[3] = {128, (cuuint32_t)bt, 1};
    int rc = encode_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->a, dims, strides, box);
    if (rc) return rc;
  }
  if (w8) {
    cuuint64_t dims[3] = {(cuuint64_t)a->n, (cuuint64_t)a->k, (cuuint64_t)a->num_experts};
    cuuint64_t strides[2] = {(cuuint64_t)a->n, (cuuint64_t)a->k * a->n};
    cuuint32_t box[3] = {128, 128, 1};
    int rc = encode_map(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->w, dims, strides, box);
    if (rc) return rc;
    traw = tw;
  } else {
    {
      // Whole 128-code blocks only: this tensor-map type wants the inner extent to be
      // a multiple of 128 codes; the row pitch stays K/2 bytes.
      cuuint64_t dims[3] = {(cuuint64_t)(a->k - a->k % 128), (cuuint64_t)a->n, (cuuint64_t)a->num_experts};
      cuuint64_t strides[2] = {(cuuint64_t)(a->k / 2), (cuuint64_t)(a->k / 2) * a->n};
      cuuint32_t box[3] = {128, (cuuint32_t)kFeat, 1};
      int rc = encode_map(&tw, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, a->w, dims, strides, box);
      if (rc) return rc;
    }
    {
      cuuint64_t dims[3] = {(cuuint64_t)(a->k / 2), (cuuint64_t)a->n, (cuuint64_t)a->num_experts};
      cuuint64_t strides[2] = {(cuuint64_t)(a->k / 2), (cuuint64_t)(a->k / 2) * a->n};
      cuuint32_t box[3] = {64, (cuuint32_t)kFeat, 1};
      int rc = encode_map(&traw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a->w, dims, strides, box,
                          CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rc) return rc;
    }
  }
  const int64_t tile_bound = ((a->m + bt - 1) / bt + a->num_experts) * (int64_t)p.n_tiles;
  int grid = sm_count();
  if (a->max_ctas > 0 && a->max_ctas < grid) grid = a->max_ctas;
  if (tile_bound < grid) grid = (int)tile_bound;
  if (grid < 1) grid = 1;
  // Small token tiles move two K blocks per pipeline stage.
#define B200_MX_CASES(W8)                                                              \
  if (x2) {                                                                            \
    if (bt == 16) return launch_mx<16, 2, 2, W8>(ta, tw, traw, p, grid, st);           \
    if (bt == 96) return launch_mx<96, 2, 1, W8>(ta, tw, traw, p, grid, st);           \
    return launch_mx<64, 2, 1, W8>(ta, tw, traw, p, grid, st);                         \
  }                                                                                    \
  if (bt == 192) return launch_mx<192, 1, 1, W8>(ta, tw, traw, p, grid, st);           \
  if (bt == 16) return launch_mx<16, 1, 2, W8>(ta, tw, traw, p, grid, st);             \
  if (bt == 64) return launch_mx<64, 1, 2, W8>(ta, tw, traw, p, grid, st);             \
  return launch_mx<128, 1, 1, W8>(ta, tw, traw, p, grid, st);
  if (w8) { B200_MX_CASES(true) }
  B200_MX_CASES(false)
#undef B200_MX_CASES
}

}  // namespace b200moe
