// Grouped NVFP4 GEMM for the routed and shared experts: tcgen05 block-scaled
// FP4 MMA (kind::mxf4nvf4, 16-element UE4M3 blocks) with TMA-fed shared-memory
// stages and double-buffered TMEM accumulators.
//
// Replaces, for all (token, expert) pairs at once, the reference's per-row host
// linear RunNvfp4LinearHost (runtime/src/backend/expert_layer.cpp:231-267:
// dequantise activation, dequantise weight, CpuMatmulRowMajor :212-229) and
// the steps fused behind it:
//   kGemmUp  : ApplyRelu2 (:269-275) and the re-quantisation of the activated
//              row that the next RunNvfp4LinearHost call performs through
//              PackRowMajorFp32ToNvfp4 (runtime/src/backend/nvfp4_packing.cpp:130-153);
//   kGemmDown: the routing-weight multiply of :951-953 (the sum over slots is
//              done by the combine kernel so that it stays in slot order).
//
// Operand roles: A = activations (128 token rows per tile, K-major packed E2M1),
// B = expert weights (BN output features per tile, K-major packed E2M1).  One
// K block is 256 elements = one 128-byte swizzled shared-memory row = four
// K=64 MMAs.  Block scales travel shared memory -> TMEM with tcgen05.cp in the
// 32-lane x 16-byte form; activations use the reference's 128x4 tile order
// (runtime/src/backend/nvfp4_scale_layout.cpp:14-28) unchanged.
//
// Warp roles (384 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2-9 = epilogue (two warps per TMEM lane quarter, splitting the
// tile's columns), warps 10-11 = block-scale copiers.  The twelve scale copies
// of a K block take longer to issue than its four MMAs and a thread's tcgen05
// operations execute in order, so the copies have threads of their own and run
// one K block ahead of the MMAs into double-buffered TMEM columns.  Every
// mbarrier wait is bounded; on a timeout the CTA records kDevWaitTimeout and
// unwinds.
#include <algorithm>
#include <cstdlib>

#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

constexpr int kEpilogueWarps = 8;
constexpr int kScaleWarp = 2 + kEpilogueWarps;  // issues the block-scale copies into TMEM
constexpr int kScaleWarps = 2;  // the copies are split between this many issuing threads
                                // (four measured no faster than two)
constexpr int kGemmThreads = (2 + kEpilogueWarps + kScaleWarps) * 32;
constexpr int kStageStride = 36;  // floats per staged row: 32 + 4 keeps float4 accesses conflict-free

template <int BN_, int A_ROWS_, int SFB_GS_, int STAGES_, bool ROW_STAGING_ = true>
struct TileCfg {
  static constexpr int BN = BN_;
  static constexpr int A_ROWS = A_ROWS_;
  static constexpr int SFB_GS = SFB_GS_;  // 32-row scale groups stored per K tile (multiple of 4:
                                          // an MMA's scale address must be 4-column aligned)
  static constexpr int STAGES = STAGES_;
  static constexpr bool PAIR = false;  // (tile_rows_of: one row tile per tile unit)
  static constexpr int B_ROWS = BN_;
  static constexpr int A_BYTES = A_ROWS * 128;
  static constexpr int B_BYTES = B_ROWS * 128;
  static constexpr int SFA_BYTES = 2048;
  static constexpr int SFB_BYTES = SFB_GS * 512;
  static constexpr int STAGE_TX = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int ACC_STRIDE = BN;  // TMEM columns per accumulator
  // block scales are double-buffered in TMEM so that the copies of K block i+1
  // do not have to wait for the MMAs of K block i to finish reading theirs
  static constexpr int SF_BUFS = 2;
  static constexpr int SF_BUF_COLS = 16 + 4 * SFB_GS;
  static constexpr int SFA_COL = 2 * ACC_STRIDE;
  static constexpr int SFB_COL = SFA_COL + 16;
  static constexpr int TMEM_USED = SFA_COL + SF_BUFS * SF_BUF_COLS;
  static constexpr int TMEM_COLS = TMEM_USED <= 32 ? 32 : TMEM_USED <= 64 ? 64 : TMEM_USED <= 128 ? 128 : TMEM_USED <= 256 ? 256 : 512;
  // full and empty per stage; accumulator full / empty; scale-ready
  // (rounded up: the epilogue's staging area behind it is accessed 16 bytes at a time)
  static constexpr int BAR_BYTES = ((2 * STAGES + 4 + SF_BUFS) * 8 + 16 + 15) / 16 * 16;
  // staging for the row-scattering epilogue of the down projection
  static constexpr bool ROW_STAGING = ROW_STAGING_;
  static constexpr int EPI_STAGE_BYTES = ROW_STAGING_ ? kEpilogueWarps * 32 * kStageStride * 4 : 0;
  // The MMA always reads 128 A rows; with a smaller box the tail rows alias the
  // following stages, which is harmless (those output rows are never stored)
  // but must stay inside the allocation: the B region follows the A region.
  static constexpr int SMEM_BYTES =
      STAGES * (A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES) + BAR_BYTES + EPI_STAGE_BYTES + 1024;
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "BN");
  static_assert(SFB_GS % 4 == 0 && SFB_GS * 32 >= BN, "weight scale groups");
  static_assert(TMEM_USED <= 512, "TMEM budget");
  static_assert(STAGES * B_BYTES >= 128 * 128, "A over-read must stay inside shared memory");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

using CfgPrefillUp = TileCfg<208, 128, 8, 4, false>;
using CfgPrefillDown = TileCfg<192, 128, 8, 4>;
using CfgDecode = TileCfg<128, 32, 4, 7>;
using CfgDecodeWide = TileCfg<128, 128, 4, 5>;

__device__ __forceinline__ void report_timeout(int32_t* error, volatile int* abort_flag) {
  *abort_flag = 1;
  if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
}

// All scale copies of one full K block that fall to copier `PART`; compile-time
// indices only, so that no copy carries a run-time predicate.
template <class C>
__device__ __forceinline__ void scale_copy(uint32_t taddr, uint64_t desc) {
  tcgen05_cp_32x128b_warpx4(taddr, desc);
}

template <class C, int PART>
__device__ __forceinline__ void issue_scale_copies(uint32_t sf_tmem, uint32_t sfa_addr,
                                                   uint32_t sfb_addr) {
#pragma unroll
  for (int c = PART; c < 4; c += kScaleWarps) {
    scale_copy<C>(sf_tmem + C::SFA_COL + 4 * c, make_smem_desc(sfa_addr + c * 512, 0, 128, 0));
  }
#pragma unroll
  for (int c = PART; c < C::SFB_GS; c += kScaleWarps) {
    scale_copy<C>(sf_tmem + C::SFB_COL + 4 * c, make_smem_desc(sfb_addr + c * 512, 0, 128, 0));
  }
}

// The row tile a CTA works on in tile unit `rt` (a row tile, or a pair of them).
struct TileRows {
  int row0;      // first row of the 128-row slot
  int rows;      // valid rows in it
  int load_row0; // where the operands are read from (a valid slot even when rows == 0)
  int expert;
};

template <class C>
__device__ __forceinline__ TileRows tile_rows_of(const GemmArgs& args, int rt, int num_row_tiles,
                                                 uint32_t cta_rank) {
  TileRows t;
  const int index = C::PAIR ? 2 * rt + static_cast<int>(cta_rank) : rt;
  if (args.row_tiles != nullptr) {
    // the plan gives every expert an even number of tiles when pairs consume them
    const int safe = min(index, num_row_tiles - 1);
    t.row0 = args.row_tiles[safe].row0;
    t.rows = index < num_row_tiles ? args.row_tiles[safe].rows : 0;
    t.expert = args.row_tiles[safe].expert;
    t.load_row0 = t.row0;
  } else {
    t.row0 = index * 128;
    t.rows = max(0, min(128, args.dense_rows - t.row0));
    t.expert = 0;
    t.load_row0 = min(t.row0, ((args.dense_rows - 1) >> 7) << 7);
  }
  return t;
}

template <class C, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs args) {
  const CUtensorMap& tmap_a = maps.a;
  const CUtensorMap& tmap_b_tail = maps.b_tail;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) &
                                             ~static_cast<uintptr_t>(1023u));
  uint8_t* sA = smem;
  uint8_t* sB = sA + C::STAGES * C::A_BYTES;
  uint8_t* sSFA = sB + C::STAGES * C::B_BYTES;
  uint8_t* sSFB = sSFA + C::STAGES * C::SFA_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sSFB + C::STAGES * C::SFB_BYTES);
  uint64_t* empty_bar = full_bar + C::STAGES;
  uint64_t* tmem_full_bar = empty_bar + C::STAGES;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* sf_ready_bar = tmem_empty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_ready_bar + C::SF_BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stage_base = reinterpret_cast<float*>(
      reinterpret_cast<uint8_t*>(full_bar) + C::BAR_BYTES);  // down epilogue staging

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int unit = static_cast<int>(blockIdx.x);
  const int units = static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], kEpilogueWarps);
    }
    for (int b = 0; b < C::SF_BUFS; ++b) {
      mbar_init(&sf_ready_bar[b], kScaleWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b_tail);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_row_tiles =
      args.row_tiles != nullptr ? *args.num_row_tiles : (args.dense_rows + 127) / 128;
  const int total_tiles = num_row_tiles * args.n_tiles;
  const int k_mmas = args.K / 64;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += units) {
        const int rt = t / args.n_tiles;
        const int nt = t - rt * args.n_tiles;
        const TileRows rows = tile_rows_of<C>(args, rt, num_row_tiles, 0u);
        const int expert = rows.expert;
        const uint8_t* sfa_src =
            args.sfa + static_cast<size_t>(rows.load_row0 >> 7) * args.k_blocks * C::SFA_BYTES;
        const uint8_t* sfb_src = args.sfb + (static_cast<size_t>(expert) * args.n_tiles + nt) *
                                                args.k_blocks * C::SFB_BYTES;
        // weights are stored K-block-major: [expert][k block][row][128 B], then the
        // partial last K block as [expert][row][tail bytes]; a pair's CTA takes the
        // half of the tile's rows that belongs to its rank
        const int b_row = nt * C::BN;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
            report_timeout(args.error, abort_flag);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_bar[stage], C::STAGE_TX);
          tma_load_2d(sA + stage * C::A_BYTES, &tmap_a, kb * 128, rows.load_row0,
                      &full_bar[stage]);
          if (kb < args.kb_full) {
            // one contiguous, pre-swizzled panel slice: a single bulk copy
            bulk_load(sB + stage * C::B_BYTES,
                      args.b_full + (static_cast<size_t>(expert * args.kb_full + kb) * args.N +
                                     b_row) * 128,
                      C::B_BYTES, &full_bar[stage]);
          } else {
            tma_load_2d(sB + stage * C::B_BYTES, &tmap_b_tail, 0, expert * args.N + b_row,
                        &full_bar[stage]);
          }
          bulk_load(sSFA + stage * C::SFA_BYTES, sfa_src + kb * C::SFA_BYTES, C::SFA_BYTES,
                    &full_bar[stage]);
          bulk_load(sSFB + stage * C::SFB_BYTES, sfb_src + kb * C::SFB_BYTES, C::SFB_BYTES,
                    &full_bar[stage]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_nvf4(C::BN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      int sf_buf = 0;
      uint32_t sf_phase = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += units, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        // both CTAs' epilogues have drained this accumulator
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u)) {
          report_timeout(args.error, abort_flag);
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::ACC_STRIDE;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          // the operands have landed (in both CTAs) and the scale copies of this K
          // block are done
          // (a pair's full barrier counts the bytes of both CTAs)
          const bool landed = mbar_wait(&full_bar[stage], phase);
          if (!landed || !mbar_wait(&sf_ready_bar[sf_buf], sf_phase)) {
            report_timeout(args.error, abort_flag);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * C::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * C::B_BYTES);
          const uint32_t sf_tmem = tmem_base + sf_buf * C::SF_BUF_COLS;
          const int kt_count = min(4, k_mmas - kb * 4);
          if (kt_count == 4) {
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              tcgen05_mma_nvf4(d_tmem, make_smem_desc(a_addr + kt * 32, 0, 1024, 2),
                               make_smem_desc(b_addr + kt * 32, 0, 1024, 2), idesc,
                               sf_tmem + C::SFA_COL + 4 * kt,
                               sf_tmem + C::SFB_COL + C::SFB_GS * kt, (kb | kt) != 0 ? 1u : 0u);
            }
          } else {
            for (int kt = 0; kt < kt_count; ++kt) {
              tcgen05_mma_nvf4(d_tmem, make_smem_desc(a_addr + kt * 32, 0, 1024, 2),
                               make_smem_desc(b_addr + kt * 32, 0, 1024, 2), idesc,
                               sf_tmem + C::SFA_COL + 4 * kt,
                               sf_tmem + C::SFB_COL + C::SFB_GS * kt, (kb | kt) != 0 ? 1u : 0u);
            }
          }
          // frees the stage for the producer(s) and, SF_BUFS K blocks later, this
          // block's scale columns for the copier
          tcgen05_commit(&empty_bar[stage]);
          if (++sf_buf == C::SF_BUFS) {
            sf_buf = 0;
            sf_phase ^= 1u;
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          tcgen05_commit(&tmem_full_bar[acc]);
        }
      }
    }
  } else if (warp >= kScaleWarp) {
    if (lane == 0) {
    // ------------------------------------------------------- block-scale copier
    // The copies of one K block's scales into TMEM take longer to issue than
    // its MMAs; a thread of their own lets them run ahead of the MMA thread.
      const int part = warp - kScaleWarp;
      int stage = 0;
      uint32_t phase = 0;
      int sf_buf = 0;
      // the scale columns written now were last read by the MMAs of the K block
      // SF_BUFS iterations back; those MMAs also release that block's stage
      int old_stage = 0;
      uint32_t old_phase = 0;
      int iteration = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += units) {
        for (int kb = 0; kb < args.k_blocks; ++kb, ++iteration) {
          bool ready = true;
          if (iteration >= C::SF_BUFS) {
            ready = mbar_wait(&empty_bar[old_stage], old_phase);
            if (++old_stage == C::STAGES) {
              old_stage = 0;
              old_phase ^= 1u;
            }
          }
          ready = ready && mbar_wait(&full_bar[stage], phase);
          if (!ready) {
            report_timeout(args.error, abort_flag);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sfa_addr = smem_u32(sSFA + stage * C::SFA_BYTES);
          const uint32_t sfb_addr = smem_u32(sSFB + stage * C::SFB_BYTES);
          const uint32_t sf_tmem = tmem_base + sf_buf * C::SF_BUF_COLS;
          // a partial last K block needs the scales of the MMAs it issues only;
          // the full block keeps its copies free of run-time predicates, which
          // slow their issue down considerably
          const int kt_count = min(4, k_mmas - kb * 4);
          constexpr int kWeightCopiesPerMma = C::SFB_GS / 4;
          if (kt_count == 4) {
            static_assert(kScaleWarps == 2, "one branch per copier");
            if (part == 0) {
              issue_scale_copies<C, 0>(sf_tmem, sfa_addr, sfb_addr);
            } else {
              issue_scale_copies<C, 1>(sf_tmem, sfa_addr, sfb_addr);
            }
          } else {
            for (int c = part; c < kt_count; c += kScaleWarps) {
              scale_copy<C>(sf_tmem + C::SFA_COL + 4 * c,
                            make_smem_desc(sfa_addr + c * 512, 0, 128, 0));
            }
            for (int c = part; c < kt_count * kWeightCopiesPerMma; c += kScaleWarps) {
              scale_copy<C>(sf_tmem + C::SFB_COL + 4 * c,
                            make_smem_desc(sfb_addr + c * 512, 0, 128, 0));
            }
          }
          tcgen05_commit(&sf_ready_bar[sf_buf]);
          if (++sf_buf == C::SF_BUFS) sf_buf = 0;
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue
    const int quarter = warp & 3;           // TMEM lanes a warp may read: 32 * (warp % 4)
    const int half = (warp - 2) >> 2;       // which half of the tile's columns
    const int r = quarter * 32 + lane;      // row inside the tile == TMEM lane
    int local = 0;
    for (int t = unit; t < total_tiles; t += units, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      const int rt = t / args.n_tiles;
      const int nt = t - rt * args.n_tiles;
      const TileRows tile = tile_rows_of<C>(args, rt, num_row_tiles, 0u);
      const int row0 = tile.row0, rows = tile.rows, expert = tile.expert;
      const bool row_valid = r < rows;
      const int grow = row0 + r;
      float scale = args.w_tensor_scale[expert];
      if (args.a_tensor_scale != nullptr && row_valid) scale *= args.a_tensor_scale[grow];

      if (!mbar_wait(&tmem_full_bar[acc], acc_phase)) {
        report_timeout(args.error, abort_flag);
        break;
      }
      tcgen05_fence_after();
      const uint32_t t_addr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::ACC_STRIDE;
      const int n0 = nt * C::BN;
      // the two warps of a lane quarter split the tile's 16-column chunks
      constexpr int kChunks = C::BN / 16;
      const int chunk_begin = half == 0 ? 0 : (kChunks + 1) / 2;
      const int chunk_end = half == 0 ? (kChunks + 1) / 2 : kChunks;

      if constexpr (MODE == kGemmUp) {
        uint8_t* packed_row = args.out_packed + static_cast<size_t>(grow) * (args.N / 2);
        float row_max = 0.0f;
        for (int ch = chunk_begin; ch < chunk_end; ++ch) {
          const int n = n0 + ch * 16;
          if (n >= args.N) break;
          float v[16];
          tmem_ld_x16(t_addr + ch * 16, v);
          float amax = 0.0f;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float x = fmaxf(__fmul_rn(v[i], scale), 0.0f);  // Relu2: x > 0 ? x*x : 0
            v[i] = __fmul_rn(x, x);
            amax = fmaxf(amax, v[i]);
          }
          row_max = fmaxf(row_max, amax);
          uint32_t lo, hi;
          const uint32_t sf = quantize_block16_unit_scale(v, amax, lo, hi);
          if (row_valid) {
            *reinterpret_cast<uint2*>(packed_row + n / 2) = make_uint2(lo, hi);
            args.out_sf[swizzled_scale_offset(grow, n / 16, args.out_k_blocks * 4)] =
                static_cast<uint8_t>(sf);
          }
        }
        if (row_valid && row_max > kFp4Max * kFp8Max && args.error != nullptr) {
          atomicCAS(args.error, kDevOk, kDevActivationRange);
        }
      } else {
        // byte address of this row's output row (0 = nothing to store); with
        // out_segments it lies in the memory of the rank the row returns to
        unsigned long long dest = 0;
        float wt = 1.0f;
        if (row_valid) {
          const int d = args.dest_row != nullptr ? args.dest_row[grow]
                                                 : grow * args.dest_mul + args.dest_add;
          const size_t row_bytes = static_cast<size_t>(args.N) * (args.out_kind == kRowF32 ? 4 : 2);
          if (d >= 0) {
            if (args.out_segments != nullptr) {
              const int slot = d + args.segment_slot0;
              const int segment = slot / args.segment_rows;
              dest = args.out_segments[segment] +
                     static_cast<size_t>(slot - segment * args.segment_rows) * row_bytes;
            } else {
              dest = reinterpret_cast<unsigned long long>(args.out_rows) + d * row_bytes;
            }
          }
          if (args.row_weight != nullptr) wt = args.row_weight[grow];
        }
        // Each thread owns one output row of the tile, but a store instruction
        // should write whole lines: stage 32 columns of 32 rows in shared memory,
        // then let every 8 lanes write 128 contiguous bytes of one row (4 rows
        // per instruction).
        float* stage = stage_base + (warp - 2) * (32 * kStageStride);
        const int sub = lane >> 3;
        const int c4 = (lane & 7) * 4;
        for (int ch = chunk_begin; ch < chunk_end; ch += 2) {
          const int n = n0 + ch * 16;
          if (n >= args.N) break;
          const bool wide = ch + 1 < chunk_end && n + 16 < args.N;
          float va[16], vb[16];
          tmem_ld_x16(t_addr + ch * 16, va);
          if (wide) {
            tmem_ld_x16(t_addr + ch * 16 + 16, vb);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) vb[i] = 0.0f;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            va[i] = __fmul_rn(va[i], scale);
            vb[i] = __fmul_rn(vb[i], scale);
            if (args.row_weight != nullptr) {
              va[i] = __fmul_rn(va[i], wt);
              vb[i] = __fmul_rn(vb[i], wt);
            }
            if (args.relu2) {  // Relu2 (expert_layer.cpp:138-140): x > 0 ? x * x : 0
              const float pa = fmaxf(va[i], 0.0f), pb = fmaxf(vb[i], 0.0f);
              va[i] = __fmul_rn(pa, pa);
              vb[i] = __fmul_rn(pb, pb);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            *reinterpret_cast<float4*>(stage + lane * kStageStride + i) =
                make_float4(va[i], va[i + 1], va[i + 2], va[i + 3]);
            if (wide) {
              *reinterpret_cast<float4*>(stage + lane * kStageStride + 16 + i) =
                  make_float4(vb[i], vb[i + 1], vb[i + 2], vb[i + 3]);
            }
          }
          __syncwarp();
          const bool col_ok = c4 < (wide ? 32 : 16);
#pragma unroll 4
          for (int it = 0; it < 8; ++it) {
            const int rr = 4 * it + sub;
            const unsigned long long d = __shfl_sync(0xffffffffu, dest, rr);
            if (d != 0 && col_ok) {
              const float4 value = *reinterpret_cast<const float4*>(stage + rr * kStageStride + c4);
              if (args.out_kind == kRowBf16) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(value.x, value.y);
                const __nv_bfloat162 hi = __floats2bfloat162_rn(value.z, value.w);
                uint2 bits;
                bits.x = *reinterpret_cast<const uint32_t*>(&lo);
                bits.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(d + static_cast<size_t>(n + c4) * 2) = bits;
              } else if (args.out_kind == kRowF16) {
                // a value beyond binary16's 65504 becomes an infinity here; the combine
                // kernel reports it
                const __half2 lo = __floats2half2_rn(value.x, value.y);
                const __half2 hi = __floats2half2_rn(value.z, value.w);
                uint2 bits;
                bits.x = *reinterpret_cast<const uint32_t*>(&lo);
                bits.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(d + static_cast<size_t>(n + c4) * 2) = bits;
              } else {
                *reinterpret_cast<float4*>(d + static_cast<size_t>(n + c4) * 4) = value;
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tmem_empty_bar[acc]);
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  // neither CTA of a pair leaves while the other may still read its shared memory
  // or signal its barriers
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// CTA-pair kernel (kVariantPairUp / kVariantPairDown): one 256 x kPairBN tile per cluster
// of two CTAs (tcgen05.mma.cta_group::2, M = 256).
//
// What bounds the grouped GEMM at prefill sizes is the rate at which an SM can pull its
// operands from L2 into shared memory (measured: ~50-58 B per cycle per SM with every SM
// streaming), not the tensor pipe: a 128 x 208 tile stages 49 KB per 256-element K block
// for 416 cycles of MMA.  A pair stages each weight tile once for 256 rows (half in each
// CTA), 33 KB per CTA and K block for 352 cycles of MMA.
//
// Two more measurements shape the kernel.  A tcgen05.cp of 512 scale bytes costs ~47
// cycles of the tensor pipe alone and more while MMAs run, and the MMAs that need the
// scales queue behind it (12 copies per K block outweigh its four MMAs), so the scales go
// shared memory -> registers -> TMEM (tcgen05.st) from four warps per CTA, one per TMEM
// lane quarter, each CTA for its own TMEM.  And an mbarrier wait costs the waiting
// thread 100-250 cycles even when the phase has completed, so every role waits at most
// twice per K block and the scales rotate through three TMEM buffers.
//
// Roles per CTA: warp 0 loads (its own 128 activation rows, its half of the weight tile,
// the scales of its rows and of the whole weight tile), warp 1 of cluster rank 0 issues
// the MMAs for both, warps 2-9 run the epilogue of the CTA's 128 rows, warps 10-13 write
// scales.  Activation and weight bytes of BOTH CTAs complete on rank 0's full barrier
// (the loads name it; no multicast); scale bytes complete on a barrier of their own CTA.
// ---------------------------------------------------------------------------
constexpr int kPairBN = 176;
constexpr int kPairBRows = kPairBN / 2;        // weight rows staged per CTA
constexpr int kPairStages = 6;
constexpr int kPairSfBufs = 3;
constexpr int kPairScaleWarps = 4;             // one per TMEM lane quarter
constexpr int kPairThreads = (2 + kEpilogueWarps + kPairScaleWarps) * 32;
constexpr int kPairABytes = 128 * 128;
constexpr int kPairBBytes = kPairBRows * 128;
constexpr int kPairSfaBytes = 2048;
constexpr int kPairSfbGroups = 8;              // two groups of 128 weight rows x 4 MMAs
constexpr int kPairSfbBytes = kPairSfbGroups * 512;
constexpr int kPairStageBytes = kPairABytes + kPairBBytes + kPairSfaBytes + kPairSfbBytes;
constexpr int kPairSfCol = 2 * kPairBN;        // TMEM: two accumulators, then the scale buffers
constexpr int kPairSfBufCols = 16 + 4 * kPairSfbGroups;
constexpr int kPairBarBytes = ((3 * kPairStages + 4 + kPairSfBufs) * 8 + 16 + 15) / 16 * 16;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + kPairBarBytes + 1024;
static_assert(kPairSfCol + kPairSfBufs * kPairSfBufCols <= 512, "TMEM budget");
static_assert(kPairBRows % 8 == 0, "half a weight tile is whole 8-row swizzle groups");
static_assert(kPairBBytes % 1024 == 0, "stage regions keep the 1024-byte swizzle alignment");
static_assert(kPairSmemBytes <= 232448, "shared memory budget");

struct PairShape {  // what tile_rows_of reads
  static constexpr bool PAIR = true;
  static constexpr int BN = kPairBN;
};

template <int MODE>
__global__ void __launch_bounds__(kPairThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs args) {
  using C = PairShape;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) &
                                             ~static_cast<uintptr_t>(1023u));
  uint8_t* sA = smem;
  uint8_t* sB = sA + kPairStages * kPairABytes;
  uint8_t* sSFA = sB + kPairStages * kPairBBytes;
  uint8_t* sSFB = sSFA + kPairStages * kPairSfaBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sSFB + kPairStages * kPairSfbBytes);
  uint64_t* sf_full_bar = full_bar + kPairStages;   // this CTA's scale bytes landed
  uint64_t* empty_bar = sf_full_bar + kPairStages;  // both CTAs: the MMAs have read the stage
  uint64_t* tmem_full_bar = empty_bar + kPairStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint64_t* sf_ready_bar = tmem_empty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_ready_bar + kPairSfBufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0u;
  const int unit = static_cast<int>(blockIdx.x >> 1);
  const int units = static_cast<int>(gridDim.x >> 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&sf_full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 2 * kEpilogueWarps);
    }
    for (int b = 0; b < kPairSfBufs; ++b) mbar_init(&sf_ready_bar[b], 2 * kPairScaleWarps);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&maps.a);
    prefetch_tensormap(&maps.b_tail);
    prefetch_tensormap(&maps.b_full);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything arrives
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_row_tiles =
      args.row_tiles != nullptr ? *args.num_row_tiles : (args.dense_rows + 127) / 128;
  const int row_units = (num_row_tiles + 1) / 2;
  const int total_tiles = row_units * args.n_tiles;
  const int k_mmas = args.K / 64;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t leader_full0 = cluster_address_of(&full_bar[0], 0);
      for (int t = unit; t < total_tiles && ok; t += units) {
        const int rt = t / args.n_tiles;
        const int nt = t - rt * args.n_tiles;
        const TileRows rows = tile_rows_of<C>(args, rt, num_row_tiles, cta_rank);
        const int expert = rows.expert;
        const uint8_t* sfa_src =
            args.sfa + static_cast<size_t>(rows.load_row0 >> 7) * args.k_blocks * kPairSfaBytes;
        const uint8_t* sfb_src = args.sfb + (static_cast<size_t>(expert) * args.n_tiles + nt) *
                                                args.k_blocks * kPairSfbBytes;
        const int b_row = nt * kPairBN + static_cast<int>(cta_rank) * kPairBRows;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
            report_timeout(args.error, abort_flag);
            ok = false;
            break;
          }
          if (args.ablate & 4) {
            if (leader) mbar_arrive(&full_bar[stage]);
            mbar_arrive(&sf_full_bar[stage]);
          } else {
            // activation and weight bytes of both CTAs are counted on the leader's barrier
            const uint32_t bar = leader_full0 + static_cast<uint32_t>(stage) * 8u;
            if (leader) {
              mbar_arrive_expect_tx(&full_bar[stage], 2 * (kPairABytes + kPairBBytes));
            }
            mbar_arrive_expect_tx(&sf_full_bar[stage], kPairSfaBytes + kPairSfbBytes);
            tma_load_2d_pair(sA + stage * kPairABytes, &maps.a, kb * 128, rows.load_row0, bar);
            if (kb < args.kb_full) {
              tma_load_2d_pair(sB + stage * kPairBBytes, &maps.b_full, 0,
                               (expert * args.kb_full + kb) * args.N + b_row, bar);
            } else {
              tma_load_2d_pair(sB + stage * kPairBBytes, &maps.b_tail, 0, expert * args.N + b_row,
                               bar);
            }
            bulk_load(sSFA + stage * kPairSfaBytes, sfa_src + kb * kPairSfaBytes, kPairSfaBytes,
                      &sf_full_bar[stage]);
            bulk_load(sSFB + stage * kPairSfbBytes, sfb_src + kb * kPairSfbBytes, kPairSfbBytes,
                      &sf_full_bar[stage]);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_nvf4_pair(kPairBN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      int sf_buf = 0;
      uint32_t sf_phase = 0;
      bool ok = true;
      for (int t = unit; t < total_tiles && ok; t += units, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        // both CTAs' epilogues have drained this accumulator
        if (!mbar_wait_cluster(&tmem_empty_bar[acc], acc_phase ^ 1u)) {
          report_timeout(args.error, abort_flag);
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kPairBN;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          // the operands of both CTAs have landed and both have written this block's scales
          if (!mbar_wait_cluster(&full_bar[stage], phase) ||
              !mbar_wait_cluster(&sf_ready_bar[sf_buf], sf_phase)) {
            report_timeout(args.error, abort_flag);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * kPairABytes);
          const uint32_t b_addr = smem_u32(sB + stage * kPairBBytes);
          const uint32_t sf_tmem = tmem_base + kPairSfCol + sf_buf * kPairSfBufCols;
          const int kt_count = (args.ablate & 8) ? 0 : min(4, k_mmas - kb * 4);
          if (kt_count == 4) {
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              tcgen05_mma_pair_nvf4(d_tmem, make_smem_desc(a_addr + kt * 32, 0, 1024, 2),
                                    make_smem_desc(b_addr + kt * 32, 0, 1024, 2), idesc,
                                    sf_tmem + 4 * kt, sf_tmem + 16 + kPairSfbGroups * kt,
                                    (kb | kt) != 0 ? 1u : 0u);
            }
          } else {
            for (int kt = 0; kt < kt_count; ++kt) {
              tcgen05_mma_pair_nvf4(d_tmem, make_smem_desc(a_addr + kt * 32, 0, 1024, 2),
                                    make_smem_desc(b_addr + kt * 32, 0, 1024, 2), idesc,
                                    sf_tmem + 4 * kt, sf_tmem + 16 + kPairSfbGroups * kt,
                                    (kb | kt) != 0 ? 1u : 0u);
            }
          }
          // frees the stage in both CTAs and, kPairSfBufs K blocks later, this block's
          // scale columns
          tcgen05_commit_pair(&empty_bar[stage], 3);
          if (++sf_buf == kPairSfBufs) {
            sf_buf = 0;
            sf_phase ^= 1u;
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tcgen05_commit_pair(&tmem_full_bar[acc], 3);
      }
    }
  } else if (warp >= kScaleWarp) {
    // ------------------------------------------------------- block-scale writers
    // Each warp writes the same 32 x 16 B of every 512-byte chunk to its own lane
    // quarter: the layout a tcgen05.cp.32x128b.warpx4 produces.
    const int quarter = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    int stage = 0;
    uint32_t phase = 0;
    int sf_buf = 0;
    // the scale columns written now were last read by the MMAs of the K block kPairSfBufs
    // iterations back; those MMAs also release that block's stage
    int old_stage = 0;
    uint32_t old_phase = 0;
    int iteration = 0;
    bool ok = true;
    for (int t = unit; t < total_tiles && ok; t += units) {
      for (int kb = 0; kb < args.k_blocks; ++kb, ++iteration) {
        bool ready = true;
        if (iteration >= kPairSfBufs) {
          ready = mbar_wait(&empty_bar[old_stage], old_phase);
          if (++old_stage == kPairStages) {
            old_stage = 0;
            old_phase ^= 1u;
          }
        }
        ready = ready && mbar_wait(&sf_full_bar[stage], phase);
        if (!ready) {
          if (lane == 0) report_timeout(args.error, abort_flag);
          ok = false;
          break;
        }
        if (!(args.ablate & 2)) {
          tcgen05_fence_after();
          const uint32_t sf_tmem = tmem_base + lane_base + kPairSfCol + sf_buf * kPairSfBufCols;
          const uint4* sfa = reinterpret_cast<const uint4*>(sSFA + stage * kPairSfaBytes) + lane;
          const uint4* sfb = reinterpret_cast<const uint4*>(sSFB + stage * kPairSfbBytes) + lane;
          uint32_t row_words[16], lo_words[16], hi_words[16];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 q = sfa[c * 32];
            row_words[4 * c] = q.x;
            row_words[4 * c + 1] = q.y;
            row_words[4 * c + 2] = q.z;
            row_words[4 * c + 3] = q.w;
            const uint4 u = sfb[c * 32];
            lo_words[4 * c] = u.x;
            lo_words[4 * c + 1] = u.y;
            lo_words[4 * c + 2] = u.z;
            lo_words[4 * c + 3] = u.w;
            const uint4 v = sfb[(c + 4) * 32];
            hi_words[4 * c] = v.x;
            hi_words[4 * c + 1] = v.y;
            hi_words[4 * c + 2] = v.z;
            hi_words[4 * c + 3] = v.w;
          }
          tmem_st_x16(sf_tmem, row_words);
          tmem_st_x16(sf_tmem + 16, lo_words);
          tmem_st_x16(sf_tmem + 32, hi_words);
          tmem_st_wait();
          tcgen05_fence_before();
        }
        __syncwarp();
        if (lane == 0) {
          if (leader) {
            mbar_arrive(&sf_ready_bar[sf_buf]);
          } else {
            mbar_arrive_remote(&sf_ready_bar[sf_buf], 0);
          }
        }
        if (++sf_buf == kPairSfBufs) sf_buf = 0;
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue
    const int quarter = warp & 3;           // TMEM lanes a warp may read: 32 * (warp % 4)
    const int half = (warp - 2) >> 2;       // which part of the tile's 16-column chunks
    const int r = quarter * 32 + lane;      // row inside this CTA's 128 rows == TMEM lane
    constexpr int kChunks = kPairBN / 16;   // 11: six for the first warp of a quarter, five
    const int chunk_begin = half == 0 ? 0 : (kChunks + 1) / 2;
    const int chunk_end = half == 0 ? (kChunks + 1) / 2 : kChunks;
    int local = 0;
    for (int t = unit; t < total_tiles; t += units, ++local) {
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      const int rt = t / args.n_tiles;
      const int nt = t - rt * args.n_tiles;
      const TileRows tile = tile_rows_of<C>(args, rt, num_row_tiles, cta_rank);
      const int row0 = tile.row0, rows = tile.rows, expert = tile.expert;
      const bool row_valid = r < rows;
      const int grow = row0 + r;
      float scale = args.w_tensor_scale[expert];
      if (args.a_tensor_scale != nullptr && row_valid) scale *= args.a_tensor_scale[grow];
      // kGemmDown: byte address of this row's output row (0 = nothing to store); with
      // out_segments it lies in the memory of the rank the row returns to
      unsigned long long dest = 0;
      float wt = 1.0f;
      if (MODE == kGemmDown && row_valid) {
        const int d = args.dest_row != nullptr ? args.dest_row[grow]
                                               : grow * args.dest_mul + args.dest_add;
        const size_t row_bytes = static_cast<size_t>(args.N) * (args.out_kind == kRowF32 ? 4 : 2);
        if (d >= 0) {
          if (args.out_segments != nullptr) {
            const int slot = d + args.segment_slot0;
            const int segment = slot / args.segment_rows;
            dest = args.out_segments[segment] +
                   static_cast<size_t>(slot - segment * args.segment_rows) * row_bytes;
          } else {
            dest = reinterpret_cast<unsigned long long>(args.out_rows) + d * row_bytes;
          }
        }
        if (args.row_weight != nullptr) wt = args.row_weight[grow];
      }
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase)) {
        report_timeout(args.error, abort_flag);
        break;
      }
      tcgen05_fence_after();
      const uint32_t t_addr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kPairBN;
      const int n0 = nt * kPairBN;
      float row_max = 0.0f;
      // two batches of up to three chunks: three loads in flight, one wait; the
      // accumulator goes back to the MMA thread once the second batch is in registers
      // (columns past N hold accumulator garbage and are never stored)
#pragma unroll 1
      for (int batch = chunk_begin; batch < chunk_end; batch += 3) {
        uint32_t raw[3][16];
        const bool last = batch + 3 >= chunk_end;
        if (!(args.ablate & 1)) {
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            if (batch + j < chunk_end) tmem_ld_x16_async(t_addr + (batch + j) * 16, raw[j]);
          }
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 3; ++j) tmem_ld_fence(raw[j]);
        }
        if (last) {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (leader) {
              mbar_arrive(&tmem_empty_bar[acc]);
            } else {
              mbar_arrive_remote(&tmem_empty_bar[acc], 0);  // the leader waits for both CTAs
            }
          }
        }
        if (args.ablate & 1) continue;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const int n = n0 + (batch + j) * 16;
          if (batch + j >= chunk_end || n >= args.N) continue;
          float v[16];
          if constexpr (MODE == kGemmUp) {
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              // Relu2: x > 0 ? x*x : 0
              const float x = fmaxf(__fmul_rn(__uint_as_float(raw[j][i]), scale), 0.0f);
              v[i] = __fmul_rn(x, x);
              amax = fmaxf(amax, v[i]);
            }
            row_max = fmaxf(row_max, amax);
            uint32_t lo, hi;
            const uint32_t sf = quantize_block16_unit_scale(v, amax, lo, hi);
            if (row_valid) {
              uint8_t* packed_row = args.out_packed + static_cast<size_t>(grow) * (args.N / 2);
              *reinterpret_cast<uint2*>(packed_row + n / 2) = make_uint2(lo, hi);
              args.out_sf[swizzled_scale_offset(grow, n / 16, args.out_k_blocks * 4)] =
                  static_cast<uint8_t>(sf);
            }
          } else if (dest != 0) {
            // every thread stores its own row: 16 columns are 32 (16-bit rows) or 64
            // bytes, whole sectors either way
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              v[i] = __fmul_rn(__uint_as_float(raw[j][i]), scale);
              if (args.row_weight != nullptr) v[i] = __fmul_rn(v[i], wt);
              if (args.relu2) {  // Relu2 (expert_layer.cpp:138-140): x > 0 ? x * x : 0
                const float p = fmaxf(v[i], 0.0f);
                v[i] = __fmul_rn(p, p);
              }
            }
            if (args.out_kind == kRowF32) {
              float4* d = reinterpret_cast<float4*>(dest + static_cast<size_t>(n) * 4);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
              }
            } else {
              uint32_t w[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (args.out_kind == kRowBf16) {
                  const __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                  w[i] = *reinterpret_cast<const uint32_t*>(&two);
                } else {
                  // a value beyond binary16's 65504 becomes an infinity here; the combine
                  // kernel reports it
                  const __half2 two = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                  w[i] = *reinterpret_cast<const uint32_t*>(&two);
                }
              }
              uint4* d = reinterpret_cast<uint4*>(dest + static_cast<size_t>(n) * 2);
              d[0] = make_uint4(w[0], w[1], w[2], w[3]);
              d[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          }
        }
      }
      if (MODE == kGemmUp && row_valid && row_max > kFp4Max * kFp8Max && args.error != nullptr) {
        atomicCAS(args.error, kDevOk, kDevActivationRange);
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  // neither CTA leaves while the other may still signal its barriers
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <int MODE>
cudaError_t launch_pair(const GemmMaps& maps, const GemmArgs& args, int num_sms,
                        cudaStream_t stream) {
  auto kernel = grouped_gemm_pair_kernel<MODE>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(num_sms & ~1), 1, 1);
  config.blockDim = dim3(kPairThreads, 1, 1);
  config.dynamicSmemBytes = kPairSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 2;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, maps, args);
}

template <class C, int MODE>
cudaError_t launch_kernel(const GemmMaps& maps, const GemmArgs& args, int grid,
                          cudaStream_t stream) {
  auto kernel = grouped_gemm_kernel<C, MODE>;
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (err != cudaSuccess) return err;
  kernel<<<grid, kGemmThreads, C::SMEM_BYTES, stream>>>(maps, args);
  return cudaGetLastError();
}

template <class C>
cudaError_t launch_cfg(GemmMode mode, const GemmMaps& maps, const GemmArgs& args, int num_sms,
                       cudaStream_t stream) {
  // one persistent CTA per SM, fewer when there is less work
  int grid = num_sms;
  if (args.row_tiles == nullptr) {
    const int tiles = ((args.dense_rows + 127) / 128) * args.n_tiles;
    if (tiles < grid) grid = tiles;
  }
  if (grid < 1) grid = 1;
  if (mode == kGemmUp) {
    return launch_kernel<C, kGemmUp>(maps, args, grid, stream);
  } else if constexpr (C::ROW_STAGING) {
    return launch_kernel<C, kGemmDown>(maps, args, grid, stream);
  } else {
    return cudaErrorInvalidValue;  // this tile shape has no staging for the down epilogue
  }
}

template <class C>
GemmVariantInfo info_of() {
  return GemmVariantInfo{C::BN, C::A_ROWS, C::SFB_GS, C::SFB_BYTES, C::SMEM_BYTES, C::B_ROWS};
}

__global__ void relayout_weight_scales_kernel(const uint8_t* __restrict__ src, int experts, int N,
                                              int K, int bn, int gs, int n_tiles, int k_blocks,
                                              uint32_t* __restrict__ out, size_t words) {
  const int blocks_per_row = K / 16;
  for (size_t w = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; w < words;
       w += static_cast<size_t>(gridDim.x) * blockDim.x) {
    // word index = ((((e*n_tiles + nt)*k_blocks + kb)*gs + chunk)*32 + lane)*4 + j
    size_t rest = w;
    const int j = rest & 3;
    rest >>= 2;
    const int lane = rest & 31;
    rest >>= 5;
    const int chunk = rest % gs;
    rest /= gs;
    const int kb = rest % k_blocks;
    rest /= k_blocks;
    const int nt = rest % n_tiles;
    const int e = static_cast<int>(rest / n_tiles);
    const int col = chunk * 4 + j;  // TMEM column inside this K block
    const int kt = col / gs;        // K tile (64 elements) inside the K block
    const int g = col - kt * gs;    // 32-row group inside the N tile
    const int local_row = g * 32 + lane;
    const int n = nt * bn + local_row;
    uint32_t word = 0;
    if (local_row < bn && n < N) {
      const uint8_t* row = src + (static_cast<size_t>(e) * N + n) * blocks_per_row;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int block = (kb * 4 + kt) * 4 + b;
        if (block < blocks_per_row) word |= static_cast<uint32_t>(row[block]) << (8 * b);
      }
    }
    out[w] = word;
  }
}

// [experts][N][K/2] row-major -> K-block-major: full 128-byte K blocks as
// [expert][k block][row][128], the partial last block as [expert][row][tail_pitch].
__global__ void relayout_weight_packed_kernel(const uint4* __restrict__ src, int experts, int N,
                                              int row_chunks, int kb_full, int tail_pitch_chunks,
                                              uint4* __restrict__ dst_full,
                                              uint4* __restrict__ dst_tail, size_t chunks) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < chunks;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % row_chunks);  // 16-byte chunk inside the row
    const size_t row = i / row_chunks;               // expert * N + n
    const int n = static_cast<int>(row % N);
    const size_t e = row / N;
    const int kb = c >> 3;
    if (kb < kb_full) {
      // 16-byte chunk j of row n is stored at position j ^ (n % 8): the 128-byte
      // shared-memory swizzle, applied here once so that a plain bulk copy of a
      // panel slice lands in shared memory exactly as a swizzling tensor copy would
      dst_full[((e * kb_full + kb) * N + n) * 8 + ((c & 7) ^ (n & 7))] = src[i];
    } else {
      dst_tail[row * tail_pitch_chunks + (c - kb_full * 8)] = src[i];
    }
  }
}

}  // namespace

cudaError_t relayout_weight_packed(const uint8_t* row_major, int experts, int N, int K,
                                   int tail_pitch_bytes, uint8_t* full, uint8_t* tail,
                                   cudaStream_t stream) {
  const int row_chunks = K / 32;
  const size_t chunks = static_cast<size_t>(experts) * N * row_chunks;
  const int blocks = static_cast<int>(std::min<size_t>((chunks + 255) / 256, 148 * 32));
  relayout_weight_packed_kernel<<<blocks, 256, 0, stream>>>(
      reinterpret_cast<const uint4*>(row_major), experts, N, row_chunks, K / 256,
      tail_pitch_bytes / 16, reinterpret_cast<uint4*>(full), reinterpret_cast<uint4*>(tail),
      chunks);
  return cudaGetLastError();
}

GemmVariantInfo gemm_variant_info(GemmVariant v) {
  switch (v) {
    case kVariantPrefillUp: return info_of<CfgPrefillUp>();
    case kVariantPrefillDown: return info_of<CfgPrefillDown>();
    case kVariantDecode: return info_of<CfgDecode>();
    case kVariantDecodeWide: return info_of<CfgDecodeWide>();
    case kVariantPairUp:
    case kVariantPairDown:
      return GemmVariantInfo{kPairBN, 128, kPairSfbGroups, kPairSfbBytes, kPairSmemBytes,
                             kPairBRows};
    default: return GemmVariantInfo{0, 0, 0, 0, 0, 0};
  }
}

cudaError_t launch_grouped_gemm(GemmVariant v, GemmMode mode, const GemmMaps& maps,
                                const GemmArgs& args, int num_sms, cudaStream_t stream) {
  switch (v) {
    case kVariantPrefillUp: return launch_cfg<CfgPrefillUp>(mode, maps, args, num_sms, stream);
    case kVariantPrefillDown: return launch_cfg<CfgPrefillDown>(mode, maps, args, num_sms, stream);
    case kVariantDecode: return launch_cfg<CfgDecode>(mode, maps, args, num_sms, stream);
    case kVariantDecodeWide: return launch_cfg<CfgDecodeWide>(mode, maps, args, num_sms, stream);
    case kVariantPairUp:
    case kVariantPairDown:
      if (num_sms < 2) return cudaErrorInvalidValue;
      return mode == kGemmUp ? launch_pair<kGemmUp>(maps, args, num_sms, stream)
                             : launch_pair<kGemmDown>(maps, args, num_sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

size_t weight_scale_layout_bytes(int experts, int N, int K, int bn, int sfb_groups) {
  const size_t n_tiles = (N + bn - 1) / bn;
  const size_t k_blocks = (K + 255) / 256;
  return static_cast<size_t>(experts) * n_tiles * k_blocks * sfb_groups * 512;
}

cudaError_t relayout_weight_scales(const uint8_t* row_major, int experts, int N, int K, int bn,
                                   int sfb_groups, uint8_t* out, cudaStream_t stream) {
  const int n_tiles = (N + bn - 1) / bn;
  const int k_blocks = (K + 255) / 256;
  const size_t words = weight_scale_layout_bytes(experts, N, K, bn, sfb_groups) / 4;
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<size_t>((words + threads - 1) / threads, 65535));
  relayout_weight_scales_kernel<<<blocks, threads, 0, stream>>>(
      row_major, experts, N, K, bn, sfb_groups, n_tiles, k_blocks,
      reinterpret_cast<uint32_t*>(out), words);
  return cudaGetLastError();
}

}  // namespace nmoe
