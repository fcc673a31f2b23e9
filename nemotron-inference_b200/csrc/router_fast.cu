// Two-pass router for large token counts.
//
// The reference computes gate logits with a sequential DOUBLE accumulation on
// the host (runtime/src/backend/linear_op.cpp:97-118) and selects experts from
// them (runtime/src/backend/expert_layer.cpp:277-367).  Matching its selected
// index sets bit for bit needs logits that round like an FP64 sum, but FP64 for
// every (token, expert) pair costs more than the expert GEMMs.  So:
//
//  pass 1  all logits on the tensor cores.  The FP32 normalised activation
//          y = (x * inv_rms) * w is recomputed in the kernel from the layer input
//          (the same two roundings as the RMSNorm kernel), split into three bf16
//          terms (hi + mid + lo carries the full 24-bit significand) that go
//          straight into shared memory in the tensor core's 128-byte swizzle;
//          the gate is bf16, products are exact and accumulate in FP32
//          (tcgen05.mma.kind::f16, accumulator in TMEM).  Nothing but the layer
//          input is read per token: no FP32 copy of y, no bf16 planes in HBM;
//  pass 2  per token, every expert whose pass-1 choice score lies within
//          `tie_margin` of the top_k-th score is re-evaluated with the FP64 sum
//          and the selection runs on those exact values.
//
// If every pass-1 score is within tie_margin/2 of its exact value, the exact
// top-k set is contained in the candidates, so indices AND weights equal the
// all-FP64 path.  tie_margin is ~20x the largest pass-1 error measured.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

// ---------------------------------------------------------------------------
// pass 1: logits[128 tokens x E] per CTA
// ---------------------------------------------------------------------------
constexpr int kFastStages = 3;
constexpr int kFastBlockK = 64;                 // bf16 elements per 128-byte row
constexpr int kFastABytes = 3 * 128 * 128;      // three planes of 128 rows x 128 B
constexpr int kSplitWarps = 8;                  // warps that build the planes, then store
constexpr int kFastThreads = (2 + kSplitWarps) * 32;

__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// kind::f16 instruction descriptor: FP32 accumulate, bf16 x bf16, K-major, M=128
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// Eight consecutive input elements of one row as FP32.
template <bool BF16>
__device__ __forceinline__ void load_x8(const void* x, size_t index, float (&v)[8]) {
  if constexpr (BF16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(
        reinterpret_cast<const __nv_bfloat16*>(x) + index);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + index);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + index + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

template <bool IN_BF16>
__global__ void __launch_bounds__(kFastThreads, 1)
router_fast_logits_kernel(const void* __restrict__ x, const float* __restrict__ inv_rms,
                          const float* __restrict__ norm_weight,
                          const __grid_constant__ CUtensorMap tmap_gate, int rows, int experts,
                          int hidden, float* __restrict__ logits, int32_t* error) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) &
                                             ~static_cast<uintptr_t>(1023u));
  const int b_bytes = experts * 128;
  uint8_t* sA = smem;
  uint8_t* sB = sA + kFastStages * kFastABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + kFastStages * b_bytes);
  uint64_t* empty_bar = full_bar + kFastStages;
  uint64_t* done_bar = empty_bar + kFastStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * 128;
  const int k_blocks = hidden / kFastBlockK;
  const uint32_t tmem_cols = experts <= 32 ? 32 : experts <= 64 ? 64 : experts <= 128 ? 128 : 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kFastStages; ++s) {
      // the gate tile arrives by TMA (one arrive + bytes), the planes are written by
      // the split warps (one arrive each)
      mbar_init(&full_bar[s], 1 + kSplitWarps);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(done_bar, 1);
    fence_barrier_init();
    prefetch_tensormap(&tmap_gate);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
          if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
          break;
        }
        mbar_arrive_expect_tx(&full_bar[stage], b_bytes);
        tma_load_2d(sB + stage * b_bytes, &tmap_gate, kb * kFastBlockK, 0, &full_bar[stage]);
        if (++stage == kFastStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(static_cast<uint32_t>(experts));
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) {
          if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(sA + stage * kFastABytes);
        const uint32_t b_addr = smem_u32(sB + stage * b_bytes);
        // smallest terms first, so that they are not absorbed by a large partial sum
        for (int plane = 2; plane >= 0; --plane) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {  // K = 16 bf16 = 32 bytes per MMA
            tcgen05_mma_bf16(tmem_base,
                             make_smem_desc(a_addr + plane * (128 * 128) + ks * 32, 0, 1024, 2),
                             make_smem_desc(b_addr + ks * 32, 0, 1024, 2), idesc,
                             (kb != 0 || plane != 2 || ks != 0) ? 1u : 0u);
          }
        }
        tcgen05_commit(&empty_bar[stage]);
        if (++stage == kFastStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) tcgen05_commit(done_bar);
    }
  } else {
    // ------------------------------------------------- split warps, then epilogue
    // Thread s of the 256 owns 16-byte chunk (s % 8) of rows (s / 8) + 32 j, j = 0..3,
    // of every K block: eight threads read one row's 128 (bf16) or 256 (FP32) bytes
    // together and write the row's three 128-byte plane rows, chunk c of row r at
    // position c ^ (r % 8) (the tensor core's 128-byte swizzle).
    const int s = threadIdx.x - 64;
    const int chunk = s & 7;
    float rinv[4];
    int row_of[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      row_of[j] = (s >> 3) + 32 * j;
      const int row = row0 + row_of[j];
      rinv[j] = row < rows ? inv_rms[row] : 0.0f;
    }
    // two K blocks of input stay in flight in registers: a row's 128-byte pieces are
    // 5 KB apart in memory, so each fetch pays a full memory latency
    float xv[2][4][8];
    auto fetch = [&](int kb, float (&dst)[4][8]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = min(row0 + row_of[j], rows - 1);
        load_x8<IN_BF16>(x, static_cast<size_t>(row) * hidden + kb * kFastBlockK + chunk * 8,
                         dst[j]);
      }
    };
    fetch(0, xv[0]);
    if (k_blocks > 1) fetch(1, xv[1]);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb = 0; kb < k_blocks; ++kb) {
      const float4 w0 = *reinterpret_cast<const float4*>(norm_weight + kb * kFastBlockK + chunk * 8);
      const float4 w1 =
          *reinterpret_cast<const float4*>(norm_weight + kb * kFastBlockK + chunk * 8 + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      uint32_t words[4][3][4];
      auto split = [&](float (&src)[4][8]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            // y exactly as the RMSNorm kernel rounds it: (x * inv_rms) * w
            float rem[2] = {__fmul_rn(__fmul_rn(src[j][i], rinv[j]), w[i]),
                            __fmul_rn(__fmul_rn(src[j][i + 1], rinv[j]), w[i + 1])};
#pragma unroll
            for (int term = 0; term < 3; ++term) {
              const __nv_bfloat16 a = __float2bfloat16_rn(rem[0]);
              const __nv_bfloat16 b = __float2bfloat16_rn(rem[1]);
              rem[0] = __fsub_rn(rem[0], __bfloat162float(a));
              rem[1] = __fsub_rn(rem[1], __bfloat162float(b));
              words[j][term][i / 2] = static_cast<uint32_t>(__bfloat16_as_ushort(a)) |
                                      (static_cast<uint32_t>(__bfloat16_as_ushort(b)) << 16);
            }
          }
        }
      };
      // (the buffer index is resolved at compile time: registers cannot be indexed)
      if (kb & 1) {
        split(xv[1]);
        if (kb + 2 < k_blocks) fetch(kb + 2, xv[1]);
      } else {
        split(xv[0]);
        if (kb + 2 < k_blocks) fetch(kb + 2, xv[0]);
      }
      if (ok && !mbar_wait(&empty_bar[stage], phase ^ 1u)) {
        if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
        ok = false;
      }
      if (ok) {
        uint8_t* planes = sA + stage * kFastABytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = row_of[j];
          const int offset = r * 128 + ((chunk ^ (r & 7)) << 4);
#pragma unroll
          for (int term = 0; term < 3; ++term) {
            *reinterpret_cast<uint4*>(planes + term * (128 * 128) + offset) =
                make_uint4(words[j][term][0], words[j][term][1], words[j][term][2],
                           words[j][term][3]);
          }
        }
        fence_proxy_async_smem();  // the tensor core reads these stores
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
      }
      if (++stage == kFastStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    // epilogue: the first four split warps own one TMEM lane quarter each
    if (warp < 6) {
      const int quarter = warp & 3;
      const int row = row0 + quarter * 32 + lane;
      if (ok && mbar_wait(done_bar, 0)) {
        tcgen05_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        for (int c = 0; c < experts; c += 16) {
          float v[16];
          tmem_ld_x16(t_addr + c, v);
          if (row < rows) {
            float* dst = logits + static_cast<size_t>(row) * experts + c;
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
          }
        }
      } else if (error != nullptr) {
        atomicCAS(error, kDevOk, kDevWaitTimeout);
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------------------
// pass 1 for bf16 layer inputs: the RMSNorm weight is folded into the gate once,
//   logit[t][e] ~= inv_rms[t] * sum_i x[t][i] * (w[i] * gate[e][i]),
// so the bf16 input itself is the (exact, single-term) A operand, loaded by TMA, and
// the three bf16 terms of fl32(w[i] * gate[e][i]) are the B operands, split once when
// the layer is created.  Same three MMAs per K step as the kernel above, but no warp
// touches the operands: one producer lane, one MMA lane, four epilogue warps.  Against
// the reference's y = fl(fl(x * inv_rms) * w) this drops two roundings of 2^-24 per term,
// the size of the FP32 accumulation error already covered by the tie margin.
// ---------------------------------------------------------------------------
constexpr int kFoldThreads = 6 * 32;
constexpr int kFoldMaxSplits = 4;
constexpr int kFoldABytes = 128 * 128;  // 128 rows x 64 bf16

__global__ void fold_gate_kernel(const __nv_bfloat16* __restrict__ gate,
                                 const float* __restrict__ norm_weight, int experts, int hidden,
                                 __nv_bfloat16* __restrict__ planes) {
  const size_t total = static_cast<size_t>(experts) * hidden;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float rem = __fmul_rn(norm_weight[i % hidden], __bfloat162float(gate[i]));
#pragma unroll
    for (int term = 0; term < 3; ++term) {
      const __nv_bfloat16 part = __float2bfloat16_rn(rem);
      rem = __fsub_rn(rem, __bfloat162float(part));
      planes[term * total + i] = part;
    }
  }
}

__global__ void __launch_bounds__(kFoldThreads, 1)
router_folded_logits_kernel(const __grid_constant__ CUtensorMap tmap_x,
                            const __grid_constant__ CUtensorMap tmap_planes,
                            const float* __restrict__ inv_rms, int rows, int experts, int hidden,
                            int stages, int splits, float* __restrict__ logits, int32_t* error) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) &
                                             ~static_cast<uintptr_t>(1023u));
  const int plane_bytes = experts * 128;
  const int b_bytes = 3 * plane_bytes;
  uint8_t* sA = smem;
  uint8_t* sB = sA + stages * kFoldABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + stages * b_bytes);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* done_bar = empty_bar + stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // With few row tiles the contraction is split over `splits` CTAs per tile (split s
  // writes its partial sums to logits + s * rows * experts; pass 2 adds them up), so that
  // a batch of a few thousand tokens still spreads over the SMs.
  const int tile = static_cast<int>(blockIdx.x) / splits;
  const int split = static_cast<int>(blockIdx.x) - tile * splits;
  const int row0 = tile * 128;
  const int all_k_blocks = hidden / kFastBlockK;
  const int kb_begin = all_k_blocks * split / splits;
  const int k_blocks = all_k_blocks * (split + 1) / splits - kb_begin;
  const uint32_t tmem_cols = experts <= 32 ? 32 : experts <= 64 ? 64 : experts <= 128 ? 128 : 256;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(done_bar, 1);
    fence_barrier_init();
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_planes);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
          if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
          break;
        }
        mbar_arrive_expect_tx(&full_bar[stage], kFoldABytes + b_bytes);
        // rows past the end of the input read as zeros (the map's extent is `rows`)
        tma_load_2d(sA + stage * kFoldABytes, &tmap_x, (kb_begin + kb) * kFastBlockK, row0,
                    &full_bar[stage]);
        for (int plane = 0; plane < 3; ++plane) {
          tma_load_2d(sB + stage * b_bytes + plane * plane_bytes, &tmap_planes,
                      (kb_begin + kb) * kFastBlockK, plane * experts, &full_bar[stage]);
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(static_cast<uint32_t>(experts));
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase)) {
          if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(sA + stage * kFoldABytes);
        const uint32_t b_addr = smem_u32(sB + stage * b_bytes);
        // smallest terms first, so that they are not absorbed by a large partial sum
        for (int plane = 2; plane >= 0; --plane) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {  // K = 16 bf16 = 32 bytes per MMA
            tcgen05_mma_bf16(tmem_base, make_smem_desc(a_addr + ks * 32, 0, 1024, 2),
                             make_smem_desc(b_addr + plane * plane_bytes + ks * 32, 0, 1024, 2),
                             idesc, (kb != 0 || plane != 2 || ks != 0) ? 1u : 0u);
          }
        }
        tcgen05_commit(&empty_bar[stage]);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) tcgen05_commit(done_bar);
    }
  } else {
    // epilogue: warp w owns TMEM lane quarter w % 4
    const int quarter = warp & 3;
    const int row = row0 + quarter * 32 + lane;
    const float rinv = row < rows ? inv_rms[row] : 0.0f;
    if (mbar_wait(done_bar, 0)) {
      tcgen05_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      for (int c = 0; c < experts; c += 16) {
        float v[16];
        tmem_ld_x16(t_addr + c, v);
        if (row < rows) {
          float* dst = logits + (static_cast<size_t>(split) * rows + row) * experts + c;
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            *reinterpret_cast<float4*>(dst + i) =
                make_float4(v[i] * rinv, v[i + 1] * rinv, v[i + 2] * rinv, v[i + 3] * rinv);
          }
        }
      }
    } else if (error != nullptr) {
      atomicCAS(error, kDevOk, kDevWaitTimeout);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------------------
// pass 2: candidates -> FP64 logits -> exact selection
// ---------------------------------------------------------------------------
constexpr int kSelectWarps = 4;
constexpr int kSelectPerLane = 8;  // experts <= 256

__device__ __forceinline__ float sigmoid_exact(float v) {
  // Sigmoid of expert_layer.cpp:129-136 with exp evaluated in double
  if (v >= 0.0f) {
    const float e = static_cast<float>(exp(-static_cast<double>(v)));
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
  }
  const float e = static_cast<float>(exp(static_cast<double>(v)));
  return __fdiv_rn(e, __fadd_rn(1.0f, e));
}

// Order-preserving map of a float onto unsigned integers (0 is below every value), so
// that a warp-wide maximum is one redux instruction.
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// The largest key of the warp and, among its holders, the smallest index
// (SelectTopExperts ranks by value; ties resolve to the lower expert index).
__device__ __forceinline__ void warp_arg_max(uint32_t key, uint32_t index, uint32_t& best_key,
                                             uint32_t& best_index) {
  best_key = __reduce_max_sync(0xffffffffu, key);
  best_index = __reduce_min_sync(0xffffffffu, key == best_key ? index : 0xffffffffu);
}

// One warp per token.  The FP64 dot products dominate; everything around them is kept
// to a few warp-wide redux steps per selected expert.
constexpr int kSelectBatch = 4;
template <bool IN_BF16>
__global__ void __launch_bounds__(kSelectWarps * 32, 8)
router_select_exact_kernel(float* __restrict__ logits, int splits, const void* __restrict__ x,
                           const float* __restrict__ inv_rms,
                           const float* __restrict__ norm_weight,
                           const __nv_bfloat16* __restrict__ gate,
                           const float* __restrict__ logit_offset, const float* __restrict__ bias,
                           int rows, int experts, int hidden, int top_k, bool norm_topk_prob,
                           float routed_scaling, float tie_margin,
                           int32_t* __restrict__ top_index, float* __restrict__ top_weight,
                           int32_t* __restrict__ expert_counts) {
  __shared__ int16_t candidate_list[kSelectWarps][256];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * kSelectWarps + warp;
  if (row >= rows) return;
  const int per_lane = experts / 32;
  float* row_logits = logits + static_cast<size_t>(row) * experts;

  // pass-1 choice scores (single precision is enough here: the margin covers it);
  // lane L holds experts L, L + 32, ...
  float choice[kSelectPerLane];
  uint32_t key[kSelectPerLane];
#pragma unroll
  for (int j = 0; j < kSelectPerLane; ++j) {
    choice[j] = -INFINITY;
    key[j] = 0u;
    if (j < per_lane) {
      const int e = lane + 32 * j;
      float l = row_logits[e];
      // partial sums of a split pass 1, in split order
      for (int sp = 1; sp < splits; ++sp) {
        l = __fadd_rn(l, row_logits[static_cast<size_t>(sp) * rows * experts + e]);
      }
      if (logit_offset != nullptr) l = __fadd_rn(l, logit_offset[e]);
      if (logit_offset != nullptr || splits > 1) {
        row_logits[e] = l;  // what the trace shows for experts that are not re-evaluated
      }
      choice[j] = __fdividef(1.0f, 1.0f + __expf(-l)) + bias[e];
      key[j] = ordered_bits(choice[j]);
    }
  }
  // the top_k-th largest pass-1 choice
  uint32_t kth_key = 0u;
  for (int r = 0; r < top_k; ++r) {
    uint32_t local_key = 0u, local_index = 0xffffffffu;
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j) {
      if (key[j] > local_key) {  // ascending j is ascending expert index: first maximum wins
        local_key = key[j];
        local_index = static_cast<uint32_t>(lane + 32 * j);
      }
    }
    uint32_t best_index;
    warp_arg_max(local_key, local_index, kth_key, best_index);
    if ((best_index & 31u) == static_cast<uint32_t>(lane)) {
#pragma unroll
      for (int j = 0; j < kSelectPerLane; ++j) {
        if (j == static_cast<int>(best_index >> 5)) key[j] = 0u;  // taken
      }
    }
  }
  // candidates: everything that could still be in the exact top-k
  float kth = 0.0f;
  {
    const uint32_t b = (kth_key & 0x80000000u) ? (kth_key & 0x7fffffffu) : ~kth_key;
    kth = __uint_as_float(b);
  }
  const float threshold = kth - tie_margin;
  uint32_t mine = 0;
#pragma unroll
  for (int j = 0; j < kSelectPerLane; ++j) {
    if (j < per_lane && choice[j] >= threshold) mine |= 1u << j;
  }
  const int my_count = __popc(mine);
  int prefix = my_count;
#pragma unroll
  for (int stride = 1; stride < 32; stride <<= 1) {
    const int other = __shfl_up_sync(0xffffffffu, prefix, stride);
    if (lane >= stride) prefix += other;
  }
  const int total = __shfl_sync(0xffffffffu, prefix, 31);
  int offset = prefix - my_count;
#pragma unroll
  for (int j = 0; j < kSelectPerLane; ++j) {
    if ((mine >> j) & 1u) candidate_list[warp][offset++] = static_cast<int16_t>(lane + 32 * j);
  }
  __syncwarp();

  // FP64 logits of the candidates, up to kSelectBatch at a time; every lane takes
  // eight consecutive hidden elements per step.  y is rebuilt from the layer input with
  // the RMSNorm kernel's own two roundings: (x * inv_rms) * w.
  const float rinv = inv_rms[row];
  const int chunks = hidden / 8;
  constexpr int kBatch = kSelectBatch;
  for (int base = 0; base < total; base += kBatch) {
    const int batch = min(kBatch, total - base);
    int e[kBatch];
    double acc[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      e[i] = candidate_list[warp][min(base + i, total - 1)];
      acc[i] = 0.0;
    }
    for (int ch = lane; ch < chunks; ch += 32) {
      float xv[8];
      load_x8<IN_BF16>(x, static_cast<size_t>(row) * hidden + ch * 8, xv);
      const float4 w0 = *reinterpret_cast<const float4*>(norm_weight + ch * 8);
      const float4 w1 = *reinterpret_cast<const float4*>(norm_weight + ch * 8 + 4);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      double a[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        a[i] = static_cast<double>(__fmul_rn(__fmul_rn(xv[i], rinv), w[i]));
      }
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (i < batch) {
          const uint4 g = *reinterpret_cast<const uint4*>(gate + static_cast<size_t>(e[i]) * hidden +
                                                          ch * 8);
          const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[i] = fma(a[2 * j], static_cast<double>(__uint_as_float(gw[j] << 16)), acc[i]);
            acc[i] = fma(a[2 * j + 1], static_cast<double>(__uint_as_float(gw[j] & 0xffff0000u)),
                         acc[i]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (i < batch) {
        double v = acc[i];
#pragma unroll
        for (int stride = 16; stride > 0; stride >>= 1) v += __shfl_xor_sync(0xffffffffu, v, stride);
        if (lane == 0) {
          float logit = static_cast<float>(v);
          if (logit_offset != nullptr) logit = __fadd_rn(logit, logit_offset[e[i]]);
          row_logits[e[i]] = logit;
        }
      }
    }
  }
  __syncwarp();

  // exact scores, compacted: lane L takes candidates L, L + 32, ... of the list, so the
  // double-precision exponential runs once per lane instead of once per expert slot
  float score[kSelectPerLane];
  uint32_t cand_key[kSelectPerLane];
  int cand_expert[kSelectPerLane];
  const int rounds = (total + 31) / 32;
#pragma unroll
  for (int j = 0; j < kSelectPerLane; ++j) {
    score[j] = 0.0f;
    cand_key[j] = 0u;
    cand_expert[j] = -1;
    if (j < rounds) {
      const int slot = lane + 32 * j;
      if (slot < total) {
        const int ex = candidate_list[warp][slot];
        const float l = *reinterpret_cast<volatile float*>(row_logits + ex);
        score[j] = sigmoid_exact(l);
        cand_key[j] = ordered_bits(__fadd_rn(score[j], bias[ex]));
        cand_expert[j] = ex;
      }
    }
  }
  int my_index = -1;
  float my_score = 0.0f;
  for (int r = 0; r < top_k; ++r) {
    uint32_t local_key = 0u, local_index = 0xffffffffu;
    float local_score = 0.0f;
    int local_slot = -1;
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j) {
      const uint32_t ex = static_cast<uint32_t>(cand_expert[j]);
      if (cand_key[j] > local_key || (cand_key[j] == local_key && cand_key[j] != 0u &&
                                      ex < local_index)) {
        local_key = cand_key[j];
        local_index = ex;
        local_score = score[j];
        local_slot = j;
      }
    }
    uint32_t best_key, best_index;
    warp_arg_max(local_key, local_index, best_key, best_index);
    const bool owner = local_key == best_key && local_index == best_index && local_slot >= 0;
    const int owner_lane = __ffs(__ballot_sync(0xffffffffu, owner)) - 1;
    const float s = __shfl_sync(0xffffffffu, local_score, owner_lane < 0 ? 0 : owner_lane);
    if (owner) {
#pragma unroll
      for (int j = 0; j < kSelectPerLane; ++j) {
        if (j == local_slot) cand_key[j] = 0u;  // taken
      }
    }
    if (lane == r) {
      my_index = static_cast<int>(best_index);
      my_score = s;
    }
  }
  float weight_sum = 0.0f;
  for (int r = 0; r < top_k; ++r) {
    weight_sum = __fadd_rn(weight_sum, __shfl_sync(0xffffffffu, my_score, r));
  }
  if (lane < top_k) {
    float w = my_score;
    if (norm_topk_prob) w = __fdiv_rn(w, __fadd_rn(weight_sum, 1.0e-20f));
    w = __fmul_rn(w, routed_scaling);
    top_index[static_cast<size_t>(row) * top_k + lane] = my_index;
    top_weight[static_cast<size_t>(row) * top_k + lane] = w;
    if (expert_counts != nullptr) atomicAdd(&expert_counts[my_index], 1);
  }
}

}  // namespace

cudaError_t launch_router_fast_logits(const void* x, bool x_bf16, const float* inv_rms,
                                      const float* norm_weight, const CUtensorMap& tmap_gate,
                                      int rows, int experts, int hidden, float* logits,
                                      int32_t* error, cudaStream_t stream) {
  if (rows <= 0 || experts % 16 != 0 || experts > 256 || hidden % kFastBlockK != 0) {
    return cudaErrorInvalidValue;
  }
  const int smem = kFastStages * (kFastABytes + experts * 128) + (2 * kFastStages + 1) * 8 + 16 + 1024;
  const int grid = (rows + 127) / 128;
  cudaError_t err;
  if (x_bf16) {
    err = cudaFuncSetAttribute(router_fast_logits_kernel<true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    router_fast_logits_kernel<true><<<grid, kFastThreads, smem, stream>>>(
        x, inv_rms, norm_weight, tmap_gate, rows, experts, hidden, logits, error);
  } else {
    err = cudaFuncSetAttribute(router_fast_logits_kernel<false>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return err;
    router_fast_logits_kernel<false><<<grid, kFastThreads, smem, stream>>>(
        x, inv_rms, norm_weight, tmap_gate, rows, experts, hidden, logits, error);
  }
  return cudaGetLastError();
}

cudaError_t launch_fold_gate(const __nv_bfloat16* gate, const float* norm_weight, int experts,
                             int hidden, __nv_bfloat16* planes, cudaStream_t stream) {
  if (experts <= 0 || hidden <= 0) return cudaErrorInvalidValue;
  fold_gate_kernel<<<148 * 4, 256, 0, stream>>>(gate, norm_weight, experts, hidden, planes);
  return cudaGetLastError();
}

int router_folded_splits(int rows, int hidden, int num_sms) {
  const int tiles = (rows + 127) / 128;
  int splits = 1;
  while (splits < kFoldMaxSplits && tiles * splits * 2 <= num_sms &&
         hidden / kFastBlockK >= 8 * splits) {
    splits *= 2;
  }
  return splits;
}

cudaError_t launch_router_folded_logits(const CUtensorMap& tmap_x, const CUtensorMap& tmap_planes,
                                        const float* inv_rms, int rows, int experts, int hidden,
                                        int splits, float* logits, int32_t* error,
                                        cudaStream_t stream) {
  if (rows <= 0 || experts % 16 != 0 || experts > 256 || hidden % kFastBlockK != 0 ||
      splits < 1 || splits > kFoldMaxSplits || hidden / kFastBlockK < splits) {
    return cudaErrorInvalidValue;
  }
  const int stage_bytes = kFoldABytes + 3 * experts * 128;
  const int stages = std::min(4, (220 * 1024) / stage_bytes);
  if (stages < 2) return cudaErrorInvalidValue;
  const int smem = stages * stage_bytes + (2 * stages + 1) * 8 + 16 + 1024;
  cudaError_t err = cudaFuncSetAttribute(router_folded_logits_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  router_folded_logits_kernel<<<((rows + 127) / 128) * splits, kFoldThreads, smem, stream>>>(
      tmap_x, tmap_planes, inv_rms, rows, experts, hidden, stages, splits, logits, error);
  return cudaGetLastError();
}

cudaError_t launch_router_select_exact(float* logits, int splits, const void* x, bool x_bf16,
                                       const float* inv_rms, const float* norm_weight,
                                       const __nv_bfloat16* gate, const float* logit_offset,
                                       const float* bias, int rows, int experts, int hidden,
                                       int top_k, bool norm_topk_prob, float routed_scaling,
                                       float tie_margin, int32_t* top_index, float* top_weight,
                                       int32_t* expert_counts, cudaStream_t stream) {
  if (rows <= 0 || experts % 32 != 0 || experts > 32 * kSelectPerLane || top_k <= 0 ||
      top_k > 32 || top_k > experts || hidden % 8 != 0 || splits < 1) {
    return cudaErrorInvalidValue;
  }
  const int grid = (rows + kSelectWarps - 1) / kSelectWarps;
  if (x_bf16) {
    router_select_exact_kernel<true><<<grid, kSelectWarps * 32, 0, stream>>>(
        logits, splits, x, inv_rms, norm_weight, gate, logit_offset, bias, rows, experts, hidden, top_k,
        norm_topk_prob, routed_scaling, tie_margin, top_index, top_weight, expert_counts);
  } else {
    router_select_exact_kernel<false><<<grid, kSelectWarps * 32, 0, stream>>>(
        logits, splits, x, inv_rms, norm_weight, gate, logit_offset, bias, rows, experts, hidden, top_k,
        norm_topk_prob, routed_scaling, tie_margin, top_index, top_weight, expert_counts);
  }
  return cudaGetLastError();
}

}  // namespace nmoe
