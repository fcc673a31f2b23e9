// Two-pass router for large token counts.
//
// The reference computes gate logits with a sequential DOUBLE accumulation on
// the host (runtime/src/backend/linear_op.cpp:97-118) and selects experts from
// them (runtime/src/backend/expert_layer.cpp:277-367).  Matching its selected
// index sets bit for bit needs logits that round like an FP64 sum, but FP64 for
// every (token, expert) pair costs more than the expert GEMMs.  So:
//
//  pass 1  all logits on the tensor cores: the FP32 normalised activations are
//          split into three bf16 terms (hi + mid + lo carries the full 24-bit
//          significand), the gate is bf16, products are exact and accumulate in
//          FP32 (tcgen05.mma.kind::f16, TMA-fed, accumulator in TMEM);
//  pass 2  per token, every expert whose pass-1 choice score lies within
//          `tie_margin` of the top_k-th score is re-evaluated with the FP64 sum
//          and the selection runs on those exact values.
//
// If every pass-1 score is within tie_margin/2 of its exact value, the exact
// top-k set is contained in the candidates, so indices AND weights equal the
// all-FP64 path.  tie_margin is ~20x the largest pass-1 error measured.
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
constexpr int kFastThreads = 192;

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

__global__ void __launch_bounds__(kFastThreads, 1)
router_fast_logits_kernel(const __grid_constant__ CUtensorMap tmap_split,
                          const __grid_constant__ CUtensorMap tmap_gate, int rows,
                          int split_plane_rows, int experts, int hidden, float* __restrict__ logits,
                          int32_t* error) {
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
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(done_bar, 1);
    fence_barrier_init();
    prefetch_tensormap(&tmap_split);
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
        mbar_arrive_expect_tx(&full_bar[stage], kFastABytes + b_bytes);
        for (int plane = 0; plane < 3; ++plane) {
          tma_load_2d(sA + stage * kFastABytes + plane * (128 * 128), &tmap_split,
                      kb * kFastBlockK, plane * split_plane_rows + row0, &full_bar[stage]);
        }
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
    const int quarter = warp & 3;
    const int row = row0 + quarter * 32 + lane;
    if (mbar_wait(done_bar, 0)) {
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

struct Pick {
  float value;
  int index;
};

__device__ __forceinline__ Pick better_pick(Pick a, Pick b) {
  if (b.index < 0) return a;
  if (a.index < 0) return b;
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ __forceinline__ Pick warp_pick(Pick mine) {
#pragma unroll
  for (int stride = 16; stride > 0; stride >>= 1) {
    Pick other;
    other.value = __shfl_xor_sync(0xffffffffu, mine.value, stride);
    other.index = __shfl_xor_sync(0xffffffffu, mine.index, stride);
    mine = better_pick(mine, other);
  }
  return mine;
}

// One warp per token runs a long dependent chain (two top-k searches, the FP64 dot
// products, their reductions), so the kernel lives on occupancy: at most 64 registers
// per thread (8 blocks of 4 warps per SM) and four candidates per FP64 batch.
constexpr int kSelectBatch = 4;
__global__ void __launch_bounds__(kSelectWarps * 32, 8)
router_select_exact_kernel(float* __restrict__ logits, const float* __restrict__ normalized,
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

  // pass-1 scores (single precision is enough here: the margin covers it)
  float fast_logit[kSelectPerLane];
  float choice[kSelectPerLane];
#pragma unroll
  for (int j = 0; j < kSelectPerLane; ++j) {
    fast_logit[j] = 0.0f;
    choice[j] = -INFINITY;
    if (j < per_lane) {
      const int e = lane + 32 * j;
      float l = row_logits[e];
      if (logit_offset != nullptr) l = __fadd_rn(l, logit_offset[e]);
      fast_logit[j] = l;
      choice[j] = __fdividef(1.0f, 1.0f + __expf(-l)) + bias[e];
    }
  }
  // top_k-th largest pass-1 choice
  uint32_t taken = 0;
  float kth = 0.0f;
  for (int r = 0; r < top_k; ++r) {
    Pick local;
    local.index = -1;
    local.value = 0.0f;
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j) {
      if (j < per_lane && ((taken >> j) & 1u) == 0u) {
        Pick cand;
        cand.value = choice[j];
        cand.index = lane + 32 * j;
        local = better_pick(local, cand);
      }
    }
    const Pick b = warp_pick(local);
    if ((b.index & 31) == lane) taken |= 1u << (b.index >> 5);
    kth = b.value;
  }
  // candidates: everything that could still be in the exact top-k
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
  // eight consecutive hidden elements per step (16-byte gate loads)
  const float* y = normalized + static_cast<size_t>(row) * hidden;
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
      const float4 y0 = *reinterpret_cast<const float4*>(y + ch * 8);
      const float4 y1 = *reinterpret_cast<const float4*>(y + ch * 8 + 4);
      const double a[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        if (i < batch) {
          const uint4 g = *reinterpret_cast<const uint4*>(gate + static_cast<size_t>(e[i]) * hidden +
                                                          ch * 8);
          const uint32_t w[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[i] = fma(a[2 * j], static_cast<double>(__uint_as_float(w[j] << 16)), acc[i]);
            acc[i] = fma(a[2 * j + 1], static_cast<double>(__uint_as_float(w[j] & 0xffff0000u)),
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

  // exact scores of the candidates; everything else is out of the running
  float score[kSelectPerLane];
#pragma unroll
  for (int j = 0; j < kSelectPerLane; ++j) {
    score[j] = 0.0f;
    if (j < per_lane) {
      const int ex = lane + 32 * j;
      if ((mine >> j) & 1u) {
        const float l = *reinterpret_cast<volatile float*>(row_logits + ex);
        score[j] = sigmoid_exact(l);
        choice[j] = __fadd_rn(score[j], bias[ex]);
      } else {
        row_logits[ex] = fast_logit[j];  // pass-1 value (with the offset) for the trace
      }
    }
  }
  taken = ~mine;  // non-candidates are never picked
  int my_index = -1;
  float my_score = 0.0f;
  for (int r = 0; r < top_k; ++r) {
    Pick local;
    local.index = -1;
    local.value = 0.0f;
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j) {
      if (j < per_lane && ((taken >> j) & 1u) == 0u) {
        Pick cand;
        cand.value = choice[j];
        cand.index = lane + 32 * j;
        local = better_pick(local, cand);
      }
    }
    const Pick b = warp_pick(local);
    const int owner = b.index & 31;
    const int slot = b.index >> 5;
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kSelectPerLane; ++j)
      if (j == slot) s = score[j];
    s = __shfl_sync(0xffffffffu, s, owner);
    if (lane == owner) taken |= 1u << slot;
    if (lane == r) {
      my_index = b.index;
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

cudaError_t launch_router_fast_logits(const CUtensorMap& tmap_split, const CUtensorMap& tmap_gate,
                                      int rows, int split_plane_rows, int experts, int hidden,
                                      float* logits, int32_t* error, cudaStream_t stream) {
  if (rows <= 0 || experts % 16 != 0 || experts > 256 || hidden % kFastBlockK != 0) {
    return cudaErrorInvalidValue;
  }
  const int smem = kFastStages * (kFastABytes + experts * 128) + (2 * kFastStages + 1) * 8 + 16 + 1024;
  cudaError_t err = cudaFuncSetAttribute(router_fast_logits_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) return err;
  router_fast_logits_kernel<<<(rows + 127) / 128, kFastThreads, smem, stream>>>(
      tmap_split, tmap_gate, rows, split_plane_rows, experts, hidden, logits, error);
  return cudaGetLastError();
}

cudaError_t launch_router_select_exact(float* logits, const float* normalized,
                                       const __nv_bfloat16* gate, const float* logit_offset,
                                       const float* bias, int rows, int experts, int hidden,
                                       int top_k, bool norm_topk_prob, float routed_scaling,
                                       float tie_margin, int32_t* top_index, float* top_weight,
                                       int32_t* expert_counts, cudaStream_t stream) {
  if (rows <= 0 || experts % 32 != 0 || experts > 32 * kSelectPerLane || top_k <= 0 ||
      top_k > 32 || top_k > experts) {
    return cudaErrorInvalidValue;
  }
  router_select_exact_kernel<<<(rows + kSelectWarps - 1) / kSelectWarps, kSelectWarps * 32, 0,
                               stream>>>(logits, normalized, gate, logit_offset, bias, rows,
                                         experts, hidden, top_k, norm_topk_prob, routed_scaling,
                                         tie_margin, top_index, top_weight, expert_counts);
  return cudaGetLastError();
}

}  // namespace nmoe
