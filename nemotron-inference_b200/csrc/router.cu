// Router: gate logits and sigmoid top-k with correction bias.
//
// Replaces the gate projection (UploadedLinearOp::Run dense fallback,
// runtime/src/backend/linear_op.cpp:97-118: sequential DOUBLE accumulation on the
// host) and SelectTopExperts (runtime/src/backend/expert_layer.cpp:277-367).
//
// Logits are accumulated in FP64 from the FP32 normalised activations and the
// gate weights widened to FP32 (as the reference's upload does): every product
// is exact in double, so the result differs
// from the reference's sequential double sum only by double rounding noise
// (~1e-16 relative) and rounds to the same FP32 logit.  That is what keeps the
// selected expert sets identical to the reference's, not merely close.
#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

constexpr int kWarps = 8;

// One warp computes TPW tokens x EPW experts; lanes split the hidden dimension.
template <int TPW, int EPW>
__global__ void __launch_bounds__(kWarps * 32)
router_logits_kernel(const float* __restrict__ y, const float* __restrict__ gate,
                     const float* __restrict__ logit_offset, int rows, int experts, int hidden,
                     float* __restrict__ logits) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kWarps + (threadIdx.x >> 5);
  const int expert_tiles = experts / EPW;
  const int token_tile = warp_global / expert_tiles;
  const int expert_tile = warp_global - token_tile * expert_tiles;
  const int t0 = token_tile * TPW;
  const int e0 = expert_tile * EPW;
  if (t0 >= rows) return;

  double acc[TPW][EPW];
#pragma unroll
  for (int i = 0; i < TPW; ++i)
#pragma unroll
    for (int j = 0; j < EPW; ++j) acc[i][j] = 0.0;

  int k_begin = lane;
  if constexpr (TPW == 1) {
    if ((hidden & 127) == 0) {
      // small batches: 16-byte loads, three steps in flight (the loop is a chain of
      // load -> FMA otherwise and costs a memory latency per step)
      const float4* y4 = reinterpret_cast<const float4*>(y + static_cast<size_t>(t0) * hidden);
      const int quads = hidden / 4;
#pragma unroll 3
      for (int q = lane; q < quads; q += 32) {
        const float4 a4 = y4[q];
        const double a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
        for (int j = 0; j < EPW; ++j) {
          const float4 w4 =
              reinterpret_cast<const float4*>(gate + static_cast<size_t>(e0 + j) * hidden)[q];
          acc[0][j] = fma(a[0], static_cast<double>(w4.x), acc[0][j]);
          acc[0][j] = fma(a[1], static_cast<double>(w4.y), acc[0][j]);
          acc[0][j] = fma(a[2], static_cast<double>(w4.z), acc[0][j]);
          acc[0][j] = fma(a[3], static_cast<double>(w4.w), acc[0][j]);
        }
      }
      k_begin = hidden;  // nothing left for the scalar loop
    }
  }
  for (int k = k_begin; k < hidden; k += 32) {
    double a[TPW];
#pragma unroll
    for (int i = 0; i < TPW; ++i) {
      const int t = min(t0 + i, rows - 1);
      a[i] = static_cast<double>(y[static_cast<size_t>(t) * hidden + k]);
    }
#pragma unroll
    for (int j = 0; j < EPW; ++j) {
      const double w = static_cast<double>(gate[static_cast<size_t>(e0 + j) * hidden + k]);
#pragma unroll
      for (int i = 0; i < TPW; ++i) acc[i][j] = fma(a[i], w, acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < TPW; ++i) {
#pragma unroll
    for (int j = 0; j < EPW; ++j) {
      double v = acc[i][j];
#pragma unroll
      for (int stride = 16; stride > 0; stride >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, stride);
      }
      if (lane == 0 && t0 + i < rows) {
        float logit = static_cast<float>(v);
        if (logit_offset != nullptr) logit = __fadd_rn(logit, logit_offset[e0 + j]);
        logits[static_cast<size_t>(t0 + i) * experts + e0 + j] = logit;
      }
    }
  }
}

// Sigmoid of expert_layer.cpp:129-136.  The host evaluates std::exp on a float;
// here exp runs in double and is rounded once, which equals the correctly
// rounded single-precision exponential.
__device__ __forceinline__ float sigmoid_ref(float v) {
  if (v >= 0.0f) {
    const float e = static_cast<float>(exp(-static_cast<double>(v)));
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
  }
  const float e = static_cast<float>(exp(static_cast<double>(v)));
  return __fdiv_rn(e, __fadd_rn(1.0f, e));
}

struct Best {
  float value;
  int index;
};

__device__ __forceinline__ Best better(Best a, Best b) {
  // descending value, lower index wins ties; index < 0 marks "none"
  if (b.index < 0) return a;
  if (a.index < 0) return b;
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ __forceinline__ Best warp_best(Best mine) {
#pragma unroll
  for (int stride = 16; stride > 0; stride >>= 1) {
    Best other;
    other.value = __shfl_xor_sync(0xffffffffu, mine.value, stride);
    other.index = __shfl_xor_sync(0xffffffffu, mine.index, stride);
    mine = better(mine, other);
  }
  return mine;
}

constexpr int kMaxPerLane = 16;  // up to 512 experts
constexpr int kTopkWarps = 4;

// One warp per token; expert e lives in lane e % 32, slot e / 32.
__global__ void __launch_bounds__(kTopkWarps * 32)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int rows,
                   int experts, int top_k, int n_group, int topk_group, bool norm_topk_prob,
                   float routed_scaling, int32_t* __restrict__ top_index,
                   float* __restrict__ top_weight, int32_t* __restrict__ expert_counts) {
  extern __shared__ float choice_smem[];  // [kTopkWarps][experts], only for n_group > 1
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * kTopkWarps + warp;
  if (row >= rows) return;
  const int per_lane = experts / 32;

  float score[kMaxPerLane];
  float choice[kMaxPerLane];
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    score[j] = 0.0f;
    choice[j] = 0.0f;
    if (j < per_lane) {
      const int e = lane + 32 * j;
      score[j] = sigmoid_ref(logits[static_cast<size_t>(row) * experts + e]);
      choice[j] = __fadd_rn(score[j], bias[e]);
    }
  }

  if (n_group > 1) {
    // group score = sum of the two largest choices of the group (:299-318);
    // keep topk_group groups, zero the others' choices (:320-339)
    float* mine = choice_smem + warp * experts;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per_lane) mine[lane + 32 * j] = choice[j];
    __syncwarp();
    const int group_size = experts / n_group;
    Best group;
    group.index = -1;
    group.value = 0.0f;
    if (lane < n_group) {
      float top1 = -INFINITY, top2 = -INFINITY;
      for (int i = 0; i < group_size; ++i) {
        const float v = mine[lane * group_size + i];
        if (v > top1) {
          top2 = top1;
          top1 = v;
        } else if (v > top2) {
          top2 = v;
        }
      }
      if (!isfinite(top2)) top2 = top1;
      group.value = __fadd_rn(top1, top2);
      group.index = lane;
    }
    uint32_t selected_groups = 0;
    const int keep = min(topk_group, n_group);
    for (int r = 0; r < keep; ++r) {
      const Best b = warp_best(group);
      selected_groups |= 1u << b.index;
      if (group.index == b.index) group.index = -1;
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      if (j < per_lane) {
        const int g = (lane + 32 * j) / group_size;
        if (((selected_groups >> g) & 1u) == 0u) choice[j] = 0.0f;
      }
    }
  }

  uint32_t taken = 0;
  int my_index = -1;    // lane r keeps the r-th selection
  float my_score = 0.0f;
  const int count = min(top_k, experts);
  for (int r = 0; r < count; ++r) {
    Best local;
    local.index = -1;
    local.value = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      if (j < per_lane && ((taken >> j) & 1u) == 0u) {
        Best cand;
        cand.value = choice[j];
        cand.index = lane + 32 * j;
        local = better(local, cand);
      }
    }
    const Best b = warp_best(local);
    const int owner = b.index & 31;
    const int slot = b.index >> 5;
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j == slot) s = score[j];
    s = __shfl_sync(0xffffffffu, s, owner);
    if (lane == owner) taken |= 1u << slot;
    if (lane == r) {
      my_index = b.index;
      my_score = s;
    }
  }

  // weight = score (no bias) normalised over the selection in selection order
  // (:349-365)
  float weight_sum = 0.0f;
  for (int r = 0; r < count; ++r) {
    weight_sum = __fadd_rn(weight_sum, __shfl_sync(0xffffffffu, my_score, r));
  }
  if (lane < count) {
    float w = my_score;
    if (norm_topk_prob) w = __fdiv_rn(w, __fadd_rn(weight_sum, 1.0e-20f));
    w = __fmul_rn(w, routed_scaling);
    top_index[static_cast<size_t>(row) * top_k + lane] = my_index;
    top_weight[static_cast<size_t>(row) * top_k + lane] = w;
    if (expert_counts != nullptr) atomicAdd(&expert_counts[my_index], 1);
  }
}

}  // namespace

cudaError_t launch_router_logits(const float* normalized, const float* gate,
                                 const float* logit_offset, int rows, int experts, int hidden,
                                 float* logits, cudaStream_t stream) {
  if (rows <= 0 || experts <= 0 || hidden <= 0) return cudaErrorInvalidValue;
  if (rows >= 256 && experts % 16 == 0) {
    const int warps = ((rows + 1) / 2) * (experts / 16);
    router_logits_kernel<2, 16><<<(warps + kWarps - 1) / kWarps, kWarps * 32, 0, stream>>>(
        normalized, gate, logit_offset, rows, experts, hidden, logits);
  } else if (experts % 4 == 0 && rows * (experts / 4) >= 148 * kWarps) {
    // four experts per warp once that still gives every SM a block
    const int warps = rows * (experts / 4);
    router_logits_kernel<1, 4><<<(warps + kWarps - 1) / kWarps, kWarps * 32, 0, stream>>>(
        normalized, gate, logit_offset, rows, experts, hidden, logits);
  } else {
    // a handful of rows: one (row, expert) pair per warp, so that the gate streams
    // through all SMs instead of a few
    const int warps = rows * experts;
    router_logits_kernel<1, 1><<<(warps + kWarps - 1) / kWarps, kWarps * 32, 0, stream>>>(
        normalized, gate, logit_offset, rows, experts, hidden, logits);
  }
  return cudaGetLastError();
}

bool router_topk_arguments_valid(int rows, int experts, int top_k, int n_group, int topk_group) {
  return rows > 0 && experts > 0 && experts % 32 == 0 && experts <= 32 * kMaxPerLane &&
         top_k > 0 && top_k <= 32 && top_k <= experts && n_group > 0 && n_group <= 32 &&
         topk_group > 0 && experts % n_group == 0;
}

cudaError_t launch_router_topk(const float* logits, const float* bias, int rows, int experts,
                               int top_k, int n_group, int topk_group, bool norm_topk_prob,
                               float routed_scaling, int32_t* top_index, float* top_weight,
                               int32_t* expert_counts, cudaStream_t stream) {
  if (!router_topk_arguments_valid(rows, experts, top_k, n_group, topk_group)) {
    return cudaErrorInvalidValue;
  }
  const size_t smem = n_group > 1 ? sizeof(float) * kTopkWarps * experts : 0;
  router_topk_kernel<<<(rows + kTopkWarps - 1) / kTopkWarps, kTopkWarps * 32, smem, stream>>>(
      logits, bias, rows, experts, top_k, n_group, topk_group, norm_topk_prob, routed_scaling,
      top_index, top_weight, expert_counts);
  return cudaGetLastError();
}

}  // namespace nmoe
