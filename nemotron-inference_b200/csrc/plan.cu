// Route plan, token permute and the weighted combine.
//
// The reference walks tokens one by one and, inside, the token's selected
// experts (runtime/src/backend/expert_layer.cpp:871-954), accumulating
// routed_row += down * weight in selection order (:951-953) and finishing with
// mixer = routed + shared, out = input + mixer (:1064-1069).  Here the
// (token, slot) pairs are bucketed by expert so that each expert's rows form
// 128-row aligned slots for the grouped GEMM, and the combine kernel adds the
// per-slot results back in the reference's order.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

__global__ void route_plan_kernel(PlanBuffers plan, int experts, int tile_rows, int max_row_tiles,
                                  int32_t* error) {
  __shared__ int32_t first_tile[513];
  const int e = threadIdx.x;
  int tiles = 0;
  int count = 0;
  if (e < experts) {
    count = plan.expert_counts[e];
    tiles = (count + tile_rows - 1) / tile_rows;
    first_tile[e + 1] = tiles;
  }
  if (e == 0) first_tile[0] = 0;
  __syncthreads();
  if (e == 0) {
    int running = 0;
    for (int i = 0; i < experts; ++i) {
      const int t = first_tile[i + 1];
      first_tile[i] = running;
      running += t;
    }
    first_tile[experts] = running;
    int total = running;
    if (total > max_row_tiles) {
      if (error != nullptr) atomicCAS(error, kDevOk, kDevPlanOverflow);
      total = max_row_tiles;
    }
    *plan.num_row_tiles = total;
  }
  __syncthreads();
  if (e < experts) {
    const int base = first_tile[e];
    plan.expert_slot0[e] = base;
    plan.expert_cursor[e] = 0;
    for (int i = 0; i < tiles; ++i) {
      if (base + i >= max_row_tiles) break;
      RowTile tile;
      tile.row0 = (base + i) * 128;
      tile.rows = min(tile_rows, count - i * tile_rows);
      tile.expert = e;
      tile.reserved = 0;
      plan.row_tiles[base + i] = tile;
    }
  }
}

constexpr int kPermuteWarps = 8;

__global__ void __launch_bounds__(kPermuteWarps * 32)
permute_kernel(PlanBuffers plan, PermuteSource src, int pairs, int tile_rows, int max_row_tiles,
               int cols, int k_tiles, uint8_t* __restrict__ sorted_packed,
               uint8_t* __restrict__ sorted_sf_tiled, float* __restrict__ sorted_tensor_scale,
               float* __restrict__ sorted_weight, int32_t* __restrict__ sorted_dest,
               int32_t* __restrict__ pair_row, int dest_stride) {
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x * kPermuteWarps + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  if (src.valid_counts != nullptr &&
      (pair % src.capacity) >= min(src.valid_counts[pair / src.capacity], src.capacity)) {
    return;  // an unused slot of a fixed-capacity segment
  }
  const int source_row = pair / src.pairs_per_row;
  const int slot = pair - source_row * src.pairs_per_row;
  const int expert = *reinterpret_cast<const int32_t*>(
      reinterpret_cast<const uint8_t*>(src.expert) + static_cast<size_t>(pair) * src.expert_stride);
  int position = 0;
  if (lane == 0) position = atomicAdd(&plan.expert_cursor[expert], 1);
  position = __shfl_sync(0xffffffffu, position, 0);
  const int tile = plan.expert_slot0[expert] + position / tile_rows;
  if (tile >= max_row_tiles) return;  // plan overflow was already reported
  const int row = tile * 128 + position % tile_rows;

  const int words = cols / 8;
  const uint8_t* from_bytes = src.packed + static_cast<size_t>(source_row) * src.packed_stride;
  uint8_t* dst_bytes = sorted_packed + static_cast<size_t>(row) * (cols / 2);
  if (((reinterpret_cast<uintptr_t>(from_bytes) | reinterpret_cast<uintptr_t>(dst_bytes)) & 15u) == 0 &&
      (cols & 31) == 0) {
    // 16 bytes per lane: a warp moves 512 contiguous bytes per instruction
    const uint4* from = reinterpret_cast<const uint4*>(from_bytes);
    uint4* dst = reinterpret_cast<uint4*>(dst_bytes);
    for (int q = lane; q < words / 4; q += 32) dst[q] = from[q];
  } else {
    const uint32_t* from = reinterpret_cast<const uint32_t*>(from_bytes);
    uint32_t* dst = reinterpret_cast<uint32_t*>(dst_bytes);
    for (int w = lane; w < words; w += 32) dst[w] = from[w];
  }

  const int blocks = cols / 16;
  const uint8_t* sf_src = src.sf + static_cast<size_t>(source_row) * src.sf_stride;
  if ((blocks & 3) == 0) {
    // four consecutive blocks are one aligned 32-bit word on both sides
    const uint32_t* sf_src_w = reinterpret_cast<const uint32_t*>(sf_src);
    for (int kt = lane; kt < blocks / 4; kt += 32) {
      *reinterpret_cast<uint32_t*>(sorted_sf_tiled + swizzled_scale_offset(row, kt * 4, k_tiles)) =
          sf_src_w[kt];
    }
  } else {
    for (int b = lane; b < blocks; b += 32) {
      sorted_sf_tiled[swizzled_scale_offset(row, b, k_tiles)] = sf_src[b];
    }
  }
  if (lane == 0) {
    sorted_tensor_scale[row] = *reinterpret_cast<const float*>(
        reinterpret_cast<const uint8_t*>(src.tensor_scale) +
        static_cast<size_t>(source_row) * src.tensor_scale_stride);
    sorted_weight[row] = *reinterpret_cast<const float*>(
        reinterpret_cast<const uint8_t*>(src.weight) + static_cast<size_t>(pair) * src.weight_stride);
    sorted_dest[row] = source_row * dest_stride + slot;
    if (pair_row != nullptr) pair_row[pair] = row;
  }
}

template <bool IN_BF16, bool OUT_BF16>
__global__ void combine_kernel(const void* __restrict__ in, const float* __restrict__ parts,
                               int rows, int hidden, int top_k, void* __restrict__ out) {
  const int quads = hidden / 4;
  const size_t total = static_cast<size_t>(rows) * quads;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / quads;
    const int c = static_cast<int>(i - t * quads) * 4;
    const float* base = parts + (t * (top_k + 1)) * hidden + c;
    float4 routed = *reinterpret_cast<const float4*>(base);
    for (int k = 1; k < top_k; ++k) {
      const float4 p = *reinterpret_cast<const float4*>(base + static_cast<size_t>(k) * hidden);
      routed.x = __fadd_rn(routed.x, p.x);
      routed.y = __fadd_rn(routed.y, p.y);
      routed.z = __fadd_rn(routed.z, p.z);
      routed.w = __fadd_rn(routed.w, p.w);
    }
    const float4 shared = *reinterpret_cast<const float4*>(base + static_cast<size_t>(top_k) * hidden);
    float x[4];
    if constexpr (IN_BF16) {
      const uint2 raw = *reinterpret_cast<const uint2*>(
          reinterpret_cast<const __nv_bfloat16*>(in) + t * hidden + c);
      x[0] = __uint_as_float(raw.x << 16);
      x[1] = __uint_as_float(raw.x & 0xffff0000u);
      x[2] = __uint_as_float(raw.y << 16);
      x[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      const float4 raw = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(in) + t * hidden + c);
      x[0] = raw.x; x[1] = raw.y; x[2] = raw.z; x[3] = raw.w;
    }
    float r[4];
    r[0] = __fadd_rn(x[0], __fadd_rn(routed.x, shared.x));
    r[1] = __fadd_rn(x[1], __fadd_rn(routed.y, shared.y));
    r[2] = __fadd_rn(x[2], __fadd_rn(routed.z, shared.z));
    r[3] = __fadd_rn(x[3], __fadd_rn(routed.w, shared.w));
    if constexpr (OUT_BF16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]);
      __nv_bfloat162 hi = __floats2bfloat162_rn(r[2], r[3]);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + t * hidden + c) = packed;
    } else {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + t * hidden + c) =
          make_float4(r[0], r[1], r[2], r[3]);
    }
  }
}

}  // namespace

cudaError_t launch_route_plan(const PlanBuffers& plan, int experts, int tile_rows,
                              int max_row_tiles, int32_t* error, cudaStream_t stream) {
  if (experts <= 0 || experts > 512) return cudaErrorInvalidValue;
  route_plan_kernel<<<1, 512, 0, stream>>>(plan, experts, tile_rows, max_row_tiles, error);
  return cudaGetLastError();
}

cudaError_t launch_permute(const PlanBuffers& plan, const PermuteSource& src, int pairs,
                           int tile_rows, int max_row_tiles, int cols, int k_blocks,
                           uint8_t* sorted_packed, uint8_t* sorted_sf_tiled,
                           float* sorted_tensor_scale, float* sorted_weight,
                           int32_t* sorted_dest, int32_t* pair_row, int dest_stride,
                           cudaStream_t stream) {
  if (pairs <= 0 || src.pairs_per_row <= 0) return cudaErrorInvalidValue;
  permute_kernel<<<(pairs + kPermuteWarps - 1) / kPermuteWarps, kPermuteWarps * 32, 0, stream>>>(
      plan, src, pairs, tile_rows, max_row_tiles, cols, k_blocks * 4, sorted_packed,
      sorted_sf_tiled, sorted_tensor_scale, sorted_weight, sorted_dest, pair_row, dest_stride);
  return cudaGetLastError();
}

cudaError_t launch_combine(const void* in, bool in_bf16, const float* parts, int rows, int hidden,
                           int top_k, void* out, bool out_bf16, cudaStream_t stream) {
  if (rows <= 0 || hidden % 4 != 0 || top_k < 1) return cudaErrorInvalidValue;
  const size_t total = static_cast<size_t>(rows) * (hidden / 4);
  const int threads = 256;
  const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
  if (in_bf16 && out_bf16) {
    combine_kernel<true, true><<<blocks, threads, 0, stream>>>(in, parts, rows, hidden, top_k, out);
  } else if (in_bf16) {
    combine_kernel<true, false><<<blocks, threads, 0, stream>>>(in, parts, rows, hidden, top_k, out);
  } else if (out_bf16) {
    combine_kernel<false, true><<<blocks, threads, 0, stream>>>(in, parts, rows, hidden, top_k, out);
  } else {
    combine_kernel<false, false><<<blocks, threads, 0, stream>>>(in, parts, rows, hidden, top_k, out);
  }
  return cudaGetLastError();
}

}  // namespace nmoe
