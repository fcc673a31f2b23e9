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

#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

__global__ void route_plan_kernel(PlanBuffers plan, int experts, int tile_rows, int tile_multiple,
                                  int max_row_tiles, int32_t* error) {
  __shared__ int32_t first_tile[513];
  const int e = threadIdx.x;
  int tiles = 0;
  int count = 0;
  if (e < experts) {
    count = plan.expert_counts[e];
    tiles = (count + tile_rows - 1) / tile_rows;
    tiles = (tiles + tile_multiple - 1) / tile_multiple * tile_multiple;
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
      tile.rows = max(0, min(tile_rows, count - i * tile_rows));
      tile.expert = e;
      tile.reserved = 0;
      plan.row_tiles[base + i] = tile;
    }
  }
}

constexpr int kPermuteWarps = 8;

__global__ void __launch_bounds__(kPermuteWarps * 32)
permute_kernel(PlanBuffers plan, PermuteSource src, int pairs, int experts, int tile_rows,
               int max_row_tiles, int cols, int k_tiles, uint8_t* __restrict__ sorted_packed,
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
  // a record that arrived corrupt or half written (a peer that timed out) names no
  // expert of this stack: the histogram kernel has reported it, nothing is indexed by it
  if (expert < 0 || expert >= experts) return;
  // Everything that does not depend on the destination is fetched BEFORE the cursor's
  // atomic, so that the row's loads, the plan's loads and the atomic are in flight
  // together instead of one global round trip after the other.
  const int words = cols / 8;
  const uint8_t* from_bytes = src.packed + static_cast<size_t>(source_row) * src.packed_stride;
  const bool wide = (reinterpret_cast<uintptr_t>(from_bytes) & 15u) == 0 && (cols & 31) == 0;
  constexpr int kAhead = 3;  // 16-byte pieces per lane held in registers: 1536 B of a row
  uint4 ahead[kAhead];
  if (wide) {
    const uint4* from = reinterpret_cast<const uint4*>(from_bytes);
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      const int q = lane + 32 * j;
      if (q < words / 4) ahead[j] = from[q];
    }
  }
  const int own_tiles = (plan.expert_counts[expert] + tile_rows - 1) / tile_rows;
  const int first_tile = plan.expert_slot0[expert];
  int position = 0;
  if (lane == 0) position = atomicAdd(&plan.expert_cursor[expert], 1);
  position = __shfl_sync(0xffffffffu, position, 0);
  // an expert's rows stay inside the tiles the plan gave it, whatever the histogram said
  if (position / tile_rows >= own_tiles) return;
  const int tile = first_tile + position / tile_rows;
  if (tile >= max_row_tiles) return;  // plan overflow was already reported
  const int row = tile * 128 + position % tile_rows;

  uint8_t* dst_bytes = sorted_packed + static_cast<size_t>(row) * (cols / 2);
  if (wide && (reinterpret_cast<uintptr_t>(dst_bytes) & 15u) == 0) {
    // 16 bytes per lane: a warp moves 512 contiguous bytes per instruction
    const uint4* from = reinterpret_cast<const uint4*>(from_bytes);
    uint4* dst = reinterpret_cast<uint4*>(dst_bytes);
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      const int q = lane + 32 * j;
      if (q < words / 4) dst[q] = ahead[j];
    }
    for (int q = lane + 32 * kAhead; q < words / 4; q += 32) dst[q] = from[q];
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

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ void unpack_f16x8(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = pair.x;
    v[2 * i + 1] = pair.y;
  }
}

// Eight consecutive elements of row `row` of a [rows][hidden] matrix of RowKind KIND.
template <int KIND>
__device__ __forceinline__ void load_row8(const void* base, size_t row, int hidden, int c,
                                          float (&v)[8]) {
  if constexpr (KIND == kRowBf16) {
    unpack_bf16x8(*reinterpret_cast<const uint4*>(
                      reinterpret_cast<const __nv_bfloat16*>(base) + row * hidden + c), v);
  } else if constexpr (KIND == kRowF16) {
    unpack_f16x8(*reinterpret_cast<const uint4*>(
                     reinterpret_cast<const __half*>(base) + row * hidden + c), v);
  } else {
    const float* p = reinterpret_cast<const float*>(base) + row * hidden + c;
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

template <bool BF16>
__device__ __forceinline__ void store_row8(void* base, size_t row, int hidden, int c,
                                           const float (&v)[8]) {
  if constexpr (BF16) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + row * hidden + c) =
        make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    float* p = reinterpret_cast<float*>(base) + row * hidden + c;
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// out[t] = in[t] + ((sum_k parts[t][k]) + parts[t][top_k]): the routed parts are
// added in selection order (expert_layer.cpp:951-953), then the shared expert's
// row and the residual (:1064-1069).  Eight elements per thread, 16- or 32-byte
// accesses; the parts are rows of RowKind PARTS.
template <bool IN_BF16, bool OUT_BF16, int PARTS>
__global__ void combine_kernel(const void* __restrict__ in, const void* __restrict__ parts,
                               int rows, int hidden, int top_k, void* __restrict__ out,
                               int32_t* __restrict__ error) {
  const int octs = hidden / 8;
  const size_t total = static_cast<size_t>(rows) * octs;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / octs;
    const int c = static_cast<int>(i - t * octs) * 8;
    const size_t first = t * (top_k + 1);
    float routed[8];
    load_row8<PARTS>(parts, first, hidden, c, routed);
    for (int k = 1; k < top_k; ++k) {
      float p[8];
      load_row8<PARTS>(parts, first + k, hidden, c, p);
#pragma unroll
      for (int j = 0; j < 8; ++j) routed[j] = __fadd_rn(routed[j], p[j]);
    }
    float shared[8], x[8], r[8];
    load_row8<PARTS>(parts, first + top_k, hidden, c, shared);
    load_row8<IN_BF16 ? kRowBf16 : kRowF32>(in, t, hidden, c, x);
    bool finite = true;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float mixer = __fadd_rn(routed[j], shared[j]);
      finite = finite && isfinite(mixer);
      r[j] = __fadd_rn(x[j], mixer);
    }
    if constexpr (PARTS == kRowF16) {
      // a row that left binary16's range on its way here (the GEMM stores an infinity)
      if (!finite && error != nullptr) atomicCAS(error, kDevOk, kDevActivationRange);
    }
    store_row8<OUT_BF16>(out, t, hidden, c, r);
  }
}

template <bool A, bool B>
void launch_combine_t(const void* in, const void* parts, RowKind parts_kind, int rows, int hidden,
                      int top_k, void* out, int32_t* error, int blocks, cudaStream_t stream) {
  if (parts_kind == kRowBf16) {
    combine_kernel<A, B, kRowBf16><<<blocks, 256, 0, stream>>>(in, parts, rows, hidden, top_k, out,
                                                               error);
  } else if (parts_kind == kRowF16) {
    combine_kernel<A, B, kRowF16><<<blocks, 256, 0, stream>>>(in, parts, rows, hidden, top_k, out,
                                                              error);
  } else {
    combine_kernel<A, B, kRowF32><<<blocks, 256, 0, stream>>>(in, parts, rows, hidden, top_k, out,
                                                              error);
  }
}

}  // namespace

cudaError_t launch_route_plan(const PlanBuffers& plan, int experts, int tile_rows,
                              int tile_multiple, int max_row_tiles, int32_t* error,
                              cudaStream_t stream) {
  if (experts <= 0 || experts > 512 || tile_multiple < 1) return cudaErrorInvalidValue;
  route_plan_kernel<<<1, 512, 0, stream>>>(plan, experts, tile_rows, tile_multiple, max_row_tiles,
                                           error);
  return cudaGetLastError();
}

cudaError_t launch_permute(const PlanBuffers& plan, const PermuteSource& src, int pairs,
                           int experts, int tile_rows, int max_row_tiles, int cols, int k_blocks,
                           uint8_t* sorted_packed, uint8_t* sorted_sf_tiled,
                           float* sorted_tensor_scale, float* sorted_weight,
                           int32_t* sorted_dest, int32_t* pair_row, int dest_stride,
                           cudaStream_t stream) {
  if (pairs <= 0 || src.pairs_per_row <= 0) return cudaErrorInvalidValue;
  permute_kernel<<<(pairs + kPermuteWarps - 1) / kPermuteWarps, kPermuteWarps * 32, 0, stream>>>(
      plan, src, pairs, experts, tile_rows, max_row_tiles, cols, k_blocks * 4, sorted_packed,
      sorted_sf_tiled, sorted_tensor_scale, sorted_weight, sorted_dest, pair_row, dest_stride);
  return cudaGetLastError();
}

cudaError_t launch_combine(const void* in, bool in_bf16, const void* parts, RowKind parts_kind,
                           int rows, int hidden, int top_k, void* out, bool out_bf16,
                           int32_t* error, cudaStream_t stream) {
  if (rows <= 0 || hidden % 8 != 0 || top_k < 1) return cudaErrorInvalidValue;
  const size_t total = static_cast<size_t>(rows) * (hidden / 8);
  const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 16));
  if (in_bf16 && out_bf16) {
    launch_combine_t<true, true>(in, parts, parts_kind, rows, hidden, top_k, out, error, blocks, stream);
  } else if (in_bf16) {
    launch_combine_t<true, false>(in, parts, parts_kind, rows, hidden, top_k, out, error, blocks, stream);
  } else if (out_bf16) {
    launch_combine_t<false, true>(in, parts, parts_kind, rows, hidden, top_k, out, error, blocks, stream);
  } else {
    launch_combine_t<false, false>(in, parts, parts_kind, rows, hidden, top_k, out, error, blocks, stream);
  }
  return cudaGetLastError();
}

}  // namespace nmoe
