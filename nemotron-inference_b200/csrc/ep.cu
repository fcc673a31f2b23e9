// Expert-parallel dispatch / return kernels.
//
// The reference has no multi-GPU code at all; correctness here is defined as
// "the expert-parallel layer equals the single-GPU layer".  Every rank routes
// its own tokens, packs one DISPATCH RECORD per (token, slot) pair -- the
// already quantised activation row, so that what an expert multiplies is bit
// for bit what it would multiply on one GPU -- grouped by destination rank, and
// an all-to-all (NCCL, issued by the host side) moves the records.  The
// receiving rank feeds them to the same plan / permute / grouped-GEMM kernels
// as local pairs and returns one weighted down_proj row per record in arrival
// order; the home rank adds them in selection order.
//
// Record layout (record_bytes, a multiple of 16):
//   [0, H/2)            packed E2M1 row
//   [H/2, H/2 + H/16)   E4M3 block scales, row-major
//   then FP32 tensor scale, FP32 routing weight, int32 expert index LOCAL to
//   the destination rank, zero padding.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

__global__ void dispatch_plan_kernel(const int32_t* __restrict__ expert_counts, int experts,
                                     int experts_per_rank, int world,
                                     int32_t* __restrict__ send_counts,
                                     int32_t* __restrict__ send_offsets,
                                     int32_t* __restrict__ rank_cursor) {
  __shared__ int32_t per_rank[64];
  const int r = threadIdx.x;
  if (r < world) {
    int total = 0;
    for (int e = r * experts_per_rank; e < (r + 1) * experts_per_rank && e < experts; ++e) {
      total += expert_counts[e];
    }
    per_rank[r] = total;
    send_counts[r] = total;
    rank_cursor[r] = 0;
  }
  __syncthreads();
  if (r == 0) {
    int running = 0;
    for (int i = 0; i < world; ++i) {
      send_offsets[i] = running;
      running += per_rank[i];
    }
  }
}

constexpr int kPackWarps = 8;

__global__ void __launch_bounds__(kPackWarps * 32)
pack_records_kernel(const int32_t* __restrict__ top_index, const float* __restrict__ top_weight,
                    int pairs, int top_k, int experts_per_rank,
                    const uint8_t* __restrict__ packed, const uint8_t* __restrict__ sf_row_major,
                    const float* __restrict__ tensor_scale, int cols, int record_bytes,
                    const int32_t* __restrict__ send_offsets, int32_t* __restrict__ rank_cursor,
                    int capacity, uint8_t* __restrict__ records,
                    const unsigned long long* __restrict__ windows,
                    int32_t* __restrict__ send_position, int32_t* __restrict__ error) {
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x * kPackWarps + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int token = pair / top_k;
  const int expert = top_index[pair];
  const int rank = expert / experts_per_rank;
  // the token's bytes are fetched before the cursor's atomic, so that their loads and the
  // atomic are in flight together
  const int packed_quads = cols / 32;  // 16-byte pieces; cols % 64 == 0
  const uint4* src = reinterpret_cast<const uint4*>(packed) + static_cast<size_t>(token) * packed_quads;
  constexpr int kAhead = 3;
  uint4 ahead[kAhead];
#pragma unroll
  for (int j = 0; j < kAhead; ++j) {
    const int w = lane + 32 * j;
    if (w < packed_quads) ahead[j] = src[w];
  }
  const int sf_bytes = cols / 16;
  const uint32_t* sf_src =
      reinterpret_cast<const uint32_t*>(sf_row_major + static_cast<size_t>(token) * sf_bytes);
  uint32_t scale_words[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int b = lane + 32 * j;
    if (b < sf_bytes / 4) scale_words[j] = sf_src[b];
  }
  int position = 0;
  int slot = 0;
  if (lane == 0) {
    slot = atomicAdd(&rank_cursor[rank], 1);
    if (capacity > 0) {
      // fixed-capacity layout: destination rank r owns records [r*capacity, (r+1)*capacity)
      position = slot < capacity ? rank * capacity + slot : -1;
      if (position < 0 && error != nullptr) atomicCAS(error, kDevOk, kDevPlanOverflow);
    } else {
      position = send_offsets[rank] + slot;
    }
  }
  position = __shfl_sync(0xffffffffu, position, 0);
  if (position < 0) {
    if (lane == 0) send_position[pair] = 0;
    return;
  }
  uint8_t* record;
  if (windows != nullptr) {
    // the record goes straight into the destination rank's receive window (its
    // own GPU's memory): windows[rank] is the start of this rank's segment there
    slot = __shfl_sync(0xffffffffu, slot, 0);
    record = reinterpret_cast<uint8_t*>(windows[rank]) + static_cast<size_t>(slot) * record_bytes;
  } else {
    record = records + static_cast<size_t>(position) * record_bytes;
  }
  uint4* dst = reinterpret_cast<uint4*>(record);
#pragma unroll
  for (int j = 0; j < kAhead; ++j) {
    const int w = lane + 32 * j;
    if (w < packed_quads) dst[w] = ahead[j];
  }
  for (int w = lane + 32 * kAhead; w < packed_quads; w += 32) dst[w] = src[w];
  uint32_t* sf_dst = reinterpret_cast<uint32_t*>(record + cols / 2);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int b = lane + 32 * j;
    if (b < sf_bytes / 4) sf_dst[b] = scale_words[j];
  }
  for (int b = lane + 64; b < sf_bytes / 4; b += 32) sf_dst[b] = sf_src[b];
  if (lane == 0) {
    // the tail starts at a multiple of 4: cols % 64 == 0 is required
    uint8_t* tail = record + cols / 2 + sf_bytes;
    *reinterpret_cast<float*>(tail) = tensor_scale[token];
    *reinterpret_cast<float*>(tail + 4) = top_weight[pair];
    *reinterpret_cast<int32_t*>(tail + 8) = expert - rank * experts_per_rank;
    send_position[pair] = position;
  }
}

__global__ void record_histogram_kernel(const uint8_t* __restrict__ records, int count,
                                        int record_bytes, int expert_offset, int local_experts,
                                        const int32_t* __restrict__ valid_counts, int capacity,
                                        int32_t* __restrict__ expert_counts,
                                        int32_t* __restrict__ error) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    if (valid_counts != nullptr && (i % capacity) >= min(valid_counts[i / capacity], capacity)) {
      continue;  // an unused slot of a fixed-capacity segment
    }
    const int e = *reinterpret_cast<const int32_t*>(
        records + static_cast<size_t>(i) * record_bytes + expert_offset);
    if (e >= 0 && e < local_experts) {
      atomicAdd(&expert_counts[e], 1);
    } else if (error != nullptr) {
      atomicCAS(error, kDevOk, kDevPlanOverflow);  // a corrupt or misrouted record
    }
  }
}

// Four consecutive elements of a row of RowKind `kind`.
__device__ __forceinline__ float4 load_row4(const void* base, int kind, size_t row, int hidden,
                                            int c) {
  if (kind == kRowF16) {
    const uint2 raw = *reinterpret_cast<const uint2*>(
        reinterpret_cast<const __half*>(base) + row * hidden + c);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
  }
  if (kind == kRowBf16) {
    const uint2 raw = *reinterpret_cast<const uint2*>(
        reinterpret_cast<const __nv_bfloat16*>(base) + row * hidden + c);
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
  }
  return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + row * hidden + c);
}

// out[t] = in[t] + ((sum_k routed[position[t][k]]) + shared[t]), routed parts
// added in selection order (expert_layer.cpp:951-953, :1064-1069).
template <bool IN_BF16, bool OUT_BF16>
__global__ void combine_indexed_kernel(const void* __restrict__ in,
                                       const void* __restrict__ returned_rows, int rows_kind,
                                       const int32_t* __restrict__ position,
                                       const void* __restrict__ shared_rows, int shared_kind,
                                       int rows, int hidden, int top_k, void* __restrict__ out,
                                       int32_t* __restrict__ error) {
  const int quads = hidden / 4;
  const size_t total = static_cast<size_t>(rows) * quads;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / quads;
    const int c = static_cast<int>(i - t * quads) * 4;
    float4 routed = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top_k; ++k) {
      const size_t row = static_cast<size_t>(position[t * top_k + k]);
      const float4 p = load_row4(returned_rows, rows_kind, row, hidden, c);
      if (k == 0) {
        routed = p;
      } else {
        routed.x = __fadd_rn(routed.x, p.x);
        routed.y = __fadd_rn(routed.y, p.y);
        routed.z = __fadd_rn(routed.z, p.z);
        routed.w = __fadd_rn(routed.w, p.w);
      }
    }
    const float4 shared = load_row4(shared_rows, shared_kind, t, hidden, c);
    const float4 x = load_row4(in, IN_BF16 ? kRowBf16 : kRowF32, t, hidden, c);
    float r[4];
    const float m0 = __fadd_rn(routed.x, shared.x), m1 = __fadd_rn(routed.y, shared.y),
                m2 = __fadd_rn(routed.z, shared.z), m3 = __fadd_rn(routed.w, shared.w);
    // a row that left binary16's range on its way here (the GEMM stores an infinity)
    if (rows_kind == kRowF16 && error != nullptr &&
        !(isfinite(m0) && isfinite(m1) && isfinite(m2) && isfinite(m3))) {
      atomicCAS(error, kDevOk, kDevActivationRange);
    }
    r[0] = __fadd_rn(x.x, m0);
    r[1] = __fadd_rn(x.y, m1);
    r[2] = __fadd_rn(x.z, m2);
    r[3] = __fadd_rn(x.w, m3);
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

// ---------------------------------------------------------------------------
// peer windows: flags that ranks raise in each other's memory
// ---------------------------------------------------------------------------

__global__ void window_epoch_kernel(uint32_t* epoch) { *epoch += 1u; }

// Thread r tells rank first+r that everything this rank's earlier kernels on
// the stream wrote into that rank's window (for the current step) is there:
// optionally one 32-bit word of payload (this rank's record count for it), then
// the step number into this rank's flag slot over there.
__global__ void window_signal_kernel(const unsigned long long* __restrict__ flag_slots,
                                     const unsigned long long* __restrict__ word_slots,
                                     const int32_t* __restrict__ words,
                                     const uint32_t* __restrict__ epoch, int first, int count) {
  if (static_cast<int>(threadIdx.x) >= count) return;
  const int r = first + static_cast<int>(threadIdx.x);
  if (word_slots != nullptr) {
    *reinterpret_cast<volatile int32_t*>(word_slots[r]) = words[r];
  }
  __threadfence_system();
  const uint32_t step = *epoch;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag_slots[r]), "r"(step) : "memory");
}

// Thread r waits until rank first+r has raised its flag for the current step.
// Bounded: after `limit_ticks` of clock64 the thread records kDevWaitTimeout
// and returns, so a missing peer costs a wrong result and an error status,
// never a hung GPU.
__global__ void window_wait_kernel(const uint32_t* __restrict__ flags,
                                   const uint32_t* __restrict__ epoch, int first, int count,
                                   long long limit_ticks, int32_t* __restrict__ error) {
  if (static_cast<int>(threadIdx.x) >= count) return;
  const uint32_t* flag = flags + first + threadIdx.x;
  const uint32_t step = *epoch;
  const long long start = clock64();
  while (true) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if (static_cast<int32_t>(seen - step) >= 0) break;
    if (clock64() - start > limit_ticks) {
      if (error != nullptr) atomicCAS(error, kDevOk, kDevWaitTimeout);
      break;
    }
    __nanosleep(200);
  }
}

}  // namespace

int dispatch_record_bytes(int cols) { return (cols / 2 + cols / 16 + 12 + 15) / 16 * 16; }

cudaError_t launch_dispatch_plan(const int32_t* expert_counts, int experts, int experts_per_rank,
                                 int world, int32_t* send_counts, int32_t* send_offsets,
                                 int32_t* rank_cursor, cudaStream_t stream) {
  if (world <= 0 || world > 64) return cudaErrorInvalidValue;
  dispatch_plan_kernel<<<1, 64, 0, stream>>>(expert_counts, experts, experts_per_rank, world,
                                             send_counts, send_offsets, rank_cursor);
  return cudaGetLastError();
}

cudaError_t launch_pack_records(const int32_t* top_index, const float* top_weight, int rows,
                                int top_k, int experts_per_rank, const uint8_t* packed,
                                const uint8_t* sf_row_major, const float* tensor_scale, int cols,
                                const int32_t* send_offsets, int32_t* rank_cursor, int capacity,
                                uint8_t* records, const unsigned long long* windows,
                                int32_t* send_position, int32_t* error, cudaStream_t stream) {
  const int pairs = rows * top_k;
  if (pairs <= 0 || cols % 64 != 0) return cudaErrorInvalidValue;
  if (windows != nullptr && capacity <= 0) return cudaErrorInvalidValue;
  pack_records_kernel<<<(pairs + kPackWarps - 1) / kPackWarps, kPackWarps * 32, 0, stream>>>(
      top_index, top_weight, pairs, top_k, experts_per_rank, packed, sf_row_major, tensor_scale,
      cols, dispatch_record_bytes(cols), send_offsets, rank_cursor, capacity, records, windows,
      send_position, error);
  return cudaGetLastError();
}

cudaError_t launch_record_histogram(const uint8_t* records, int count, int cols,
                                    int local_experts, const int32_t* valid_counts, int capacity,
                                    int32_t* expert_counts, int32_t* error, cudaStream_t stream) {
  if (count <= 0) return cudaSuccess;
  const int blocks = (count + 255) / 256 < 592 ? (count + 255) / 256 : 592;
  record_histogram_kernel<<<blocks, 256, 0, stream>>>(records, count, dispatch_record_bytes(cols),
                                                      cols / 2 + cols / 16 + 8, local_experts,
                                                      valid_counts, capacity, expert_counts,
                                                      error);
  return cudaGetLastError();
}

cudaError_t launch_combine_indexed(const void* in, bool in_bf16, const void* returned_rows,
                                   RowKind rows_kind, const int32_t* position,
                                   const void* shared_rows, RowKind shared_kind, int rows,
                                   int hidden, int top_k, void* out, bool out_bf16,
                                   int32_t* error, cudaStream_t stream) {
  if (rows <= 0 || hidden % 4 != 0 || top_k < 1) return cudaErrorInvalidValue;
  const size_t total = static_cast<size_t>(rows) * (hidden / 4);
  const int blocks = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (in_bf16 && out_bf16) {
    combine_indexed_kernel<true, true><<<blocks, 256, 0, stream>>>(
        in, returned_rows, rows_kind, position, shared_rows, shared_kind, rows, hidden, top_k, out,
        error);
  } else if (in_bf16) {
    combine_indexed_kernel<true, false><<<blocks, 256, 0, stream>>>(
        in, returned_rows, rows_kind, position, shared_rows, shared_kind, rows, hidden, top_k, out,
        error);
  } else if (out_bf16) {
    combine_indexed_kernel<false, true><<<blocks, 256, 0, stream>>>(
        in, returned_rows, rows_kind, position, shared_rows, shared_kind, rows, hidden, top_k, out,
        error);
  } else {
    combine_indexed_kernel<false, false><<<blocks, 256, 0, stream>>>(
        in, returned_rows, rows_kind, position, shared_rows, shared_kind, rows, hidden, top_k, out,
        error);
  }
  return cudaGetLastError();
}

cudaError_t launch_window_epoch(uint32_t* epoch, cudaStream_t stream) {
  window_epoch_kernel<<<1, 1, 0, stream>>>(epoch);
  return cudaGetLastError();
}

cudaError_t launch_window_signal(const unsigned long long* flag_slots,
                                 const unsigned long long* word_slots, const int32_t* words,
                                 const uint32_t* epoch, int first, int count,
                                 cudaStream_t stream) {
  if (count <= 0 || count > 64) return cudaErrorInvalidValue;
  window_signal_kernel<<<1, 64, 0, stream>>>(flag_slots, word_slots, words, epoch, first, count);
  return cudaGetLastError();
}

cudaError_t launch_window_wait(const uint32_t* flags, const uint32_t* epoch, int first, int count,
                               long long limit_ticks, int32_t* error, cudaStream_t stream) {
  if (count <= 0 || count > 64 || limit_ticks <= 0) return cudaErrorInvalidValue;
  window_wait_kernel<<<1, 64, 0, stream>>>(flags, epoch, first, count, limit_ticks, error);
  return cudaGetLastError();
}

}  // namespace nmoe
