// RMSNorm + dynamic NVFP4 activation quantiser, dequantiser and scale re-tiling.
//
// Replaces RmsNormKernel (runtime/src/backend/primitive_ops.cu:26-59), the host
// packer PackRowMajorFp32ToNvfp4 (runtime/src/backend/nvfp4_packing.cpp:90-157),
// its device mirror (runtime/src/backend/device_nvfp4_matrix.cu:64-171: amax,
// tensor scale, pack, swizzle -- four kernels and four synchronisations) and
// SwizzleRowMajorNvfp4ScalesForExecution
// (runtime/src/backend/nvfp4_scale_layout.cpp:68-87) with one pass per row.
//
// One warp owns one row.  The sum of squares reproduces the reference kernel's
// association exactly (256 strided FMA partials, halving tree), so that the
// normalised activations -- and therefore every FP4 code derived from them --
// are a pure function of the input bits.  inv_rms is 1/sqrt(mean+eps) with two
// correctly rounded operations (the reference kernel's rsqrtf is within 2 ulp
// of it).
#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

constexpr int kWarpsPerBlock = 8;

template <bool BF16>
__device__ __forceinline__ float load_scalar(const void* base, size_t index) {
  if constexpr (BF16) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[index]);
  } else {
    return reinterpret_cast<const float*>(base)[index];
  }
}

template <bool BF16>
__device__ __forceinline__ void load8(const void* base, size_t index, float (&v)[8]) {
  if constexpr (BF16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(
        reinterpret_cast<const __nv_bfloat16*>(base) + index);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + index);
    const float4 b =
        *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + index + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

// tensor scale rule of nvfp4_packing.cpp:119-126
__device__ __forceinline__ float tensor_scale_from_amax(float amax) {
  return amax > kFp4Max * kFp8Max ? clamp_scale(__fdiv_rn(amax, kFp4Max * kFp8Max)) : 1.0f;
}

template <bool BF16, bool PER_ROW_SCALE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
norm_quant_kernel(const void* __restrict__ in, int rows, int cols,
                  const float* __restrict__ norm_weight, float eps,
                  float* __restrict__ normalized, uint8_t* __restrict__ packed,
                  uint8_t* __restrict__ sf_row_major, uint8_t* __restrict__ sf_tiled, int k_tiles,
                  float* __restrict__ tensor_scale, const float* __restrict__ global_amax,
                  float* __restrict__ inv_rms_out) {
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerBlock + warp;
  if (row >= rows) return;
  const size_t row_base = static_cast<size_t>(row) * cols;

  float inv_rms = 1.0f;
  if (norm_weight != nullptr) {
    // The reference kernel keeps 256 partial sums, partial[t] accumulating columns
    // t, t+256, ... in order, and folds them with a halving tree.  Lane L owns
    // t = 8L .. 8L+7: its it-th 8-element chunk (columns 8(L+32 it) ..) is exactly
    // columns t + 256 it, so 16-byte loads reproduce the same partial sums.
    float partial[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int row_chunks = cols / 8;
#pragma unroll 4
    for (int ch = lane; ch < row_chunks; ch += 32) {
      float x[8];
      load8<BF16>(in, row_base + static_cast<size_t>(ch) * 8, x);
#pragma unroll
      for (int i = 0; i < 8; ++i) partial[i] = __fmaf_rn(x[i], x[i], partial[i]);
    }
    // halving tree: strides 128, 64, 32, 16, 8 pair lane L with L+16, +8, +4, +2, +1
    // (same i); strides 4, 2, 1 stay inside the lane
#pragma unroll
    for (int stride = 16; stride > 0; stride >>= 1) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        partial[i] = __fadd_rn(partial[i], __shfl_down_sync(0xffffffffu, partial[i], stride));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) partial[i] = __fadd_rn(partial[i], partial[i + 4]);
    partial[0] = __fadd_rn(partial[0], partial[2]);
    partial[1] = __fadd_rn(partial[1], partial[3]);
    float sum = __fadd_rn(partial[0], partial[1]);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float mean = __fdiv_rn(sum, static_cast<float>(cols));
    inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    if (lane == 0 && inv_rms_out != nullptr) inv_rms_out[row] = inv_rms;
  }

  const int chunks = cols / 8;
  float ts = 1.0f;
  if constexpr (PER_ROW_SCALE) {
    float amax = 0.0f;
#pragma unroll 4
    for (int ch = lane; ch < chunks; ch += 32) {
      float v[8];
      load8<BF16>(in, row_base + static_cast<size_t>(ch) * 8, v);
      if (norm_weight != nullptr) {
        const float4 w0 = *reinterpret_cast<const float4*>(norm_weight + ch * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(norm_weight + ch * 8 + 4);
        const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], inv_rms), w[i]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int stride = 16; stride > 0; stride >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, stride));
    }
    ts = tensor_scale_from_amax(amax);
    if (lane == 0 && tensor_scale != nullptr) tensor_scale[row] = ts;
  } else {
    ts = tensor_scale_from_amax(*global_amax);
    if (row == 0 && lane == 0 && tensor_scale != nullptr) tensor_scale[0] = ts;
  }

  const int blocks_per_row = cols / 16;
  const int iterations = (chunks + 31) / 32;
  for (int it = 0; it < iterations; ++it) {
    const int ch = it * 32 + lane;
    const bool active = ch < chunks;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (active) {
      load8<BF16>(in, row_base + static_cast<size_t>(ch) * 8, v);
      if (norm_weight != nullptr) {
        const float4 w0 = *reinterpret_cast<const float4*>(norm_weight + ch * 8);
        const float4 w1 = *reinterpret_cast<const float4*>(norm_weight + ch * 8 + 4);
        const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], inv_rms), w[i]);
      }
      if (normalized != nullptr) {
        float* dst = normalized + row_base + static_cast<size_t>(ch) * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    }
    // a 16-block is shared by lanes (2i, 2i+1)
    float half_max = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) half_max = fmaxf(half_max, fabsf(v[i]));
    const float block_max = fmaxf(half_max, __shfl_xor_sync(0xffffffffu, half_max, 1));
    float bs = 1.0f;
    if (block_max > 0.0f) bs = clamp_scale(__fdiv_rn(block_max, __fmul_rn(kFp4Max, ts)));
    const float divisor = __fmul_rn(ts, bs);
    uint32_t word = 0;
    // x / divisor, IEEE-rounded: one reciprocal per block and a residual correction per
    // value give the correctly rounded quotient unless the divisor's significand is all
    // ones (div_by_reciprocal), where the division itself is used
    if ((__float_as_uint(divisor) & 0x007fffffu) != 0x007fffffu) {
      const float r = __frcp_rn(divisor);
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const uint32_t byte = encode_e2m1x2(div_by_reciprocal(v[i], divisor, r),
                                            div_by_reciprocal(v[i + 1], divisor, r));
        word |= (byte & 0xffu) << (4 * i);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const uint32_t byte =
            encode_e2m1x2(__fdiv_rn(v[i], divisor), __fdiv_rn(v[i + 1], divisor));
        word |= (byte & 0xffu) << (4 * i);
      }
    }
    if (active && packed != nullptr) {
      *reinterpret_cast<uint32_t*>(packed + row_base / 2 + static_cast<size_t>(ch) * 4) = word;
      if ((lane & 1) == 0) {
        const uint8_t sf = static_cast<uint8_t>(encode_e4m3(bs));
        const int block = ch >> 1;
        if (sf_row_major != nullptr) {
          sf_row_major[static_cast<size_t>(row) * blocks_per_row + block] = sf;
        }
        if (sf_tiled != nullptr) sf_tiled[swizzled_scale_offset(row, block, k_tiles)] = sf;
      }
    }
  }
}

// ComputeGlobalMaxAbsKernel, device_nvfp4_matrix.cu:64-75
__global__ void global_amax_kernel(const float* __restrict__ in, size_t count,
                                   float* __restrict__ amax) {
  float local = 0.0f;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    local = fmaxf(local, fabsf(in[i]));
  }
#pragma unroll
  for (int stride = 16; stride > 0; stride >>= 1) {
    local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, stride));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(reinterpret_cast<int*>(amax), __float_as_int(local));  // non-negative floats
  }
}

// DequantizeNvfp4Matrix, expert_layer.cpp:154-186: scale product first.
__global__ void dequant_kernel(const uint8_t* __restrict__ packed,
                               const uint8_t* __restrict__ sf_row_major,
                               const float* __restrict__ tensor_scale, bool per_row, int rows,
                               int cols, float* __restrict__ out) {
  const size_t bytes = static_cast<size_t>(rows) * cols / 2;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < bytes;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t element = i * 2;
    const size_t row = element / cols;
    const size_t col = element - row * cols;
    const float ts = tensor_scale[per_row ? row : 0];
    const float s = __fmul_rn(decode_e4m3(sf_row_major[row * (cols / 16) + col / 16]), ts);
    const uint32_t byte = packed[i];
    out[element] = __fmul_rn(decode_e2m1(byte & 15u), s);
    out[element + 1] = __fmul_rn(decode_e2m1(byte >> 4), s);
  }
}

__global__ void swizzle_kernel(const uint8_t* __restrict__ row_major, int rows, int blocks,
                               int k_tiles, uint8_t* __restrict__ tiled) {
  const size_t count = static_cast<size_t>(rows) * blocks;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = i / blocks;
    const size_t block = i - row * blocks;
    tiled[swizzled_scale_offset(row, block, k_tiles)] = row_major[i];
  }
}

int grid_for(size_t work, int threads) {
  const size_t blocks = (work + threads - 1) / threads;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace

cudaError_t launch_norm_quant(const void* in, bool in_bf16, int rows, int cols,
                              const float* norm_weight, float eps, float* normalized,
                              uint8_t* packed, uint8_t* sf_row_major, uint8_t* sf_tiled,
                              int k_blocks, float* tensor_scale, cudaStream_t stream,
                              float* inv_rms) {
  if (rows <= 0 || cols <= 0 || cols % 16 != 0) return cudaErrorInvalidValue;
  const int grid = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int threads = kWarpsPerBlock * 32;
  if (in_bf16) {
    norm_quant_kernel<true, true><<<grid, threads, 0, stream>>>(
        in, rows, cols, norm_weight, eps, normalized, packed, sf_row_major, sf_tiled,
        k_blocks * 4, tensor_scale, nullptr, inv_rms);
  } else {
    norm_quant_kernel<false, true><<<grid, threads, 0, stream>>>(
        in, rows, cols, norm_weight, eps, normalized, packed, sf_row_major, sf_tiled,
        k_blocks * 4, tensor_scale, nullptr, inv_rms);
  }
  return cudaGetLastError();
}

cudaError_t launch_quant_matrix(const float* in, int rows, int cols, uint8_t* packed,
                                uint8_t* sf_row_major, float* tensor_scale, float* amax_scratch,
                                cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 16 != 0) return cudaErrorInvalidValue;
  cudaError_t err = cudaMemsetAsync(amax_scratch, 0, sizeof(float), stream);
  if (err != cudaSuccess) return err;
  const size_t count = static_cast<size_t>(rows) * cols;
  global_amax_kernel<<<grid_for(count, 256), 256, 0, stream>>>(in, count, amax_scratch);
  const int grid = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  norm_quant_kernel<false, false><<<grid, kWarpsPerBlock * 32, 0, stream>>>(
      in, rows, cols, nullptr, 0.0f, nullptr, packed, sf_row_major, nullptr, 0, tensor_scale,
      amax_scratch, nullptr);
  return cudaGetLastError();
}

cudaError_t launch_dequant(const uint8_t* packed, const uint8_t* sf_row_major,
                           const float* tensor_scale, bool per_row_scale, int rows, int cols,
                           float* out, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 16 != 0) return cudaErrorInvalidValue;
  const size_t bytes = static_cast<size_t>(rows) * cols / 2;
  dequant_kernel<<<grid_for(bytes, 256), 256, 0, stream>>>(packed, sf_row_major, tensor_scale,
                                                           per_row_scale, rows, cols, out);
  return cudaGetLastError();
}

cudaError_t launch_swizzle_scales(const uint8_t* row_major, int rows, int cols, uint8_t* tiled,
                                  cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || cols % 16 != 0) return cudaErrorInvalidValue;
  const int blocks = cols / 16;
  const int k_tiles = (blocks + 3) / 4;
  const size_t padded = static_cast<size_t>((rows + 127) / 128) * 128 * k_tiles * 4;
  cudaError_t err = cudaMemsetAsync(tiled, 0, padded, stream);
  if (err != cudaSuccess) return err;
  swizzle_kernel<<<grid_for(static_cast<size_t>(rows) * blocks, 256), 256, 0, stream>>>(
      row_major, rows, blocks, k_tiles, tiled);
  return cudaGetLastError();
}

}  // namespace nmoe
