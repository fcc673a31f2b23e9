// Element-wise helpers around the dense and scaled-FP8 linear families of the
// expert layer and the latent-MoE data flow.
//
// The reference runs fc1_latent / fc2_latent / shared_up (and shared_down when it
// is not NVFP4) as UploadedLinearOp (runtime/src/backend/linear_op.cpp:97-118) or
// ScaledFp8LinearOp (runtime/src/backend/scaled_fp8_linear.cu:222-283): FP32
// activations, FP32 weights, sequential DOUBLE accumulation.  The matmul itself
// is launch_router_logits (csrc/router.cu), which accumulates the same exact
// products in FP64; this file holds what goes around it:
//   * the activation round trip through E4M3 of the scaled-FP8 family
//     (QuantizeFp8RoundTripKernel, scaled_fp8_linear.cu:94-106, and the host loop
//     of ScaledFp8LinearOp::Run :231-236),
//   * the weight dequantisation DecodeFp8(byte) * weight_scale (:121-139),
//   * relu^2 in place (expert_layer.cpp:956-964),
//   * the routed sum in selection order (:951-953) when it feeds fc2_latent,
//   * mixer + residual (:1064-1069) from separate projected / shared rows.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

int blocks_for(size_t work, int threads) {
  const size_t blocks = (work + threads - 1) / threads;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

__global__ void fp8_round_trip_kernel(const float* __restrict__ in, size_t count, float scale,
                                      float* __restrict__ out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float normalized = __fdiv_rn(in[i], scale);
    out[i] = __fmul_rn(decode_e4m3(encode_e4m3(normalized)), scale);
  }
}

__global__ void fp8_weight_kernel(const uint8_t* __restrict__ bytes, size_t count, float scale,
                                  float* __restrict__ out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    out[i] = __fmul_rn(decode_e4m3(bytes[i]), scale);
  }
}

__global__ void relu2_kernel(float* __restrict__ values, size_t count) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float v = values[i];
    values[i] = v > 0.0f ? __fmul_rn(v, v) : 0.0f;
  }
}

// out[t] = ((0 + parts[t][0]) + parts[t][1]) + ... : routed_row of expert_layer.cpp:951-953
__global__ void sum_parts_kernel(const float* __restrict__ parts, int rows, int cols, int top_k,
                                 float* __restrict__ out) {
  const int quads = cols / 4;
  const size_t total = static_cast<size_t>(rows) * quads;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / quads;
    const int c = static_cast<int>(i - t * quads) * 4;
    const float* base = parts + t * top_k * cols + c;
    float4 acc = *reinterpret_cast<const float4*>(base);
    for (int k = 1; k < top_k; ++k) {
      const float4 p = *reinterpret_cast<const float4*>(base + static_cast<size_t>(k) * cols);
      acc.x = __fadd_rn(acc.x, p.x);
      acc.y = __fadd_rn(acc.y, p.y);
      acc.z = __fadd_rn(acc.z, p.z);
      acc.w = __fadd_rn(acc.w, p.w);
    }
    *reinterpret_cast<float4*>(out + t * cols + c) = acc;
  }
}

template <bool IN_BF16, bool OUT_BF16>
__global__ void mixer_kernel(const void* __restrict__ in, const float* __restrict__ projected,
                             const float* __restrict__ shared, size_t count,
                             void* __restrict__ out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    float x;
    if constexpr (IN_BF16) {
      x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in)[i]);
    } else {
      x = reinterpret_cast<const float*>(in)[i];
    }
    const float r = __fadd_rn(x, __fadd_rn(projected[i], shared[i]));
    if constexpr (OUT_BF16) {
      reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(r);
    } else {
      reinterpret_cast<float*>(out)[i] = r;
    }
  }
}

__global__ void gather_rows_kernel(const float* __restrict__ rows, const int32_t* __restrict__ row_of,
                                   int count, int cols, float* __restrict__ out) {
  const int i = blockIdx.x;
  if (i >= count) return;
  const int row = row_of != nullptr ? row_of[i] : i;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    out[static_cast<size_t>(i) * cols + c] = rows[static_cast<size_t>(row) * cols + c];
  }
}

}  // namespace

cudaError_t launch_fp8_round_trip(const float* in, size_t count, float input_scale, float* out,
                                  cudaStream_t stream) {
  if (count == 0) return cudaErrorInvalidValue;
  // ClampScale (scaled_fp8_linear.cu:27-33)
  const float scale = clamp_scale_host(input_scale);
  fp8_round_trip_kernel<<<blocks_for(count, 256), 256, 0, stream>>>(in, count, scale, out);
  return cudaGetLastError();
}

cudaError_t launch_fp8_weight_dequant(const uint8_t* bytes, size_t count, float weight_scale,
                                      float* out, cudaStream_t stream) {
  if (count == 0) return cudaErrorInvalidValue;
  fp8_weight_kernel<<<blocks_for(count, 256), 256, 0, stream>>>(bytes, count, weight_scale, out);
  return cudaGetLastError();
}

cudaError_t launch_relu2(float* values, size_t count, cudaStream_t stream) {
  if (count == 0) return cudaErrorInvalidValue;
  relu2_kernel<<<blocks_for(count, 256), 256, 0, stream>>>(values, count);
  return cudaGetLastError();
}

cudaError_t launch_sum_parts(const float* parts, int rows, int cols, int top_k, float* out,
                             cudaStream_t stream) {
  if (rows <= 0 || cols % 4 != 0 || top_k < 1) return cudaErrorInvalidValue;
  sum_parts_kernel<<<blocks_for(static_cast<size_t>(rows) * (cols / 4), 256), 256, 0, stream>>>(
      parts, rows, cols, top_k, out);
  return cudaGetLastError();
}

cudaError_t launch_mixer(const void* in, bool in_bf16, const float* projected, const float* shared,
                         int rows, int hidden, void* out, bool out_bf16, cudaStream_t stream) {
  if (rows <= 0 || hidden <= 0) return cudaErrorInvalidValue;
  const size_t count = static_cast<size_t>(rows) * hidden;
  const int blocks = blocks_for(count, 256);
  if (in_bf16 && out_bf16) {
    mixer_kernel<true, true><<<blocks, 256, 0, stream>>>(in, projected, shared, count, out);
  } else if (in_bf16) {
    mixer_kernel<true, false><<<blocks, 256, 0, stream>>>(in, projected, shared, count, out);
  } else if (out_bf16) {
    mixer_kernel<false, true><<<blocks, 256, 0, stream>>>(in, projected, shared, count, out);
  } else {
    mixer_kernel<false, false><<<blocks, 256, 0, stream>>>(in, projected, shared, count, out);
  }
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const float* rows, const int32_t* row_of, int count, int cols,
                               float* out, cudaStream_t stream) {
  if (count <= 0 || cols <= 0) return cudaErrorInvalidValue;
  gather_rows_kernel<<<count, 256, 0, stream>>>(rows, row_of, count, cols, out);
  return cudaGetLastError();
}

}  // namespace nmoe
