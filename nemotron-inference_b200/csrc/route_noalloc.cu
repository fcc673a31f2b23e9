// nmoe_route_tokens_noalloc: RMSNorm -> gate logits -> top-k expert selection in
// one call that never allocates.
//
// Who needs it: hosts that may not call cudaMalloc (or any allocating routine)
// at the point where they route tokens -- a runtime that hands out all device
// memory from its own arena at start-up and forbids later driver allocations, a
// latency-critical serving loop where an allocation could stall or fail, a
// plugin that runs under somebody else's memory accounting.  The other entry
// points that route tokens either take caller-provided intermediates
// (nmoe_rmsnorm / nmoe_router_logits / nmoe_router_topk, three calls and two
// intermediate buffers the caller must own) or live inside nmoe_layer, whose
// creation allocates.  Here the two intermediates (normalised activations and
// logits) live in a fixed array that is part of the library image.
//
// The price: the array has a fixed size (limits below), every GPU that loads
// the library holds it until the process exits, and all calls on one GPU share
// it.
#include <mutex>

#include "../../include/nmoe.h"
#include "common.cuh"
#include "kernels.h"

namespace {

// rows * hidden floats of normalised activations, then rows * experts floats
// of logits: 4.5 MiB.
constexpr size_t kMaxNormalizedFloats = NMOE_NOALLOC_MAX_ROWS_X_HIDDEN;
constexpr size_t kMaxLogitFloats = NMOE_NOALLOC_MAX_ROWS_X_EXPERTS;

static __device__ __align__(256) float g_route_scratch[kMaxNormalizedFloats + kMaxLogitFloats];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_address[kMaxDevices] = {};

// In host code `g_route_scratch` is only a handle for the symbol, not a device
// address; the address on the CURRENT device comes from cudaGetSymbolAddress.
// Looked up once per device, with that device current.
cudaError_t scratch_for_current_device(float** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_route_scratch);
    if (err != cudaSuccess) return err;
    g_scratch_address[device] = static_cast<float*>(address);
  }
  *out = g_scratch_address[device];
  return cudaSuccess;
}

}  // namespace

extern "C" nmoe_status nmoe_route_tokens_noalloc(
    void* stream_ptr, const void* input, nmoe_dtype dtype, int64_t rows, int32_t hidden,
    const float* norm_weight, float epsilon, const float* gate, const float* bias, int32_t experts,
    int32_t top_k, int32_t n_group, int32_t topk_group, int32_t norm_topk_prob,
    float routed_scaling, int32_t* top_index, float* top_weight) {
  if (input == nullptr || norm_weight == nullptr || gate == nullptr || bias == nullptr ||
      top_index == nullptr || top_weight == nullptr || rows <= 0 || hidden <= 0 ||
      hidden % 16 != 0 || experts <= 0 || !(epsilon > 0.0f)) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  // the selection's own argument rules, checked before anything is enqueued
  if (!nmoe::router_topk_arguments_valid(static_cast<int>(rows), experts, top_k, n_group,
                                         topk_group)) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  // the kernels read `input`, `norm_weight` and `gate` 16 bytes at a time
  if (((reinterpret_cast<uintptr_t>(input) | reinterpret_cast<uintptr_t>(norm_weight) |
        reinterpret_cast<uintptr_t>(gate)) & 15u) != 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (static_cast<size_t>(rows) * static_cast<size_t>(hidden) > kMaxNormalizedFloats ||
      static_cast<size_t>(rows) * static_cast<size_t>(experts) > kMaxLogitFloats) {
    return NMOE_ERR_CAPACITY;  // the fixed scratch cannot hold this many rows
  }
  float* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != cudaSuccess) return NMOE_ERR_CUDA;
  float* normalized = scratch;
  float* logits = scratch + kMaxNormalizedFloats;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const int r = static_cast<int>(rows);
  // Nothing in the scratch has to start at zero: both regions are fully
  // written for `rows` rows before they are read.
  // a launcher that rejects its arguments says cudaErrorInvalidValue; anything else
  // is a failure of the CUDA runtime
  auto status_of = [](cudaError_t err) {
    return err == cudaSuccess ? NMOE_OK
                              : err == cudaErrorInvalidValue ? NMOE_ERR_INVALID_ARGUMENT
                                                             : NMOE_ERR_CUDA;
  };
  nmoe_status status = status_of(nmoe::launch_norm_quant(
      input, dtype == NMOE_BF16, r, hidden, norm_weight, epsilon, normalized, nullptr, nullptr,
      nullptr, 0, nullptr, stream));
  if (status != NMOE_OK) return status;
  status = status_of(
      nmoe::launch_router_logits(normalized, gate, nullptr, r, experts, hidden, logits, stream));
  if (status != NMOE_OK) return status;
  return status_of(nmoe::launch_router_topk(logits, bias, r, experts, top_k, n_group, topk_group,
                                            norm_topk_prob != 0, routed_scaling, top_index,
                                            top_weight, nullptr, stream));
}
