// Drop-in definitions of nemotron::ExpertLayerSlice over the C ABI of nmoe.h.
//
// This file is compiled inside the reference project: it includes the reference's own
// header (runtime/include/nemotron/expert_layer.h) and defines the member functions that
// header declares, replacing their definitions in runtime/src/backend/expert_layer.cpp
// (Create :494-709, Run :752-1092); BuildExpertLayerBindings (:369-492) is catalogue
// bookkeeping and stays where it is.  The callers
// (runtime/src/api/single_token_forward_model.cpp:392-419, :637-647) do not change.
// Device scratch starts at NMOE_SHIM_MAX_TOKENS rows per layer (default 256) and grows to
// the largest token count a Run has seen.
//
// Build (inside the reference tree):
//   g++ -std=c++20 -I runtime/include -I <this repo>/include -c expert_layer_shim.cpp
//   ... -L <this repo>/nemotron-inference_b200 -lnmoe_b200 -lcudart
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "nemotron/expert_layer.h"
#include "nmoe.h"

namespace nemotron {
namespace {
nmoe_nvfp4_matrix ToMatrix(const GemmDescriptor& d) {          // gemm_catalog.h:20-42
  return {d.output_rows, d.input_cols, d.packed_data, d.packed_nbytes,
          d.block_scales_data, d.block_scales_nbytes, d.tensor_scale_data, d.tensor_scale_nbytes};
}
nmoe_dense_tensor ToDense(const std::uint8_t* data, std::size_t nbytes, const std::string& dtype,
                          std::size_t rows, std::size_t cols) {
  return {data, nbytes, dtype == "bf16" || dtype == "bfloat16" ? NMOE_BF16 : NMOE_F32, rows, cols};
}

bool Copy(nmoe_layer* layer, cudaStream_t stream, int field, void* dst, std::size_t nbytes) {
  return nmoe_layer_copy_trace_field(layer, stream, field, dst, nbytes) == NMOE_OK;
}

// ExpertLayerRunTrace for one token (expert_layer.h:63-76), every field the reference
// fills (expert_layer.cpp:929-977, :1078-1090), from a run on the unfused path.
bool FillTrace(nmoe_layer* layer, cudaStream_t stream, const ExpertLayerConfig& c,
               ExpertLayerRunTrace* trace) {
  const std::size_t k = c.top_k, hidden = c.hidden_size, latent = c.moe_latent_size,
                    inter = c.routed_expert_intermediate_size,
                    shared_inter = c.shared_expert_intermediate_size;
  nmoe_trace_view view{};
  if (nmoe_layer_trace_view(layer, &view) != NMOE_OK) return false;
  const bool has_latent = view.latent_output != nullptr;
  trace->normalized_input.resize(hidden);
  trace->router_logits.resize(c.n_routed_experts);
  std::vector<std::int32_t> index(k);
  std::vector<float> weight(k);
  std::vector<float> parts((has_latent ? k : k + 1) * latent);
  trace->routed_expert_activated_hidden.resize(k * inter);
  trace->routed_expert_outputs.resize(k * latent);
  // nmoe_layer_export_unfused gathers on the device: stage its rows in device memory
  float* staged = nullptr;
  const std::size_t staged_floats = k * inter + k * latent + shared_inter;
  if (cudaMalloc(reinterpret_cast<void**>(&staged), staged_floats * sizeof(float)) != cudaSuccess) {
    return false;
  }
  bool ok = Copy(layer, stream, 0, trace->normalized_input.data(), hidden * sizeof(float)) &&
            Copy(layer, stream, 1, trace->router_logits.data(),
                 trace->router_logits.size() * sizeof(float)) &&
            Copy(layer, stream, 2, index.data(), k * sizeof(std::int32_t)) &&
            Copy(layer, stream, 3, weight.data(), k * sizeof(float)) &&
            Copy(layer, stream, 7, parts.data(), parts.size() * sizeof(float)) &&
            nmoe_layer_export_unfused(layer, stream, staged, staged + k * inter,
                                      staged + k * inter + k * latent) == NMOE_OK &&
            cudaMemcpyAsync(trace->routed_expert_activated_hidden.data(), staged,
                            k * inter * sizeof(float), cudaMemcpyDeviceToHost,
                            stream) == cudaSuccess &&
            cudaMemcpyAsync(trace->routed_expert_outputs.data(), staged + k * inter,
                            k * latent * sizeof(float), cudaMemcpyDeviceToHost,
                            stream) == cudaSuccess;
  trace->latent_output.resize(latent);
  trace->routed_latent_output.assign(latent, 0.0f);
  trace->projected_routed_output.resize(hidden);
  trace->shared_output.resize(hidden);
  if (ok && has_latent) {
    ok = Copy(layer, stream, 8, trace->latent_output.data(), latent * sizeof(float)) &&
         Copy(layer, stream, 9, trace->routed_latent_output.data(), latent * sizeof(float)) &&
         Copy(layer, stream, 10, trace->projected_routed_output.data(), hidden * sizeof(float)) &&
         Copy(layer, stream, 11, trace->shared_output.data(), hidden * sizeof(float));
  }
  ok = ok && cudaStreamSynchronize(stream) == cudaSuccess;
  cudaFree(staged);
  if (!ok) return false;
  trace->selected_experts.resize(k);
  trace->routed_expert_order.resize(k);
  for (std::size_t i = 0; i < k; ++i) {
    trace->selected_experts[i].expert_index = static_cast<std::size_t>(index[i]);
    trace->selected_experts[i].weight = weight[i];
    trace->routed_expert_order[i] = static_cast<std::size_t>(index[i]);
  }
  // weighted contributions in selection order
  trace->routed_expert_weighted_contributions.assign(parts.begin(), parts.begin() + k * latent);
  if (!has_latent) {
    // identity projections: latent = normalised input, projected = routed sum, taken in
    // the reference's order (:951-953); the shared expert's row follows the routed parts
    trace->latent_output = trace->normalized_input;
    for (std::size_t slot = 0; slot < k; ++slot) {
      for (std::size_t i = 0; i < latent; ++i) {
        trace->routed_latent_output[i] += parts[slot * latent + i];
      }
    }
    trace->projected_routed_output = trace->routed_latent_output;
    trace->shared_output.assign(parts.begin() + k * latent, parts.end());
  }
  trace->mixer_output.resize(hidden);
  for (std::size_t i = 0; i < hidden; ++i) {                    // :1064-1069
    trace->mixer_output[i] = trace->projected_routed_output[i] + trace->shared_output[i];
  }
  return true;
}

// BuildScaledFp8LinearConfig (expert_layer.cpp:84-105): the scaled-FP8 family needs the
// weight bytes and two scalar FP32 tensors; anything else falls back to the dense family.
bool ReadScalar(const KernelTensorDescriptor* d, float* out) {
  if (d == nullptr || d->packed_data == nullptr) return false;
  if (d->storage_dtype == "fp32" && d->packed_nbytes == sizeof(float)) {
    std::memcpy(out, d->packed_data, sizeof(float));
    return true;
  }
  if ((d->storage_dtype == "bf16" || d->storage_dtype == "bfloat16") && d->packed_nbytes == 2) {
    std::uint32_t bits = static_cast<std::uint32_t>(d->packed_data[0]) << 16 |
                         static_cast<std::uint32_t>(d->packed_data[1]) << 24;
    std::memcpy(out, &bits, sizeof(float));
    return true;
  }
  return false;
}

// fc1_latent / shared_up / shared_down in the dense or scaled-FP8 family
// (expert_layer.cpp:534-617); `absent` when neither form is bound.
nmoe_linear ToLinear(const GemmDescriptor* dense, const KernelTensorDescriptor* fp8_weight,
                     const KernelTensorDescriptor* weight_scale,
                     const KernelTensorDescriptor* input_scale) {
  nmoe_linear l{};
  l.family = NMOE_LINEAR_ABSENT;
  float ws = 0.0f, is = 0.0f;
  if (fp8_weight != nullptr && fp8_weight->logical_shape.size() == 2 &&
      fp8_weight->packed_data != nullptr && ReadScalar(weight_scale, &ws) &&
      ReadScalar(input_scale, &is)) {
    l.family = NMOE_LINEAR_SCALED_FP8;
    l.weight = {fp8_weight->packed_data, fp8_weight->packed_nbytes, NMOE_F32,
                fp8_weight->logical_shape[0], fp8_weight->logical_shape[1]};
    l.weight_scale = ws;
    l.input_scale = is;
  } else if (dense != nullptr && dense->kernel_family == GemmKernelFamily::kDenseRowMajor) {
    l.family = NMOE_LINEAR_DENSE;
    l.weight = ToDense(dense->packed_data, dense->packed_nbytes, dense->storage_dtype,
                       dense->output_rows, dense->input_cols);
  }
  return l;
}

std::int32_t InitialTokenCapacity() {
  // scratch grows on demand (nmoe_layer_reserve_tokens); this is only where it starts
  if (const char* env = std::getenv("NMOE_SHIM_MAX_TOKENS")) {
    const long v = std::strtol(env, nullptr, 10);
    if (v > 0 && v < (1 << 24)) return static_cast<std::int32_t>(v);
  }
  return 256;
}
}  // namespace

struct ExpertLayerSlice::Impl {
  ExpertLayerConfig config;
  nmoe_layer* layer = nullptr;
  std::int64_t capacity = 0;
  ~Impl() { nmoe_layer_destroy(layer); }
};

ExpertLayerSlice::ExpertLayerSlice(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
ExpertLayerSlice::ExpertLayerSlice(ExpertLayerSlice&&) noexcept = default;
ExpertLayerSlice& ExpertLayerSlice::operator=(ExpertLayerSlice&&) noexcept = default;
ExpertLayerSlice::~ExpertLayerSlice() = default;

bool ExpertLayerSlice::valid() const { return impl_ != nullptr && impl_->layer != nullptr; }
const ExpertLayerConfig& ExpertLayerSlice::config() const { return impl_->config; }

std::unique_ptr<ExpertLayerSlice> ExpertLayerSlice::Create(const ExpertLayerConfig& c,
                                                           const ExpertLayerBindings& b) {
  if (b.input_norm_weight == nullptr || b.gate_weight == nullptr ||
      b.gate_score_correction_bias == nullptr || b.routed_experts.size() != c.n_routed_experts) {
    return nullptr;                                            // expert_layer.cpp:505-528
  }
  nmoe_config cfg{};
  cfg.layer_index = static_cast<std::int32_t>(c.layer_index);
  cfg.hidden_size = static_cast<std::int32_t>(c.hidden_size);
  cfg.moe_latent_size = static_cast<std::int32_t>(c.moe_latent_size);
  cfg.top_k = static_cast<std::int32_t>(c.top_k);
  cfg.routed_expert_intermediate_size = static_cast<std::int32_t>(c.routed_expert_intermediate_size);
  cfg.shared_expert_intermediate_size = static_cast<std::int32_t>(c.shared_expert_intermediate_size);
  cfg.n_routed_experts = static_cast<std::int32_t>(c.n_routed_experts);
  cfg.n_group = static_cast<std::int32_t>(c.n_group);
  cfg.topk_group = static_cast<std::int32_t>(c.topk_group);
  cfg.norm_topk_prob = c.norm_topk_prob ? 1 : 0;
  cfg.rms_epsilon = c.rms_epsilon;
  cfg.routed_scaling_factor = c.routed_scaling_factor;
  cfg.max_tokens = InitialTokenCapacity();

  std::vector<nmoe_nvfp4_matrix> up, down;
  for (const ExpertWeightPair& p : b.routed_experts) {
    if (p.up_proj == nullptr || p.down_proj == nullptr) return nullptr;
    up.push_back(ToMatrix(*p.up_proj));
    down.push_back(ToMatrix(*p.down_proj));
  }
  nmoe_weights w{};
  const auto& norm = *b.input_norm_weight;                     // kernel_catalog.h:14-34
  w.input_norm_weight = ToDense(norm.packed_data, norm.packed_nbytes, norm.storage_dtype, 1, c.hidden_size);
  const auto& gate = *b.gate_weight;
  w.gate_weight = ToDense(gate.packed_data, gate.packed_nbytes, gate.storage_dtype,
                          gate.output_rows, gate.input_cols);
  const auto& bias = *b.gate_score_correction_bias;
  w.gate_score_correction_bias = ToDense(bias.packed_data, bias.packed_nbytes, bias.storage_dtype,
                                         1, c.n_routed_experts);
  w.routed_up = up.data();  w.routed_down = down.data();
  w.n_local_experts = static_cast<int32_t>(up.size());  w.first_local_expert = 0;
  w.gate_logit_offset = nullptr;
  // latent projections: absent only when the layer has none (moe_latent_size == hidden_size
  // and neither projection bound); the reference itself insists on both (:519-521)
  w.fc1_latent = ToLinear(b.fc1_latent_gemm_weight, b.fc1_latent_kernel_weight,
                          b.fc1_latent_weight_scale, b.fc1_latent_input_scale);
  w.fc2_latent = ToLinear(b.fc2_latent_weight, nullptr, nullptr, nullptr);
  // shared expert: an NVFP4 descriptor goes to the block-scaled GEMM, everything else to
  // the scaled-FP8 or dense family, in the reference's order of preference (:560-617)
  const bool up_nvfp4 = b.shared_up_gemm_weight != nullptr &&
                        b.shared_up_gemm_weight->kernel_family ==
                            GemmKernelFamily::kCublasLtNvfp4BlockScaled;
  if (up_nvfp4) {
    w.shared_up = ToMatrix(*b.shared_up_gemm_weight);
  } else {
    w.shared_up_linear = ToLinear(b.shared_up_gemm_weight, b.shared_up_kernel_weight,
                                  b.shared_up_weight_scale, b.shared_up_input_scale);
    if (w.shared_up_linear.family == NMOE_LINEAR_ABSENT) return nullptr;
  }
  const bool down_nvfp4 = b.shared_down_gemm_weight != nullptr &&
                          b.shared_down_gemm_weight->kernel_family ==
                              GemmKernelFamily::kCublasLtNvfp4BlockScaled;
  if (down_nvfp4) {
    w.shared_down = ToMatrix(*b.shared_down_gemm_weight);
  } else {
    const bool fp8 = b.shared_down_kernel_weight != nullptr &&
                     b.shared_down_kernel_weight->storage_dtype == "fp8_e4m3fn";
    w.shared_down_linear = ToLinear(b.shared_down_gemm_weight,
                                    fp8 ? b.shared_down_kernel_weight : nullptr,
                                    b.shared_down_weight_scale, b.shared_down_input_scale);
    if (w.shared_down_linear.family == NMOE_LINEAR_ABSENT) return nullptr;
  }

  auto impl = std::make_unique<Impl>();
  impl->config = c;
  impl->capacity = cfg.max_tokens;
  if (nmoe_layer_create(&cfg, &w, &impl->layer) != NMOE_OK) return nullptr;   // Create -> nullptr
  nmoe_layer_keep_trace(impl->layer, 0);  // a trace is for one token (:775): nothing to keep
  return std::unique_ptr<ExpertLayerSlice>(new ExpertLayerSlice(std::move(impl)));
}

bool ExpertLayerSlice::Run(CublasLtHandle&, GemmHeuristicCache*, const DeviceTensorFp32& input,
                           DeviceTensorFp32* output, ExpertLayerRunTrace* trace) const {
  if (!valid() || output == nullptr || input.shape().size() != 2 ||
      input.shape()[1] != impl_->config.hidden_size || output->shape() != input.shape() ||
      (trace != nullptr && input.shape()[0] != 1)) {
    return false;                                              // expert_layer.cpp:760-780
  }
  nmoe_layer* layer = impl_->layer;
  const std::int64_t tokens = static_cast<std::int64_t>(input.shape()[0]);
  // diagnostics go to stderr under NEMOTRON_FORWARD_DEBUG only, as in the reference (:758)
  const bool debug = std::getenv("NEMOTRON_FORWARD_DEBUG") != nullptr;
  auto fail = [&](const char* what, nmoe_status status) {
    if (debug) {
      std::fprintf(stderr, "expert_layer: %s: %s (%s)\n", what, nmoe_status_string(status),
                   nmoe_layer_last_error(layer));
    }
    return false;
  };
  cudaStream_t stream = nullptr;                               // the reference runs on the default stream
  // the reference sizes its scratch per call (:782-787): any token count is accepted
  if (tokens > impl_->capacity) {
    const nmoe_status grown = nmoe_layer_reserve_tokens(layer, static_cast<std::int32_t>(tokens));
    if (grown != NMOE_OK) return fail("growing the scratch", grown);
    impl_->capacity = tokens;
  }
  // a trace needs the FP32 activated rows, which only the unfused path keeps
  bool unfused = trace != nullptr;
  if (unfused) {
    const nmoe_status set = nmoe_layer_set_unfused_activation(layer, 1);
    if (set != NMOE_OK) return fail("switching to the unfused path", set);
  }
  nmoe_status status = NMOE_ERR_CUDA;
  for (int attempt = 0; attempt < 2; ++attempt) {
    status = nmoe_layer_run(layer, stream, input.data(), NMOE_F32, tokens, output->data(),
                            NMOE_F32);
    if (status != NMOE_OK) break;
    status = nmoe_layer_sync_status(layer, stream);            // Run is synchronous
    if (status != NMOE_ERR_ACTIVATION_RANGE || unfused) break;
    // an activated row beyond 6*448 takes a tensor scale != 1 (nvfp4_packing.cpp:119-126):
    // redo the call on the path that quantises rows the way RunNvfp4LinearHost does
    if (nmoe_layer_set_unfused_activation(layer, 1) != NMOE_OK) break;
    unfused = true;
  }
  bool ok = status == NMOE_OK;
  if (!ok) fail("run", status);
  if (ok && trace != nullptr) {
    ok = FillTrace(layer, stream, impl_->config, trace);
    if (!ok) fail("reading the trace", NMOE_ERR_CUDA);
  }
  if (unfused) nmoe_layer_set_unfused_activation(layer, 0);
  return ok;
}
}  // namespace nemotron
