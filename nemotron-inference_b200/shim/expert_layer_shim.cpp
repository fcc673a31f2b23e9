// Drop-in definitions of nemotron::ExpertLayerSlice over the C ABI of nmoe.h.
//
// This file is compiled inside the reference project: it includes the reference's own
// header (runtime/include/nemotron/expert_layer.h) and defines the member functions that
// header declares, replacing their definitions in runtime/src/backend/expert_layer.cpp
// (Create :494-709, Run :752-1092); BuildExpertLayerBindings (:369-492) is catalogue
// bookkeeping and stays where it is.  The callers
// (runtime/src/api/single_token_forward_model.cpp:392-419, :637-647) do not change.
//
// Build (inside the reference tree):
//   g++ -std=c++20 -I runtime/include -I <this repo>/include -c expert_layer_shim.cpp
//   ... -L <this repo>/nemotron-inference_b200 -lnmoe_b200 -lcudart
#include <cuda_runtime_api.h>

#include <cstdint>
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
}  // namespace

struct ExpertLayerSlice::Impl {
  ExpertLayerConfig config;
  nmoe_layer* layer = nullptr;
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
      b.gate_score_correction_bias == nullptr || b.shared_up_gemm_weight == nullptr ||
      b.shared_down_gemm_weight == nullptr || b.routed_experts.size() != c.n_routed_experts) {
    return nullptr;                                            // expert_layer.cpp:505-528
  }
  nmoe_config cfg{};
  cfg.layer_index = c.layer_index;            cfg.hidden_size = c.hidden_size;
  cfg.moe_latent_size = c.moe_latent_size;    cfg.top_k = c.top_k;
  cfg.routed_expert_intermediate_size = c.routed_expert_intermediate_size;
  cfg.shared_expert_intermediate_size = c.shared_expert_intermediate_size;
  cfg.n_routed_experts = c.n_routed_experts;  cfg.n_group = c.n_group;
  cfg.topk_group = c.topk_group;              cfg.norm_topk_prob = c.norm_topk_prob;
  cfg.rms_epsilon = c.rms_epsilon;            cfg.routed_scaling_factor = c.routed_scaling_factor;
  cfg.max_tokens = 8192;                      // prefill chunk size of the caller

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
  w.shared_up = ToMatrix(*b.shared_up_gemm_weight);
  w.shared_down = ToMatrix(*b.shared_down_gemm_weight);
  w.gate_logit_offset = nullptr;

  auto impl = std::make_unique<Impl>();
  impl->config = c;
  if (nmoe_layer_create(&cfg, &w, &impl->layer) != NMOE_OK) return nullptr;   // Create -> nullptr
  return std::unique_ptr<ExpertLayerSlice>(new ExpertLayerSlice(std::move(impl)));
}

bool ExpertLayerSlice::Run(CublasLtHandle&, GemmHeuristicCache*, const DeviceTensorFp32& input,
                           DeviceTensorFp32* output, ExpertLayerRunTrace* trace) const {
  if (!valid() || output == nullptr || input.shape().size() != 2 ||
      input.shape()[1] != impl_->config.hidden_size || output->shape() != input.shape() ||
      (trace != nullptr && input.shape()[0] != 1)) {
    return false;                                              // expert_layer.cpp:760-780
  }
  cudaStream_t stream = nullptr;                               // the reference runs on the default stream
  if (nmoe_layer_run(impl_->layer, stream, input.data(), NMOE_F32,
                     static_cast<int64_t>(input.shape()[0]), output->data(), NMOE_F32) != NMOE_OK) {
    return false;
  }
  if (nmoe_layer_sync_status(impl_->layer, stream) != NMOE_OK) return false;  // Run is synchronous
  if (trace != nullptr) {                                      // expert_layer.h:63-76
    trace->normalized_input.resize(impl_->config.hidden_size);
    nmoe_layer_copy_trace_field(impl_->layer, stream, 0, trace->normalized_input.data(),
                                trace->normalized_input.size() * sizeof(float));
    trace->router_logits.resize(impl_->config.n_routed_experts);
    nmoe_layer_copy_trace_field(impl_->layer, stream, 1, trace->router_logits.data(),
                                trace->router_logits.size() * sizeof(float));
    const std::size_t k = impl_->config.top_k, hidden = impl_->config.hidden_size;
    std::vector<std::int32_t> index(k);
    std::vector<float> weight(k), parts((k + 1) * hidden);
    nmoe_layer_copy_trace_field(impl_->layer, stream, 2, index.data(), k * sizeof(std::int32_t));
    nmoe_layer_copy_trace_field(impl_->layer, stream, 3, weight.data(), k * sizeof(float));
    nmoe_layer_copy_trace_field(impl_->layer, stream, 7, parts.data(),
                                parts.size() * sizeof(float));
    cudaStreamSynchronize(stream);
    trace->selected_experts.resize(k);
    trace->routed_expert_order.resize(k);
    for (std::size_t i = 0; i < k; ++i) {
      trace->selected_experts[i].expert_index = static_cast<std::size_t>(index[i]);
      trace->selected_experts[i].weight = weight[i];
      trace->routed_expert_order[i] = static_cast<std::size_t>(index[i]);
    }
    // weighted contributions in selection order, then the shared expert's row
    trace->routed_expert_weighted_contributions.assign(parts.begin(), parts.begin() + k * hidden);
    trace->shared_output.assign(parts.begin() + k * hidden, parts.end());
    cudaStreamSynchronize(stream);
  }
  return true;
}
}  // namespace nemotron
