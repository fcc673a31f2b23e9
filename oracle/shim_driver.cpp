// TEST INFRASTRUCTURE ONLY.  Drives the drop-in shim through the reference's own
// C++ types: builds GemmDescriptor / KernelTensorDescriptor objects over byte
// buffers read from a file (the way the reference's tests hand-build them,
// runtime/tests/expert_layer_oracle_test.cpp:626-645), calls
// nemotron::ExpertLayerSlice::Create and ::Run (defined by
// nemotron-inference_b200/shim/expert_layer_shim.cpp over libnmoe_b200.so) with
// nemotron::DeviceTensorFp32 tensors, and writes the output rows (and, for one
// token, the trace) to a file.  Compiled against the reference's headers and its
// device_tensor.cpp / cublaslt_handle.cpp where they lie in the reference
// checkout; the binary lands in oracle/_ref/.
//
// Input file (little endian): int64 header[10] = {hidden, routed_intermediate,
// shared_intermediate, experts, top_k, tokens, norm_topk_prob, 0, 0, 0},
// float rms_epsilon, float routed_scaling, then the arrays in the order read below.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <string>
#include <vector>

#include "nemotron/cublaslt_handle.h"
#include "nemotron/device_tensor.h"
#include "nemotron/expert_layer.h"

namespace {

struct Blob {
  std::vector<std::uint8_t> bytes;
};

bool ReadExact(std::FILE* f, void* dst, std::size_t n) { return std::fread(dst, 1, n, f) == n; }

bool ReadBlob(std::FILE* f, std::size_t n, Blob* blob) {
  blob->bytes.resize(n);
  return ReadExact(f, blob->bytes.data(), n);
}

struct Nvfp4Storage {
  Blob packed, scales, tensor_scale;
};

bool ReadNvfp4(std::FILE* f, std::size_t rows, std::size_t cols, Nvfp4Storage* s) {
  return ReadBlob(f, rows * cols / 2, &s->packed) && ReadBlob(f, rows * cols / 16, &s->scales) &&
         ReadBlob(f, 4, &s->tensor_scale);
}

nemotron::GemmDescriptor Nvfp4Descriptor(const std::string& name, std::size_t rows,
                                         std::size_t cols, const Nvfp4Storage& s) {
  nemotron::GemmDescriptor d;
  d.tensor_name = name;
  d.op_class = "gemm_nvfp4";
  d.kernel_family = nemotron::GemmKernelFamily::kCublasLtNvfp4BlockScaled;
  d.output_rows = rows;
  d.input_cols = cols;
  d.storage_dtype = "nvfp4_e2m1";
  d.compute_dtype = "fp32_accum";
  d.layout_tag = "cublaslt_fp4_tn_v1";
  d.alignment_bytes = 16;
  d.packed_data = s.packed.bytes.data();
  d.packed_nbytes = s.packed.bytes.size();
  d.block_scales_data = s.scales.bytes.data();
  d.block_scales_nbytes = s.scales.bytes.size();
  d.tensor_scale_data = s.tensor_scale.bytes.data();
  d.tensor_scale_nbytes = s.tensor_scale.bytes.size();
  return d;
}

nemotron::KernelTensorDescriptor VectorDescriptor(const std::string& name, std::size_t n,
                                                  const Blob& blob) {
  nemotron::KernelTensorDescriptor d;
  d.tensor_name = name;
  d.op_class = "vector";
  d.logical_shape = {n};
  d.packed_shape = {n};
  d.storage_dtype = "fp32";
  d.compute_dtype = "fp32";
  d.layout_tag = "row_major";
  d.packed_data = blob.bytes.data();
  d.packed_nbytes = blob.bytes.size();
  return d;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 3) {
    std::fprintf(stderr, "usage: shim_driver <input file> <output file>\n");
    return 2;
  }
  std::FILE* f = std::fopen(argv[1], "rb");
  if (f == nullptr) return 2;
  std::int64_t header[10];
  float eps = 0.0f, scaling = 0.0f;
  if (!ReadExact(f, header, sizeof(header)) || !ReadExact(f, &eps, 4) || !ReadExact(f, &scaling, 4)) {
    return 2;
  }
  const std::size_t H = header[0], I = header[1], S = header[2], E = header[3], K = header[4],
                    T = header[5];

  nemotron::ExpertLayerConfig config;
  config.layer_index = 0;
  config.hidden_size = H;
  config.moe_latent_size = H;
  config.routed_expert_intermediate_size = I;
  config.shared_expert_intermediate_size = S;
  config.n_routed_experts = E;
  config.top_k = K;
  config.rms_epsilon = eps;
  config.routed_scaling_factor = scaling;
  config.norm_topk_prob = header[6] != 0;

  Blob norm_weight, gate_weight, bias, tokens;
  Nvfp4Storage shared_up, shared_down;
  std::vector<Nvfp4Storage> up(E), down(E);
  bool ok = ReadBlob(f, H * 4, &norm_weight) && ReadBlob(f, E * H * 2, &gate_weight) &&
            ReadBlob(f, E * 4, &bias);
  for (std::size_t e = 0; ok && e < E; ++e) {
    ok = ReadNvfp4(f, I, H, &up[e]) && ReadNvfp4(f, H, I, &down[e]);
  }
  ok = ok && ReadNvfp4(f, S, H, &shared_up) && ReadNvfp4(f, H, S, &shared_down) &&
       ReadBlob(f, T * H * 4, &tokens);
  std::fclose(f);
  if (!ok) {
    std::fprintf(stderr, "short input file\n");
    return 2;
  }

  const nemotron::KernelTensorDescriptor norm_d = VectorDescriptor("norm.weight", H, norm_weight);
  const nemotron::KernelTensorDescriptor bias_d = VectorDescriptor("gate.bias", E, bias);
  nemotron::GemmDescriptor gate_d;
  gate_d.tensor_name = "gate.weight";
  gate_d.op_class = "gemm_dense";
  gate_d.kernel_family = nemotron::GemmKernelFamily::kDenseRowMajor;
  gate_d.output_rows = E;
  gate_d.input_cols = H;
  gate_d.storage_dtype = "bf16";
  gate_d.compute_dtype = "fp32";
  gate_d.layout_tag = "row_major";
  gate_d.packed_data = gate_weight.bytes.data();
  gate_d.packed_nbytes = gate_weight.bytes.size();
  std::vector<nemotron::GemmDescriptor> up_d, down_d;
  for (std::size_t e = 0; e < E; ++e) {
    up_d.push_back(Nvfp4Descriptor("up." + std::to_string(e), I, H, up[e]));
    down_d.push_back(Nvfp4Descriptor("down." + std::to_string(e), H, I, down[e]));
  }
  const nemotron::GemmDescriptor shared_up_d = Nvfp4Descriptor("shared.up", S, H, shared_up);
  const nemotron::GemmDescriptor shared_down_d = Nvfp4Descriptor("shared.down", H, S, shared_down);

  nemotron::ExpertLayerBindings bindings;
  bindings.input_norm_weight = &norm_d;
  bindings.gate_weight = &gate_d;
  bindings.gate_score_correction_bias = &bias_d;
  bindings.shared_up_gemm_weight = &shared_up_d;
  bindings.shared_down_gemm_weight = &shared_down_d;
  for (std::size_t e = 0; e < E; ++e) bindings.routed_experts.push_back({&up_d[e], &down_d[e]});

  std::unique_ptr<nemotron::ExpertLayerSlice> slice =
      nemotron::ExpertLayerSlice::Create(config, bindings);
  if (slice == nullptr || !slice->valid()) {
    std::fprintf(stderr, "ExpertLayerSlice::Create returned nullptr\n");
    return 1;
  }
  auto cublas = nemotron::CublasLtHandle::Create();
  auto input = nemotron::DeviceTensorFp32::Create({T, H});
  auto output = nemotron::DeviceTensorFp32::Create({T, H});
  if (cublas == nullptr || input == nullptr || output == nullptr ||
      !input->CopyFromHost(reinterpret_cast<const float*>(tokens.bytes.data()), T * H)) {
    return 1;
  }
  nemotron::ExpertLayerRunTrace trace;
  if (!slice->Run(*cublas, nullptr, *input, output.get(), T == 1 ? &trace : nullptr)) {
    std::fprintf(stderr, "ExpertLayerSlice::Run returned false\n");
    return 1;
  }
  // the reference contract: a trace is only allowed for one token, shapes must match
  auto wrong = nemotron::DeviceTensorFp32::Create({T, H + 16});
  const bool rejected = !slice->Run(*cublas, nullptr, *input, wrong.get(), nullptr);

  std::vector<float> result(T * H);
  if (!output->CopyToHost(result.data(), result.size())) return 1;
  std::FILE* out = std::fopen(argv[2], "wb");
  if (out == nullptr) return 2;
  const std::int64_t out_header[4] = {static_cast<std::int64_t>(T), static_cast<std::int64_t>(H),
                                      rejected ? 1 : 0,
                                      static_cast<std::int64_t>(trace.selected_experts.size())};
  std::fwrite(out_header, sizeof(out_header), 1, out);
  std::fwrite(result.data(), sizeof(float), result.size(), out);
  for (const nemotron::ExpertSelection& s : trace.selected_experts) {
    const std::int64_t index = static_cast<std::int64_t>(s.expert_index);
    std::fwrite(&index, sizeof(index), 1, out);
    std::fwrite(&s.weight, sizeof(float), 1, out);
  }
  if (T == 1) {
    // every vector of ExpertLayerRunTrace (expert_layer.h:63-76): int64 length, then values
    const std::vector<float>* fields[10] = {
        &trace.normalized_input, &trace.router_logits, &trace.latent_output,
        &trace.routed_latent_output, &trace.routed_expert_activated_hidden,
        &trace.routed_expert_outputs, &trace.routed_expert_weighted_contributions,
        &trace.projected_routed_output, &trace.shared_output, &trace.mixer_output};
    for (const std::vector<float>* field : fields) {
      const std::int64_t n = static_cast<std::int64_t>(field->size());
      std::fwrite(&n, sizeof(n), 1, out);
      std::fwrite(field->data(), sizeof(float), field->size(), out);
    }
    const std::int64_t n = static_cast<std::int64_t>(trace.routed_expert_order.size());
    std::fwrite(&n, sizeof(n), 1, out);
    for (std::size_t e : trace.routed_expert_order) {
      const std::int64_t index = static_cast<std::int64_t>(e);
      std::fwrite(&index, sizeof(index), 1, out);
    }
  }
  std::fclose(out);
  return 0;
}
