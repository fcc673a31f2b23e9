// ref_driver.cpp -- thin command-line driver around the REFERENCE's own host
// functions for the NVFP4 expert layer.  TEST INFRASTRUCTURE ONLY.
//
// It is compiled against the reference sources where they lie (never copied):
// this translation unit textually includes runtime/src/backend/expert_layer.cpp
// so that the functions of its anonymous namespace (Sigmoid, Relu2, DecodeFp4,
// DecodeFp8, DequantizeNvfp4Matrix, RunNvfp4LinearHost, SelectTopExperts) are
// callable, and links runtime/src/backend/nvfp4_packing.cpp and
// nvfp4_scale_layout.cpp.  The device-side members of that file
// (ExpertLayerSlice::Create/Run) are unreferenced and dropped by
// --gc-sections.  Built by oracle/build_oracle.py into oracle/_ref/ref_driver.
//
// Usage: ref_driver <command> <args...>; every tensor travels as a raw
// little-endian binary file.
#include "runtime/src/backend/expert_layer.cpp"

#include <chrono>
#include <cstdio>
#include <fstream>
#include <sstream>

#include "nemotron/nvfp4_scale_layout.h"

extern "C" void ref_dense_matmul_double(const float* activations, std::size_t rows,
                                        const float* weights, std::size_t output_rows,
                                        std::size_t input_cols, float* output);

namespace {

template <typename T>
std::vector<T> ReadFile(const std::string& path) {
  std::ifstream in(path, std::ios::binary | std::ios::ate);
  if (!in) {
    std::fprintf(stderr, "ref_driver: cannot open %s\n", path.c_str());
    std::exit(2);
  }
  const std::streamsize size = in.tellg();
  in.seekg(0);
  std::vector<T> data(static_cast<std::size_t>(size) / sizeof(T));
  in.read(reinterpret_cast<char*>(data.data()), size);
  return data;
}

template <typename T>
void WriteFile(const std::string& path, const std::vector<T>& data) {
  std::ofstream out(path, std::ios::binary);
  out.write(reinterpret_cast<const char*>(data.data()),
            static_cast<std::streamsize>(data.size() * sizeof(T)));
}

nemotron::GemmDescriptor MakeNvfp4Descriptor(std::size_t out_rows, std::size_t in_cols,
                                             const std::vector<std::uint8_t>& packed,
                                             const std::vector<std::uint8_t>& scales,
                                             const float* tensor_scale) {
  nemotron::GemmDescriptor d;
  d.kernel_family = nemotron::GemmKernelFamily::kCublasLtNvfp4BlockScaled;
  d.output_rows = out_rows;
  d.input_cols = in_cols;
  d.storage_dtype = "nvfp4_e2m1";
  d.compute_dtype = "fp32_accum";
  d.layout_tag = "cublaslt_fp4_tn_v1";
  d.packed_data = packed.data();
  d.packed_nbytes = packed.size();
  d.block_scales_data = scales.data();
  d.block_scales_nbytes = scales.size();
  d.tensor_scale_data = reinterpret_cast<const std::uint8_t*>(tensor_scale);
  d.tensor_scale_nbytes = sizeof(float);
  return d;
}

std::size_t ToSize(const char* s) { return static_cast<std::size_t>(std::strtoull(s, nullptr, 10)); }

}  // namespace

int main(int argc, char** argv) {
  using namespace nemotron;
  if (argc < 2) {
    std::fprintf(stderr, "usage: ref_driver <command> ...\n");
    return 2;
  }
  const std::string cmd = argv[1];

  if (cmd == "decode_tables" && argc == 3) {
    // 16 E2M1 values followed by 256 E4M3 values (DecodeFp4 / DecodeFp8).
    std::vector<float> out;
    for (int i = 0; i < 16; ++i) out.push_back(DecodeFp4(static_cast<std::uint8_t>(i)));
    for (int i = 0; i < 256; ++i) out.push_back(DecodeFp8(static_cast<std::uint8_t>(i)));
    WriteFile(argv[2], out);
    return 0;
  }
  if ((cmd == "encode_fp4" || cmd == "encode_fp8") && argc == 4) {
    // The toolkit conversions the reference packer calls
    // (nvfp4_packing.cpp:37-46), applied to a list of floats.
    const auto in = ReadFile<float>(argv[2]);
    std::vector<std::uint8_t> out(in.size());
    for (std::size_t i = 0; i < in.size(); ++i) {
      out[i] = cmd == "encode_fp4"
                   ? static_cast<std::uint8_t>(
                         __nv_cvt_float_to_fp4(in[i], __NV_E2M1, cudaRoundNearest) & 0x0f)
                   : static_cast<std::uint8_t>(
                         __nv_cvt_float_to_fp8(in[i], __NV_SATFINITE, __NV_E4M3));
    }
    WriteFile(argv[3], out);
    return 0;
  }
  if (cmd == "sigmoid" && argc == 4) {
    auto v = ReadFile<float>(argv[2]);
    for (float& x : v) x = Sigmoid(x);
    WriteFile(argv[3], v);
    return 0;
  }
  if (cmd == "pack" && argc == 7) {
    // pack <rows> <cols> <fixed_scale or 0> in.f32 out.bin
    // out = tensor_scale (4 bytes) | packed | block scales; empty file on reject.
    const std::size_t rows = ToSize(argv[2]), cols = ToSize(argv[3]);
    const float fixed = std::strtof(argv[4], nullptr);
    const auto in = ReadFile<float>(argv[5]);
    Nvfp4PackOptions options;
    if (fixed != 0.0f) options.fixed_tensor_scale = fixed;
    const auto packed = PackRowMajorFp32ToNvfp4(in.data(), rows, cols, options);
    std::vector<std::uint8_t> out;
    if (packed.has_value()) {
      out.resize(4);
      std::memcpy(out.data(), &packed->tensor_scale, 4);
      out.insert(out.end(), packed->packed.begin(), packed->packed.end());
      out.insert(out.end(), packed->block_scales.begin(), packed->block_scales.end());
    }
    WriteFile(argv[6], out);
    return 0;
  }
  if (cmd == "swizzle" && argc == 6) {
    const std::size_t rows = ToSize(argv[2]), cols = ToSize(argv[3]);
    const auto in = ReadFile<std::uint8_t>(argv[4]);
    WriteFile(argv[5], SwizzleRowMajorNvfp4ScalesForExecution(in.data(), rows, cols));
    return 0;
  }
  if (cmd == "dequant" && argc == 8) {
    // dequant <rows> <cols> packed.u8 scales.u8 tensor_scale out.f32
    const std::size_t rows = ToSize(argv[2]), cols = ToSize(argv[3]);
    const auto packed = ReadFile<std::uint8_t>(argv[4]);
    const auto scales = ReadFile<std::uint8_t>(argv[5]);
    const float ts = std::strtof(argv[6], nullptr);
    WriteFile(argv[7], DequantizeNvfp4Matrix(packed.data(), packed.size(), scales.data(),
                                             scales.size(), ts, rows, cols));
    return 0;
  }
  if (cmd == "topk" && argc == 12) {
    // topk T E k n_group topk_group norm scaling logits.f32 bias.f32 out.bin
    // out = per token k x (int32 index) then k x (float weight)
    ExpertLayerConfig config;
    const std::size_t T = ToSize(argv[2]);
    config.n_routed_experts = ToSize(argv[3]);
    config.top_k = ToSize(argv[4]);
    config.n_group = ToSize(argv[5]);
    config.topk_group = ToSize(argv[6]);
    config.norm_topk_prob = ToSize(argv[7]) != 0;
    config.routed_scaling_factor = std::strtof(argv[8], nullptr);
    const auto logits = ReadFile<float>(argv[9]);
    const auto bias = ReadFile<float>(argv[10]);
    std::vector<std::uint8_t> out;
    for (std::size_t t = 0; t < T; ++t) {
      const std::vector<float> row(logits.begin() + t * config.n_routed_experts,
                                   logits.begin() + (t + 1) * config.n_routed_experts);
      const auto selections = SelectTopExperts(config, row, bias);
      for (const auto& s : selections) {
        const std::int32_t index = static_cast<std::int32_t>(s.expert_index);
        const auto* p = reinterpret_cast<const std::uint8_t*>(&index);
        out.insert(out.end(), p, p + 4);
      }
      for (const auto& s : selections) {
        const auto* p = reinterpret_cast<const std::uint8_t*>(&s.weight);
        out.insert(out.end(), p, p + 4);
      }
    }
    WriteFile(argv[11], out);
    return 0;
  }
  if (cmd == "linear" && argc == 10) {
    // linear rows N K act.f32 w_packed.u8 w_scales.u8 w_tensor_scale out.f32
    // RunNvfp4LinearHost called once per activation row (rows == 1), the way
    // ExpertLayerSlice::Run calls it (expert_layer.cpp:913, :922, :990).
    const std::size_t rows = ToSize(argv[2]), N = ToSize(argv[3]), K = ToSize(argv[4]);
    const auto act = ReadFile<float>(argv[5]);
    const auto packed = ReadFile<std::uint8_t>(argv[6]);
    const auto scales = ReadFile<std::uint8_t>(argv[7]);
    const float ts = std::strtof(argv[8], nullptr);
    const GemmDescriptor d = MakeNvfp4Descriptor(N, K, packed, scales, &ts);
    std::vector<float> out;
    for (std::size_t r = 0; r < rows; ++r) {
      const std::vector<float> row(act.begin() + r * K, act.begin() + (r + 1) * K);
      const auto y = RunNvfp4LinearHost(row, 1, d);
      if (!y.has_value()) return 3;
      out.insert(out.end(), y->begin(), y->end());
    }
    WriteFile(argv[9], out);
    return 0;
  }
  if (cmd == "expert" && argc == 14) {
    // expert rows H I act.f32 up_p up_s up_ts down_p down_s down_ts hidden_out.f32 out.f32
    // down( relu2( up(x) ) ) per row through RunNvfp4LinearHost + ApplyRelu2
    // (expert_layer.cpp:913-922); also writes the relu^2 intermediate.
    const std::size_t rows = ToSize(argv[2]), H = ToSize(argv[3]), I = ToSize(argv[4]);
    const auto act = ReadFile<float>(argv[5]);
    const auto up_p = ReadFile<std::uint8_t>(argv[6]);
    const auto up_s = ReadFile<std::uint8_t>(argv[7]);
    const float up_ts = std::strtof(argv[8], nullptr);
    const auto down_p = ReadFile<std::uint8_t>(argv[9]);
    const auto down_s = ReadFile<std::uint8_t>(argv[10]);
    const float down_ts = std::strtof(argv[11], nullptr);
    const GemmDescriptor up = MakeNvfp4Descriptor(I, H, up_p, up_s, &up_ts);
    const GemmDescriptor down = MakeNvfp4Descriptor(H, I, down_p, down_s, &down_ts);
    std::vector<float> hidden, out;
    for (std::size_t r = 0; r < rows; ++r) {
      const std::vector<float> row(act.begin() + r * H, act.begin() + (r + 1) * H);
      const auto u = RunNvfp4LinearHost(row, 1, up);
      if (!u.has_value()) return 3;
      const std::vector<float> activated = ApplyRelu2(*u);
      const auto y = RunNvfp4LinearHost(activated, 1, down);
      if (!y.has_value()) return 3;
      hidden.insert(hidden.end(), activated.begin(), activated.end());
      out.insert(out.end(), y->begin(), y->end());
    }
    WriteFile(argv[12], hidden);
    WriteFile(argv[13], out);
    return 0;
  }
  if (cmd == "dense" && argc == 8) {
    // dense rows N K act.f32 weights.f32 out.f32 -- the double-accumulate host
    // matmul of the dense linear fallback (linear_op.cpp:97-118).
    const std::size_t rows = ToSize(argv[2]), N = ToSize(argv[3]), K = ToSize(argv[4]);
    const auto act = ReadFile<float>(argv[5]);
    const auto weights = ReadFile<float>(argv[6]);
    std::vector<float> out(rows * N);
    ref_dense_matmul_double(act.data(), rows, weights.data(), N, K, out.data());
    WriteFile(argv[7], out);
    return 0;
  }
  if (cmd == "layer_rows" && argc == 13) {
    // layer_rows dir rows H I S E k scaling normalized.f32 x.f32 out.f32
    // The per-token loop of ExpertLayerSlice::Run (expert_layer.cpp:871-1005,
    // :1064-1069) built from the reference's own functions: gate projection by
    // the double-accumulate host matmul, SelectTopExperts, RunNvfp4LinearHost +
    // ApplyRelu2 per selected expert, the NVFP4 shared expert, weighted
    // accumulate, mixer and residual.  RMSNorm is a device kernel in the
    // reference, so normalised rows come in from the caller.  Weights are raw
    // files in `dir`: gate.f32, bias.f32, up_p.u8, up_s.u8, up_ts.f32 (stacked
    // over experts), down_*, sup_*, sdown_*.  Prints the seconds spent in the
    // token loop (weights already in memory).
    const std::string dir = argv[2];
    const std::size_t rows = ToSize(argv[3]), H = ToSize(argv[4]), I = ToSize(argv[5]),
                      S = ToSize(argv[6]), E = ToSize(argv[7]);
    ExpertLayerConfig config;
    config.n_routed_experts = E;
    config.top_k = ToSize(argv[8]);
    config.routed_scaling_factor = std::strtof(argv[9], nullptr);
    const auto normalized = ReadFile<float>(argv[10]);
    const auto x = ReadFile<float>(argv[11]);
    const auto gate = ReadFile<float>(dir + "/gate.f32");
    const auto bias = ReadFile<float>(dir + "/bias.f32");
    const auto up_p = ReadFile<std::uint8_t>(dir + "/up_p.u8");
    const auto up_s = ReadFile<std::uint8_t>(dir + "/up_s.u8");
    const auto up_ts = ReadFile<float>(dir + "/up_ts.f32");
    const auto down_p = ReadFile<std::uint8_t>(dir + "/down_p.u8");
    const auto down_s = ReadFile<std::uint8_t>(dir + "/down_s.u8");
    const auto down_ts = ReadFile<float>(dir + "/down_ts.f32");
    const auto sup_p = ReadFile<std::uint8_t>(dir + "/sup_p.u8");
    const auto sup_s = ReadFile<std::uint8_t>(dir + "/sup_s.u8");
    const auto sup_ts = ReadFile<float>(dir + "/sup_ts.f32");
    const auto sdown_p = ReadFile<std::uint8_t>(dir + "/sdown_p.u8");
    const auto sdown_s = ReadFile<std::uint8_t>(dir + "/sdown_s.u8");
    const auto sdown_ts = ReadFile<float>(dir + "/sdown_ts.f32");
    auto slice = [](const std::vector<std::uint8_t>& v, std::size_t e, std::size_t each) {
      return std::vector<std::uint8_t>(v.begin() + e * each, v.begin() + (e + 1) * each);
    };
    std::vector<std::vector<std::uint8_t>> upp(E), ups(E), dnp(E), dns(E);
    std::vector<GemmDescriptor> up(E), down(E);
    for (std::size_t e = 0; e < E; ++e) {
      upp[e] = slice(up_p, e, I * H / 2);
      ups[e] = slice(up_s, e, I * H / 16);
      dnp[e] = slice(down_p, e, I * H / 2);
      dns[e] = slice(down_s, e, I * H / 16);
      up[e] = MakeNvfp4Descriptor(I, H, upp[e], ups[e], &up_ts[e]);
      down[e] = MakeNvfp4Descriptor(H, I, dnp[e], dns[e], &down_ts[e]);
    }
    const GemmDescriptor shared_up = MakeNvfp4Descriptor(S, H, sup_p, sup_s, &sup_ts[0]);
    const GemmDescriptor shared_down = MakeNvfp4Descriptor(H, S, sdown_p, sdown_s, &sdown_ts[0]);
    std::vector<float> out(rows * H);
    const auto start = std::chrono::steady_clock::now();
    std::vector<float> logits(rows * E);
    ref_dense_matmul_double(normalized.data(), rows, gate.data(), E, H, logits.data());
    for (std::size_t t = 0; t < rows; ++t) {
      const std::vector<float> logit_row(logits.begin() + t * E, logits.begin() + (t + 1) * E);
      const std::vector<float> row(normalized.begin() + t * H, normalized.begin() + (t + 1) * H);
      const auto selections = SelectTopExperts(config, logit_row, bias);
      std::vector<float> routed(H, 0.0f);
      for (const auto& selection : selections) {
        const auto u = RunNvfp4LinearHost(row, 1, up[selection.expert_index]);
        const auto d = RunNvfp4LinearHost(ApplyRelu2(*u), 1, down[selection.expert_index]);
        for (std::size_t i = 0; i < H; ++i) routed[i] += (*d)[i] * selection.weight;
      }
      const auto su = RunNvfp4LinearHost(row, 1, shared_up);
      const auto sd = RunNvfp4LinearHost(ApplyRelu2(*su), 1, shared_down);
      for (std::size_t i = 0; i < H; ++i) {
        const float mixer = routed[i] + (*sd)[i];
        out[t * H + i] = x[t * H + i] + mixer;
      }
    }
    const double seconds =
        std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
    WriteFile(argv[12], out);
    std::printf("%.6f\n", seconds);
    return 0;
  }
  std::fprintf(stderr, "ref_driver: unknown command or wrong argument count: %s\n", cmd.c_str());
  return 2;
}
