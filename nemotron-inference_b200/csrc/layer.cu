// Host side of the C ABI declared in include/nmoe.h: weight upload, scratch,
// tensor maps and the launch sequence of the expert layer.
//
// Mirrors ExpertLayerSlice::Create / ::Run
// (runtime/src/backend/expert_layer.cpp:494-709, :752-1092) with three
// differences that follow from running on the device: all weights are
// uploaded once (the reference keeps host pointers to the routed experts,
// :707), scratch is allocated once for `max_tokens` (the reference allocates
// six tensors per call, :782-787) and nothing synchronises inside Run.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "../../include/nmoe.h"
#include "common.cuh"
#include "kernels.h"

namespace nmoe {
namespace {

// ---------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------

struct Failure {
  nmoe_status status;
  std::string message;
};

#define NMOE_CUDA(expr)                                                                    \
  do {                                                                                     \
    const cudaError_t err__ = (expr);                                                      \
    if (err__ != cudaSuccess) {                                                            \
      throw Failure{NMOE_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(err__)}; \
    }                                                                                      \
  } while (0)

#define NMOE_REQUIRE(cond, text)                                        \
  do {                                                                  \
    if (!(cond)) throw Failure{NMOE_ERR_INVALID_ARGUMENT, (text)};      \
  } while (0)

class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  ~DeviceBuffer() { reset(); }
  void allocate(size_t bytes, bool zero = false) {
    reset();
    bytes_ = bytes == 0 ? 16 : bytes;
    NMOE_CUDA(cudaMalloc(&ptr_, bytes_));
    if (zero) NMOE_CUDA(cudaMemset(ptr_, 0, bytes_));
  }
  void reset() {
    if (ptr_ != nullptr) cudaFree(ptr_);
    ptr_ = nullptr;
    bytes_ = 0;
  }
  template <typename T>
  T* as() const {
    return reinterpret_cast<T*>(ptr_);
  }
  size_t bytes() const { return bytes_; }

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult query;
    NMOE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query));
    if (sym == nullptr || query != cudaDriverEntryPointSuccess) {
      throw Failure{NMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver"};
    }
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Packed E2M1 rows viewed as bytes: [rows][row_bytes], box = 128 bytes x
// box_rows, 128-byte swizzle (one box row = one K block of 256 elements).
CUtensorMap make_packed_map(const void* base, size_t rows, size_t row_bytes, int box_rows) {
  NMOE_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "tensor map base must be 16-byte aligned");
  NMOE_REQUIRE(row_bytes % 16 == 0, "packed row pitch must be a multiple of 16 bytes (K % 32 == 0)");
  CUtensorMap map;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult rc = encode_tiled_fn()(
      &map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    throw Failure{NMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(rc)};
  }
  return map;
}

// bf16 rows [rows][cols], box = 64 elements (128 bytes) x box_rows, 128-byte swizzle.
CUtensorMap make_bf16_map(const void* base, size_t rows, size_t cols, int box_rows) {
  NMOE_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "tensor map base must be 16-byte aligned");
  NMOE_REQUIRE((cols * 2) % 16 == 0, "bf16 row pitch must be a multiple of 16 bytes");
  CUtensorMap map;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult rc = encode_tiled_fn()(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    throw Failure{NMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(rc)};
  }
  return map;
}

// Bytes that are already in their shared-memory order, viewed as [rows][128 B]: box =
// 128 bytes x box_rows, no swizzle.  The CTA-pair GEMM loads its weight panels through
// such a map.
CUtensorMap make_raw_map(const void* base, size_t rows, int box_rows) {
  NMOE_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "tensor map base must be 16-byte aligned");
  CUtensorMap map;
  const cuuint64_t dims[2] = {128u, rows};
  const cuuint64_t strides[1] = {128u};
  const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem_strides[2] = {1u, 1u};
  const CUresult rc = encode_tiled_fn()(
      &map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
      elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    throw Failure{NMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(rc)};
  }
  return map;
}

int k_blocks_of(int k) { return (k + 255) / 256; }
size_t tiled_sf_bytes(size_t row_slots, int k) { return row_slots * k_blocks_of(k) * 2048; }

// clock64 ticks in `ms` milliseconds at the device's maximum SM clock
long long ticks_from_ms(double ms) {
  int device = 0, khz = 0;
  NMOE_CUDA(cudaGetDevice(&device));
  NMOE_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device));
  const double ticks = ms * static_cast<double>(khz);
  return ticks < 1.0 ? 1 : static_cast<long long>(ticks);
}

int device_sm_count() {
  int device = 0, sms = 0;
  NMOE_CUDA(cudaGetDevice(&device));
  NMOE_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  return sms;
}

void validate_matrix(const nmoe_nvfp4_matrix& m, size_t rows, size_t cols, const char* name) {
  // shape checks of expert_layer.cpp:646-689 plus the byte counts of
  // DequantizeNvfp4Matrix (:162-169) and the 4-byte tensor scale (:189-195)
  const std::string n(name);
  NMOE_REQUIRE(m.output_rows == rows && m.input_cols == cols, n + ": shape mismatch");
  NMOE_REQUIRE(cols % 64 == 0, n + ": input_cols must be a multiple of 64");
  NMOE_REQUIRE(m.packed_data != nullptr && m.packed_nbytes == rows * cols / 2,
               n + ": packed bytes");
  NMOE_REQUIRE(m.block_scales_data != nullptr && m.block_scales_nbytes == rows * (cols / 16),
               n + ": block scale bytes");
  NMOE_REQUIRE(m.tensor_scale_data != nullptr && m.tensor_scale_nbytes == sizeof(float),
               n + ": tensor scale must be one FP32");
}

// ---------------------------------------------------------------------------
// A stack of same-shaped NVFP4 matrices resident in HBM with the scale layouts
// and tensor maps of every GEMM tile shape that may consume it.
// ---------------------------------------------------------------------------
// kClassPair: 256 x 176 tiles over CTA pairs (cta_group::2), each CTA staging half of the
// weight tile; measured slower than the single-CTA shapes, selected only by NMOE_GEMM_PAIR.
enum TileClass : int { kClassPrefill = 0, kClassDecode = 1, kClassDecodeWide = 2, kClassPair = 3 };

struct WeightStack {
  int experts = 0;
  int n = 0;  // output rows per expert
  int k = 0;  // input cols
  // K-block-major packed weights: every (expert, 256-element K block) is a
  // contiguous [n][128 B] panel, so a weight tile is one contiguous read; the
  // partial last K block lives in `packed_tail` as [experts * n][tail_pitch].
  DeviceBuffer packed;        // [experts][k/256][n][128]
  DeviceBuffer packed_tail;   // [experts][n][tail_pitch]
  int kb_full = 0;
  DeviceBuffer tensor_scale;  // [experts]
  DeviceBuffer sf_prefill;    // scale layout for the prefill tile of this projection
  DeviceBuffer sf_decode;     // scale layout for the BN=128 tiles
  DeviceBuffer sf_pair;       // scale layout for the CTA-pair tile
  GemmVariant prefill_variant = kVariantPrefillUp;
  GemmVariant decode_variant = kVariantDecode;
  GemmVariant decode_wide_variant = kVariantDecodeWide;
  GemmVariant pair_variant = kVariantPairUp;
  // tensor maps exist only for the partial last K block; full K blocks are
  // plain bulk copies of contiguous, pre-swizzled panels
  CUtensorMap tail_prefill;
  CUtensorMap tail_decode;
  CUtensorMap tail_pair;
  CUtensorMap full_pair;  // the K-block-major panels as [rows][128 B], for the CTA-pair variants

  void upload(const nmoe_nvfp4_matrix* matrices, int count, int rows, int cols, bool is_up,
              const char* name, cudaStream_t stream) {
    experts = count;
    n = rows;
    k = cols;
    prefill_variant = is_up ? kVariantPrefillUp : kVariantPrefillDown;
    pair_variant = is_up ? kVariantPairUp : kVariantPairDown;
    const size_t packed_each = static_cast<size_t>(rows) * cols / 2;
    const size_t sf_each = static_cast<size_t>(rows) * (cols / 16);
    tensor_scale.allocate(sizeof(float) * count);
    for (int e = 0; e < count; ++e) validate_matrix(matrices[e], rows, cols, name);
    const GemmVariantInfo pi = gemm_variant_info(prefill_variant);
    const GemmVariantInfo di = gemm_variant_info(decode_variant);
    const int pair_rows = gemm_variant_info(pair_variant).b_rows;
    const size_t sf_prefill_each = weight_scale_layout_bytes(1, rows, cols, pi.bn, pi.sfb_groups);
    const size_t sf_decode_each = weight_scale_layout_bytes(1, rows, cols, di.bn, di.sfb_groups);
    const GemmVariantInfo qi = gemm_variant_info(pair_variant);
    const size_t sf_pair_each = weight_scale_layout_bytes(1, rows, cols, qi.bn, qi.sfb_groups);
    sf_prefill.allocate(sf_prefill_each * count);
    sf_decode.allocate(sf_decode_each * count);
    sf_pair.allocate(sf_pair_each * count);
    kb_full = cols / 256;
    const int tail_bytes = (cols % 256) / 2;
    const size_t panel_rows = static_cast<size_t>(count) * rows;
    packed.allocate(panel_rows * kb_full * 128 + 256 * 128, true);  // + one tile of slack: the last
                                                                    // tile of the last panel over-reads
    // The tail map reads `tail_bytes` per row and lets TMA zero-fill the rest of
    // the 128-byte box; if the driver refuses a box wider than the tensor, the
    // tail rows are padded to 128 bytes instead.
    int tail_pitch = tail_bytes;
    bool narrow_tail = tail_bytes > 0;
    if (narrow_tail) {
      packed_tail.allocate(panel_rows * tail_pitch);
      try {
        tail_prefill = make_packed_map(packed_tail.as<uint8_t>(), panel_rows, tail_pitch, pi.bn);
        tail_decode = make_packed_map(packed_tail.as<uint8_t>(), panel_rows, tail_pitch, di.bn);
        tail_pair = make_packed_map(packed_tail.as<uint8_t>(), panel_rows, tail_pitch, pair_rows);
      } catch (const Failure&) {
        narrow_tail = false;
      }
    }
    if (!narrow_tail && tail_bytes > 0) {
      tail_pitch = 128;
      packed_tail.allocate(panel_rows * tail_pitch, true);
      tail_prefill = make_packed_map(packed_tail.as<uint8_t>(), panel_rows, tail_pitch, pi.bn);
      tail_decode = make_packed_map(packed_tail.as<uint8_t>(), panel_rows, tail_pitch, di.bn);
      tail_pair = make_packed_map(packed_tail.as<uint8_t>(), panel_rows, tail_pitch, pair_rows);
    }
    if (tail_bytes == 0) {
      tail_pitch = 16;
      packed_tail.allocate(16);
    }
    // One expert at a time through a staging buffer of one matrix: descriptor bytes
    // (host or device) -> staging -> K-block-major panels and per-tile scale layouts.
    // Copies and kernels share the stream, so the staging buffer is reused in order;
    // no second copy of the whole stack exists and the host waits once, at the end.
    DeviceBuffer staging_packed, staging_sf;
    staging_packed.allocate(packed_each);
    staging_sf.allocate(sf_each);
    const size_t panel_each = static_cast<size_t>(rows) * kb_full * 128;
    const size_t tail_each = static_cast<size_t>(rows) * tail_pitch;
    for (int e = 0; e < count; ++e) {
      NMOE_CUDA(cudaMemcpyAsync(staging_packed.as<void>(), matrices[e].packed_data, packed_each,
                                cudaMemcpyDefault, stream));
      NMOE_CUDA(cudaMemcpyAsync(staging_sf.as<void>(), matrices[e].block_scales_data, sf_each,
                                cudaMemcpyDefault, stream));
      NMOE_CUDA(cudaMemcpyAsync(tensor_scale.as<float>() + e, matrices[e].tensor_scale_data,
                                sizeof(float), cudaMemcpyDefault, stream));
      NMOE_CUDA(relayout_weight_packed(staging_packed.as<uint8_t>(), 1, rows, cols, tail_pitch,
                                       packed.as<uint8_t>() + panel_each * e,
                                       packed_tail.as<uint8_t>() + (tail_bytes > 0 ? tail_each * e : 0),
                                       stream));
      NMOE_CUDA(relayout_weight_scales(staging_sf.as<uint8_t>(), 1, rows, cols, pi.bn,
                                       pi.sfb_groups, sf_prefill.as<uint8_t>() + sf_prefill_each * e,
                                       stream));
      NMOE_CUDA(relayout_weight_scales(staging_sf.as<uint8_t>(), 1, rows, cols, di.bn,
                                       di.sfb_groups, sf_decode.as<uint8_t>() + sf_decode_each * e,
                                       stream));
      NMOE_CUDA(relayout_weight_scales(staging_sf.as<uint8_t>(), 1, rows, cols, qi.bn,
                                       qi.sfb_groups, sf_pair.as<uint8_t>() + sf_pair_each * e,
                                       stream));
    }
    NMOE_CUDA(cudaStreamSynchronize(stream));  // the staging buffers die here
    if (kb_full > 0) {
      full_pair = make_raw_map(packed.as<uint8_t>(), panel_rows * kb_full + 256, pair_rows);
    } else {
      full_pair = make_raw_map(packed.as<uint8_t>(), 256, pair_rows);  // never read
    }
    if (tail_bytes == 0) {
      // never read (k_blocks == kb_full), but the kernel takes a valid map
      tail_prefill = make_packed_map(packed.as<uint8_t>(), panel_rows * kb_full, 128, pi.bn);
      tail_decode = make_packed_map(packed.as<uint8_t>(), panel_rows * kb_full, 128, di.bn);
      tail_pair = make_packed_map(packed.as<uint8_t>(), panel_rows * kb_full, 128, pair_rows);
    }
  }

  GemmVariant variant(TileClass c) const {
    return c == kClassPrefill ? prefill_variant
           : c == kClassPair  ? pair_variant
           : c == kClassDecode ? decode_variant : decode_wide_variant;
  }
  const CUtensorMap& tail_map(TileClass c) const {
    return c == kClassPrefill ? tail_prefill : c == kClassPair ? tail_pair : tail_decode;
  }
  const uint8_t* sf(TileClass c) const {
    return (c == kClassPrefill ? sf_prefill : c == kClassPair ? sf_pair : sf_decode).as<uint8_t>();
  }
};

// Packed activation rows + tiled scales as a GEMM A operand.
struct ActivationOperand {
  const uint8_t* packed = nullptr;
  const uint8_t* sf_tiled = nullptr;
  CUtensorMap map_box128;
  CUtensorMap map_box32;
  void bind(const uint8_t* packed_rows, const uint8_t* sf, size_t rows, int k) {
    packed = packed_rows;
    sf_tiled = sf;
    map_box128 = make_packed_map(packed_rows, rows, static_cast<size_t>(k) / 2, 128);
    map_box32 = make_packed_map(packed_rows, rows, static_cast<size_t>(k) / 2, 32);
  }
  const CUtensorMap& map(TileClass c) const { return c == kClassDecode ? map_box32 : map_box128; }
};


GemmMaps gemm_maps(const WeightStack& weights, TileClass tile_class, const ActivationOperand& a) {
  GemmMaps maps;
  maps.a = a.map(tile_class);
  maps.b_tail = weights.tail_map(tile_class);
  maps.b_full = weights.full_pair;
  return maps;
}

// NMOE_GEMM_ABLATE: timing experiments only (GemmArgs::ablate); results are wrong when set.
int gemm_ablation() {
  static const int value = [] {
    const char* env = std::getenv("NMOE_GEMM_ABLATE");
    return env != nullptr ? std::atoi(env) : 0;
  }();
  return value;
}

struct Schedule {
  const RowTile* row_tiles = nullptr;  // grouped when non-null
  const int32_t* num_row_tiles = nullptr;
  int dense_rows = 0;
};

// Where the down projection's rows go when they return straight to the ranks
// their records came from (GemmArgs::out_segments).
struct RowSegments {
  const unsigned long long* bases = nullptr;
  int rows = 0;
  int slot0 = 0;
};

// One GEMM with the row-storing epilogue: rows = A x W^T times the tensor scales
// [x routing weight] [-> relu^2], scattered by dest_row.
void run_down_gemm(const WeightStack& weights, TileClass tile_class, const ActivationOperand& a,
                   const float* a_tensor_scale, const Schedule& schedule, void* out_rows,
                   const int32_t* dest_row, int dest_mul, int dest_add, const float* row_weight,
                   bool relu2, int32_t* error, int num_sms, cudaStream_t stream, RowKind out_kind,
                   RowSegments segments) {
  GemmArgs d;
  const GemmVariant variant = weights.variant(tile_class);
  const int bn = gemm_variant_info(variant).bn;
  d.K = weights.k;
  d.N = weights.n;
  d.n_tiles = (weights.n + bn - 1) / bn;
  d.k_blocks = k_blocks_of(weights.k);
  d.kb_full = weights.kb_full;
  d.b_full = weights.packed.as<uint8_t>();
  d.sfa = a.sf_tiled;
  d.sfb = weights.sf(tile_class);
  d.a_tensor_scale = a_tensor_scale;
  d.w_tensor_scale = weights.tensor_scale.as<float>();
  d.row_tiles = schedule.row_tiles;
  d.num_row_tiles = schedule.num_row_tiles;
  d.dense_rows = schedule.dense_rows;
  d.out_rows = out_rows;
  d.out_kind = out_kind;
  d.dest_row = dest_row;
  d.dest_mul = dest_mul;
  d.dest_add = dest_add;
  d.row_weight = row_weight;
  d.relu2 = relu2 ? 1 : 0;
  d.out_segments = segments.bases;
  d.segment_rows = segments.rows;
  d.segment_slot0 = segments.slot0;
  d.error = error;
  d.ablate = gemm_ablation();
  NMOE_CUDA(launch_grouped_gemm(variant, kGemmDown, gemm_maps(weights, tile_class, a), d, num_sms,
                                stream));
}

// up GEMM (relu^2 + quantise) followed by down GEMM (scale, weight, scatter).
void run_expert_gemms(const WeightStack& up, const WeightStack& down, TileClass tile_class,
                      const ActivationOperand& a, const float* a_tensor_scale,
                      const Schedule& schedule, uint8_t* hidden_packed, uint8_t* hidden_sf,
                      const ActivationOperand& hidden, void* out_rows, const int32_t* dest_row,
                      int dest_mul, int dest_add, const float* row_weight, int32_t* error,
                      int num_sms, cudaStream_t stream, cudaEvent_t between = nullptr,
                      RowKind out_kind = kRowF32, RowSegments segments = RowSegments()) {
  GemmArgs g;
  const GemmVariant up_variant = up.variant(tile_class);
  g.K = up.k;
  g.N = up.n;
  g.n_tiles = (up.n + gemm_variant_info(up_variant).bn - 1) / gemm_variant_info(up_variant).bn;
  g.k_blocks = k_blocks_of(up.k);
  g.kb_full = up.kb_full;
  g.b_full = up.packed.as<uint8_t>();
  g.sfa = a.sf_tiled;
  g.sfb = up.sf(tile_class);
  g.a_tensor_scale = a_tensor_scale;
  g.w_tensor_scale = up.tensor_scale.as<float>();
  g.row_tiles = schedule.row_tiles;
  g.num_row_tiles = schedule.num_row_tiles;
  g.dense_rows = schedule.dense_rows;
  g.out_packed = hidden_packed;
  g.out_sf = hidden_sf;
  g.out_k_blocks = k_blocks_of(up.n);
  g.error = error;
  g.ablate = gemm_ablation();
  NMOE_CUDA(launch_grouped_gemm(up_variant, kGemmUp, gemm_maps(up, tile_class, a), g, num_sms,
                                stream));

  if (between != nullptr) cudaEventRecord(between, stream);

  // the fused quantiser always uses tensor scale 1
  run_down_gemm(down, tile_class, hidden, nullptr, schedule, out_rows, dest_row, dest_mul,
                dest_add, row_weight, false, error, num_sms, stream, out_kind, segments);
}

nmoe_status status_from_device(int code) {
  switch (code) {
    case kDevOk: return NMOE_OK;
    case kDevWaitTimeout: return NMOE_ERR_DEVICE_TIMEOUT;
    case kDevActivationRange: return NMOE_ERR_ACTIVATION_RANGE;
    case kDevPlanOverflow: return NMOE_ERR_CAPACITY;
    default: return NMOE_ERR_CUDA;
  }
}

struct ErrorSlot {
  DeviceBuffer device;
  int32_t* host = nullptr;  // pinned
  void create() {
    device.allocate(sizeof(int32_t), true);
    NMOE_CUDA(cudaMallocHost(&host, sizeof(int32_t)));
    *host = 0;
  }
  ~ErrorSlot() {
    if (host != nullptr) cudaFreeHost(host);
  }
  nmoe_status sync(cudaStream_t stream) {
    NMOE_CUDA(cudaMemcpyAsync(host, device.as<int32_t>(), sizeof(int32_t), cudaMemcpyDeviceToHost,
                              stream));
    NMOE_CUDA(cudaMemsetAsync(device.as<int32_t>(), 0, sizeof(int32_t), stream));
    NMOE_CUDA(cudaStreamSynchronize(stream));
    return status_from_device(*host);
  }
};

// Un-tile block scales of selected rows into row-major order (trace export).
__global__ void export_rows_kernel(const uint8_t* __restrict__ packed,
                                   const uint8_t* __restrict__ sf_tiled,
                                   const int32_t* __restrict__ row_of, int count, int cols,
                                   int k_tiles, uint8_t* __restrict__ out_packed,
                                   uint8_t* __restrict__ out_sf) {
  const int i = blockIdx.x;
  if (i >= count) return;
  const int row = row_of != nullptr ? row_of[i] : i;
  if (out_packed != nullptr) {
    for (int b = threadIdx.x; b < cols / 2; b += blockDim.x) {
      out_packed[static_cast<size_t>(i) * (cols / 2) + b] =
          packed[static_cast<size_t>(row) * (cols / 2) + b];
    }
  }
  if (out_sf != nullptr) {
    for (int b = threadIdx.x; b < cols / 16; b += blockDim.x) {
      out_sf[static_cast<size_t>(i) * (cols / 16) + b] =
          sf_tiled[swizzled_scale_offset(row, b, k_tiles)];
    }
  }
}

__global__ void widen_bf16_kernel(const __nv_bfloat16* __restrict__ in, size_t count,
                                  float* __restrict__ out) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    out[i] = __bfloat162float(in[i]);
  }
}

// ReadVectorWeightToHostFp32 / UploadVectorWeightToDeviceFp32 and the dense
// upload of linear_op.cpp:274-303: FP32 as is, bf16 widened.
void upload_dense_fp32(const nmoe_dense_tensor& t, size_t count, const char* name,
                       DeviceBuffer* out, cudaStream_t stream) {
  NMOE_REQUIRE(t.data != nullptr, std::string(name) + ": null data");
  NMOE_REQUIRE(t.rows * t.cols == count, std::string(name) + ": shape mismatch");
  out->allocate(count * sizeof(float));
  if (t.dtype == NMOE_F32) {
    NMOE_REQUIRE(t.nbytes == count * 4, std::string(name) + ": byte count");
    NMOE_CUDA(cudaMemcpyAsync(out->as<float>(), t.data, count * 4, cudaMemcpyDefault, stream));
  } else {
    NMOE_REQUIRE(t.nbytes == count * 2, std::string(name) + ": byte count");
    DeviceBuffer staging;
    staging.allocate(count * 2);
    NMOE_CUDA(cudaMemcpyAsync(staging.as<void>(), t.data, count * 2, cudaMemcpyDefault, stream));
    widen_bf16_kernel<<<148, 256, 0, stream>>>(staging.as<__nv_bfloat16>(), count, out->as<float>());
    NMOE_CUDA(cudaGetLastError());
    NMOE_CUDA(cudaStreamSynchronize(stream));
  }
}

// A dense or scaled-FP8 linear resident in HBM as FP32 [out][in], the form the
// reference's UploadedLinearOp / ScaledFp8LinearOp multiply with
// (linear_op.cpp:274-303, scaled_fp8_linear.cu:121-139).
struct DenseLinear {
  bool present = false;
  bool fp8 = false;
  int out = 0, in = 0;
  float input_scale = 1.0f;
  DeviceBuffer weight;

  void upload(const nmoe_linear& linear, size_t out_rows, size_t in_cols, const char* name,
              cudaStream_t stream) {
    const std::string n(name);
    out = static_cast<int>(out_rows);
    in = static_cast<int>(in_cols);
    const size_t count = out_rows * in_cols;
    if (linear.family == NMOE_LINEAR_DENSE) {
      nmoe_dense_tensor t = linear.weight;
      NMOE_REQUIRE(t.rows == out_rows && t.cols == in_cols, n + ": shape mismatch");
      upload_dense_fp32(t, count, name, &weight, stream);
    } else if (linear.family == NMOE_LINEAR_SCALED_FP8) {
      // DequantizeScaledFp8WeightToHostFp32 (scaled_fp8_linear.cu:121-139)
      NMOE_REQUIRE(linear.weight.data != nullptr && linear.weight.nbytes == count &&
                       linear.weight.rows == out_rows && linear.weight.cols == in_cols,
                   n + ": FP8 weight bytes");
      NMOE_REQUIRE(linear.weight_scale > 0.0f && linear.weight_scale < 3.0e38f,
                   n + ": weight_scale must be finite and positive");
      DeviceBuffer staging;
      staging.allocate(count);
      NMOE_CUDA(cudaMemcpyAsync(staging.as<void>(), linear.weight.data, count, cudaMemcpyDefault,
                                stream));
      weight.allocate(count * sizeof(float));
      NMOE_CUDA(launch_fp8_weight_dequant(staging.as<uint8_t>(), count, linear.weight_scale,
                                          weight.as<float>(), stream));
      NMOE_CUDA(cudaStreamSynchronize(stream));
      fp8 = true;
      input_scale = linear.input_scale;
    } else {
      throw Failure{NMOE_ERR_INVALID_ARGUMENT, n + ": unknown linear family"};
    }
    present = true;
  }
};

}  // namespace
}  // namespace nmoe

using namespace nmoe;

// ===========================================================================
// nmoe_ffn
// ===========================================================================
struct nmoe_ffn {
  int hidden = 0;
  int inter = 0;
  int max_rows = 0;
  int num_sms = 0;
  WeightStack up, down;
  DeviceBuffer a_packed, a_sf, a_ts, h_packed, h_sf;
  ActivationOperand a_op, h_op;
  ErrorSlot error;
  int last_rows = 0;
  std::string last_error;
};

extern "C" {

const char* nmoe_status_string(nmoe_status status) {
  switch (status) {
    case NMOE_OK: return "ok";
    case NMOE_ERR_INVALID_ARGUMENT: return "invalid argument";
    case NMOE_ERR_CUDA: return "CUDA error";
    case NMOE_ERR_UNSUPPORTED: return "unsupported configuration";
    case NMOE_ERR_DEVICE_TIMEOUT: return "a device-side wait timed out";
    case NMOE_ERR_ACTIVATION_RANGE: return "activated row exceeds the NVFP4 range for tensor scale 1";
    case NMOE_ERR_CAPACITY: return "token or row-tile capacity exceeded";
  }
  return "unknown status";
}

nmoe_status nmoe_ffn_create(const nmoe_nvfp4_matrix* up, const nmoe_nvfp4_matrix* down,
                            int32_t max_rows, nmoe_ffn** out_ffn) {
  if (up == nullptr || down == nullptr || out_ffn == nullptr || max_rows <= 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  *out_ffn = nullptr;
  std::unique_ptr<nmoe_ffn> f(new (std::nothrow) nmoe_ffn);
  if (!f) return NMOE_ERR_CUDA;
  try {
    f->hidden = static_cast<int>(up->input_cols);
    f->inter = static_cast<int>(up->output_rows);
    f->max_rows = max_rows;
    f->num_sms = device_sm_count();
    cudaStream_t stream = nullptr;
    f->up.upload(up, 1, f->inter, f->hidden, true, "up_proj", stream);
    f->down.upload(down, 1, f->hidden, f->inter, false, "down_proj", stream);
    const size_t slots = (static_cast<size_t>(max_rows) + 127) / 128;
    f->a_packed.allocate(slots * 128 * f->hidden / 2, true);
    f->a_sf.allocate(tiled_sf_bytes(slots, f->hidden), true);
    f->a_ts.allocate(slots * 128 * sizeof(float), true);
    f->h_packed.allocate(slots * 128 * f->inter / 2, true);
    f->h_sf.allocate(tiled_sf_bytes(slots, f->inter), true);
    f->a_op.bind(f->a_packed.as<uint8_t>(), f->a_sf.as<uint8_t>(), slots * 128, f->hidden);
    f->h_op.bind(f->h_packed.as<uint8_t>(), f->h_sf.as<uint8_t>(), slots * 128, f->inter);
    f->error.create();
    NMOE_CUDA(cudaDeviceSynchronize());
  } catch (const Failure& failure) {
    std::fprintf(stderr, "nmoe_ffn_create: %s\n", failure.message.c_str());
    return failure.status;
  }
  *out_ffn = f.release();
  return NMOE_OK;
}

void nmoe_ffn_destroy(nmoe_ffn* ffn) { delete ffn; }

nmoe_status nmoe_ffn_run(nmoe_ffn* ffn, void* stream_ptr, const void* input,
                         nmoe_dtype input_dtype, int64_t rows, float* output,
                         int32_t gemm_variant) {
  if (ffn == nullptr || input == nullptr || output == nullptr || rows <= 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (rows > ffn->max_rows) return NMOE_ERR_CAPACITY;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  try {
    TileClass tile_class = rows <= 32 ? kClassDecode : rows <= 256 ? kClassDecodeWide : kClassPrefill;
    if (gemm_variant >= 1 && gemm_variant <= 4) tile_class = static_cast<TileClass>(gemm_variant - 1);
    if (tile_class == kClassDecode && rows > 32) return NMOE_ERR_INVALID_ARGUMENT;
    NMOE_CUDA(launch_norm_quant(input, input_dtype == NMOE_BF16, static_cast<int>(rows),
                                ffn->hidden, nullptr, 0.0f, nullptr, ffn->a_packed.as<uint8_t>(),
                                nullptr, ffn->a_sf.as<uint8_t>(), k_blocks_of(ffn->hidden),
                                ffn->a_ts.as<float>(), stream));
    Schedule schedule;
    schedule.dense_rows = static_cast<int>(rows);
    run_expert_gemms(ffn->up, ffn->down, tile_class, ffn->a_op, ffn->a_ts.as<float>(), schedule,
                     ffn->h_packed.as<uint8_t>(), ffn->h_sf.as<uint8_t>(), ffn->h_op, output,
                     nullptr, 1, 0, nullptr, ffn->error.device.as<int32_t>(), ffn->num_sms,
                     stream);
    ffn->last_rows = static_cast<int>(rows);
  } catch (const Failure& failure) {
    ffn->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ffn_sync_status(nmoe_ffn* ffn, void* stream_ptr) {
  if (ffn == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  try {
    return ffn->error.sync(static_cast<cudaStream_t>(stream_ptr));
  } catch (const Failure& failure) {
    ffn->last_error = failure.message;
    return failure.status;
  }
}

nmoe_status nmoe_ffn_export_hidden(nmoe_ffn* ffn, void* stream_ptr, uint8_t* packed,
                                   uint8_t* scales) {
  if (ffn == nullptr || ffn->last_rows <= 0) return NMOE_ERR_INVALID_ARGUMENT;
  export_rows_kernel<<<ffn->last_rows, 128, 0, static_cast<cudaStream_t>(stream_ptr)>>>(
      ffn->h_packed.as<uint8_t>(), ffn->h_sf.as<uint8_t>(), nullptr, ffn->last_rows, ffn->inter,
      k_blocks_of(ffn->inter) * 4, packed, scales);
  return cudaGetLastError() == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}

}  // extern "C"

// ===========================================================================
// nmoe_layer
// ===========================================================================
enum { kStageCount = NMOE_STAGE_COUNT };

struct nmoe_layer {
  nmoe_config cfg{};
  int num_sms = 0;
  int local_experts = 0;
  int first_local_expert = 0;
  int max_row_tiles = 0;
  int decode_pairs_limit = 0;

  DeviceBuffer norm_weight, gate, bias, logit_offset;
  bool has_logit_offset = false;
  // two-pass router (tensor-core logits + FP64 re-evaluation of near-ties)
  bool fast_router = false;
  int fast_router_min_tokens = 256;
  float router_tie_margin = 2.0e-4f;
  DeviceBuffer gate_bf16, inv_rms;
  CUtensorMap gate_map;
  // bf16 inputs: the norm weight folded into the gate as three bf16 planes, and the map of
  // the last input the layer saw (its address and row count are part of the map)
  DeviceBuffer gate_planes;
  CUtensorMap planes_map;
  bool folded_router = false;
  CUtensorMap input_map;
  const void* input_map_base = nullptr;
  int input_map_rows = 0;
  // The FP32 normalised rows are needed by the FP64 logits kernel of small batches,
  // by the dense / scaled-FP8 linears and by the trace; the two-pass router of large
  // batches rebuilds them on the fly, so they are only written there while a trace may
  // be asked for (nmoe_layer_keep_trace).
  bool keep_trace = true;
  WeightStack up, down, shared_up, shared_down;

  // Latent projections and the dense / scaled-FP8 families (fc1_latent, fc2_latent,
  // shared_up, shared_down of expert_layer.cpp:534-617).  `latent` is the row length
  // the routed experts see; without projections it is the hidden size.
  int latent = 0;
  bool latent_mode = false;
  DenseLinear fc1, fc2, shared_up_dense, shared_down_dense;
  DeviceBuffer latent_rows, lat_packed, lat_sf_row_major, lat_ts;  // fc1 output and its NVFP4 form
  DeviceBuffer routed_latent, projected, shared_rows;               // [T][latent], [T][H], [T][H]
  DeviceBuffer fp8_tmp;                                             // activation round trip
  DeviceBuffer shared_raw;  // [T][S] FP32: shared_up output, activated in place
  DeviceBuffer sh_ts;       // per-row tensor scale of the quantised shared intermediate

  // The unfused activation path (nmoe_layer_set_unfused_activation): the up
  // projection's rows stay FP32 and are quantised in a pass of their own.
  bool unfused = false;
  DeviceBuffer u_raw, h_ts, unweighted_rows;
  int unweighted_tokens = 0;  // the unweighted down rows are kept for up to this many tokens

  // token-order scratch
  DeviceBuffer normalized, logits, top_index, top_weight;
  DeviceBuffer y_packed, y_sf_row_major, y_sf_tiled, y_ts;
  DeviceBuffer sh_packed, sh_sf;
  DeviceBuffer parts;
  // plan
  DeviceBuffer counts, cursor, slot0, row_tiles, num_row_tiles, pair_row;
  // expert-sorted scratch
  DeviceBuffer a_packed, a_sf, a_ts, a_weight, a_dest, h_packed, h_sf;

  // expert parallelism
  int ep_world = 1;
  int ep_rank = 0;
  int64_t max_pairs = 0;
  int64_t send_record_slots = 0;
  int record_bytes = 0;
  DeviceBuffer send_records, send_position, send_counts, send_offsets, rank_cursor, shared_out;

  // Peer window (nmoe_ep_window_*): one allocation per rank that the other
  // ranks map and write into: [records][returned rows][flags and counts].
  struct PeerWindow {
    bool attached = false;
    int64_t capacity = 0;  // pairs per (source rank, destination rank)
    RowKind rows_kind = kRowF16;
    DeviceBuffer local;
    size_t records_off = 0, rows_off = 0, flags_off = 0;
    std::vector<void*> peer_base;  // opened mappings, nullptr for this rank
    // u64[world] tables on the device: where this rank writes in rank r's window
    DeviceBuffer record_segments, row_segments, record_flag_slots, row_flag_slots, count_slots;
    DeviceBuffer epoch;  // uint32 step counter
    uint32_t* record_flags() const { return reinterpret_cast<uint32_t*>(local.as<uint8_t>() + flags_off); }
    uint32_t* row_flags() const { return record_flags() + 64; }
    int32_t* counts() const { return reinterpret_cast<int32_t*>(record_flags() + 128); }
    void close_peers() {
      for (void*& base : peer_base) {
        if (base != nullptr) cudaIpcCloseMemHandle(base);
        base = nullptr;
      }
      attached = false;
    }
  } window;

  ActivationOperand y_op, sh_op, a_op, h_op;
  ErrorSlot error;
  int last_tokens = 0;
  std::string last_error;
  RowKind last_parts_kind = kRowF32;
  bool last_unfused = false;
  bool last_normalized = true;
  bool force_fp32_parts = false;  // NMOE_PARTS_FP32=1: FP32 rows whatever the output type
  // CTA pairs for the prefill GEMMs (NMOE_GEMM_PAIR=1 turns them on), used once an
  // expert has this many rows on average.  Off by default: with the partner CTA's
  // "operands landed" relayed through a thread they measured slower than single CTAs.
  bool pair_gemms = false;
  int pair_min_rows = 640;
  // how long a kernel waits for a flag another GPU raises before it gives up with
  // kDevWaitTimeout (clock64 ticks; nmoe_layer_set_wait_limit_ms, NMOE_WAIT_LIMIT_MS)
  long long wait_limit_ticks = 1ll << 34;
  DeviceBuffer probe_epoch;  // nmoe_layer_wait_flag

  // Small batches: the shared expert runs on a stream of the layer's own beside the
  // router, plan and permute kernels (it needs only the quantised rows) and joins
  // before the combine.  Its GEMMs use a few dozen SMs at these sizes.
  cudaStream_t side_stream = nullptr;
  cudaEvent_t quant_done = nullptr, shared_done = nullptr;
  int fork_max_tokens = 1 << 30;  // (NMOE_FORK_MAX_TOKENS)
  bool window_fork_shared = false;    // nmoe_ep_window_fork_shared
  bool window_shared_pending = false;
  RowKind window_shared_kind = kRowF32;  // type of shared_out for the pending combine

  // Small batches are bound by launch overhead: the whole run is recorded once per
  // (token count, buffers, types) as a CUDA graph and replayed afterwards.
  // NMOE_GRAPH_MAX_TOKENS sets the largest batch handled this way (0 = never).
  struct RecordedRun {
    const void* input;
    void* output;
    int tokens;
    int in_dtype, out_dtype;
    RowKind parts_kind;
    bool normalized;
    cudaGraphExec_t exec;
    uint64_t last_use;
  };
  std::vector<RecordedRun> recorded;
  int graph_max_tokens = 256;
  uint64_t run_counter = 0;
  void drop_recorded() {
    for (RecordedRun& r : recorded) cudaGraphExecDestroy(r.exec);
    recorded.clear();
  }

  // optional per-stage CUDA events (nmoe_layer_enable_stage_timing)
  bool stage_timing = false;
  cudaEvent_t stage_events[kStageCount + 1] = {};
  ~nmoe_layer() {
    drop_recorded();
    window.close_peers();
    if (quant_done != nullptr) cudaEventDestroy(quant_done);
    if (shared_done != nullptr) cudaEventDestroy(shared_done);
    if (side_stream != nullptr) cudaStreamDestroy(side_stream);
    for (cudaEvent_t e : stage_events)
      if (e != nullptr) cudaEventDestroy(e);
  }
  void mark(int index, cudaStream_t stream) {
    if (stage_timing) cudaEventRecord(stage_events[index], stream);
  }
};

namespace {

// Everything whose size follows the token capacity.  Called at creation and by
// nmoe_layer_reserve_tokens; weights are not touched.
void allocate_scratch(nmoe_layer* L, size_t T) {
  L->drop_recorded();  // recorded runs hold the old buffers' addresses
  const nmoe_config& c = L->cfg;
  const int H = c.hidden_size, I = c.routed_expert_intermediate_size,
            S = c.shared_expert_intermediate_size, E = c.n_routed_experts, K = c.top_k;
  const int EL = L->local_experts, Lr = L->latent;
  const size_t token_slots = (T + 127) / 128;
  L->inv_rms.allocate(T * sizeof(float));
  L->normalized.allocate(T * H * sizeof(float));
  // (a split router pass 1 keeps up to four partial sums per logit for small batches)
  L->logits.allocate(std::min<size_t>(T, 4736) * 3 * E * sizeof(float) + T * E * sizeof(float));
  L->top_index.allocate(T * K * sizeof(int32_t));
  L->top_weight.allocate(T * K * sizeof(float));
  L->y_packed.allocate(token_slots * 128 * H / 2, true);
  L->y_sf_row_major.allocate(T * (H / 16));
  L->y_sf_tiled.allocate(tiled_sf_bytes(token_slots, H), true);
  L->y_ts.allocate(token_slots * 128 * sizeof(float), true);
  L->sh_packed.allocate(token_slots * 128 * S / 2, true);
  L->sh_sf.allocate(tiled_sf_bytes(token_slots, S), true);
  L->sh_ts.allocate(token_slots * 128 * sizeof(float), true);
  if (L->latent_mode) {
    L->latent_rows.allocate(T * Lr * sizeof(float));
    L->lat_packed.allocate(T * Lr / 2);
    L->lat_sf_row_major.allocate(T * (Lr / 16));
    L->lat_ts.allocate(T * sizeof(float));
    L->routed_latent.allocate(T * Lr * sizeof(float));
    L->projected.allocate(T * H * sizeof(float));
    L->shared_rows.allocate(T * H * sizeof(float));
  }
  if (L->fc1.fp8 || L->shared_up_dense.fp8 || L->shared_down_dense.fp8) {
    L->fp8_tmp.allocate(T * static_cast<size_t>(std::max(H, S)) * sizeof(float));
  }
  if (L->shared_up_dense.present || L->shared_down_dense.present || L->unfused) {
    L->shared_raw.allocate(T * S * sizeof(float));
  }
  if (L->ep_world == 1) {
    L->parts.allocate(T * (K + 1) * static_cast<size_t>(std::max(H, Lr)) * sizeof(float));
  }

  // Row tiles: every expert may leave one partly filled slot.  Small batches
  // use 32-row tiles (decode tile class), large ones 128-row tiles.
  // With expert parallelism the rows come from every rank: the capacity is
  // max_recv_pairs (default: twice the local pairs, i.e. 2x the uniform share).
  L->decode_pairs_limit = 32 * EL;
  const size_t local_pairs = T * K;
  const size_t pairs = L->ep_world == 1 ? local_pairs
                       : c.max_recv_pairs > 0 ? static_cast<size_t>(c.max_recv_pairs)
                                              : 2 * local_pairs;
  L->max_pairs = static_cast<int64_t>(pairs);
  // (an expert may leave a partly filled slot, and an empty one when pairs consume them)
  const size_t tiles_prefill = 2 * static_cast<size_t>(EL) + (pairs + 127) / 128;
  const size_t tiles_decode = EL + (std::min<size_t>(pairs, L->decode_pairs_limit) + 31) / 32;
  L->max_row_tiles = static_cast<int>(std::max(tiles_prefill, tiles_decode));
  const size_t slots = static_cast<size_t>(L->max_row_tiles);
  L->counts.allocate(E * sizeof(int32_t), true);
  L->cursor.allocate(E * sizeof(int32_t), true);
  L->slot0.allocate(E * sizeof(int32_t), true);
  L->row_tiles.allocate(slots * sizeof(RowTile), true);
  L->num_row_tiles.allocate(sizeof(int32_t), true);
  L->pair_row.allocate(pairs * sizeof(int32_t), true);
  if (L->ep_world > 1) {
    L->record_bytes = dispatch_record_bytes(H);
    // room for the compact layout and for fixed-capacity segments up to 2x the mean
    L->send_record_slots = static_cast<int64_t>(2 * local_pairs + 64 * 16);
    L->send_records.allocate(static_cast<size_t>(L->send_record_slots) * L->record_bytes, true);
    L->send_position.allocate(local_pairs * sizeof(int32_t), true);
    L->send_counts.allocate(64 * sizeof(int32_t), true);
    L->send_offsets.allocate(64 * sizeof(int32_t), true);
    L->rank_cursor.allocate(64 * sizeof(int32_t), true);
    L->shared_out.allocate(T * H * sizeof(float));
  }
  L->a_packed.allocate(slots * 128 * Lr / 2, true);
  L->a_sf.allocate(tiled_sf_bytes(slots, Lr), true);
  L->a_ts.allocate(slots * 128 * sizeof(float), true);
  L->a_weight.allocate(slots * 128 * sizeof(float), true);
  L->a_dest.allocate(slots * 128 * sizeof(int32_t), true);
  L->h_packed.allocate(slots * 128 * I / 2, true);
  L->h_sf.allocate(tiled_sf_bytes(slots, I), true);
  L->h_ts.allocate(slots * 128 * sizeof(float), true);
  if (L->unfused) {
    L->u_raw.allocate(slots * 128 * I * sizeof(float), true);
    L->unweighted_tokens = static_cast<int>(std::min<size_t>(T, 64));
    L->unweighted_rows.allocate(static_cast<size_t>(L->unweighted_tokens) * (K + 1) *
                                std::max(H, Lr) * sizeof(float), true);
  }

  L->y_op.bind(L->y_packed.as<uint8_t>(), L->y_sf_tiled.as<uint8_t>(), token_slots * 128, H);
  L->sh_op.bind(L->sh_packed.as<uint8_t>(), L->sh_sf.as<uint8_t>(), token_slots * 128, S);
  L->a_op.bind(L->a_packed.as<uint8_t>(), L->a_sf.as<uint8_t>(), slots * 128, Lr);
  L->h_op.bind(L->h_packed.as<uint8_t>(), L->h_sf.as<uint8_t>(), slots * 128, I);
  L->cfg.max_tokens = static_cast<int32_t>(T);
  L->last_tokens = 0;
}

void layer_create_impl(nmoe_layer* L, const nmoe_config& c, const nmoe_weights& w) {
  // config checks of expert_layer.cpp:505-528
  NMOE_REQUIRE(c.hidden_size > 0 && c.moe_latent_size > 0 &&
                   c.routed_expert_intermediate_size > 0 &&
                   c.shared_expert_intermediate_size > 0 && c.n_routed_experts > 0 &&
                   c.top_k > 0 && c.top_k <= c.n_routed_experts && c.n_group > 0 &&
                   c.topk_group > 0 && c.n_routed_experts % c.n_group == 0 &&
                   c.rms_epsilon > 0.0f && c.max_tokens > 0,
               "invalid config");
  const bool has_fc1 = w.fc1_latent.family != NMOE_LINEAR_ABSENT;
  const bool has_fc2 = w.fc2_latent.family != NMOE_LINEAR_ABSENT;
  NMOE_REQUIRE(has_fc1 == has_fc2, "fc1_latent and fc2_latent come together");
  NMOE_REQUIRE(has_fc1 || c.moe_latent_size == c.hidden_size,
               "moe_latent_size != hidden_size needs the fc1_latent / fc2_latent projections");
  NMOE_REQUIRE(w.fc2_latent.family != NMOE_LINEAR_SCALED_FP8,
               "fc2_latent is a dense projection (expert_layer.cpp:617-626)");
  NMOE_REQUIRE(c.n_routed_experts % 32 == 0 && c.n_routed_experts <= 512 && c.top_k <= 32 &&
                   c.n_group <= 32,
               "router limits: experts % 32 == 0, experts <= 512, top_k <= 32, n_group <= 32");
  NMOE_REQUIRE(c.hidden_size % 64 == 0 && c.moe_latent_size % 64 == 0 &&
                   c.routed_expert_intermediate_size % 64 == 0 &&
                   c.shared_expert_intermediate_size % 64 == 0,
               "hidden, latent and intermediate sizes must be multiples of 64");
  // Expert parallelism: this device holds experts [first_local_expert,
  // first_local_expert + n_local_experts), an equal share of all of them.
  NMOE_REQUIRE(w.n_local_experts > 0 && c.n_routed_experts % w.n_local_experts == 0 &&
                   w.first_local_expert >= 0 && w.first_local_expert % w.n_local_experts == 0 &&
                   w.first_local_expert + w.n_local_experts <= c.n_routed_experts &&
                   c.n_routed_experts / w.n_local_experts <= 64,
               "local experts must be an equal, aligned share of the routed experts");
  NMOE_REQUIRE(w.routed_up != nullptr && w.routed_down != nullptr, "missing routed expert weights");

  L->cfg = c;
  L->num_sms = device_sm_count();
  L->force_fp32_parts = std::getenv("NMOE_PARTS_FP32") != nullptr;
  if (const char* env = std::getenv("NMOE_GEMM_PAIR")) L->pair_gemms = std::atoi(env) != 0;
  if (const char* env = std::getenv("NMOE_GRAPH_MAX_TOKENS")) L->graph_max_tokens = std::atoi(env);
  if (const char* env = std::getenv("NMOE_GEMM_PAIR_MIN_ROWS")) L->pair_min_rows = std::atoi(env);
  if (const char* env = std::getenv("NMOE_WAIT_LIMIT_MS")) {
    const double ms = std::strtod(env, nullptr);
    if (ms > 0.0) L->wait_limit_ticks = ticks_from_ms(ms);
  }
  if (const char* env = std::getenv("NMOE_FORK_MAX_TOKENS")) L->fork_max_tokens = std::atoi(env);
  if (std::getenv("NMOE_NO_SHARED_FORK") == nullptr) {
    NMOE_CUDA(cudaStreamCreateWithFlags(&L->side_stream, cudaStreamNonBlocking));
    NMOE_CUDA(cudaEventCreateWithFlags(&L->quant_done, cudaEventDisableTiming));
    NMOE_CUDA(cudaEventCreateWithFlags(&L->shared_done, cudaEventDisableTiming));
  }
  L->local_experts = w.n_local_experts;
  L->first_local_expert = w.first_local_expert;
  cudaStream_t stream = nullptr;
  const int H = c.hidden_size, I = c.routed_expert_intermediate_size,
            S = c.shared_expert_intermediate_size, E = c.n_routed_experts;
  const int EL = w.n_local_experts;
  L->ep_world = E / EL;
  L->ep_rank = w.first_local_expert / EL;
  L->latent = c.moe_latent_size;
  L->latent_mode = has_fc1;
  const int Lr = L->latent;
  const bool dense_shared = w.shared_up_linear.family != NMOE_LINEAR_ABSENT ||
                            w.shared_down_linear.family != NMOE_LINEAR_ABSENT;
  if (L->ep_world > 1 && (L->latent_mode || dense_shared)) {
    throw Failure{NMOE_ERR_UNSUPPORTED,
                  "expert parallelism is built for the all-NVFP4 layer without latent projections"};
  }

  upload_dense_fp32(w.input_norm_weight, H, "input_norm_weight", &L->norm_weight, stream);
  upload_dense_fp32(w.gate_weight, static_cast<size_t>(E) * H, "gate_weight", &L->gate, stream);
  upload_dense_fp32(w.gate_score_correction_bias, E, "gate_score_correction_bias", &L->bias, stream);
  if (w.gate_logit_offset != nullptr) {
    L->logit_offset.allocate(E * sizeof(float));
    NMOE_CUDA(cudaMemcpyAsync(L->logit_offset.as<float>(), w.gate_logit_offset,
                              E * sizeof(float), cudaMemcpyDefault, stream));
    L->has_logit_offset = true;
  }
  // routed experts act on latent rows: up_proj [I][latent], down_proj [latent][I]
  // (shape checks of expert_layer.cpp:646-689)
  L->up.upload(w.routed_up, EL, I, Lr, true, "routed up_proj", stream);
  L->down.upload(w.routed_down, EL, Lr, I, false, "routed down_proj", stream);
  if (L->latent_mode) {
    L->fc1.upload(w.fc1_latent, Lr, H, "fc1_latent", stream);
    L->fc2.upload(w.fc2_latent, H, Lr, "fc2_latent", stream);
  }
  if (w.shared_up_linear.family != NMOE_LINEAR_ABSENT) {
    L->shared_up_dense.upload(w.shared_up_linear, S, H, "shared up_proj", stream);
  } else {
    L->shared_up.upload(&w.shared_up, 1, S, H, true, "shared up_proj", stream);
  }
  if (w.shared_down_linear.family != NMOE_LINEAR_ABSENT) {
    L->shared_down_dense.upload(w.shared_down_linear, H, S, "shared down_proj", stream);
  } else {
    L->shared_down.upload(&w.shared_down, 1, H, S, false, "shared down_proj", stream);
  }

  // The tensor-core pass needs the gate exactly in bf16.
  L->fast_router = w.gate_weight.dtype == NMOE_BF16 && c.n_group == 1 && E % 32 == 0 &&
                   E <= 256 && H % 64 == 0 && std::getenv("NMOE_ROUTER_FP64_ONLY") == nullptr;
  if (L->fast_router) {
    L->gate_bf16.allocate(static_cast<size_t>(E) * H * 2);
    NMOE_CUDA(cudaMemcpyAsync(L->gate_bf16.as<void>(), w.gate_weight.data,
                              static_cast<size_t>(E) * H * 2, cudaMemcpyDefault, stream));
    L->gate_map = make_bf16_map(L->gate_bf16.as<void>(), E, H, E);
    L->folded_router = std::getenv("NMOE_ROUTER_SPLIT_INPUT") == nullptr;
    if (L->folded_router) {
      L->gate_planes.allocate(static_cast<size_t>(3) * E * H * 2);
      NMOE_CUDA(launch_fold_gate(L->gate_bf16.as<__nv_bfloat16>(), L->norm_weight.as<float>(), E, H,
                                 L->gate_planes.as<__nv_bfloat16>(), stream));
      L->planes_map = make_bf16_map(L->gate_planes.as<void>(), static_cast<size_t>(3) * E, H, E);
    }
    if (const char* env = std::getenv("NMOE_ROUTER_TIE_MARGIN")) L->router_tie_margin = std::strtof(env, nullptr);
    if (const char* env = std::getenv("NMOE_ROUTER_FAST_MIN_TOKENS")) L->fast_router_min_tokens = std::atoi(env);
  }
  L->unfused = std::getenv("NMOE_UNFUSED_ACTIVATION") != nullptr;
  allocate_scratch(L, static_cast<size_t>(c.max_tokens));
  L->error.create();
  NMOE_CUDA(cudaDeviceSynchronize());
}

// y = x W^T of a dense / scaled-FP8 linear, FP64 accumulation.
void run_linear(nmoe_layer* L, const DenseLinear& linear, const float* in_rows, int rows,
                float* out_rows, cudaStream_t stream) {
  const float* source = in_rows;
  if (linear.fp8) {
    NMOE_CUDA(launch_fp8_round_trip(in_rows, static_cast<size_t>(rows) * linear.in,
                                    linear.input_scale, L->fp8_tmp.as<float>(), stream));
    source = L->fp8_tmp.as<float>();
  }
  NMOE_CUDA(launch_router_logits(source, linear.weight.as<float>(), nullptr, rows, linear.out,
                                 linear.in, out_rows, stream));
}

// RMSNorm + activation quantiser + router: fills normalized, y_*, logits,
// top_index / top_weight and the per-expert histogram `counts` (global ids).
void route_tokens(nmoe_layer* L, cudaStream_t stream, const void* input, nmoe_dtype in_dtype,
                  int tokens, cudaEvent_t after_quantise = nullptr,
                  bool fork_after_logits = false) {
  const nmoe_config& c = L->cfg;
  const int H = c.hidden_size, E = c.n_routed_experts, K = c.top_k;
  int32_t* error = L->error.device.as<int32_t>();
  L->mark(0, stream);
  const bool two_pass_router = L->fast_router && tokens >= L->fast_router_min_tokens;
  const bool in_bf16 = in_dtype == NMOE_BF16;
  const bool want_normalized = !two_pass_router || L->keep_trace || L->latent_mode ||
                               L->shared_up_dense.present;
  // RMSNorm (:795-796) fused with the activation quantiser every expert's
  // up_proj applies to the same normalised row (:913 -> nvfp4_packing.cpp:90)
  NMOE_CUDA(launch_norm_quant(input, in_bf16, tokens, H, L->norm_weight.as<float>(),
                              c.rms_epsilon, want_normalized ? L->normalized.as<float>() : nullptr,
                              L->y_packed.as<uint8_t>(), L->y_sf_row_major.as<uint8_t>(),
                              L->y_sf_tiled.as<uint8_t>(), k_blocks_of(H), L->y_ts.as<float>(),
                              stream, L->inv_rms.as<float>()));
  L->last_normalized = want_normalized;
  if (after_quantise != nullptr && !fork_after_logits) {
    NMOE_CUDA(cudaEventRecord(after_quantise, stream));
  }
  L->mark(1, stream);
  // gate projection (:797-799) and top-k (:881)
  NMOE_CUDA(cudaMemsetAsync(L->counts.as<int32_t>(), 0, E * sizeof(int32_t), stream));
  const float* offset = L->has_logit_offset ? L->logit_offset.as<float>() : nullptr;
  if (two_pass_router) {
    int logit_splits = 1;
    if (L->folded_router && in_bf16 && reinterpret_cast<uintptr_t>(input) % 16 == 0) {
      if (L->input_map_base != input || L->input_map_rows != tokens) {
        L->input_map = make_bf16_map(input, tokens, H, 128);
        L->input_map_base = input;
        L->input_map_rows = tokens;
      }
      logit_splits = router_folded_splits(tokens, H, L->num_sms);
      NMOE_CUDA(launch_router_folded_logits(L->input_map, L->planes_map, L->inv_rms.as<float>(),
                                            tokens, E, H, logit_splits, L->logits.as<float>(),
                                            error, stream));
    } else {
      NMOE_CUDA(launch_router_fast_logits(input, in_bf16, L->inv_rms.as<float>(),
                                          L->norm_weight.as<float>(), L->gate_map, tokens, E, H,
                                          L->logits.as<float>(), error, stream));
    }
    // A stream forked here runs the shared expert beside the selection, plan and permute
    // kernels; forked before pass 1 its persistent GEMM CTAs would hold the shared memory
    // the pass-1 CTAs need.
    if (after_quantise != nullptr && fork_after_logits) {
      NMOE_CUDA(cudaEventRecord(after_quantise, stream));
    }
    L->mark(2, stream);
    NMOE_CUDA(launch_router_select_exact(
        L->logits.as<float>(), logit_splits, input, in_bf16, L->inv_rms.as<float>(),
        L->norm_weight.as<float>(), L->gate_bf16.as<__nv_bfloat16>(), offset,
        L->bias.as<float>(), tokens, E, H, K, c.norm_topk_prob != 0, c.routed_scaling_factor,
        L->router_tie_margin, L->top_index.as<int32_t>(), L->top_weight.as<float>(),
        L->counts.as<int32_t>(), stream));
  } else {
    NMOE_CUDA(launch_router_logits(L->normalized.as<float>(), L->gate.as<float>(), offset, tokens,
                                   E, H, L->logits.as<float>(), stream));
    L->mark(2, stream);
    NMOE_CUDA(launch_router_topk(L->logits.as<float>(), L->bias.as<float>(), tokens, E, K,
                                 c.n_group, c.topk_group, c.norm_topk_prob != 0,
                                 c.routed_scaling_factor, L->top_index.as<int32_t>(),
                                 L->top_weight.as<float>(), L->counts.as<int32_t>(), stream));
  }
  L->mark(3, stream);
}

// One expert FFN over rows that are already quantised, fused or unfused.
//   fused:   up GEMM (relu^2 + NVFP4 quantise in the epilogue, tensor scale 1) -> down GEMM
//   unfused: up GEMM keeps relu^2 rows in FP32 (`raw_rows`) -> per-row quantiser with
//            the row's own tensor scale (nvfp4_packing.cpp:119-153) -> down GEMM
struct FfnBuffers {
  uint8_t* hidden_packed;
  uint8_t* hidden_sf;
  float* hidden_ts;
  const ActivationOperand* hidden;
  float* raw_rows;  // unfused only: [row slots * 128][intermediate] FP32
  int raw_row_count;
};

void run_ffn(nmoe_layer* L, bool unfused, const WeightStack& up, const WeightStack& down,
             TileClass tile_class, const ActivationOperand& a, const float* a_ts,
             const Schedule& schedule, const FfnBuffers& buffers, void* out_rows,
             const int32_t* dest_row, int dest_mul, int dest_add, const float* row_weight,
             cudaStream_t stream, cudaEvent_t between, RowKind out_kind, RowSegments segments) {
  int32_t* error = L->error.device.as<int32_t>();
  if (!unfused) {
    run_expert_gemms(up, down, tile_class, a, a_ts, schedule, buffers.hidden_packed,
                     buffers.hidden_sf, *buffers.hidden, out_rows, dest_row, dest_mul, dest_add,
                     row_weight, error, L->num_sms, stream, between, out_kind, segments);
    return;
  }
  // the row-storing epilogue exists for the BN = 128 tile shapes
  const TileClass raw_class =
      tile_class == kClassPrefill || tile_class == kClassPair ? kClassDecodeWide : tile_class;
  run_down_gemm(up, raw_class, a, a_ts, schedule, buffers.raw_rows, nullptr, 1, 0, nullptr,
                /*relu2=*/true, error, L->num_sms, stream, kRowF32, RowSegments());
  NMOE_CUDA(launch_norm_quant(buffers.raw_rows, false, buffers.raw_row_count, up.n, nullptr, 0.0f,
                              nullptr, buffers.hidden_packed, nullptr, buffers.hidden_sf,
                              k_blocks_of(up.n), buffers.hidden_ts, stream));
  if (between != nullptr) cudaEventRecord(between, stream);
  run_down_gemm(down, tile_class, *buffers.hidden, buffers.hidden_ts, schedule, out_rows, dest_row,
                dest_mul, dest_add, row_weight, /*relu2=*/false, error, L->num_sms, stream,
                out_kind, segments);
}

// Plan + permute + the two grouped GEMMs over `pairs` (row, slot) pairs whose
// per-local-expert histogram is already in `counts`.
void routed_experts(nmoe_layer* L, cudaStream_t stream, const PermuteSource& source, int pairs,
                    int dest_stride, void* out_rows, RowKind out_kind,
                    RowSegments segments = RowSegments()) {
  const int Lr = L->latent;
  int32_t* error = L->error.device.as<int32_t>();
  const bool decode = static_cast<long long>(pairs) <= L->decode_pairs_limit / 2;
  const bool pair = !decode && L->pair_gemms && !L->unfused && (L->num_sms & 1) == 0 &&
                    pairs / L->local_experts >= L->pair_min_rows;
  const TileClass routed_class = decode ? kClassDecode : pair ? kClassPair : kClassPrefill;
  const int tile_rows = decode ? 32 : 128;
  PlanBuffers plan;
  plan.expert_counts = L->counts.as<int32_t>();
  plan.expert_cursor = L->cursor.as<int32_t>();
  plan.expert_slot0 = L->slot0.as<int32_t>();
  plan.row_tiles = L->row_tiles.as<RowTile>();
  plan.num_row_tiles = L->num_row_tiles.as<int32_t>();
  NMOE_CUDA(launch_route_plan(plan, L->local_experts, tile_rows, pair ? 2 : 1, L->max_row_tiles,
                              error, stream));
  L->mark(4, stream);
  NMOE_CUDA(launch_permute(plan, source, pairs, L->local_experts, tile_rows, L->max_row_tiles, Lr,
                           k_blocks_of(Lr),
                           L->a_packed.as<uint8_t>(), L->a_sf.as<uint8_t>(), L->a_ts.as<float>(),
                           L->a_weight.as<float>(), L->a_dest.as<int32_t>(),
                           L->ep_world == 1 ? L->pair_row.as<int32_t>() : nullptr, dest_stride,
                           stream));
  L->mark(5, stream);
  // routed experts (:896-954)
  Schedule routed;
  routed.row_tiles = L->row_tiles.as<RowTile>();
  routed.num_row_tiles = L->num_row_tiles.as<int32_t>();
  FfnBuffers buffers{L->h_packed.as<uint8_t>(), L->h_sf.as<uint8_t>(), L->h_ts.as<float>(),
                     &L->h_op, L->u_raw.as<float>(), L->max_row_tiles * 128};
  run_ffn(L, L->unfused, L->up, L->down, routed_class, L->a_op, L->a_ts.as<float>(), routed,
          buffers, out_rows, L->a_dest.as<int32_t>(), 1, 0, L->a_weight.as<float>(), stream,
          L->stage_timing ? L->stage_events[6] : nullptr, out_kind, segments);
  if (L->unfused && L->ep_world == 1 && pairs <= L->unweighted_tokens * L->cfg.top_k) {
    // the down_proj rows before the routing weight (routed_expert_outputs of the trace)
    run_down_gemm(L->down, routed_class, L->h_op, L->h_ts.as<float>(), routed,
                  L->unweighted_rows.as<float>(), L->a_dest.as<int32_t>(), 1, 0, nullptr, false,
                  error, L->num_sms, stream, kRowF32, RowSegments());
  }
}

// shared expert (:814-818, :956-964, :981-1005) on the token-order rows
void shared_expert(nmoe_layer* L, cudaStream_t stream, int tokens, void* out_rows, int dest_mul,
                   int dest_add, cudaEvent_t between, RowKind out_kind = kRowF32) {
  const int H = L->cfg.hidden_size, S = L->cfg.shared_expert_intermediate_size;
  const bool pair = L->pair_gemms && (L->num_sms & 1) == 0 && tokens >= 1024;
  const TileClass shared_class = tokens <= 32    ? kClassDecode
                                 : tokens <= 256 ? kClassDecodeWide
                                 : pair          ? kClassPair
                                                 : kClassPrefill;
  Schedule shared;
  shared.dense_rows = tokens;
  int32_t* error = L->error.device.as<int32_t>();
  if (!L->shared_up_dense.present && !L->shared_down_dense.present) {
    FfnBuffers buffers{L->sh_packed.as<uint8_t>(), L->sh_sf.as<uint8_t>(), L->sh_ts.as<float>(),
                       &L->sh_op, L->shared_raw.as<float>(), tokens};
    run_ffn(L, L->unfused, L->shared_up, L->shared_down, shared_class, L->y_op,
            L->y_ts.as<float>(), shared, buffers, out_rows, nullptr, dest_mul, dest_add, nullptr,
            stream, between, out_kind, RowSegments());
    return;
  }
  // shared_up -> FP32 rows -> relu^2 in place (:956-964)
  float* raw = L->shared_raw.as<float>();
  if (L->shared_up_dense.present) {
    run_linear(L, L->shared_up_dense, L->normalized.as<float>(), tokens, raw, stream);
    NMOE_CUDA(launch_relu2(raw, static_cast<size_t>(tokens) * S, stream));
  } else {
    run_down_gemm(L->shared_up,
                  shared_class == kClassPrefill || shared_class == kClassPair ? kClassDecodeWide
                                                                              : shared_class,
                  L->y_op, L->y_ts.as<float>(), shared, raw, nullptr, 1, 0, nullptr, true, error,
                  L->num_sms, stream, kRowF32, RowSegments());
  }
  if (between != nullptr) cudaEventRecord(between, stream);
  if (L->shared_down_dense.present) {
    // dense / scaled-FP8 down projection (:1006-1045) straight from the FP32 rows;
    // only the latent data flow (FP32 rows of `hidden` per token) reaches this
    NMOE_REQUIRE(dest_mul == 1 && dest_add == 0 && out_kind == kRowF32,
                 "a dense shared_down writes FP32 token rows");
    run_linear(L, L->shared_down_dense, raw, tokens, static_cast<float*>(out_rows), stream);
    (void)H;
    return;
  }
  // NVFP4 down projection through the host linear's own packing step (:981-1005)
  NMOE_CUDA(launch_norm_quant(raw, false, tokens, S, nullptr, 0.0f, nullptr,
                              L->sh_packed.as<uint8_t>(), nullptr, L->sh_sf.as<uint8_t>(),
                              k_blocks_of(S), L->sh_ts.as<float>(), stream));
  run_down_gemm(L->shared_down, shared_class, L->sh_op, L->sh_ts.as<float>(), shared, out_rows,
                nullptr, dest_mul, dest_add, nullptr, false, error, L->num_sms, stream, out_kind,
                RowSegments());
}

PermuteSource local_source(nmoe_layer* L) {
  const int H = L->cfg.hidden_size;
  PermuteSource source;
  source.packed = L->y_packed.as<uint8_t>();
  source.packed_stride = static_cast<size_t>(H) / 2;
  source.sf = L->y_sf_row_major.as<uint8_t>();
  source.sf_stride = static_cast<size_t>(H) / 16;
  source.tensor_scale = L->y_ts.as<float>();
  source.tensor_scale_stride = sizeof(float);
  source.weight = L->top_weight.as<float>();
  source.weight_stride = sizeof(float);
  source.expert = L->top_index.as<int32_t>();
  source.expert_stride = sizeof(int32_t);
  source.pairs_per_row = L->cfg.top_k;
  return source;
}

void layer_run_impl(nmoe_layer* L, cudaStream_t stream, const void* input, nmoe_dtype in_dtype,
                    int tokens, void* output, nmoe_dtype out_dtype) {
  const nmoe_config& c = L->cfg;
  const int H = c.hidden_size, K = c.top_k, Lr = L->latent;
  const bool dense_shared = L->shared_up_dense.present || L->shared_down_dense.present;
  // The per-(token, slot) rows of the down projection and the shared expert's row
  // wait in `parts` for the combine.  They carry the precision the output needs: FP32
  // rows for an FP32 result (the reference's arithmetic, bit for bit in the sums),
  // binary16 rows for a bf16 result: half the bytes of the layer's largest write and
  // read, and eight times finer than the bf16 the sum is rounded to in the end.
  const RowKind parts_kind = out_dtype == NMOE_BF16 && !L->force_fp32_parts && !L->latent_mode
                                 ? kRowF16 : kRowF32;
  const bool fork = L->side_stream != nullptr && !L->stage_timing &&
                    tokens <= L->fork_max_tokens && !L->latent_mode && !dense_shared;
  const bool two_pass = L->fast_router && tokens >= L->fast_router_min_tokens;
  route_tokens(L, stream, input, in_dtype, tokens, fork ? L->quant_done : nullptr,
               fork && two_pass);
  L->last_tokens = tokens;
  L->last_parts_kind = parts_kind;
  L->last_unfused = L->unfused;
  if (L->latent_mode) {
    // latent = fc1_latent(normalized) (:809-813); every routed expert's up_proj packs
    // the same latent row (:913 -> nvfp4_packing.cpp:90)
    run_linear(L, L->fc1, L->normalized.as<float>(), tokens, L->latent_rows.as<float>(), stream);
    NMOE_CUDA(launch_norm_quant(L->latent_rows.as<float>(), false, tokens, Lr, nullptr, 0.0f,
                                nullptr, L->lat_packed.as<uint8_t>(),
                                L->lat_sf_row_major.as<uint8_t>(), nullptr, 0,
                                L->lat_ts.as<float>(), stream));
    PermuteSource source = local_source(L);
    source.packed = L->lat_packed.as<uint8_t>();
    source.packed_stride = static_cast<size_t>(Lr) / 2;
    source.sf = L->lat_sf_row_major.as<uint8_t>();
    source.sf_stride = static_cast<size_t>(Lr) / 16;
    source.tensor_scale = L->lat_ts.as<float>();
    routed_experts(L, stream, source, tokens * K, K, L->parts.as<void>(), kRowF32);
    L->mark(7, stream);
    shared_expert(L, stream, tokens, L->shared_rows.as<void>(), 1, 0,
                  L->stage_timing ? L->stage_events[8] : nullptr, kRowF32);
    L->mark(9, stream);
    // routed sum in selection order (:951-953), fc2_latent (:1047-1053), mixer and
    // residual (:1064-1069)
    NMOE_CUDA(launch_sum_parts(L->parts.as<float>(), tokens, Lr, K, L->routed_latent.as<float>(),
                               stream));
    run_linear(L, L->fc2, L->routed_latent.as<float>(), tokens, L->projected.as<float>(), stream);
    NMOE_CUDA(launch_mixer(input, in_dtype == NMOE_BF16, L->projected.as<float>(),
                           L->shared_rows.as<float>(), tokens, H, output, out_dtype == NMOE_BF16,
                           stream));
    L->mark(10, stream);
    return;
  }
  if (fork) {
    NMOE_CUDA(cudaStreamWaitEvent(L->side_stream, L->quant_done, 0));
    shared_expert(L, L->side_stream, tokens, L->parts.as<void>(), K + 1, K, nullptr, parts_kind);
    NMOE_CUDA(cudaEventRecord(L->shared_done, L->side_stream));
  }
  routed_experts(L, stream, local_source(L), tokens * K, K + 1, L->parts.as<void>(), parts_kind);
  L->mark(7, stream);
  if (fork) {
    NMOE_CUDA(cudaStreamWaitEvent(stream, L->shared_done, 0));
  } else {
    shared_expert(L, stream, tokens, L->parts.as<void>(), K + 1, K,
                  L->stage_timing ? L->stage_events[8] : nullptr, parts_kind);
  }
  // routed sum in selection order, mixer and residual (:951-953, :1064-1069)
  L->mark(9, stream);
  NMOE_CUDA(launch_combine(input, in_dtype == NMOE_BF16, L->parts.as<void>(), parts_kind, tokens,
                           H, K, output, out_dtype == NMOE_BF16, L->error.device.as<int32_t>(),
                           stream));
  L->mark(10, stream);
}

// nmoe_layer_run: small batches replay a recorded CUDA graph of the same run.
void run_recorded_or_eager(nmoe_layer* L, cudaStream_t stream, const void* input,
                           nmoe_dtype in_dtype, int tokens, void* output, nmoe_dtype out_dtype) {
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  const bool can_query = cudaStreamIsCapturing(stream, &capturing) == cudaSuccess;
  if (!can_query) cudaGetLastError();
  const bool eligible = tokens <= L->graph_max_tokens && !L->stage_timing && !L->unfused &&
                        can_query && capturing == cudaStreamCaptureStatusNone &&
                        stream != nullptr && stream != cudaStreamLegacy;
  if (!eligible) {
    layer_run_impl(L, stream, input, in_dtype, tokens, output, out_dtype);
    return;
  }
  ++L->run_counter;
  for (nmoe_layer::RecordedRun& r : L->recorded) {
    if (r.input == input && r.output == output && r.tokens == tokens &&
        r.in_dtype == in_dtype && r.out_dtype == out_dtype) {
      r.last_use = L->run_counter;
      NMOE_CUDA(cudaGraphLaunch(r.exec, stream));
      L->last_tokens = tokens;
      L->last_parts_kind = r.parts_kind;
      L->last_normalized = r.normalized;
      L->last_unfused = false;
      return;
    }
  }
  // record: the launches below go into a graph instead of onto the stream
  if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    cudaGetLastError();      // this stream cannot be captured (e.g. the legacy default stream)
    L->graph_max_tokens = 0;  // stay eager from now on
    layer_run_impl(L, stream, input, in_dtype, tokens, output, out_dtype);
    return;
  }
  cudaGraph_t graph = nullptr;
  try {
    layer_run_impl(L, stream, input, in_dtype, tokens, output, out_dtype);
  } catch (...) {
    cudaStreamEndCapture(stream, &graph);
    if (graph != nullptr) cudaGraphDestroy(graph);
    cudaGetLastError();
    throw;
  }
  NMOE_CUDA(cudaStreamEndCapture(stream, &graph));
  cudaGraphExec_t exec = nullptr;
  const cudaError_t made = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (made != cudaSuccess) {
    cudaGetLastError();
    L->graph_max_tokens = 0;
    layer_run_impl(L, stream, input, in_dtype, tokens, output, out_dtype);
    return;
  }
  if (L->recorded.size() >= 16) {  // forget the run that was used longest ago
    size_t oldest = 0;
    for (size_t i = 1; i < L->recorded.size(); ++i) {
      if (L->recorded[i].last_use < L->recorded[oldest].last_use) oldest = i;
    }
    cudaGraphExecDestroy(L->recorded[oldest].exec);
    L->recorded.erase(L->recorded.begin() + static_cast<long>(oldest));
  }
  L->recorded.push_back(nmoe_layer::RecordedRun{input, output, tokens, in_dtype, out_dtype,
                                                L->last_parts_kind, L->last_normalized, exec,
                                                L->run_counter});
  NMOE_CUDA(cudaGraphLaunch(exec, stream));
}

}  // namespace

extern "C" {

nmoe_status nmoe_layer_create(const nmoe_config* config, const nmoe_weights* weights,
                              nmoe_layer** out_layer) {
  if (config == nullptr || weights == nullptr || out_layer == nullptr) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  *out_layer = nullptr;
  std::unique_ptr<nmoe_layer> layer(new (std::nothrow) nmoe_layer);
  if (!layer) return NMOE_ERR_CUDA;
  try {
    layer_create_impl(layer.get(), *config, *weights);
  } catch (const Failure& failure) {
    if (std::getenv("NEMOTRON_FORWARD_DEBUG") != nullptr) {
      std::fprintf(stderr, "expert_layer_create: layer %d failed: %s\n", config->layer_index,
                   failure.message.c_str());
    }
    return failure.status;
  }
  *out_layer = layer.release();
  return NMOE_OK;
}

void nmoe_layer_destroy(nmoe_layer* layer) { delete layer; }

nmoe_status nmoe_layer_run(nmoe_layer* layer, void* stream, const void* input,
                           nmoe_dtype input_dtype, int64_t tokens, void* output,
                           nmoe_dtype output_dtype) {
  if (layer == nullptr || input == nullptr || output == nullptr || tokens <= 0 ||
      input == output || (input_dtype != NMOE_F32 && input_dtype != NMOE_BF16) ||
      (output_dtype != NMOE_F32 && output_dtype != NMOE_BF16)) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (tokens > layer->cfg.max_tokens) return NMOE_ERR_CAPACITY;
  if (layer->ep_world != 1) return NMOE_ERR_INVALID_ARGUMENT;  // use the nmoe_ep_* stages
  try {
    run_recorded_or_eager(layer, static_cast<cudaStream_t>(stream), input, input_dtype,
                          static_cast<int>(tokens), output, output_dtype);
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    if (std::getenv("NEMOTRON_FORWARD_DEBUG") != nullptr) {
      std::fprintf(stderr, "expert_layer: %s\n", failure.message.c_str());
    }
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_layer_sync_status(nmoe_layer* layer, void* stream) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  try {
    const nmoe_status status = layer->error.sync(static_cast<cudaStream_t>(stream));
    if (status != NMOE_OK) layer->last_error = nmoe_status_string(status);
    return status;
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
}

nmoe_status nmoe_layer_reserve_sms(nmoe_layer* layer, int32_t reserved_sms) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  const int all = device_sm_count();
  if (reserved_sms < 0 || reserved_sms >= all) return NMOE_ERR_INVALID_ARGUMENT;
  layer->drop_recorded();
  layer->num_sms = all - reserved_sms;
  return NMOE_OK;
}

nmoe_status nmoe_layer_set_wait_limit_ms(nmoe_layer* layer, double milliseconds) {
  if (layer == nullptr || !(milliseconds > 0.0) || milliseconds > 60000.0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  try {
    layer->wait_limit_ticks = ticks_from_ms(milliseconds);
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_layer_wait_flag(nmoe_layer* layer, void* stream_ptr, const uint32_t* flag,
                                 uint32_t expected) {
  if (layer == nullptr || flag == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  try {
    if (layer->probe_epoch.bytes() == 0) layer->probe_epoch.allocate(sizeof(uint32_t), true);
    NMOE_CUDA(cudaMemcpyAsync(layer->probe_epoch.as<uint32_t>(), &expected, sizeof(uint32_t),
                              cudaMemcpyHostToDevice, stream));
    NMOE_CUDA(launch_window_wait(flag, layer->probe_epoch.as<uint32_t>(), 0, 1,
                                 layer->wait_limit_ticks, layer->error.device.as<int32_t>(),
                                 stream));
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_layer_enable_stage_timing(nmoe_layer* layer, int32_t enable) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  if (enable != 0) {
    for (cudaEvent_t& e : layer->stage_events) {
      if (e == nullptr && cudaEventCreate(&e) != cudaSuccess) return NMOE_ERR_CUDA;
    }
  }
  layer->stage_timing = enable != 0;
  return NMOE_OK;
}

nmoe_status nmoe_layer_stage_times(nmoe_layer* layer, float* milliseconds, int32_t count) {
  if (layer == nullptr || milliseconds == nullptr || count < kStageCount || !layer->stage_timing) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  // A stage the last run did not pass through (the expert-parallel stages record only
  // some of the marks) reports 0.
  for (int i = 0; i <= kStageCount; ++i) {
    const cudaError_t state = cudaEventQuery(layer->stage_events[i]);
    if (state == cudaErrorNotReady) {
      if (cudaEventSynchronize(layer->stage_events[i]) != cudaSuccess) return NMOE_ERR_CUDA;
    } else if (state != cudaSuccess) {
      cudaGetLastError();
    }
  }
  for (int i = 0; i < kStageCount; ++i) {
    if (cudaEventElapsedTime(&milliseconds[i], layer->stage_events[i],
                             layer->stage_events[i + 1]) != cudaSuccess) {
      cudaGetLastError();
      milliseconds[i] = 0.0f;
    }
  }
  return NMOE_OK;
}

// ---------------------------------------------------------------------------
// expert-parallel stages
// ---------------------------------------------------------------------------

size_t nmoe_ep_record_bytes(const nmoe_layer* layer) {
  return layer == nullptr ? 0 : static_cast<size_t>(dispatch_record_bytes(layer->cfg.hidden_size));
}

nmoe_status nmoe_ep_dispatch(nmoe_layer* layer, void* stream_ptr, const void* input,
                             nmoe_dtype input_dtype, int64_t tokens, int64_t capacity_per_rank,
                             const void** send_records, const int32_t** send_counts) {
  if (layer == nullptr || input == nullptr || send_records == nullptr || send_counts == nullptr ||
      tokens <= 0 || layer->ep_world <= 1) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (tokens > layer->cfg.max_tokens) return NMOE_ERR_CAPACITY;
  if (capacity_per_rank < 0 ||
      capacity_per_rank * layer->ep_world > layer->send_record_slots) {
    return NMOE_ERR_CAPACITY;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  try {
    const nmoe_config& c = layer->cfg;
    route_tokens(layer, stream, input, input_dtype, static_cast<int>(tokens));
    NMOE_CUDA(launch_dispatch_plan(layer->counts.as<int32_t>(), c.n_routed_experts,
                                   layer->local_experts, layer->ep_world,
                                   layer->send_counts.as<int32_t>(),
                                   layer->send_offsets.as<int32_t>(),
                                   layer->rank_cursor.as<int32_t>(), stream));
    NMOE_CUDA(launch_pack_records(layer->top_index.as<int32_t>(), layer->top_weight.as<float>(),
                                  static_cast<int>(tokens), c.top_k, layer->local_experts,
                                  layer->y_packed.as<uint8_t>(),
                                  layer->y_sf_row_major.as<uint8_t>(), layer->y_ts.as<float>(),
                                  c.hidden_size, layer->send_offsets.as<int32_t>(),
                                  layer->rank_cursor.as<int32_t>(),
                                  static_cast<int>(capacity_per_rank),
                                  layer->send_records.as<uint8_t>(), nullptr,
                                  layer->send_position.as<int32_t>(),
                                  layer->error.device.as<int32_t>(), stream));
    layer->last_tokens = static_cast<int>(tokens);
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  *send_records = layer->send_records.as<uint8_t>();
  *send_counts = layer->send_counts.as<int32_t>();
  return NMOE_OK;
}

nmoe_status nmoe_ep_experts(nmoe_layer* layer, void* stream_ptr, const void* recv_records,
                            int64_t count, const int32_t* valid_counts, int64_t capacity_per_rank,
                            void* out_rows, nmoe_dtype rows_dtype) {
  if (layer == nullptr || layer->ep_world <= 1 || count < 0 ||
      (count > 0 && (recv_records == nullptr || out_rows == nullptr))) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (rows_dtype != NMOE_F32 && rows_dtype != NMOE_BF16 && rows_dtype != NMOE_F16) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (count > layer->max_pairs) return NMOE_ERR_CAPACITY;
  if (count == 0) return NMOE_OK;
  if (valid_counts != nullptr && capacity_per_rank <= 0) return NMOE_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  try {
    const int H = layer->cfg.hidden_size;
    NMOE_CUDA(cudaMemsetAsync(layer->counts.as<int32_t>(), 0,
                              layer->local_experts * sizeof(int32_t), stream));
    NMOE_CUDA(launch_record_histogram(static_cast<const uint8_t*>(recv_records),
                                      static_cast<int>(count), H, layer->local_experts,
                                      valid_counts, static_cast<int>(capacity_per_rank),
                                      layer->counts.as<int32_t>(),
                                      layer->error.device.as<int32_t>(), stream));
    const uint8_t* records = static_cast<const uint8_t*>(recv_records);
    const size_t stride = static_cast<size_t>(layer->record_bytes);
    const size_t tail = static_cast<size_t>(H) / 2 + static_cast<size_t>(H) / 16;
    PermuteSource source;
    source.packed = records;
    source.packed_stride = stride;
    source.sf = records + H / 2;
    source.sf_stride = stride;
    source.tensor_scale = reinterpret_cast<const float*>(records + tail);
    source.tensor_scale_stride = stride;
    source.weight = reinterpret_cast<const float*>(records + tail + 4);
    source.weight_stride = stride;
    source.expert = reinterpret_cast<const int32_t*>(records + tail + 8);
    source.expert_stride = stride;
    source.pairs_per_row = 1;
    source.valid_counts = valid_counts;
    source.capacity = static_cast<int>(capacity_per_rank);
    routed_experts(layer, stream, source, static_cast<int>(count), 1, out_rows,
                   static_cast<RowKind>(rows_dtype));
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ep_shared(nmoe_layer* layer, void* stream_ptr) {
  if (layer == nullptr || layer->ep_world <= 1 || layer->last_tokens <= 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  try {
    shared_expert(layer, static_cast<cudaStream_t>(stream_ptr), layer->last_tokens,
                  layer->shared_out.as<float>(), 1, 0, nullptr);
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ep_combine(nmoe_layer* layer, void* stream_ptr, const void* input,
                            nmoe_dtype input_dtype, const void* returned_rows,
                            nmoe_dtype rows_dtype, void* output, nmoe_dtype output_dtype) {
  if (layer == nullptr || layer->ep_world <= 1 || layer->last_tokens <= 0 || input == nullptr ||
      returned_rows == nullptr || output == nullptr) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  const cudaError_t err = launch_combine_indexed(
      input, input_dtype == NMOE_BF16, returned_rows, static_cast<RowKind>(rows_dtype),
      layer->send_position.as<int32_t>(), layer->shared_out.as<void>(), kRowF32, layer->last_tokens,
      layer->cfg.hidden_size, layer->cfg.top_k, output, output_dtype == NMOE_BF16,
      layer->error.device.as<int32_t>(), static_cast<cudaStream_t>(stream_ptr));
  return err == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}


// --- peer windows: the exchanges done by the stages' own kernels ------------

namespace {

// the part of nmoe_ep_experts after the records are known to be in place
void experts_over_records(nmoe_layer* layer, cudaStream_t stream, const uint8_t* records,
                          int count, const int32_t* valid_counts, int capacity, void* out_rows,
                          RowKind rows_kind, RowSegments segments) {
  const int H = layer->cfg.hidden_size;
  NMOE_CUDA(cudaMemsetAsync(layer->counts.as<int32_t>(), 0,
                            layer->local_experts * sizeof(int32_t), stream));
  NMOE_CUDA(launch_record_histogram(records, count, H, layer->local_experts, valid_counts,
                                    capacity, layer->counts.as<int32_t>(),
                                    layer->error.device.as<int32_t>(), stream));
  const size_t stride = static_cast<size_t>(layer->record_bytes);
  const size_t tail = static_cast<size_t>(H) / 2 + static_cast<size_t>(H) / 16;
  PermuteSource source;
  source.packed = records;
  source.packed_stride = stride;
  source.sf = records + H / 2;
  source.sf_stride = stride;
  source.tensor_scale = reinterpret_cast<const float*>(records + tail);
  source.tensor_scale_stride = stride;
  source.weight = reinterpret_cast<const float*>(records + tail + 4);
  source.weight_stride = stride;
  source.expert = reinterpret_cast<const int32_t*>(records + tail + 8);
  source.expert_stride = stride;
  source.pairs_per_row = 1;
  source.valid_counts = valid_counts;
  source.capacity = capacity;
  routed_experts(layer, stream, source, count, 1, out_rows, rows_kind, segments);
}

}  // namespace

nmoe_status nmoe_ep_window_create(nmoe_layer* layer, int64_t capacity_per_rank,
                                  nmoe_dtype rows_dtype, void* handle_out) {
  if (layer == nullptr || handle_out == nullptr || layer->ep_world <= 1 ||
      layer->ep_world > 64 || capacity_per_rank <= 0 ||
      (rows_dtype != NMOE_F32 && rows_dtype != NMOE_BF16 && rows_dtype != NMOE_F16)) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == NMOE_EP_WINDOW_HANDLE_BYTES, "handle size");
  const int64_t slots = capacity_per_rank * layer->ep_world;
  if (slots > layer->max_pairs) return NMOE_ERR_CAPACITY;
  try {
    auto& w = layer->window;
    w.close_peers();
    w.capacity = capacity_per_rank;
    w.rows_kind = static_cast<RowKind>(rows_dtype);
    const size_t H = static_cast<size_t>(layer->cfg.hidden_size);
    auto round_up = [](size_t v) { return (v + 255) / 256 * 256; };
    w.records_off = 0;
    w.rows_off = round_up(static_cast<size_t>(slots) * layer->record_bytes);
    w.flags_off = w.rows_off + round_up(static_cast<size_t>(slots) * H * row_kind_bytes(w.rows_kind));
    w.local.allocate(w.flags_off + 3 * 64 * sizeof(uint32_t), true);
    w.epoch.allocate(sizeof(uint32_t), true);
    NMOE_CUDA(cudaDeviceSynchronize());  // the zeroes are in place before any peer maps it
    cudaIpcMemHandle_t handle;
    NMOE_CUDA(cudaIpcGetMemHandle(&handle, w.local.as<void>()));
    std::memcpy(handle_out, &handle, sizeof(handle));
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ep_window_attach(nmoe_layer* layer, const void* handles) {
  if (layer == nullptr || handles == nullptr || layer->ep_world <= 1 ||
      layer->window.capacity <= 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  try {
    auto& w = layer->window;
    const int W = layer->ep_world, me = layer->ep_rank;
    w.close_peers();
    w.peer_base.assign(W, nullptr);
    std::vector<unsigned long long> record_segments(W), row_segments(W), record_flags(W),
        row_flags(W), counts(W);
    const size_t H = static_cast<size_t>(layer->cfg.hidden_size);
    const size_t row_bytes = H * row_kind_bytes(w.rows_kind);
    for (int r = 0; r < W; ++r) {
      uint8_t* base = w.local.as<uint8_t>();
      if (r != me) {
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, static_cast<const uint8_t*>(handles) + r * sizeof(handle),
                    sizeof(handle));
        void* mapped = nullptr;
        NMOE_CUDA(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess));
        w.peer_base[r] = mapped;
        base = static_cast<uint8_t*>(mapped);
      }
      // in rank r's window this rank owns segment `me` of every region
      const size_t segment = static_cast<size_t>(me) * w.capacity;
      record_segments[r] = reinterpret_cast<unsigned long long>(
          base + w.records_off + segment * layer->record_bytes);
      row_segments[r] =
          reinterpret_cast<unsigned long long>(base + w.rows_off + segment * row_bytes);
      uint32_t* flags = reinterpret_cast<uint32_t*>(base + w.flags_off);
      record_flags[r] = reinterpret_cast<unsigned long long>(flags + me);
      row_flags[r] = reinterpret_cast<unsigned long long>(flags + 64 + me);
      counts[r] = reinterpret_cast<unsigned long long>(flags + 128 + me);
    }
    auto upload = [&](DeviceBuffer& buffer, const std::vector<unsigned long long>& host) {
      buffer.allocate(host.size() * sizeof(unsigned long long));
      NMOE_CUDA(cudaMemcpy(buffer.as<void>(), host.data(),
                           host.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice));
    };
    upload(w.record_segments, record_segments);
    upload(w.row_segments, row_segments);
    upload(w.record_flag_slots, record_flags);
    upload(w.row_flag_slots, row_flags);
    upload(w.count_slots, counts);
    w.attached = true;
  } catch (const Failure& failure) {
    layer->window.close_peers();
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ep_window_detach(nmoe_layer* layer) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  cudaDeviceSynchronize();
  layer->window.close_peers();
  return NMOE_OK;
}

nmoe_status nmoe_ep_window_fork_shared(nmoe_layer* layer, int32_t enable) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  if (enable != 0 && layer->side_stream == nullptr) return NMOE_ERR_UNSUPPORTED;
  layer->window_fork_shared = enable != 0;
  return NMOE_OK;
}

nmoe_status nmoe_ep_window_dispatch(nmoe_layer* layer, void* stream_ptr, const void* input,
                                    nmoe_dtype input_dtype, int64_t tokens) {
  if (layer == nullptr || input == nullptr || tokens <= 0 || !layer->window.attached) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  if (tokens > layer->cfg.max_tokens) return NMOE_ERR_CAPACITY;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  try {
    const nmoe_config& c = layer->cfg;
    auto& w = layer->window;
    NMOE_CUDA(launch_window_epoch(w.epoch.as<uint32_t>(), stream));
    // The shared expert needs only the quantised rows: with `fork_shared` it starts on
    // the layer's own stream right after the quantiser and runs beside the router and
    // the packing; nmoe_ep_window_combine joins it.
    const bool fork = layer->side_stream != nullptr && layer->window_fork_shared;
    route_tokens(layer, stream, input, input_dtype, static_cast<int>(tokens),
                 fork ? layer->quant_done : nullptr);
    if (fork) {
      NMOE_CUDA(cudaStreamWaitEvent(layer->side_stream, layer->quant_done, 0));
      // the shared expert's rows take the type of the returned rows, so that the
      // combine adds what the single-device layer adds for the same output type
      shared_expert(layer, layer->side_stream, static_cast<int>(tokens),
                    layer->shared_out.as<void>(), 1, 0, nullptr, w.rows_kind);
      NMOE_CUDA(cudaEventRecord(layer->shared_done, layer->side_stream));
    }
    layer->window_shared_pending = fork;
    layer->window_shared_kind = fork ? w.rows_kind : kRowF32;
    NMOE_CUDA(launch_dispatch_plan(layer->counts.as<int32_t>(), c.n_routed_experts,
                                   layer->local_experts, layer->ep_world,
                                   layer->send_counts.as<int32_t>(),
                                   layer->send_offsets.as<int32_t>(),
                                   layer->rank_cursor.as<int32_t>(), stream));
    NMOE_CUDA(launch_pack_records(layer->top_index.as<int32_t>(), layer->top_weight.as<float>(),
                                  static_cast<int>(tokens), c.top_k, layer->local_experts,
                                  layer->y_packed.as<uint8_t>(),
                                  layer->y_sf_row_major.as<uint8_t>(), layer->y_ts.as<float>(),
                                  c.hidden_size, layer->send_offsets.as<int32_t>(),
                                  layer->rank_cursor.as<int32_t>(), static_cast<int>(w.capacity),
                                  nullptr, w.record_segments.as<unsigned long long>(),
                                  layer->send_position.as<int32_t>(),
                                  layer->error.device.as<int32_t>(), stream));
    // every destination learns its record count and that the records are there
    NMOE_CUDA(launch_window_signal(w.record_flag_slots.as<unsigned long long>(),
                                   w.count_slots.as<unsigned long long>(),
                                   layer->send_counts.as<int32_t>(), w.epoch.as<uint32_t>(), 0,
                                   layer->ep_world, stream));
    layer->last_tokens = static_cast<int>(tokens);
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ep_window_experts(nmoe_layer* layer, void* stream_ptr, int32_t first_source_rank,
                                   int32_t source_ranks) {
  if (layer == nullptr || !layer->window.attached || first_source_rank < 0 ||
      source_ranks <= 0 || first_source_rank + source_ranks > layer->ep_world) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  try {
    auto& w = layer->window;
    const int cap = static_cast<int>(w.capacity);
    NMOE_CUDA(launch_window_wait(w.record_flags(), w.epoch.as<uint32_t>(), first_source_rank,
                                 source_ranks, layer->wait_limit_ticks,
                                 layer->error.device.as<int32_t>(), stream));
    RowSegments segments;
    segments.bases = w.row_segments.as<unsigned long long>();
    segments.rows = cap;
    segments.slot0 = first_source_rank * cap;
    const uint8_t* records = w.local.as<uint8_t>() + w.records_off +
                             static_cast<size_t>(first_source_rank) * cap * layer->record_bytes;
    experts_over_records(layer, stream, records, source_ranks * cap,
                         w.counts() + first_source_rank, cap, nullptr, w.rows_kind, segments);
    NMOE_CUDA(launch_window_signal(w.row_flag_slots.as<unsigned long long>(), nullptr, nullptr,
                                   w.epoch.as<uint32_t>(), first_source_rank, source_ranks,
                                   stream));
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_ep_window_combine(nmoe_layer* layer, void* stream_ptr, const void* input,
                                   nmoe_dtype input_dtype, void* output,
                                   nmoe_dtype output_dtype) {
  if (layer == nullptr || !layer->window.attached || layer->last_tokens <= 0 ||
      input == nullptr || output == nullptr) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  auto& w = layer->window;
  cudaError_t err = launch_window_wait(w.row_flags(), w.epoch.as<uint32_t>(), 0, layer->ep_world,
                                       layer->wait_limit_ticks,
                                       layer->error.device.as<int32_t>(), stream);
  if (err == cudaSuccess && layer->window_shared_pending) {
    err = cudaStreamWaitEvent(stream, layer->shared_done, 0);
    layer->window_shared_pending = false;
  }
  if (err == cudaSuccess) {
    err = launch_combine_indexed(input, input_dtype == NMOE_BF16,
                                 w.local.as<uint8_t>() + w.rows_off, w.rows_kind,
                                 layer->send_position.as<int32_t>(), layer->shared_out.as<void>(),
                                 layer->window_shared_kind, layer->last_tokens, layer->cfg.hidden_size, layer->cfg.top_k,
                                 output, output_dtype == NMOE_BF16,
                                 layer->error.device.as<int32_t>(), stream);
  }
  return err == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}

const char* nmoe_layer_last_error(const nmoe_layer* layer) {
  return layer == nullptr ? "null layer" : layer->last_error.c_str();
}

nmoe_status nmoe_layer_trace_view(nmoe_layer* layer, nmoe_trace_view* out) {
  if (layer == nullptr || out == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  out->normalized_input = layer->last_normalized ? layer->normalized.as<float>() : nullptr;
  out->router_logits = layer->logits.as<float>();
  out->selected_index = layer->top_index.as<int32_t>();
  out->selected_weight = layer->top_weight.as<float>();
  const bool lat = layer->latent_mode;
  out->act_packed = lat ? layer->lat_packed.as<uint8_t>() : layer->y_packed.as<uint8_t>();
  out->act_scales = lat ? layer->lat_sf_row_major.as<uint8_t>() : layer->y_sf_row_major.as<uint8_t>();
  out->act_tensor_scale = lat ? layer->lat_ts.as<float>() : layer->y_ts.as<float>();
  out->parts = layer->last_parts_kind != kRowF32 ? nullptr : layer->parts.as<float>();
  out->latent_output = lat ? layer->latent_rows.as<float>() : nullptr;
  out->routed_latent_output = lat ? layer->routed_latent.as<float>() : nullptr;
  out->projected_routed_output = lat ? layer->projected.as<float>() : nullptr;
  out->shared_output = lat ? layer->shared_rows.as<float>() : nullptr;
  return NMOE_OK;
}

nmoe_status nmoe_layer_copy_trace_field(nmoe_layer* layer, void* stream, int32_t field, void* dst,
                                        size_t nbytes) {
  if (layer == nullptr || dst == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  nmoe_trace_view view;
  nmoe_layer_trace_view(layer, &view);
  const void* sources[12] = {view.normalized_input, view.router_logits, view.selected_index,
                             view.selected_weight,  view.act_packed,    view.act_scales,
                             view.act_tensor_scale, view.parts,         view.latent_output,
                             view.routed_latent_output, view.projected_routed_output,
                             view.shared_output};
  if (field < 0 || field >= 12 || sources[field] == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  return cudaMemcpyAsync(dst, sources[field], nbytes, cudaMemcpyDefault,
                         static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? NMOE_OK
             : NMOE_ERR_CUDA;
}

nmoe_status nmoe_layer_keep_trace(nmoe_layer* layer, int32_t enable) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  if (layer->keep_trace != (enable != 0)) layer->drop_recorded();
  layer->keep_trace = enable != 0;
  return NMOE_OK;
}

nmoe_status nmoe_layer_reserve_tokens(nmoe_layer* layer, int32_t max_tokens) {
  if (layer == nullptr || max_tokens <= 0) return NMOE_ERR_INVALID_ARGUMENT;
  if (max_tokens <= layer->cfg.max_tokens) return NMOE_OK;
  if (layer->window.attached) return NMOE_ERR_INVALID_ARGUMENT;  // peers hold the old window
  try {
    NMOE_CUDA(cudaDeviceSynchronize());
    allocate_scratch(layer, static_cast<size_t>(max_tokens));
    NMOE_CUDA(cudaDeviceSynchronize());
  } catch (const Failure& failure) {
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_layer_set_unfused_activation(nmoe_layer* layer, int32_t enable) {
  if (layer == nullptr) return NMOE_ERR_INVALID_ARGUMENT;
  const bool want = enable != 0;
  if (want == layer->unfused) return NMOE_OK;
  if (want && layer->ep_world > 1) return NMOE_ERR_UNSUPPORTED;
  try {
    NMOE_CUDA(cudaDeviceSynchronize());
    layer->unfused = want;
    if (want && layer->u_raw.bytes() == 0) {
      allocate_scratch(layer, static_cast<size_t>(layer->cfg.max_tokens));
      NMOE_CUDA(cudaDeviceSynchronize());
    }
  } catch (const Failure& failure) {
    layer->unfused = false;
    layer->last_error = failure.message;
    return failure.status;
  }
  return NMOE_OK;
}

nmoe_status nmoe_layer_export_unfused(nmoe_layer* layer, void* stream_ptr, float* routed_activated,
                                      float* routed_outputs, float* shared_activated) {
  if (layer == nullptr || layer->last_tokens <= 0 || !layer->last_unfused) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const nmoe_config& c = layer->cfg;
  const int tokens = layer->last_tokens, pairs = tokens * c.top_k;
  cudaError_t err = cudaSuccess;
  if (routed_activated != nullptr) {
    err = launch_gather_rows(layer->u_raw.as<float>(), layer->pair_row.as<int32_t>(), pairs,
                             c.routed_expert_intermediate_size, routed_activated, stream);
  }
  if (err == cudaSuccess && routed_outputs != nullptr) {
    if (tokens > layer->unweighted_tokens) return NMOE_ERR_CAPACITY;
    // kept in the layout of `parts`: [token][top_k (+1 unless latent)][row]
    const int stride = layer->latent_mode ? c.top_k : c.top_k + 1;
    const int cols = layer->latent;
    for (int t = 0; t < tokens && err == cudaSuccess; ++t) {
      err = cudaMemcpyAsync(routed_outputs + static_cast<size_t>(t) * c.top_k * cols,
                            layer->unweighted_rows.as<float>() +
                                static_cast<size_t>(t) * stride * cols,
                            static_cast<size_t>(c.top_k) * cols * sizeof(float),
                            cudaMemcpyDefault, stream);
    }
  }
  if (err == cudaSuccess && shared_activated != nullptr) {
    err = cudaMemcpyAsync(shared_activated, layer->shared_raw.as<float>(),
                          static_cast<size_t>(tokens) * c.shared_expert_intermediate_size *
                              sizeof(float),
                          cudaMemcpyDefault, stream);
  }
  return err == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}

nmoe_status nmoe_layer_export_hidden(nmoe_layer* layer, void* stream_ptr, uint8_t* routed_packed,
                                     uint8_t* routed_scales, uint8_t* shared_packed,
                                     uint8_t* shared_scales) {
  if (layer == nullptr || layer->last_tokens <= 0) return NMOE_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const nmoe_config& c = layer->cfg;
  const int pairs = layer->last_tokens * c.top_k;
  if (routed_packed != nullptr || routed_scales != nullptr) {
    export_rows_kernel<<<pairs, 128, 0, stream>>>(
        layer->h_packed.as<uint8_t>(), layer->h_sf.as<uint8_t>(), layer->pair_row.as<int32_t>(),
        pairs, c.routed_expert_intermediate_size,
        k_blocks_of(c.routed_expert_intermediate_size) * 4, routed_packed, routed_scales);
  }
  if (shared_packed != nullptr || shared_scales != nullptr) {
    export_rows_kernel<<<layer->last_tokens, 128, 0, stream>>>(
        layer->sh_packed.as<uint8_t>(), layer->sh_sf.as<uint8_t>(), nullptr, layer->last_tokens,
        c.shared_expert_intermediate_size, k_blocks_of(c.shared_expert_intermediate_size) * 4,
        shared_packed, shared_scales);
  }
  return cudaGetLastError() == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// unit operators
// ---------------------------------------------------------------------------

nmoe_status nmoe_quantize_nvfp4(void* stream_ptr, const void* input, nmoe_dtype dtype,
                                int64_t rows, int64_t cols, int32_t per_row, uint8_t* packed,
                                uint8_t* scales_row_major, uint8_t* scales_swizzled,
                                float* tensor_scale) {
  // argument checks of nvfp4_packing.cpp:95-97
  if (input == nullptr || packed == nullptr || scales_row_major == nullptr ||
      tensor_scale == nullptr || rows <= 0 || cols <= 0 || cols % 16 != 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  cudaError_t err;
  if (per_row != 0) {
    if (scales_swizzled != nullptr) {
      err = cudaMemsetAsync(scales_swizzled, 0, nmoe_swizzled_scale_bytes(rows, cols), stream);
      if (err != cudaSuccess) return NMOE_ERR_CUDA;
    }
    // the tiled layout of this entry point pads blocks to 4, not to a K block
    err = launch_norm_quant(input, dtype == NMOE_BF16, static_cast<int>(rows),
                            static_cast<int>(cols), nullptr, 0.0f, nullptr, packed,
                            scales_row_major, nullptr, 0, tensor_scale, stream);
    if (err == cudaSuccess && scales_swizzled != nullptr) {
      err = launch_swizzle_scales(scales_row_major, static_cast<int>(rows),
                                  static_cast<int>(cols), scales_swizzled, stream);
    }
  } else {
    if (dtype != NMOE_F32) return NMOE_ERR_INVALID_ARGUMENT;
    float* scratch = nullptr;
    if (cudaMallocAsync(reinterpret_cast<void**>(&scratch), sizeof(float), stream) != cudaSuccess) {
      return NMOE_ERR_CUDA;
    }
    err = launch_quant_matrix(static_cast<const float*>(input), static_cast<int>(rows),
                              static_cast<int>(cols), packed, scales_row_major, tensor_scale,
                              scratch, stream);
    cudaFreeAsync(scratch, stream);
    if (err == cudaSuccess && scales_swizzled != nullptr) {
      err = launch_swizzle_scales(scales_row_major, static_cast<int>(rows),
                                  static_cast<int>(cols), scales_swizzled, stream);
    }
  }
  return err == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}

nmoe_status nmoe_dequant_nvfp4(void* stream, const uint8_t* packed,
                               const uint8_t* scales_row_major, const float* tensor_scale,
                               int32_t per_row, int64_t rows, int64_t cols, float* output) {
  if (packed == nullptr || scales_row_major == nullptr || tensor_scale == nullptr ||
      output == nullptr || rows <= 0 || cols <= 0 || cols % 16 != 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  return launch_dequant(packed, scales_row_major, tensor_scale, per_row != 0,
                        static_cast<int>(rows), static_cast<int>(cols), output,
                        static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? NMOE_OK
             : NMOE_ERR_CUDA;
}

size_t nmoe_swizzled_scale_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0 || cols % 16 != 0) return 0;
  const size_t padded_rows = (static_cast<size_t>(rows) + 127) / 128 * 128;
  const size_t padded_blocks = (static_cast<size_t>(cols) / 16 + 3) / 4 * 4;
  return padded_rows * padded_blocks;
}

nmoe_status nmoe_swizzle_scales(void* stream, const uint8_t* scales_row_major, int64_t rows,
                                int64_t cols, uint8_t* scales_swizzled) {
  if (scales_row_major == nullptr || scales_swizzled == nullptr || rows <= 0 || cols <= 0 ||
      cols % 16 != 0) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  return launch_swizzle_scales(scales_row_major, static_cast<int>(rows), static_cast<int>(cols),
                               scales_swizzled, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? NMOE_OK
             : NMOE_ERR_CUDA;
}

nmoe_status nmoe_rmsnorm(void* stream_ptr, const void* input, nmoe_dtype dtype, int64_t rows,
                         int64_t hidden, const float* weight, float epsilon, float* output) {
  if (input == nullptr || weight == nullptr || output == nullptr || rows <= 0 || hidden <= 0 ||
      hidden % 16 != 0 || !(epsilon > 0.0f)) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const cudaError_t err = launch_norm_quant(input, dtype == NMOE_BF16, static_cast<int>(rows),
                                            static_cast<int>(hidden), weight, epsilon, output,
                                            nullptr, nullptr, nullptr, 0, nullptr, stream);
  return err == cudaSuccess ? NMOE_OK : NMOE_ERR_CUDA;
}

nmoe_status nmoe_router_logits(void* stream, const float* normalized, const float* gate,
                               int64_t rows, int32_t experts, int32_t hidden, float* logits) {
  if (normalized == nullptr || gate == nullptr || logits == nullptr) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  return launch_router_logits(normalized, gate, nullptr, static_cast<int>(rows), experts, hidden,
                              logits,
                              static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? NMOE_OK
             : NMOE_ERR_INVALID_ARGUMENT;
}

nmoe_status nmoe_router_topk(void* stream, const float* logits, const float* bias, int64_t rows,
                             int32_t experts, int32_t top_k, int32_t n_group, int32_t topk_group,
                             int32_t norm_topk_prob, float routed_scaling, int32_t* top_index,
                             float* top_weight) {
  if (logits == nullptr || bias == nullptr || top_index == nullptr || top_weight == nullptr) {
    return NMOE_ERR_INVALID_ARGUMENT;
  }
  return launch_router_topk(logits, bias, static_cast<int>(rows), experts, top_k, n_group,
                            topk_group, norm_topk_prob != 0, routed_scaling, top_index,
                            top_weight, nullptr,
                            static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? NMOE_OK
             : NMOE_ERR_INVALID_ARGUMENT;
}

}  // extern "C"
