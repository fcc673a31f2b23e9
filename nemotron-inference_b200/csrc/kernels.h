// Host-visible declarations of the kernel launchers.  Everything takes an
// explicit stream and returns cudaError_t from the launch.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace nmoe {

// A row tile is a 128-row aligned slot of the expert-sorted activation buffer
// holding `rows` (<= 128) valid rows that all belong to `expert`.
struct RowTile {
  int32_t row0;    // first row of the slot (multiple of 128)
  int32_t rows;    // valid rows in the slot
  int32_t expert;  // index into the stacked expert weights
  int32_t reserved;
};

// Element type of the per-(token, slot) rows the down projection produces and the
// combine kernels add up: FP32, or a 16-bit type that halves the layer's largest
// write and read.  The numbering is nmoe_dtype's.
enum RowKind : int { kRowF32 = 0, kRowBf16 = 1, kRowF16 = 2 };
inline size_t row_kind_bytes(RowKind kind) { return kind == kRowF32 ? 4 : 2; }

enum GemmMode : int {
  kGemmUp = 0,    // D -> *scales -> relu^2 -> NVFP4 (packed + tiled scales)
  kGemmDown = 1,  // D -> *scales [* routing weight] -> FP32 rows scattered by dest_row
};

struct GemmArgs {
  int32_t K = 0;         // contraction length, multiple of 64
  int32_t N = 0;         // output features per expert
  int32_t n_tiles = 0;   // ceil(N / BN)
  int32_t k_blocks = 0;  // ceil(K / 256)
  int32_t kb_full = 0;   // K / 256: K blocks stored in the full-block weight region
  const uint8_t* b_full = nullptr;  // [expert][kb_full][N][128 B], 16-byte chunks pre-swizzled
  // A-side block scales, tiled: [row slot][k_blocks][2048 bytes]
  const uint8_t* sfa = nullptr;
  // weight block scales, [expert][n_tile][k_block][sfb_bytes] in the layout
  // produced by relayout_weight_scales()
  const uint8_t* sfb = nullptr;
  const float* a_tensor_scale = nullptr;  // per activation row, nullptr => 1.0
  const float* w_tensor_scale = nullptr;  // [expert]
  // schedule: grouped (row_tiles + device count) or dense (row_tiles == nullptr)
  const RowTile* row_tiles = nullptr;
  const int32_t* num_row_tiles = nullptr;
  int32_t dense_rows = 0;
  // kGemmUp outputs
  uint8_t* out_packed = nullptr;  // [row][N/2]
  uint8_t* out_sf = nullptr;      // tiled [row slot][out_k_blocks][2048]
  int32_t out_k_blocks = 0;       // ceil(N / 256)
  // kGemmDown outputs
  void* out_rows = nullptr;           // [dest][N] of out_kind elements
  int32_t out_kind = kRowF32;         // RowKind
  const int32_t* dest_row = nullptr;  // per activation row; nullptr => row*dest_mul+dest_add
  int32_t dest_mul = 1;
  int32_t dest_add = 0;
  const float* row_weight = nullptr;  // per activation row routing weight, nullptr => none
  int32_t relu2 = 0;                  // kGemmDown: store relu^2 of the scaled value (the
                                      // unfused up projection keeps its rows in FP32)
  // Expert-parallel return straight into the source ranks' memory: destination
  // index d means row (d + segment_slot0) % segment_rows of the buffer that
  // out_segments[(d + segment_slot0) / segment_rows] points to (a peer's GPU).
  const unsigned long long* out_segments = nullptr;
  int32_t segment_rows = 0;
  int32_t segment_slot0 = 0;
  int32_t* error = nullptr;           // device error slot (DeviceError)
  // Timing experiments on the CTA-pair kernel only (results are WRONG when set):
  // bit 0 the epilogue drains nothing, bit 1 no scale writes, bit 2 no operand loads,
  // bit 3 no MMAs.  Every barrier handshake stays in place.
  int32_t ablate = 0;
};

// Tile shapes compiled into the library.  The block scales of every MMA must
// start on a 4-column TMEM boundary, so a weight tile stores its scales in
// whole groups of 128 rows; BN = 128 makes that exact for the HBM-bound sizes.
enum GemmVariant : int {
  kVariantPrefillUp = 0,    // BN 208, 128-row A box
  kVariantPrefillDown = 1,  // BN 192, 128-row A box
  kVariantDecode = 2,       // BN 128, 32-row A box, deep pipeline
  kVariantDecodeWide = 3,   // BN 128, 128-row A box
  kVariantPairUp = 4,       // 256 x 176 over a CTA pair (cta_group::2), quantising epilogue
  kVariantPairDown = 5,     // the same tile, row-storing epilogue
  kVariantCount = 6,
};

struct GemmVariantInfo {
  int bn;            // output features per tile
  int a_rows;        // rows of the activation box / valid rows per row tile
  int sfb_groups;    // 32-row groups of weight scales stored per K-tile
  int sfb_bytes;     // bytes of weight scales per (n_tile, k_block)
  int smem_bytes;    // dynamic shared memory of the kernel
  int b_rows;        // weight rows one CTA stages per K block (half a tile in a pair)
};

// Tensor maps of one GEMM launch.  `a` (activation rows, 128-byte swizzle) and `b_tail`
// (the partial last K block of the weights) are used by every variant; the CTA-pair
// variants also load the full weight K blocks through a map (`b_full`: the K-block-major
// panels as [rows][128 B], no swizzle), so that both CTAs' copies can complete on the
// leader's barrier.
struct GemmMaps {
  CUtensorMap a;
  CUtensorMap b_tail;
  CUtensorMap b_full;
};

GemmVariantInfo gemm_variant_info(GemmVariant v);
cudaError_t launch_grouped_gemm(GemmVariant v, GemmMode mode, const GemmMaps& maps,
                                const GemmArgs& args, int num_sms, cudaStream_t stream);

// Packed weights [experts][N][K/2] -> K-block-major (device to device): every
// (expert, 128-byte K block) becomes a contiguous [N][128 B] panel in `full`, so a
// weight tile of any height is ONE contiguous read; the partial last K block
// goes to `tail` as [experts * N][tail_pitch_bytes].
cudaError_t relayout_weight_packed(const uint8_t* row_major, int experts, int N, int K,
                                   int tail_pitch_bytes, uint8_t* full, uint8_t* tail,
                                   cudaStream_t stream);

// Re-tile row-major E4M3 weight block scales [experts][N][K/16] into the layout
// the GEMM variant consumes (device to device).
cudaError_t relayout_weight_scales(const uint8_t* row_major, int experts, int N, int K, int bn,
                                   int sfb_groups, uint8_t* out, cudaStream_t stream);
size_t weight_scale_layout_bytes(int experts, int N, int K, int bn, int sfb_groups);

// --- quantiser / norm ------------------------------------------------------
// RMSNorm (optional) + per-row dynamic NVFP4 quantisation.
//   in: [rows][cols] fp32 or bf16; norm_weight nullptr => no normalisation
//   normalized (optional) fp32 [rows][cols]
//   packed [rows][cols/2]; sf_row_major (optional) [rows][cols/16];
//   sf_tiled (optional) tiled layout with k_blocks*4 K-tiles per 128-row slot;
//   tensor_scale (optional) [rows]; inv_rms (optional) [rows]: 1/sqrt(mean(x^2)+eps)
cudaError_t launch_norm_quant(const void* in, bool in_bf16, int rows, int cols,
                              const float* norm_weight, float eps, float* normalized,
                              uint8_t* packed, uint8_t* sf_row_major, uint8_t* sf_tiled,
                              int k_blocks, float* tensor_scale, cudaStream_t stream,
                              float* inv_rms = nullptr);
// Whole-matrix dynamic quantisation with ONE tensor scale (the reference
// packer's semantics for rows > 1).  `amax_scratch` is one float of device
// memory; it is overwritten.
cudaError_t launch_quant_matrix(const float* in, int rows, int cols, uint8_t* packed,
                                uint8_t* sf_row_major, float* tensor_scale,
                                float* amax_scratch, cudaStream_t stream);
cudaError_t launch_dequant(const uint8_t* packed, const uint8_t* sf_row_major,
                           const float* tensor_scale, bool per_row_scale, int rows, int cols,
                           float* out, cudaStream_t stream);
cudaError_t launch_swizzle_scales(const uint8_t* row_major, int rows, int cols, uint8_t* tiled,
                                  cudaStream_t stream);

// --- router ------------------------------------------------------------------
cudaError_t launch_router_logits(const float* normalized, const float* gate,
                                 const float* logit_offset /* nullable [experts] */, int rows,
                                 int experts, int hidden, float* logits, cudaStream_t stream);
// The argument rules of launch_router_topk, for callers that must know before they
// enqueue anything.
bool router_topk_arguments_valid(int rows, int experts, int top_k, int n_group, int topk_group);
cudaError_t launch_router_topk(const float* logits, const float* bias, int rows, int experts,
                               int top_k, int n_group, int topk_group, bool norm_topk_prob,
                               float routed_scaling, int32_t* top_index, float* top_weight,
                               int32_t* expert_counts /* nullable, += histogram */,
                               cudaStream_t stream);

// Two-pass router for large batches.  Pass 1: logits on the tensor cores (FP32
// accumulate) from the bf16 gate and the normalised activations, which the kernel
// rebuilds from the layer input `x` as (x * inv_rms) * norm_weight and splits into
// three bf16 terms on the fly.  Pass 2, per token: every expert whose pass-1 choice
// score is within `tie_margin` of the top_k-th is re-evaluated in FP64 (and written
// back into `logits`), then top-k runs on the exact values.  Requires n_group == 1,
// experts % 32 == 0, experts <= 256, hidden % 64 == 0.
cudaError_t launch_router_fast_logits(const void* x, bool x_bf16, const float* inv_rms,
                                      const float* norm_weight, const CUtensorMap& tmap_gate,
                                      int rows, int experts, int hidden, float* logits,
                                      int32_t* error, cudaStream_t stream);
// Pass 1 for bf16 layer inputs: the RMSNorm weight folded into the gate (three bf16 terms of
// fl32(w[i] * gate[e][i]), `planes` = [3][experts][hidden], built once by launch_fold_gate),
// the input rows read by TMA through `tmap_x` ([rows][hidden] bf16, box 64 x 128, 128-byte
// swizzle; `tmap_planes` = [3 * experts][hidden], box 64 x experts), inv_rms applied to the sums.
cudaError_t launch_fold_gate(const __nv_bfloat16* gate, const float* norm_weight, int experts,
                             int hidden, __nv_bfloat16* planes, cudaStream_t stream);
// `splits` CTAs share the contraction of one 128-row tile; split s writes its partial sums to
// logits + s * rows * experts, and launch_router_select_exact adds them up.
// router_folded_splits picks the split count (1, 2 or 4) for a batch.
int router_folded_splits(int rows, int hidden, int num_sms);
cudaError_t launch_router_folded_logits(const CUtensorMap& tmap_x, const CUtensorMap& tmap_planes,
                                        const float* inv_rms, int rows, int experts, int hidden,
                                        int splits, float* logits, int32_t* error,
                                        cudaStream_t stream);
cudaError_t launch_router_select_exact(float* logits, int splits, const void* x, bool x_bf16,
                                       const float* inv_rms, const float* norm_weight,
                                       const __nv_bfloat16* gate, const float* logit_offset,
                                       const float* bias, int rows, int experts, int hidden,
                                       int top_k, bool norm_topk_prob, float routed_scaling,
                                       float tie_margin, int32_t* top_index, float* top_weight,
                                       int32_t* expert_counts, cudaStream_t stream);

// --- dense and scaled-FP8 linear families, latent-MoE data flow (csrc/dense.cu) -
// The dense matmul itself is launch_router_logits: out[rows][experts] =
// a[rows][hidden] x w[experts][hidden]^T, FP64 accumulation, FP32 result.
// Activation round trip through E4M3 with a per-tensor input scale.
cudaError_t launch_fp8_round_trip(const float* in, size_t count, float input_scale, float* out,
                                  cudaStream_t stream);
// E4M3 weight bytes -> FP32 values times the per-tensor weight scale.
cudaError_t launch_fp8_weight_dequant(const uint8_t* bytes, size_t count, float weight_scale,
                                      float* out, cudaStream_t stream);
cudaError_t launch_relu2(float* values, size_t count, cudaStream_t stream);
// out[t] = sum_k parts[t][k] in slot order; parts FP32 [rows][top_k][cols].
cudaError_t launch_sum_parts(const float* parts, int rows, int cols, int top_k, float* out,
                             cudaStream_t stream);
// out = in + (projected + shared), all [rows][hidden].
cudaError_t launch_mixer(const void* in, bool in_bf16, const float* projected, const float* shared,
                         int rows, int hidden, void* out, bool out_bf16, cudaStream_t stream);
// out[i] = rows[row_of[i]] (row_of == nullptr: identity), FP32 rows of `cols`.
cudaError_t launch_gather_rows(const float* rows, const int32_t* row_of, int count, int cols,
                               float* out, cudaStream_t stream);

// --- plan / permute / combine -------------------------------------------------
struct PlanBuffers {
  int32_t* expert_counts;   // [experts]  (input, filled by the router)
  int32_t* expert_cursor;   // [experts]  (scratch, zeroed by the plan kernel)
  int32_t* expert_slot0;    // [experts]  first row slot of each expert
  RowTile* row_tiles;       // [max_row_tiles]
  int32_t* num_row_tiles;   // [1]
};
// `tile_multiple`: every expert gets a multiple of this many row tiles (2 when CTA
// pairs consume them: the second tile of an odd expert is left empty).
cudaError_t launch_route_plan(const PlanBuffers& plan, int experts, int tile_rows,
                              int tile_multiple, int max_row_tiles, int32_t* error,
                              cudaStream_t stream);
// Where permute reads a (row, slot) pair from.  Quantised rows are indexed by
// source row = pair / pairs_per_row, routing weight and expert id by pair; all
// strides are in bytes.  Local routing: pairs_per_row = top_k over the token
// arrays.  Expert-parallel receive: pairs_per_row = 1 over dispatch records.
struct PermuteSource {
  const uint8_t* packed;
  size_t packed_stride;
  const uint8_t* sf;  // row-major E4M3 block scales
  size_t sf_stride;
  const float* tensor_scale;
  size_t tensor_scale_stride;
  const float* weight;
  size_t weight_stride;
  const int32_t* expert;  // index into the LOCAL expert stack
  size_t expert_stride;
  int pairs_per_row;
  // fixed-capacity receive buffers: pair i is valid iff (i % capacity) <
  // valid_counts[i / capacity]; nullptr = every pair is valid
  const int32_t* valid_counts = nullptr;
  int capacity = 0;
};
// Copies each pair's quantised activation row into its expert's row slots and
// records where it went; sorted_dest[row] = source_row * dest_stride + slot.
cudaError_t launch_permute(const PlanBuffers& plan, const PermuteSource& src, int pairs,
                           int experts /* size of the local expert stack */, int tile_rows,
                           int max_row_tiles, int cols, int k_blocks,
                           uint8_t* sorted_packed, uint8_t* sorted_sf_tiled,
                           float* sorted_tensor_scale, float* sorted_weight,
                           int32_t* sorted_dest, int32_t* pair_row /* nullable */,
                           int dest_stride, cudaStream_t stream);
// --- expert-parallel dispatch / return (csrc/ep.cu) ---------------------------
int dispatch_record_bytes(int cols);
cudaError_t launch_dispatch_plan(const int32_t* expert_counts, int experts, int experts_per_rank,
                                 int world, int32_t* send_counts, int32_t* send_offsets,
                                 int32_t* rank_cursor, cudaStream_t stream);
cudaError_t launch_pack_records(const int32_t* top_index, const float* top_weight, int rows,
                                int top_k, int experts_per_rank, const uint8_t* packed,
                                const uint8_t* sf_row_major, const float* tensor_scale, int cols,
                                const int32_t* send_offsets, int32_t* rank_cursor,
                                int capacity /* per destination rank, 0 = compact */,
                                uint8_t* records,
                                const unsigned long long* windows /* nullable: per destination
                                rank, where this rank's segment starts in that rank's memory */,
                                int32_t* send_position, int32_t* error, cudaStream_t stream);
// Peer windows: a step counter on the device, flags raised in other ranks'
// memory (one thread per rank first..first+count-1), and a bounded wait.
cudaError_t launch_window_epoch(uint32_t* epoch, cudaStream_t stream);
cudaError_t launch_window_signal(const unsigned long long* flag_slots,
                                 const unsigned long long* word_slots, const int32_t* words,
                                 const uint32_t* epoch, int first, int count, cudaStream_t stream);
// `limit_ticks`: clock64 ticks after which a waiting thread gives up and records
// kDevWaitTimeout in `error`.
cudaError_t launch_window_wait(const uint32_t* flags, const uint32_t* epoch, int first, int count,
                               long long limit_ticks, int32_t* error, cudaStream_t stream);
cudaError_t launch_record_histogram(const uint8_t* records, int count, int cols,
                                    int local_experts, const int32_t* valid_counts, int capacity,
                                    int32_t* expert_counts, int32_t* error, cudaStream_t stream);
cudaError_t launch_combine_indexed(const void* in, bool in_bf16, const void* returned_rows,
                                   RowKind rows_kind, const int32_t* position,
                                   const void* shared_rows, RowKind shared_kind, int rows,
                                   int hidden, int top_k, void* out, bool out_bf16,
                                   int32_t* error, cudaStream_t stream);

// out[t] = in[t] + ((sum_k parts[t][k]) + parts[t][top_k]) with the routed
// parts (rows of `parts_kind`, [rows][top_k + 1][hidden]) added in slot order.
// `error` (nullable): kDevActivationRange when a binary16 part arrived as an infinity.
cudaError_t launch_combine(const void* in, bool in_bf16, const void* parts, RowKind parts_kind,
                           int rows, int hidden, int top_k, void* out, bool out_bf16,
                           int32_t* error, cudaStream_t stream);

}  // namespace nmoe
