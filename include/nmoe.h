/*
 * nmoe.h -- C ABI of the B200 NVFP4 mixture-of-experts expert layer.
 *
 * Drop-in replacement for the expert-layer operator of kwindla/nemotron-inference
 * (nemotron::ExpertLayerSlice, runtime/include/nemotron/expert_layer.h:84-105):
 * RMSNorm, sigmoid top-k router with correction bias, token permute, routed
 * expert grouped GEMMs (up_proj -> relu^2 -> down_proj, dynamic per-16-block
 * NVFP4 activation quantisation), shared expert, weighted combine, residual.
 *
 * Plain pointers and sizes only.  Weight pointers may be host or device
 * addresses (unified addressing); they are copied at creation and need not
 * outlive it.  Activation pointers are device addresses.  Every call takes the
 * CUDA stream to run on (passed as void*, a cudaStream_t); nothing here
 * synchronises unless it says so.  All functions return an nmoe_status
 * (0 = success); nmoe_status_string() and nmoe_layer_last_error() describe a
 * failure.  The library has no CPU fallback: without a CUDA device every
 * compute entry point fails with NMOE_ERR_CUDA.
 *
 * Citations are file:line inside the reference project.
 */
#ifndef NMOE_H_
#define NMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NMOE_API __attribute__((visibility("default")))

typedef enum nmoe_status {
  NMOE_OK = 0,
  NMOE_ERR_INVALID_ARGUMENT = 1,
  NMOE_ERR_CUDA = 2,            /* a CUDA runtime / driver call failed */
  NMOE_ERR_UNSUPPORTED = 3,     /* valid in the reference, not built here */
  NMOE_ERR_DEVICE_TIMEOUT = 4,  /* a bounded device-side wait gave up */
  NMOE_ERR_ACTIVATION_RANGE = 5,/* an activated row exceeded 6*448 (tensor scale != 1) */
  NMOE_ERR_CAPACITY = 6         /* more tokens / row tiles than the layer was created for */
} nmoe_status;

/* NMOE_F16 (binary16) is accepted only for the rows expert-parallel ranks return
 * (rows_dtype of the nmoe_ep_* entry points); activations are FP32 or bf16. */
typedef enum nmoe_dtype { NMOE_F32 = 0, NMOE_BF16 = 1, NMOE_F16 = 2 } nmoe_dtype;

/* Mirrors nemotron::ExpertLayerConfig (expert_layer.h:18-31).  The routed
 * experts act on rows of moe_latent_size elements: the output of fc1_latent
 * (expert_layer.cpp:809-813), projected back by fc2_latent (:1047-1053).  With
 * moe_latent_size == hidden_size both projections may be absent (identity). */
typedef struct nmoe_config {
  int32_t layer_index;
  int32_t hidden_size;
  int32_t moe_latent_size;
  int32_t routed_expert_intermediate_size;
  int32_t shared_expert_intermediate_size;
  int32_t n_routed_experts;
  int32_t top_k;
  int32_t n_group;
  int32_t topk_group;
  int32_t norm_topk_prob;
  float rms_epsilon;
  float routed_scaling_factor;
  int32_t max_tokens; /* capacity of one nmoe_layer_run call (not in the reference,
                         which allocates scratch per call, expert_layer.cpp:782-787) */
  int32_t max_recv_pairs; /* expert parallelism only: most (token, slot) pairs this rank
                             accepts from all ranks in one step; 0 = 2*max_tokens*top_k */
} nmoe_config;

/* One NVFP4 matrix in the reference's weight layout: the byte fields of
 * nemotron::GemmDescriptor (gemm_catalog.h:20-42) for kernel family
 * kCublasLtNvfp4BlockScaled / layout "cublaslt_fp4_tn_v1"
 * (nvfp4_weight.cpp:59-70).  packed: [output_rows][input_cols/2], column 2j in
 * the low nibble; block_scales: [output_rows][input_cols/16] E4M3, row-major;
 * tensor_scale: 4-byte FP32. */
typedef struct nmoe_nvfp4_matrix {
  size_t output_rows;
  size_t input_cols;
  const uint8_t* packed_data;
  size_t packed_nbytes;
  const uint8_t* block_scales_data;
  size_t block_scales_nbytes;
  const uint8_t* tensor_scale_data;
  size_t tensor_scale_nbytes;
} nmoe_nvfp4_matrix;

/* A dense row-major tensor (KernelTensorDescriptor / dense GemmDescriptor,
 * kernel_catalog.h:14-34): norm weight [hidden], gate weight [experts][hidden],
 * e_score_correction_bias [experts]; FP32 or bf16. */
typedef struct nmoe_dense_tensor {
  const void* data;
  size_t nbytes;
  nmoe_dtype dtype;
  size_t rows;
  size_t cols;
} nmoe_dense_tensor;

/* A linear of the dense or the scaled-FP8 family, the two families the
 * reference accepts for fc1_latent, shared_up and (when it is not NVFP4)
 * shared_down (expert_layer.cpp:534-617), and the dense family of fc2_latent.
 *   DENSE       weight FP32 or bf16 [out][in]; y = x W^T with DOUBLE accumulation
 *               (UploadedLinearOp, linear_op.cpp:97-118, :238-271).
 *   SCALED_FP8  weight E4M3 bytes [out][in] (weight.dtype is ignored, nbytes =
 *               out * in), dequantised as DecodeFp8(byte) * weight_scale; the
 *               activations take a round trip through E4M3 at input_scale first
 *               (ScaledFp8LinearOp, scaled_fp8_linear.cu:121-139, :222-283). */
typedef enum nmoe_linear_family {
  NMOE_LINEAR_ABSENT = 0,
  NMOE_LINEAR_DENSE = 1,
  NMOE_LINEAR_SCALED_FP8 = 2
} nmoe_linear_family;

typedef struct nmoe_linear {
  nmoe_linear_family family;
  nmoe_dense_tensor weight;
  float weight_scale; /* SCALED_FP8 only */
  float input_scale;  /* SCALED_FP8 only */
} nmoe_linear;

/* Mirrors nemotron::ExpertLayerBindings (expert_layer.h:38-56).
 * routed_up/routed_down hold n_local_experts entries: the experts
 * [first_local_expert, first_local_expert + n_local_experts) of the layer,
 * up_proj [intermediate][latent], down_proj [latent][intermediate]. */
typedef struct nmoe_weights {
  nmoe_dense_tensor input_norm_weight;
  nmoe_dense_tensor gate_weight;
  nmoe_dense_tensor gate_score_correction_bias;
  const nmoe_nvfp4_matrix* routed_up;   /* each [intermediate][hidden] */
  const nmoe_nvfp4_matrix* routed_down; /* each [hidden][intermediate] */
  int32_t n_local_experts;
  int32_t first_local_expert;
  nmoe_nvfp4_matrix shared_up;   /* [shared_intermediate][hidden] */
  nmoe_nvfp4_matrix shared_down; /* [hidden][shared_intermediate] */
  /* Optional FP32 [experts] added to the gate logits (NULL = none).  Not in the
   * reference: a hook for synthetic workloads with skewed expert load. */
  const float* gate_logit_offset;
  /* Latent projections (fc1_latent_*, fc2_latent_weight of the reference's
   * bindings): fc1 [latent][hidden], fc2 [hidden][latent] (dense only).  Both
   * ABSENT means identity and requires moe_latent_size == hidden_size. */
  nmoe_linear fc1_latent;
  nmoe_linear fc2_latent;
  /* Shared expert in the dense / scaled-FP8 families the real checkpoint uses
   * (shared_up_kernel_weight + scales, or a dense shared_up_gemm_weight): when
   * not ABSENT they replace the NVFP4 shared_up / shared_down above, whose
   * pointers may then be NULL. */
  nmoe_linear shared_up_linear;   /* [shared_intermediate][hidden] */
  nmoe_linear shared_down_linear; /* [hidden][shared_intermediate] */
} nmoe_weights;

typedef struct nmoe_layer nmoe_layer;

NMOE_API const char* nmoe_status_string(nmoe_status status);

/* ExpertLayerSlice::Create (expert_layer.cpp:494-709): validates config and
 * shapes (:505-528, :646-689), uploads every weight to HBM (the reference keeps
 * host pointers to the routed experts, :707) and allocates all scratch for
 * max_tokens.  Synchronises the device once. */
NMOE_API nmoe_status nmoe_layer_create(const nmoe_config* config, const nmoe_weights* weights,
                                       nmoe_layer** out_layer);
NMOE_API void nmoe_layer_destroy(nmoe_layer* layer);

/* ExpertLayerSlice::Run (expert_layer.cpp:752-1092) for `tokens` rows:
 * output = input + routed + shared with the input RMSNorm inside.  input and
 * output are device [tokens][hidden] in the given dtypes and must not alias.
 * With FP32 output the per-slot rows are summed from FP32, in the reference's
 * order (:951-953, :1064-1069); with bf16 output they are rounded to binary16
 * first (a row beyond 65504 is reported as NMOE_ERR_ACTIVATION_RANGE).
 * Enqueues on `stream` and returns; device-side failures surface through
 * nmoe_layer_sync_status().  Batches of up to 256 tokens (NMOE_GRAPH_MAX_TOKENS)
 * on a capturable stream are recorded once per (token count, buffers, types) as a
 * CUDA graph and replayed by later calls with the same arguments; the legacy
 * default stream, and a stream the caller is capturing itself, run eagerly. */
NMOE_API nmoe_status nmoe_layer_run(nmoe_layer* layer, void* stream, const void* input,
                                    nmoe_dtype input_dtype, int64_t tokens, void* output,
                                    nmoe_dtype output_dtype);

/* Grows the layer's scratch to `max_tokens` rows per call (no effect when it is
 * already that large).  Frees and reallocates device memory and synchronises the
 * device: call it between runs.  The reference allocates its scratch per call
 * (expert_layer.cpp:782-787) and therefore accepts any token count; a caller
 * that wants that behaviour calls this when nmoe_layer_run answers
 * NMOE_ERR_CAPACITY. */
NMOE_API nmoe_status nmoe_layer_reserve_tokens(nmoe_layer* layer, int32_t max_tokens);

/* The unfused activation path.  By default the up projection's epilogue applies
 * relu^2 and quantises the row to NVFP4 on the fly, which is the reference's
 * arithmetic only while the row's tensor scale is 1, i.e. while no activated
 * value exceeds 6*448 (nvfp4_packing.cpp:119-126); a run that meets a larger
 * value reports NMOE_ERR_ACTIVATION_RANGE.  With enable != 0 the layer keeps
 * the activated rows in FP32 and quantises them in a pass of its own with the
 * per-row tensor scale, as RunNvfp4LinearHost does (expert_layer.cpp:913-922):
 * any range is handled, at about twice the cost of the expert GEMMs.  It also
 * retains what ExpertLayerRunTrace needs beyond the fused path's buffers: the
 * FP32 activated rows and the unweighted down_proj rows
 * (nmoe_layer_export_unfused).  Allocates on the first enable and synchronises
 * the device: call it between runs. */
NMOE_API nmoe_status nmoe_layer_set_unfused_activation(nmoe_layer* layer, int32_t enable);
/* After a run with the unfused path, in (token, slot) order, DEVICE pointers, any of
 * which may be NULL: routed_activated [tokens][top_k][intermediate] FP32 = relu^2(up_proj),
 * routed_outputs [tokens][top_k][latent] FP32 = down_proj rows before the
 * routing weight, shared_activated [tokens][shared_intermediate] FP32
 * (routed_expert_activated_hidden / routed_expert_outputs of
 * expert_layer.h:63-76). */
NMOE_API nmoe_status nmoe_layer_export_unfused(nmoe_layer* layer, void* stream,
                                               float* routed_activated, float* routed_outputs,
                                               float* shared_activated);

/* Waits for `stream` and reports what the kernels left in the layer's device
 * error slot (and clears it): the boolean the reference's synchronous Run
 * returns. */
NMOE_API nmoe_status nmoe_layer_sync_status(nmoe_layer* layer, void* stream);
NMOE_API const char* nmoe_layer_last_error(const nmoe_layer* layer);

/* Failure detection.  No reference counterpart (one process, one GPU; every
 * failure there is `return false`).  Kernels of this library that wait for
 * another GPU -- the flag waits of the peer-window stages below -- give up after
 * a limit, leave NMOE_ERR_DEVICE_TIMEOUT in the layer's error slot and return,
 * so a peer that died or skipped a step costs an error status, never a hung
 * GPU.  nmoe_layer_set_wait_limit_ms sets that limit (default about eight
 * seconds; the environment variable NMOE_WAIT_LIMIT_MS sets it at creation).
 * nmoe_layer_wait_flag enqueues the same bounded wait on a caller-owned device
 * word: it returns when *flag >= expected (as a wrapping 32-bit step counter) or
 * when the limit runs out; health checks and tests use it to see the timeout
 * path without a second GPU. */
NMOE_API nmoe_status nmoe_layer_set_wait_limit_ms(nmoe_layer* layer, double milliseconds);
NMOE_API nmoe_status nmoe_layer_wait_flag(nmoe_layer* layer, void* stream, const uint32_t* flag,
                                          uint32_t expected);

/* Per-stage device timing (the reference has no profiler hooks; its benchmarks
 * time with steady_clock around synchronous calls,
 * benchmarks/gb10_nvfp4_gemm/gb10_nvfp4_gemm_bench.cpp:655-676).  When enabled,
 * nmoe_layer_run records a CUDA event before every stage; after the run,
 * nmoe_layer_stage_times waits for the last one and returns the elapsed
 * milliseconds of the NMOE_STAGE_COUNT stages, in this order: norm+quantise,
 * router logits, top-k, route plan, permute, routed up GEMM, routed down GEMM,
 * shared up GEMM, shared down GEMM, combine. */
#define NMOE_STAGE_COUNT 10
NMOE_API nmoe_status nmoe_layer_enable_stage_timing(nmoe_layer* layer, int32_t enable);
NMOE_API nmoe_status nmoe_layer_stage_times(nmoe_layer* layer, float* milliseconds,
                                            int32_t count);

/* Expert parallelism runs collectives on a second stream while the grouped
 * GEMMs execute.  The GEMMs are persistent kernels with one CTA per SM and
 * nearly all of its shared memory, so a communication kernel launched beside
 * them would not start before they finish.  This call makes the layer launch
 * its GEMMs on (SM count - reserved_sms) SMs; 0 restores the default.  No
 * reference counterpart (the reference runs one GPU per process without
 * overlap). */
NMOE_API nmoe_status nmoe_layer_reserve_sms(nmoe_layer* layer, int32_t reserved_sms);

/* The intermediates ExpertLayerRunTrace exposes (expert_layer.h:63-76), for any
 * token count, as device buffers of the LAST run.  A field stays NULL when the
 * layer does not hold it.  Valid until the next run or destroy. */
typedef struct nmoe_trace_view {
  const float* normalized_input;   /* [tokens][hidden]; NULL after a large-batch run with
                                      nmoe_layer_keep_trace off */
  const float* router_logits;      /* [tokens][experts] */
  const int32_t* selected_index;   /* [tokens][top_k], selection order */
  const float* selected_weight;    /* [tokens][top_k] */
  const uint8_t* act_packed;       /* [tokens][hidden/2]  quantised normalised input */
  const uint8_t* act_scales;       /* [tokens][hidden/16] row-major E4M3 */
  const float* act_tensor_scale;   /* [tokens] */
  const float* parts;              /* [tokens][top_k+1][hidden]: weighted routed
                                      contributions in selection order, then shared.
                                      FP32 when the last run's output was FP32; a run
                                      with bf16 output keeps these rows in binary16
                                      and leaves this field NULL.  With latent
                                      projections: [tokens][top_k][latent], routed
                                      rows only */
  const float* latent_output;      /* [tokens][latent]: fc1_latent(normalized); NULL when
                                      the projection is the identity */
  const float* routed_latent_output; /* [tokens][latent]: the routed sum fed to fc2_latent */
  const float* projected_routed_output; /* [tokens][hidden]: fc2_latent of it */
  const float* shared_output;      /* [tokens][hidden] FP32; NULL without latent projections
                                      (the shared row is parts[t][top_k] there) */
} nmoe_trace_view;
NMOE_API nmoe_status nmoe_layer_trace_view(nmoe_layer* layer, nmoe_trace_view* out);
/* A layer keeps everything a trace may ask for (the default).  With enable == 0 it
 * stops writing the FP32 normalised rows where nothing but a trace reads them --
 * batches large enough for the two-pass router, whose kernels rebuild the rows
 * from the input -- which removes the largest write of the routing front end.
 * The reference captures a trace for one token only (expert_layer.cpp:775). */
NMOE_API nmoe_status nmoe_layer_keep_trace(nmoe_layer* layer, int32_t enable);
/* Copies one nmoe_trace_view field (index in declaration order, 0 =
 * normalized_input) of the last run into `dst` (device or host), `nbytes`
 * bytes, in stream order; NMOE_ERR_INVALID_ARGUMENT for a field that is NULL. */
NMOE_API nmoe_status nmoe_layer_copy_trace_field(nmoe_layer* layer, void* stream, int32_t field,
                                                 void* dst, size_t nbytes);

/* Copies the quantised relu^2 intermediates of the LAST run into
 * (token, slot)-ordered row-major buffers (device pointers):
 * routed_packed [tokens][top_k][I/2], routed_scales [tokens][top_k][I/16],
 * shared_packed [tokens][S/2], shared_scales [tokens][S/16].  Any may be NULL. */
NMOE_API nmoe_status nmoe_layer_export_hidden(nmoe_layer* layer, void* stream,
                                              uint8_t* routed_packed, uint8_t* routed_scales,
                                              uint8_t* shared_packed, uint8_t* shared_scales);

/* --- expert parallelism ------------------------------------------------------
 * No counterpart in the reference (single GPU, no collectives).  A layer created
 * with n_local_experts < n_routed_experts holds an equal share of the routed
 * experts (rank = first_local_expert / n_local_experts) and replicated router
 * and shared-expert weights.  One step = four device stages with two
 * all-to-all exchanges between them, which the HOST issues (NCCL): the library
 * never communicates.  Results equal the single-device layer's (bit for bit
 * with FP32 return rows).
 *
 *   nmoe_ep_dispatch   routes `tokens` own tokens and packs one record of
 *                      nmoe_ep_record_bytes() bytes per (token, slot) pair,
 *                      grouped by destination rank; returns the device address
 *                      of the records and of the int32[world] per-rank counts.
 *   -- exchange counts, then records (all-to-all-v, rows = records) --
 *   nmoe_ep_experts    runs this rank's experts over `count` received records
 *                      and writes one weighted down_proj row per record, in
 *                      arrival order, to out_rows [count][hidden] (FP32, bf16
 *                      or binary16).
 *   nmoe_ep_shared     shared expert over the tokens of the last dispatch (any
 *                      stream; independent of the exchange).
 *   -- return the rows (all-to-all-v with the splits swapped) --
 *   nmoe_ep_combine    output = input + (sum of the returned rows of each token
 *                      in selection order + shared).  returned_rows holds one
 *                      row per pair in the order the records were sent.
 *
 * Two record layouts.  capacity_per_rank == 0: records are compact, grouped by
 * destination rank, and the host must read the counts to size the exchange.
 * capacity_per_rank > 0: destination rank r owns the fixed segment
 * [r*capacity, (r+1)*capacity) of the send buffer, so every exchange has equal,
 * host-known splits and a step needs no host synchronisation (it can be recorded
 * once and replayed); the receiver passes the device counts it received
 * (valid_counts[source rank]) and count = world*capacity slots, and returns rows
 * in the same segmented layout.  A destination that would get more than
 * `capacity` pairs sets NMOE_ERR_CAPACITY (reported by nmoe_layer_sync_status).
 */
NMOE_API size_t nmoe_ep_record_bytes(const nmoe_layer* layer);
NMOE_API nmoe_status nmoe_ep_dispatch(nmoe_layer* layer, void* stream, const void* input,
                                      nmoe_dtype input_dtype, int64_t tokens,
                                      int64_t capacity_per_rank, const void** send_records,
                                      const int32_t** send_counts);
NMOE_API nmoe_status nmoe_ep_experts(nmoe_layer* layer, void* stream, const void* recv_records,
                                     int64_t count, const int32_t* valid_counts,
                                     int64_t capacity_per_rank, void* out_rows,
                                     nmoe_dtype rows_dtype);
NMOE_API nmoe_status nmoe_ep_shared(nmoe_layer* layer, void* stream);
NMOE_API nmoe_status nmoe_ep_combine(nmoe_layer* layer, void* stream, const void* input,
                                     nmoe_dtype input_dtype, const void* returned_rows,
                                     nmoe_dtype rows_dtype, void* output, nmoe_dtype output_dtype);

/* --- expert parallelism over peer windows ------------------------------------
 * The same four stages, with both exchanges done by the stages' own kernels
 * over NVLink instead of host-issued collectives (fixed-capacity layout only).
 * Every rank owns a "window": one device allocation holding its receive
 * segments for records, its segments for returned rows, and flag words.  The
 * other ranks of the node map it (CUDA IPC) and
 *   - the record packer stores each record directly into the destination
 *     rank's window,
 *   - the down-projection epilogue of the grouped GEMM stores each weighted
 *     row directly into the window of the rank the record came from, tile by
 *     tile while the GEMM runs,
 *   - small kernels raise a per-source flag (the step number) in the peer's
 *     window after the data, and the consumer's stream waits on its own flags
 *     with a bounded spin (NMOE_ERR_DEVICE_TIMEOUT after the limit of
 *     nmoe_layer_set_wait_limit_ms, about eight seconds by default; never a hang).
 * One buffer per direction suffices: a rank overwrites a peer's segment for
 * step s+1 only after its own combine of step s, which needed that peer's
 * rows of step s, which the peer produced after reading the segment.
 * A step records no host synchronisation and launches no collective.
 *
 * Setup (host): every rank calls nmoe_ep_window_create and receives a
 * NMOE_EP_WINDOW_HANDLE_BYTES handle; the host all-gathers the handles in rank
 * order and passes them to nmoe_ep_window_attach; a host barrier follows.
 * Teardown: host barrier, nmoe_ep_window_detach on every rank, host barrier,
 * then nmoe_layer_destroy.  All ranks must be processes on one node whose GPUs
 * have peer access.  No reference counterpart. */
#define NMOE_EP_WINDOW_HANDLE_BYTES 64
NMOE_API nmoe_status nmoe_ep_window_create(nmoe_layer* layer, int64_t capacity_per_rank,
                                           nmoe_dtype rows_dtype, void* handle_out);
NMOE_API nmoe_status nmoe_ep_window_attach(nmoe_layer* layer, const void* handles_in_rank_order);
NMOE_API nmoe_status nmoe_ep_window_detach(nmoe_layer* layer);
/* With enable != 0, nmoe_ep_window_dispatch also starts the shared expert, on a
 * stream of the layer's own, as soon as the rows are quantised, and
 * nmoe_ep_window_combine joins it: nmoe_ep_shared must then not be called. */
NMOE_API nmoe_status nmoe_ep_window_fork_shared(nmoe_layer* layer, int32_t enable);
/* route + pack into the peers' windows + raise the record flags */
NMOE_API nmoe_status nmoe_ep_window_dispatch(nmoe_layer* layer, void* stream, const void* input,
                                             nmoe_dtype input_dtype, int64_t tokens);
/* wait for the records of source ranks [first, first+count), run this rank's
 * experts over them, rows land in those ranks' windows, raise their row flags */
NMOE_API nmoe_status nmoe_ep_window_experts(nmoe_layer* layer, void* stream,
                                            int32_t first_source_rank, int32_t source_ranks);
/* wait for every rank's rows, then combine as nmoe_ep_combine does */
NMOE_API nmoe_status nmoe_ep_window_combine(nmoe_layer* layer, void* stream, const void* input,
                                            nmoe_dtype input_dtype, void* output,
                                            nmoe_dtype output_dtype);

/* --- one expert FFN: down(relu^2(up(x))) with NVFP4 weights ----------------
 * The composition ExpertLayerSlice::Run applies per (token, expert)
 * (expert_layer.cpp:913-922: RunNvfp4LinearHost, ApplyRelu2,
 * RunNvfp4LinearHost).  No norm, no residual. */
typedef struct nmoe_ffn nmoe_ffn;
NMOE_API nmoe_status nmoe_ffn_create(const nmoe_nvfp4_matrix* up, const nmoe_nvfp4_matrix* down,
                                     int32_t max_rows, nmoe_ffn** out_ffn);
NMOE_API void nmoe_ffn_destroy(nmoe_ffn* ffn);
/* input [rows][hidden] device FP32/bf16 -> output [rows][hidden] device FP32.
 * gemm_variant: 0 = choose by size, otherwise 1 + a tile-shape class (for tests):
 * 1 prefill tiles, 2 decode tiles (rows <= 32), 3 wide decode tiles, 4 prefill tiles
 * over CTA pairs. */
NMOE_API nmoe_status nmoe_ffn_run(nmoe_ffn* ffn, void* stream, const void* input,
                                  nmoe_dtype input_dtype, int64_t rows, float* output,
                                  int32_t gemm_variant);
NMOE_API nmoe_status nmoe_ffn_sync_status(nmoe_ffn* ffn, void* stream);
/* Quantised relu^2 intermediate of the last run: [rows][I/2], [rows][I/16]. */
NMOE_API nmoe_status nmoe_ffn_export_hidden(nmoe_ffn* ffn, void* stream, uint8_t* packed,
                                            uint8_t* scales);

/* --- unit operators (all pointers device, all asynchronous) ---------------- */

/* PackRowMajorFp32ToNvfp4 (nvfp4_packing.cpp:90-157) /
 * PackDeviceRowMajorFp32ToNvfp4 (device_nvfp4_matrix.cu:339-435).
 * per_row != 0: every row is packed as its own call (rows == 1 semantics, the
 * way the layer calls it, expert_layer.cpp:913) and tensor_scale has `rows`
 * entries; per_row == 0: one tensor scale for the whole matrix (input must be
 * FP32).  scales_row_major [rows][cols/16]; scales_swizzled (nullable) in the
 * 128x4 tile order of nvfp4_scale_layout.cpp:14-28, nmoe_swizzled_scale_bytes()
 * bytes, zero padded. */
NMOE_API nmoe_status nmoe_quantize_nvfp4(void* stream, const void* input, nmoe_dtype dtype,
                                         int64_t rows, int64_t cols, int32_t per_row,
                                         uint8_t* packed, uint8_t* scales_row_major,
                                         uint8_t* scales_swizzled, float* tensor_scale);
/* DequantizeNvfp4Matrix (expert_layer.cpp:154-186). */
NMOE_API nmoe_status nmoe_dequant_nvfp4(void* stream, const uint8_t* packed,
                                        const uint8_t* scales_row_major,
                                        const float* tensor_scale, int32_t per_row, int64_t rows,
                                        int64_t cols, float* output);
/* SwizzleRowMajorNvfp4ScalesForExecution (nvfp4_scale_layout.cpp:68-87). */
NMOE_API size_t nmoe_swizzled_scale_bytes(int64_t rows, int64_t cols);
NMOE_API nmoe_status nmoe_swizzle_scales(void* stream, const uint8_t* scales_row_major,
                                         int64_t rows, int64_t cols, uint8_t* scales_swizzled);
/* RmsNormFp32 (primitive_ops.cu:92-108) on [rows][hidden]. */
NMOE_API nmoe_status nmoe_rmsnorm(void* stream, const void* input, nmoe_dtype dtype, int64_t rows,
                                  int64_t hidden, const float* weight, float epsilon,
                                  float* output);
/* Gate projection (linear_op.cpp:97-118): logits[rows][experts] from FP32
 * activations and FP32 gate weights [experts][hidden]. */
NMOE_API nmoe_status nmoe_router_logits(void* stream, const float* normalized, const float* gate,
                                        int64_t rows, int32_t experts, int32_t hidden,
                                        float* logits);
/* SelectTopExperts (expert_layer.cpp:277-367) per row: indices (int32) and
 * weights in selection order. */
NMOE_API nmoe_status nmoe_router_topk(void* stream, const float* logits, const float* bias,
                                      int64_t rows, int32_t experts, int32_t top_k,
                                      int32_t n_group, int32_t topk_group,
                                      int32_t norm_topk_prob, float routed_scaling,
                                      int32_t* top_index, float* top_weight);

/* --- routing without any allocation ------------------------------------------
 * Has no counterpart in the reference (whose Run allocates six scratch tensors
 * per call, expert_layer.cpp:782-787).  For callers that are not allowed to
 * allocate device memory when they route tokens: a host whose memory all comes
 * from an arena reserved at start-up, a serving loop that cannot risk an
 * allocation stalling or failing, a plugin under foreign memory accounting.
 *
 * Computes, for `rows` rows of `input` [rows][hidden] (FP32 or bf16, device):
 * RMSNorm with `norm_weight`, gate logits against `gate` [experts][hidden] FP32,
 * then SelectTopExperts -- the same three kernels as nmoe_rmsnorm,
 * nmoe_router_logits and nmoe_router_topk, with identical results -- and writes
 * top_index / top_weight [rows][top_k].  The normalised rows and the logits
 * live in a fixed 4.5 MiB array inside the library image instead of in
 * caller buffers; the call performs no cudaMalloc, cudaFree or any other
 * allocating routine.
 *
 * Limits: rows*hidden <= NMOE_NOALLOC_MAX_ROWS_X_HIDDEN and rows*experts <=
 * NMOE_NOALLOC_MAX_ROWS_X_EXPERTS, otherwise NMOE_ERR_CAPACITY (e.g. 390 rows at
 * hidden 2688, 256 rows at hidden 4096 or at 512 experts).
 * Every GPU that loads the library holds the array until the process exits.
 * All calls on one GPU share it and it keeps the previous call's contents
 * (nothing in it needs clearing: each call overwrites what it reads), so two
 * calls whose kernels can overlap on the GPU -- different streams, no ordering
 * between them -- race; serialise them.
 * The first call on each device looks up the array's device address (the
 * device must be current); make that first call outside any stream capture.
 * The address is kept for the life of the process: after a cudaDeviceReset of a
 * device do not call this entry point on it again.
 * `input`, `norm_weight` and `gate` must be 16-byte aligned (the kernels read 16
 * bytes at a time); every argument is validated before the first kernel is
 * enqueued, so a rejected call leaves no work on the stream. */
#define NMOE_NOALLOC_MAX_ROWS_X_HIDDEN 1048576
#define NMOE_NOALLOC_MAX_ROWS_X_EXPERTS 131072
NMOE_API nmoe_status nmoe_route_tokens_noalloc(
    void* stream, const void* input, nmoe_dtype dtype, int64_t rows, int32_t hidden,
    const float* norm_weight, float epsilon, const float* gate, const float* bias,
    int32_t experts, int32_t top_k, int32_t n_group, int32_t topk_group,
    int32_t norm_topk_prob, float routed_scaling, int32_t* top_index, float* top_weight);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* NMOE_H_ */
