/*
 * nmoe_oracle.c -- CPU restatement of the NVFP4 mixture-of-experts layer of
 * kwindla/nemotron-inference.  TEST INFRASTRUCTURE ONLY: it is the checker for
 * the CUDA path and the timed CPU baseline; nothing in the shipped library
 * links, loads or calls it.
 *
 * Every function cites the reference file:line it restates (paths are
 * relative to the reference project root).  The arithmetic follows the
 * reference's host path operation by operation: FP32 multiplies and adds are
 * kept separate (build with -ffp-contract=off), the routed/shared matmuls
 * accumulate sequentially in FP32 along K, the router matmul accumulates
 * sequentially in double.
 *
 * Parity pin: the E2M1/E4M3 codecs, the packer, the scale swizzle, the top-k
 * selection and the single-row NVFP4 linear are compared with the reference's
 * own host functions (compiled from the reference sources into
 * oracle/_ref/ref_driver) by tests/test_oracle_vs_reference.py and with the
 * committed vectors in tests/golden/.
 *
 * Two things here have no counterpart in the reference and are marked as
 * such: the seeded weight quantiser (the reference only consumes
 * checkpoint-quantised weights) and the "admissible code" override used for
 * tie-aware parity.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define NMO_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Number formats                                                            */
/* ------------------------------------------------------------------------ */

/* E2M1 magnitudes, nibble bit 3 is the sign.  Restates DecodeFp4,
 * runtime/src/backend/expert_layer.cpp:142-146 (which defers to the CUDA
 * toolkit's __nv_fp4_e2m1 conversion). */
static const float kE2m1Magnitude[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

NMO_EXPORT float nmo_decode_e2m1(uint8_t nibble) {
  const float magnitude = kE2m1Magnitude[nibble & 7u];
  return (nibble & 8u) ? -magnitude : magnitude;
}

/* E4M3 (fn variant: no infinities, S.1111.111 is NaN, bias 7).  Restates
 * DecodeFp8, runtime/src/backend/expert_layer.cpp:148-152. */
NMO_EXPORT float nmo_decode_e4m3(uint8_t byte) {
  const int sign = byte >> 7;
  const int exponent = (byte >> 3) & 15;
  const int mantissa = byte & 7;
  float value;
  if (exponent == 15 && mantissa == 7) {
    value = NAN;
  } else if (exponent == 0) {
    value = ldexpf((float)mantissa, -9);
  } else {
    value = ldexpf((float)(8 + mantissa), exponent - 10);
  }
  return sign ? -value : value;
}

/* Round-to-nearest-even E2M1 with saturation to +-6.  Restates EncodeFp4,
 * runtime/src/backend/nvfp4_packing.cpp:37-41
 * (__nv_cvt_float_to_fp4(value, __NV_E2M1, cudaRoundNearest)).  Ties go to the
 * code with an even mantissa bit: 0.25->0, 0.75->1, 1.25->1, 1.75->2, 2.5->2,
 * 3.5->4, 5->4.  NaN encodes as +6 (0x7), like the toolkit conversion. */
NMO_EXPORT uint8_t nmo_encode_e2m1(float value) {
  uint32_t bits;
  memcpy(&bits, &value, sizeof(bits));
  const uint8_t sign = (uint8_t)((bits >> 31) << 3);
  const float a = fabsf(value);
  uint8_t code;
  if (a != a) {
    return 0x7u;
  }
  if (a <= 0.25f) {
    code = 0;
  } else if (a < 0.75f) {
    code = 1;
  } else if (a <= 1.25f) {
    code = 2;
  } else if (a < 1.75f) {
    code = 3;
  } else if (a <= 2.5f) {
    code = 4;
  } else if (a < 3.5f) {
    code = 5;
  } else if (a <= 5.0f) {
    code = 6;
  } else {
    code = 7;
  }
  return (uint8_t)(sign | code);
}

/* Round-to-nearest-even E4M3 with saturation to +-448 (NaN -> 0x7f).
 * Restates EncodeFp8Scale, runtime/src/backend/nvfp4_packing.cpp:43-46
 * (__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3)). */
NMO_EXPORT uint8_t nmo_encode_e4m3(float value) {
  uint32_t bits;
  memcpy(&bits, &value, sizeof(bits));
  const uint8_t sign = (uint8_t)((bits >> 31) << 7);
  const float a = fabsf(value);
  if (a != a) {
    return (uint8_t)(sign | 0x7fu);
  }
  if (a >= 464.0f) { /* halfway between 448 and the unrepresentable 480 */
    return (uint8_t)(sign | 0x7eu);
  }
  if (a < ldexpf(1.0f, -10)) { /* below half of the smallest subnormal 2^-9 */
    return sign;
  }
  int exponent;
  (void)frexpf(a, &exponent); /* a = m * 2^exponent, m in [0.5, 1) */
  int unbiased = exponent - 1;
  if (unbiased < -6) {
    unbiased = -6; /* subnormal range shares the quantum of the smallest normal */
  }
  /* quantum = 2^(unbiased-3); a/quantum is exact (power-of-two scaling). */
  const float scaled = ldexpf(a, 3 - unbiased);
  float rounded = nearbyintf(scaled); /* default rounding mode: nearest even */
  int biased = unbiased + 7;
  int q = (int)rounded;
  if (q >= 16) { /* mantissa carry into the next binade */
    q = 8;
    biased += 1;
  }
  uint8_t code;
  if (q < 8) { /* subnormal (only reachable with unbiased == -6) */
    code = (uint8_t)q;
  } else {
    code = (uint8_t)((biased << 3) | (q - 8));
  }
  if (code > 0x7eu) {
    code = 0x7eu;
  }
  return (uint8_t)(sign | code);
}

/* ------------------------------------------------------------------------ */
/* NVFP4 packer and scale layout                                             */
/* ------------------------------------------------------------------------ */

#define NMO_BLOCK 16
static const float kFp4Max = 6.0f;
static const float kFp8Max = 448.0f;
static const float kMinScale = 1.0f / 1024.0f;

/* ClampScale, runtime/src/backend/nvfp4_packing.cpp:19-24 */
static float clamp_scale(float value) {
  if (!isfinite(value) || value < kMinScale) {
    return kMinScale;
  }
  return value;
}

/* PackRowMajorFp32ToNvfp4, runtime/src/backend/nvfp4_packing.cpp:90-157.
 * One tensor scale for the whole [rows, cols] call (1.0 unless the global
 * amax exceeds 6*448); per 16-block scale = clamp(amax_b / (6*ts)) stored as
 * E4M3, all-zero block -> 1.0; values are divided by ts*block_scale with the
 * UNROUNDED block scale (:145) and encoded to E2M1, even column in the low
 * nibble (:146-152).  fixed_tensor_scale <= 0 means "dynamic".
 * Returns 0 on success, -1 on invalid arguments or non-finite input. */
NMO_EXPORT int nmo_pack_nvfp4(const float* data, size_t rows, size_t cols,
                              float fixed_tensor_scale, uint8_t* packed,
                              uint8_t* block_scales, float* tensor_scale_out) {
  if (data == NULL || rows == 0 || cols == 0 || cols % NMO_BLOCK != 0) {
    return -1;
  }
  float global_max = 0.0f;
  for (size_t i = 0; i < rows * cols; ++i) {
    if (!isfinite(data[i])) {
      return -1;
    }
    const float a = fabsf(data[i]);
    if (a > global_max) global_max = a;
  }
  float tensor_scale = 1.0f;
  if (fixed_tensor_scale > 0.0f && isfinite(fixed_tensor_scale)) {
    tensor_scale = clamp_scale(fixed_tensor_scale);
  } else if (global_max > kFp4Max * kFp8Max) {
    tensor_scale = clamp_scale(global_max / (kFp4Max * kFp8Max));
  }
  size_t packed_index = 0;
  size_t scale_index = 0;
  for (size_t row = 0; row < rows; ++row) {
    const float* row_data = data + row * cols;
    for (size_t block = 0; block < cols / NMO_BLOCK; ++block) {
      const float* b = row_data + block * NMO_BLOCK;
      float block_max = 0.0f;
      for (int i = 0; i < NMO_BLOCK; ++i) {
        const float a = fabsf(b[i]);
        if (a > block_max) block_max = a;
      }
      float block_scale = 1.0f;
      if (block_max > 0.0f) {
        block_scale = clamp_scale(block_max / (kFp4Max * tensor_scale));
      }
      block_scales[scale_index++] = nmo_encode_e4m3(block_scale);
      const float scale = tensor_scale * block_scale;
      for (int i = 0; i < NMO_BLOCK; i += 2) {
        const uint8_t lo = nmo_encode_e2m1(b[i] / scale) & 0x0fu;
        const uint8_t hi = nmo_encode_e2m1(b[i + 1] / scale) & 0x0fu;
        packed[packed_index++] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
  *tensor_scale_out = tensor_scale;
  return 0;
}

/* DequantizeNvfp4Matrix, runtime/src/backend/expert_layer.cpp:154-186:
 * value = E2M1(nibble) * (E4M3(scale) * tensor_scale), scale product first. */
NMO_EXPORT int nmo_dequant_nvfp4(const uint8_t* packed, const uint8_t* block_scales,
                                 float tensor_scale, size_t rows, size_t cols,
                                 float* out) {
  if (packed == NULL || block_scales == NULL || cols == 0 || cols % NMO_BLOCK != 0) {
    return -1;
  }
  size_t packed_index = 0;
  size_t scale_index = 0;
  for (size_t row = 0; row < rows; ++row) {
    for (size_t block = 0; block < cols / NMO_BLOCK; ++block) {
      const float s = nmo_decode_e4m3(block_scales[scale_index++]) * tensor_scale;
      float* o = out + row * cols + block * NMO_BLOCK;
      for (int i = 0; i < NMO_BLOCK; i += 2) {
        const uint8_t byte = packed[packed_index++];
        o[i] = nmo_decode_e2m1(byte & 0x0fu) * s;
        o[i + 1] = nmo_decode_e2m1((byte >> 4) & 0x0fu) * s;
      }
    }
  }
  return 0;
}

/* ExecutionScaleOffset / BuildNvfp4ExecutionScaleLayout,
 * runtime/src/backend/nvfp4_scale_layout.cpp:14-28, :45-66.  Rows pad to 128,
 * 16-blocks pad to 4; a 512-byte tile holds 128 rows x 4 blocks. */
NMO_EXPORT size_t nmo_swizzled_scale_bytes(size_t rows, size_t cols) {
  if (rows == 0 || cols == 0 || cols % NMO_BLOCK != 0) return 0;
  const size_t padded_rows = (rows + 127u) / 128u * 128u;
  const size_t padded_blocks = (cols / NMO_BLOCK + 3u) / 4u * 4u;
  return padded_rows * padded_blocks;
}

NMO_EXPORT size_t nmo_swizzled_scale_offset(size_t row, size_t block_col,
                                            size_t padded_blocks_per_row) {
  const size_t k_tiles = padded_blocks_per_row / 4u;
  const size_t m_tile = row / 128u;
  const size_t k_tile = block_col / 4u;
  return (((m_tile * k_tiles) + k_tile) << 9) | ((row & 31u) << 4) |
         (((row >> 5) & 3u) << 2) | (block_col & 3u);
}

/* SwizzleRowMajorNvfp4ScalesForExecution,
 * runtime/src/backend/nvfp4_scale_layout.cpp:68-87.  out must hold
 * nmo_swizzled_scale_bytes(rows, cols) bytes; padding bytes are zero. */
NMO_EXPORT int nmo_swizzle_scales(const uint8_t* row_major, size_t rows, size_t cols,
                                  uint8_t* out) {
  const size_t nbytes = nmo_swizzled_scale_bytes(rows, cols);
  if (nbytes == 0 || row_major == NULL) return -1;
  const size_t blocks = cols / NMO_BLOCK;
  const size_t padded_blocks = (blocks + 3u) / 4u * 4u;
  memset(out, 0, nbytes);
  for (size_t row = 0; row < rows; ++row) {
    for (size_t b = 0; b < blocks; ++b) {
      out[nmo_swizzled_scale_offset(row, b, padded_blocks)] = row_major[row * blocks + b];
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------ */
/* Seeded weight quantiser (NOT in the reference: it only loads checkpoint   */
/* NVFP4).  global = amax/(6*448); block scale = E4M3(amax_b/(6*global));    */
/* code = E2M1(w / (global * decoded_block_scale)).  The DECODED block scale */
/* divides the value here, the standard NVFP4 weight recipe.                 */
/* ------------------------------------------------------------------------ */
NMO_EXPORT int nmo_quantize_weight(const float* w, size_t rows, size_t cols,
                                   uint8_t* packed, uint8_t* block_scales,
                                   float* tensor_scale_out) {
  if (w == NULL || rows == 0 || cols == 0 || cols % NMO_BLOCK != 0) return -1;
  float amax = 0.0f;
  for (size_t i = 0; i < rows * cols; ++i) {
    const float a = fabsf(w[i]);
    if (a > amax) amax = a;
  }
  float global = amax / (kFp4Max * kFp8Max);
  if (!(global > 0.0f)) global = 1.0f;
  const size_t blocks = cols / NMO_BLOCK;
#pragma omp parallel for schedule(static)
  for (size_t row = 0; row < rows; ++row) {
    for (size_t blk = 0; blk < blocks; ++blk) {
      const float* b = w + row * cols + blk * NMO_BLOCK;
      float block_max = 0.0f;
      for (int i = 0; i < NMO_BLOCK; ++i) {
        const float a = fabsf(b[i]);
        if (a > block_max) block_max = a;
      }
      uint8_t code = nmo_encode_e4m3(block_max / (kFp4Max * global));
      float decoded = nmo_decode_e4m3(code);
      if (!(decoded > 0.0f)) { /* all-zero or underflowing block */
        code = 0x38u;          /* 1.0 */
        decoded = 1.0f;
      }
      block_scales[row * blocks + blk] = code;
      const float scale = global * decoded;
      uint8_t* out = packed + (row * cols + blk * NMO_BLOCK) / 2;
      for (int i = 0; i < NMO_BLOCK; i += 2) {
        const uint8_t lo = nmo_encode_e2m1(b[i] / scale) & 0x0fu;
        const uint8_t hi = nmo_encode_e2m1(b[i + 1] / scale) & 0x0fu;
        out[i / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
  *tensor_scale_out = global;
  return 0;
}

/* ------------------------------------------------------------------------ */
/* RMSNorm, router, top-k                                                    */
/* ------------------------------------------------------------------------ */

/* RmsNormKernel, runtime/src/backend/primitive_ops.cu:26-59, restated on the
 * host: 256 strided partial sums of squares (nvcc contracts value*value+sum
 * into an FMA, hence fmaf), a halving tree over the 256 partials, then
 * y = x * inv_rms * w evaluated left to right.  The device kernel uses
 * rsqrtf (<= 2 ulp); here inv_rms = 1/sqrt(mean+eps) with two correctly
 * rounded FP32 operations, which the CUDA path reproduces bit for bit. */
NMO_EXPORT void nmo_rmsnorm(const float* x, const float* weight, size_t rows,
                            size_t hidden, float eps, float* y) {
#pragma omp parallel for schedule(static)
  for (size_t row = 0; row < rows; ++row) {
    const float* xr = x + row * hidden;
    float partial[256];
    for (size_t t = 0; t < 256; ++t) {
      float s = 0.0f;
      for (size_t c = t; c < hidden; c += 256) {
        s = fmaf(xr[c], xr[c], s);
      }
      partial[t] = s;
    }
    for (size_t stride = 128; stride > 0; stride /= 2) {
      for (size_t t = 0; t < stride; ++t) {
        partial[t] += partial[t + stride];
      }
    }
    const float mean = partial[0] / (float)hidden;
    const float inv_rms = 1.0f / sqrtf(mean + eps);
    float* yr = y + row * hidden;
    for (size_t c = 0; c < hidden; ++c) {
      yr[c] = xr[c] * inv_rms * weight[c];
    }
  }
}

/* Router logits: the dense fallback of UploadedLinearOp::Run,
 * runtime/src/backend/linear_op.cpp:97-118 -- sequential DOUBLE accumulation
 * of FP32 activations times FP32-upcast gate weights, rounded to FP32. */
NMO_EXPORT void nmo_router_logits(const float* y, const float* gate, size_t rows,
                                  size_t experts, size_t hidden, float* logits) {
#pragma omp parallel for schedule(static)
  for (size_t row = 0; row < rows; ++row) {
    for (size_t e = 0; e < experts; ++e) {
      double accum = 0.0;
      const float* a = y + row * hidden;
      const float* w = gate + e * hidden;
      for (size_t c = 0; c < hidden; ++c) {
        accum += (double)a[c] * (double)w[c];
      }
      logits[row * experts + e] = (float)accum;
    }
  }
}

/* Sigmoid, runtime/src/backend/expert_layer.cpp:129-136 (std::exp on float). */
NMO_EXPORT float nmo_sigmoid(float value) {
  if (value >= 0.0f) {
    const float exp_neg = expf(-value);
    return 1.0f / (1.0f + exp_neg);
  }
  const float exp_pos = expf(value);
  return exp_pos / (1.0f + exp_pos);
}

typedef struct {
  float score;
  int index;
} nmo_scored;

/* Selection of the `count` largest entries in descending order.  The
 * reference uses std::partial_sort (expert_layer.cpp:321-325, :342-346) whose
 * order among equal keys is unspecified; this restatement breaks ties by the
 * lower index. */
static void select_top(nmo_scored* items, int n, int count) {
  for (int i = 0; i < count; ++i) {
    int best = i;
    for (int j = i + 1; j < n; ++j) {
      if (items[j].score > items[best].score ||
          (items[j].score == items[best].score && items[j].index < items[best].index)) {
        best = j;
      }
    }
    const nmo_scored tmp = items[i];
    items[i] = items[best];
    items[best] = tmp;
  }
}

/* SelectTopExperts, runtime/src/backend/expert_layer.cpp:277-367, for one
 * token.  scores = sigmoid(logits); choice = scores + bias; group score =
 * sum of the two largest choices in the group (:299-318); the best
 * topk_group groups are kept, other groups' choices become 0.0 (:332-339);
 * top_k by choice; weight = score WITHOUT bias (:350-355), normalised by
 * (sum + 1e-20) when norm_topk_prob (:357-362), then times the routed
 * scaling factor (:363-365).  Returns the number of selections written. */
NMO_EXPORT int nmo_select_top_experts(const float* logits, const float* bias, int experts,
                                      int top_k, int n_group, int topk_group,
                                      int norm_topk_prob, float routed_scaling,
                                      int32_t* out_index, float* out_weight) {
  if (experts <= 0 || top_k <= 0 || n_group <= 0 || topk_group <= 0 ||
      experts % n_group != 0) {
    return 0;
  }
  float* scores = (float*)malloc(sizeof(float) * (size_t)experts);
  float* choice = (float*)malloc(sizeof(float) * (size_t)experts);
  nmo_scored* groups = (nmo_scored*)malloc(sizeof(nmo_scored) * (size_t)n_group);
  nmo_scored* masked = (nmo_scored*)malloc(sizeof(nmo_scored) * (size_t)experts);
  char* group_selected = (char*)calloc((size_t)n_group, 1);
  for (int i = 0; i < experts; ++i) {
    scores[i] = nmo_sigmoid(logits[i]);
    choice[i] = scores[i] + bias[i];
  }
  const int group_size = experts / n_group;
  for (int g = 0; g < n_group; ++g) {
    float top1 = -INFINITY, top2 = -INFINITY;
    for (int i = 0; i < group_size; ++i) {
      const float v = choice[g * group_size + i];
      if (v > top1) {
        top2 = top1;
        top1 = v;
      } else if (v > top2) {
        top2 = v;
      }
    }
    if (!isfinite(top2)) top2 = top1;
    groups[g].score = top1 + top2;
    groups[g].index = g;
  }
  const int group_count = topk_group < n_group ? topk_group : n_group;
  select_top(groups, n_group, group_count);
  for (int i = 0; i < group_count; ++i) group_selected[groups[i].index] = 1;
  for (int i = 0; i < experts; ++i) {
    masked[i].score = group_selected[i / group_size] ? choice[i] : 0.0f;
    masked[i].index = i;
  }
  const int count = top_k < experts ? top_k : experts;
  select_top(masked, experts, count);
  float weight_sum = 0.0f;
  for (int i = 0; i < count; ++i) {
    out_index[i] = masked[i].index;
    out_weight[i] = scores[masked[i].index];
    weight_sum += out_weight[i];
  }
  if (norm_topk_prob) {
    const float denominator = weight_sum + 1.0e-20f;
    for (int i = 0; i < count; ++i) out_weight[i] /= denominator;
  }
  for (int i = 0; i < count; ++i) out_weight[i] *= routed_scaling;
  free(scores);
  free(choice);
  free(groups);
  free(masked);
  free(group_selected);
  return count;
}

/* Smallest gap between the top_k-th and (top_k+1)-th choice score of one
 * token (n_group == 1 view); the parity harness reports it so that a routing
 * mismatch can be attributed to a near-tie. */
NMO_EXPORT float nmo_selection_margin(const float* logits, const float* bias, int experts,
                                      int top_k) {
  nmo_scored* items = (nmo_scored*)malloc(sizeof(nmo_scored) * (size_t)experts);
  for (int i = 0; i < experts; ++i) {
    items[i].score = nmo_sigmoid(logits[i]) + bias[i];
    items[i].index = i;
  }
  const int count = top_k + 1 < experts ? top_k + 1 : experts;
  select_top(items, experts, count);
  const float margin = count > top_k ? items[top_k - 1].score - items[top_k].score : INFINITY;
  free(items);
  return margin;
}

/* ------------------------------------------------------------------------ */
/* NVFP4 linear                                                              */
/* ------------------------------------------------------------------------ */

/* Relu2, runtime/src/backend/expert_layer.cpp:138-140 */
static inline float relu2(float v) { return v > 0.0f ? v * v : 0.0f; }

/* Literal RunNvfp4LinearHost for ONE activation row,
 * runtime/src/backend/expert_layer.cpp:231-267: pack the row (dynamic tensor
 * scale), dequantise it, dequantise the whole weight, then
 * CpuMatmulRowMajor (:212-229): out[o] = sum_c a[c]*w[o][c], FP32, c
 * ascending.  Slow on purpose; the grouped path below is proven bit-equal to
 * it in tests/test_oracle.py. */
NMO_EXPORT int nmo_nvfp4_linear_row_literal(const float* activation, size_t out_rows,
                                            size_t in_cols, const uint8_t* w_packed,
                                            const uint8_t* w_scales, float w_tensor_scale,
                                            float* out) {
  uint8_t* a_packed = (uint8_t*)malloc(in_cols / 2);
  uint8_t* a_scales = (uint8_t*)malloc(in_cols / NMO_BLOCK);
  float* a_deq = (float*)malloc(sizeof(float) * in_cols);
  float* w_deq = (float*)malloc(sizeof(float) * out_rows * in_cols);
  float a_ts = 1.0f;
  int rc = nmo_pack_nvfp4(activation, 1, in_cols, 0.0f, a_packed, a_scales, &a_ts);
  if (rc == 0) rc = nmo_dequant_nvfp4(a_packed, a_scales, a_ts, 1, in_cols, a_deq);
  if (rc == 0) rc = nmo_dequant_nvfp4(w_packed, w_scales, w_tensor_scale, out_rows, in_cols, w_deq);
  if (rc == 0) {
    for (size_t o = 0; o < out_rows; ++o) {
      float accum = 0.0f;
      for (size_t c = 0; c < in_cols; ++c) {
        accum += a_deq[c] * w_deq[o * in_cols + c];
      }
      out[o] = accum;
    }
  }
  free(a_packed);
  free(a_scales);
  free(a_deq);
  free(w_deq);
  return rc;
}

/* Dequantise a weight into K-major ("transposed") FP32 so that the grouped
 * matmul can run K outermost and vectorise across output rows while every
 * output still sees the same sequential FP32 accumulation along K. */
static void dequant_weight_transposed(const uint8_t* packed, const uint8_t* scales,
                                      float tensor_scale, size_t out_rows, size_t in_cols,
                                      float* wt /* [in_cols][out_rows] */) {
  const size_t blocks = in_cols / NMO_BLOCK;
  for (size_t o = 0; o < out_rows; ++o) {
    for (size_t blk = 0; blk < blocks; ++blk) {
      const float s = nmo_decode_e4m3(scales[o * blocks + blk]) * tensor_scale;
      const uint8_t* p = packed + (o * in_cols + blk * NMO_BLOCK) / 2;
      for (int i = 0; i < NMO_BLOCK; i += 2) {
        const uint8_t byte = p[i / 2];
        wt[(blk * NMO_BLOCK + i) * out_rows + o] = nmo_decode_e2m1(byte & 0x0fu) * s;
        wt[(blk * NMO_BLOCK + i + 1) * out_rows + o] = nmo_decode_e2m1(byte >> 4) * s;
      }
    }
  }
}

/* out[o] = sum_c a[c] * wt[c][o], c ascending, separate FP32 multiply and
 * add: the same operations in the same order as CpuMatmulRowMajor
 * (expert_layer.cpp:212-229) for every output o. */
static void matvec_transposed(const float* a, const float* wt, size_t out_rows,
                              size_t in_cols, float* out) {
  for (size_t o = 0; o < out_rows; ++o) out[o] = 0.0f;
  for (size_t c = 0; c < in_cols; ++c) {
    const float ac = a[c];
    const float* w = wt + c * out_rows;
    for (size_t o = 0; o < out_rows; ++o) {
      out[o] += ac * w[o];
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Admissible-code override (tie-aware parity; not in the reference)         */
/* ------------------------------------------------------------------------ */

/* A device result may legitimately differ from this oracle in a quantised
 * intermediate when the FP32 value being quantised sits within rounding
 * noise of a code boundary: both sides accumulate the K products of the up
 * projection in FP32, in different orders.  Given the oracle's own
 * pre-activation row `u` (h = relu^2(u) is what gets quantised) and a
 * candidate (packed, scales) row from the device, a differing code or scale
 * byte is ADOPTED when the smallest shift of the pre-activation that makes the
 * reference packer emit the device's byte is at most `limit` noise units, and
 * counted as INADMISSIBLE otherwise.
 *
 * Noise unit of output i: 2^-24 * sum_c |a[c] * w[i][c]|.  A sequential FP32
 * sum of K random-sign terms carries an rms error of about half that unit
 * (each add rounds at relative 2^-24 of a partial sum that performs a random
 * walk), so a handful of units covers the largest accumulation error among
 * ~10^8 outputs, while a systematic error in the GEMM or its epilogue (a wrong
 * scale, a dropped K block) is thousands of units.  A code is also given the
 * pre-activation equivalent of the block maximum's noise, because the divisor
 * of every value of a block derives from that maximum.
 *
 * Only rows whose tensor scale is 1.0 are considered (larger rows keep the
 * oracle's codes).  The largest adopted distance is reported so that a test
 * can assert how close to the boundary the adopted values really were. */
typedef struct {
  int64_t adopted_codes;
  int64_t adopted_scales;
  int64_t inadmissible_codes;
  int64_t inadmissible_scales;
  double max_noise_units; /* largest adopted shift, in noise units */
  double max_rel_shift;   /* the same shift relative to |u| */
} nmo_override_stats;

static int e2m1_rank(uint8_t code) {
  const int mag = code & 7;
  return (code & 8) ? -mag : mag;
}

/* what the packer needs to know about the row being checked */
typedef struct {
  const float* u;    /* [cols] pre-activation (before relu^2) */
  const float* a;    /* [K] dequantised activation row */
  const float* wt;   /* [K][cols] dequantised up_proj, transposed */
  size_t k;
  size_t cols;
} nmo_override_row;

static double noise_unit(const nmo_override_row* row, size_t i) {
  double sum = 0.0;
  for (size_t c = 0; c < row->k; ++c) sum += fabs((double)row->a[c] * (double)row->wt[c * row->cols + i]);
  return sum * 5.9604644775390625e-08; /* 2^-24 */
}

static float relu2_shifted(float u, double shift) {
  const float v = (float)((double)u + shift);
  return v > 0.0f ? v * v : 0.0f;
}

/* smallest |shift| (searched up to `bound`, direction `dir`) for which
 * rank(shifted value) reaches `target`; negative when even `bound` does not. */
static double code_shift(float u, float bs, int target, int dir, double bound) {
  const int at_bound = e2m1_rank(nmo_encode_e2m1(relu2_shifted(u, dir * bound) / bs));
  if (dir > 0 ? at_bound < target : at_bound > target) return -1.0;
  double lo = 0.0, hi = bound;
  for (int it = 0; it < 48; ++it) {
    const double mid = 0.5 * (lo + hi);
    const int r = e2m1_rank(nmo_encode_e2m1(relu2_shifted(u, dir * mid) / bs));
    if (dir > 0 ? r >= target : r <= target) hi = mid; else lo = mid;
  }
  return hi;
}

static double scale_shift(float u, int target, int dir, double bound) {
  float m = relu2_shifted(u, dir * bound);
  int at_bound = nmo_encode_e4m3(m > 0.0f ? clamp_scale(m / kFp4Max) : 1.0f);
  if (dir > 0 ? at_bound < target : at_bound > target) return -1.0;
  double lo = 0.0, hi = bound;
  for (int it = 0; it < 48; ++it) {
    const double mid = 0.5 * (lo + hi);
    m = relu2_shifted(u, dir * mid);
    const int r = nmo_encode_e4m3(m > 0.0f ? clamp_scale(m / kFp4Max) : 1.0f);
    if (dir > 0 ? r >= target : r <= target) hi = mid; else lo = mid;
  }
  return hi;
}

static void note_adopted(nmo_override_stats* stats, double shift, double unit, float u) {
  const double units = shift / unit;
  if (units > stats->max_noise_units) stats->max_noise_units = units;
  const double rel = fabs((double)u) > 0.0 ? shift / fabs((double)u) : 0.0;
  if (rel > stats->max_rel_shift) stats->max_rel_shift = rel;
}

/* Returns 1 when anything was adopted. */
static int apply_override(const nmo_override_row* row, float tensor_scale, uint8_t* packed,
                          uint8_t* scales, const uint8_t* cand_packed,
                          const uint8_t* cand_scales, float limit, nmo_override_stats* stats) {
  if (tensor_scale != 1.0f) return 0;
  int adopted = 0;
  for (size_t blk = 0; blk < row->cols / NMO_BLOCK; ++blk) {
    const float* ub = row->u + blk * NMO_BLOCK;
    const int scale_differs = cand_scales[blk] != scales[blk];
    int codes_differ = 0;
    for (size_t j = 0; j < NMO_BLOCK / 2; ++j) {
      codes_differ |= packed[blk * (NMO_BLOCK / 2) + j] != cand_packed[blk * (NMO_BLOCK / 2) + j];
    }
    if (!scale_differs && !codes_differ) continue;
    /* the block maximum decides the block scale */
    int i_max = 0;
    for (int i = 1; i < NMO_BLOCK; ++i) {
      if (ub[i] > ub[i_max]) i_max = i;
    }
    const float block_max = relu2(ub[i_max]);
    const float bs = block_max > 0.0f ? clamp_scale(block_max / kFp4Max) : 1.0f;
    const double unit_max = noise_unit(row, blk * NMO_BLOCK + (size_t)i_max);
    if (scale_differs) {
      const int dir = cand_scales[blk] > scales[blk] ? 1 : -1;
      const double shift = scale_shift(ub[i_max], cand_scales[blk], dir, unit_max * limit);
      if (shift >= 0.0 && unit_max > 0.0) {
        scales[blk] = cand_scales[blk];
        stats->adopted_scales++;
        note_adopted(stats, shift, unit_max, ub[i_max]);
        adopted = 1;
      } else {
        stats->inadmissible_scales++;
      }
    }
    for (int i = 0; i < NMO_BLOCK; ++i) {
      const size_t byte_index = (blk * NMO_BLOCK + (size_t)i) / 2;
      const int shift_bits = (i & 1) ? 4 : 0;
      const uint8_t mine = (packed[byte_index] >> shift_bits) & 0x0fu;
      const uint8_t theirs = (cand_packed[byte_index] >> shift_bits) & 0x0fu;
      if (mine == theirs) continue;
      const int r_mine = e2m1_rank(mine), r_theirs = e2m1_rank(theirs);
      if (r_mine == r_theirs) continue; /* +0 and -0 */
      /* own accumulation noise plus the share of the block maximum's */
      double unit = noise_unit(row, blk * NMO_BLOCK + (size_t)i);
      if (ub[i_max] > 0.0f && ub[i] > 0.0f) unit += (double)ub[i] * unit_max / (double)ub[i_max];
      const double shift =
          code_shift(ub[i], bs, r_theirs, r_theirs > r_mine ? 1 : -1, unit * limit);
      if (shift >= 0.0 && unit > 0.0) {
        packed[byte_index] =
            (uint8_t)((packed[byte_index] & ~(0x0fu << shift_bits)) | (theirs << shift_bits));
        stats->adopted_codes++;
        note_adopted(stats, shift, unit, ub[i]);
        adopted = 1;
      } else {
        stats->inadmissible_codes++;
      }
    }
  }
  return adopted;
}

static void merge_override_stats(nmo_override_stats* total, const nmo_override_stats* local) {
  total->adopted_codes += local->adopted_codes;
  total->adopted_scales += local->adopted_scales;
  total->inadmissible_codes += local->inadmissible_codes;
  total->inadmissible_scales += local->inadmissible_scales;
  if (local->max_noise_units > total->max_noise_units) total->max_noise_units = local->max_noise_units;
  if (local->max_rel_shift > total->max_rel_shift) total->max_rel_shift = local->max_rel_shift;
}

/* ------------------------------------------------------------------------ */
/* The layer                                                                 */
/* ------------------------------------------------------------------------ */

typedef struct {
  const uint8_t* packed; /* [out_rows][in_cols/2] */
  const uint8_t* scales; /* [out_rows][in_cols/16] E4M3 */
  float tensor_scale;
} nmo_nvfp4_weight;

typedef struct {
  int32_t hidden;              /* H */
  int32_t routed_intermediate; /* I */
  int32_t shared_intermediate; /* S */
  int32_t experts;             /* E */
  int32_t top_k;
  int32_t n_group;
  int32_t topk_group;
  int32_t norm_topk_prob;
  float rms_eps;
  float routed_scaling;
  int32_t latent;  /* moe_latent_size; 0 = hidden (no latent projections) */
} nmo_layer_config;

typedef struct {
  const float* norm_weight; /* [H] */
  const float* gate;        /* [E][H], bf16 values widened to FP32 */
  const float* bias;        /* [E] e_score_correction_bias */
  const nmo_nvfp4_weight* up;   /* [E] each [I][H] */
  const nmo_nvfp4_weight* down; /* [E] each [H][I] */
  nmo_nvfp4_weight shared_up;   /* [S][H] */
  nmo_nvfp4_weight shared_down; /* [H][S] */
  const float* logit_offset;    /* optional [E] added to the FP32 logits (not in the
                                   reference: synthetic skewed-load hook) */
  /* Dense / scaled-FP8 linears as the FP32 matrices the reference multiplies with
   * (UploadedLinearOp, linear_op.cpp:274-303; DequantizeScaledFp8WeightToHostFp32,
   * scaled_fp8_linear.cu:121-139).  NULL = absent.  *_input_scale > 0 selects the
   * scaled-FP8 family's activation round trip (scaled_fp8_linear.cu:231-236). */
  const float* fc1;             /* [latent][H] */
  float fc1_input_scale;
  const float* fc2;             /* [H][latent] */
  const float* shared_up_dense; /* [S][H]; replaces shared_up */
  float shared_up_input_scale;
  const float* shared_down_dense; /* [H][S]; replaces shared_down */
  float shared_down_input_scale;
} nmo_layer_weights;

/* Optional outputs (NULL to skip) and optional device candidates for the
 * admissible-code override (NULL to skip). */
typedef struct {
  float* normalized;      /* [T][H] */
  float* logits;          /* [T][E] */
  int32_t* top_index;     /* [T][k] */
  float* top_weight;      /* [T][k] */
  uint8_t* act_packed;    /* [T][H/2]   quantised normalised activations */
  uint8_t* act_scales;    /* [T][H/16] */
  float* act_tensor_scale;/* [T] */
  uint8_t* hid_packed;    /* [T][k][I/2]  quantised relu^2 intermediates */
  uint8_t* hid_scales;    /* [T][k][I/16] */
  float* routed_out;      /* [T][k][H]  unweighted down_proj outputs */
  uint8_t* shid_packed;   /* [T][S/2] */
  uint8_t* shid_scales;   /* [T][S/16] */
  float* shared_out;      /* [T][H] */
  const uint8_t* cand_hid_packed;  /* device candidates, same shapes */
  const uint8_t* cand_hid_scales;
  const uint8_t* cand_shid_packed;
  const uint8_t* cand_shid_scales;
  float override_limit;     /* admissible shift of a pre-activation, in noise units */
  nmo_override_stats stats;
  uint8_t* adopted_token;   /* optional [T]: 1 where a code or scale of the token was adopted */
  float* latent;            /* optional [T][latent]: fc1_latent output */
  float* routed_latent;     /* optional [T][latent]: routed sum */
  float* projected;         /* optional [T][H]: fc2_latent of it */
  float* hid_values;        /* optional [T][k][I]: relu^2(up_proj) before quantisation */
  float* shid_values;       /* optional [T][S]: the same for the shared expert */
} nmo_layer_trace;

/* One expert FFN on a single activation row that is ALREADY dequantised:
 * up -> relu^2 -> pack(row) -> [override] -> dequant -> down.
 * Follows expert_layer.cpp:913-922 (routed) and :814-818/:956-964/:981-1005
 * (shared, with shared_up taken through the NVFP4 host linear as well). */
static int expert_row(const float* a_deq, size_t H, size_t I, const float* up_t,
                      const float* down_t, float* scratch_u /* [I] */, float* scratch_h /* [I] */,
                      float* scratch_hd /* [I] */, uint8_t* hq /* [I/2] */,
                      uint8_t* hs /* [I/16] */, const uint8_t* cand_q,
                      const uint8_t* cand_s, float limit, nmo_override_stats* stats,
                      int* adopted, float* out /* [H] */) {
  matvec_transposed(a_deq, up_t, I, H, scratch_u);
  for (size_t i = 0; i < I; ++i) scratch_h[i] = relu2(scratch_u[i]);
  float ts = 1.0f;
  if (nmo_pack_nvfp4(scratch_h, 1, I, 0.0f, hq, hs, &ts) != 0) return -1;
  if (cand_q != NULL && cand_s != NULL) {
    const nmo_override_row row = {scratch_u, a_deq, up_t, H, I};
    const int any = apply_override(&row, ts, hq, hs, cand_q, cand_s, limit, stats);
    if (adopted != NULL && any) *adopted = 1;
  }
  nmo_dequant_nvfp4(hq, hs, ts, 1, I, scratch_hd);
  matvec_transposed(scratch_hd, down_t, H, I, out);
  return 0;
}

/* ScaledFp8LinearOp::Run's activation round trip (scaled_fp8_linear.cu:231-236):
 * value / scale -> E4M3 satfinite -> decode -> * scale, scale clamped as in :27-33. */
NMO_EXPORT void nmo_fp8_round_trip(const float* in, size_t count, float input_scale, float* out) {
  const float scale = clamp_scale(input_scale);
  for (size_t i = 0; i < count; ++i) {
    out[i] = nmo_decode_e4m3(nmo_encode_e4m3(in[i] / scale)) * scale;
  }
}

/* A dense or scaled-FP8 linear over `rows` rows: DOUBLE accumulation
 * (linear_op.cpp:97-118, scaled_fp8_linear.cu:40-62). */
static void dense_linear(const float* in, size_t rows, size_t in_cols, const float* weight,
                         size_t out_rows, float input_scale, float* out) {
  if (input_scale > 0.0f) {
    float* tmp = (float*)malloc(sizeof(float) * rows * in_cols);
    nmo_fp8_round_trip(in, rows * in_cols, input_scale, tmp);
    nmo_router_logits(tmp, weight, rows, out_rows, in_cols, out);
    free(tmp);
  } else {
    nmo_router_logits(in, weight, rows, out_rows, in_cols, out);
  }
}

/* The whole layer for T tokens of FP32 input, restructured for speed but
 * arithmetically identical per (token, expert) to the reference's loop
 * (expert_layer.cpp:795-1069).  Latent projections fc1 / fc2 dense or scaled
 * FP8 or absent (identity); routed experts NVFP4 on latent rows; shared_up and
 * shared_down NVFP4, dense or scaled FP8.  Returns 0 on success. */
NMO_EXPORT int nmo_layer_forward(const nmo_layer_config* cfg, const nmo_layer_weights* w,
                                 const float* x, int64_t T, float* out,
                                 nmo_layer_trace* trace) {
  const size_t H = (size_t)cfg->hidden, I = (size_t)cfg->routed_intermediate,
               S = (size_t)cfg->shared_intermediate, E = (size_t)cfg->experts,
               K = (size_t)cfg->top_k;
  const size_t L = cfg->latent > 0 ? (size_t)cfg->latent : H;
  if (T <= 0 || H % NMO_BLOCK || I % NMO_BLOCK || S % NMO_BLOCK || L % NMO_BLOCK) return -1;
  if ((w->fc1 == NULL) != (w->fc2 == NULL) || (w->fc1 == NULL && L != H)) return -1;
  const size_t Tn = (size_t)T;
  int status = 0;

  float* y = (float*)malloc(sizeof(float) * Tn * H);
  float* logits = (float*)malloc(sizeof(float) * Tn * E);
  int32_t* top_index = (int32_t*)malloc(sizeof(int32_t) * Tn * K);
  float* top_weight = (float*)malloc(sizeof(float) * Tn * K);
  float* lat = w->fc1 ? (float*)malloc(sizeof(float) * Tn * L) : y;
  float* a_deq = (float*)malloc(sizeof(float) * Tn * L);  /* what the routed up_proj sees */
  float* y_deq = NULL;                                     /* what an NVFP4 shared_up sees */
  float* routed = (float*)malloc(sizeof(float) * Tn * K * L);
  float* routed_sum = (float*)malloc(sizeof(float) * Tn * L);
  float* projected = w->fc2 ? (float*)malloc(sizeof(float) * Tn * H) : routed_sum;
  float* shared = (float*)malloc(sizeof(float) * Tn * H);
  uint8_t* aq = (uint8_t*)malloc(Tn * L / 2);
  uint8_t* as = (uint8_t*)malloc(Tn * L / NMO_BLOCK);
  float* ats = (float*)malloc(sizeof(float) * Tn);

  /* :795-799 RMSNorm + gate projection */
  nmo_rmsnorm(x, w->norm_weight, Tn, H, cfg->rms_eps, y);
  nmo_router_logits(y, w->gate, Tn, E, H, logits);
  if (w->logit_offset != NULL) {
    for (size_t i = 0; i < Tn * E; ++i) logits[i] = logits[i] + w->logit_offset[i % E];
  }
  /* :809-813 latent = fc1_latent(normalized) */
  if (w->fc1) dense_linear(y, Tn, H, w->fc1, L, w->fc1_input_scale, lat);

  /* :881 top-k per token; :913 activation pack per row (rows == 1) */
#pragma omp parallel for schedule(static)
  for (size_t t = 0; t < Tn; ++t) {
    const int n = nmo_select_top_experts(logits + t * E, w->bias, (int)E, (int)K,
                                         cfg->n_group, cfg->topk_group, cfg->norm_topk_prob,
                                         cfg->routed_scaling, top_index + t * K,
                                         top_weight + t * K);
    if (n != (int)K) {
#pragma omp atomic write
      status = -2;
    }
    if (nmo_pack_nvfp4(lat + t * L, 1, L, 0.0f, aq + t * L / 2, as + t * L / NMO_BLOCK,
                       ats + t) != 0) {
#pragma omp atomic write
      status = -3;
    }
    nmo_dequant_nvfp4(aq + t * L / 2, as + t * L / NMO_BLOCK, ats[t], 1, L, a_deq + t * L);
  }
  if (status != 0) goto done;
  if (w->fc1 && w->shared_up_dense == NULL) {
    /* an NVFP4 shared_up packs the normalised hidden row itself */
    y_deq = (float*)malloc(sizeof(float) * Tn * H);
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < Tn; ++t) {
      uint8_t* q = (uint8_t*)malloc(H / 2);
      uint8_t* sc = (uint8_t*)malloc(H / NMO_BLOCK);
      float ts = 1.0f;
      nmo_pack_nvfp4(y + t * H, 1, H, 0.0f, q, sc, &ts);
      nmo_dequant_nvfp4(q, sc, ts, 1, H, y_deq + t * H);
      free(q);
      free(sc);
    }
  }

  /* bucket (token, slot) pairs by expert */
  {
    size_t* count = (size_t*)calloc(E + 1, sizeof(size_t));
    size_t* start = (size_t*)calloc(E + 1, sizeof(size_t));
    size_t* pairs = (size_t*)malloc(sizeof(size_t) * Tn * K);
    for (size_t p = 0; p < Tn * K; ++p) count[top_index[p]]++;
    for (size_t e = 0; e < E; ++e) start[e + 1] = start[e] + count[e];
    memset(count, 0, sizeof(size_t) * (E + 1));
    for (size_t p = 0; p < Tn * K; ++p) {
      const size_t e = (size_t)top_index[p];
      pairs[start[e] + count[e]++] = p;
    }

    nmo_override_stats total = {0, 0, 0, 0, 0.0, 0.0};
    if (trace && trace->adopted_token) memset(trace->adopted_token, 0, Tn);
#pragma omp parallel
    {
      float* up_t = (float*)malloc(sizeof(float) * L * I);
      float* down_t = (float*)malloc(sizeof(float) * L * I);
      float* u = (float*)malloc(sizeof(float) * I);
      float* h = (float*)malloc(sizeof(float) * I);
      float* hd = (float*)malloc(sizeof(float) * I);
      uint8_t* hq = (uint8_t*)malloc(I / 2);
      uint8_t* hs = (uint8_t*)malloc(I / NMO_BLOCK);
      nmo_override_stats local = {0, 0, 0, 0, 0.0, 0.0};
#pragma omp for schedule(dynamic, 1)
      for (size_t e = 0; e < E; ++e) {
        if (count[e] == 0) continue;
        dequant_weight_transposed(w->up[e].packed, w->up[e].scales, w->up[e].tensor_scale,
                                  I, L, up_t);
        dequant_weight_transposed(w->down[e].packed, w->down[e].scales,
                                  w->down[e].tensor_scale, L, I, down_t);
        for (size_t j = 0; j < count[e]; ++j) {
          const size_t p = pairs[start[e] + j];
          const size_t t = p / K;
          const uint8_t* cq = NULL;
          const uint8_t* cs = NULL;
          if (trace && trace->cand_hid_packed && trace->cand_hid_scales) {
            cq = trace->cand_hid_packed + p * (I / 2);
            cs = trace->cand_hid_scales + p * (I / NMO_BLOCK);
          }
          int adopted = 0;
          if (expert_row(a_deq + t * L, L, I, up_t, down_t, u, h, hd, hq, hs, cq, cs,
                         trace ? trace->override_limit : 0.0f, &local, &adopted,
                         routed + p * L) != 0) {
#pragma omp atomic write
            status = -4;
          }
          if (adopted && trace && trace->adopted_token) {
#pragma omp atomic write
            trace->adopted_token[t] = 1;
          }
          if (trace && trace->hid_packed) memcpy(trace->hid_packed + p * (I / 2), hq, I / 2);
          if (trace && trace->hid_scales)
            memcpy(trace->hid_scales + p * (I / NMO_BLOCK), hs, I / NMO_BLOCK);
          if (trace && trace->hid_values) memcpy(trace->hid_values + p * I, h, sizeof(float) * I);
        }
      }
      free(up_t);
      free(down_t);
      free(u);
      free(h);
      free(hd);
      free(hq);
      free(hs);
#pragma omp critical
      merge_override_stats(&total, &local);
    }

    /* shared expert, one "expert" over all tokens (:814-818, :956-964, :981-1045) */
    if (w->shared_up_dense == NULL && w->shared_down_dense == NULL) {
      const float* shared_in = y_deq ? y_deq : a_deq;
      float* up_t = (float*)malloc(sizeof(float) * H * S);
      float* down_t = (float*)malloc(sizeof(float) * H * S);
      dequant_weight_transposed(w->shared_up.packed, w->shared_up.scales,
                                w->shared_up.tensor_scale, S, H, up_t);
      dequant_weight_transposed(w->shared_down.packed, w->shared_down.scales,
                                w->shared_down.tensor_scale, H, S, down_t);
#pragma omp parallel
      {
        float* u = (float*)malloc(sizeof(float) * S);
        float* h = (float*)malloc(sizeof(float) * S);
        float* hd = (float*)malloc(sizeof(float) * S);
        uint8_t* hq = (uint8_t*)malloc(S / 2);
        uint8_t* hs = (uint8_t*)malloc(S / NMO_BLOCK);
        nmo_override_stats local = {0, 0, 0, 0, 0.0, 0.0};
#pragma omp for schedule(dynamic, 4)
        for (size_t t = 0; t < Tn; ++t) {
          const uint8_t* cq = NULL;
          const uint8_t* cs = NULL;
          if (trace && trace->cand_shid_packed && trace->cand_shid_scales) {
            cq = trace->cand_shid_packed + t * (S / 2);
            cs = trace->cand_shid_scales + t * (S / NMO_BLOCK);
          }
          int adopted = 0;
          if (expert_row(shared_in + t * H, H, S, up_t, down_t, u, h, hd, hq, hs, cq, cs,
                         trace ? trace->override_limit : 0.0f, &local, &adopted,
                         shared + t * H) != 0) {
#pragma omp atomic write
            status = -5;
          }
          if (adopted && trace && trace->adopted_token) {
#pragma omp atomic write
            trace->adopted_token[t] = 1;
          }
          if (trace && trace->shid_packed) memcpy(trace->shid_packed + t * (S / 2), hq, S / 2);
          if (trace && trace->shid_scales)
            memcpy(trace->shid_scales + t * (S / NMO_BLOCK), hs, S / NMO_BLOCK);
          if (trace && trace->shid_values) memcpy(trace->shid_values + t * S, h, sizeof(float) * S);
        }
        free(u);
        free(h);
        free(hd);
        free(hq);
        free(hs);
#pragma omp critical
        merge_override_stats(&total, &local);
      }
      free(up_t);
      free(down_t);
    } else {
      /* dense / scaled-FP8 shared_up (:814-818) and relu^2 (:956-964); an NVFP4
       * shared_up beside a dense shared_down goes through the host linear too */
      float* su = (float*)malloc(sizeof(float) * Tn * S);
      if (w->shared_up_dense) {
        dense_linear(y, Tn, H, w->shared_up_dense, S, w->shared_up_input_scale, su);
      } else {
        const float* shared_in = y_deq ? y_deq : a_deq;
        float* up_t = (float*)malloc(sizeof(float) * H * S);
        dequant_weight_transposed(w->shared_up.packed, w->shared_up.scales,
                                  w->shared_up.tensor_scale, S, H, up_t);
#pragma omp parallel for schedule(static)
        for (size_t t = 0; t < Tn; ++t) matvec_transposed(shared_in + t * H, up_t, S, H, su + t * S);
        free(up_t);
      }
      for (size_t i = 0; i < Tn * S; ++i) su[i] = relu2(su[i]);
      if (trace && trace->shid_values) memcpy(trace->shid_values, su, sizeof(float) * Tn * S);
      if (w->shared_down_dense) {
        dense_linear(su, Tn, S, w->shared_down_dense, H, w->shared_down_input_scale, shared);
      } else {
        /* NVFP4 shared_down through RunNvfp4LinearHost per row (:981-1005) */
        float* down_t = (float*)malloc(sizeof(float) * H * S);
        dequant_weight_transposed(w->shared_down.packed, w->shared_down.scales,
                                  w->shared_down.tensor_scale, H, S, down_t);
#pragma omp parallel
        {
          float* hd = (float*)malloc(sizeof(float) * S);
          uint8_t* hq = (uint8_t*)malloc(S / 2);
          uint8_t* hs = (uint8_t*)malloc(S / NMO_BLOCK);
#pragma omp for schedule(dynamic, 4)
          for (size_t t = 0; t < Tn; ++t) {
            float ts = 1.0f;
            nmo_pack_nvfp4(su + t * S, 1, S, 0.0f, hq, hs, &ts);
            nmo_dequant_nvfp4(hq, hs, ts, 1, S, hd);
            matvec_transposed(hd, down_t, H, S, shared + t * H);
            if (trace && trace->shid_packed) memcpy(trace->shid_packed + t * (S / 2), hq, S / 2);
            if (trace && trace->shid_scales)
              memcpy(trace->shid_scales + t * (S / NMO_BLOCK), hs, S / NMO_BLOCK);
          }
          free(hd);
          free(hq);
          free(hs);
        }
        free(down_t);
      }
      free(su);
    }
    if (trace) trace->stats = total;
    free(count);
    free(start);
    free(pairs);
  }

  /* :951-953 weighted accumulate in selection order */
#pragma omp parallel for schedule(static)
  for (size_t t = 0; t < Tn; ++t) {
    for (size_t i = 0; i < L; ++i) {
      float acc = 0.0f;
      for (size_t k = 0; k < K; ++k) {
        acc += routed[(t * K + k) * L + i] * top_weight[t * K + k];
      }
      routed_sum[t * L + i] = acc;
    }
  }
  /* :1047-1053 fc2_latent; :1064-1069 mixer and residual */
  if (w->fc2) dense_linear(routed_sum, Tn, L, w->fc2, H, 0.0f, projected);
#pragma omp parallel for schedule(static)
  for (size_t t = 0; t < Tn; ++t) {
    for (size_t i = 0; i < H; ++i) {
      const float mixer = projected[t * H + i] + shared[t * H + i];
      out[t * H + i] = x[t * H + i] + mixer;
    }
  }

  if (trace) {
    if (trace->normalized) memcpy(trace->normalized, y, sizeof(float) * Tn * H);
    if (trace->logits) memcpy(trace->logits, logits, sizeof(float) * Tn * E);
    if (trace->top_index) memcpy(trace->top_index, top_index, sizeof(int32_t) * Tn * K);
    if (trace->top_weight) memcpy(trace->top_weight, top_weight, sizeof(float) * Tn * K);
    if (trace->act_packed) memcpy(trace->act_packed, aq, Tn * L / 2);
    if (trace->act_scales) memcpy(trace->act_scales, as, Tn * L / NMO_BLOCK);
    if (trace->act_tensor_scale) memcpy(trace->act_tensor_scale, ats, sizeof(float) * Tn);
    if (trace->routed_out) memcpy(trace->routed_out, routed, sizeof(float) * Tn * K * L);
    if (trace->shared_out) memcpy(trace->shared_out, shared, sizeof(float) * Tn * H);
    if (trace->latent) memcpy(trace->latent, lat, sizeof(float) * Tn * L);
    if (trace->routed_latent) memcpy(trace->routed_latent, routed_sum, sizeof(float) * Tn * L);
    if (trace->projected) memcpy(trace->projected, projected, sizeof(float) * Tn * H);
  }

done:
  free(y);
  free(logits);
  free(top_index);
  free(top_weight);
  if (w->fc1) free(lat);
  free(a_deq);
  free(y_deq);
  free(routed);
  free(routed_sum);
  if (w->fc2) free(projected);
  free(shared);
  free(aq);
  free(as);
  free(ats);
  return status;
}

/* One expert FFN over `rows` FP32 activation rows: pack(row) -> dequant ->
 * up -> relu^2 -> pack(row) -> [override] -> dequant -> down, i.e. two
 * RunNvfp4LinearHost calls (expert_layer.cpp:913-922) per row with the weights
 * dequantised once.  Optional outputs may be NULL. */
NMO_EXPORT int nmo_expert_ffn_forward(const float* x, int64_t rows, int32_t hidden,
                                      int32_t inter, const nmo_nvfp4_weight* up,
                                      const nmo_nvfp4_weight* down, float* out,
                                      uint8_t* hid_packed, uint8_t* hid_scales,
                                      const uint8_t* cand_packed, const uint8_t* cand_scales,
                                      float override_limit, nmo_override_stats* stats,
                                      uint8_t* adopted_row) {
  const size_t H = (size_t)hidden, I = (size_t)inter, R = (size_t)rows;
  if (rows <= 0 || H % NMO_BLOCK || I % NMO_BLOCK) return -1;
  int status = 0;
  float* up_t = (float*)malloc(sizeof(float) * H * I);
  float* down_t = (float*)malloc(sizeof(float) * H * I);
  dequant_weight_transposed(up->packed, up->scales, up->tensor_scale, I, H, up_t);
  dequant_weight_transposed(down->packed, down->scales, down->tensor_scale, H, I, down_t);
  nmo_override_stats total = {0, 0, 0, 0, 0.0, 0.0};
#pragma omp parallel
  {
    float* a = (float*)malloc(sizeof(float) * H);
    uint8_t* aq = (uint8_t*)malloc(H / 2);
    uint8_t* as = (uint8_t*)malloc(H / NMO_BLOCK);
    float* u = (float*)malloc(sizeof(float) * I);
    float* h = (float*)malloc(sizeof(float) * I);
    float* hd = (float*)malloc(sizeof(float) * I);
    uint8_t* hq = (uint8_t*)malloc(I / 2);
    uint8_t* hs = (uint8_t*)malloc(I / NMO_BLOCK);
    nmo_override_stats local = {0, 0, 0, 0, 0.0, 0.0};
#pragma omp for schedule(dynamic, 4)
    for (size_t r = 0; r < R; ++r) {
      float ats = 1.0f;
      int adopted = 0;
      if (nmo_pack_nvfp4(x + r * H, 1, H, 0.0f, aq, as, &ats) != 0) {
#pragma omp atomic write
        status = -3;
        continue;
      }
      nmo_dequant_nvfp4(aq, as, ats, 1, H, a);
      if (expert_row(a, H, I, up_t, down_t, u, h, hd, hq, hs,
                     cand_packed ? cand_packed + r * (I / 2) : NULL,
                     cand_scales ? cand_scales + r * (I / NMO_BLOCK) : NULL, override_limit,
                     &local, &adopted, out + r * H) != 0) {
#pragma omp atomic write
        status = -4;
      }
      if (hid_packed) memcpy(hid_packed + r * (I / 2), hq, I / 2);
      if (hid_scales) memcpy(hid_scales + r * (I / NMO_BLOCK), hs, I / NMO_BLOCK);
      if (adopted_row) adopted_row[r] = (uint8_t)adopted;
    }
    free(a); free(aq); free(as); free(u); free(h); free(hd); free(hq); free(hs);
#pragma omp critical
    merge_override_stats(&total, &local);
  }
  if (stats) *stats = total;
  free(up_t);
  free(down_t);
  return status;
}

/* The literal per-token loop (expert_layer.cpp:871-1005, :1064-1069) built
 * from nmo_nvfp4_linear_row_literal: re-packs the activation and
 * re-dequantises the whole weight for every (token, expert, projection).
 * Used on tiny shapes to prove nmo_layer_forward bit-equal to it. */
NMO_EXPORT int nmo_layer_forward_literal(const nmo_layer_config* cfg,
                                         const nmo_layer_weights* w, const float* x,
                                         int64_t T, float* out) {
  const size_t H = (size_t)cfg->hidden, I = (size_t)cfg->routed_intermediate,
               S = (size_t)cfg->shared_intermediate, E = (size_t)cfg->experts,
               K = (size_t)cfg->top_k;
  const size_t Tn = (size_t)T;
  float* y = (float*)malloc(sizeof(float) * Tn * H);
  float* logits = (float*)malloc(sizeof(float) * Tn * E);
  float* up = (float*)malloc(sizeof(float) * (I > S ? I : S));
  float* down = (float*)malloc(sizeof(float) * H);
  float* routed = (float*)malloc(sizeof(float) * H);
  int32_t* idx = (int32_t*)malloc(sizeof(int32_t) * K);
  float* wt = (float*)malloc(sizeof(float) * K);
  int status = 0;
  nmo_rmsnorm(x, w->norm_weight, Tn, H, cfg->rms_eps, y);
  nmo_router_logits(y, w->gate, Tn, E, H, logits);
  if (w->logit_offset != NULL) {
    for (size_t i = 0; i < Tn * E; ++i) logits[i] = logits[i] + w->logit_offset[i % E];
  }
  for (size_t t = 0; t < Tn && status == 0; ++t) {
    if (nmo_select_top_experts(logits + t * E, w->bias, (int)E, (int)K, cfg->n_group,
                               cfg->topk_group, cfg->norm_topk_prob, cfg->routed_scaling,
                               idx, wt) != (int)K) {
      status = -2;
      break;
    }
    for (size_t i = 0; i < H; ++i) routed[i] = 0.0f;
    for (size_t k = 0; k < K; ++k) {
      const nmo_nvfp4_weight* wu = &w->up[idx[k]];
      const nmo_nvfp4_weight* wd = &w->down[idx[k]];
      status |= nmo_nvfp4_linear_row_literal(y + t * H, I, H, wu->packed, wu->scales,
                                             wu->tensor_scale, up);
      for (size_t i = 0; i < I; ++i) up[i] = relu2(up[i]);
      status |= nmo_nvfp4_linear_row_literal(up, H, I, wd->packed, wd->scales,
                                             wd->tensor_scale, down);
      for (size_t i = 0; i < H; ++i) routed[i] += down[i] * wt[k];
    }
    status |= nmo_nvfp4_linear_row_literal(y + t * H, S, H, w->shared_up.packed,
                                           w->shared_up.scales, w->shared_up.tensor_scale, up);
    for (size_t i = 0; i < S; ++i) up[i] = relu2(up[i]);
    status |= nmo_nvfp4_linear_row_literal(up, H, S, w->shared_down.packed,
                                           w->shared_down.scales,
                                           w->shared_down.tensor_scale, down);
    for (size_t i = 0; i < H; ++i) {
      const float mixer = routed[i] + down[i];
      out[t * H + i] = x[t * H + i] + mixer;
    }
  }
  free(y);
  free(logits);
  free(up);
  free(down);
  free(routed);
  free(idx);
  free(wt);
  return status;
}

NMO_EXPORT int nmo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
