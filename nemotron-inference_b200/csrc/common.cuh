// Shared device helpers: number formats, PTX wrappers for mbarrier / TMA /
// tcgen05, and small utilities.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace nmoe {

// Status words a kernel can leave in the layer's device error slot.
enum DeviceError : int {
  kDevOk = 0,
  kDevWaitTimeout = 1,      // a bounded mbarrier wait gave up
  kDevActivationRange = 2,  // a relu^2 row exceeded 6*448: per-row tensor scale != 1
  kDevPlanOverflow = 3,     // more row tiles than the workspace was sized for
};

constexpr int kQuantBlock = 16;
constexpr float kFp4Max = 6.0f;
constexpr float kFp8Max = 448.0f;
constexpr float kMinScale = 1.0f / 1024.0f;

// ---------------------------------------------------------------------------
// Number formats.  The reference decodes through the toolkit's __nv_fp4_e2m1 /
// __nv_fp8_e4m3 (runtime/src/backend/expert_layer.cpp:142-152) and encodes with
// __nv_cvt_float_to_fp4(.., cudaRoundNearest) / __nv_cvt_float_to_fp8(..,
// __NV_SATFINITE, __NV_E4M3) (runtime/src/backend/nvfp4_packing.cpp:37-46).
// The device side calls the same toolkit conversions, which lower to the
// cvt.rn.satfinite.e2m1x2.f32 / e4m3x2 hardware instructions on sm_100a.
// ---------------------------------------------------------------------------

__device__ __forceinline__ float decode_e2m1(uint32_t nibble) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign
  const uint32_t m = nibble & 7u;
  const float mag = m < 2u ? 0.5f * static_cast<float>(m)
                           : __uint_as_float((((m >> 1) + 126u) << 23) | ((m & 1u) << 22));
  return (nibble & 8u) ? -mag : mag;
}

__device__ __forceinline__ float decode_e4m3(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ uint32_t encode_e4m3(float v) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// Two floats -> one byte, `even` in the low nibble, `odd` in the high nibble
// (nvfp4_packing.cpp:146-152).
__device__ __forceinline__ uint32_t encode_e2m1x2(float even, float odd) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp4x2(make_float2(even, odd), __NV_E2M1, cudaRoundNearest));
}

// ClampScale, nvfp4_packing.cpp:19-24
__device__ __forceinline__ float clamp_scale(float v) {
  return (!isfinite(v) || v < kMinScale) ? kMinScale : v;
}

inline float clamp_scale_host(float v) {
  return (!(v == v) || v > 3.0e38f || v < kMinScale) ? kMinScale : v;
}

// Quantise 16 FP32 values that share one block (per-row tensor scale `ts`):
// returns the E4M3 scale byte, writes 8 packed bytes into two 32-bit words.
// Follows nvfp4_packing.cpp:130-153 with IEEE divisions.
__device__ __forceinline__ uint32_t quantize_block16(const float (&v)[16], float ts,
                                                     uint32_t& lo_word, uint32_t& hi_word) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  float bs = 1.0f;
  if (amax > 0.0f) bs = clamp_scale(__fdiv_rn(amax, __fmul_rn(kFp4Max, ts)));
  const uint32_t scale_byte = encode_e4m3(bs);
  const float divisor = __fmul_rn(ts, bs);
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    const uint32_t byte = encode_e2m1x2(__fdiv_rn(v[i], divisor), __fdiv_rn(v[i + 1], divisor));
    w[i / 8] |= (byte & 0xffu) << (8 * ((i / 2) & 3));
  }
  lo_word = w[0];
  hi_word = w[1];
  return scale_byte;
}

// Correctly rounded x / d for d > 0 given r = RN(1/d): one multiply and two
// FMAs (q = RN(x r); q + r * RN(x - q d)).  The residual correction yields the
// IEEE quotient whenever r is the correctly rounded reciprocal and d's
// significand is not all ones (Markstein); the caller handles that one
// significand with a full division.
__device__ __forceinline__ float div_by_reciprocal(float x, float d, float r) {
  const float q = __fmul_rn(x, r);
  const float e = __fmaf_rn(-q, d, x);
  return __fmaf_rn(e, r, q);
}

// The fused quantiser of the up-projection epilogue: 16 non-negative values
// whose maximum is `amax`, per-row tensor scale 1 (nvfp4_packing.cpp:119-153
// with tensor_scale == 1.0).  Bit-identical to quantize_block16(v, 1.0f, ..).
__device__ __forceinline__ uint32_t quantize_block16_unit_scale(const float (&v)[16], float amax,
                                                                uint32_t& lo_word,
                                                                uint32_t& hi_word) {
  float bs = 1.0f;
  if (amax > 0.0f) bs = clamp_scale(__fdiv_rn(amax, kFp4Max));
  const uint32_t scale_byte = encode_e4m3(bs);
  uint32_t w[2] = {0u, 0u};
  if ((__float_as_uint(bs) & 0x007fffffu) != 0x007fffffu) {
    const float r = __frcp_rn(bs);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const uint32_t byte = encode_e2m1x2(div_by_reciprocal(v[i], bs, r),
                                          div_by_reciprocal(v[i + 1], bs, r));
      w[i / 8] |= (byte & 0xffu) << (8 * ((i / 2) & 3));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const uint32_t byte = encode_e2m1x2(__fdiv_rn(v[i], bs), __fdiv_rn(v[i + 1], bs));
      w[i / 8] |= (byte & 0xffu) << (8 * ((i / 2) & 3));
    }
  }
  lo_word = w[0];
  hi_word = w[1];
  return scale_byte;
}

// Offset of the scale of (row, 16-block) inside the 128-row x 4-block tiled
// layout of runtime/src/backend/nvfp4_scale_layout.cpp:14-28.  `k_tiles` is the
// number of 4-block groups each 128-row tile stores.
__host__ __device__ __forceinline__ size_t swizzled_scale_offset(size_t row, size_t block,
                                                                 size_t k_tiles) {
  return ((((row >> 7) * k_tiles) + (block >> 2)) << 9) | ((row & 31u) << 4) |
         (((row >> 5) & 3u) << 2) | (block & 3u);
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait: gives up after ~2^31 clock ticks (about a second) so that a
// protocol bug or a lost copy can never hang the GPU.  Returns false on
// timeout; the caller records kDevWaitTimeout and unwinds.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - start > (1ll << 31)) return false;
  }
  return true;
}

// The same bounded wait polling with test_wait, which returns at once instead of
// suspending the thread for a hardware-chosen time: lower wake-up latency for the waits
// on a kernel's critical path, at the price of a hot spin.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_test_wait(bar, parity)) {
    if (clock64() - start > (1ll << 31)) return false;
  }
  return true;
}

// 2-D tiled TMA load (no multicast) into this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// 1-D bulk copy global -> shared (16-byte aligned addresses and size).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// --- tcgen05 ---------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrive on an mbarrier once every tcgen05 operation this thread issued so far
// has completed.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor (sm_100 format, version 1).
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version (1)
//   bits 61-63 swizzle (0 none, 2 = 128 B)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swizzle) {
  return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) |
         (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(swizzle) << 61);
}

// Copy 32 rows x 16 bytes of scale factors from shared memory into 4 TMEM
// columns, replicated to all four 32-lane quarters.
__device__ __forceinline__ void tcgen05_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
               : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-16 UE4M3 block scales taken from
// TMEM; E2M1 operands, K = 64 per instruction.
__device__ __forceinline__ void tcgen05_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t sfa_tmem,
                                                 uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
      "r"(sfb_tmem)
      : "memory");
}

// Instruction descriptor for kind::mxf4nvf4: E2M1 x E2M1, UE4M3 scales,
// both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t make_idesc_nvf4(uint32_t n) {
  return (1u << 7) /* A = E2M1 */ | (1u << 10) /* B = E2M1 */ | ((n >> 3) << 17) |
         (0u << 23) /* scale format UE4M3 */ | ((128u >> 4) << 24);
}

// 32 lanes x 16 consecutive FP32 columns: thread i receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  // The wait shares the asm statement with the load so that no use of the
  // destination registers can be scheduled between them.
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without its wait: several may be in flight before one tmem_ld_fence()
// per destination array.  The destination registers are undefined until then.
__device__ __forceinline__ void tmem_ld_x16_async(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns from registers: thread i writes row (lane
// base + i).  Complete after tmem_st_wait().
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// After tmem_ld_wait(): ties every later use of `r` to a volatile statement behind the
// wait, so that the compiler cannot schedule a use of the registers before it.
__device__ __forceinline__ void tmem_ld_fence(uint32_t (&r)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) asm volatile("" : "+r"(r[i]));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

// --- CTA pairs (cta_group::2) -------------------------------------------------
// Two CTAs of a cluster of size 2 drive one tcgen05.mma with M = 256: each CTA
// holds 128 rows of A and half of B's rows in its own shared memory (at the same
// offsets), each accumulates its own 128 rows in its own TMEM.  One thread of the
// leader (cluster rank 0) issues the MMAs and the scale copies for both.

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Arrive on the mbarrier at the same shared-memory offset in CTA `target_rank`
// of this cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t target_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(smem_u32(bar)), "r"(target_rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote)
               : "memory");
}

// try_wait that acquires at cluster scope: pairs with mbar_arrive_remote.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (clock64() - start > (1ll << 31)) return false;
  }
  return true;
}

// 2-D tiled TMA load into this CTA's shared memory whose completion bytes are counted
// on the mbarrier `leader_bar`, a shared::cluster address that may lie in the partner
// CTA of the pair (cluster_address_of): both CTAs' loads of a stage complete on the
// leader's barrier.  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x,
                                                 int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}

// The shared::cluster address of `local` (an address in this CTA's shared memory) in
// CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_address_of(const void* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote)
               : "r"(smem_u32(local)), "r"(rank));
  return remote;
}

// TMEM allocation for a pair: one warp of EACH CTA executes it, the same columns
// are allocated in both.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(columns)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
               : "memory");
}

// Arrive, once every tcgen05 operation this thread issued so far has completed, on
// the mbarrier at this offset in every CTA of `cta_mask` (bit i = cluster rank i).
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(smem_u32(bar)),
      "h"(cta_mask)
      : "memory");
}

// Scale copy in both CTAs of the pair: each copies from its own shared memory (same
// offset) into its own TMEM.
__device__ __forceinline__ void tcgen05_cp_pair_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
               : "memory");
}

__device__ __forceinline__ void tcgen05_mma_pair_nvf4(uint32_t d_tmem, uint64_t a_desc,
                                                      uint64_t b_desc, uint32_t idesc,
                                                      uint32_t sfa_tmem, uint32_t sfb_tmem,
                                                      uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"
      " [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
      "r"(sfb_tmem)
      : "memory");
}

// Instruction descriptor of make_idesc_nvf4 with M = 256 (a CTA pair).
__host__ __device__ constexpr uint32_t make_idesc_nvf4_pair(uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (0u << 23) | ((256u >> 4) << 24);
}

}  // namespace nmoe
