// Shared pieces of the W4A16 decode kernels (w4a16_gemv.cu, w4a16_gemv_persist.cu): launch
// parameters, workspace layout, mbarrier / bulk-copy / shared-memory primitives.
#pragma once

#include "common.cuh"
#include "peer.cuh"

namespace pare {
namespace gemv {


constexpr int kMaxStepsPerWarp = 8;   // 16-row blocks x 128-column steps per warp: RB * steps <= 8
constexpr int kTabCols = 16;          // activation rows per call (two MMA column blocks)
constexpr uint32_t kSpinLimit = 1u << 22;

// Workspace layout: [counters | status word][prepared activations][step table][partials fp32].  The counter region has a FIXED
// size so the partial sums of one call can never land where another call keeps its counters;
// the counters are the only part that must be zero between calls.
constexpr size_t kCounterInts = 16384;
constexpr size_t kCounterBytes = kCounterInts * sizeof(int);
constexpr size_t kStatusIndex = kCounterInts - 1;

struct GemvParams {
  const void* x;
  int64_t ldx;
  const uint8_t* packed;
  const float* scale;
  const float* zero;
  const uint32_t* meta_h2;
  const int32_t* col_perm;
  const float* input_scale;
  const void* bias;
  void* y;
  int64_t ldy;
  int M, N, K;
  int ngroups;          // K / group_size
  int steps_per_group;  // group_size / 128
  int steps_per_split;  // 128-column steps per CTA
  int splits;
  void* xp;             // [M][K] fp16 activations in operand order (workspace)
  float4* tabg;         // [K/128][kTabCols] (E, SX, g, -) per step and activation row (workspace)
  float* partial;       // [splits][M][N]
  int* counters;        // [row tiles]; counters[kStatusIndex] is the status word
  int x_vec_ok;
  // activations computed inside the kernel (stage.cuh) instead of read from xp / tabg
  int producer;         // 0 = none, PARE_PRODUCER_RMSNORM, PARE_PRODUCER_SILU_MUL
  const void* pa;       // rmsnorm: residual stream x [M][lda]; silu_mul: fused gate|up [M][lda], lda >= 2 K
  const void* pb;       // rmsnorm: delta added to x first (may be NULL)
  const void* pc;       // rmsnorm: norm weight [K]
  void* resid_out;      // rmsnorm: x + delta is stored here by the first CTA (may be NULL; must not alias x)
  int64_t lda;
  float eps;
  // row-parallel layer of a tensor-parallel model: the ranks' partial outputs are added inside the epilogue (peer.cuh)
  PeerCtx peer;
};

// ---- mbarrier / bulk-copy primitives -----------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and records the failure in the status word) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, int* status, uint32_t limit) {
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_test(bar, parity)) return true;
  if (status) atomicExch(status, PARE_ERR_TIMEOUT);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status) {
  return mbar_wait_limit(bar, parity, status, kSpinLimit);
}
// contiguous global -> shared copy of `bytes` (multiple of 16, both addresses 16-byte aligned)
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// explicit shared-space accesses through 32-bit shared addresses
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds_v4f(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts_v4(uint32_t a, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_v4f(uint32_t a, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1,%2,%3,%4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

// D = A * B (accumulator starts at zero: no register initialisation, no dependency on a previous value)
template <typename T>
__device__ __forceinline__ void mma16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816_zero<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                      uint32_t b0, uint32_t b1) {
  const float z = 0.f;
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}
template <>
__device__ __forceinline__ void mma16816_zero<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  const float z = 0.f;
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

}  // namespace gemv
}  // namespace pare
