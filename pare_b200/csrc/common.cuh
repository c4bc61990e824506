// Shared device helpers for the sm_100a kernels of libpare_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "pare_b200.h"

namespace pare {

// ---- status helpers (host) -------------------------------------------------
#define PARE_REQUIRE(cond, code) \
  do {                           \
    if (!(cond)) return (code);  \
  } while (0)

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? PARE_OK : PARE_ERR_CUDA; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Streaming multiprocessors of the current device (cached per device; 148 on a B200).  Schedules are sized by it;
// nothing depends on it for correctness.
inline int sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    cached[dev] = v;
  }
  return cached[dev];
}

// cudaFuncSetAttribute(max dynamic shared memory) once per (kernel, device), thread-safe.  Keyed by the kernel's
// address: instantiations of one kernel template share a function-pointer type, so a static per type would not do.
inline bool ensure_smem_attr(const void* kern, int bytes) {
  static std::mutex mu;
  static const void* seen[256][2] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return false;
  const void* tag = reinterpret_cast<const void*>(static_cast<uintptr_t>(dev) + 1);
  std::lock_guard<std::mutex> lock(mu);
  int free_slot = -1;
  for (int i = 0; i < 256; ++i) {
    if (seen[i][0] == kern && seen[i][1] == tag) return true;
    if (seen[i][0] == nullptr) {
      free_slot = i;
      break;
    }
  }
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  if (free_slot >= 0) {
    seen[free_slot][0] = kern;
    seen[free_slot][1] = tag;
  }
  return true;
}

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start
// while its predecessor still runs.  Everything that does not depend on the
// predecessor's output (weight streaming) is issued before pdl_wait(); without the
// attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with the programmatic-stream-serialization attribute (host).
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? PARE_OK : PARE_ERR_CUDA;
}

// ---- streaming 128-bit load: read-only path, no L1 allocation ---------------
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// (a & b) | c in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// ---- warp-level tensor-core step, fp32 accumulate ---------------------------
// D[16x8] += A[16x16] * B[16x8]; used by the streaming kernels only to get exact
// products with fp32 accumulation out of integer-valued 16-bit operands.
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm(  // not volatile: a pure function of its operands, the compiler may schedule around it
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- 4-bit code -> 16-bit float without a conversion instruction ------------
// OR-ing a code into the mantissa of a power of two gives an exact integer-valued
// float.  A 32-bit word holds codes c0..c7 (c_i at bits 4i..4i+3); the four results
// are the pairs (c0,c4) (c1,c5) (c2,c6) (c3,c7).
//
// fp16 (10 mantissa bits, magic 1024.0 = 0x6400): a code at bits 0..3 reads
// 1024 + c, a code at bits 4..7 reads 1024 + 16c.  Pairs 0 and 2 are of the first
// kind, pairs 1 and 3 of the second; the other operand of those products is stored
// pre-divided by 16, so every product is (offset + value * c) with one shift per word.
//
// bf16 (7 mantissa bits, magic 128.0 = 0x4300): only bits 0..3 fit, so each pair
// gets its own shift and reads 128 + c.
template <typename T>
struct Nibbles;

template <>
struct Nibbles<__half> {
  static constexpr float kOffsetLo = 1024.f;   // pairs 0, 2
  static constexpr float kOffsetHi = 1024.f;   // pairs 1, 3 (operand pre-divided by 16 -> 64 per unit)
  static constexpr float kHiPrescale = 1.f / 16.f;
  __device__ static __forceinline__ void unpack(uint32_t w, uint32_t (&p)[4]) {
    const uint32_t t = w >> 8;
    p[0] = and_or(w, 0x000f000fu, 0x64006400u);
    p[1] = and_or(w, 0x00f000f0u, 0x64006400u);
    p[2] = and_or(t, 0x000f000fu, 0x64006400u);
    p[3] = and_or(t, 0x00f000f0u, 0x64006400u);
  }
};

// Exact variant for the attention kernel: the mantissa offset is removed before the product (one
// half2 op per pair), so the accumulator never carries the 1024-per-element offset and nothing
// large has to cancel (logits are exponentiated, so their absolute error matters).  Every
// output is code - CENTER for all four pairs; CENTER = 8 maps the codes to -8..7, which halves
// the magnitude of the products and with it the effect of rounding the other operand to fp16.
template <int CENTER>
__device__ __forceinline__ void unpack_codes_exact(uint32_t w, uint32_t (&p)[4]) {
  const uint32_t t = w >> 8;
  const __half2 off_lo = __float2half2_rn(1024.f + CENTER);        // exact in fp16
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const __half2 off_hi = __float2half2_rn(-(64.f + CENTER));
  uint32_t r0 = and_or(w, 0x000f000fu, 0x64006400u), r1 = and_or(w, 0x00f000f0u, 0x64006400u);
  uint32_t r2 = and_or(t, 0x000f000fu, 0x64006400u), r3 = and_or(t, 0x00f000f0u, 0x64006400u);
  __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&r0), off_lo);
  __half2 h1 = __hfma2(*reinterpret_cast<__half2*>(&r1), sixteenth, off_hi);
  __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&r2), off_lo);
  __half2 h3 = __hfma2(*reinterpret_cast<__half2*>(&r3), sixteenth, off_hi);
  p[0] = *reinterpret_cast<uint32_t*>(&h0);
  p[1] = *reinterpret_cast<uint32_t*>(&h1);
  p[2] = *reinterpret_cast<uint32_t*>(&h2);
  p[3] = *reinterpret_cast<uint32_t*>(&h3);
}

// Same for 2-bit codes: a word holds c0..c15 (c_i at bits 2i); the eight results are the pairs (c_j, c_{j+8}),
// each code - CENTER exactly.
template <int CENTER>
__device__ __forceinline__ void unpack_codes2_exact(uint32_t w, uint32_t (&p)[8]) {
  const __half2 off = __float2half2_rn(1024.f + CENTER);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t r = and_or(w >> (2 * j), 0x00030003u, 0x64006400u);
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), off);
    p[j] = *reinterpret_cast<uint32_t*>(&h);
  }
}

template <>
struct Nibbles<__nv_bfloat16> {
  static constexpr float kOffsetLo = 128.f;
  static constexpr float kOffsetHi = 128.f;
  static constexpr float kHiPrescale = 1.f;
  __device__ static __forceinline__ void unpack(uint32_t w, uint32_t (&p)[4]) {
    p[0] = and_or(w, 0x000f000fu, 0x43004300u);
    p[1] = and_or(w >> 4, 0x000f000fu, 0x43004300u);
    p[2] = and_or(w >> 8, 0x000f000fu, 0x43004300u);
    p[3] = and_or(w >> 12, 0x000f000fu, 0x43004300u);
  }
};

// ---- storage position of a channel in the KIVI key scale / zero rows -----------------------
// Inside every block of 128 channels the rows are stored as [word i = (c>>3)&3][lane quad = (c>>5)&3][c&7]:
// the decode-attention kernel reads, for one code word i, the eight channels of each of the four lanes of a
// quad, and this order puts those four 32-byte pieces next to each other (no shared-memory bank conflicts
// after the row has been bulk-copied as it is).  Head dims that are not a multiple of 128 keep channel order.
__host__ __device__ __forceinline__ int kmeta_pos(int c, int D) {
  if (D & 127) return c;
  return (c & ~127) | (((c >> 3) & 3) << 5) | (((c >> 5) & 3) << 3) | (c & 7);
}

// ---- scalar conversions -----------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace pare
