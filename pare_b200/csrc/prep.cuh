// Prepared activations of the W4A16 decode kernels, produced in place by whichever kernel
// computes the activation (activation prep, RMSNorm, SwiGLU, attention merge).
//
// The streaming kernels multiply integer-valued fp16 codes (1024 + c, see common.cuh) with
// fp16 activations on the warp-level MMA unit whatever the activation dtype is: bf16 has too
// few mantissa bits for the cheap code conversion.  To make the fp16 operand safe for any
// input range, every 128-column step of every activation row carries its own power-of-two
// factor f (its largest magnitude lands in [256, 512)); products and sums are exact in fp32,
// and the step's inverse factor g = 1 / f is applied when the step is folded into the output.
//
// Layout of a prepared buffer for M rows of K columns (K % 128 == 0):
//   xp  [M][K]  fp16, each 128-column step holds its sixteen 8-column chunks at position
//               (c & 3) * 4 + (c >> 2) with the elements of a chunk in slot order 0,4,1,5,2,6,3,7
//               (the order in which one unpacked code word meets its MMA operand); odd code
//               positions are pre-divided by 16 (their codes read 1024 + 16 c)
//   tab [K/128][kTabCols] float4 at byte offset prepared_tab_offset(M, K):
//               E  = what the mantissa offsets of the codes add to a step's accumulator,
//               SX = plain sum of the step's (scaled) activations, g = inverse step factor.
#pragma once

#include "gemv_common.cuh"

namespace pare {

__host__ __device__ inline size_t prepared_tab_offset(int M, int K) { return (((size_t)M * K * 2) + 255) & ~(size_t)255; }
__host__ __device__ inline size_t prepared_bytes(int M, int K) {
  return prepared_tab_offset(M, K) + ((size_t)((K >> 7) + 1) * gemv::kTabCols * sizeof(float4) + 255) / 256 * 256;
}

// Sum / max over the 16 lanes (aligned half warp) that hold one step; every lane of the warp must call.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Warp-collective: the 16 lanes of an aligned half warp hold one 128-column step of one activation
// row, lane c its columns 8c .. 8c+7 (already divided by any input scale).  T is the activation
// dtype: values are rounded to T first (the activation the oracle sees).  Writes the step in operand
// order to step_base[0..127] and, from lane c == 0, its table entry.  Lanes that are not `live`
// (beyond the row) take part in the shuffles only.
template <typename T>
__device__ __forceinline__ void prep_store_step(const float (&v)[8], bool live, __half* step_base, int c, float4* tab_entry) {
  float r[8];
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    r[e] = live ? to_float<T>(from_float<T>(v[e])) : 0.f;
    amax = fmaxf(amax, fabsf(r[e]));
  }
  amax = half_warp_max(amax);
  // f = 2^(8 - floor(log2 amax)), exponent clamped so that f and g = 1 / f stay normal numbers
  const int ex = (__float_as_int(amax) >> 23) & 0xff;
  int fe = 262 - ex;
  fe = fe > 253 ? 253 : fe;
  const float f = ex ? __int_as_float(fe << 23) : 1.f;
  const float g = ex ? __int_as_float((254 - fe) << 23) : 1.f;
  __half b[8];
  float lo = 0.f, hi = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    b[e] = __float2half_rn((e & 1) ? r[e] * f * Nibbles<__half>::kHiPrescale : r[e] * f);   // exact unless it underflows
    if (e & 1) hi += __half2float(b[e]); else lo += __half2float(b[e]);
  }
  if (live) {
    uint4 out;
    __half* o = reinterpret_cast<__half*>(&out);
    o[0] = b[0]; o[1] = b[4]; o[2] = b[1]; o[3] = b[5]; o[4] = b[2]; o[5] = b[6]; o[6] = b[3]; o[7] = b[7];
    *reinterpret_cast<uint4*>(step_base + ((c & 3) * 4 + (c >> 2)) * 8) = out;
  }
  lo = half_warp_sum(lo);
  hi = half_warp_sum(hi);
  if (live && c == 0)
    *tab_entry = make_float4(Nibbles<__half>::kOffsetLo * lo + Nibbles<__half>::kOffsetHi * hi,
                             lo + hi / Nibbles<__half>::kHiPrescale, g, 0.f);
}

}  // namespace pare
