// Prepared activations of the W4A16 decode kernels, produced in place by whichever kernel
// computes the activation (activation prep, RMSNorm, SwiGLU, attention merge).
//
// Layout of a prepared buffer for M rows of K columns (K % 128 == 0):
//   xp  [M][K]  16-bit, each 128-column step holds its sixteen 8-column chunks at position
//               (c & 3) * 4 + (c >> 2) with the elements of a chunk in slot order 0,4,1,5,2,6,3,7
//               (the order in which one unpacked code word meets its MMA operand); odd code
//               positions carry Nibbles<T>::kHiPrescale
//   tab [K/128][kTabCols] float2 at byte offset prepared_tab_offset(M, K):
//               E  = what the mantissa offsets of the codes add to a step's accumulator,
//               SX = plain sum of the step's activations.
#pragma once

#include "gemv_common.cuh"

namespace pare {

__host__ __device__ inline size_t prepared_tab_offset(int M, int K) { return (((size_t)M * K * 2) + 255) & ~(size_t)255; }
__host__ __device__ inline size_t prepared_bytes(int M, int K) {
  return prepared_tab_offset(M, K) + ((size_t)((K >> 7) + 1) * gemv::kTabCols * sizeof(float2) + 255) / 256 * 256;
}

// One thread holds columns 8c .. 8c+7 of a step (values already divided by any input scale).
// Stores the chunk in operand order and returns this thread's share of the two step sums.
template <typename T>
__device__ __forceinline__ void prep_chunk8(const float (&v)[8], T* step_base, int c, float& lo, float& hi) {
  T b[8];
  lo = 0.f;
  hi = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    // round to the operand type first (the activation the oracle sees), then the exact power-of-two prescale
    const float r = to_float<T>(from_float<T>(v[e]));
    b[e] = from_float<T>((e & 1) ? r * Nibbles<T>::kHiPrescale : r);
    if (e & 1) hi += to_float<T>(b[e]); else lo += to_float<T>(b[e]);
  }
  uint4 out;
  T* o = reinterpret_cast<T*>(&out);
  o[0] = b[0]; o[1] = b[4]; o[2] = b[1]; o[3] = b[5]; o[4] = b[2]; o[5] = b[6]; o[6] = b[3]; o[7] = b[7];
  *reinterpret_cast<uint4*>(step_base + ((c & 3) * 4 + (c >> 2)) * 8) = out;
}

// Sum over the 16 lanes (aligned half warp) that hold one step; every lane of the warp must call.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__device__ __forceinline__ float2 prep_tab_entry(float lo, float hi) {
  return make_float2(Nibbles<T>::kOffsetLo * lo + Nibbles<T>::kOffsetHi * hi, lo + hi / Nibbles<T>::kHiPrescale);
}

}  // namespace pare
