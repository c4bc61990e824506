// Elementwise glue between the two hot kernels of a decode step (RMSNorm with residual add,
// SwiGLU gate).  Not part of the reference library (a caller's model code does these); they
// exist so that a decode stack can be chained and captured in a CUDA graph without leaving
// this library.  One CTA per activation row.

#include "common.cuh"

namespace pare {
namespace {

// Each thread keeps its elements in registers (8 per 16-byte vector, up to kVecs vectors), so the
// row is read once and all loads are in flight together; n must be a multiple of 8.
constexpr int kNormThreads = 256;
constexpr int kVecs = 8;  // rows up to 256 * 8 * 8 = 16384 elements

template <typename T>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_residual_kernel(const T* __restrict__ x, const T* __restrict__ delta,
                                                                        const T* __restrict__ weight, T* resid_out,
                                                                        T* __restrict__ y, int n, float eps) {
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * n;
  const int nvec = n >> 3;
  uint4 xv[kVecs], dv[kVecs];
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      xv[j] = *reinterpret_cast<const uint4*>(x + row + v * 8);
      if (delta) dv[j] = *reinterpret_cast<const uint4*>(delta + row + v * 8);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      T* xe = reinterpret_cast<T*>(&xv[j]);
      const T* de = reinterpret_cast<const T*>(&dv[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float f = to_float<T>(xe[e]);
        if (delta) f += to_float<T>(de[e]);
        xe[e] = from_float<T>(f);            // the residual stream is kept in T
        const float r = to_float<T>(xe[e]);
        ss += r * r;
      }
      if (resid_out) *reinterpret_cast<uint4*>(resid_out + row + v * 8) = xv[j];
    }
  }
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (kNormThreads >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / n + eps);
  }
  __syncthreads();
  const float inv = red[0];
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      const uint4 wv = *reinterpret_cast<const uint4*>(weight + v * 8);
      const T* we = reinterpret_cast<const T*>(&wv);
      const T* xe = reinterpret_cast<const T*>(&xv[j]);
      uint4 ov;
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int e = 0; e < 8; ++e) oe[e] = from_float<T>(to_float<T>(xe[e]) * inv * to_float<T>(we[e]));
      *reinterpret_cast<uint4*>(y + row + v * 8) = ov;
    }
  }
}

template <typename T>
__global__ void silu_mul_kernel(const T* gate_up, T* out, int n, int64_t ld) {
  pdl_wait();
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = to_float<T>(gate_up[(size_t)row * ld + i]);
  const float u = to_float<T>(gate_up[(size_t)row * ld + n + i]);
  out[(size_t)row * n + i] = from_float<T>(g / (1.f + __expf(-g)) * u);
}

}  // namespace
}  // namespace pare

extern "C" {

// y = rmsnorm(x + delta) * weight; optionally stores x + delta (the new residual stream).
// x, delta (may be NULL), resid_out (may be NULL, may alias x), y: [rows][n]; weight [n].
int pare_rmsnorm_residual(const void* x, const void* delta, const void* weight, void* resid_out, void* y, int rows,
                          int n, float eps, int dtype, void* stream) {
  PARE_REQUIRE(x && weight && y && rows > 0 && n > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n % 8 == 0 && n <= pare::kNormThreads * pare::kVecs * 8, PARE_ERR_UNSUPPORTED);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == PARE_F16)
    pare::rmsnorm_residual_kernel<__half><<<rows, 256, 0, s>>>((const __half*)x, (const __half*)delta, (const __half*)weight,
                                                               (__half*)resid_out, (__half*)y, n, eps);
  else if (dtype == PARE_BF16)
    pare::rmsnorm_residual_kernel<__nv_bfloat16><<<rows, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)delta,
                                                                      (const __nv_bfloat16*)weight, (__nv_bfloat16*)resid_out,
                                                                      (__nv_bfloat16*)y, n, eps);
  else
    return PARE_ERR_DTYPE;
  return pare::launch_status();
}

// out[r][i] = silu(gate_up[r][i]) * gate_up[r][n + i]; gate_up rows have leading dimension ld >= 2n.
int pare_silu_mul(const void* gate_up, void* out, int rows, int n, int64_t ld, int dtype, void* stream) {
  PARE_REQUIRE(gate_up && out && rows > 0 && n > 0 && ld >= 2 * (int64_t)n, PARE_ERR_SHAPE);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((n + 255) / 256, rows);
  if (dtype == PARE_F16)
    pare::silu_mul_kernel<__half><<<grid, 256, 0, s>>>((const __half*)gate_up, (__half*)out, n, ld);
  else if (dtype == PARE_BF16)
    pare::silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n, ld);
  else
    return PARE_ERR_DTYPE;
  return pare::launch_status();
}

}  // extern "C"
