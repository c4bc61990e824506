// Elementwise glue between the two hot kernels of a decode step (RMSNorm with residual add,
// SwiGLU gate).  Not part of the reference library (a caller's model code does these); they
// exist so that a decode stack can be chained and captured in a CUDA graph without leaving
// this library.  One CTA per activation row.

#include "common.cuh"

namespace pare {
namespace {

template <typename T>
__global__ void rmsnorm_residual_kernel(const T* x, const T* delta, const T* weight, T* resid_out, T* y, int n, float eps) {
  pdl_wait();
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * n;
  const T* dr = delta ? delta + (size_t)row * n : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_float<T>(xr[i]) + (dr ? to_float<T>(dr[i]) : 0.f);
    const float r = to_float<T>(from_float<T>(v));  // the residual stream is kept in T
    if (resid_out) resid_out[(size_t)row * n + i] = from_float<T>(v);
    ss += r * r;
  }
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) red[0] = rsqrtf(v / n + eps);
  }
  __syncthreads();
  const float inv = red[0];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    // resid_out may alias x: once it is written, read the sum back instead of adding delta twice
    const float v = resid_out ? to_float<T>(resid_out[(size_t)row * n + i])
                              : to_float<T>(from_float<T>(to_float<T>(xr[i]) + (dr ? to_float<T>(dr[i]) : 0.f)));
    y[(size_t)row * n + i] = from_float<T>(v * inv * to_float<T>(weight[i]));
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
