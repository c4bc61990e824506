// Elementwise glue between the two hot kernels of a decode step (RMSNorm with residual add,
// SwiGLU gate).  Not part of the reference library (a caller's model code does these); they
// exist so that a decode stack can be chained and captured in a CUDA graph without leaving
// this library.  Both can write their result directly as prepared activations of the next
// W4A16 linear (prep.cuh), which saves that linear's activation-prep launch.

#include "prep.cuh"

namespace pare {
namespace {

// Each thread keeps its elements in registers (8 per 16-byte vector, up to kVecs vectors), so the
// row is read once and all loads are in flight together; n must be a multiple of 8.  One CTA per row.
constexpr int kNormThreads = 256;
constexpr int kVecs = 8;  // rows up to 256 * 8 * 8 = 16384 elements

template <typename T>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_residual_kernel(const T* __restrict__ x, const T* __restrict__ delta,
                                                                        const T* __restrict__ weight, T* resid_out,
                                                                        T* __restrict__ y, __half* __restrict__ prep_xp,
                                                                        float4* __restrict__ prep_tab, int n, float eps) {
  pdl_launch_dependents();
  const size_t row = (size_t)blockIdx.x * n;
  const int nvec = n >> 3;
  uint4 wv[kVecs];   // the norm weights do not depend on the previous kernel
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    if (j * kNormThreads >= nvec) break;   // block-uniform: no vector of this round is inside the row
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) wv[j] = *reinterpret_cast<const uint4*>(weight + v * 8);
  }
  pdl_wait();
  uint4 xv[kVecs], dv[kVecs];
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    if (j * kNormThreads >= nvec) break;   // block-uniform: no vector of this round is inside the row
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec) {
      xv[j] = *reinterpret_cast<const uint4*>(x + row + v * 8);
      if (delta) dv[j] = *reinterpret_cast<const uint4*>(delta + row + v * 8);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kVecs; ++j) {
    if (j * kNormThreads >= nvec) break;   // block-uniform: no vector of this round is inside the row
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
    if (j * kNormThreads >= nvec) break;   // block-uniform: no vector of this round is inside the row
    const int v = threadIdx.x + j * kNormThreads;
    const bool live = v < nvec;
    float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) {
      const T* we = reinterpret_cast<const T*>(&wv[j]);
      const T* xe = reinterpret_cast<const T*>(&xv[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = to_float<T>(xe[e]) * inv * to_float<T>(we[e]);
      if (y) {
        uint4 ov;
        T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int e = 0; e < 8; ++e) oe[e] = from_float<T>(o[e]);
        *reinterpret_cast<uint4*>(y + row + v * 8) = ov;
      }
    }
    if (prep_xp) {   // n % 128 == 0: the sixteen lanes of a step are live or idle together
      const int st = v >> 4, c = v & 15;
      prep_store_step<T>(o, live, prep_xp + row + st * 128, c, prep_tab + (size_t)st * gemv::kTabCols + blockIdx.x);
    }
  }
}

// thread = 8 columns of one row
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                                                       __half* __restrict__ prep_xp, float4* __restrict__ prep_tab, int n,
                                                       int64_t ld, int vec_ok) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = v * 8 < n;
  float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
    const T* g = gate_up + (size_t)row * ld + v * 8;
    uint4 gv, uv;
    if (vec_ok) {
      gv = *reinterpret_cast<const uint4*>(g);
      uv = *reinterpret_cast<const uint4*>(g + n);
    } else {
      T* ge = reinterpret_cast<T*>(&gv);
      T* ue = reinterpret_cast<T*>(&uv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const bool in = v * 8 + e < n;
        ge[e] = in ? g[e] : from_float<T>(0.f);
        ue[e] = in ? g[n + e] : from_float<T>(0.f);
      }
    }
    const T* ge = reinterpret_cast<const T*>(&gv);
    const T* ue = reinterpret_cast<const T*>(&uv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = to_float<T>(ge[e]);
      o[e] = a / (1.f + __expf(-a)) * to_float<T>(ue[e]);
    }
    if (out) {
      T* dst = out + (size_t)row * n + v * 8;
      if (vec_ok) {
        uint4 ov;
        T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
        for (int e = 0; e < 8; ++e) oe[e] = from_float<T>(o[e]);
        *reinterpret_cast<uint4*>(dst) = ov;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (v * 8 + e < n) dst[e] = from_float<T>(o[e]);
      }
    }
  }
  if (prep_xp) {   // n % 128 == 0
    const int st = v >> 4, c = v & 15;
    prep_store_step<T>(o, live, prep_xp + (size_t)row * n + st * 128, c, prep_tab + (size_t)st * gemv::kTabCols + row);
  }
}

template <typename T>
int rmsnorm_launch(const void* x, const void* delta, const void* weight, void* resid_out, void* y, void* prepared, int rows,
                   int n, float eps, cudaStream_t s) {
  __half* xp = reinterpret_cast<__half*>(prepared);
  float4* tab = prepared ? reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(prepared) + prepared_tab_offset(rows, n)) : nullptr;
  return launch_pdl(rmsnorm_residual_kernel<T>, dim3(rows), dim3(kNormThreads), 0, s, (const T*)x, (const T*)delta,
                    (const T*)weight, (T*)resid_out, (T*)y, xp, tab, n, eps);
}

template <typename T>
int silu_launch(const void* gate_up, void* out, void* prepared, int rows, int n, int64_t ld, cudaStream_t s) {
  __half* xp = reinterpret_cast<__half*>(prepared);
  float4* tab = prepared ? reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(prepared) + prepared_tab_offset(rows, n)) : nullptr;
  const int vec_ok = (n % 8 == 0) && (ld % 8 == 0) && aligned16(gate_up) && (out == nullptr || aligned16(out));
  const int nvec = (n + 7) / 8;
  return launch_pdl(silu_mul_kernel<T>, dim3((nvec + 255) / 256, rows), dim3(256), 0, s, (const T*)gate_up, (T*)out, xp, tab,
                    n, ld, vec_ok);
}

// Rotary embedding of x [B][H][T][D] (element strides sb / sh / st, channels contiguous) into a dense out [B][H][T][D]:
// pairs (i, i + D/2), rows [T][D] = cos[0..D/2) | sin[0..D/2) per token.  Products and sum in fp32, each rounded
// separately (no fused multiply-add), then rounded to T: the arithmetic of the decode-attention kernel's rope8 and of
// an fp32 restatement.  One thread per pair of channels.
template <typename T>
__global__ void rope_kernel(const T* x, int64_t sb, int64_t sh, int64_t st, T* out, const float* rows, int B, int H, int Tn, int D) {
  const int half = D >> 1;
  const int64_t total = (int64_t)B * H * Tn * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int64_t row = idx / half;                 // (b * H + h) * Tn + t
    const int t = (int)(row % Tn);
    const int64_t bh = row / Tn;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const T* src = x + (int64_t)b * sb + (int64_t)h * sh + (int64_t)t * st;
    const float a = to_float<T>(src[i]), bb = to_float<T>(src[i + half]);
    const float co = rows[(int64_t)t * D + i], si = rows[(int64_t)t * D + half + i];
    T* dst = out + row * D;
    dst[i] = from_float<T>(__fsub_rn(__fmul_rn(a, co), __fmul_rn(bb, si)));
    dst[i + half] = from_float<T>(__fadd_rn(__fmul_rn(bb, co), __fmul_rn(a, si)));
  }
}

// The same, eight channel pairs per thread with 16-byte accesses (rows 16-byte aligned, D a multiple of 16).
template <typename T>
__global__ void rope_vec_kernel(const T* x, int64_t sb, int64_t sh, int64_t st, T* out, const float* rows, int B, int H, int Tn, int D) {
  const int half = D >> 1, per_row = half >> 3;
  const int64_t total = (int64_t)B * H * Tn * per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % per_row) * 8;
    const int64_t row = idx / per_row;              // (b * H + h) * Tn + t
    const int t = (int)(row % Tn);
    const int64_t bh = row / Tn;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const T* src = x + (int64_t)b * sb + (int64_t)h * sh + (int64_t)t * st;
    const uint4 ra = *reinterpret_cast<const uint4*>(src + i), rb = *reinterpret_cast<const uint4*>(src + half + i);
    const T* a = reinterpret_cast<const T*>(&ra);
    const T* bb = reinterpret_cast<const T*>(&rb);
    const float* cs = rows + (int64_t)t * D;
    const float4 c0 = *reinterpret_cast<const float4*>(cs + i), c1 = *reinterpret_cast<const float4*>(cs + i + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(cs + half + i), s1 = *reinterpret_cast<const float4*>(cs + half + i + 4);
    const float co[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float si[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint4 oa, ob;
    T* pa = reinterpret_cast<T*>(&oa);
    T* pb = reinterpret_cast<T*>(&ob);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float av = to_float<T>(a[j]), bv = to_float<T>(bb[j]);
      pa[j] = from_float<T>(__fsub_rn(__fmul_rn(av, co[j]), __fmul_rn(bv, si[j])));
      pb[j] = from_float<T>(__fadd_rn(__fmul_rn(bv, co[j]), __fmul_rn(av, si[j])));
    }
    T* dst = out + row * D;
    *reinterpret_cast<uint4*>(dst + i) = oa;
    *reinterpret_cast<uint4*>(dst + half + i) = ob;
  }
}

}  // namespace
}  // namespace pare

extern "C" {

// y = rmsnorm(x + delta) * weight; optionally stores x + delta (the new residual stream).
// x, delta (may be NULL), resid_out (may be NULL, may alias x), y: [rows][n]; weight [n].
// prepared_out (may be NULL; then y must not be): the result as prepared activations of a W4A16 linear with K = n.
int pare_rmsnorm_residual(const void* x, const void* delta, const void* weight, void* resid_out, void* y,
                          void* prepared_out, int rows, int n, float eps, int dtype, void* stream) {
  PARE_REQUIRE(x && weight && (y || prepared_out) && rows > 0 && n > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n % 8 == 0 && n <= pare::kNormThreads * pare::kVecs * 8, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(prepared_out == nullptr || (n % 128 == 0 && rows <= pare::gemv::kTabCols && pare::aligned16(prepared_out)),
               PARE_ERR_UNSUPPORTED);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == PARE_F16) return pare::rmsnorm_launch<__half>(x, delta, weight, resid_out, y, prepared_out, rows, n, eps, s);
  if (dtype == PARE_BF16) return pare::rmsnorm_launch<__nv_bfloat16>(x, delta, weight, resid_out, y, prepared_out, rows, n, eps, s);
  return PARE_ERR_DTYPE;
}

// out[r][i] = silu(gate_up[r][i]) * gate_up[r][n + i]; gate_up rows have leading dimension ld >= 2n.
// prepared_out (may be NULL; then out must not be): the result as prepared activations of a W4A16 linear with K = n.
int pare_silu_mul(const void* gate_up, void* out, void* prepared_out, int rows, int n, int64_t ld, int dtype, void* stream) {
  PARE_REQUIRE(gate_up && (out || prepared_out) && rows > 0 && n > 0 && ld >= 2 * (int64_t)n, PARE_ERR_SHAPE);
  PARE_REQUIRE(prepared_out == nullptr ||
                   (n % 128 == 0 && ld % 8 == 0 && rows <= pare::gemv::kTabCols && pare::aligned16(prepared_out) && pare::aligned16(gate_up)),
               PARE_ERR_UNSUPPORTED);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == PARE_F16) return pare::silu_launch<__half>(gate_up, out, prepared_out, rows, n, ld, s);
  if (dtype == PARE_BF16) return pare::silu_launch<__nv_bfloat16>(gate_up, out, prepared_out, rows, n, ld, s);
  return PARE_ERR_DTYPE;
}

// out [B][H][T][D] (dense) = rotary embedding of x [B][H][T][D] (element strides given, channels contiguous) with one
// row of D floats (cos | sin) per token: the step a model takes between its q|k|v projection and the prompt's
// attention (the reference's callers hand update() keys that are already rotated).
int pare_rope(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_t, void* out, const float* rows, int B, int H,
              int T, int D, int dtype, void* stream) {
  PARE_REQUIRE(x && out && rows && B > 0 && H > 0 && T > 0 && D > 0 && (D % 2) == 0, PARE_ERR_SHAPE);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const bool vec = (D % 16) == 0 && pare::aligned16(x) && pare::aligned16(out) && pare::aligned16(rows) && stride_b % 8 == 0 &&
                   stride_h % 8 == 0 && stride_t % 8 == 0;
  const int64_t total = (int64_t)B * H * T * (vec ? D / 16 : D / 2);
  const unsigned blocks = (unsigned)((total + 255) / 256 < 65535 * 16 ? (total + 255) / 256 : 65535 * 16);
  if (vec) {
    if (dtype == PARE_F16)
      pare::rope_vec_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)x, stride_b, stride_h, stride_t, (__half*)out, rows, B, H, T, D);
    else if (dtype == PARE_BF16)
      pare::rope_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, stride_b, stride_h, stride_t, (__nv_bfloat16*)out, rows, B, H, T, D);
    else
      return PARE_ERR_DTYPE;
    return pare::launch_status();
  }
  if (dtype == PARE_F16)
    pare::rope_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)x, stride_b, stride_h, stride_t, (__half*)out, rows, B, H, T, D);
  else if (dtype == PARE_BF16)
    pare::rope_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, stride_b, stride_h, stride_t, (__nv_bfloat16*)out, rows, B, H, T, D);
  else
    return PARE_ERR_DTYPE;
  return pare::launch_status();
}

}  // extern "C"
