// KIVI cache maintenance kernels: quantize-on-append and dense dequantize, sm_100a.
//
// Storage of one layer (caller-owned, preallocated for `cap` tokens, cap % 128 == 0):
//   k_codes [B][H][cap][D*bits/8]            codes packed along CHANNELS: channel c of a token
//                                            sits at bit (c*bits) of the token's row (little endian)
//   k_scale, k_zero [B][H][cap/group][D]     fp32 per (group of `group` tokens, channel); channel c at
//                                            position kmeta_pos(c, D) of the row (common.cuh)
//   v_codes [B][H][cap/128][D][128*bits/8]   codes packed along TOKENS inside blocks of 128 tokens:
//                                            token t of the block sits at bit (t*bits) of row d
//   v_scale, v_zero [B][H][cap][D/v_group]   fp32 per (token, group of v_group channels); v_group == D (one per
//                                            token, the reference's form) or 32
// The two code layouts follow the two contractions of attention: q.K^T contracts channels,
// P.V contracts tokens, so each packs along the axis its consumer reads 128 bits at a time.
//
// Arithmetic restates pare/kv_cache.py:75-156 in IEEE fp32 with the same operation order, so
// codes, scales and zeros are bit-identical to the reference:
//   scale = max((max - min) / qmax, 1e-8)          true division
//   code  = rint(min(max((x - min) / scale, 0), qmax))   true division, clamp, then half-to-even
//   x^    = code * scale + min                     separate multiply and add (no FMA contraction)

#include "common.cuh"

namespace pare {
namespace {

struct CachePtrs {
  uint8_t* k_codes;
  float* k_scale;
  float* k_zero;
  uint8_t* v_codes;
  float* v_scale;
  float* v_zero;
  int B, H, D, bits, group, cap;
  int v_group;   // channels that share a value scale / zero: D, or a multiple of 32 that divides D
};

template <typename T>
__device__ __forceinline__ float load_as_float(const void* base, int64_t idx) {
  return to_float<T>(reinterpret_cast<const T*>(base)[idx]);
}

__device__ __forceinline__ uint8_t affine_code(float x, float lo, float scale, float qmax) {
  const float q = fminf(fmaxf(__fdiv_rn(__fsub_rn(x, lo), scale), 0.f), qmax);
  return (uint8_t)rintf(q);
}

// One CTA per (token group, head, batch); blockDim.x == D.
template <typename T>
__global__ void kivi_append_kernel(const void* k_src, const void* v_src, int64_t sb, int64_t sh, int64_t st, int t0,
                                   CachePtrs c) {
  extern __shared__ unsigned char smem[];
  const int G = c.group, D = c.D, bits = c.bits;
  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int d = threadIdx.x, warp = d >> 5, lane = d & 31, nwarps = D >> 5;
  const float qmax = (float)((1 << bits) - 1);
  const int tok0 = t0 + g * G;                      // first destination token of this group
  const int64_t src0 = (int64_t)b * sb + (int64_t)h * sh + (int64_t)g * G * st;
  const size_t bh = (size_t)b * c.H + h;

  uint8_t* codes = smem;                                                   // [G][D]
  const int VG = D / c.v_group;                                            // value groups per token
  float* v_lo = reinterpret_cast<float*>(smem + (size_t)G * D);            // [G][VG]
  float* v_sc = v_lo + G * VG;                                             // [G][VG]

  // ---- keys: per channel over the G tokens of the group ----
  {
    float lo = INFINITY, hi = -INFINITY;
    for (int t = 0; t < G; ++t) {
      const float x = load_as_float<T>(k_src, src0 + (int64_t)t * st + d);
      lo = fminf(lo, x);
      hi = fmaxf(hi, x);
    }
    const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), qmax), 1e-8f);
    const size_t mi = (bh * (c.cap / G) + tok0 / G) * D + kmeta_pos(d, D);
    c.k_scale[mi] = scale;
    c.k_zero[mi] = lo;
    for (int t = 0; t < G; ++t) {
      const float x = load_as_float<T>(k_src, src0 + (int64_t)t * st + d);
      codes[t * D + d] = affine_code(x, lo, scale, qmax);
    }
  }
  __syncthreads();
  {
    // pack along channels: every thread emits whole bytes of the [G][D*bits/8] block
    const int row_bytes = D * bits / 8, per_byte = 8 / bits;
    uint8_t* dst = c.k_codes + (bh * c.cap + tok0) * (size_t)row_bytes;
    for (int i = d; i < G * row_bytes; i += D) {
      const int t = i / row_bytes, j = i - t * row_bytes;
      uint32_t v = 0;
      for (int e = 0; e < per_byte; ++e) v |= (uint32_t)codes[t * D + j * per_byte + e] << (e * bits);
      dst[i] = (uint8_t)v;
    }
  }
  __syncthreads();

  // ---- values: per token over each group of v_group channels (all D of them in the reference's form) ----
  for (int t = warp; t < G; t += nwarps) {
    for (int vg = 0; vg < VG; ++vg) {
      float lo = INFINITY, hi = -INFINITY;
      for (int cc = vg * c.v_group + lane; cc < (vg + 1) * c.v_group; cc += 32) {
        const float x = load_as_float<T>(v_src, src0 + (int64_t)t * st + cc);
        lo = fminf(lo, x);
        hi = fmaxf(hi, x);
      }
      lo = warp_min(lo);
      hi = warp_max(hi);
      const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), qmax), 1e-8f);
      if (lane == 0) {
        v_lo[t * VG + vg] = lo;
        v_sc[t * VG + vg] = scale;
        c.v_scale[(bh * c.cap + tok0 + t) * VG + vg] = scale;
        c.v_zero[(bh * c.cap + tok0 + t) * VG + vg] = lo;
      }
    }
  }
  __syncthreads();
  {
    // pack along tokens: thread d owns row d of the 128-token block(s) this group falls into
    const int row_bytes = 128 * bits / 8, per_byte = 8 / bits;
    for (int tb = 0; tb < G; tb += per_byte) {
      uint32_t v = 0;
      for (int e = 0; e < per_byte; ++e) {
        const int t = tb + e;
        const float x = load_as_float<T>(v_src, src0 + (int64_t)t * st + d);
        v |= (uint32_t)affine_code(x, v_lo[t * VG + d / c.v_group], v_sc[t * VG + d / c.v_group], qmax) << (e * bits);
      }
      const int tok = tok0 + tb;
      uint8_t* row = c.v_codes + ((bh * (c.cap / 128) + tok / 128) * D + d) * (size_t)row_bytes;
      row[(tok % 128) * bits / 8] = (uint8_t)v;
    }
  }
}

// One CTA per (128-token block, head, batch); blockDim.x == D.  Writes tokens [0, n_comp).
template <typename T>
__global__ void kivi_dequant_kernel(CachePtrs c, int n_comp, void* out_k, void* out_v, int64_t ob, int64_t oh, int64_t ot) {
  const int D = c.D, bits = c.bits, G = c.group;
  const int blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
  const size_t bh = (size_t)b * c.H + h;
  const uint32_t mask = (1u << bits) - 1u;
  T* ok = reinterpret_cast<T*>(out_k) + (int64_t)b * ob + (int64_t)h * oh;
  T* ov = reinterpret_cast<T*>(out_v) + (int64_t)b * ob + (int64_t)h * oh;
  const int t_end = min(n_comp, (blk + 1) * 128);
  const int k_row_bytes = D * bits / 8, v_row_bytes = 128 * bits / 8;
  const uint8_t* vrow = c.v_codes + ((bh * (c.cap / 128) + blk) * D + d) * (size_t)v_row_bytes;
  for (int t = blk * 128; t < t_end; ++t) {
    const uint8_t kb = c.k_codes[(bh * c.cap + t) * (size_t)k_row_bytes + (d * bits >> 3)];
    const float kq = (float)((kb >> ((d * bits) & 7)) & mask);
    const size_t mi = (bh * (c.cap / G) + t / G) * D + kmeta_pos(d, D);
    ok[(int64_t)t * ot + d] = from_float<T>(__fadd_rn(__fmul_rn(kq, c.k_scale[mi]), c.k_zero[mi]));
    const int tl = t & 127;
    const uint8_t vb = vrow[tl * bits >> 3];
    const float vq = (float)((vb >> ((tl * bits) & 7)) & mask);
    const size_t vi = (bh * c.cap + t) * (D / c.v_group) + d / c.v_group;
    ov[(int64_t)t * ot + d] = from_float<T>(__fadd_rn(__fmul_rn(vq, c.v_scale[vi]), c.v_zero[vi]));
  }
}

int check_cache(const CachePtrs& c) {
  PARE_REQUIRE(c.B > 0 && c.H > 0 && c.D > 0 && c.cap > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(c.D % 32 == 0 && c.D <= 256, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(c.bits == 2 || c.bits == 4 || c.bits == 8, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(c.group == 16 || c.group == 32 || c.group == 64 || c.group == 128, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(c.cap % 128 == 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(c.v_group > 0 && c.v_group % 32 == 0 && c.D % c.v_group == 0, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(c.k_codes && c.k_scale && c.k_zero && c.v_codes && c.v_scale && c.v_zero, PARE_ERR_SHAPE);
  return PARE_OK;
}

}  // namespace
}  // namespace pare

using pare::CachePtrs;

extern "C" {

int pare_kivi_append(const void* k_src, const void* v_src, int src_dtype, int64_t stride_b, int64_t stride_h,
                     int64_t stride_t, int n_tokens, int t0, uint8_t* k_codes, float* k_scale, float* k_zero,
                     uint8_t* v_codes, float* v_scale, float* v_zero, int B, int H, int D, int bits, int group, int v_group,
                     int cap, void* stream) {
  CachePtrs c{k_codes, k_scale, k_zero, v_codes, v_scale, v_zero, B, H, D, bits, group, cap, v_group > 0 ? v_group : D};
  const int rc = pare::check_cache(c);
  if (rc != PARE_OK) return rc;
  PARE_REQUIRE(k_src && v_src && n_tokens > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n_tokens % group == 0 && t0 >= 0 && t0 % group == 0 && t0 + n_tokens <= cap, PARE_ERR_SHAPE);
  const dim3 grid(n_tokens / group, H, B);
  const size_t smem = (size_t)group * D + 2 * group * (D / c.v_group) * sizeof(float);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (src_dtype) {
    case PARE_F16:
      pare::kivi_append_kernel<__half><<<grid, D, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c);
      break;
    case PARE_BF16:
      pare::kivi_append_kernel<__nv_bfloat16><<<grid, D, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c);
      break;
    case PARE_F32:
      pare::kivi_append_kernel<float><<<grid, D, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c);
      break;
    default:
      return PARE_ERR_DTYPE;
  }
  return pare::launch_status();
}

int pare_kivi_dequant(const uint8_t* k_codes, const float* k_scale, const float* k_zero, const uint8_t* v_codes,
                      const float* v_scale, const float* v_zero, int B, int H, int D, int bits, int group, int v_group,
                      int cap, int n_comp, void* out_k, void* out_v, int out_dtype, int64_t stride_b, int64_t stride_h,
                      int64_t stride_t, void* stream) {
  CachePtrs c{const_cast<uint8_t*>(k_codes), const_cast<float*>(k_scale), const_cast<float*>(k_zero),
              const_cast<uint8_t*>(v_codes), const_cast<float*>(v_scale), const_cast<float*>(v_zero),
              B, H, D, bits, group, cap, v_group > 0 ? v_group : D};
  const int rc = pare::check_cache(c);
  if (rc != PARE_OK) return rc;
  PARE_REQUIRE(out_k && out_v && n_comp >= 0 && n_comp <= cap && n_comp % group == 0, PARE_ERR_SHAPE);
  if (n_comp == 0) return PARE_OK;
  const dim3 grid((n_comp + 127) / 128, H, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case PARE_F16:
      pare::kivi_dequant_kernel<__half><<<grid, D, 0, s>>>(c, n_comp, out_k, out_v, stride_b, stride_h, stride_t);
      break;
    case PARE_BF16:
      pare::kivi_dequant_kernel<__nv_bfloat16><<<grid, D, 0, s>>>(c, n_comp, out_k, out_v, stride_b, stride_h, stride_t);
      break;
    case PARE_F32:
      pare::kivi_dequant_kernel<float><<<grid, D, 0, s>>>(c, n_comp, out_k, out_v, stride_b, stride_h, stride_t);
      break;
    default:
      return PARE_ERR_DTYPE;
  }
  return pare::launch_status();
}

}  // extern "C"
