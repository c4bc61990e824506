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

// The same code without a division per element.  The quotient is approximated by a product with the correctly
// rounded reciprocal (error below 2 units in the last place of a number below 16, i.e. < 4e-6) and rounded to the
// nearest integer by adding 1.5 * 2^23 (round-to-nearest-even, like rintf; the integer then sits in the low mantissa
// bits).  Only an approximation within 1e-4 of a rounding boundary could round differently from the exact quotient:
// those elements (about one in ten thousand) take the division.  x >= lo by construction, so only the upper clamp is
// needed.  Bit-identical to affine_code.
__device__ __forceinline__ uint32_t affine_code_fast(float x, float lo, float inv, const float* scale_ptr, float qmax) {
  const float q = fminf(__fmul_rn(__fsub_rn(x, lo), inv), qmax);
  const float r = __fadd_rn(q, 12582912.f);
  const float frac = __fsub_rn(__fsub_rn(r, 12582912.f), q);
  if (fabsf(frac) > 0.4999f) return affine_code(x, lo, *scale_ptr, qmax);
  return __float_as_uint(r) & 0xffu;
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

// Vectorised quantize-on-append for the attention geometry (D == 128, 2- or 4-bit codes, 16-bit source, groups of up
// to 64 tokens, 16-byte aligned source rows): one CTA of 128 threads per (token group, head, batch).  The group's keys
// and values (G x 256 bytes each) come in with 16-byte loads into shared memory and every later pass reads them from
// there; the codes leave as 16-byte vectors -- a token's key codes in runs of 16 bytes, a channel's value codes of
// the group as one piece of its row.  Same arithmetic, in the same order, as the element-wise kernel above.
template <typename T, int BITS, int VG>
__global__ void __launch_bounds__(128) kivi_append128_kernel(const void* k_src, const void* v_src, int64_t sb, int64_t sh, int64_t st,
                                                              int t0, CachePtrs c) {
  constexpr int D = 128;
  extern __shared__ __align__(16) unsigned char sm[];
  const int G = c.group;
  T* kt = reinterpret_cast<T*>(sm);                         // [G][D]
  T* vt = kt + G * D;                                       // [G][D]
  float* ks_s = reinterpret_cast<float*>(vt + G * D);       // [D] scale, channel order
  float* kl_s = ks_s + D;                                   // [D] group minimum
  float* ki_s = kl_s + D;                                   // [D] 1 / scale
  float* vs_s = ki_s + D;                                   // [G][VG]
  float* vl_s = vs_s + G * VG;                              // [G][VG]
  float* vi_s = vl_s + G * VG;                              // [G][VG] 1 / scale
  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float qmax = (float)((1 << BITS) - 1);
  const int tok0 = t0 + g * G;
  const size_t bh = (size_t)b * c.H + h;
  const T* kg = reinterpret_cast<const T*>(k_src) + (int64_t)b * sb + (int64_t)h * sh + (int64_t)g * G * st;
  const T* vg_ = reinterpret_cast<const T*>(v_src) + (int64_t)b * sb + (int64_t)h * sh + (int64_t)g * G * st;
  for (int i = tid; i < G * 16; i += 128) {
    const int t = i >> 4, part = i & 15;
    reinterpret_cast<uint4*>(kt)[i] = __ldg(reinterpret_cast<const uint4*>(kg + (int64_t)t * st) + part);
    reinterpret_cast<uint4*>(vt)[i] = __ldg(reinterpret_cast<const uint4*>(vg_ + (int64_t)t * st) + part);
  }
  __syncthreads();
  // ---- keys: per channel over the G tokens of the group ----
  {
    const int d = tid;
    float lo = INFINITY, hi = -INFINITY;
    for (int t = 0; t < G; ++t) {
      const float x = to_float<T>(kt[t * D + d]);
      lo = fminf(lo, x);
      hi = fmaxf(hi, x);
    }
    const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), qmax), 1e-8f);
    const size_t mi = (bh * (c.cap / G) + tok0 / G) * D + kmeta_pos(d, D);
    c.k_scale[mi] = scale;
    c.k_zero[mi] = lo;
    ks_s[d] = scale;
    kl_s[d] = lo;
    ki_s[d] = __frcp_rn(scale);
  }
  // ---- values: per token over each group of D / VG channels (a warp per token, a lane per four channels) ----
  for (int t = warp; t < G; t += 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(vt + t * D + lane * 4);
    const T* e = reinterpret_cast<const T*>(&raw);
    float lo = fminf(fminf(to_float<T>(e[0]), to_float<T>(e[1])), fminf(to_float<T>(e[2]), to_float<T>(e[3])));
    float hi = fmaxf(fmaxf(to_float<T>(e[0]), to_float<T>(e[1])), fmaxf(to_float<T>(e[2]), to_float<T>(e[3])));
    constexpr int kLanes = 32 / VG;                         // lanes that share a value group
#pragma unroll
    for (int o = kLanes / 2; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if ((lane & (kLanes - 1)) == 0) {
      const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), qmax), 1e-8f);
      vs_s[t * VG + lane / kLanes] = scale;
      vl_s[t * VG + lane / kLanes] = lo;
      vi_s[t * VG + lane / kLanes] = __frcp_rn(scale);
    }
  }
  __syncthreads();
  for (int i = tid; i < G * VG; i += 128) {                 // the group's value scales / zeros: contiguous in the cache
    c.v_scale[(bh * c.cap + tok0) * VG + i] = vs_s[i];
    c.v_zero[(bh * c.cap + tok0) * VG + i] = vl_s[i];
  }
  // ---- key codes: 16 bytes (32 or 64 channels) of one token per step ----
  {
    constexpr int CPI = 128 / BITS;                         // channels per 16 bytes of codes
    constexpr int IPT = D / CPI;                            // such pieces per token
    uint8_t* dst = c.k_codes + (bh * c.cap + tok0) * (size_t)(D * BITS / 8);
    for (int i = tid; i < G * IPT; i += 128) {
      const int t = i / IPT, c0 = (i % IPT) * CPI;
      uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int j = 0; j < CPI; j += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(kt + t * D + c0 + j);
        const T* e = reinterpret_cast<const T*>(&raw);
        const float4 l0 = *reinterpret_cast<const float4*>(kl_s + c0 + j), l1 = *reinterpret_cast<const float4*>(kl_s + c0 + j + 4);
        const float4 i0 = *reinterpret_cast<const float4*>(ki_s + c0 + j), i1 = *reinterpret_cast<const float4*>(ki_s + c0 + j + 4);
        const float lo8[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const float in8[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t code = affine_code_fast(to_float<T>(e[k]), lo8[k], in8[k], ks_s + c0 + j + k, qmax);
          w[((j + k) * BITS) >> 5] |= code << (((j + k) * BITS) & 31);
        }
      }
      *reinterpret_cast<uint4*>(dst + (size_t)i * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  // ---- value codes: thread d packs the group's G tokens of channel d into its row of the 128-token block ----
  {
    const int d = tid, gi = VG == 1 ? 0 : (d >> 5);
    constexpr int TPW = 32 / BITS;                          // tokens per 32-bit word
    uint8_t* row = c.v_codes + ((bh * (c.cap / 128) + tok0 / 128) * D + d) * (size_t)(128 * BITS / 8) + (tok0 % 128) * BITS / 8;
    const int words = G / TPW;
    for (int w0 = 0; w0 < words; w0 += 4) {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
      const int nw = min(4, words - w0);
      for (int wi = 0; wi < nw; ++wi)
#pragma unroll
        for (int k = 0; k < TPW; ++k) {
          const int t = (w0 + wi) * TPW + k;
          w[wi] |= affine_code_fast(to_float<T>(vt[t * D + d]), vl_s[t * VG + gi], vi_s[t * VG + gi], vs_s + t * VG + gi, qmax) << (k * BITS);
        }
      if (nw == 4) *reinterpret_cast<uint4*>(row + w0 * 4) = make_uint4(w[0], w[1], w[2], w[3]);
      else if (nw == 2) *reinterpret_cast<uint2*>(row + w0 * 4) = make_uint2(w[0], w[1]);
      else for (int wi = 0; wi < nw; ++wi) *reinterpret_cast<uint32_t*>(row + (w0 + wi) * 4) = w[wi];
    }
  }
}

// Element-wise form of the dequantize kernel for any supported geometry (head dims other than 128, 8-bit codes):
// one CTA per (128-token block, head, batch); blockDim.x == D.  Writes tokens [0, n_comp).
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

// eight dequantized values (code * scale + zero, separately rounded product and sum) as one 16-byte vector of T,
// or two of them for T = float
template <typename T>
__device__ __forceinline__ void store8(T* dst, const float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 o;
    T* e = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = from_float<T>(v[j]);
    *reinterpret_cast<uint4*>(dst) = o;
  } else {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// Vectorised dequantize for the attention geometry (D == 128, 2- or 4-bit codes, 16-byte aligned output rows): one
// CTA of 256 threads per (128-token block, head, batch).  The block's codes and metadata (about 21 KB) come in with
// 16-byte loads into shared memory; a thread then produces eight consecutive channels of one token at a time --
// the key codes of such a run are one 32-bit (16-bit) word, the value codes one nibble from each of eight channel
// rows -- and stores them as one 16-byte vector, a token's 256 output bytes contiguous across 16 threads.
template <typename T, int BITS, int VG>
__global__ void __launch_bounds__(256) kivi_dequant128_kernel(CachePtrs c, int n_comp, void* out_k, void* out_v, int64_t ob, int64_t oh,
                                                               int64_t ot) {
  constexpr int D = 128, KROW = D * BITS / 8, VROW = 128 * BITS / 8, VPITCH = VROW + 4;   // value rows padded: conflict-free column reads
  extern __shared__ __align__(16) unsigned char sm[];
  const int G = c.group, ngr = 128 / G;
  unsigned char* kc = sm;                                              // [128][KROW]
  unsigned char* vc = kc + 128 * KROW;                                 // [D][VPITCH]
  float* ks = reinterpret_cast<float*>(vc + D * VPITCH);               // [ngr][D] in kmeta_pos order
  float* kz = ks + ngr * D;
  float* vs = kz + ngr * D;                                            // [128][VG]
  float* vz = vs + 128 * VG;
  const int blk = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  const size_t bh = (size_t)b * c.H + h;
  const int t0 = blk * 128, valid = min(128, n_comp - t0);             // a multiple of G
  const int vgroups = valid / G;
  {
    const uint4* src = reinterpret_cast<const uint4*>(c.k_codes + (bh * c.cap + t0) * (size_t)KROW);
    for (int i = tid; i < valid * KROW / 16; i += 256) reinterpret_cast<uint4*>(kc)[i] = __ldg(src + i);
    const uint4* vsrc = reinterpret_cast<const uint4*>(c.v_codes + (bh * (c.cap / 128) + blk) * (size_t)(D * VROW));
    for (int i = tid; i < D * VROW / 16; i += 256) {
      const uint4 v = __ldg(vsrc + i);
      const int row = i / (VROW / 16), part = i % (VROW / 16);
      uint32_t* dst = reinterpret_cast<uint32_t*>(vc + row * VPITCH + part * 16);   // rows are only 4-byte aligned
      dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    const size_t grow = (bh * (c.cap / G) + t0 / G) * D;
    for (int i = tid; i < vgroups * D / 4; i += 256) {
      reinterpret_cast<float4*>(ks)[i] = __ldg(reinterpret_cast<const float4*>(c.k_scale + grow) + i);
      reinterpret_cast<float4*>(kz)[i] = __ldg(reinterpret_cast<const float4*>(c.k_zero + grow) + i);
    }
    const size_t vrow0 = (bh * c.cap + t0) * VG;
    for (int i = tid; i < valid * VG / 4; i += 256) {
      reinterpret_cast<float4*>(vs)[i] = __ldg(reinterpret_cast<const float4*>(c.v_scale + vrow0) + i);
      reinterpret_cast<float4*>(vz)[i] = __ldg(reinterpret_cast<const float4*>(c.v_zero + vrow0) + i);
    }
  }
  __syncthreads();
  T* okp = reinterpret_cast<T*>(out_k) + (int64_t)b * ob + (int64_t)h * oh;
  T* ovp = reinterpret_cast<T*>(out_v) + (int64_t)b * ob + (int64_t)h * oh;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  for (int item = tid; item < valid * 16; item += 256) {   // (token, run of eight channels)
    const int t = item >> 4, r = item & 15, c8 = r * 8;
    // ---- keys: the run's codes are BITS bytes of the token's row ----
    uint32_t kw;
    if constexpr (BITS == 4) kw = *reinterpret_cast<const uint32_t*>(kc + t * KROW + r * 4);
    else kw = *reinterpret_cast<const uint16_t*>(kc + t * KROW + r * 2);
    const int mp = (t / G) * D + kmeta_pos(c8, D);          // the eight channels of a run are adjacent in the stored order
    const float4 s0 = *reinterpret_cast<const float4*>(ks + mp), s1 = *reinterpret_cast<const float4*>(ks + mp + 4);
    const float4 z0 = *reinterpret_cast<const float4*>(kz + mp), z1 = *reinterpret_cast<const float4*>(kz + mp + 4);
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float zv[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
    float kv[8], vv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) kv[j] = __fadd_rn(__fmul_rn((float)((kw >> (j * BITS)) & MASK), sv[j]), zv[j]);
    store8<T>(okp + (int64_t)(t0 + t) * ot + c8, kv);
    // ---- values: one code from each of the run's eight channel rows ----
    const int vgi = VG == 1 ? 0 : (c8 >> 5);
    const float vsc = vs[t * VG + vgi], vzr = vz[t * VG + vgi];
    const int byte = (t * BITS) >> 3, sh = (t * BITS) & 7;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t code = (vc[(c8 + j) * VPITCH + byte] >> sh) & MASK;
      vv[j] = __fadd_rn(__fmul_rn((float)code, vsc), vzr);
    }
    store8<T>(ovp + (int64_t)(t0 + t) * ot + c8, vv);
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
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int vg = D / c.v_group;
  if (D == 128 && (bits == 2 || bits == 4) && (vg == 1 || vg == 4) && group <= 64 && (src_dtype == PARE_F16 || src_dtype == PARE_BF16) &&
      pare::aligned16(k_src) && pare::aligned16(v_src) && stride_b % 8 == 0 && stride_h % 8 == 0 && stride_t % 8 == 0 &&
      pare::aligned16(k_codes) && pare::aligned16(v_codes)) {
    const size_t smem = (size_t)2 * group * 128 * 2 + 3 * 128 * sizeof(float) + 3 * (size_t)group * vg * sizeof(float);
#define PARE_AP(T)                                                                                                                   \
  do {                                                                                                                               \
    if (bits == 4 && vg == 1) pare::kivi_append128_kernel<T, 4, 1><<<grid, 128, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c); \
    else if (bits == 4) pare::kivi_append128_kernel<T, 4, 4><<<grid, 128, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c);       \
    else if (vg == 1) pare::kivi_append128_kernel<T, 2, 1><<<grid, 128, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c);         \
    else pare::kivi_append128_kernel<T, 2, 4><<<grid, 128, smem, s>>>(k_src, v_src, stride_b, stride_h, stride_t, t0, c);                      \
  } while (0)
    if (src_dtype == PARE_F16) PARE_AP(__half);
    else PARE_AP(__nv_bfloat16);
#undef PARE_AP
    return pare::launch_status();
  }
  const size_t smem = (size_t)group * D + 2 * group * (D / c.v_group) * sizeof(float);
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
  const int vg = D / c.v_group;
  const size_t esz = out_dtype == PARE_F32 ? 4 : 2;
  const bool fast = D == 128 && (bits == 2 || bits == 4) && (vg == 1 || vg == 4) && pare::aligned16(out_k) && pare::aligned16(out_v) &&
                    (stride_b * esz) % 16 == 0 && (stride_h * esz) % 16 == 0 && (stride_t * esz) % 16 == 0 &&
                    pare::aligned16(k_codes) && pare::aligned16(v_codes) && pare::aligned16(k_scale) && pare::aligned16(k_zero) &&
                    pare::aligned16(v_scale) && pare::aligned16(v_zero);
  if (fast) {
    const size_t smem = (size_t)128 * (128 * bits / 8) + (size_t)128 * (128 * bits / 8 + 4) + 2 * (size_t)(128 / group) * 128 * 4 +
                        2 * (size_t)128 * vg * 4;
    auto launch = [&](auto kern) -> int {
      if (smem > 48 * 1024 && !pare::ensure_smem_attr(reinterpret_cast<const void*>(kern), 64 * 1024)) return PARE_ERR_CUDA;
      kern<<<grid, 256, smem, s>>>(c, n_comp, out_k, out_v, stride_b, stride_h, stride_t);
      return pare::launch_status();
    };
#define PARE_DQ(T)                                                                                        \
  (bits == 4 ? (vg == 1 ? launch(pare::kivi_dequant128_kernel<T, 4, 1>) : launch(pare::kivi_dequant128_kernel<T, 4, 4>)) \
             : (vg == 1 ? launch(pare::kivi_dequant128_kernel<T, 2, 1>) : launch(pare::kivi_dequant128_kernel<T, 2, 4>)))
    switch (out_dtype) {
      case PARE_F16: return PARE_DQ(__half);
      case PARE_BF16: return PARE_DQ(__nv_bfloat16);
      case PARE_F32: return PARE_DQ(float);
      default: return PARE_ERR_DTYPE;
    }
#undef PARE_DQ
  }
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
