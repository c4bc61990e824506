// Fused KIVI dequantize + decode attention (one query token per sequence), sm_100a.
//
// The reference reconstructs the whole cache to dense fp32 on every step
// (pare/kv_cache.py:249-250, 315-325) and leaves attention to the caller
// (pare/kv_cache.py:183-186).  This kernel reads the packed cache directly and never
// materialises K or V.  Dequantization is folded into the operands that are small:
//     S[h][t] = sum_c (q[h][c] * ks[g][c]) * code_k[t][c]  +  sum_c q[h][c] * kz[g][c]
//     O[h][c] = sum_t (p[h][t] * vs[t]) * (code_v[t][c] - 8)  +  sum_t p[h][t] * (vz[t] + 8 vs[t])
// so the 4-bit codes go to the warp-level MMA unit as exact integer-valued fp16 (OR-ed into
// the mantissa of 1024.0 and the offset subtracted again, see common.cuh; logits are
// exponentiated, so nothing large is left to cancel in the accumulator) and the
// per-channel / per-token scales multiply the
// query row (once per 32-token group) and the probabilities instead of every cache element.
// The up to 8 query heads that share a KV head sit in the 8 MMA columns, so the cache is read
// once for all of them.
//
// Grid: (splits, kv heads, batch).  Each split owns a chunk of compressed tokens (split-KV
// for long contexts); one extra split owns the full-precision residual window.  Phases of a
// CTA: (A) scores of its chunk into shared memory, (B) softmax statistics and scaled
// probabilities in operand order (warp-shuffle reductions), (C) P.V with the V codes as the
// MMA A operand.  Partial (max, sum, O) go to a workspace; the CTA that arrives last at the
// per-(batch, head) counter merges them in split order and resets the counter.

#include "common.cuh"

namespace pare {
namespace {

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kD = 128;
constexpr int kHeads = 8;
constexpr int kMaxChunk = 1024;
constexpr int kMaxResidual = 512;
constexpr size_t kCounterInts = 16384;
constexpr size_t kCounterBytes = kCounterInts * sizeof(int);
constexpr float kNegBig = -1e30f;

struct AttnParams {
  const void* q;
  int64_t q_sb, q_sh;
  const uint8_t* k_codes;
  const float* k_scale;
  const float* k_zero;
  const uint8_t* v_codes;
  const float* v_scale;
  const float* v_zero;
  const void* res_k;
  const void* res_v;
  int64_t r_sb, r_sh, r_st;
  int n_res;
  void* out;
  int64_t o_sb, o_sh;
  float sm_scale;
  int B, Hq, H, rep, group, cap, n_comp;
  int chunk, n_csplit, n_split;
  int s_stride;  // floats per score row
  int p_stride;  // bytes per probability row
  float* part_o;
  float* part_ml;
  int* counters;
};

__device__ __forceinline__ uint32_t h2_bits(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// (a, b) -> hi = fp16 pair, lo = fp16 pair of the rounding residuals
__device__ __forceinline__ void split_h2(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __half2 h = __floats2half2_rn(a, b);
  const __half2 l = __floats2half2_rn(a - __low2float(h), b - __high2float(h));
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <typename T>
__device__ __forceinline__ uint32_t pair_to_h2(uint32_t raw);
template <>
__device__ __forceinline__ uint32_t pair_to_h2<__half>(uint32_t raw) { return raw; }
template <>
__device__ __forceinline__ uint32_t pair_to_h2<__nv_bfloat16>(uint32_t raw) {
  return h2_bits(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u));
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads) kivi_decode_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * p.H + h;
  const bool is_res = (split >= p.n_csplit);

  float* qf = reinterpret_cast<float*>(smem);                       // [8][128]
  float* S = qf + kHeads * kD;                                      // [8][s_stride]
  unsigned char* P = reinterpret_cast<unsigned char*>(S + kHeads * p.s_stride);  // [8][p_stride] fp16 hi parts
  unsigned char* P2 = P + kHeads * p.p_stride;                                   // [8][p_stride] fp16 lo parts
  float* st_m = reinterpret_cast<float*>(P2 + kHeads * p.p_stride);  // [8]
  float* st_l = st_m + kHeads;
  float* st_c = st_l + kHeads;

  // ---- query rows of this KV head as fp32 (rows >= rep are zero) ----
  {
    const T* qg = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.rep * p.q_sh;
    for (int i = threadIdx.x; i < kHeads * kD; i += kAttnThreads) {
      const int hh = i >> 7, c = i & 127;
      qf[i] = hh < p.rep ? to_float<T>(qg[(int64_t)hh * p.q_sh + c]) : 0.f;
    }
  }
  __syncthreads();

  int valid;   // tokens this CTA attends to
  float o_acc[4] = {0.f, 0.f, 0.f, 0.f};   // phase C result, layout depends on the branch

  if (!is_res) {
    const int chunk_start = split * p.chunk;
    valid = min(p.chunk, p.n_comp - chunk_start);
    const int G = p.group;
    const int ngroups = valid / G;
    const int gbase = chunk_start / G;

    // ================= phase A: scores =================
    for (int gl = warp; gl < ngroups; gl += kAttnWarps) {
      const int tok0 = chunk_start + gl * G;
      // issue the code loads of the whole group first (up to 8 tiles of 16 tokens)
      const uint8_t* krow = p.k_codes + (bh * p.cap + tok0) * 64 + tig * 16;
      const float* ks = p.k_scale + (bh * (p.cap / G) + gbase + gl) * kD + tig * 32;
      const float* kz = p.k_zero + (bh * (p.cap / G) + gbase + gl) * kD + tig * 32;
      // q * scale as a two-term fp16 expansion (hi + lo, ~22 bits): a single fp16 rounding of
      // this operand would move the logits by more than the reference's own fp16 cast of K^
      uint32_t xh[4][4], xl[4][4];
      float bias = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(ks + i * 8));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(ks + i * 8 + 4));
        const float4 z0 = __ldg(reinterpret_cast<const float4*>(kz + i * 8));
        const float4 z1 = __ldg(reinterpret_cast<const float4*>(kz + i * 8 + 4));
        const float4 q0 = *reinterpret_cast<const float4*>(qf + gid * kD + tig * 32 + i * 8);
        const float4 q1 = *reinterpret_cast<const float4*>(qf + gid * kD + tig * 32 + i * 8 + 4);
        bias = fmaf(q0.x, z0.x, bias); bias = fmaf(q0.y, z0.y, bias); bias = fmaf(q0.z, z0.z, bias); bias = fmaf(q0.w, z0.w, bias);
        bias = fmaf(q1.x, z1.x, bias); bias = fmaf(q1.y, z1.y, bias); bias = fmaf(q1.z, z1.z, bias); bias = fmaf(q1.w, z1.w, bias);
        // operand order of one code word: (c0,c4) (c1,c5) (c2,c6) (c3,c7)
        split_h2(q0.x * s0.x, q1.x * s1.x, xh[i][0], xl[i][0]);
        split_h2(q0.y * s0.y, q1.y * s1.y, xh[i][1], xl[i][1]);
        split_h2(q0.z * s0.z, q1.z * s1.z, xh[i][2], xl[i][2]);
        split_h2(q0.w * s0.w, q1.w * s1.w, xh[i][3], xl[i][3]);
      }
      bias += __shfl_xor_sync(0xffffffffu, bias, 1);
      bias += __shfl_xor_sync(0xffffffffu, bias, 2);
      const float c0 = __shfl_sync(0xffffffffu, bias, (tig * 2) * 4);
      const float c1 = __shfl_sync(0xffffffffu, bias, (tig * 2 + 1) * 4);

      for (int tile = 0; tile < G / 16; ++tile) {
        const uint4 wa4 = ld_stream_v4(krow + (size_t)(tile * 16 + gid) * 64);
        const uint4 wb4 = ld_stream_v4(krow + (size_t)(tile * 16 + gid + 8) * 64);
        const uint32_t wa[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
        const uint32_t wb[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
        float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t pa[4], pb[4];
          unpack_codes_exact<0>(wa[i], pa);
          unpack_codes_exact<0>(wb[i], pb);
          mma16816<__half>(d0, pa[0], pb[0], pa[1], pb[1], xh[i][0], xh[i][1]);
          mma16816<__half>(d1, pa[2], pb[2], pa[3], pb[3], xh[i][2], xh[i][3]);
          mma16816<__half>(d0, pa[0], pb[0], pa[1], pb[1], xl[i][0], xl[i][1]);
          mma16816<__half>(d1, pa[2], pb[2], pa[3], pb[3], xl[i][2], xl[i][3]);
        }
        const int tl = gl * G + tile * 16 + gid;
        float* s0 = S + (tig * 2) * p.s_stride + tl;
        float* s1 = S + (tig * 2 + 1) * p.s_stride + tl;
        s0[0] = (d0[0] + d1[0] + c0) * p.sm_scale;
        s1[0] = (d0[1] + d1[1] + c1) * p.sm_scale;
        s0[8] = (d0[2] + d1[2] + c0) * p.sm_scale;
        s1[8] = (d0[3] + d1[3] + c1) * p.sm_scale;
      }
    }
    __syncthreads();

    // ================= phase B: softmax statistics, scaled probabilities =================
    const int nblk = (valid + 127) >> 7;
    if (warp < p.rep) {
      const float* srow = S + warp * p.s_stride;
      float m = kNegBig;
      for (int t = lane; t < valid; t += 32) m = fmaxf(m, srow[t]);
      m = warp_max(m);
      float l = 0.f, z = 0.f;
      unsigned char* prow = P + warp * p.p_stride;
      const float* vs = p.v_scale + bh * p.cap + chunk_start;
      const float* vz = p.v_zero + bh * p.cap + chunk_start;
      for (int t = lane; t < nblk * 128; t += 32) {
        float pv = 0.f;
        if (t < valid) {
          const float e = __expf(srow[t] - m);
          l += e;
          const float sc = __ldg(vs + t);
          z = fmaf(e, fmaf(8.f, sc, __ldg(vz + t)), z);   // value codes are centred at 8 in phase C
          pv = e * sc;
        }
        // operand layout of a 128-token block: [word 0..3][quad 0..3] chunks of 8 halves, slots 0,4,1,5,2,6,3,7
        const int tl = t & 127, pos = tl & 7;
        const int slot = ((pos & 3) << 1) | (pos >> 2);
        // two-term fp16 expansion of p * scale (hi + residual): keeps P.V at fp32-level accuracy
        const int off = (t >> 7) * 256 + ((tl >> 3) & 3) * 64 + (tl >> 5) * 16 + slot * 2;
        const __half hv = __float2half_rn(pv);
        *reinterpret_cast<__half*>(prow + off) = hv;
        *reinterpret_cast<__half*>(prow + kHeads * p.p_stride + off) = __float2half_rn(pv - __half2float(hv));
      }
      l = warp_sum(l);
      z = warp_sum(z);
      if (lane == 0) {
        st_m[warp] = m;
        st_l[warp] = l;
        st_c[warp] = z;
      }
    }
    __syncthreads();

    // ================= phase C: O^T[c][h] = sum_t code_v[t][c] * P'[t][h] =================
    {
      const int row = warp * 16 + gid;  // channel
      const uint8_t* vbase = p.v_codes + ((bh * (p.cap / 128) + (chunk_start >> 7)) * kD + row) * 64 + tig * 16;
      float o0[4] = {0.f, 0.f, 0.f, 0.f}, o1[4] = {0.f, 0.f, 0.f, 0.f};
      uint4 va = ld_stream_v4(vbase), vb = ld_stream_v4(vbase + 8 * 64);
      for (int blk = 0; blk < nblk; ++blk) {
        const uint32_t wa[4] = {va.x, va.y, va.z, va.w};
        const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w};
        if (blk + 1 < nblk) {
          va = ld_stream_v4(vbase + (size_t)(blk + 1) * kD * 64);
          vb = ld_stream_v4(vbase + (size_t)(blk + 1) * kD * 64 + 8 * 64);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 pf = make_uint4(0u, 0u, 0u, 0u), pl = make_uint4(0u, 0u, 0u, 0u);
          if (gid < p.rep) {
            pf = *reinterpret_cast<const uint4*>(P + gid * p.p_stride + blk * 256 + i * 64 + tig * 16);
            pl = *reinterpret_cast<const uint4*>(P2 + gid * p.p_stride + blk * 256 + i * 64 + tig * 16);
          }
          uint32_t pa[4], pb[4];
          unpack_codes_exact<8>(wa[i], pa);
          unpack_codes_exact<8>(wb[i], pb);
          mma16816<__half>(o0, pa[0], pb[0], pa[1], pb[1], pf.x, pf.y);
          mma16816<__half>(o1, pa[2], pb[2], pa[3], pb[3], pf.z, pf.w);
          mma16816<__half>(o0, pa[0], pb[0], pa[1], pb[1], pl.x, pl.y);
          mma16816<__half>(o1, pa[2], pb[2], pa[3], pb[3], pl.z, pl.w);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) o_acc[i] = o0[i] + o1[i];
    }
    // write partial O: lane holds channels (row, row+8) x heads (tig*2, tig*2+1)
    {
      float* po = p.part_o + (bh * p.n_split + split) * (size_t)(kHeads * kD);
      const int row = warp * 16 + gid;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int hh = tig * 2 + (i & 1), c = row + 8 * (i >> 1);
        if (hh < p.rep) __stcg(po + hh * kD + c, o_acc[i] + st_c[hh]);
      }
    }
  } else {
    // ================= residual window: dense fp16/bf16 tokens =================
    valid = p.n_res;
    const T* rk = reinterpret_cast<const T*>(p.res_k) + (int64_t)b * p.r_sb + (int64_t)h * p.r_sh;
    const T* rv = reinterpret_cast<const T*>(p.res_v) + (int64_t)b * p.r_sb + (int64_t)h * p.r_sh;
    for (int tile = warp; tile * 16 < valid; tile += kAttnWarps) {
      const int tA = min(tile * 16 + gid, valid - 1), tB = min(tile * 16 + gid + 8, valid - 1);
      float d0[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = (j * 4 + tig) * 8;
        const uint4 ka = *reinterpret_cast<const uint4*>(rk + (int64_t)tA * p.r_st + c0);
        const uint4 kb = *reinterpret_cast<const uint4*>(rk + (int64_t)tB * p.r_st + c0);
        const float4 q0 = *reinterpret_cast<const float4*>(qf + gid * kD + c0);
        const float4 q1 = *reinterpret_cast<const float4*>(qf + gid * kD + c0 + 4);
        mma16816<__half>(d0, pair_to_h2<T>(ka.x), pair_to_h2<T>(kb.x), pair_to_h2<T>(ka.y), pair_to_h2<T>(kb.y),
                         h2_bits(q0.x, q0.y), h2_bits(q0.z, q0.w));
        mma16816<__half>(d0, pair_to_h2<T>(ka.z), pair_to_h2<T>(kb.z), pair_to_h2<T>(ka.w), pair_to_h2<T>(kb.w),
                         h2_bits(q1.x, q1.y), h2_bits(q1.z, q1.w));
      }
      const int tl = tile * 16 + gid;
      float* s0 = S + (tig * 2) * p.s_stride + tl;
      float* s1 = S + (tig * 2 + 1) * p.s_stride + tl;
      s0[0] = d0[0] * p.sm_scale;
      s1[0] = d0[1] * p.sm_scale;
      s0[8] = d0[2] * p.sm_scale;
      s1[8] = d0[3] * p.sm_scale;
    }
    __syncthreads();
    if (warp < p.rep) {
      float* srow = S + warp * p.s_stride;
      float m = kNegBig;
      for (int t = lane; t < valid; t += 32) m = fmaxf(m, srow[t]);
      m = warp_max(m);
      float l = 0.f;
      for (int t = lane; t < valid; t += 32) {
        const float e = __expf(srow[t] - m);
        srow[t] = e;
        l += e;
      }
      l = warp_sum(l);
      if (lane == 0) {
        st_m[warp] = m;
        st_l[warp] = l;
        st_c[warp] = 0.f;
      }
    }
    __syncthreads();
    // P.V on the CUDA cores: thread = (channel, token half); 8 heads per thread
    {
      const int c = threadIdx.x & 127, half = threadIdx.x >> 7;
      const int t_mid = (valid + 1) >> 1;
      const int tb = half ? t_mid : 0, te = half ? valid : t_mid;
      float acc[kHeads];
#pragma unroll
      for (int hh = 0; hh < kHeads; ++hh) acc[hh] = 0.f;
      for (int t = tb; t < te; ++t) {
        const float v = to_float<T>(rv[(int64_t)t * p.r_st + c]);
#pragma unroll
        for (int hh = 0; hh < kHeads; ++hh) acc[hh] = fmaf(S[hh * p.s_stride + t], v, acc[hh]);
      }
      float* red = reinterpret_cast<float*>(P);  // [8][128], reused
      if (half) {
#pragma unroll
        for (int hh = 0; hh < kHeads; ++hh) red[hh * kD + c] = acc[hh];
      }
      __syncthreads();
      if (!half) {
        float* po = p.part_o + (bh * p.n_split + split) * (size_t)(kHeads * kD);
        for (int hh = 0; hh < p.rep; ++hh) __stcg(po + hh * kD + c, acc[hh] + red[hh * kD + c]);
      }
    }
  }

  if (threadIdx.x < p.rep) {
    float* pm = p.part_ml + (bh * p.n_split + split) * (size_t)(kHeads * 2);
    __stcg(pm + threadIdx.x * 2, st_m[threadIdx.x]);
    __stcg(pm + threadIdx.x * 2 + 1, st_l[threadIdx.x]);
  }

  // ================= merge of the splits by the last CTA of this (batch, head) =================
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counters + bh, 1) == p.n_split - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  T* og = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_sb + (int64_t)h * p.rep * p.o_sh;
  const float* pm = p.part_ml + bh * p.n_split * (size_t)(kHeads * 2);
  const float* po = p.part_o + bh * p.n_split * (size_t)(kHeads * kD);
  for (int i = threadIdx.x; i < p.rep * kD; i += kAttnThreads) {
    const int hh = i >> 7, c = i & 127;
    float M = kNegBig;
    for (int s = 0; s < p.n_split; ++s) M = fmaxf(M, __ldcg(pm + (s * kHeads + hh) * 2));
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < p.n_split; ++s) {
      const float w = __expf(__ldcg(pm + (s * kHeads + hh) * 2) - M);
      L = fmaf(w, __ldcg(pm + (s * kHeads + hh) * 2 + 1), L);
      acc = fmaf(w, __ldcg(po + (size_t)s * (kHeads * kD) + hh * kD + c), acc);
    }
    og[(int64_t)hh * p.o_sh + c] = from_float<T>(acc / L);
  }
  if (threadIdx.x == 0) p.counters[bh] = 0;
}

int g_attn_chunk = 0;

int pick_chunk(int B, int H, int n_comp) {
  if (g_attn_chunk) return g_attn_chunk;
  const long long want = ((long long)n_comp * B * H + 443) / 444;  // ~3 CTAs per SM
  int chunk = (int)((want + 127) / 128 * 128);
  if (chunk < 256) chunk = 256;
  if (chunk > kMaxChunk) chunk = kMaxChunk;
  return chunk;
}

}  // namespace
}  // namespace pare

extern "C" {

size_t pare_kivi_attn_workspace_bytes(int B, int H, int n_comp, int n_res) {
  if (B <= 0 || H <= 0 || n_comp < 0 || n_res < 0) return 0;
  const int chunk = 128;  // smallest chunk any plan uses -> upper bound on the split count
  const size_t n_split = (size_t)(n_comp + chunk - 1) / chunk + 1;
  return pare::kCounterBytes + (size_t)B * H * n_split * (pare::kHeads * pare::kD + pare::kHeads * 2) * sizeof(float);
}

void pare_kivi_attn_set_tuning(int chunk) { pare::g_attn_chunk = chunk; }

int pare_kivi_decode_attn(const void* q, int dtype, int64_t q_stride_b, int64_t q_stride_h, const uint8_t* k_codes,
                          const float* k_scale, const float* k_zero, const uint8_t* v_codes, const float* v_scale,
                          const float* v_zero, int n_comp, const void* res_k, const void* res_v, int64_t res_stride_b,
                          int64_t res_stride_h, int64_t res_stride_t, int n_res, void* out, int64_t out_stride_b,
                          int64_t out_stride_h, float softmax_scale, int B, int Hq, int H, int D, int bits, int group,
                          int cap, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace pare;
  PARE_REQUIRE(B > 0 && Hq > 0 && H > 0 && Hq % H == 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(D == kD && bits == 4, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(Hq / H <= kHeads, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(group == 16 || group == 32 || group == 64 || group == 128, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(dtype == PARE_F16 || dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(n_comp >= 0 && n_res >= 0 && n_comp + n_res > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n_comp % group == 0 && n_comp <= cap && cap % 128 == 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n_res <= kMaxResidual, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(q && out && (n_comp == 0 || (k_codes && k_scale && k_zero && v_codes && v_scale && v_zero)), PARE_ERR_SHAPE);
  PARE_REQUIRE(n_res == 0 || (res_k && res_v), PARE_ERR_SHAPE);
  PARE_REQUIRE((size_t)B * H < kCounterInts, PARE_ERR_UNSUPPORTED);
  if (n_res > 0) {
    PARE_REQUIRE(aligned16(res_k) && aligned16(res_v), PARE_ERR_ALIGN);
    PARE_REQUIRE(res_stride_b % 8 == 0 && res_stride_h % 8 == 0 && res_stride_t % 8 == 0, PARE_ERR_ALIGN);
  }
  if (n_comp > 0) PARE_REQUIRE(aligned16(k_codes) && aligned16(v_codes) && aligned16(k_scale) && aligned16(k_zero), PARE_ERR_ALIGN);

  AttnParams p{};
  p.q = q; p.q_sb = q_stride_b; p.q_sh = q_stride_h;
  p.k_codes = k_codes; p.k_scale = k_scale; p.k_zero = k_zero;
  p.v_codes = v_codes; p.v_scale = v_scale; p.v_zero = v_zero;
  p.res_k = res_k; p.res_v = res_v; p.r_sb = res_stride_b; p.r_sh = res_stride_h; p.r_st = res_stride_t; p.n_res = n_res;
  p.out = out; p.o_sb = out_stride_b; p.o_sh = out_stride_h;
  p.sm_scale = softmax_scale;
  p.B = B; p.Hq = Hq; p.H = H; p.rep = Hq / H; p.group = group; p.cap = cap; p.n_comp = n_comp;
  p.chunk = pick_chunk(B, H, n_comp);
  PARE_REQUIRE(p.chunk % 128 == 0 && p.chunk >= 128 && p.chunk <= kMaxChunk, PARE_ERR_UNSUPPORTED);
  p.n_csplit = (n_comp + p.chunk - 1) / p.chunk;
  p.n_split = p.n_csplit + (n_res > 0 ? 1 : 0);
  const int span = p.chunk > ((n_res + 127) / 128 * 128) ? p.chunk : ((n_res + 127) / 128 * 128);
  p.s_stride = span + 4;
  p.p_stride = (span / 128) * 256 + 64;
  if (p.p_stride * kHeads < (int)(kHeads * kD * sizeof(float))) p.p_stride = kD * sizeof(float);  // residual reduction buffer
  const size_t need = kCounterBytes + (size_t)B * H * p.n_split * (kHeads * kD + kHeads * 2) * sizeof(float);
  PARE_REQUIRE(workspace && workspace_bytes >= need, PARE_ERR_WORKSPACE);
  p.counters = reinterpret_cast<int*>(workspace);
  p.part_o = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + kCounterBytes);
  p.part_ml = p.part_o + (size_t)B * H * p.n_split * kHeads * kD;

  const size_t smem = (size_t)kHeads * kD * sizeof(float) + (size_t)kHeads * p.s_stride * sizeof(float) +
                      2 * (size_t)kHeads * p.p_stride + 3 * kHeads * sizeof(float) + 16;
  const dim3 grid(p.n_split, H, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto launch = [&](auto kern) -> int {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess) return PARE_ERR_CUDA;
    kern<<<grid, kAttnThreads, smem, s>>>(p);
    return launch_status();
  };
  PARE_REQUIRE(smem <= 96 * 1024, PARE_ERR_UNSUPPORTED);
  return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half>) : launch(kivi_decode_attn_kernel<__nv_bfloat16>);
}

}  // extern "C"
