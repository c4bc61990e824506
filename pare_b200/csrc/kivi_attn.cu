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
// for long contexts) or up to 64 tokens of the full-precision residual window.  A CTA first
// puts everything it will read into shared memory with a handful of bulk async copies on one
// mbarrier (codes, scales and zeros of a chunk are contiguous in the cache layout), so the
// phases that follow never wait on global memory: (A) scores of its chunk, (B) softmax
// statistics and scaled probabilities in operand order (warp-shuffle reductions), (C) P.V with
// the V codes as the MMA A operand.  Partial (max, sum, O) go to a workspace; the CTA that
// arrives last at the per-(batch, head) counter merges them in split order and resets the counter.
//
// Launched with programmatic stream serialization: the compressed cache of this step is
// immutable, so its copies are issued before griddepcontrol.wait and overlap the tail of the
// kernel that produces q; the residual window and q are read after the wait.  The newest
// token can be handed in separately (new_k / new_v, e.g. straight out of the q|k|v projection):
// the CTA that owns the last window position attends to it and stores it into the window.
//
// The merged output can also be written as prepared activations of the next W4A16 linear
// (operand order + per-step sums, see prep.cuh): head h is exactly one 128-column step.

#include "gemv_common.cuh"
#include "prep.cuh"

namespace pare {
namespace {

using gemv::bulk_load;
using gemv::kStatusIndex;
using gemv::mbar_expect_tx;
using gemv::mbar_init;
using gemv::mbar_wait;
using gemv::smem_u32;

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kD = 128;
constexpr int kHeads = 8;
constexpr int kMaxVG = 4;        // value scale / zero groups per token at most (32 channels each)
// bytes of shared memory in front of q: mbarrier, flag, statistics [2 + vg][8]
__host__ __device__ constexpr int attn_header(int vg) { return vg == 1 ? 128 : 256; }
constexpr int kMaxChunk = 512;
constexpr int kResChunk = 64;            // residual tokens per split
constexpr int kResPitch = 320;           // bytes per staged residual row (256 + 64: conflict-free 16-byte reads down a column)
constexpr int kMaxResidual = 512;
constexpr size_t kCounterInts = gemv::kCounterInts;
constexpr size_t kCounterBytes = gemv::kCounterBytes;
constexpr size_t kAttnSmemCap = 200 * 1024;
constexpr float kNegBig = -1e30f;
constexpr int kQS = 132;   // floats per staged query row: channel c at (c>>3 & 3)*32 + (c>>5)*8 + (c&7), rows 16 bytes off a bank period
// Rotary position embedding of eight consecutive channels c8 .. c8+7 of a head (pairing i <-> i + D/2): own = the
// channels themselves, other = their partners, cs = cos | sin of the position.  Separately rounded products and
// sum (no fused multiply-add), then rounded to T: what an fp32 restatement computes.
template <typename T>
__device__ __forceinline__ uint4 rope8(const uint4& own, const uint4& other, const float* cs, int c8) {
  const T* a = reinterpret_cast<const T*>(&own);
  const T* b = reinterpret_cast<const T*>(&other);
  const int c = c8 & (kD / 2 - 1);
  const float4 co0 = *reinterpret_cast<const float4*>(cs + c), co1 = *reinterpret_cast<const float4*>(cs + c + 4);
  const float4 si0 = *reinterpret_cast<const float4*>(cs + kD / 2 + c), si1 = *reinterpret_cast<const float4*>(cs + kD / 2 + c + 4);
  const float co[8] = {co0.x, co0.y, co0.z, co0.w, co1.x, co1.y, co1.z, co1.w};
  const float si[8] = {si0.x, si0.y, si0.z, si0.w, si1.x, si1.y, si1.z, si1.w};
  const float sign = c8 < kD / 2 ? -1.f : 1.f;
  uint4 out;
  T* o = reinterpret_cast<T*>(&out);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    o[j] = from_float<T>(__fadd_rn(__fmul_rn(to_float<T>(a[j]), co[j]), sign * __fmul_rn(to_float<T>(b[j]), si[j])));
  return out;
}

__device__ __forceinline__ int q_pos(int c) { return (((c >> 3) & 3) << 5) | ((c >> 5) << 3) | (c & 7); }

struct AttnParams {
  const void* q;
  int64_t q_sb, q_sh;
  int q_vec;           // q rows can be read as 16-byte vectors
  const uint8_t* k_codes;
  const float* k_scale;
  const float* k_zero;
  const uint8_t* v_codes;
  const float* v_scale;
  const float* v_zero;
  void* res_k;
  void* res_v;
  int64_t r_sb, r_sh, r_st;
  int n_res;
  const void* new_k;   // newest token [B][H][D] (may be NULL: the window already holds all n_res tokens)
  const void* new_v;
  const float* rope;    // NULL, or cos[0..D/2) | sin[0..D/2) of the newest token's position: q and new_k are rotated
  int64_t n_sb, n_sh;
  void* out;           // may be NULL when prep_xp is given
  int64_t o_sb, o_sh;
  void* prep_xp;       // prepared activations [B][Hq * 128] + table, or NULL
  float4* prep_tab;
  float sm_scale;
  int B, Hq, H, rep, group, cap, n_comp;
  int vg;        // value scale / zero groups per token (1: one per token; 4: one per 32 channels)
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

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// bytes of the operand stage of a compressed split
__host__ __device__ inline int stage_bytes(int chunk, int group, int bits, int vg) {
  return chunk * (kD * bits / 8) + 2 * (chunk / group) * kD * 4 + (chunk / 128) * kD * (128 * bits / 8) + 2 * chunk * 4 * vg;
}

// codes - CENTER of one word as exact fp16 pairs: four pairs (c_k, c_k+4) at 4 bits, eight pairs (c_j, c_j+8) at 2 bits
template <int BITS, int CENTER>
__device__ __forceinline__ void unpack_exact(uint32_t w, uint32_t (&p)[BITS == 4 ? 4 : 8]) {
  if constexpr (BITS == 4) unpack_codes_exact<CENTER>(w, p);
  else unpack_codes2_exact<CENTER>(w, p);
}

template <typename T, int BITS, int VG>
__global__ void __launch_bounds__(kAttnThreads) kivi_decode_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int NW = BITS == 4 ? 4 : 2;          // code words of the 32 channels / tokens a lane owns
  constexpr int PW = BITS == 4 ? 4 : 8;          // fp16 pairs per word
  constexpr int LB = 4 * BITS;                   // bytes of those 32 codes
  constexpr int KROW = kD * BITS / 8;            // bytes of a token's key codes
  constexpr int VROW = 128 * BITS / 8;           // bytes of a channel's value codes in a 128-token block
  constexpr int VCENTER = BITS == 4 ? 8 : 2;     // value codes are centred (halves the magnitude of the products)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * p.H + h;
  const bool is_res = (split >= p.n_csplit);

  // header: mbarrier, flags, statistics | q fp32 | scores | probabilities (hi, lo) | operand stage
  uint64_t* bar_p = reinterpret_cast<uint64_t*>(smem);
  int* s_last = reinterpret_cast<int*>(smem + 8);
  float* st_m = reinterpret_cast<float*>(smem + 16);                // [8]
  float* st_l = st_m + kHeads;
  float* st_c = st_l + kHeads;                                      // [vg][8]
  float* qf = reinterpret_cast<float*>(smem + attn_header(VG));         // [8][kQS], channels in q_pos order
  float* S = qf + kHeads * kQS;                                     // [8][s_stride]
  // per value group: [8][p_stride] fp16 hi parts, then [8][p_stride] fp16 lo parts
  unsigned char* P = reinterpret_cast<unsigned char*>(S + kHeads * p.s_stride);
  const int pgs = 2 * kHeads * p.p_stride;           // bytes per value group
  unsigned char* stage = P + VG * pgs;             // 128-byte aligned by construction of the strides
  const uint32_t bar = smem_u32(bar_p);
  int* status = p.counters + kStatusIndex;

  int valid;           // tokens this CTA attends to
  int chunk_start = 0;
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();

  // operand stage of a compressed split
  const int ngr_full = p.chunk / p.group;
  unsigned char* kc_s = stage;
  float* ks_s = reinterpret_cast<float*>(kc_s + p.chunk * KROW);
  float* kz_s = ks_s + ngr_full * kD;
  unsigned char* vc_s = reinterpret_cast<unsigned char*>(kz_s + ngr_full * kD);
  float* vs_s = reinterpret_cast<float*>(vc_s + (p.chunk / 128) * kD * VROW);
  float* vz_s = vs_s + p.chunk * VG;               // [token][vg] both

  if (!is_res) {
    chunk_start = split * p.chunk;
    valid = min(p.chunk, p.n_comp - chunk_start);
    if (threadIdx.x == 0) {
      // the compressed cache does not change during a decode step: fetch before the dependency wait
      const int ngroups = valid / p.group, nblk = (valid + 127) >> 7;
      const size_t grow = bh * (p.cap / p.group) + chunk_start / p.group;
      mbar_expect_tx(bar, valid * KROW + 2 * ngroups * kD * 4 + nblk * kD * VROW + 2 * valid * 4 * VG);
      bulk_load(smem_u32(kc_s), p.k_codes + (bh * p.cap + chunk_start) * (size_t)KROW, valid * KROW, bar);
      bulk_load(smem_u32(ks_s), p.k_scale + grow * kD, ngroups * kD * 4, bar);
      bulk_load(smem_u32(kz_s), p.k_zero + grow * kD, ngroups * kD * 4, bar);
      bulk_load(smem_u32(vc_s), p.v_codes + (bh * (p.cap / 128) + (chunk_start >> 7)) * (size_t)(kD * VROW), nblk * kD * VROW, bar);
      bulk_load(smem_u32(vs_s), p.v_scale + (bh * p.cap + chunk_start) * VG, valid * 4 * VG, bar);
      bulk_load(smem_u32(vz_s), p.v_zero + (bh * p.cap + chunk_start) * VG, valid * 4 * VG, bar);
    }
  }
  __syncthreads();   // the barrier is initialised for everybody
  pdl_wait();   // q, the newest token and the residual window may come from the previous kernels

  unsigned char* rk_s = stage;
  unsigned char* rv_s = stage + kResChunk * kResPitch;
  if (is_res) {
    chunk_start = (split - p.n_csplit) * kResChunk;
    valid = min(kResChunk, p.n_res - chunk_start);
    T* rk = reinterpret_cast<T*>(p.res_k) + (int64_t)b * p.r_sb + (int64_t)h * p.r_sh;
    T* rv = reinterpret_cast<T*>(p.res_v) + (int64_t)b * p.r_sb + (int64_t)h * p.r_sh;
    // the newest token, if handed in separately, is the last window position
    const bool has_new = p.new_k != nullptr && chunk_start + valid == p.n_res;
    const int ncopy = has_new ? valid - 1 : valid;
    if (warp == 0) {
      if (lane == 0) mbar_expect_tx(bar, ncopy * 2 * kD * (int)sizeof(T));
      __syncwarp();
      for (int i = lane; i < ncopy; i += 32) {
        bulk_load(smem_u32(rk_s + i * kResPitch), rk + (int64_t)(chunk_start + i) * p.r_st, kD * sizeof(T), bar);
        bulk_load(smem_u32(rv_s + i * kResPitch), rv + (int64_t)(chunk_start + i) * p.r_st, kD * sizeof(T), bar);
      }
    } else if (warp == 1 && has_new) {
      const bool is_v = lane >= 16;
      const int part = lane & 15;   // 16 bytes each
      const T* src = reinterpret_cast<const T*>(is_v ? p.new_v : p.new_k) + (int64_t)b * p.n_sb + (int64_t)h * p.n_sh;
      uint4 val = *reinterpret_cast<const uint4*>(src + part * 8);
      if (p.rope && !is_v) val = rope8<T>(val, *reinterpret_cast<const uint4*>(src + (part ^ 8) * 8), p.rope, part * 8);
      *reinterpret_cast<uint4*>((is_v ? rv_s : rk_s) + (valid - 1) * kResPitch + part * 16) = val;
      *reinterpret_cast<uint4*>((is_v ? rv : rk) + (int64_t)(p.n_res - 1) * p.r_st + part * 8) = val;
    }
  }

  // ---- query rows of this KV head as fp32 (rows >= rep are zero) ----
  {
    const T* qg = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.rep * p.q_sh;
    for (int i = threadIdx.x; i < kHeads * (kD / 8); i += kAttnThreads) {
      const int hh = i >> 4, c8 = (i & 15) * 8;
      float4 lo4 = make_float4(0.f, 0.f, 0.f, 0.f), hi4 = lo4;
      if (hh < p.rep) {
        uint4 raw;
        auto load8 = [&](int c0) {
          uint4 r4;
          if (p.q_vec) {
            r4 = *reinterpret_cast<const uint4*>(qg + (int64_t)hh * p.q_sh + c0);
          } else {
            T* r = reinterpret_cast<T*>(&r4);
#pragma unroll
            for (int j = 0; j < 8; ++j) r[j] = qg[(int64_t)hh * p.q_sh + c0 + j];
          }
          return r4;
        };
        raw = load8(c8);
        if (p.rope) raw = rope8<T>(raw, load8(c8 ^ (kD / 2)), p.rope, c8);
        const T* e = reinterpret_cast<const T*>(&raw);
        lo4 = make_float4(to_float<T>(e[0]), to_float<T>(e[1]), to_float<T>(e[2]), to_float<T>(e[3]));
        hi4 = make_float4(to_float<T>(e[4]), to_float<T>(e[5]), to_float<T>(e[6]), to_float<T>(e[7]));
      }
      *reinterpret_cast<float4*>(qf + hh * kQS + q_pos(c8)) = lo4;
      *reinterpret_cast<float4*>(qf + hh * kQS + q_pos(c8) + 4) = hi4;
    }
  }
  __syncthreads();
  mbar_wait(bar, 0, status);   // bounded; a timeout is reported through the status word

  float o_acc[4] = {0.f, 0.f, 0.f, 0.f};   // phase C result, layout depends on the branch

  if (!is_res) {
    const int G = p.group;
    const int ngroups = valid / G;

    // ================= phase A: scores =================
    // one (group, 16-token tile) item per warp when that occupies no more than the eight warps (short chunks:
    // the per-group operand preparation is repeated, the serial tile loop is cut); else one group per warp
    const int tpg = G / 16;
    const bool split_tiles = ngroups * tpg <= kAttnWarps;
    const int n_items = split_tiles ? ngroups * tpg : ngroups;
    for (int item = warp; item < n_items; item += kAttnWarps) {
      const int gl = split_tiles ? item / tpg : item;
      const int tile_lo = split_tiles ? item - gl * tpg : 0, tile_hi = split_tiles ? tile_lo + 1 : tpg;
      const unsigned char* krow = kc_s + (gl * G) * KROW + tig * LB;
      const float* ks = ks_s + gl * kD + tig * 8;   // rows in kmeta_pos order: channels 8u .. 8u+7 of this lane at u * 32 + tig * 8
      const float* kz = kz_s + gl * kD + tig * 8;
      const float* qrow = qf + gid * kQS + tig * 8;
      // q * scale as a two-term fp16 expansion (hi + lo, ~22 bits): a single fp16 rounding of
      // this operand would move the logits by more than the reference's own fp16 cast of K^.
      // xh / xl[w * PW + j]: the operand pair that meets pair j of code word w.
      uint32_t xh[16], xl[16];
      float bias = 0.f;
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {   // sixteen channels (two runs of eight) at a time
        float pr[2][8];
#pragma unroll
        for (int u2 = 0; u2 < 2; ++u2) {
          const int u = h2 * 2 + u2;
          const float4 s0 = *reinterpret_cast<const float4*>(ks + u * 32);
          const float4 s1 = *reinterpret_cast<const float4*>(ks + u * 32 + 4);
          const float4 z0 = *reinterpret_cast<const float4*>(kz + u * 32);
          const float4 z1 = *reinterpret_cast<const float4*>(kz + u * 32 + 4);
          const float4 q0 = *reinterpret_cast<const float4*>(qrow + u * 32);
          const float4 q1 = *reinterpret_cast<const float4*>(qrow + u * 32 + 4);
          bias = fmaf(q0.x, z0.x, bias); bias = fmaf(q0.y, z0.y, bias); bias = fmaf(q0.z, z0.z, bias); bias = fmaf(q0.w, z0.w, bias);
          bias = fmaf(q1.x, z1.x, bias); bias = fmaf(q1.y, z1.y, bias); bias = fmaf(q1.z, z1.z, bias); bias = fmaf(q1.w, z1.w, bias);
          pr[u2][0] = q0.x * s0.x; pr[u2][1] = q0.y * s0.y; pr[u2][2] = q0.z * s0.z; pr[u2][3] = q0.w * s0.w;
          pr[u2][4] = q1.x * s1.x; pr[u2][5] = q1.y * s1.y; pr[u2][6] = q1.z * s1.z; pr[u2][7] = q1.w * s1.w;
        }
        if constexpr (BITS == 4) {   // a word is one run of eight channels: pairs (c_k, c_k+4)
#pragma unroll
          for (int u2 = 0; u2 < 2; ++u2)
#pragma unroll
            for (int k = 0; k < 4; ++k) split_h2(pr[u2][k], pr[u2][k + 4], xh[(h2 * 2 + u2) * 4 + k], xl[(h2 * 2 + u2) * 4 + k]);
        } else {                      // a word is both runs: pairs (c_j, c_j+8)
#pragma unroll
          for (int j = 0; j < 8; ++j) split_h2(pr[0][j], pr[1][j], xh[h2 * 8 + j], xl[h2 * 8 + j]);
        }
      }
      bias += __shfl_xor_sync(0xffffffffu, bias, 1);
      bias += __shfl_xor_sync(0xffffffffu, bias, 2);
      const float c0 = __shfl_sync(0xffffffffu, bias, (tig * 2) * 4);
      const float c1 = __shfl_sync(0xffffffffu, bias, (tig * 2 + 1) * 4);

      for (int tile = tile_lo; tile < tile_hi; ++tile) {
        uint32_t wa[NW], wb[NW];
        if constexpr (BITS == 4) {
          const uint4 wa4 = *reinterpret_cast<const uint4*>(krow + (tile * 16 + gid) * KROW);
          const uint4 wb4 = *reinterpret_cast<const uint4*>(krow + (tile * 16 + gid + 8) * KROW);
          wa[0] = wa4.x; wa[1] = wa4.y; wa[2] = wa4.z; wa[3] = wa4.w;
          wb[0] = wb4.x; wb[1] = wb4.y; wb[2] = wb4.z; wb[3] = wb4.w;
        } else {
          const uint2 wa2 = *reinterpret_cast<const uint2*>(krow + (tile * 16 + gid) * KROW);
          const uint2 wb2 = *reinterpret_cast<const uint2*>(krow + (tile * 16 + gid + 8) * KROW);
          wa[0] = wa2.x; wa[1] = wa2.y;
          wb[0] = wb2.x; wb[1] = wb2.y;
        }
        float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          uint32_t pa[PW], pb[PW];
          unpack_exact<BITS, 0>(wa[w], pa);
          unpack_exact<BITS, 0>(wb[w], pb);
#pragma unroll
          for (int q4 = 0; q4 < PW / 4; ++q4) {
            const int x0 = w * PW + q4 * 4;
            mma16816<__half>(d0, pa[q4 * 4], pb[q4 * 4], pa[q4 * 4 + 1], pb[q4 * 4 + 1], xh[x0], xh[x0 + 1]);
            mma16816<__half>(d1, pa[q4 * 4 + 2], pb[q4 * 4 + 2], pa[q4 * 4 + 3], pb[q4 * 4 + 3], xh[x0 + 2], xh[x0 + 3]);
            mma16816<__half>(d0, pa[q4 * 4], pb[q4 * 4], pa[q4 * 4 + 1], pb[q4 * 4 + 1], xl[x0], xl[x0 + 1]);
            mma16816<__half>(d1, pa[q4 * 4 + 2], pb[q4 * 4 + 2], pa[q4 * 4 + 3], pb[q4 * 4 + 3], xl[x0 + 2], xl[x0 + 3]);
          }
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
      float l = 0.f, z[VG] = {};
      unsigned char* prow = P + warp * p.p_stride;
      for (int t = lane; t < nblk * 128; t += 32) {
        float e = 0.f;
        if (t < valid) {
          e = __expf(srow[t] - m);
          l += e;
        }
        // operand layout of a 128-token block: [4 operand quads][lane quad 0..3] chunks of 8 halves = four pairs, in the
        // order the pairs of the value code words come out of the unpack (4 bits: (t_k, t_k+4) per 8 tokens; 2 bits:
        // (t_j, t_j+8) per 16 tokens)
        const int tl = t & 127;
        int off;
        if constexpr (BITS == 4) {
          const int pos = tl & 7;
          off = (t >> 7) * 256 + ((tl >> 3) & 3) * 64 + (tl >> 5) * 16 + ((((pos & 3) << 1) | (pos >> 2)) * 2);
        } else {
          const int e = tl & 15, j = e & 7;
          off = (t >> 7) * 256 + ((((tl >> 4) & 1) * 2 + (j >> 2)) * 64) + (tl >> 5) * 16 + (((j & 3) * 2 + (e >> 3)) * 2);
        }
#pragma unroll
        for (int g = 0; g < VG; ++g) {
          {
            float pv = 0.f;
            if (t < valid) {
              const float sc = vs_s[t * VG + g];
              z[g] = fmaf(e, fmaf((float)VCENTER, sc, vz_s[t * VG + g]), z[g]);   // value codes are centred in phase C
              pv = e * sc;
            }
            // two-term fp16 expansion of p * scale (hi + residual): keeps P.V at fp32-level accuracy
            const __half hv = __float2half_rn(pv);
            *reinterpret_cast<__half*>(prow + g * pgs + off) = hv;
            *reinterpret_cast<__half*>(prow + g * pgs + kHeads * p.p_stride + off) = __float2half_rn(pv - __half2float(hv));
          }
        }
      }
      l = warp_sum(l);
#pragma unroll
      for (int g = 0; g < VG; ++g) z[g] = warp_sum(z[g]);
      if (lane == 0) {
        st_m[warp] = m;
        st_l[warp] = l;
#pragma unroll
        for (int g = 0; g < VG; ++g)
          st_c[g * kHeads + warp] = z[g];
      }
    }
    __syncthreads();

    // ================= phase C: O^T[c][h] = sum_t code_v[t][c] * P'[t][h] =================
    {
      const int row = warp * 16 + gid;  // channel
      const unsigned char* Pg = P + ((warp * 16 * VG) / kD) * pgs;   // probabilities scaled for this warp's channel group
      const unsigned char* vbase = vc_s + row * VROW + tig * LB;
      float o0[4] = {0.f, 0.f, 0.f, 0.f}, o1[4] = {0.f, 0.f, 0.f, 0.f};
      for (int blk = 0; blk < nblk; ++blk) {
        uint32_t wa[NW], wb[NW];
        if constexpr (BITS == 4) {
          const uint4 va = *reinterpret_cast<const uint4*>(vbase + blk * (kD * VROW));
          const uint4 vb = *reinterpret_cast<const uint4*>(vbase + blk * (kD * VROW) + 8 * VROW);
          wa[0] = va.x; wa[1] = va.y; wa[2] = va.z; wa[3] = va.w;
          wb[0] = vb.x; wb[1] = vb.y; wb[2] = vb.z; wb[3] = vb.w;
        } else {
          const uint2 va = *reinterpret_cast<const uint2*>(vbase + blk * (kD * VROW));
          const uint2 vb = *reinterpret_cast<const uint2*>(vbase + blk * (kD * VROW) + 8 * VROW);
          wa[0] = va.x; wa[1] = va.y;
          wb[0] = vb.x; wb[1] = vb.y;
        }
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          uint32_t pa[PW], pb[PW];
          unpack_exact<BITS, VCENTER>(wa[w], pa);
          unpack_exact<BITS, VCENTER>(wb[w], pb);
#pragma unroll
          for (int q4 = 0; q4 < PW / 4; ++q4) {
            const int i = w * (PW / 4) + q4;   // operand quad
            uint4 pf = make_uint4(0u, 0u, 0u, 0u), pl = make_uint4(0u, 0u, 0u, 0u);
            if (gid < p.rep) {
              pf = *reinterpret_cast<const uint4*>(Pg + gid * p.p_stride + blk * 256 + i * 64 + tig * 16);
              pl = *reinterpret_cast<const uint4*>(Pg + kHeads * p.p_stride + gid * p.p_stride + blk * 256 + i * 64 + tig * 16);
            }
            mma16816<__half>(o0, pa[q4 * 4], pb[q4 * 4], pa[q4 * 4 + 1], pb[q4 * 4 + 1], pf.x, pf.y);
            mma16816<__half>(o1, pa[q4 * 4 + 2], pb[q4 * 4 + 2], pa[q4 * 4 + 3], pb[q4 * 4 + 3], pf.z, pf.w);
            mma16816<__half>(o0, pa[q4 * 4], pb[q4 * 4], pa[q4 * 4 + 1], pb[q4 * 4 + 1], pl.x, pl.y);
            mma16816<__half>(o1, pa[q4 * 4 + 2], pb[q4 * 4 + 2], pa[q4 * 4 + 3], pb[q4 * 4 + 3], pl.z, pl.w);
          }
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
        if (hh < p.rep) __stcg(po + hh * kD + c, o_acc[i] + st_c[((warp * 16 * VG) / kD) * kHeads + hh]);
      }
    }
  } else {
    // ================= residual window: dense fp16/bf16 tokens from the stage =================
    for (int tile = warp; tile * 16 < valid; tile += kAttnWarps) {
      const int tA = min(tile * 16 + gid, valid - 1), tB = min(tile * 16 + gid + 8, valid - 1);
      float d0[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = (j * 4 + tig) * 8;
        const uint4 ka = *reinterpret_cast<const uint4*>(rk_s + tA * kResPitch + c0 * 2);
        const uint4 kb = *reinterpret_cast<const uint4*>(rk_s + tB * kResPitch + c0 * 2);
        const float4 q0 = *reinterpret_cast<const float4*>(qf + gid * kQS + q_pos(c0));
        const float4 q1 = *reinterpret_cast<const float4*>(qf + gid * kQS + q_pos(c0) + 4);
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
        const float v = to_float<T>(*reinterpret_cast<const T*>(rv_s + t * kResPitch + c * 2));
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
  if (threadIdx.x == 0) *s_last = (atomicAdd(p.counters + bh, 1) == p.n_split - 1);
  __syncthreads();
  if (!*s_last) return;
  __threadfence();
  const float* pm = p.part_ml + bh * p.n_split * (size_t)(kHeads * 2);
  const float* po = p.part_o + bh * p.n_split * (size_t)(kHeads * kD);
  // Everything the merge needs from global memory is requested before anything waits: first the partial outputs
  // of this thread (registers), then the statistics of all splits (shared memory).
  // thread = (split group, head, 8 channels): the groups take contiguous ranges of splits; their partial sums
  // meet in shared memory and are added in group order
  const int rep_pad = p.rep <= 1 ? 1 : (p.rep <= 2 ? 2 : (p.rep <= 4 ? 4 : 8));
  const int pairs = 16 * rep_pad, n_sg = kAttnThreads / pairs;
  const int pair = threadIdx.x % pairs, sg = threadIdx.x / pairs;
  const int mh = pair >> 4, mc = pair & 15;
  const bool head_ok = mh < p.rep;
  const int per = (p.n_split + n_sg - 1) / n_sg;
  const int s_lo = sg * per, s_hi = min(p.n_split, s_lo + per);
  constexpr int kPer = 5;   // splits per thread whose partial outputs are held in registers
  float4 pa0[kPer], pa1[kPer];
  const float* psrc = po + mh * kD + mc * 8;
#pragma unroll
  for (int k = 0; k < kPer; ++k) {
    const int sp = s_lo + k;
    pa0[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    pa1[k] = pa0[k];
    if (head_ok && sp < s_hi) {
      pa0[k] = __ldcg(reinterpret_cast<const float4*>(psrc + (size_t)sp * (kHeads * kD)));
      pa1[k] = __ldcg(reinterpret_cast<const float4*>(psrc + (size_t)sp * (kHeads * kD) + 4));
    }
  }
  float* w_s = reinterpret_cast<float*>(stage);   // [n_split][8]: max, then weight (the operand stage is free by now)
  float* l_s = w_s + p.n_split * kHeads;          // [n_split][8]: sum
  for (int i = threadIdx.x; i < p.n_split * kHeads; i += kAttnThreads) {
    const int hh = i & 7;
    w_s[i] = hh < p.rep ? __ldcg(pm + i * 2) : kNegBig;
    l_s[i] = hh < p.rep ? __ldcg(pm + i * 2 + 1) : 0.f;
  }
  __syncthreads();
  if (warp < p.rep) {   // one warp per head: weights of the splits and their sum
    const int hh = warp;
    float M = kNegBig;
    for (int sp = lane; sp < p.n_split; sp += 32) M = fmaxf(M, w_s[sp * kHeads + hh]);
    M = warp_max(M);
    float L = 0.f;
    for (int sp = lane; sp < p.n_split; sp += 32) {
      const float w = __expf(w_s[sp * kHeads + hh] - M);
      w_s[sp * kHeads + hh] = w;
      L = fmaf(w, l_s[sp * kHeads + hh], L);
    }
    L = warp_sum(L);
    if (lane == 0) st_l[hh] = L;
  }
  __syncthreads();
  {
    const int hh = mh, c = mc;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (head_ok) {
#pragma unroll
      for (int k = 0; k < kPer; ++k) {
        const int sp = s_lo + k;
        const float w = sp < s_hi ? w_s[sp * kHeads + hh] : 0.f;
        acc[0] = fmaf(w, pa0[k].x, acc[0]); acc[1] = fmaf(w, pa0[k].y, acc[1]); acc[2] = fmaf(w, pa0[k].z, acc[2]); acc[3] = fmaf(w, pa0[k].w, acc[3]);
        acc[4] = fmaf(w, pa1[k].x, acc[4]); acc[5] = fmaf(w, pa1[k].y, acc[5]); acc[6] = fmaf(w, pa1[k].z, acc[6]); acc[7] = fmaf(w, pa1[k].w, acc[7]);
      }
#pragma unroll 4
      for (int sp = s_lo + kPer; sp < s_hi; ++sp) {   // long contexts: the rest in batches of four
        const float w = w_s[sp * kHeads + hh];
        const float4 a0 = __ldcg(reinterpret_cast<const float4*>(psrc + (size_t)sp * (kHeads * kD)));
        const float4 a1 = __ldcg(reinterpret_cast<const float4*>(psrc + (size_t)sp * (kHeads * kD) + 4));
        acc[0] = fmaf(w, a0.x, acc[0]); acc[1] = fmaf(w, a0.y, acc[1]); acc[2] = fmaf(w, a0.z, acc[2]); acc[3] = fmaf(w, a0.w, acc[3]);
        acc[4] = fmaf(w, a1.x, acc[4]); acc[5] = fmaf(w, a1.y, acc[5]); acc[6] = fmaf(w, a1.z, acc[6]); acc[7] = fmaf(w, a1.w, acc[7]);
      }
    }
    float* red = reinterpret_cast<float*>(stage + 16384);   // [n_sg][pairs][8], 8 KB
    if (sg > 0) {
      *reinterpret_cast<float4*>(red + (sg * pairs + pair) * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(red + (sg * pairs + pair) * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    __syncthreads();
    const bool active = head_ok && sg == 0;
    if (active) {
      for (int g2 = 1; g2 < n_sg; ++g2) {
        const float4 a0 = *reinterpret_cast<const float4*>(red + (g2 * pairs + pair) * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(red + (g2 * pairs + pair) * 8 + 4);
        acc[0] += a0.x; acc[1] += a0.y; acc[2] += a0.z; acc[3] += a0.w;
        acc[4] += a1.x; acc[5] += a1.y; acc[6] += a1.z; acc[7] += a1.w;
      }
      const float L = st_l[hh];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = acc[e] / L;
    }
    if (active && p.out) {
      T* og = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_sb + (int64_t)(h * p.rep + hh) * p.o_sh + c * 8;
      uint4 ov;
      T* oe = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int e = 0; e < 8; ++e) oe[e] = from_float<T>(acc[e]);
      if (p.o_sh % 8 == 0 && p.o_sb % 8 == 0 && aligned16_dev(p.out)) {
        *reinterpret_cast<uint4*>(og) = ov;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) og[e] = oe[e];
      }
    }
    if (p.prep_xp) {
      // query head (h * rep + hh) is step (h * rep + hh) of activation row b of the next linear
      const int K = p.Hq * kD, st = h * p.rep + hh;
      prep_store_step<T>(acc, active, reinterpret_cast<__half*>(p.prep_xp) + (size_t)b * K + st * kD, c,
                         p.prep_tab + (size_t)st * gemv::kTabCols + b);
    }
  }
  if (threadIdx.x == 0) p.counters[bh] = 0;
}

int pick_chunk(int B, int H, int n_comp, int group) {
  int chunk;
  {
    // 256 tokens per CTA: every warp has a 32-token group to score, three CTAs stay resident per SM (what overlaps
    // one CTA's copies with another's arithmetic once the grid is larger than the machine), and the merge of
    // a 4096-token context reads each split's partial output in one round trip
    chunk = n_comp <= 128 ? 128 : 256;
    // a grid that does not even fill the machine is all latency: longer chunks mean fewer splits to merge
    // (measured at batch 1, 4096 tokens: 11.6 us with 512-token chunks, 12.9 us with 256)
    if ((long long)B * H * ((n_comp + 255) / 256) <= sm_count() && n_comp > 256) chunk = 512;
    while (chunk < kMaxChunk && (n_comp + chunk - 1) / chunk > 96) chunk += 128;   // bound the merge
  }
  if (chunk % group) chunk = (chunk + group - 1) / group * group;
  return chunk;
}

struct AttnPlan {
  int chunk, n_csplit, n_rsplit, n_split, s_stride, p_stride;
  size_t smem;
};

AttnPlan make_attn_plan(int B, int H, int n_comp, int n_res, int group, int bits, int vg) {
  AttnPlan a;
  a.chunk = pick_chunk(B, H, n_comp, group);
  a.n_csplit = (n_comp + a.chunk - 1) / a.chunk;
  a.n_rsplit = (n_res + kResChunk - 1) / kResChunk;
  a.n_split = a.n_csplit + a.n_rsplit;
  const int span = a.chunk > 128 ? a.chunk : 128;
  a.s_stride = span + 4;
  a.p_stride = (span / 128) * 256 + 64;
  if (a.p_stride < 512) a.p_stride = 512;   // the residual branch reuses the buffer for an [8][128] fp32 reduction
  const int st = stage_bytes(a.chunk, group, bits, vg), rs = 2 * kResChunk * kResPitch;
  a.smem = attn_header(vg) + (size_t)kHeads * kQS * sizeof(float) + (size_t)kHeads * a.s_stride * sizeof(float) +
           2 * (size_t)kHeads * a.p_stride * vg + (size_t)(st > rs ? st : rs);
  return a;
}

}  // namespace
}  // namespace pare

extern "C" {

size_t pare_kivi_attn_workspace_bytes(int B, int H, int n_comp, int n_res) {
  if (B <= 0 || H <= 0 || n_comp < 0 || n_res < 0) return 0;
  // smallest chunk any plan uses -> upper bound on the split count
  const size_t n_split = (size_t)(n_comp + 127) / 128 + (size_t)(n_res + pare::kResChunk - 1) / pare::kResChunk + 1;
  return pare::kCounterBytes + (size_t)B * H * n_split * (pare::kHeads * pare::kD + pare::kHeads * 2) * sizeof(float);
}

int pare_kivi_decode_attn(const void* q, int dtype, int64_t q_stride_b, int64_t q_stride_h, const uint8_t* k_codes,
                          const float* k_scale, const float* k_zero, const uint8_t* v_codes, const float* v_scale,
                          const float* v_zero, int n_comp, void* res_k, void* res_v, int64_t res_stride_b,
                          int64_t res_stride_h, int64_t res_stride_t, int n_res, const void* new_k, const void* new_v,
                          int64_t new_stride_b, int64_t new_stride_h, const float* rope, void* out, int64_t out_stride_b,
                          int64_t out_stride_h, void* prepared_out, float softmax_scale, int B, int Hq, int H, int D,
                          int bits, int group, int v_group, int cap, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace pare;
  PARE_REQUIRE(v_group == 0 || v_group == D || v_group == 32, PARE_ERR_UNSUPPORTED);
  const int vg = (v_group == 0 || v_group == D) ? 1 : D / v_group;
  PARE_REQUIRE(B > 0 && Hq > 0 && H > 0 && Hq % H == 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(D == kD && (bits == 4 || bits == 2), PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(Hq / H <= kHeads, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(group == 16 || group == 32 || group == 64 || group == 128, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(dtype == PARE_F16 || dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(n_comp >= 0 && n_res >= 0 && n_comp + n_res > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n_comp % group == 0 && n_comp <= cap && cap % 128 == 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(n_res <= kMaxResidual, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(q && (out || prepared_out) && (n_comp == 0 || (k_codes && k_scale && k_zero && v_codes && v_scale && v_zero)),
               PARE_ERR_SHAPE);
  PARE_REQUIRE(n_res == 0 || (res_k && res_v), PARE_ERR_SHAPE);
  PARE_REQUIRE((new_k == nullptr) == (new_v == nullptr), PARE_ERR_SHAPE);
  PARE_REQUIRE(new_k == nullptr || n_res > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE((size_t)B * H < kStatusIndex, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(prepared_out == nullptr || B <= gemv::kTabCols, PARE_ERR_UNSUPPORTED);
  if (n_res > 0) {
    PARE_REQUIRE(aligned16(res_k) && aligned16(res_v), PARE_ERR_ALIGN);
    PARE_REQUIRE(res_stride_b % 8 == 0 && res_stride_h % 8 == 0 && res_stride_t % 8 == 0, PARE_ERR_ALIGN);
  }
  if (new_k) {
    PARE_REQUIRE(aligned16(new_k) && aligned16(new_v) && new_stride_b % 8 == 0 && new_stride_h % 8 == 0, PARE_ERR_ALIGN);
  }
  if (prepared_out) PARE_REQUIRE(aligned16(prepared_out), PARE_ERR_ALIGN);
  if (rope) PARE_REQUIRE(aligned16(rope), PARE_ERR_ALIGN);
  if (n_comp > 0)
    PARE_REQUIRE(aligned16(k_codes) && aligned16(v_codes) && aligned16(k_scale) && aligned16(k_zero) && aligned16(v_scale) &&
                     aligned16(v_zero),
                 PARE_ERR_ALIGN);

  const AttnPlan plan = make_attn_plan(B, H, n_comp, n_res, group, bits, vg);
  PARE_REQUIRE(plan.chunk % 128 == 0 && plan.chunk % group == 0 && plan.chunk <= kMaxChunk, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(plan.smem <= kAttnSmemCap && (size_t)plan.n_split * 2 * kHeads * sizeof(float) <= 16384, PARE_ERR_UNSUPPORTED);

  AttnParams p{};
  p.q = q; p.q_sb = q_stride_b; p.q_sh = q_stride_h;
  p.q_vec = aligned16(q) && q_stride_b % 8 == 0 && q_stride_h % 8 == 0;
  p.k_codes = k_codes; p.k_scale = k_scale; p.k_zero = k_zero;
  p.v_codes = v_codes; p.v_scale = v_scale; p.v_zero = v_zero;
  p.res_k = res_k; p.res_v = res_v; p.r_sb = res_stride_b; p.r_sh = res_stride_h; p.r_st = res_stride_t; p.n_res = n_res;
  p.new_k = new_k; p.new_v = new_v; p.n_sb = new_stride_b; p.n_sh = new_stride_h;
  p.rope = rope;
  p.out = out; p.o_sb = out_stride_b; p.o_sh = out_stride_h;
  if (prepared_out) {
    p.prep_xp = prepared_out;
    p.prep_tab = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(prepared_out) + prepared_tab_offset(B, Hq * kD));
  }
  p.sm_scale = softmax_scale;
  p.B = B; p.Hq = Hq; p.H = H; p.rep = Hq / H; p.group = group; p.cap = cap; p.n_comp = n_comp;
  p.vg = vg;
  p.chunk = plan.chunk; p.n_csplit = plan.n_csplit; p.n_split = plan.n_split;
  p.s_stride = plan.s_stride; p.p_stride = plan.p_stride;
  const size_t need = kCounterBytes + (size_t)B * H * p.n_split * (kHeads * kD + kHeads * 2) * sizeof(float);
  PARE_REQUIRE(workspace && workspace_bytes >= need, PARE_ERR_WORKSPACE);
  p.counters = reinterpret_cast<int*>(workspace);
  p.part_o = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + kCounterBytes);
  p.part_ml = p.part_o + (size_t)B * H * p.n_split * kHeads * kD;

  auto launch = [&](auto kern) -> int {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmemCap) != cudaSuccess) return PARE_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_split, H, B);
    cfg.blockDim = dim3(kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = plan.smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, p) == cudaSuccess ? PARE_OK : PARE_ERR_CUDA;
  };
  if (vg == 1) {
    if (bits == 4) return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 4, 1>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 4, 1>);
    return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 2, 1>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 2, 1>);
  }
  if (bits == 4) return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 4, kMaxVG>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 4, kMaxVG>);
  return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 2, kMaxVG>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 2, kMaxVG>);
}

}  // extern "C"
