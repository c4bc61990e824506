// Fused KIVI dequantize + decode attention (one query token per sequence), sm_100a.
//
// The reference reconstructs the whole cache to dense fp32 on every step
// (pare/kv_cache.py:249-250, 315-325) and leaves attention to the caller
// (pare/kv_cache.py:183-186).  This kernel reads the packed cache directly and never
// materialises K or V.  Dequantization is folded into the operands that are small:
//     S[h][t] = sum_c (q[h][c] * ks[g][c]) * code_k[t][c]  +  sum_c q[h][c] * kz[g][c]
//     O[h][c] = sum_t (p[h][t] * vs[t]) * code_v[t][c]     +  sum_t p[h][t] * vz[t]
// so the codes go to the warp-level MMA unit as exact small integers and the per-channel / per-token scales
// multiply the query row (once per token group) and the probabilities instead of every cache element.  The up
// to 8 query heads that share a KV head sit in the 8 MMA columns, so the cache is read once for all of them.
//
// Grid: one CTA per split, compressed splits of all (batch, KV head) pairs first, then the residual splits (they
// are short and fill the gaps of the last wave).  A split is either a run of up to `nb` blocks of 128 compressed
// tokens or up to 64 tokens of the full-precision residual window.
//
// A compressed split is a software pipeline over its blocks, with no CTA-wide barrier inside:
//   * a ring of stages: the six pieces of a block (key codes, key scales, key zeros, value codes, value scales,
//     value zeros) are contiguous in the cache layout and arrive by six bulk async copies on one mbarrier.  The
//     compressed cache is immutable during a decode step, so the first copies start before griddepcontrol.wait
//     and overlap the kernel that produces q.
//   * two teams of four warps; team t takes blocks t, t + 2, ...  Inside a team every warp does both halves of
//     the work on the team's block: scaled-query operand of its token group, scores of its 32 tokens by MMA,
//     block maximum (named barrier of the team), online-softmax rescale, probabilities times the value scale
//     into the team's operand buffer (second named barrier), then O = O * alpha + codes_v^T . P for its 32
//     channels.  The teams never wait for each other, so one team's barrier or dependency stalls are the other
//     one's issue slots.  One lane of the team refills the slot once its four warps have released it.
//   * the two teams' (max, sum, O) are combined in shared memory into the split's partial.
// Key codes enter the MMA as fp16 subnormals (a mask per pair, no offset to remove; the query is pre-multiplied
// by the position factor); value codes as exact centred integers (c - 8 or c - 2), see below why.
// Partial (max, sum, O) of a split go to a workspace; the CTA that arrives last at the per-(batch, head)
// counter (one release/acquire atomic) merges them in split order and resets the counter.
//
// The residual window, q and the newest token are read after the dependency wait: the window rows by plain
// 16-byte loads of all threads, scores and P.V by MMA (transposing matrix loads for V).  The newest token can be
// handed in separately (new_k / new_v, e.g. straight out of the q|k|v projection): the CTA that owns the last
// window position attends to it and stores it into the window.  The merged output can also be written as
// prepared activations of the next W4A16 linear (operand order + per-step sums, see prep.cuh): head h is exactly
// one 128-column step.
//
// Every mbarrier wait is bounded: on expiry the thread records PARE_ERR_TIMEOUT in the workspace
// status word and never waits again; the CTA still reaches every named barrier and returns.

#include <type_traits>

#include "gemv_common.cuh"
#include "prep.cuh"

namespace pare {
namespace {

using gemv::bulk_load;
using gemv::kStatusIndex;
using gemv::mbar_expect_tx;
using gemv::mbar_init;
using gemv::mbar_test;
using gemv::smem_u32;

constexpr int kComputeThreads = 256;     // two teams of four warps
constexpr int kAttnThreads = kComputeThreads;
constexpr int kAttnWarps = 8;            // the residual branch and the merge use all warps alike
constexpr int kD = 128;
constexpr int kHeads = 8;
constexpr int kMaxVG = 4;                // value scale / zero groups per token at most (32 channels each)
constexpr int kBlk = 128;                // compressed tokens per pipeline block
constexpr int kMaxStages = 4;
constexpr int kMaxNb = 64;               // blocks per compressed split the planner chooses at most
constexpr int kMaxSplits = 250;          // splits per (batch, head) the merge takes
constexpr int kResChunk = 64;            // residual tokens per split
constexpr int kResPitch = 320;           // bytes per staged residual row (256 + 64: conflict-free 16-byte reads down a column)
constexpr int kMaxResidual = 512;
constexpr int kPHead = 320;              // bytes per head row of a probability operand buffer (256 + 64)
constexpr size_t kCounterBytes = gemv::kCounterBytes;
constexpr float kNegBig = -1e30f;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kQS = 132;   // floats per staged query row: channel c at (c>>3 & 3)*32 + (c>>5)*8 + (c&7), rows 16 bytes off a bank period
constexpr uint32_t kSpin = 1u << 22;

// ---- shared-memory map (bytes) ----
constexpr int kOffBars = 0;       // data_full[4] data_empty[4]
constexpr int kOffLast = 104;
constexpr int kOffStM = 128;      // [8]
constexpr int kOffStL = 160;      // [8]
constexpr int kOffAlpha = 320;    // [2][8]
constexpr int kOffGmax = 384;     // [2][4][8]
constexpr int kOffFin = 640;      // [8 warps][8 heads][1 + kMaxVG]: sum, constant term per value group
constexpr int kFinStride = 1 + kMaxVG;
constexpr int kOffQ = 2048;       // [8][kQS] fp32
constexpr int kOffP = kOffQ + kHeads * kQS * 4;            // 6272
__host__ __device__ constexpr int p_stage_bytes(int vg) { return vg * 2 * kHeads * kPHead; }   // per stage: [vg][hi, lo][8][kPHead]
__host__ __device__ constexpr int ring_offset(int vg) { return kOffP + 2 * p_stage_bytes(vg); }
constexpr size_t kAttnSmemBudget = 112 * 1024;   // two CTAs per SM

// bytes of one pipeline stage (a block of 128 compressed tokens)
__host__ __device__ inline int stage_bytes(int group, int bits, int vg) {
  return kBlk * (kD * bits / 8) + 2 * (kBlk / group) * kD * 4 + kD * (kBlk * bits / 8) + 2 * kBlk * 4 * vg;
}

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
  int nb;              // blocks of 128 compressed tokens per compressed split
  int stages;          // pipeline stages in shared memory
  int n_csplit, n_split;
  float* part_o;
  float* part_ml;
  int* counters;
};

__device__ __forceinline__ uint32_t h2_bits(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
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

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sts_h(uint32_t addr, __half v) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(*reinterpret_cast<const unsigned short*>(&v)) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// Bounded wait; `dead` is sticky per thread: after one expiry nothing waits any more.
__device__ __forceinline__ void wait_bar(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  if (dead) return;
#pragma unroll 1
  for (uint32_t i = 0; i < kSpin; ++i)
    if (mbar_test(bar, parity)) return;
  dead = true;
  atomicExch(status, PARE_ERR_TIMEOUT);
}

// ---- codes as fp16 subnormals ----
// A code field that lies inside the ten mantissa bits of an fp16 whose exponent bits are zero IS the number
// code * 2^(b - 24) (b = the field's lowest bit): masking alone yields an exact tensor-core operand, with no
// offset to remove.  A 4-bit word gives the pairs (c_k, c_k+4) at b = 0 (k even) or 4 (k odd); a 2-bit word the
// pairs (c_j, c_j+8) at b = 2j (j <= 4) or 2(j - 5) after one shift.  The other operand of position e = k or j is
// pre-multiplied by code_factor(e) = 2^(S - b), so every product carries the same 2^(S - 24) = 1 / kCodeOut.
template <int BITS>
__host__ __device__ constexpr float code_factor(int e) {
  if (BITS == 4) return (e & 1) ? 0.0625f : 1.f;
  const int b = (e & 7) <= 4 ? 2 * (e & 7) : 2 * ((e & 7) - 5);
  return 4.f / (float)(1 << b);
}
template <int BITS>
constexpr float kCodeOut = BITS == 4 ? 16777216.f : 4194304.f;

// The value side keeps offset-free CENTRED codes instead (code - kVCentre, one more half2 operation per pair): its
// other operand, the probabilities, is all positive, so with uncentred codes the tensor-core sum and the fp32 zero
// term would be two large numbers that cancel, and the accumulation error of the former showed up a hundredfold in
// the output (1e-2 instead of 5e-4 against the fp32 restatement at 32768 tokens).  The key side's other operand has
// random signs and no such cancellation.
template <int BITS>
constexpr int kVCentre = BITS == 4 ? 8 : 2;
template <int BITS>
__device__ __forceinline__ void unpack_centred(uint32_t w, uint32_t (&p)[BITS == 4 ? 4 : 8]) {
  if constexpr (BITS == 4) unpack_codes_exact<kVCentre<BITS>>(w, p);
  else unpack_codes2_exact<kVCentre<BITS>>(w, p);
}

template <int BITS>
__device__ __forceinline__ void unpack_sub(uint32_t w, uint32_t (&p)[BITS == 4 ? 4 : 8]) {
  if constexpr (BITS == 4) {
    const uint32_t t = w >> 8;
    p[0] = w & 0x000f000fu; p[1] = w & 0x00f000f0u; p[2] = t & 0x000f000fu; p[3] = t & 0x00f000f0u;
  } else {
    const uint32_t t = w >> 10;
#pragma unroll
    for (int j = 0; j < 5; ++j) p[j] = w & (0x00030003u << (2 * j));
#pragma unroll
    for (int j = 5; j < 8; ++j) p[j] = t & (0x00030003u << (2 * (j - 5)));
  }
}

// two independent fp32 operations per instruction
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%2, %3};\n\tmov.b64 y, {%4, %5};\n\tmul.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 x, y, z;\n\tmov.b64 x, {%2, %3};\n\tmov.b64 y, {%4, %5};\n\tmov.b64 z, {%6, %7};\n\tfma.rn.f32x2 x, x, y, z;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

// byte offset, inside a head row of a probability buffer, of token tl (0..127) of the block: the operand order of the
// value MMA ([4 code words of a lane][4 lanes of a quad: the token's 32-token range, XOR-ed with the head pair so that
// neither the scattered stores nor the 16-byte loads meet bank conflicts][8 halves in pair order])
template <int BITS>
__device__ __forceinline__ int p_offset(int tl, int head) {
  const int chunk = ((tl >> 5) ^ (head >> 1)) & 3;
  if constexpr (BITS == 4) {
    const int pos = tl & 7;
    return ((tl >> 3) & 3) * 64 + chunk * 16 + ((((pos & 3) << 1) | (pos >> 2)) * 2);
  } else {
    const int e = tl & 15, j = e & 7;
    return ((((tl >> 4) & 1) * 2 + (j >> 2)) * 64) + chunk * 16 + (((j & 3) * 2 + (e >> 3)) * 2);
  }
}

// MODE bit 0: the scaled query q * k_scale as a two-term fp16 expansion (hi + rounding residual); bit 1: the same for the
// probabilities times the value scale.  Single terms are the faster, less accurate choice.
template <typename T, int BITS, int VG, int MODE>
__global__ void __launch_bounds__(kAttnThreads, 2) kivi_decode_attn_kernel(const AttnParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr bool K2 = (MODE & 1) != 0, P2 = (MODE & 2) != 0;
  constexpr int NW = BITS == 4 ? 4 : 2;          // code words of the 32 channels / tokens a lane owns
  constexpr int PW = BITS == 4 ? 4 : 8;          // fp16 pairs per word
  constexpr int LB = 4 * BITS;                   // bytes of those 32 codes
  constexpr int KROW = kD * BITS / 8;            // bytes of a token's key codes
  constexpr int VROW = kBlk * BITS / 8;          // bytes of a channel's value codes in a 128-token block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  // Launch order = block index: the long compressed splits of every (batch, head) come first, the short residual
  // splits last, where they fill the gaps of the final wave instead of delaying a compressed split by a wave.
  const int n_rsplit = p.n_split - p.n_csplit;
  const int total_c = p.B * p.H * p.n_csplit;
  const bool is_res = (int)blockIdx.x >= total_c;
  const int pair_idx = is_res ? ((int)blockIdx.x - total_c) / n_rsplit : (int)blockIdx.x / p.n_csplit;
  const int split = is_res ? p.n_csplit + ((int)blockIdx.x - total_c) % n_rsplit : (int)blockIdx.x % p.n_csplit;
  const int b = pair_idx / p.H, h = pair_idx % p.H;
  const size_t bh = (size_t)pair_idx;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
  const uint32_t data_full = smem_u32(bars), data_empty = smem_u32(bars + 4);
  int* s_last = reinterpret_cast<int*>(smem + kOffLast);
  float* st_m = reinterpret_cast<float*>(smem + kOffStM);
  float* st_l = reinterpret_cast<float*>(smem + kOffStL);
  float* alpha_s = reinterpret_cast<float*>(smem + kOffAlpha);  // [2][8]
  float* gmax_s = reinterpret_cast<float*>(smem + kOffGmax);    // [2][4][8]
  float* fin_s = reinterpret_cast<float*>(smem + kOffFin);      // [4][8][kFinStride]
  float* qf = reinterpret_cast<float*>(smem + kOffQ);           // [8][kQS], channels in q_pos order
  unsigned char* Pring = smem + kOffP;
  unsigned char* stage = smem + ring_offset(VG);
  int* status = p.counters + kStatusIndex;
  bool dead = false;

  const int G = p.group;
  const int sbytes = stage_bytes(G, BITS, VG);
  // pieces of a stage
  const int off_ks = kBlk * KROW, off_kz = off_ks + (kBlk / G) * kD * 4, off_vc = off_kz + (kBlk / G) * kD * 4;
  const int off_vs = off_vc + kD * VROW, off_vz = off_vs + kBlk * 4 * VG;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(data_full + i * 8, 1);
      mbar_init(data_empty + i * 8, 4);   // the four warps of the team that owns the block
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  __syncthreads();   // the barriers are initialised for everybody

  // blocks of this compressed split
  const int nblk_total = (p.n_comp + kBlk - 1) / kBlk;
  const int blk0 = split * p.nb;
  const int nblk = is_res ? 0 : min(p.nb, nblk_total - blk0);

  // one block of the compressed cache into its ring slot (six bulk copies on the slot's barrier); issued by one thread
  const int lg = 31 - __clz(G);   // G is a power of two
  auto issue_block = [&](int i, int slot) {
    const int t0 = (blk0 + i) * kBlk;
    const int valid = min(kBlk, p.n_comp - t0), ngroups = valid >> lg;
    const size_t grow = bh * (size_t)(p.cap >> lg) + (t0 >> lg);
    const uint32_t dst = smem_u32(stage + slot * sbytes), bar = data_full + slot * 8;
    mbar_expect_tx(bar, valid * KROW + 2 * ngroups * kD * 4 + kD * VROW + 2 * valid * 4 * VG);
    bulk_load(dst, p.k_codes + (bh * p.cap + t0) * (size_t)KROW, valid * KROW, bar);
    bulk_load(dst + off_ks, p.k_scale + grow * kD, ngroups * kD * 4, bar);
    bulk_load(dst + off_kz, p.k_zero + grow * kD, ngroups * kD * 4, bar);
    bulk_load(dst + off_vc, p.v_codes + (bh * (p.cap / kBlk) + (t0 >> 7)) * (size_t)(kD * VROW), kD * VROW, bar);
    bulk_load(dst + off_vs, p.v_scale + (bh * p.cap + t0) * VG, valid * 4 * VG, bar);
    bulk_load(dst + off_vz, p.v_zero + (bh * p.cap + t0) * VG, valid * 4 * VG, bar);
  };
  // the compressed cache does not change during a decode step, so the first stages are fetched before the dependency wait
  if (warp == kAttnWarps - 1 && lane == 0)
    for (int i = 0; i < nblk && i < p.stages; ++i) issue_block(i, i);

  pdl_wait();   // q, the newest token and the residual window may come from the previous kernels

  unsigned char* rk_s = stage;
  unsigned char* rv_s = stage + kResChunk * kResPitch;
  int valid = 0;           // tokens a residual split attends to
  int chunk_start = 0;
  constexpr int kResLoads = kResChunk * 32 / kComputeThreads;   // 16-byte pieces of the window per thread
  uint4 res_regs[kResLoads];
  int res_total = 0;
  if (is_res) {
    chunk_start = (split - p.n_csplit) * kResChunk;
    valid = min(kResChunk, p.n_res - chunk_start);
    T* rk = reinterpret_cast<T*>(p.res_k) + (int64_t)b * p.r_sb + (int64_t)h * p.r_sh;
    T* rv = reinterpret_cast<T*>(p.res_v) + (int64_t)b * p.r_sb + (int64_t)h * p.r_sh;
    // the newest token, if handed in separately, is the last window position
    const bool has_new = p.new_k != nullptr && chunk_start + valid == p.n_res;
    const int ncopy = has_new ? valid - 1 : valid;
    // the window rows as 16-byte pieces straight into registers (all in flight at once); they are stored to the
    // padded stage after the query rows below have been staged
    {
      const int total = res_total = ncopy * 32;   // 16 pieces of K and 16 of V per token
#pragma unroll
      for (int j = 0; j < kResLoads; ++j) {
        const int idx = threadIdx.x + j * kComputeThreads;
        res_regs[j] = make_uint4(0u, 0u, 0u, 0u);
        if (idx < total) {
          const int row = idx >> 5, part = idx & 31;
          const T* src = (part < 16 ? rk : rv) + (int64_t)(chunk_start + row) * p.r_st + (part & 15) * 8;
          res_regs[j] = __ldcg(reinterpret_cast<const uint4*>(src));
        }
      }
    }
    if (warp == 1 && has_new) {
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
    for (int i = threadIdx.x; i < kHeads * (kD / 8); i += kComputeThreads) {
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
        if (!is_res) {   // the compressed splits multiply q by the factor of its channel's position in a code word
          lo4.x *= code_factor<BITS>(0); lo4.y *= code_factor<BITS>(1); lo4.z *= code_factor<BITS>(2); lo4.w *= code_factor<BITS>(3);
          hi4.x *= code_factor<BITS>(4); hi4.y *= code_factor<BITS>(5); hi4.z *= code_factor<BITS>(6); hi4.w *= code_factor<BITS>(7);
        }
      }
      *reinterpret_cast<float4*>(qf + hh * kQS + q_pos(c8)) = lo4;
      *reinterpret_cast<float4*>(qf + hh * kQS + q_pos(c8) + 4) = hi4;
    }
  }
  if (is_res) {
#pragma unroll
    for (int j = 0; j < kResLoads; ++j) {
      const int idx = threadIdx.x + j * kComputeThreads;
      if (idx < res_total) {
        const int row = idx >> 5, part = idx & 31;
        *reinterpret_cast<uint4*>((part < 16 ? rk_s : rv_s) + row * kResPitch + (part & 15) * 16) = res_regs[j];
      }
    }
  }
  named_sync(1, kComputeThreads);

  if (!is_res) {
    // ================= compressed split: two teams of four warps, team t takes blocks t, t + 2, ... =================
    // Inside a team every warp plays both parts on the team's current block: scores and probabilities of its 32 tokens,
    // then O += codes_v^T . P for its 32 channels; two named barriers per block order the team's probability buffer.
    // The teams never wait for each other: while one is in a barrier or a dependency stall the other one issues.
    const float scale2 = p.sm_scale * kLog2e;   // scores in base-2 units: p = exp2(s2 - m2)
    const float scale2o = scale2 * kCodeOut<BITS>;   // the code products carry 1 / kCodeOut
    const int team = warp >> 2, tw = warp & 3;
    const int team_bar = 2 + team;
    const float* qrow = qf + gid * kQS + tig * 8;   // this lane's query row (head gid, channels 32 tig .. + 31 in runs of eight)
    unsigned char* pst = Pring + team * p_stage_bytes(VG);   // the team's probability buffer
    float* gm = gmax_s + team * (4 * kHeads);
    // where this lane's four (tile, row half) tokens go in a probability row, per head of its pair
    uint32_t paddr[2][2][2];   // shared-memory addresses
#pragma unroll
    for (int tile = 0; tile < 2; ++tile)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tl = 32 * tw + 16 * tile + gid + 8 * hf, head = 2 * tig + e;
          paddr[tile][hf][e] = smem_u32(pst) + head * kPHead + p_offset<BITS>(tl, head);
        }
    const int pg = VG == 1 ? 0 : tw;   // value part: channels [32 tw, 32 tw + 32) = one value group
    const int pchunk = ((tig ^ (gid >> 1)) & 3) * 16;

    float m_run[2] = {kNegBig, kNegBig}, l_run[2] = {0.f, 0.f};
    float z_run[VG][2];   // sum of p * (value zero + centre * value scale): the constant term of the output
#pragma unroll
    for (int g = 0; g < VG; ++g) z_run[g][0] = z_run[g][1] = 0.f;
    float oacc[2][4];     // value part: channels (32 tw + 16 mt + gid, + 8) x heads (2 tig, 2 tig + 1)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) oacc[mt][e] = 0.f;

    int slot = team, phase = 0;   // ring position of block i = team, team + 2, ...: slot i mod stages, parity of i / stages
    if (slot >= p.stages) { slot -= p.stages; phase ^= 1; }
    for (int i = team; i < nblk; i += 2) {
      const unsigned char* st = stage + slot * sbytes;
      const int t0 = (blk0 + i) * kBlk;
      const int bvalid = min(kBlk, p.n_comp - t0);
      const int wvalid = max(0, min(32, bvalid - 32 * tw));   // 0, 16 or 32 tokens of this warp (16 only when G == 16)
      wait_bar(data_full + slot * 8, phase, status, dead);

      // ---------------- scores of this warp's 32 tokens ----------------
      float s[2][4];
      float alpha[2];
      {
        const int warp_tok = tw;   // (kept as a name: the lambdas below index tokens by it)
        uint32_t xh[16], xl[K2 ? 16 : 1];
        float c0 = 0.f, c1 = 0.f;
        // ---- scaled query of a token group: x = q * k_scale as fp16 operand pairs (two-term: value + rounding
        // residual, ~22 bits), and the constant sum_c q k_zero of the group for this lane's two heads ----
        auto prep = [&](int gl) {
          const float* ks = reinterpret_cast<const float*>(st + off_ks) + gl * kD + tig * 8;   // rows in kmeta_pos order
          const float* kz = reinterpret_cast<const float*>(st + off_kz) + gl * kD + tig * 8;
          float2 bacc[4];   // sum of (pre-scaled q) * k_zero per channel position pair (e, e + 1) of a run
#pragma unroll
          for (int j = 0; j < 4; ++j) bacc[j] = make_float2(0.f, 0.f);
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {   // sixteen channels (two runs of eight) at a time
            float pr[2][8], qv[2][8], sv[2][8];
#pragma unroll
            for (int u2 = 0; u2 < 2; ++u2) {
              const int u = h2 * 2 + u2;
#pragma unroll
              for (int v4 = 0; v4 < 2; ++v4) {
                const float4 s4 = *reinterpret_cast<const float4*>(ks + u * 32 + v4 * 4);
                const float4 z4 = *reinterpret_cast<const float4*>(kz + u * 32 + v4 * 4);
                const float4 q4 = *reinterpret_cast<const float4*>(qrow + u * 32 + v4 * 4);
                const float2 p01 = mul2(make_float2(q4.x, q4.y), make_float2(s4.x, s4.y));
                const float2 p23 = mul2(make_float2(q4.z, q4.w), make_float2(s4.z, s4.w));
                bacc[v4 * 2] = fma2(make_float2(q4.x, q4.y), make_float2(z4.x, z4.y), bacc[v4 * 2]);
                bacc[v4 * 2 + 1] = fma2(make_float2(q4.z, q4.w), make_float2(z4.z, z4.w), bacc[v4 * 2 + 1]);
                pr[u2][v4 * 4] = p01.x; pr[u2][v4 * 4 + 1] = p01.y; pr[u2][v4 * 4 + 2] = p23.x; pr[u2][v4 * 4 + 3] = p23.y;
                if constexpr (K2) {
                  qv[u2][v4 * 4] = q4.x; qv[u2][v4 * 4 + 1] = q4.y; qv[u2][v4 * 4 + 2] = q4.z; qv[u2][v4 * 4 + 3] = q4.w;
                  sv[u2][v4 * 4] = s4.x; sv[u2][v4 * 4 + 1] = s4.y; sv[u2][v4 * 4 + 2] = s4.z; sv[u2][v4 * 4 + 3] = s4.w;
                }
              }
            }
            // operand pair (channels ua:ea, ub:eb): the fp16 value and, as the second term, the exact residual of the product
            auto put = [&](int idx, int ua, int ea, int ub, int eb) {
              const __half2 hv = __floats2half2_rn(pr[ua][ea], pr[ub][eb]);
              xh[idx] = *reinterpret_cast<const uint32_t*>(&hv);
              if constexpr (K2) {
                const float2 hf = __half22float2(hv);
                const __half2 lv = __floats2half2_rn(fmaf(qv[ua][ea], sv[ua][ea], -hf.x), fmaf(qv[ub][eb], sv[ub][eb], -hf.y));
                xl[idx] = *reinterpret_cast<const uint32_t*>(&lv);
              }
            };
            if constexpr (BITS == 4) {   // a word is one run of eight channels: pairs (c_k, c_k+4)
#pragma unroll
              for (int u2 = 0; u2 < 2; ++u2)
#pragma unroll
                for (int k = 0; k < 4; ++k) put((h2 * 2 + u2) * 4 + k, u2, k, u2, k + 4);
            } else {                      // a word is both runs: pairs (c_j, c_j+8)
#pragma unroll
              for (int j = 0; j < 8; ++j) put(h2 * 8 + j, 0, j, 1, j);
            }
          }
          // undo the per-position pre-scaling of q in the constant term
          float bias = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            bias = fmaf(bacc[j].x, 1.f / code_factor<BITS>(2 * j), bias);
            bias = fmaf(bacc[j].y, 1.f / code_factor<BITS>(2 * j + 1), bias);
          }
          bias += __shfl_xor_sync(0xffffffffu, bias, 1);
          bias += __shfl_xor_sync(0xffffffffu, bias, 2);
          c0 = __shfl_sync(0xffffffffu, bias, (tig * 2) * 4) * scale2;
          c1 = __shfl_sync(0xffffffffu, bias, (tig * 2 + 1) * 4) * scale2;
        };
        // ---- scores of NT tiles of 16 tokens that share the operand: their MMA chains are independent and interleave ----
        auto run_tiles = [&](auto nt_tag, int tile0) {
          constexpr int NT = decltype(nt_tag)::value;
          uint32_t wa[NT][NW], wb[NT][NW];
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const unsigned char* krow = st + (32 * warp_tok + 16 * (tile0 + t) + gid) * KROW + tig * LB;
            if constexpr (BITS == 4) {
              const uint4 wa4 = *reinterpret_cast<const uint4*>(krow);
              const uint4 wb4 = *reinterpret_cast<const uint4*>(krow + 8 * KROW);
              wa[t][0] = wa4.x; wa[t][1] = wa4.y; wa[t][2] = wa4.z; wa[t][3] = wa4.w;
              wb[t][0] = wb4.x; wb[t][1] = wb4.y; wb[t][2] = wb4.z; wb[t][3] = wb4.w;
            } else {
              const uint2 wa2 = *reinterpret_cast<const uint2*>(krow);
              const uint2 wb2 = *reinterpret_cast<const uint2*>(krow + 8 * KROW);
              wa[t][0] = wa2.x; wa[t][1] = wa2.y;
              wb[t][0] = wb2.x; wb[t][1] = wb2.y;
            }
          }
          float d0[NT][4], d1[NT][4];
#pragma unroll
          for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) d0[t][e] = d1[t][e] = 0.f;
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            uint32_t pa[NT][PW], pb[NT][PW];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
              unpack_sub<BITS>(wa[t][w], pa[t]);
              unpack_sub<BITS>(wb[t][w], pb[t]);
            }
#pragma unroll
            for (int q4 = 0; q4 < PW / 4; ++q4) {
              const int x0 = w * PW + q4 * 4;
#pragma unroll
              for (int t = 0; t < NT; ++t) {
                mma16816<__half>(d0[t], pa[t][q4 * 4], pb[t][q4 * 4], pa[t][q4 * 4 + 1], pb[t][q4 * 4 + 1], xh[x0], xh[x0 + 1]);
                mma16816<__half>(d1[t], pa[t][q4 * 4 + 2], pb[t][q4 * 4 + 2], pa[t][q4 * 4 + 3], pb[t][q4 * 4 + 3], xh[x0 + 2], xh[x0 + 3]);
              }
              if constexpr (K2) {
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                  mma16816<__half>(d0[t], pa[t][q4 * 4], pb[t][q4 * 4], pa[t][q4 * 4 + 1], pb[t][q4 * 4 + 1], xl[x0], xl[x0 + 1]);
                  mma16816<__half>(d1[t], pa[t][q4 * 4 + 2], pb[t][q4 * 4 + 2], pa[t][q4 * 4 + 3], pb[t][q4 * 4 + 3], xl[x0 + 2], xl[x0 + 3]);
                }
              }
            }
          }
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            s[tile0 + t][0] = fmaf(d0[t][0] + d1[t][0], scale2o, c0);   // token gid,     head 2 tig
            s[tile0 + t][1] = fmaf(d0[t][1] + d1[t][1], scale2o, c1);   // token gid,     head 2 tig + 1
            s[tile0 + t][2] = fmaf(d0[t][2] + d1[t][2], scale2o, c0);   // token gid + 8, head 2 tig
            s[tile0 + t][3] = fmaf(d0[t][3] + d1[t][3], scale2o, c1);   // token gid + 8, head 2 tig + 1
          }
        };
#pragma unroll
        for (int t = 0; t < 2; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = kNegBig;
        if (G >= 32) {
          if (wvalid > 0) {   // both tiles lie in one token group
            prep((32 * warp_tok) >> lg);
            run_tiles(std::integral_constant<int, 2>{}, 0);
          }
        } else {
          for (int tile = 0; tile * 16 < wvalid; ++tile) {
            prep((32 * warp_tok + 16 * tile) >> lg);
            if (tile == 0) run_tiles(std::integral_constant<int, 1>{}, 0);
            else run_tiles(std::integral_constant<int, 1>{}, 1);
          }
        }
      }
      // ---- block maximum per head: this warp's 32 tokens, then the team's four warps through shared memory ----
      float mx0 = fmaxf(fmaxf(s[0][0], s[0][2]), fmaxf(s[1][0], s[1][2]));
      float mx1 = fmaxf(fmaxf(s[0][1], s[0][3]), fmaxf(s[1][1], s[1][3]));
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
      }
      if (gid == 0) *reinterpret_cast<float2*>(gm + tw * kHeads + 2 * tig) = make_float2(mx0, mx1);
      named_sync(team_bar, 128);   // the maxima are in; every warp of the team is done with the previous block's probabilities
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float mb = kNegBig;
#pragma unroll
        for (int w = 0; w < 4; ++w) mb = fmaxf(mb, gm[w * kHeads + 2 * tig + e]);
        const float m_new = fmaxf(m_run[e], mb);
        alpha[e] = exp2f(m_run[e] - m_new);
        m_run[e] = m_new;
        l_run[e] *= alpha[e];
#pragma unroll
        for (int g = 0; g < VG; ++g) z_run[g][e] *= alpha[e];
      }
      // ---------------- probabilities times the value scale into the team's operand buffer ----------------
      // (FULL: all 128 tokens of the block exist, which is every block but the last one of a context: no predicates)
      auto write_probs = [&](auto full_tag) {
        constexpr bool FULL = decltype(full_tag)::value;
        const float* vs = reinterpret_cast<const float*>(st + off_vs);
        const float* vz = reinterpret_cast<const float*>(st + off_vz);
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int tl = 32 * tw + 16 * tile + gid + 8 * hf;
            const bool live = FULL || tl < bvalid;
            float pe[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              pe[e] = live ? exp2f(s[tile][hf * 2 + e] - m_run[e]) : 0.f;
              l_run[e] += pe[e];
            }
#pragma unroll
            for (int g = 0; g < VG; ++g) {
              const float sc = live ? vs[tl * VG + g] : 0.f;
              const float zc = live ? fmaf((float)kVCentre<BITS>, sc, vz[tl * VG + g]) : 0.f;
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const float pv = pe[e] * sc;
                z_run[g][e] = fmaf(pe[e], zc, z_run[g][e]);
                const __half hv = __float2half_rn(pv);
                const uint32_t dst = paddr[tile][hf][e] + g * (2 * kHeads * kPHead);
                sts_h(dst, hv);
                if constexpr (P2) sts_h(dst + kHeads * kPHead, __float2half_rn(pv - __half2float(hv)));
              }
            }
          }
      };
      if (bvalid == kBlk) write_probs(std::true_type{});
      else write_probs(std::false_type{});
      named_sync(team_bar, 128);   // the block's probabilities are complete
      // ---------------- O = O * alpha + codes_v^T . P for this warp's 32 channels ----------------
      {
        uint32_t wa[2][NW], wb[2][NW];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          const unsigned char* vrow = st + off_vc + (32 * tw + 16 * mt + gid) * VROW + tig * LB;
          if constexpr (BITS == 4) {
            const uint4 va = *reinterpret_cast<const uint4*>(vrow);
            const uint4 vb = *reinterpret_cast<const uint4*>(vrow + 8 * VROW);
            wa[mt][0] = va.x; wa[mt][1] = va.y; wa[mt][2] = va.z; wa[mt][3] = va.w;
            wb[mt][0] = vb.x; wb[mt][1] = vb.y; wb[mt][2] = vb.z; wb[mt][3] = vb.w;
          } else {
            const uint2 va = *reinterpret_cast<const uint2*>(vrow);
            const uint2 vb = *reinterpret_cast<const uint2*>(vrow + 8 * VROW);
            wa[mt][0] = va.x; wa[mt][1] = va.y;
            wb[mt][0] = vb.x; wb[mt][1] = vb.y;
          }
        }
        const unsigned char* ph = pst + pg * (2 * kHeads * kPHead) + gid * kPHead + pchunk;
        // independent accumulator chains: (row tile, pair half, term)
        float o0[2][4], o1[2][4], o0l[2][4], o1l[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) o0[mt][e] = o1[mt][e] = o0l[mt][e] = o1l[mt][e] = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          uint32_t pa[2][PW], pb[2][PW];
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            unpack_centred<BITS>(wa[mt][w], pa[mt]);
            unpack_centred<BITS>(wb[mt][w], pb[mt]);
          }
#pragma unroll
          for (int q4 = 0; q4 < PW / 4; ++q4) {
            const int ci = w * (PW / 4) + q4;   // operand quad
            const uint4 pf = *reinterpret_cast<const uint4*>(ph + ci * 64);
            uint4 pl = make_uint4(0u, 0u, 0u, 0u);
            if constexpr (P2) pl = *reinterpret_cast<const uint4*>(ph + kHeads * kPHead + ci * 64);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
              mma16816<__half>(o0[mt], pa[mt][q4 * 4], pb[mt][q4 * 4], pa[mt][q4 * 4 + 1], pb[mt][q4 * 4 + 1], pf.x, pf.y);
              mma16816<__half>(o1[mt], pa[mt][q4 * 4 + 2], pb[mt][q4 * 4 + 2], pa[mt][q4 * 4 + 3], pb[mt][q4 * 4 + 3], pf.z, pf.w);
              if constexpr (P2) {
                mma16816<__half>(o0l[mt], pa[mt][q4 * 4], pb[mt][q4 * 4], pa[mt][q4 * 4 + 1], pb[mt][q4 * 4 + 1], pl.x, pl.y);
                mma16816<__half>(o1l[mt], pa[mt][q4 * 4 + 2], pb[mt][q4 * 4 + 2], pa[mt][q4 * 4 + 3], pb[mt][q4 * 4 + 3], pl.z, pl.w);
              }
            }
          }
        }
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(data_empty + slot * 8);
          if (tw == 3 && i + p.stages < nblk) {   // refill the slot once the team's four warps have released it
            wait_bar(data_empty + slot * 8, phase, status, dead);
            issue_block(i + p.stages, slot);
          }
        }
        slot += 2;
        if (slot >= p.stages) { slot -= p.stages; phase ^= 1; }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          oacc[mt][0] = fmaf(oacc[mt][0], alpha[0], (o0[mt][0] + o1[mt][0]) + (o0l[mt][0] + o1l[mt][0]));
          oacc[mt][1] = fmaf(oacc[mt][1], alpha[1], (o0[mt][1] + o1[mt][1]) + (o0l[mt][1] + o1l[mt][1]));
          oacc[mt][2] = fmaf(oacc[mt][2], alpha[0], (o0[mt][2] + o1[mt][2]) + (o0l[mt][2] + o1l[mt][2]));
          oacc[mt][3] = fmaf(oacc[mt][3], alpha[1], (o0[mt][3] + o1[mt][3]) + (o0l[mt][3] + o1l[mt][3]));
        }
      }
    }

    // ---------------- the two teams' results become the split's partial (max, sum, O) ----------------
    float* tm_s = alpha_s;   // [2 teams][8]: running maximum (base-2 units)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float lsum = l_run[e];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
      float cs[VG];
#pragma unroll
      for (int g = 0; g < VG; ++g) {
        float c = z_run[g][e];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
        cs[g] = c;
      }
      if (gid == 0) {
        float* f = fin_s + (warp * kHeads + 2 * tig + e) * kFinStride;
        f[0] = lsum;
#pragma unroll
        for (int g = 0; g < VG; ++g) f[1 + g] = cs[g];
        if (tw == 0) tm_s[team * kHeads + 2 * tig + e] = m_run[e];
      }
    }
    named_sync(1, kComputeThreads);
    float wt[2], corr[2];   // this team's weight in the split, and its constant term, for heads 2 tig, 2 tig + 1
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int hh = 2 * tig + e;
      const float M = fmaxf(tm_s[hh], tm_s[kHeads + hh]);
      wt[e] = exp2f(tm_s[team * kHeads + hh] - M);
      float c = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) c += fin_s[((team * 4 + w) * kHeads + hh) * kFinStride + 1 + pg];
      corr[e] = c;
    }
    float* obuf = reinterpret_cast<float*>(Pring);   // [8 heads][128 channels] fp32: team 1 -> team 0 (the probability buffers are free)
    if (team == 1) {
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int hh = 2 * tig + e, c = 32 * tw + 16 * mt + gid;
          obuf[hh * kD + c] = (oacc[mt][e] + corr[e]) * wt[e];
          obuf[hh * kD + c + 8] = (oacc[mt][2 + e] + corr[e]) * wt[e];
        }
    }
    named_sync(1, kComputeThreads);
    if (team == 0) {
      float* po = p.part_o + (bh * p.n_split + split) * (size_t)(kHeads * kD);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int hh = 2 * tig + e;
        if (hh < p.rep) {
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            const int c = 32 * tw + 16 * mt + gid;
            __stcg(po + hh * kD + c, (oacc[mt][e] + corr[e]) * wt[e] + obuf[hh * kD + c]);
            __stcg(po + hh * kD + c + 8, (oacc[mt][2 + e] + corr[e]) * wt[e] + obuf[hh * kD + c + 8]);
          }
        }
      }
      if (warp == 0 && lane < kHeads) {
        const float mA = tm_s[lane], mB = tm_s[kHeads + lane], M = fmaxf(mA, mB);
        float lA = 0.f, lB = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          lA += fin_s[(w * kHeads + lane) * kFinStride];
          lB += fin_s[((4 + w) * kHeads + lane) * kFinStride];
        }
        st_m[lane] = M * kLn2;
        st_l[lane] = lA * exp2f(mA - M) + lB * exp2f(mB - M);
      }
    }
    named_sync(1, kComputeThreads);   // st_m / st_l are complete
  } else {
    // ================= residual window: dense fp16/bf16 tokens from the stage =================
    float* S = reinterpret_cast<float*>(Pring);                 // [8][s_stride] scores
    constexpr int s_stride = kResChunk + 4;
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
      float* s0 = S + (tig * 2) * s_stride + tl;
      float* s1 = S + (tig * 2 + 1) * s_stride + tl;
      s0[0] = d0[0] * p.sm_scale;
      s1[0] = d0[1] * p.sm_scale;
      s0[8] = d0[2] * p.sm_scale;
      s1[8] = d0[3] * p.sm_scale;
    }
    named_sync(1, kComputeThreads);
    if (warp < p.rep) {
      float* srow = S + warp * s_stride;
      float m = kNegBig;
      for (int t = lane; t < valid; t += 32) m = fmaxf(m, srow[t]);
      m = warp_max(m);
      float l = 0.f;
      for (int t = lane; t < ((valid + 15) & ~15); t += 32) {   // the padding of the last 16-token step reads as zero
        const float e = t < valid ? __expf(srow[t] - m) : 0.f;
        srow[t] = e;
        l += e;
      }
      l = warp_sum(l);
      if (lane == 0) {
        st_m[warp] = m;
        st_l[warp] = l;
      }
    }
    named_sync(1, kComputeThreads);
    // P.V on the tensor cores: O^T[channel][head] = V^T[channel][token] . P[token][head], a warp per 16 channels.
    // The transposing matrix load turns the staged rows (token-major) into the row operand; the probabilities go
    // in as value + rounding residual in the window's own 16-bit type.
    {
      const int c0 = warp * 16;
      float dh[4] = {0.f, 0.f, 0.f, 0.f}, dl[4] = {0.f, 0.f, 0.f, 0.f};
      const int ksteps = (valid + 15) >> 4;
      for (int ks = 0; ks < ksteps; ++ks) {
        // lane -> row of matrix (lane >> 3): tokens 0-7 | 0-7 | 8-15 | 8-15 of the step, channels 0-7 | 8-15 | 0-7 | 8-15;
        // rows past the window repeat its last token (their probabilities are zero)
        const int trow = min(ks * 16 + (lane >> 4) * 8 + (lane & 7), valid - 1);
        const uint32_t addr = smem_u32(rv_s + trow * kResPitch + (c0 + ((lane >> 3) & 1) * 8) * 2);
        uint32_t a0, a1, a2, a3;
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                     : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(addr));
        const float* sp = S + gid * s_stride + ks * 16 + 2 * tig;
        const float2 p0 = *reinterpret_cast<const float2*>(sp), p1 = *reinterpret_cast<const float2*>(sp + 8);
        T hi[4] = {from_float<T>(p0.x), from_float<T>(p0.y), from_float<T>(p1.x), from_float<T>(p1.y)};
        T lo[4] = {from_float<T>(p0.x - to_float<T>(hi[0])), from_float<T>(p0.y - to_float<T>(hi[1])),
                   from_float<T>(p1.x - to_float<T>(hi[2])), from_float<T>(p1.y - to_float<T>(hi[3]))};
        const uint32_t* hb = reinterpret_cast<const uint32_t*>(hi);
        const uint32_t* lb = reinterpret_cast<const uint32_t*>(lo);
        mma16816<T>(dh, a0, a1, a2, a3, hb[0], hb[1]);
        mma16816<T>(dl, a0, a1, a2, a3, lb[0], lb[1]);
      }
      float* po = p.part_o + (bh * p.n_split + split) * (size_t)(kHeads * kD);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int hh = 2 * tig + e;
        if (hh < p.rep) {
          __stcg(po + hh * kD + c0 + gid, dh[e] + dl[e]);
          __stcg(po + hh * kD + c0 + gid + 8, dh[2 + e] + dl[2 + e]);
        }
      }
    }
  }

  if (threadIdx.x < p.rep) {
    float* pm = p.part_ml + (bh * p.n_split + split) * (size_t)(kHeads * 2);
    __stcg(pm + threadIdx.x * 2, st_m[threadIdx.x]);
    __stcg(pm + threadIdx.x * 2 + 1, st_l[threadIdx.x]);
  }

  // ================= merge of the splits by the last CTA of this (batch, head) =================
  // The partials of all threads are ordered before the counter by the barrier and thread 0's release; the last
  // arriver's acquire, followed by the second barrier, orders every other split's partials before the reads below.
  named_sync(1, kComputeThreads);
  if (threadIdx.x == 0) {
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + bh) : "memory");
    *s_last = (old == p.n_split - 1);
  }
  named_sync(1, kComputeThreads);
  if (!*s_last) return;
  const float* pm = p.part_ml + bh * p.n_split * (size_t)(kHeads * 2);
  const float* po = p.part_o + bh * p.n_split * (size_t)(kHeads * kD);
  // Everything the merge needs from global memory is requested before anything waits: first the partial outputs
  // of this thread (registers), then the statistics of all splits (shared memory).
  // thread = (split group, head, 8 channels): the groups take contiguous ranges of splits; their partial sums
  // meet in shared memory and are added in group order
  const int rep_pad = p.rep <= 1 ? 1 : (p.rep <= 2 ? 2 : (p.rep <= 4 ? 4 : 8));
  const int pairs = 16 * rep_pad, n_sg = kComputeThreads / pairs;
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
  float* w_s = reinterpret_cast<float*>(stage);   // [n_split][8]: max, then weight (the operand stages are free by now)
  float* l_s = w_s + p.n_split * kHeads;          // [n_split][8]: sum
  for (int i = threadIdx.x; i < p.n_split * kHeads; i += kComputeThreads) {
    const int hh = i & 7;
    w_s[i] = hh < p.rep ? __ldcg(pm + i * 2) : kNegBig;
    l_s[i] = hh < p.rep ? __ldcg(pm + i * 2 + 1) : 0.f;
  }
  named_sync(1, kComputeThreads);
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
  named_sync(1, kComputeThreads);
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
    named_sync(1, kComputeThreads);
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

struct AttnPlan {
  int nb, n_csplit, n_rsplit, n_split, stages;
  size_t smem;
};

// Blocks per compressed split: enough CTAs for two per SM, few enough splits for the merge, and as little of a
// nearly empty last wave as the choice allows (cost in block times: a CTA's fixed part counts as two blocks).
AttnPlan make_attn_plan(int B, int H, int n_comp, int n_res, int group, int bits, int vg) {
  AttnPlan a{};
  const int nblk = (n_comp + kBlk - 1) / kBlk;
  a.n_rsplit = (n_res + kResChunk - 1) / kResChunk;
  const long long slots = 2LL * sm_count();
  int nb_min = (nblk + (kMaxSplits - a.n_rsplit) - 1) / (kMaxSplits - a.n_rsplit);
  if (nb_min < 1) nb_min = 1;
  int nb_max = nblk < kMaxNb ? nblk : kMaxNb;
  if (nb_max < nb_min) nb_max = nb_min;
  // Makespan model in microseconds.  A compressed split runs its blocks on two teams side by side, so it takes
  // ceil(nb / 2) block times plus a fixed part (first data, the teams' merge, the partial's store and the counter);
  // block and fixed times are longer when every SM holds two CTAs.  Residual splits are short and fill the gaps of
  // the last wave; the merge by the last arriver grows with the number of splits.
  int best = nb_min;
  double best_cost = 1e30;
  const double pairs = (double)B * H;
  for (int nb = nb_min; nb <= nb_max && nblk > 0; ++nb) {
    const long long cs = (nblk + nb - 1) / nb;
    const int nb_even = (int)((nblk + cs - 1) / cs);   // blocks of the largest split when the blocks are spread evenly
    if (nb_even != nb) continue;                        // the same split count with fewer blocks per split comes later
    const double c_ctas = pairs * cs, r_ctas = pairs * a.n_rsplit;
    const bool light = c_ctas + r_ctas <= 0.6 * (double)slots;
    const double t_blk = light ? 2.0 : 3.1, t_fix = light ? 3.0 : 4.5, t_res = light ? 2.5 : 3.5;
    const double t_cta = t_fix + ((nb + 1) / 2) * t_blk;
    const double waves = (double)((long long)((c_ctas + slots - 1) / slots));
    double span = waves * t_cta;
    const double area = (c_ctas * t_cta + r_ctas * t_res) / (double)slots;
    if (area > span) span = area;
    if (span < t_res) span = t_res;
    const double cost = span + 2.5 + 0.035 * (double)(cs + a.n_rsplit);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = nb;
    }
  }
  a.nb = best;
  a.n_csplit = nblk ? (nblk + a.nb - 1) / a.nb : 0;
  a.n_split = a.n_csplit + a.n_rsplit;
  const int sb = stage_bytes(group, bits, vg);
  const size_t fixed = ring_offset(vg);
  int stages = (int)((kAttnSmemBudget - fixed) / sb);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > a.nb) stages = a.nb;
  if (stages < 2) stages = 2;
  a.stages = stages;
  size_t ring = (size_t)stages * sb;
  const size_t need_other = 2 * kResChunk * kResPitch;   // the residual stage; the merge scratch (24 KB) is smaller
  if (ring < need_other) ring = need_other;
  a.smem = fixed + ring;
  return a;
}

}  // namespace
}  // namespace pare

extern "C" {

size_t pare_kivi_attn_workspace_bytes(int B, int H, int n_comp, int n_res) {
  if (B <= 0 || H <= 0 || n_comp < 0 || n_res < 0) return 0;
  // one block per split is the finest plan -> upper bound on the split count
  size_t n_split = (size_t)(n_comp + 127) / 128 + (size_t)(n_res + pare::kResChunk - 1) / pare::kResChunk + 1;
  if (n_split > (size_t)pare::kMaxSplits + 1) n_split = pare::kMaxSplits + 1;
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
  // The merge takes kMaxSplits splits per (batch, head); a split runs as many blocks of 128 compressed tokens as that
  // bound needs, so the context itself is not limited here (beyond kMaxNb blocks per split the planner only stops
  // balancing waves).
  PARE_REQUIRE(plan.n_split <= kMaxSplits, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(plan.smem <= kAttnSmemBudget, PARE_ERR_UNSUPPORTED);

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
  p.nb = plan.nb; p.stages = plan.stages; p.n_csplit = plan.n_csplit; p.n_split = plan.n_split;
  const size_t need = kCounterBytes + (size_t)B * H * p.n_split * (kHeads * kD + kHeads * 2) * sizeof(float);
  PARE_REQUIRE(workspace && workspace_bytes >= need, PARE_ERR_WORKSPACE);
  p.counters = reinterpret_cast<int*>(workspace);
  p.part_o = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + kCounterBytes);
  p.part_ml = p.part_o + (size_t)B * H * p.n_split * kHeads * kD;

  auto launch = [&](auto kern) -> int {
    if (!ensure_smem_attr(reinterpret_cast<const void*>(kern), (int)kAttnSmemBudget)) return PARE_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.n_split * H * B), 1, 1);
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
  constexpr int kMode = 3;   // two-term scaled query and two-term probabilities: what the parity bars need
  if (vg == 1) {
    if (bits == 4) return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 4, 1, kMode>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 4, 1, kMode>);
    return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 2, 1, kMode>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 2, 1, kMode>);
  }
  if (bits == 4) return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 4, kMaxVG, kMode>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 4, kMaxVG, kMode>);
  return dtype == PARE_F16 ? launch(kivi_decode_attn_kernel<__half, 2, kMaxVG, kMode>) : launch(kivi_decode_attn_kernel<__nv_bfloat16, 2, kMaxVG, kMode>);
}

}  // extern "C"
