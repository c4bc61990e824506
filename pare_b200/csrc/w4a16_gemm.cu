// W4A16 tensor-core path for M > 16 (prefill), sm_100a: dequantize to shared memory, tcgen05.mma
// with the accumulator in tensor memory.
//
// Replaces the Triton tile kernel of the reference (pare/kernels/matmul_int4.py:54-176) where
// tiles are worth it.  Orientation: the 128 rows of a weight tile sit on the MMA M axis (the 128
// TMEM lanes), the activation rows on the MMA N axis, so a 64-row batch does not waste half of
// every instruction:   Y^T[n][m] = sum_k W[n][k] * X[m][k].
//
// One CTA = 128 output rows x one tile of up to 128 activation rows x one K range.  Warp roles:
//   warps 0-7  dequantize (two groups of four warps, one per 64-column block of a 128-column stage, one thread per weight row), then
//              run the epilogue
//   warp 8     producer, two lanes: packed codes by TMA (cp.async.bulk.tensor.2d over the [N][K/2] byte matrix,
//              one 128-row x 128-byte box per 256-column stage, 128B swizzle) into a four-stage ring, requested up
//              to three stages ahead; activation tiles by TMA (128B swizzle) one operand stage ahead of the MMA
//   warp 9     one elected thread issues tcgen05.mma (UMMA 128 x MT x 16, fp32 accumulate in TMEM)
// Per 64-column block a dequantizing thread reads 16 bytes of codes, computes (q - zero) * scale in fp32 (packed
// two-wide fp32 instructions, codes read in place as subnormal floats: dequant_word below), rounds to the 16-bit
// type and writes four 16-byte chunks of the K-major, 128B-swizzled operand tile that the MMA reads through a
// shared-memory descriptor.  Weights therefore reach the tensor core as exactly dtype(fp32((q - zero) * scale)),
// bit for bit what the reference's own dequantize-then-matmul path feeds its GEMM (pare/layers/linear.py:112-118, 129).
// All mbarrier waits are bounded; on expiry the CTA records PARE_ERR_TIMEOUT, stops waiting,
// frees its tensor memory and returns.

#include <cuda.h>

#include "common.cuh"

namespace pare {
namespace {

constexpr int kRows = 128;             // weight rows per CTA (UMMA M)
constexpr int kBlockK = 64;            // columns per MMA stage: 128 bytes of 16-bit elements = one swizzle row
constexpr int kRawK = 256;             // columns per raw (packed) stage: four 64-column blocks, one tensor-map box
constexpr int kRawBytes = kRows * 128; // bytes of a raw stage: 128 rows x 128 bytes, 128B swizzle
constexpr int kRawStages = 4;          // three stages (3 x 1.2 us of work) in flight cover the 2.5 - 3.5 us a box takes to arrive
constexpr int kRawKb = kRawK / kBlockK;
constexpr int kStages = 2;             // operand ring depth, in stages of two 64-column blocks (one barrier round per 128 columns)
constexpr int kStageBytes = 32768;     // per operand and stage: two K-major 128B-swizzled tiles of up to 128 rows
constexpr int kDequantThreads = 256;
constexpr int kGemmThreads = kDequantThreads + 64;
constexpr uint32_t kSpin = 1u << 22;
constexpr size_t kCounterInts = 16384;
constexpr size_t kCounterBytes = kCounterInts * sizeof(int);
constexpr size_t kStatusIndex = kCounterInts - 1;

struct GemmParams {
  const uint8_t* packed;
  const float* scale;
  const float* zero;
  const void* bias;
  void* y;
  int64_t ldy;
  int M, N, K, ngroups, group_size;
  int mt;               // activation rows per tile (UMMA N): 32, 64, 128 or 256
  int raw_stages;       // depth of the packed-code ring (4; 2 when the 256-row activation tiles take the shared memory)
  int kblocks_per_split;
  int splits;
  float* partial;       // [splits][M][N]
  int* counters;
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  `dead` is sticky per thread: after one expiry nothing waits any more.
__device__ __forceinline__ void bar_wait(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  if (dead) return;
#pragma unroll 1
  for (uint32_t i = 0; i < kSpin; ++i)
    if (bar_test(bar, parity)) return;
  dead = true;
  if (status) atomicExch(status, PARE_ERR_TIMEOUT);
}
__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ uint4 ld_s128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void st_s128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// K-major operand tile, 128-byte rows, 128B swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- activations for the tensor-core path when they need work: the act-order gather and / or the run-time input
// scale, into a dense [M][K] copy in column order.  Plain layers skip this launch: the activation tiles are then
// fetched by TMA straight from the caller's tensor. ----
template <typename T>
__global__ void w4a16_gemm_prep_kernel(const T* x, int64_t ldx, const int32_t* col_perm, const float* input_scale, T* xq,
                                       int M, int K) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)M * K) return;
  const int m = (int)(idx / K), k = (int)(idx - (int64_t)m * K);
  const int src = col_perm ? col_perm[k] : k;
  float v = to_float<T>(x[(int64_t)m * ldx + src]);
  if (input_scale) v = __fdiv_rn(v, input_scale[src]);
  xq[(int64_t)m * K + k] = from_float<T>(v);
}

template <typename T>
struct Pair;
template <>
struct Pair<__half> {
  static constexpr uint32_t kFmt = 0;
  // (lo, hi) fp32 -> one word of two fp16, round to nearest even
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
};
template <>
struct Pair<__nv_bfloat16> {
  static constexpr uint32_t kFmt = 1;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
};

// Packed fp32 pairs (two independent IEEE operations per instruction).
__device__ __forceinline__ void fma_pair2(float& a, float& b, float m, float c0, float c1) {   // (a, b) = (a, b) * m + (c0, c1)
  asm("{\n\t.reg .b64 x, y, z;\n\t"
      "mov.b64 x, {%0, %1};\n\t"
      "mov.b64 y, {%2, %2};\n\t"
      "mov.b64 z, {%3, %4};\n\t"
      "fma.rn.f32x2 x, x, y, z;\n\t"
      "mov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a), "+f"(b)
      : "f"(m), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void mul_pair2(float& a, float& b, float m0, float m1) {   // (a, b) = (a, b) * (m0, m1)
  asm("{\n\t.reg .b64 x, y;\n\t"
      "mov.b64 x, {%0, %1};\n\t"
      "mov.b64 y, {%2, %3};\n\t"
      "mul.rn.f32x2 x, x, y;\n\t"
      "mov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a), "+f"(b)
      : "f"(m0), "f"(m1));
}

// Per (weight row, group) constants of the dequantization below.
struct DqConst {
  float zc[4];   // -zero * 2^(4k - 22)
  float sc[4];   // scale * 2^(22 - 4k)
  __device__ __forceinline__ void set(float scale, float zero) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      zc[k] = -zero * __int_as_float((127 + 4 * k - 22) << 23);
      sc[k] = scale * __int_as_float((127 + 22 - 4 * k) << 23);
    }
  }
};

// One 32-bit word of codes -> 8 dequantized 16-bit values in COLUMN ORDER as one 16-byte chunk, each EXACTLY
// dtype(fp32((q - zero) * scale)): the weight the reference's eager path feeds its GEMM
// (pare/layers/linear.py:112-118, 129: fp32 subtract, fp32 multiply, cast).  A code nibble left in place at bits
// 4k .. 4k+3 (k = 0..3; the upper four codes after one shift by 16) and read as a float's bit pattern is the subnormal
// q * 2^(4k - 149); one fused multiply-add by 2^127 with -zero * 2^(4k - 22) gives (q - zero) * 2^(4k - 22) with the
// single rounding of the reference's fp32 subtraction (powers of two do not change a rounding; no rounding at all for
// the integer zero-points of the reference's quantizers), one multiply by scale * 2^(22 - 4k) its fp32 product, one
// conversion per pair the cast.  The two lanes of a packed instruction are neighbouring columns (positions k, k + 1),
// each with its own constants, so the operand tile is in the activations' own column order and the activations need
// no re-ordering pass.
template <typename T>
__device__ __forceinline__ uint4 dequant_word(uint32_t w, const DqConst& c) {
  const uint32_t t = w >> 16;
  constexpr float kTwo127 = 1.7014118346046923e38f;
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {   // columns 2j, 2j + 1
    const uint32_t src = j < 2 ? w : t;
    const int k = (2 * j) & 3;
    float a = __uint_as_float(src & (0xFu << (4 * k)));
    float b = __uint_as_float(src & (0xFu << (4 * k + 4)));
    fma_pair2(a, b, kTwo127, c.zc[k], c.zc[k + 1]);
    mul_pair2(a, b, c.sc[k], c.sc[k + 1]);
    o[j] = Pair<T>::pack(a, b);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <typename T>
__global__ void __launch_bounds__(kGemmThreads) w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                                                                 const GemmParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // an activation block is mt rows x 128 bytes: 16 KB up to 128 rows, 32 KB at 256
  const uint32_t b_blk = p.mt > 128 ? 32768u : 16384u, b_stage = 2 * b_blk;
  const int rstages = p.raw_stages;
  unsigned char* a_ring = smem;                                   // kStages x 2 blocks x 16 KB
  unsigned char* b_ring = a_ring + kStages * kStageBytes;         // kStages x 2 blocks x b_blk
  unsigned char* raw = b_ring + kStages * b_stage;                // rstages x 16 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw + rstages * kRawBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
  const uint32_t raw_full = s_u32(bars), raw_empty = s_u32(bars + 4), a_full = s_u32(bars + 8), b_full = s_u32(bars + 12),
                 ab_empty = s_u32(bars + 16), acc_full = s_u32(bars + 20);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * kRows;
  const int m0 = blockIdx.z * p.mt;
  const int kb_total = p.K / kBlockK;
  const int kb0 = blockIdx.y * p.kblocks_per_split;
  const int nkb = min(p.kblocks_per_split, kb_total - kb0);       // multiple of 4 (host guarantees)
  int* status = p.counters ? p.counters + kStatusIndex : nullptr;
  bool dead = false;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kRawStages; ++i) {
      bar_init(raw_full + i * 8, 1);
      bar_init(raw_empty + i * 8, kDequantThreads / 32);
    }
    for (int i = 0; i < kStages; ++i) {
      // one barrier per operand stage for both operands: the eight dequantizing warps that write A (one group per
      // 64-column block) and the producer's expect-tx arrival for the two activation tiles (a wait costs the MMA
      // thread ~230 cycles even when the phase is complete, and that thread's loop is what paces the kernel)
      bar_init(a_full + i * 8, kDequantThreads / 32 + 1);
      bar_init(b_full + i * 8, 1);
      bar_init(ab_empty + i * 8, 1);
    }
    bar_init(acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {  // tensor memory: one power-of-two block of columns for the fp32 accumulator
    const uint32_t ncols = p.mt < 32 ? 32 : p.mt;
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_u32(tmem_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 8) {
    // ================= producer =================
    // Two independent lanes: lane 1 keeps the raw ring full (a stage is requested as soon as its slot is free, a
    // whole stage before the dequantizing threads reach it), lane 0 feeds the activation ring four blocks ahead
    // of the MMA.  A raw stage is one tensor-map copy of 128 rows x 128 bytes.
    if (lane == 1) {
      for (int rs = 0; rs < nkb / kRawKb; ++rs) {
        const int slot = rs % rstages;
        bar_wait(raw_empty + slot * 8, ((rs / rstages) & 1) ^ 1, status, dead);
        bar_expect(raw_full + slot * 8, kRawBytes);
        const int xb = (kb0 + rs * kRawKb) * (kBlockK / 2);   // byte column of the stage
        tma_tile(s_u32(raw) + slot * kRawBytes, &tm_w, xb, row0, raw_full + slot * 8);
      }
    } else if (lane == 0) {
      for (int kd = 0; kd < nkb / 2; ++kd) {  // the two activation tiles of each stage
        const int s = kd % kStages;
        bar_wait(ab_empty + s * 8, ((kd / kStages) & 1) ^ 1, status, dead);
        bar_expect(a_full + s * 8, 2 * p.mt * 128);
        tma_tile(s_u32(b_ring) + s * b_stage, &tm_x, (kb0 + 2 * kd) * kBlockK, m0, a_full + s * 8);
        tma_tile(s_u32(b_ring) + s * b_stage + b_blk, &tm_x, (kb0 + 2 * kd + 1) * kBlockK, m0, a_full + s * 8);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ================= MMA issuer =================
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (Pair<T>::kFmt << 7) | (Pair<T>::kFmt << 10) | ((uint32_t)(p.mt >> 3) << 17) |
                             ((uint32_t)(kRows >> 4) << 24);
      // This thread's loop paces the kernel (every instruction waits for the one before), so it carries as little
      // as possible: descriptors of stage 0 built once, a stage or a 16-column step further is an addition to the
      // descriptor's address field (units of 16 bytes).
      const uint64_t a_desc0 = umma_desc(s_u32(a_ring)), b_desc0 = umma_desc(s_u32(b_ring));
      for (int kd = 0; kd < nkb / 2; ++kd) {
        const int s = kd % kStages;
        const uint32_t par = (kd / kStages) & 1;
        bar_wait(a_full + s * 8, par, status, dead);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a_desc = a_desc0 + (uint64_t)(s * (kStageBytes >> 4)), b_desc = b_desc0 + (uint64_t)(s * (b_stage >> 4));
        umma_f16(tmem_acc, a_desc, b_desc, idesc, kd != 0);
#pragma unroll
        for (int j = 1; j < 2 * (kBlockK / 16); ++j) {   // the second block's tiles start one block after the first's
          const uint64_t oa = (uint64_t)((j >> 2) * (16384 >> 4) + (j & 3) * 2);
          const uint64_t ob = (uint64_t)((j >> 2) * (b_blk >> 4) + (j & 3) * 2);
          umma_f16(tmem_acc, a_desc + oa, b_desc + ob, idesc, 1u);
        }
        umma_commit(ab_empty + s * 8);  // frees the operand stage when these MMAs have read it
      }
      umma_commit(acc_full);
    }
    __syncwarp();
  } else {
    // ================= dequantize =================
    // Two groups of four warps, one thread per weight row; group g writes block g of every stage (the blocks
    // kb = g mod 2), so a thread's fixed cost per stage (barrier wait, arrival, loop: more cycles than its
    // arithmetic) is spread over 64 weights.
    const int r = threadIdx.x & 127, grp = threadIdx.x >> 7;
    const int gr = min(row0 + r, p.N - 1);
    const int spg = p.group_size / 128;                     // 128-column halves of a raw stage per group
    const uint32_t a_row = (r >> 3) * 1024 + (r & 7) * 128;
    float sc[2], zc[2], sc_n[2], zc_n[2];
    // scale / zero of the two 128-column halves of a raw stage: a row-strided (one line per thread) read that
    // often comes from DRAM, so the next stage's values are requested a whole stage before they are needed
    auto load_meta = [&](int kb, float (&s4)[2], float (&z4)[2]) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int g = min(((kb0 + kb) / 2 + i) / spg, p.ngroups - 1);
        s4[i] = __ldg(p.scale + (size_t)gr * p.ngroups + g);
        z4[i] = __ldg(p.zero + (size_t)gr * p.ngroups + g);
      }
    };
    load_meta(0, sc_n, zc_n);
    for (int kb = grp; kb < nkb; kb += 2) {
      const int rsi = kb / kRawKb, slot = rsi % rstages;
      if ((kb & (kRawKb - 1)) == grp) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          sc[i] = sc_n[i];
          zc[i] = zc_n[i];
        }
        if (kb - grp + kRawKb < nkb) load_meta(kb - grp + kRawKb, sc_n, zc_n);
        bar_wait(raw_full + slot * 8, (rsi / rstages) & 1, status, dead);
      }
      const int kd = kb >> 1, s = kd % kStages;   // this group writes block grp of stage kd
      bar_wait(ab_empty + s * 8, ((kd / kStages) & 1) ^ 1, status, dead);
      // 16-byte chunks (kb & 3) * 2 and + 1 of row r of the stage, where the 128B swizzle put them
      const uint32_t raw_row = s_u32(raw) + slot * kRawBytes + r * 128;
      const uint4 codes0 = ld_s128(raw_row + ((((kb & 3) * 2) ^ (r & 7)) << 4));
      const uint4 codes1 = ld_s128(raw_row + ((((kb & 3) * 2 + 1) ^ (r & 7)) << 4));
      const bool second = (kb & 2) != 0;   // which 128-column half of the stage
      DqConst dq;
      dq.set(second ? sc[1] : sc[0], second ? zc[1] : zc[0]);
      const uint32_t wv[8] = {codes0.x, codes0.y, codes0.z, codes0.w, codes1.x, codes1.y, codes1.z, codes1.w};
      const uint32_t dst = s_u32(a_ring) + s * kStageBytes + grp * 16384 + a_row;
#pragma unroll
      for (int wi = 0; wi < 8; ++wi) {
        const uint4 v = dequant_word<T>(wv[wi], dq);
        st_s128(dst + ((wi ^ (r & 7)) << 4), v.x, v.y, v.z, v.w);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // make the tile visible to the MMA unit
      __syncwarp();
      if (lane == 0) {
        bar_arrive(a_full + s * 8);
        if ((kb & (kRawKb - 1)) == kRawKb - 2 + grp) bar_arrive(raw_empty + slot * 8);   // this group's last block of the raw stage
      }
    }

    // ================= epilogue: TMEM -> registers -> global =================
    bar_wait(acc_full, 0, status, dead);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int q4 = warp & 3, chalf = warp >> 2;
    const int n = row0 + q4 * 32 + lane;
    const int cpw = p.mt / 2;  // columns per warp group
    T* yg = reinterpret_cast<T*>(p.y);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const float bv = (bias && n < p.N && p.splits == 1) ? to_float<T>(bias[n]) : 0.f;
    float* part = p.splits > 1 ? p.partial + (size_t)blockIdx.y * p.M * p.N : nullptr;
    // Whole-K tiles with an aligned output go through a per-warp transpose in shared memory (the operand ring is
    // free by now): a lane holds ONE output column n for 16 activation rows, i.e. 2-byte stores 64 bytes per
    // instruction; after the transpose a lane stores 8 consecutive n of one row as 16 bytes.
    const bool vec_out = part == nullptr && (reinterpret_cast<uintptr_t>(p.y) & 15u) == 0 && (p.ldy & 7) == 0 && row0 + kRows <= p.N;
    const uint32_t tbuf = s_u32(a_ring) + warp * 1024;   // [16 activation rows][32 n] of T
    for (int c = chalf * cpw; c < (chalf + 1) * cpw; c += 16) {
      uint32_t v[16];
      const uint32_t taddr = tmem_acc + ((uint32_t)(q4 * 32) << 16) + (uint32_t)c;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
            "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (vec_out) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const T h = from_float<T>(__uint_as_float(v[i]) + bv);
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(tbuf + (i * 32 + lane) * 2), "h"(*reinterpret_cast<const unsigned short*>(&h)) : "memory");
        }
        __syncwarp();
        if (!dead) {
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            const int mi = pass * 8 + (lane >> 2), seg = lane & 3;
            const int m = m0 + c + mi;
            const uint4 o = ld_s128(tbuf + (mi * 32 + seg * 8) * 2);
            if (m < p.M) *reinterpret_cast<uint4*>(yg + (size_t)m * p.ldy + row0 + q4 * 32 + seg * 8) = o;
          }
        }
        __syncwarp();
      } else if (n < p.N && !dead) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int m = m0 + c + i;
          if (m < p.M) {
            const float f = __uint_as_float(v[i]);
            if (part)
              __stcg(part + (size_t)m * p.N + n, f);
            else
              yg[(size_t)m * p.ldy + n] = from_float<T>(f + bv);
          }
        }
      }
    }
  }

  // ---- teardown: everyone done with tensor memory, then free it ----
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    const uint32_t ncols = p.mt < 32 ? 32 : p.mt;
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(ncols) : "memory");
  }
  if (p.splits == 1) return;

  // ---- K spans several CTAs: the last one to arrive adds the partial sums in split order ----
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  const int tile_id = blockIdx.z * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counters + tile_id, 1) == p.splits - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int tile_rows = min(kRows, p.N - row0), tile_m = min(p.mt, p.M - m0);
  T* yg = reinterpret_cast<T*>(p.y);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  const bool vec = tile_rows == kRows && (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 7u) == 0 && (p.ldy & 3) == 0;
  if (vec) {
    // Four outputs per 16-byte load, four such pieces per thread and up to four splits requested before anything is
    // added: the loop is a chain of L2 round trips, so what counts is how many loads each trip carries.  Every
    // output is still the sum of its partials in split order.
    constexpr int kU = 4, kS = 4, kQ = kRows / 4;
    const int total = tile_m * kQ;
    for (int base = threadIdx.x; base < total; base += kGemmThreads * kU) {
      float4 acc[kU];
      const float* src[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int idx = min(base + u * kGemmThreads, total - 1);
        acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        src[u] = p.partial + (size_t)(m0 + idx / kQ) * p.N + row0 + (idx % kQ) * 4;
      }
      for (int s0 = 0; s0 < p.splits; s0 += kS) {
        float4 t[kS][kU];
#pragma unroll
        for (int si = 0; si < kS; ++si)
#pragma unroll
          for (int u = 0; u < kU; ++u)
            t[si][u] = s0 + si < p.splits ? __ldcg(reinterpret_cast<const float4*>(src[u] + (size_t)(s0 + si) * p.M * p.N))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int si = 0; si < kS; ++si)
#pragma unroll
          for (int u = 0; u < kU; ++u) {
            acc[u].x += t[si][u].x; acc[u].y += t[si][u].y; acc[u].z += t[si][u].z; acc[u].w += t[si][u].w;
          }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int idx = base + u * kGemmThreads;
        if (idx < total) {
          const int m = m0 + idx / kQ, n = row0 + (idx % kQ) * 4;
          float4 v = acc[u];
          if (bias) {
            v.x += to_float<T>(bias[n]); v.y += to_float<T>(bias[n + 1]); v.z += to_float<T>(bias[n + 2]); v.w += to_float<T>(bias[n + 3]);
          }
          T o[4] = {from_float<T>(v.x), from_float<T>(v.y), from_float<T>(v.z), from_float<T>(v.w)};
          *reinterpret_cast<uint2*>(yg + (size_t)m * p.ldy + n) = *reinterpret_cast<const uint2*>(o);
        }
      }
    }
  } else {
    for (int idx = threadIdx.x; idx < tile_rows * tile_m; idx += kGemmThreads) {
      const int mi = idx / tile_rows, n = row0 + (idx - mi * tile_rows), m = m0 + mi;
      float v = 0.f;
      for (int s = 0; s < p.splits; ++s) v += __ldcg(p.partial + ((size_t)s * p.M + m) * p.N + n);
      if (bias) v += to_float<T>(bias[n]);
      yg[(size_t)m * p.ldy + n] = from_float<T>(v);
    }
  }
  if (threadIdx.x == 0) p.counters[tile_id] = 0;
}

// ---- host side --------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// alignment slack + dequantized-weight ring + activation ring + packed-code ring + barriers and the TMEM slot
constexpr size_t gemm_smem_bytes(int mt, int raw_stages) {
  return 1024 + (size_t)kStages * kStageBytes + (size_t)kStages * 2 * (mt > 128 ? 32768 : 16384) + (size_t)raw_stages * kRawBytes + 25 * 8 + 64;
}
constexpr size_t kGemmSmemMax = gemm_smem_bytes(256, 2);   // 224 KB of rings: the 256-row tile leaves room for two packed stages
static_assert(kGemmSmemMax >= gemm_smem_bytes(128, kRawStages) && kGemmSmemMax <= 227 * 1024, "shared memory plan");

struct GemmPlan {
  int mt, mtiles, mpad, splits, kblocks_per_split;
};

// K splits by a cost model in microseconds: whole waves of one CTA per SM, each CTA a fixed part (launch, first
// loads, epilogue: ~10) plus a time per 64-column block that grows mildly with the activation tile, plus the
// cross-CTA sum when K is split (it grows with the rows: splitting pays below about a hundred rows only).  It also
// avoids a second, nearly empty wave.
GemmPlan gemm_plan_for(int mt, int M, int N, int K, double* cost_out) {
  GemmPlan g{};
  g.mt = mt;
  g.mtiles = (M + g.mt - 1) / g.mt;
  g.mpad = g.mtiles * g.mt;
  const int row_tiles = (N + kRows - 1) / kRows;
  const int raw_stages = K / kRawK;
  const int tiles = row_tiles * g.mtiles;
  const int sms = sm_count();
  const double per_block = mt > 128 ? 0.40 : 0.35;
  int best_per = raw_stages;
  double best_cost = 1e30;
  for (int s = 1; s <= 16 && s <= raw_stages; ++s) {
    const int per = (raw_stages + s - 1) / s, s_eff = (raw_stages + per - 1) / per;
    const int waves = (tiles * s_eff + sms - 1) / sms;
    // a split costs its fp32 partials written and read again by the one CTA per tile that adds them: measured at
    // about 1 us per MB of partials (qkv 6144 x 4096, 256 rows: 43 us unsplit, 54 / 55 us in 2 / 3 splits)
    const double cost = waves * (10.0 + per * kRawKb * per_block) + (s_eff > 1 ? 3.0 + (double)s_eff * M * N * 8e-6 : 0.0);
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best_per = per;
    }
  }
  g.splits = (raw_stages + best_per - 1) / best_per;
  g.kblocks_per_split = best_per * kRawKb;
  *cost_out = best_cost;
  return g;
}

// Above 128 rows a CTA may take 256 activation rows (UMMA N = 256, 256 TMEM columns): a weight stage is then
// dequantized once per 256 rows, and dequantization, not the tensor pipe, is what bounds this kernel.  Layers with few
// row tiles can be better off with twice the CTAs of 128 rows; the cost model decides.
GemmPlan gemm_plan(int M, int N, int K) {
  double c = 0.0;
  if (M <= 128) return gemm_plan_for(M <= 32 ? 32 : (M <= 64 ? 64 : 128), M, N, K, &c);
  double c128 = 0.0, c256 = 0.0;
  const GemmPlan g128 = gemm_plan_for(128, M, N, K, &c128), g256 = gemm_plan_for(256, M, N, K, &c256);
  return c256 <= c128 ? g256 : g128;
}

}  // namespace

bool gemm_supported(int M, int K, int G, const float* scale, const float* zero) {
  // 512 rather than the raw stage's 256: shapes between the two keep the streaming kernel's fp32-weight semantics
  return M > 16 && (K % 512) == 0 && (G % 128) == 0 && scale != nullptr && zero != nullptr;
}

size_t gemm_workspace_bytes(int M, int N, int K) {
  const GemmPlan g = gemm_plan(M, N, K);
  // the same formula as gemm_forward's own check: partial sums only when the plan splits K, and only its splits
  return kCounterBytes + ((size_t)g.mpad * K * 2 + 255) / 256 * 256 + (g.splits > 1 ? (size_t)g.splits * M * N * sizeof(float) : 0);
}

int gemm_forward(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale, const float* zero,
                 const int32_t* col_perm, const float* input_scale, const void* bias, void* y, int64_t ldy, int M, int N,
                 int K, int G, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  const GemmPlan g = gemm_plan(M, N, K);
  const size_t xq_bytes = ((size_t)g.mpad * K * 2 + 255) / 256 * 256;
  const size_t need = kCounterBytes + xq_bytes + (g.splits > 1 ? (size_t)g.splits * M * N * sizeof(float) : 0);
  PARE_REQUIRE(workspace != nullptr && workspace_bytes >= need, PARE_ERR_WORKSPACE);
  PARE_REQUIRE(aligned16(packed), PARE_ERR_ALIGN);
  const int row_tiles = (N + kRows - 1) / kRows;
  PARE_REQUIRE((size_t)row_tiles * g.mtiles < kStatusIndex, PARE_ERR_UNSUPPORTED);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  void* xq = ws + kCounterBytes;

  // 1) activations: gathered / scaled into the workspace if the layer asks for that (or the caller's rows cannot be
  //    described by a tensor map: 16-byte aligned base and row pitch), otherwise used where they are
  const bool direct = col_perm == nullptr && input_scale == nullptr && aligned16(x) && (ldx % 8) == 0;
  if (!direct) {
    const int64_t total = (int64_t)M * K;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (x_dtype == PARE_F16)
      w4a16_gemm_prep_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)x, ldx, col_perm, input_scale, (__half*)xq, M, K);
    else
      w4a16_gemm_prep_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, col_perm, input_scale,
                                                                        (__nv_bfloat16*)xq, M, K);
    if (cudaGetLastError() != cudaSuccess) return PARE_ERR_CUDA;
  }

  // 2) tensor map over the activations [M][K] (rows of the last tile beyond M read as zeros), box 64 columns x mt
  //    rows, 128B swizzle
  EncodeTiledFn enc = encode_fn();
  PARE_REQUIRE(enc != nullptr, PARE_ERR_CUDA);
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)(direct ? ldx : K) * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)g.mt};
  const cuuint32_t estr[2] = {1, 1};
  PARE_REQUIRE(enc(&tm, x_dtype == PARE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   direct ? const_cast<void*>(x) : xq, dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
               PARE_ERR_CUDA);

  // tensor map over the packed codes [N][K/2] bytes, box 128 bytes x 128 rows, 128B swizzle (rows beyond N read as zeros)
  CUtensorMap tw;
  const cuuint64_t wdims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)N};
  const cuuint64_t wstrides[1] = {(cuuint64_t)(K / 2)};
  const cuuint32_t wbox[2] = {128u, (cuuint32_t)kRows};
  PARE_REQUIRE(enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(packed), wdims, wstrides, wbox, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
               PARE_ERR_CUDA);

  GemmParams p{};
  p.packed = packed;
  p.scale = scale;
  p.zero = zero;
  p.bias = bias;
  p.y = y;
  p.ldy = ldy;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ngroups = K / G;
  p.group_size = G;
  p.mt = g.mt;
  p.raw_stages = g.mt > 128 ? 2 : kRawStages;
  p.kblocks_per_split = g.kblocks_per_split;
  p.splits = g.splits;
  p.counters = reinterpret_cast<int*>(ws);
  p.partial = reinterpret_cast<float*>(ws + kCounterBytes + xq_bytes);

  const dim3 grid(row_tiles, g.splits, g.mtiles);
  auto launch = [&](auto kern) -> int {
    if (!ensure_smem_attr(reinterpret_cast<const void*>(kern), (int)kGemmSmemMax)) return PARE_ERR_CUDA;
    kern<<<grid, kGemmThreads, gemm_smem_bytes(p.mt, p.raw_stages), stream>>>(tm, tw, p);
    return launch_status();
  };
  return x_dtype == PARE_F16 ? launch(w4a16_gemm_kernel<__half>) : launch(w4a16_gemm_kernel<__nv_bfloat16>);
}

}  // namespace pare
