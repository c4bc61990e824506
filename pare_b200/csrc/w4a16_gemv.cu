// W4A16 streaming dequant-GEMV for M <= 16 (decode), sm_100a.
//
// Replaces the Triton tile kernel of the reference (pare/kernels/matmul_int4.py:54-176)
// for small M, where that kernel wastes >= 31/32 of every tile.  Per output row n
//     y[m][n] = sum_g  scale[n][g] * ( sum_{k in g} x[m][k] * q[n][k]  -  zero[n][g] * sum_{k in g} x[m][k] )
// which is the reference formula (q - zero) * scale (pare/core/functional.py:78-91) with
// the zero-point and the scale hoisted out of the inner loop.
//
// The kernel is HBM-bound; every weight byte is read exactly once and the design goal is
// to keep instructions per weight low and bytes in flight high:
//   * A CTA owns 64 output rows x one K range.  One elected thread streams that tile with
//     TMA (cp.async.bulk.tensor.2d, 128-byte-swizzled boxes of 64 rows x 128 B) into a ring
//     of shared-memory stages guarded by mbarriers; scale and zero ride in the same stages
//     (boxes of 64 rows x 4 groups).  Registers hold one step at a time, so many warps stay
//     resident and the whole tile can be in flight at once.
//   * Four consumer warps take 16 rows each.  Per 128-column step a lane reads 2 x 16 bytes
//     of codes (conflict-free thanks to the swizzle and a row permutation), turns them into
//     exact integer-valued fp16/bf16 by OR-ing into the mantissa of a power of two, and
//     multiplies them with the activations on the warp-level MMA unit (fp32 accumulation;
//     the 8 MMA columns carry up to 8 activation rows at the cost of one).
//   * Activations are staged once per CTA in shared memory in operand order, with the
//     per-group sums the hoisted zero-point needs (warp-shuffle reductions).
//   * Split-K partial sums go to a workspace; the CTA that arrives last at a per-row-tile
//     counter adds them in split order (deterministic) and resets the counter.
//   * Programmatic dependent launch: the weight stream starts before griddepcontrol.wait.
// Every mbarrier wait is bounded; on expiry the kernel records PARE_ERR_TIMEOUT in the
// workspace status word and runs to completion without waiting again.

#include <cuda.h>

#include "common.cuh"

namespace pare {
namespace {

constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kTileRows = kConsumerWarps * 16;  // 64
constexpr int kBoxBytes = kTileRows * 128;      // one swizzled weight box: 64 rows x 128 B
constexpr int kStageBytes = 2 * kBoxBytes + 2048;  // 512 columns: two boxes + scale box + zero box
constexpr int kMaxDepth = 12;
constexpr uint32_t kSpinLimit = 1u << 22;

// Workspace layout: [counters | status word][partials fp32].  The counter region has a FIXED
// size so the partial sums of one call can never land where another call keeps its counters;
// the counters are the only part that must be zero between calls.
constexpr size_t kCounterInts = 16384;
constexpr size_t kCounterBytes = kCounterInts * sizeof(int);
constexpr size_t kStatusIndex = kCounterInts - 1;

struct GemvParams {
  const void* x;
  int64_t ldx;
  const float* scale;
  const float* zero;
  const uint32_t* meta_h2;
  const int32_t* col_perm;
  const float* input_scale;
  const void* bias;
  void* y;
  int64_t ldy;
  int M, N, K;
  int ngroups;          // K / group_size
  int steps_per_group;  // group_size / 128
  int steps_per_split;  // 128-column steps per CTA (multiple of 4)
  int splits;
  int depth;            // ring stages
  float* partial;       // [splits][M][N]
  int* counters;        // [row tiles]; counters[kStatusIndex] is the status word
  int x_vec_ok;
};

// ---- mbarrier / TMA primitives -------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
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
// Bounded wait: returns false (and records the failure) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  if (dead) return false;
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_test(bar, parity)) return true;
  dead = true;
  if (status) atomicExch(status, PARE_ERR_TIMEOUT);
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

template <typename T>
__device__ __forceinline__ void mma_zero_c(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  d[0] = d[1] = d[2] = d[3] = 0.f;
  mma16816<T>(d, a0, a1, a2, a3, b0, b1);
}

// META: 0 = fp32 scale/zero through TMA, 1 = fp16 pairs through TMA, 2 = plain loads at fold time
template <typename T, int MB, int META>
__global__ void __launch_bounds__(kThreads) w4a16_gemv_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                             const __grid_constant__ CUtensorMap tm_s,
                                                             const __grid_constant__ CUtensorMap tm_z,
                                                             const GemvParams p) {
  extern __shared__ unsigned char smem_raw[];
  constexpr int MP = 8 * MB;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int steps_total = (p.K + 127) >> 7;
  const int st0 = blockIdx.y * p.steps_per_split;
  const int nst = min(p.steps_per_split, steps_total - st0);  // 128-column steps of this CTA
  const int nstg = (nst + 3) >> 2;                            // ring stages of this CTA
  const int k0 = st0 << 7;
  const int tile_row0 = blockIdx.x * kTileRows;
  const int spg = p.steps_per_group;
  const int g_first = st0 / spg;
  const int nseg = (st0 + nst - 1) / spg - g_first + 1;
  const int depth = p.depth;

  // ---- shared memory carve-up (ring must be 1024-byte aligned for the 128B swizzle) ----
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* ring = smem;
  const int xrows = min(p.M, MP);
  const int xstride = nstg * 1024 + 64;  // bytes per activation row; == 64 (mod 128)
  unsigned char* xs = ring + (size_t)depth * kStageBytes;
  float2* tab = reinterpret_cast<float2*>(xs + (size_t)xrows * xstride);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(tab) + (size_t)nseg * MP * sizeof(float2));
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxDepth);
  const uint32_t ring_u32 = smem_u32(ring);
  int* status = p.counters ? p.counters + kStatusIndex : nullptr;
  bool dead = false;

  const bool is_producer = (warp == kConsumerWarps);
  constexpr uint32_t kTxBytes = 2 * kBoxBytes + (META == 0 ? 2048 : (META == 1 ? 1024 : 0));

  auto issue_stage = [&](int it) {
    const int slot = it % depth;
    const uint32_t dst = ring_u32 + slot * kStageBytes;
    const uint32_t bar = full0 + slot * 8;
    const int kb = (k0 >> 1) + it * 256;  // byte column of the stage
    mbar_expect_tx(bar, kTxBytes);
    tma_load_2d(dst, &tm_w, kb, tile_row0, bar);
    tma_load_2d(dst + kBoxBytes, &tm_w, kb + 128, tile_row0, bar);
    if (META == 0) {
      const int gb = ((k0 >> 7) + it * 4) * 4;  // byte column in the [N][ngroups] fp32 arrays
      tma_load_2d(dst + 2 * kBoxBytes, &tm_s, gb, tile_row0, bar);
      tma_load_2d(dst + 2 * kBoxBytes + 1024, &tm_z, gb, tile_row0, bar);
    } else if (META == 1) {
      const int gb = ((k0 >> 7) + it * 4) * 4;  // [N][ngroups] half2 pairs, 4 B each
      tma_load_2d(dst + 2 * kBoxBytes, &tm_s, gb, tile_row0, bar);
    }
  };

  if (threadIdx.x == kConsumerWarps * 32) {
    for (int i = 0; i < depth; ++i) {
      mbar_init(full0 + i * 8, 1);
      mbar_init(empty0 + i * 8, kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // weights do not depend on the previous kernel: fill the ring before the dependency wait
  if (threadIdx.x == kConsumerWarps * 32) {
    const int first = min(depth, nstg);
    for (int it = 0; it < first; ++it) issue_stage(it);
  }
  pdl_launch_dependents();
  pdl_wait();

  // ---- stage activations: operand order + per-segment sums (all five warps) ----
  {
    const T* xg = reinterpret_cast<const T*>(p.x);
    const int c = lane >> 1, hsel = lane & 1;
    const int chunk_off = (c & 3) * 64 + (c >> 2) * 16;  // [word][quad] order inside a step
    // only rows m < M are staged; table entries of the unused MMA columns are never read back
    for (int pr = warp; pr < nseg * p.M; pr += kConsumerWarps + 1) {
      const int seg = pr / p.M, m = pr - seg * p.M;
      const int pair = seg * MP + m;
      const int sb = max(0, (g_first + seg) * spg - st0);
      const int se = min(nst, (g_first + seg + 1) * spg - st0);
      float lo = 0.f, hi = 0.f;
      {
        for (int st = sb; st < se; ++st) {
          const int k = k0 + st * 128 + lane * 4;
          float v[4];
          if (p.col_perm == nullptr && p.x_vec_ok) {
            const uint2 raw = *reinterpret_cast<const uint2*>(xg + (size_t)m * p.ldx + k);
            const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = to_float<T>(e[i]);
            if (p.input_scale) {
#pragma unroll
              for (int i = 0; i < 4; ++i) v[i] = __fdiv_rn(v[i], __ldg(p.input_scale + k + i));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int src = p.col_perm ? __ldg(p.col_perm + k + i) : k + i;
              v[i] = to_float<T>(xg[(size_t)m * p.ldx + src]);
              if (p.input_scale) v[i] = __fdiv_rn(v[i], __ldg(p.input_scale + src));
            }
          }
          // round to the operand type first (the activation the oracle sees), then apply the
          // exact power-of-two prescale of the odd code positions
          T b[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float r = to_float<T>(from_float<T>(v[i]));
            b[i] = from_float<T>((i & 1) ? r * Nibbles<T>::kHiPrescale : r);
          }
          lo += to_float<T>(b[0]) + to_float<T>(b[2]);
          hi += to_float<T>(b[1]) + to_float<T>(b[3]);
          T* dst = reinterpret_cast<T*>(xs + (size_t)m * xstride + st * 256 + chunk_off);
          dst[0 + hsel] = b[0];
          dst[2 + hsel] = b[1];
          dst[4 + hsel] = b[2];
          dst[6 + hsel] = b[3];
        }
      }
      lo = warp_sum(lo);
      hi = warp_sum(hi);
      if (lane == 0) {
        // E: what the mantissa offsets add to the accumulator; SX: plain sum of x
        const float E = Nibbles<T>::kOffsetLo * lo + Nibbles<T>::kOffsetHi * hi;
        const float SX = lo + hi / Nibbles<T>::kHiPrescale;
        tab[pair] = make_float2(E, SX);
      }
    }
  }
  __syncthreads();

  float yacc[MB][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int i = 0; i < 4; ++i) yacc[mb][i] = 0.f;

  // fragment row gid maps to tile row rho: rows of one quarter-warp differ in bit 2, which the
  // 128B swizzle turns into different 64-byte halves -> conflict-free 16-byte reads
  const int rho = ((gid & 1) << 2) | (gid >> 1);
  const int rowA = warp * 16 + rho, rowB = rowA + 8;  // rows inside the tile (consumer warps)

  if (is_producer) {
    if (lane == 0) {
      for (int it = depth; it < nstg; ++it) {
        const int slot = it % depth;
        mbar_wait(empty0 + slot * 8, ((it / depth) & 1) ^ 1, status, dead);
        issue_stage(it);
      }
    }
    __syncwarp();
  } else {
    float d0[MB][4], d1[MB][4];
    int pos_in_group = st0 - g_first * spg;
    bool fresh = true;  // accumulators hold nothing yet for the current group
    for (int it = 0; it < nstg; ++it) {
      const int slot = it % depth;
      mbar_wait(full0 + slot * 8, (it / depth) & 1, status, dead);
      const unsigned char* stage = ring + (size_t)slot * kStageBytes;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const int st = it * 4 + s;
        if (st < nst) {
          const unsigned char* box = stage + (s >> 1) * kBoxBytes;
          const int chunk = (((s & 1) * 4 + tig) ^ rho) * 16;
          const uint4 wa4 = *reinterpret_cast<const uint4*>(box + rowA * 128 + chunk);
          const uint4 wb4 = *reinterpret_cast<const uint4*>(box + rowB * 128 + chunk);
          const uint32_t wa[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
          const uint32_t wb[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
          uint4 xb[MB][4];
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            const int m = mb * 8 + gid;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (m < p.M)
                xb[mb][i] = *reinterpret_cast<const uint4*>(xs + (size_t)m * xstride + st * 256 + i * 64 + tig * 16);
              else
                xb[mb][i] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t pa[4], pb[4];
            Nibbles<T>::unpack(wa[i], pa);
            Nibbles<T>::unpack(wb[i], pb);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              if (i == 0 && fresh) {
                mma_zero_c<T>(d0[mb], pa[0], pb[0], pa[1], pb[1], xb[mb][i].x, xb[mb][i].y);
                mma_zero_c<T>(d1[mb], pa[2], pb[2], pa[3], pb[3], xb[mb][i].z, xb[mb][i].w);
              } else {
                mma16816<T>(d0[mb], pa[0], pb[0], pa[1], pb[1], xb[mb][i].x, xb[mb][i].y);
                mma16816<T>(d1[mb], pa[2], pb[2], pa[3], pb[3], xb[mb][i].z, xb[mb][i].w);
              }
            }
          }
          fresh = false;
          // end of a quantization group (or of this CTA's K range): fold with scale / zero
          const bool fold = (pos_in_group == spg - 1) || (st == nst - 1);
          if (fold) {
            const int g = (st0 + st) / spg;
            float sA, zA, sB, zB;
            if (META == 0) {
              sA = *reinterpret_cast<const float*>(stage + 2 * kBoxBytes + rowA * 16 + s * 4);
              sB = *reinterpret_cast<const float*>(stage + 2 * kBoxBytes + rowB * 16 + s * 4);
              zA = *reinterpret_cast<const float*>(stage + 2 * kBoxBytes + 1024 + rowA * 16 + s * 4);
              zB = *reinterpret_cast<const float*>(stage + 2 * kBoxBytes + 1024 + rowB * 16 + s * 4);
            } else if (META == 1) {
              const __half2 ha = *reinterpret_cast<const __half2*>(stage + 2 * kBoxBytes + rowA * 16 + s * 4);
              const __half2 hb = *reinterpret_cast<const __half2*>(stage + 2 * kBoxBytes + rowB * 16 + s * 4);
              sA = __low2float(ha);
              zA = __high2float(ha);
              sB = __low2float(hb);
              zB = __high2float(hb);
            } else {
              const size_t ia = (size_t)min(tile_row0 + rowA, p.N - 1) * p.ngroups + g;
              const size_t ib = (size_t)min(tile_row0 + rowB, p.N - 1) * p.ngroups + g;
              if (p.meta_h2) {
                const uint32_t va = __ldg(p.meta_h2 + ia), vb = __ldg(p.meta_h2 + ib);
                const __half2 ha = *reinterpret_cast<const __half2*>(&va), hb = *reinterpret_cast<const __half2*>(&vb);
                sA = __low2float(ha);
                zA = __high2float(ha);
                sB = __low2float(hb);
                zB = __high2float(hb);
              } else {
                sA = __ldg(p.scale + ia);
                zA = __ldg(p.zero + ia);
                sB = __ldg(p.scale + ib);
                zB = __ldg(p.zero + ib);
              }
            }
            const int seg = g - g_first;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              const float4 t = *reinterpret_cast<const float4*>(&tab[seg * MP + mb * 8 + tig * 2]);  // E0 SX0 E1 SX1
              yacc[mb][0] = fmaf(sA, fmaf(-zA, t.y, (d0[mb][0] + d1[mb][0]) - t.x), yacc[mb][0]);
              yacc[mb][1] = fmaf(sA, fmaf(-zA, t.w, (d0[mb][1] + d1[mb][1]) - t.z), yacc[mb][1]);
              yacc[mb][2] = fmaf(sB, fmaf(-zB, t.y, (d0[mb][2] + d1[mb][2]) - t.x), yacc[mb][2]);
              yacc[mb][3] = fmaf(sB, fmaf(-zB, t.w, (d0[mb][3] + d1[mb][3]) - t.z), yacc[mb][3]);
            }
            fresh = true;
          }
          pos_in_group = (pos_in_group == spg - 1) ? 0 : pos_in_group + 1;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + slot * 8);
    }
  }

  // ---- epilogue ----
  T* yg = reinterpret_cast<T*>(p.y);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  if (p.splits == 1) {
    if (!is_producer) {
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = tile_row0 + ((i >> 1) ? rowB : rowA);
          const int m = mb * 8 + tig * 2 + (i & 1);
          if (n < p.N && m < p.M) {
            float v = yacc[mb][i];
            if (bias) v += to_float<T>(bias[n]);
            yg[(size_t)m * p.ldy + n] = from_float<T>(v);
          }
        }
    }
    return;
  }

  float* part = p.partial + (size_t)blockIdx.y * p.M * p.N;
  if (!is_producer) {
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = tile_row0 + ((i >> 1) ? rowB : rowA);
        const int m = mb * 8 + tig * 2 + (i & 1);
        if (n < p.N && m < p.M) __stcg(part + (size_t)m * p.N + n, yacc[mb][i]);
      }
  }
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counters + blockIdx.x, 1) == p.splits - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int tile_rows = min(kTileRows, p.N - tile_row0);
  for (int idx = threadIdx.x; idx < tile_rows * p.M; idx += kThreads) {
    const int m = idx / tile_rows, n = tile_row0 + (idx - m * tile_rows);
    float v = 0.f;
    for (int s = 0; s < p.splits; ++s) v += __ldcg(p.partial + ((size_t)s * p.M + m) * p.N + n);
    if (bias) v += to_float<T>(bias[n]);
    yg[(size_t)m * p.ldy + n] = from_float<T>(v);
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;  // leave the workspace ready for the next call
}

// ---- any-shape fallback: one thread per output, used when K or the group size is not a
// multiple of 128 (tiny layers); correctness path, not a performance path ----
template <typename T>
__global__ void w4a16_generic_kernel(const GemvParams p, const uint8_t* packed, int group_size) {
  pdl_wait();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)p.M * p.N) return;
  const int m = (int)(idx / p.N), n = (int)(idx - (int64_t)m * p.N);
  const T* xg = reinterpret_cast<const T*>(p.x);
  const uint8_t* wrow = packed + (size_t)n * (p.K >> 1);
  float acc = 0.f;
  for (int g = 0; g < p.ngroups; ++g) {
    float s, z;
    if (p.meta_h2) {
      const uint32_t v = p.meta_h2[(size_t)n * p.ngroups + g];
      const __half2 hv = *reinterpret_cast<const __half2*>(&v);
      s = __low2float(hv);
      z = __high2float(hv);
    } else {
      s = p.scale[(size_t)n * p.ngroups + g];
      z = p.zero[(size_t)n * p.ngroups + g];
    }
    float dot = 0.f, sx = 0.f;
    for (int k = g * group_size; k < (g + 1) * group_size; ++k) {
      const int src = p.col_perm ? p.col_perm[k] : k;
      float xv = to_float<T>(xg[(size_t)m * p.ldx + src]);
      if (p.input_scale) xv = to_float<T>(from_float<T>(__fdiv_rn(xv, p.input_scale[src])));
      const uint8_t byte = wrow[k >> 1];
      const float q = (float)((k & 1) ? (byte >> 4) : (byte & 0xF));
      dot = fmaf(xv, q, dot);
      sx += xv;
    }
    acc = fmaf(s, fmaf(-z, sx, dot), acc);
  }
  if (p.bias) acc += to_float<T>(reinterpret_cast<const T*>(p.bias)[n]);
  reinterpret_cast<T*>(p.y)[(size_t)m * p.ldy + n] = from_float<T>(acc);
}

// ---- host side ----------------------------------------------------------------------
int g_tune_splits = 0, g_tune_depth = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D byte tensor [rows][row_bytes] with box [kTileRows][box_bytes]
bool make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes, bool swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_bytes, (cuuint32_t)kTileRows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Plan {
  bool fast;
  int meta;  // 0 fp32 TMA, 1 fp16 TMA, 2 plain loads
  int splits, steps_per_split, depth;
  size_t smem;
};

constexpr int kSmCount = 148;
constexpr size_t kSmemCap = 200 * 1024;

size_t gemv_smem(int M, int MB, int nst, int spg, int depth) {
  const int xrows = M < 8 * MB ? M : 8 * MB;
  const int nstg = (nst + 3) / 4;
  const int nseg = (nst + spg - 1) / spg + 1;
  return 1024 + (size_t)depth * kStageBytes + (size_t)xrows * (nstg * 1024 + 64) + (size_t)nseg * 8 * MB * sizeof(float2) +
         2 * kMaxDepth * sizeof(uint64_t) + 16;
}

Plan make_plan(int M, int N, int K, int G, bool meta16) {
  Plan pl{};
  pl.fast = (K % 128 == 0) && (G % 128 == 0);
  if (!pl.fast) return pl;
  const int MB = M <= 8 ? 1 : 2;
  const int steps = K / 128;
  const int ngroups = K / G;
  pl.meta = (G == 128 && ngroups % 4 == 0) ? (meta16 ? 1 : 0) : 2;
  const int row_tiles = (N + kTileRows - 1) / kTileRows;
  const int stages = (steps + 3) / 4;
  int splits;
  if (g_tune_splits) {
    splits = g_tune_splits;
  } else {
    // aim at ~4 CTAs per SM so the whole layer is in flight at once when it fits
    splits = (4 * kSmCount + row_tiles - 1) / row_tiles;
  }
  if (splits > stages) splits = stages;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  int stg_per_split = (stages + splits - 1) / splits;
  int depth = g_tune_depth ? g_tune_depth : 4;
  if (depth > stg_per_split) depth = stg_per_split;
  if (depth > kMaxDepth) depth = kMaxDepth;
  // the activation tile must fit beside the ring: shorten the K range if it does not
  while (gemv_smem(M, MB, stg_per_split * 4, G / 128, depth) > kSmemCap && stg_per_split > 1) {
    stg_per_split = (stg_per_split + 1) / 2;
    if (depth > stg_per_split) depth = stg_per_split;
  }
  splits = (stages + stg_per_split - 1) / stg_per_split;
  pl.splits = splits;
  pl.steps_per_split = stg_per_split * 4;
  pl.depth = depth;
  pl.smem = gemv_smem(M, MB, pl.steps_per_split, G / 128, depth);
  return pl;
}

template <typename T, int MB, int META>
int launch_gemv(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const GemvParams& p, const Plan& pl,
                cudaStream_t stream) {
  auto kern = w4a16_gemv_kernel<T, MB, META>;
  static bool attr_done[64] = {};  // per instantiation and device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PARE_ERR_CUDA;
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemCap) != cudaSuccess)
      return PARE_ERR_CUDA;
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + kTileRows - 1) / kTileRows, pl.splits, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, tw, ts, tz, p) != cudaSuccess) return PARE_ERR_CUDA;
  return PARE_OK;
}

template <typename T>
int dispatch_gemv(const CUtensorMap& tw, const CUtensorMap& ts, const CUtensorMap& tz, const GemvParams& p,
                  const Plan& pl, cudaStream_t stream) {
  if (p.M <= 8) {
    if (pl.meta == 0) return launch_gemv<T, 1, 0>(tw, ts, tz, p, pl, stream);
    if (pl.meta == 1) return launch_gemv<T, 1, 1>(tw, ts, tz, p, pl, stream);
    return launch_gemv<T, 1, 2>(tw, ts, tz, p, pl, stream);
  }
  if (pl.meta == 0) return launch_gemv<T, 2, 0>(tw, ts, tz, p, pl, stream);
  if (pl.meta == 1) return launch_gemv<T, 2, 1>(tw, ts, tz, p, pl, stream);
  return launch_gemv<T, 2, 2>(tw, ts, tz, p, pl, stream);
}

template <typename T>
int launch_generic(const GemvParams& p, const uint8_t* packed, int G, cudaStream_t stream) {
  const int64_t total = (int64_t)p.M * p.N;
  const int threads = 128;
  w4a16_generic_kernel<T><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(p, packed, G);
  return launch_status();
}

}  // namespace

size_t gemv_workspace_bytes(int M, int N, int K, int G) {
  const int m = M < 16 ? M : 16;
  size_t splits = 1;
  if (K % 128 == 0 && G % 128 == 0) splits = (size_t)((K / 128 + 3) / 4);  // upper bound on any plan
  if (splits > 64) splits = 64;
  return kCounterBytes + splits * (size_t)m * N * sizeof(float);
}

// Called by pare_w4a16_forward for every chunk of at most 16 activation rows.
int gemv_forward(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale,
                 const float* zero, const void* meta_h2, const int32_t* col_perm, const float* input_scale,
                 const void* bias, void* y, int64_t ldy, int M, int N, int K, int G, void* workspace,
                 size_t workspace_bytes, cudaStream_t stream) {
  GemvParams p{};
  p.x = x;
  p.ldx = ldx;
  p.scale = scale;
  p.zero = zero;
  p.meta_h2 = reinterpret_cast<const uint32_t*>(meta_h2);
  p.col_perm = col_perm;
  p.input_scale = input_scale;
  p.bias = bias;
  p.y = y;
  p.ldy = ldy;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ngroups = K / G;
  p.steps_per_group = G / 128;
  p.x_vec_ok = ((reinterpret_cast<uintptr_t>(x) & 7u) == 0 && (ldx % 4) == 0) ? 1 : 0;

  Plan pl = make_plan(M, N, K, G, meta_h2 != nullptr);
  if (!pl.fast) {
    return x_dtype == PARE_F16 ? launch_generic<__half>(p, packed, G, stream)
                               : launch_generic<__nv_bfloat16>(p, packed, G, stream);
  }
  PARE_REQUIRE(aligned16(packed) && (K % 32) == 0, PARE_ERR_ALIGN);
  PARE_REQUIRE((size_t)(N + kTileRows - 1) / kTileRows < kStatusIndex, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(pl.smem <= kSmemCap, PARE_ERR_UNSUPPORTED);
  p.splits = pl.splits;
  p.steps_per_split = pl.steps_per_split;
  p.depth = pl.depth;
  if (workspace != nullptr && workspace_bytes >= kCounterBytes) p.counters = reinterpret_cast<int*>(workspace);
  if (pl.splits > 1) {
    const size_t need = kCounterBytes + (size_t)pl.splits * M * N * sizeof(float);
    PARE_REQUIRE(workspace != nullptr && workspace_bytes >= need, PARE_ERR_WORKSPACE);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + kCounterBytes);
  }

  CUtensorMap tw, ts, tz;
  PARE_REQUIRE(make_map(&tw, packed, (uint64_t)K / 2, (uint64_t)N, 128, true), PARE_ERR_CUDA);
  ts = tw;
  tz = tw;
  if (pl.meta == 0) {
    PARE_REQUIRE(aligned16(scale) && aligned16(zero), PARE_ERR_ALIGN);
    PARE_REQUIRE(make_map(&ts, scale, (uint64_t)p.ngroups * 4, (uint64_t)N, 16, false), PARE_ERR_CUDA);
    PARE_REQUIRE(make_map(&tz, zero, (uint64_t)p.ngroups * 4, (uint64_t)N, 16, false), PARE_ERR_CUDA);
  } else if (pl.meta == 1) {
    PARE_REQUIRE(aligned16(meta_h2), PARE_ERR_ALIGN);
    PARE_REQUIRE(make_map(&ts, meta_h2, (uint64_t)p.ngroups * 4, (uint64_t)N, 16, false), PARE_ERR_CUDA);
  }
  return x_dtype == PARE_F16 ? dispatch_gemv<__half>(tw, ts, tz, p, pl, stream)
                             : dispatch_gemv<__nv_bfloat16>(tw, ts, tz, p, pl, stream);
}

void gemv_set_tuning(int rb, int splits, int depth) {
  (void)rb;
  g_tune_splits = splits;
  g_tune_depth = depth;
}

}  // namespace pare
