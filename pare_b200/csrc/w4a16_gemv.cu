// W4A16 streaming dequant-GEMV for M <= 16 (decode), sm_100a.
//
// Replaces the Triton tile kernel of the reference (pare/kernels/matmul_int4.py:54-176)
// for small M, where that kernel wastes >= 31/32 of every tile.  Per output row n
//     y[m][n] = sum_g  scale[n][g] * ( sum_{k in g} x[m][k] * q[n][k]  -  zero[n][g] * sum_{k in g} x[m][k] )
// which is the reference formula (q - zero) * scale (pare/core/functional.py:78-91) with
// the zero-point and the scale hoisted out of the inner loop.
//
// The path is HBM-bound by design; every weight byte is read exactly once.  This file holds the tile kernel
// (small layers, and the fallback of every fast-path shape), the activation-preparation kernel, the
// any-shape fallback and the host-side routing; large layers run the persistent schedule of
// w4a16_gemv_persist.cu.  Tile kernel:
//   * A CTA owns 16 (or 32) output rows x one K range of up to 4096 columns.  Lanes 0..15 of warp 0
//     issue one bulk async copy (cp.async.bulk, the non-tensor TMA path) per row: a row's
//     whole K range is one contiguous request of up to 2 KB, which is what HBM and the copy
//     engine like; all 16 complete on one mbarrier.  Every CTA has its whole tile in flight
//     from its first instructions, and several CTAs are resident per SM.
//   * The shared-memory row pitch is (bytes + 64), so the 16-byte reads of a quarter-warp
//     (two adjacent rows x four chunks) fall in distinct banks without any swizzle.
//   * The WARPS warps of the CTA split the K range; each takes all 16 rows.  Per 128-column
//     step a lane reads 2 x 16 bytes of codes, turns them into exact integer-valued fp16
//     by OR-ing into the mantissa of 1024.0, and multiplies them with the (fp16, per-step scaled) activations
//     on the warp-level MMA unit (fp32 accumulation; the 8 MMA columns carry up to 8
//     activation rows at the cost of one).  Scale and zero of the warp's groups are
//     prefetched into registers before anything else.
//   * Activations arrive prepared (prep.cuh: operand order + per-step table), written once per call by
//     w4a16_prep_kernel or by the kernel that computed them; the CTAs only copy their slice into shared
//     memory -- or compute it themselves from the residual stream / the fused gate|up tensor (stage.cuh).
//   * The warps' partial sums meet in shared memory.  Only when K exceeds one CTA's range do
//     partial sums go through the global workspace: the CTA that arrives last at a
//     per-row-tile counter adds them in split order (deterministic) and resets the counter.
//   * Programmatic dependent launch: weights and metadata do not depend on the previous
//     kernel, so their loads are issued before griddepcontrol.wait.
// The mbarrier wait is bounded; on expiry the kernel records PARE_ERR_TIMEOUT in the
// workspace status word and runs to completion without waiting again.

#include "gemv_common.cuh"
#include "prep.cuh"
#include "stage.cuh"

namespace pare {

// what stage.cuh computes the activations from
struct ProducerArgs {
  int kind;
  const void* a;
  const void* b;
  const void* c;
  void* resid_out;
  int64_t lda;
  float eps;
};

namespace {

using namespace gemv;

// ---- activation preparation: once per call, not per CTA ------------------------------------
// Writes x as fp16 in the operand order of the inner product with its per-step table (prep.cuh).
// The act-order column gather and the run-time input scale are applied here.  One half warp per
// (row m, 128-column step), eight columns per thread.
template <typename T>
__global__ void __launch_bounds__(128) w4a16_prep_kernel(const GemvParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int item = (blockIdx.x * 128 + threadIdx.x) >> 4;   // (row, step)
  const int c = threadIdx.x & 15;
  const int steps = p.K >> 7;
  const bool live = item < p.M * steps;
  const int m = live ? item / steps : 0, st = live ? item - m * steps : 0;
  const T* xg = reinterpret_cast<const T*>(p.x);
  const int k = st * 128 + c * 8;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
    if (p.col_perm == nullptr && p.x_vec_ok) {
      const uint4 raw = *reinterpret_cast<const uint4*>(xg + (size_t)m * p.ldx + k);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = to_float<T>(e[i]);
      if (p.input_scale) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = to_float<T>(from_float<T>(__fdiv_rn(v[i], __ldg(p.input_scale + k + i))));   // quotient rounded to the activation type, in every kernel
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int src = p.col_perm ? __ldg(p.col_perm + k + i) : k + i;
        v[i] = to_float<T>(xg[(size_t)m * p.ldx + src]);
        if (p.input_scale) v[i] = to_float<T>(from_float<T>(__fdiv_rn(v[i], __ldg(p.input_scale + src))));
      }
    }
  }
  prep_store_step<T>(v, live, reinterpret_cast<__half*>(p.xp) + (size_t)m * p.K + st * 128, c,
                     p.tabg + (size_t)st * kTabCols + m);
}

// RB = 16-row blocks per CTA (every warp takes all of them over its share of K: the activation
// fragments are read once per step for all RB blocks, and the per-warp prologue / epilogue is paid
// once for RB times the work).
// PROD: the activations are computed by this kernel (stage.cuh, M <= 4) instead of copied from a prepared buffer.
template <typename T, int MB, int WARPS, bool META16, int RB, bool PROD>
__global__ void __launch_bounds__(WARPS * 32) w4a16_gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int MP = 8 * MB;
  constexpr int THREADS = WARPS * 32;
  constexpr int kTileRows = 16 * RB;
  constexpr int kSteps = kMaxStepsPerWarp / RB;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int steps_total = p.K >> 7;
  const int st0 = blockIdx.y * p.steps_per_split;
  const int nst = min(p.steps_per_split, steps_total - st0);  // 128-column steps of this CTA (even)
  const int k0 = st0 << 7;
  const int row0 = blockIdx.x * kTileRows;
  const int spg = p.steps_per_group;

  // ---- shared memory carve-up ----
  const int seg_bytes = nst * 64;        // one row's codes for this K range
  const int pitch = seg_bytes + 64;      // == 64 (mod 128): adjacent rows land in different bank halves
  const int xrows = min(p.M, MP);
  const int xstride = nst * 256 + 64;    // bytes per activation row; == 64 (mod 128)
  unsigned char* wt = smem;
  unsigned char* xs = wt + kTileRows * pitch;
  float4* tab = reinterpret_cast<float4*>(xs + (size_t)xrows * xstride);           // [nst][kTabCols] (E, SX, g, -)
  const int mcols = (xrows + 1) & ~1;   // table columns kept in shared memory: activation rows in use, rounded up to a pair
  float* red = reinterpret_cast<float*>(tab + (size_t)nst * mcols);                // [WARPS][RB][MB][32][4]
  uint32_t* zero_blk = reinterpret_cast<uint32_t*>(red + WARPS * RB * MB * 128);   // 256 zero bytes
  uint64_t* bar_ptr = reinterpret_cast<uint64_t*>(zero_blk + 64);
  const uint32_t bar = smem_u32(bar_ptr);
  const uint32_t wt_u32 = smem_u32(wt), xs_u32 = smem_u32(xs), tab_u32 = smem_u32(tab);
  int* status = p.counters ? p.counters + kStatusIndex : nullptr;

  // ---- this warp's share of the K range ----
  const int spw = (nst + WARPS - 1) / WARPS;
  const int ws = warp * spw;
  const int nsw = max(0, min(nst, ws + spw) - ws);   // <= kSteps (host guarantees)

  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 64) zero_blk[threadIdx.x] = 0u;
  __syncthreads();

  // ---- weights: one contiguous bulk copy per row, all on one mbarrier (independent of the previous kernel) ----
  if (warp == 0) {
    if (lane == 0) mbar_expect_tx(bar, kTileRows * seg_bytes);
    __syncwarp();
    if (lane < kTileRows) {
      const int r = min(row0 + lane, p.N - 1);
      bulk_load(wt_u32 + lane * pitch, p.packed + (size_t)r * (p.K >> 1) + (k0 >> 1), seg_bytes, bar);
    }
  }
  // ---- scale / zero of this warp's steps, rows gid and gid + 8, straight into registers ----
  float ms[kSteps][RB][2], mz[kSteps][RB][2];
#pragma unroll
  for (int j = 0; j < kSteps; ++j) {
    if (j < nsw) {
      const int g = spg == 1 ? st0 + ws + j : (st0 + ws + j) / spg;   // group_size 128: no division
#pragma unroll
      for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const size_t idx = (size_t)min(row0 + rb * 16 + gid + 8 * h, p.N - 1) * p.ngroups + g;
          if (META16) {
            const uint32_t v = __ldg(p.meta_h2 + idx);
            const __half2 hv = *reinterpret_cast<const __half2*>(&v);
            ms[j][rb][h] = __low2float(hv);
            mz[j][rb][h] = __high2float(hv);
          } else {
            ms[j][rb][h] = __ldg(p.scale + idx);
            mz[j][rb][h] = __ldg(p.zero + idx);
          }
        }
    }
  }

  // staging threads per 128-column step: THREADS / 16 half warps, so K <= 4096 takes 4096 / (8 THREADS) rounds
  constexpr int kRounds = WARPS == 8 ? 2 : 4;
  uint4 norm_w[kRounds];
  if constexpr (PROD) stage_prefetch_norm<T, kRounds>(p, nst, threadIdx.x, THREADS, norm_w);
  pdl_launch_dependents();
  pdl_wait();  // from here on the previous kernel's output (x) is visible

  // ---- activations arrive in operand order with their per-step sums (prepared once per call by
  // w4a16_prep_kernel or by the kernel that computed them): straight 16-byte copies into shared
  // memory; or this CTA computes them itself (stage.cuh) ----
  if constexpr (PROD) {
    stage_produce<T, kRounds>(p, st0, nst, xs, xstride, tab, mcols, threadIdx.x, THREADS, red, blockIdx.x == 0 && blockIdx.y == 0,
                              norm_w, [] { __syncthreads(); });
  } else {
    const int vec_per_row = nst * 16;  // 256 bytes per step
    const unsigned char* xp = reinterpret_cast<const unsigned char*>(p.xp);
    for (int m = 0; m < xrows; ++m) {
      const uint4* src = reinterpret_cast<const uint4*>(xp + ((size_t)m * p.K + k0) * 2);
      for (int v = threadIdx.x; v < vec_per_row; v += THREADS) sts_v4(xs_u32 + m * xstride + v * 16, __ldcg(src + v));
    }
    const uint4* tg = reinterpret_cast<const uint4*>(p.tabg + (size_t)st0 * kTabCols);
    // only the table columns of activation rows in use; threads whose rows are beyond them read
    // whatever follows (always inside this CTA's shared memory) and their results are discarded
    for (int i = threadIdx.x; i < nst * mcols; i += THREADS) {
      const int st = i / mcols, c = i - st * mcols;
      sts_v4(tab_u32 + i * 16, __ldcg(tg + st * kTabCols + c));
    }
  }
  __syncthreads();
  mbar_wait(bar, 0, status);

  // ---- main loop over this warp's steps ----
  float yacc[RB][MB][4];
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 4; ++i) yacc[rb][mb][i] = 0.f;
  {
    const uint32_t wa_addr = wt_u32 + gid * pitch + ws * 64 + tig * 16;
    const uint32_t tab_addr = tab_u32 + ws * (mcols * 16) + tig * 32;
    uint32_t xaddr[MB], xstep[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      const int m = mb * 8 + gid;
      // columns beyond M read a block of zeros that does not advance with the step
      xaddr[mb] = (m < p.M ? xs_u32 + m * xstride + ws * 256 : smem_u32(zero_blk)) + tig * 16;
      xstep[mb] = m < p.M ? 256u : 0u;
    }
#pragma unroll
    for (int j = 0; j < kSteps; ++j) {
      if (j < nsw) {
        uint4 xb[MB][4];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
          for (int i = 0; i < 4; ++i) xb[mb][i] = lds_v4(xaddr[mb] + j * xstep[mb] + i * 64);
        float4 t0[MB], t1[MB];   // (E, SX, g, -) of activation rows mb*8 + 2 tig and + 1
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          t0[mb] = lds_v4f(tab_addr + j * (mcols * 16) + mb * 128);
          t1[mb] = lds_v4f(tab_addr + j * (mcols * 16) + mb * 128 + 16);
        }
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
          const uint4 wa4 = lds_v4(wa_addr + rb * 16 * pitch + j * 64);
          const uint4 wb4 = lds_v4(wa_addr + (rb * 16 + 8) * pitch + j * 64);
          const uint32_t wa[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
          const uint32_t wb[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
          float d0[MB][4], d1[MB][4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t pa[4], pb[4];
            Nibbles<__half>::unpack(wa[i], pa);
            Nibbles<__half>::unpack(wb[i], pb);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              if (i == 0) {
                mma16816_zero<__half>(d0[mb], pa[0], pb[0], pa[1], pb[1], xb[mb][i].x, xb[mb][i].y);
                mma16816_zero<__half>(d1[mb], pa[2], pb[2], pa[3], pb[3], xb[mb][i].z, xb[mb][i].w);
              } else {
                mma16816<__half>(d0[mb], pa[0], pb[0], pa[1], pb[1], xb[mb][i].x, xb[mb][i].y);
                mma16816<__half>(d1[mb], pa[2], pb[2], pa[3], pb[3], xb[mb][i].z, xb[mb][i].w);
              }
            }
          }
          // fold this step with its group's scale / zero (linear, so folding per step is exact for any group size)
          const float sA = ms[j][rb][0], zA = mz[j][rb][0], sB = ms[j][rb][1], zB = mz[j][rb][1];
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            yacc[rb][mb][0] = fmaf(sA * t0[mb].z, fmaf(-zA, t0[mb].y, (d0[mb][0] + d1[mb][0]) - t0[mb].x), yacc[rb][mb][0]);
            yacc[rb][mb][1] = fmaf(sA * t1[mb].z, fmaf(-zA, t1[mb].y, (d0[mb][1] + d1[mb][1]) - t1[mb].x), yacc[rb][mb][1]);
            yacc[rb][mb][2] = fmaf(sB * t0[mb].z, fmaf(-zB, t0[mb].y, (d0[mb][2] + d1[mb][2]) - t0[mb].x), yacc[rb][mb][2]);
            yacc[rb][mb][3] = fmaf(sB * t1[mb].z, fmaf(-zB, t1[mb].y, (d0[mb][3] + d1[mb][3]) - t1[mb].x), yacc[rb][mb][3]);
          }
        }
      }
    }
  }

  // ---- the warps' partial sums meet in shared memory ----
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
      sts_v4f(smem_u32(red) + (((warp * RB + rb) * MB + mb) * 32 + lane) * 16, yacc[rb][mb][0], yacc[rb][mb][1],
              yacc[rb][mb][2], yacc[rb][mb][3]);
  __syncthreads();

  T* yg = reinterpret_cast<T*>(p.y);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  float* part = p.splits > 1 ? p.partial + (size_t)blockIdx.y * p.M * p.N : nullptr;
  const bool peer = peer_on(p.peer);
  const uint32_t pe = peer ? peer_epoch(p.peer) : 0u;   // after the dependency wait above
  bool peer_timeout = false;
  if (threadIdx.x < 32 * MB * RB) {   // one warp per (row block, column block)
    const int rb = (threadIdx.x >> 5) / MB, mb = (threadIdx.x >> 5) % MB;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float4 v = lds_v4f(smem_u32(red) + (((w * RB + rb) * MB + mb) * 32 + lane) * 16);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    float out[4] = {acc.x, acc.y, acc.z, acc.w};
    if (peer && !part) {   // the ranks' partial outputs meet here: send all four, then collect them
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = row0 + rb * 16 + gid + 8 * (i >> 1), m = mb * 8 + tig * 2 + (i & 1);
        if (n < p.N && m < p.M) peer_send(p.peer, pe, (size_t)m * p.N + n, out[i] + (bias ? to_float<T>(bias[n]) : 0.f));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = row0 + rb * 16 + gid + 8 * (i >> 1), m = mb * 8 + tig * 2 + (i & 1);
        if (n < p.N && m < p.M) yg[(size_t)m * p.ldy + n] = from_float<T>(peer_recv(p.peer, pe, (size_t)m * p.N + n, peer_timeout));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = row0 + rb * 16 + gid + 8 * (i >> 1);
        const int m = mb * 8 + tig * 2 + (i & 1);
        if (n < p.N && m < p.M) {
          if (part) {
            __stcg(part + (size_t)m * p.N + n, out[i]);
          } else {
            float v = out[i];
            if (bias) v += to_float<T>(bias[n]);
            yg[(size_t)m * p.ldy + n] = from_float<T>(v);
          }
        }
      }
    }
  }
  if (p.splits == 1) {
    if (peer) {   // one exchanging unit per row tile
      const int any_timeout = __syncthreads_or(peer_timeout);
      if (threadIdx.x == 0) peer_unit_done(p.peer, pe, gridDim.x, any_timeout != 0);
    }
    return;
  }

  // ---- K spans several CTAs: the last one to arrive adds the partial sums in split order ----
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counters + blockIdx.x, 1) == p.splits - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int tile_rows = min(kTileRows, p.N - row0);
  for (int idx = threadIdx.x; idx < tile_rows * p.M; idx += THREADS) {
    const int m = idx / tile_rows, n = row0 + (idx - m * tile_rows);
    float v = 0.f;
    for (int s = 0; s < p.splits; ++s) v += __ldcg(p.partial + ((size_t)s * p.M + m) * p.N + n);
    if (bias) v += to_float<T>(bias[n]);
    if (peer) peer_send(p.peer, pe, (size_t)m * p.N + n, v);
    else yg[(size_t)m * p.ldy + n] = from_float<T>(v);
  }
  if (peer) {
    for (int idx = threadIdx.x; idx < tile_rows * p.M; idx += THREADS) {
      const int m = idx / tile_rows, n = row0 + (idx - m * tile_rows);
      yg[(size_t)m * p.ldy + n] = from_float<T>(peer_recv(p.peer, pe, (size_t)m * p.N + n, peer_timeout));
    }
    const int any_timeout = __syncthreads_or(peer_timeout);
    if (threadIdx.x == 0) peer_unit_done(p.peer, pe, gridDim.x, any_timeout != 0);
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;  // leave the workspace ready for the next call
}

// ---- any-shape fallback: one thread per output, used when K is not a multiple of 256 or the
// group size not a multiple of 128 (tiny layers); correctness path, not a performance path ----
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

struct Plan {
  bool fast;
  int warps, rb, splits, steps_per_split;
  size_t smem;
};

constexpr size_t kSmemCap = 110 * 1024;

size_t gemv_smem(int M, int MB, int nst, int warps, int rb) {
  const int xrows = M < 8 * MB ? M : 8 * MB;
  return (size_t)16 * rb * (nst * 64 + 64) + (size_t)xrows * (nst * 256 + 64) + (size_t)nst * ((xrows + 1) & ~1) * sizeof(float4) +
         (size_t)warps * rb * MB * 128 * sizeof(float) + 256 + 16 + 128;
}


Plan make_plan_rb(int M, int N, int K, int G, int rb_request);

Plan make_plan(int M, int N, int K, int G) {
  Plan pl = make_plan_rb(M, N, K, G, 0);
  if (pl.fast && pl.rb == 2 && pl.smem > kSmemCap) pl = make_plan_rb(M, N, K, G, 1);  // tile too large with 32 rows
  return pl;
}

Plan make_plan_rb(int M, int N, int K, int G, int rb_request) {
  Plan pl{};
  const int kSmCount = sm_count();
  pl.fast = (K % 256 == 0) && (G % 128 == 0);  // K ranges are cut in multiples of 256 columns (an even number of steps)
  if (!pl.fast) return pl;
  const int MB = M <= 8 ? 1 : 2;
  const int chunks = K / 256;
  // two 16-row blocks per CTA when that still leaves at least two CTAs per SM (big layers): half the
  // per-warp overhead per weight.  Small layers keep 16-row CTAs for parallelism.
  int rb = rb_request ? rb_request : (((N + 31) / 32 >= 2 * kSmCount && MB == 1) ? 2 : 1);
  if (rb != 1 && rb != 2) rb = 1;
  const int row_tiles = (N + 16 * rb - 1) / (16 * rb);
  // columns per CTA: bounded by the activation tile that must sit in shared memory beside the weights
  int kc = M <= 4 ? 4096 : (M <= 8 ? 2048 : 1024);
  // very small layers only: cut K further until there is at least one CTA per SM (going through the
  // global split-K reduction costs more latency than it buys otherwise)
  while (kc > 512 && (long long)row_tiles * ((K + kc - 1) / kc) < kSmCount) kc >>= 1;
  int cps = kc / 256;                     // 256-column chunks per CTA
  if (cps < 1) cps = 1;
  if (cps > chunks) cps = chunks;
  int splits = (chunks + cps - 1) / cps;
  cps = (chunks + splits - 1) / splits;   // balance the splits
  if (splits > 64) {
    splits = 64;
    cps = (chunks + 63) / 64;
  }
  splits = (chunks + cps - 1) / cps;
  const int nst = cps * 2;
  const int max_steps = kMaxStepsPerWarp / rb;
  // enough CTAs to fill the machine three times over: fewer, longer warps (less per-warp overhead);
  // otherwise more warps per CTA to shorten each CTA's critical path
  int warps = (nst >= 16 && (long long)row_tiles * splits < 3 * kSmCount) ? 8 : 4;
  if ((nst + warps - 1) / warps > max_steps || rb == 2) warps = 8;
  pl.warps = warps;
  pl.rb = rb;
  pl.splits = splits;
  pl.steps_per_split = nst;
  pl.smem = gemv_smem(M, MB, nst, warps, rb);
  return pl;
}

template <typename T, int MB, int WARPS, bool META16, int RB, bool PROD = false>
int launch_gemv(const GemvParams& p, const Plan& pl, cudaStream_t stream) {
  auto kern = w4a16_gemv_kernel<T, MB, WARPS, META16, RB, PROD>;
  // the shared-memory opt-in once per instantiation and device (a function-local static per template
  // instantiation, guarded by a mutex: the entry points may be called from several host threads)
  static std::mutex mu;
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PARE_ERR_CUDA;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_done[dev]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemCap) != cudaSuccess)
        return PARE_ERR_CUDA;
      attr_done[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + 16 * RB - 1) / (16 * RB), pl.splits, 1);
  cfg.blockDim = dim3(WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return PARE_ERR_CUDA;
  return PARE_OK;
}

template <typename T, int MB>
int dispatch_warps(const GemvParams& p, const Plan& pl, cudaStream_t stream) {
  const bool m16 = p.meta_h2 != nullptr;
  if constexpr (MB == 1) {
    if (p.producer) {   // M <= 4
      if (pl.rb == 2) return m16 ? launch_gemv<T, 1, 8, true, 2, true>(p, pl, stream) : launch_gemv<T, 1, 8, false, 2, true>(p, pl, stream);
      if (pl.warps == 8) return m16 ? launch_gemv<T, 1, 8, true, 1, true>(p, pl, stream) : launch_gemv<T, 1, 8, false, 1, true>(p, pl, stream);
      return m16 ? launch_gemv<T, 1, 4, true, 1, true>(p, pl, stream) : launch_gemv<T, 1, 4, false, 1, true>(p, pl, stream);
    }
  }
  if (p.producer) return PARE_ERR_UNSUPPORTED;
  if (MB == 1 && pl.rb == 2)   // 32-row CTAs always run 8 warps (4 steps x 2 row blocks per warp)
    return m16 ? launch_gemv<T, 1, 8, true, 2>(p, pl, stream) : launch_gemv<T, 1, 8, false, 2>(p, pl, stream);
  if (pl.warps == 8)
    return m16 ? launch_gemv<T, MB, 8, true, 1>(p, pl, stream) : launch_gemv<T, MB, 8, false, 1>(p, pl, stream);
  return m16 ? launch_gemv<T, MB, 4, true, 1>(p, pl, stream) : launch_gemv<T, MB, 4, false, 1>(p, pl, stream);
}

template <typename T>
int dispatch_gemv(const GemvParams& p, const Plan& pl, cudaStream_t stream) {
  return p.M <= 8 ? dispatch_warps<T, 1>(p, pl, stream) : dispatch_warps<T, 2>(p, pl, stream);
}

template <typename T>
int launch_generic(const GemvParams& p, const uint8_t* packed, int G, cudaStream_t stream) {
  const int64_t total = (int64_t)p.M * p.N;
  const int threads = 128;
  w4a16_generic_kernel<T><<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(p, packed, G);
  return launch_status();
}

}  // namespace

bool gemv_persist_supported(int M, int N, int K, int G, bool producer = false);
size_t gemv_persist_partial_floats(int M, int N, int K);
int gemv_persist_launch(const gemv::GemvParams& p, int x_dtype, cudaStream_t stream);

size_t prep_bytes(int M, int K) {  // prepared activations + step table, each rounded to 256 bytes
  const size_t xp = ((size_t)M * K * 2 + 255) / 256 * 256;
  const size_t tab = ((size_t)(K / 128 + 1) * kTabCols * sizeof(float4) + 255) / 256 * 256;
  return xp + tab;
}

size_t gemv_workspace_bytes(int M, int N, int K, int G) {
  const int m = M < 16 ? M : 16;
  size_t splits = 1;
  if (K % 256 == 0 && G % 128 == 0) splits = (size_t)(K / 256);  // upper bound on any plan
  if (splits > 64) splits = 64;
  // split-K partial sums of either schedule (the persistent one adds at most one 32-row block per SM)
  return kCounterBytes + prep_bytes(m, K) + (splits * (size_t)m * N + (size_t)sm_count() * 32 * m) * sizeof(float);
}

// Called by pare_w4a16_forward for every chunk of at most 16 activation rows.
int gemv_forward(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale,
                 const float* zero, const void* meta_h2, const int32_t* col_perm, const float* input_scale,
                 const void* bias, void* y, int64_t ldy, int M, int N, int K, int G, void* workspace,
                 size_t workspace_bytes, cudaStream_t stream, const void* prepared, const ProducerArgs* prod,
                 const PeerCtx* peer) {
  GemvParams p{};
  p.x = x;
  p.ldx = ldx;
  p.packed = packed;
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
  p.x_vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (ldx % 8) == 0) ? 1 : 0;

  Plan pl = make_plan(M, N, K, G);
  if (prepared) PARE_REQUIRE(pl.fast && col_perm == nullptr && input_scale == nullptr && aligned16(prepared), PARE_ERR_UNSUPPORTED);
  if (prod) {
    PARE_REQUIRE(pl.fast && col_perm == nullptr && input_scale == nullptr && prepared == nullptr && M <= 4, PARE_ERR_UNSUPPORTED);
    p.producer = prod->kind;
    p.pa = prod->a; p.pb = prod->b; p.pc = prod->c; p.resid_out = prod->resid_out; p.lda = prod->lda; p.eps = prod->eps;
  }
  if (peer) {   // the ranks' partial outputs are added in the epilogue: streaming kernels only, one fp32 unit per output
    PARE_REQUIRE(pl.fast, PARE_ERR_UNSUPPORTED);
    PARE_REQUIRE((size_t)M * N * 8 <= peer->slot_bytes, PARE_ERR_WORKSPACE);
    p.peer = *peer;
  }
  if (!pl.fast) {
    return x_dtype == PARE_F16 ? launch_generic<__half>(p, packed, G, stream)
                               : launch_generic<__nv_bfloat16>(p, packed, G, stream);
  }
  PARE_REQUIRE(aligned16(packed), PARE_ERR_ALIGN);
  PARE_REQUIRE((size_t)(N + 15) / 16 < kStatusIndex, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(pl.smem <= kSmemCap, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE((pl.steps_per_split + pl.warps - 1) / pl.warps <= kMaxStepsPerWarp / pl.rb, PARE_ERR_UNSUPPORTED);
  p.splits = pl.splits;
  p.steps_per_split = pl.steps_per_split;
  const bool persist = gemv_persist_supported(M, N, K, G, prod != nullptr);
  const size_t need = kCounterBytes + prep_bytes(M, K) +
                      (persist ? gemv_persist_partial_floats(M, N, K) * sizeof(float)
                               : (pl.splits > 1 ? (size_t)pl.splits * M * N * sizeof(float) : 0));
  PARE_REQUIRE(workspace != nullptr && workspace_bytes >= need, PARE_ERR_WORKSPACE);
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  p.counters = reinterpret_cast<int*>(ws);
  p.xp = ws + kCounterBytes;
  p.tabg = reinterpret_cast<float4*>(ws + kCounterBytes + ((size_t)M * K * 2 + 255) / 256 * 256);
  p.partial = reinterpret_cast<float*>(ws + kCounterBytes + prep_bytes(M, K));

  if (prepared) {   // the producer of the activations already wrote them in operand order
    p.xp = const_cast<void*>(prepared);
    p.tabg = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(p.xp) + prepared_tab_offset(M, K));
  }
  if (prod) {
    // RMSNorm needs the whole row in one CTA, and few enough steps per half warp of the staging threads
    if (persist) {
      PARE_REQUIRE(prod->kind != PARE_PRODUCER_RMSNORM || K <= 4096, PARE_ERR_UNSUPPORTED);
    } else {
      PARE_REQUIRE(prod->kind != PARE_PRODUCER_RMSNORM || (pl.splits == 1 && K <= 4096),
                   PARE_ERR_UNSUPPORTED);
    }
  }
  // 1) activations into operand order (one warp per row and 128-column step)
  if (!prepared && !prod) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((M * (K / 128) + 7) / 8, 1, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = x_dtype == PARE_F16 ? cudaLaunchKernelEx(&cfg, w4a16_prep_kernel<__half>, p)
                                              : cudaLaunchKernelEx(&cfg, w4a16_prep_kernel<__nv_bfloat16>, p);
    if (e != cudaSuccess) return PARE_ERR_CUDA;
  }
  // 2) the streaming kernel: persistent schedule for large layers at M <= 4, one tile per CTA otherwise
  if (persist) return gemv_persist_launch(p, x_dtype, stream);
  return x_dtype == PARE_F16 ? dispatch_gemv<__half>(p, pl, stream) : dispatch_gemv<__nv_bfloat16>(p, pl, stream);
}

// Activation prep alone, into a caller-owned prepared buffer (prepared_bytes(M, K) bytes).
int gemv_prepare(const void* x, int x_dtype, int64_t ldx, const int32_t* col_perm, const float* input_scale, int M, int K,
                 void* prepared, cudaStream_t stream) {
  PARE_REQUIRE(M > 0 && M <= kTabCols && K > 0 && K % 128 == 0 && aligned16(prepared), PARE_ERR_UNSUPPORTED);
  GemvParams p{};
  p.x = x;
  p.ldx = ldx;
  p.col_perm = col_perm;
  p.input_scale = input_scale;
  p.M = M;
  p.K = K;
  p.x_vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (ldx % 8) == 0) ? 1 : 0;
  p.xp = prepared;
  p.tabg = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(prepared) + prepared_tab_offset(M, K));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((M * (K / 128) + 7) / 8, 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = x_dtype == PARE_F16 ? cudaLaunchKernelEx(&cfg, w4a16_prep_kernel<__half>, p)
                                            : cudaLaunchKernelEx(&cfg, w4a16_prep_kernel<__nv_bfloat16>, p);
  return e == cudaSuccess ? PARE_OK : PARE_ERR_CUDA;
}

}  // namespace pare
