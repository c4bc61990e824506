// Persistent variant of the W4A16 streaming dequant-GEMV for large layers at M <= 4, sm_100a.
//
// Same arithmetic and data layout as w4a16_gemv.cu (see there).  What changes is the schedule:
// one CTA per SM stays resident and walks over tiles of 32 output rows x this CTA's K range, so
//   * activations and their per-step table are staged in shared memory ONCE per CTA, not per tile;
//   * a producer warp keeps the next tile's weights in flight (two-slot ring of row-contiguous
//     bulk async copies, full / empty mbarriers) while the eight consumer warps work on the
//     current one, so loading and computing overlap instead of alternating;
//   * each consumer warp owns a fixed 1/8 of the K range for both 16-row blocks of the tile;
//     scale / zero of the next tile are fetched into the registers the current tile has just
//     finished with.
// The eight partial sums of a tile meet in shared memory (double-buffered, one named barrier per
// tile); warps 0 and 1 write the outputs.  With a K split the same two warps run the
// last-arriver reduction through the workspace.  All mbarrier waits are bounded.

#include "gemv_common.cuh"

namespace pare {
namespace {

using namespace gemv;

constexpr int kDepth = 2;              // ring slots
constexpr int kRowsPerTile = 32;
constexpr int kMaxSteps = 32;          // K range per CTA <= 4096 columns

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ bool wait_or_die(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  if (dead) return false;
  if (mbar_wait(bar, parity, status)) return true;
  dead = true;
  return false;
}

// kCW consumer warps, each with kMaxSteps / kCW 128-column steps of the K range.
template <typename T, bool META16, int kCW>
__global__ void __launch_bounds__((kCW + 1) * 32, 1) w4a16_gemv_persist_kernel(const GemvParams p, int n_tiles) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int kStepsPW = kMaxSteps / kCW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int steps_total = p.K >> 7;
  const int st0 = blockIdx.y * p.steps_per_split;
  const int nst = min(p.steps_per_split, steps_total - st0);   // multiple of 4, <= 32
  const int k0 = st0 << 7;
  const int spg = p.steps_per_group;

  const int seg_bytes = nst * 64;
  const int pitch = seg_bytes + 64;          // == 64 (mod 128)
  const int xstride = nst * 256 + 64;
  unsigned char* ring = smem;                                                     // [kDepth][32][pitch]
  unsigned char* xs = ring + kDepth * kRowsPerTile * pitch;                       // [M][xstride]
  float2* tab = reinterpret_cast<float2*>(xs + (size_t)p.M * xstride);            // [nst][kTabCols]
  float* red = reinterpret_cast<float*>(tab + (size_t)nst * kTabCols);            // [2][kCW][2][32][4]
  uint32_t* zero_blk = reinterpret_cast<uint32_t*>(red + 2 * kCW * 2 * 128);      // 256 zero bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(zero_blk + 64);                    // full[2], empty[2]
  int* s_flag = reinterpret_cast<int*>(bars + 2 * kDepth);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kDepth);
  const uint32_t ring_u32 = smem_u32(ring), xs_u32 = smem_u32(xs), tab_u32 = smem_u32(tab), red_u32 = smem_u32(red);
  int* status = p.counters ? p.counters + kStatusIndex : nullptr;
  bool dead = false;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kDepth; ++i) {
      mbar_init(full0 + i * 8, 1);
      mbar_init(empty0 + i * 8, kCW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 64) zero_blk[threadIdx.x] = 0u;
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kCW) {
    // ================= producer: weights never depend on the previous kernel =================
    int i = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i) {
      const int slot = i & 1;
      wait_or_die(empty0 + slot * 8, ((i >> 1) & 1) ^ 1, status, dead);
      if (lane == 0) mbar_expect_tx(full0 + slot * 8, kRowsPerTile * seg_bytes);
      __syncwarp();
      const int r = t * kRowsPerTile + lane;
      bulk_load(ring_u32 + (slot * kRowsPerTile + lane) * pitch, p.packed + (size_t)r * (p.K >> 1) + (k0 >> 1), seg_bytes,
                full0 + slot * 8);
    }
    return;
  }

  // ================= consumers =================
  const int spw = (nst + kCW - 1) / kCW;     // <= kStepsPW
  const int ws = warp * spw;
  const int nsw = max(0, min(nst, ws + spw) - ws);   // kStepsPW or 0 (host guarantees whole shares)
  // scale / zero of this warp's kStepsPW consecutive groups for rows (rb*16 + gid + 8h) of a tile: one
  // vector load per row and array; the pointers advance by a constant stride from tile to tile
  float ms[kStepsPW][2][2], mz[kStepsPW][2][2];
  const size_t tile_stride = (size_t)gridDim.x * kRowsPerTile * p.ngroups;
  size_t meta_idx[2][2];
#pragma unroll
  for (int rb = 0; rb < 2; ++rb)
#pragma unroll
    for (int h = 0; h < 2; ++h)
      meta_idx[rb][h] = (size_t)(blockIdx.x * kRowsPerTile + rb * 16 + gid + 8 * h) * p.ngroups + st0 + ws;
  auto load_meta = [&]() {
#pragma unroll
    for (int rb = 0; rb < 2; ++rb)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (META16) {
          uint32_t v[kStepsPW];
          if (kStepsPW == 2) {
            const uint2 t2 = __ldg(reinterpret_cast<const uint2*>(p.meta_h2 + meta_idx[rb][h]));
            v[0] = t2.x;
            v[1] = t2.y;
          } else {
            const uint4 t4 = __ldg(reinterpret_cast<const uint4*>(p.meta_h2 + meta_idx[rb][h]));
            v[0] = t4.x; v[1] = t4.y; v[2 % kStepsPW] = t4.z; v[3 % kStepsPW] = t4.w;
          }
#pragma unroll
          for (int j = 0; j < kStepsPW; ++j) {
            const __half2 hv = *reinterpret_cast<const __half2*>(&v[j]);
            ms[j][rb][h] = __low2float(hv);
            mz[j][rb][h] = __high2float(hv);
          }
        } else if (kStepsPW == 2) {
          const float2 a = __ldg(reinterpret_cast<const float2*>(p.scale + meta_idx[rb][h]));
          const float2 b = __ldg(reinterpret_cast<const float2*>(p.zero + meta_idx[rb][h]));
          ms[0][rb][h] = a.x; ms[1][rb][h] = a.y;
          mz[0][rb][h] = b.x; mz[1][rb][h] = b.y;
        } else {
          const float4 a = __ldg(reinterpret_cast<const float4*>(p.scale + meta_idx[rb][h]));
          const float4 b = __ldg(reinterpret_cast<const float4*>(p.zero + meta_idx[rb][h]));
          ms[0][rb][h] = a.x; ms[1][rb][h] = a.y; ms[2 % kStepsPW][rb][h] = a.z; ms[3 % kStepsPW][rb][h] = a.w;
          mz[0][rb][h] = b.x; mz[1][rb][h] = b.y; mz[2 % kStepsPW][rb][h] = b.z; mz[3 % kStepsPW][rb][h] = b.w;
        }
        meta_idx[rb][h] += tile_stride;
      }
  };
  if (nsw == kStepsPW) load_meta();   // first tile (blockIdx.x < n_tiles by construction of the grid)

  pdl_wait();  // the activations are the previous kernel's output
  {
    const int vec_per_row = nst * 16;
    const unsigned char* xp = reinterpret_cast<const unsigned char*>(p.xp);
    for (int m = 0; m < p.M; ++m) {
      const uint4* src = reinterpret_cast<const uint4*>(xp + ((size_t)m * p.K + k0) * 2);
      for (int v = threadIdx.x; v < vec_per_row; v += kCW * 32) sts_v4(xs_u32 + m * xstride + v * 16, __ldcg(src + v));
    }
    const uint4* tg = reinterpret_cast<const uint4*>(p.tabg + (size_t)st0 * kTabCols);
    for (int i = threadIdx.x; i < nst * (kTabCols / 2); i += kCW * 32) sts_v4(tab_u32 + i * 16, __ldcg(tg + i));
  }
  named_sync(1, kCW * 32);

  // Offsets into the shared array (plain C++ loads from it compile to ld.shared and, unlike asm, leave
  // the compiler free to software-pipeline the eight independent (step, row block) units of a tile).
  const int w_off = gid * pitch + ws * 64 + tig * 16;
  const int tab_off = (int)(reinterpret_cast<unsigned char*>(tab) - smem) + ws * (kTabCols * 8) + tig * 16;
  const int x_off = (gid < p.M ? (int)(xs - smem) + gid * xstride + ws * 256
                               : (int)(reinterpret_cast<unsigned char*>(zero_blk) - smem)) + tig * 16;
  const int xstep = gid < p.M ? 256 : 0;
  T* yg = reinterpret_cast<T*>(p.y);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  float* part = p.splits > 1 ? p.partial + (size_t)blockIdx.y * p.M * p.N : nullptr;

  int i = 0, par = 0;
  for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++i, par ^= 1) {
    const int slot = i & 1;
    wait_or_die(full0 + slot * 8, (i >> 1) & 1, status, dead);
    const unsigned char* stage = smem + slot * kRowsPerTile * pitch + w_off;
    float yacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (nsw == kStepsPW) {   // warp-uniform; one basic block for the whole tile
#pragma unroll
      for (int j = 0; j < kStepsPW; ++j) {
        uint4 xb[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) xb[q] = *reinterpret_cast<const uint4*>(smem + x_off + j * xstep + q * 64);
        const float4 tt = *reinterpret_cast<const float4*>(smem + tab_off + j * (kTabCols * 8));  // E0 SX0 E1 SX1
#pragma unroll
        for (int rb = 0; rb < 2; ++rb) {
          const uint4 wa4 = *reinterpret_cast<const uint4*>(stage + rb * 16 * pitch + j * 64);
          const uint4 wb4 = *reinterpret_cast<const uint4*>(stage + (rb * 16 + 8) * pitch + j * 64);
          const uint32_t wa[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
          const uint32_t wb[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
          float d0[4], d1[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t pa[4], pb[4];
            Nibbles<T>::unpack(wa[q], pa);
            Nibbles<T>::unpack(wb[q], pb);
            if (q == 0) {
              mma16816_zero<T>(d0, pa[0], pb[0], pa[1], pb[1], xb[q].x, xb[q].y);
              mma16816_zero<T>(d1, pa[2], pb[2], pa[3], pb[3], xb[q].z, xb[q].w);
            } else {
              mma16816<T>(d0, pa[0], pb[0], pa[1], pb[1], xb[q].x, xb[q].y);
              mma16816<T>(d1, pa[2], pb[2], pa[3], pb[3], xb[q].z, xb[q].w);
            }
          }
          const float sA = ms[j][rb][0], zA = mz[j][rb][0], sB = ms[j][rb][1], zB = mz[j][rb][1];
          yacc[rb][0] = fmaf(sA, fmaf(-zA, tt.y, (d0[0] + d1[0]) - tt.x), yacc[rb][0]);
          yacc[rb][1] = fmaf(sA, fmaf(-zA, tt.w, (d0[1] + d1[1]) - tt.z), yacc[rb][1]);
          yacc[rb][2] = fmaf(sB, fmaf(-zB, tt.y, (d0[2] + d1[2]) - tt.x), yacc[rb][2]);
          yacc[rb][3] = fmaf(sB, fmaf(-zB, tt.w, (d0[3] + d1[3]) - tt.z), yacc[rb][3]);
        }
      }
      if (t + (int)gridDim.x < n_tiles) load_meta();   // the registers are free again: fetch the next tile's scale / zero
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + slot * 8);   // this warp has read all it needs from the slot

    // ---- the eight partial sums of the tile meet in shared memory (buffer `par`) ----
    const uint32_t red_base = red_u32 + par * (kCW * 2 * 32 * 16);
    sts_v4f(red_base + ((warp * 2 + 0) * 32 + lane) * 16, yacc[0][0], yacc[0][1], yacc[0][2], yacc[0][3]);
    sts_v4f(red_base + ((warp * 2 + 1) * 32 + lane) * 16, yacc[1][0], yacc[1][1], yacc[1][2], yacc[1][3]);
    named_sync(1, kCW * 32);
    if (warp < 2) {
      const int rb = warp;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < kCW; ++w) {
        const float4 v = lds_v4f(red_base + ((w * 2 + rb) * 32 + lane) * 16);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      const float out[4] = {acc.x, acc.y, acc.z, acc.w};
      const int row0 = t * kRowsPerTile;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int n = row0 + rb * 16 + gid + 8 * (q >> 1);
        const int m = tig * 2 + (q & 1);
        if (n < p.N && m < p.M) {
          if (part) {
            __stcg(part + (size_t)m * p.N + n, out[q]);
          } else {
            float v = out[q];
            if (bias) v += to_float<T>(bias[n]);
            yg[(size_t)m * p.ldy + n] = from_float<T>(v);
          }
        }
      }
      if (part) {
        // K spans several CTAs: the last one to arrive at this tile's counter adds the partial sums in split order
        __threadfence();
        named_sync(2, 64);
        if (threadIdx.x == 0) *s_flag = (atomicAdd(p.counters + t, 1) == p.splits - 1);
        named_sync(2, 64);
        if (*s_flag) {
          __threadfence();
          const int tile_rows = min(kRowsPerTile, p.N - row0);
          for (int idx = threadIdx.x; idx < tile_rows * p.M; idx += 64) {
            const int m = idx / tile_rows, n = row0 + (idx - m * tile_rows);
            float v = 0.f;
            for (int s = 0; s < p.splits; ++s) v += __ldcg(p.partial + ((size_t)s * p.M + m) * p.N + n);
            if (bias) v += to_float<T>(bias[n]);
            yg[(size_t)m * p.ldy + n] = from_float<T>(v);
          }
          if (threadIdx.x == 0) p.counters[t] = 0;
        }
        named_sync(2, 64);
      }
    }
  }
}

constexpr size_t kPersistSmemCap = 220 * 1024;

int g_persist_warps = 16;

size_t persist_smem(int M, int nst) {
  return (size_t)kDepth * kRowsPerTile * (nst * 64 + 64) + (size_t)M * (nst * 256 + 64) + (size_t)nst * kTabCols * sizeof(float2) +
         (size_t)2 * 16 * 2 * 128 * sizeof(float) + 256 + 2 * kDepth * 8 + 16 + 128;
}

}  // namespace

void gemv_persist_set_warps(int w) { g_persist_warps = (w == 8) ? 8 : 16; }

// Large layers at M <= 4 with 128-column groups aligned to the per-warp K shares.
bool gemv_persist_supported(int M, int N, int steps_per_split, int steps_per_group, int splits) {
  if (steps_per_group != 1) return false;                               // group size 128: a warp's groups are contiguous
  // every consumer warp's share must be whole: 4 steps with 8 warps, 2 with 16 (or empty)
  if (M > 4 || steps_per_split > kMaxSteps || (steps_per_split % 4) != 0 || steps_per_split <= 24) return false;
  if (N % kRowsPerTile) return false;                                   // whole tiles only: no row clamping in the loop
  // Fewer than two tiles per resident CTA leaves nothing to pipeline (measured: the 4096 x 14336
  // layer with four K splits is 13 % slower here than as independent tiles).
  if (N / kRowsPerTile < 2 * (148 / splits)) return false;
  if (splits > 1 && N / kRowsPerTile < 2 * 148) return false;
  return persist_smem(M, steps_per_split) <= kPersistSmemCap;
}

int gemv_persist_launch(const gemv::GemvParams& p, int x_dtype, cudaStream_t stream) {
  using namespace gemv;
  const int n_tiles = (p.N + kRowsPerTile - 1) / kRowsPerTile;
  if ((size_t)n_tiles >= kStatusIndex) return PARE_ERR_UNSUPPORTED;
  const size_t smem = persist_smem(p.M, p.steps_per_split);
  int ctas = 148 / p.splits;
  if (ctas < 1) ctas = 1;
  if (ctas > n_tiles) ctas = n_tiles;
  auto launch = [&](auto kern, int threads) -> int {
    // set on every launch: the kernels share one function-pointer type, so a per-lambda flag would not do
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPersistSmemCap) != cudaSuccess)
      return PARE_ERR_CUDA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, p.splits, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, p, n_tiles) == cudaSuccess ? PARE_OK : PARE_ERR_CUDA;
  };
  const bool m16 = p.meta_h2 != nullptr;
  if (g_persist_warps == 8) {
    if (x_dtype == PARE_F16)
      return m16 ? launch(w4a16_gemv_persist_kernel<__half, true, 8>, 288) : launch(w4a16_gemv_persist_kernel<__half, false, 8>, 288);
    return m16 ? launch(w4a16_gemv_persist_kernel<__nv_bfloat16, true, 8>, 288)
               : launch(w4a16_gemv_persist_kernel<__nv_bfloat16, false, 8>, 288);
  }
  if (x_dtype == PARE_F16)
    return m16 ? launch(w4a16_gemv_persist_kernel<__half, true, 16>, 544) : launch(w4a16_gemv_persist_kernel<__half, false, 16>, 544);
  return m16 ? launch(w4a16_gemv_persist_kernel<__nv_bfloat16, true, 16>, 544)
             : launch(w4a16_gemv_persist_kernel<__nv_bfloat16, false, 16>, 544);
}

}  // namespace pare
