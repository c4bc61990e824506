// Persistent, work-balanced variant of the W4A16 streaming dequant-GEMV (M <= 8, group size 128), sm_100a.
//
// Same arithmetic and data layout as w4a16_gemv.cu (see there).  What changes is the schedule.
// One CTA per SM stays resident.  K is cut into slices of <= 4096 columns and the SMs are divided
// evenly among the slices; within a slice the layer is cut into items of 32 output rows, and
// CTA b of the slice takes items b, b + Gs, b + 2 Gs, ...  The items that are left over when the
// count is not a multiple of Gs are cut further along K into P pieces, one per CTA, so every SM
// gets the same amount of work to within a fraction of an item instead of one whole extra item.
// Inside a CTA three kinds of warps talk through mbarriers only:
//   * a producer warp keeps the next items' weights in flight (ring of two to four slots of
//     row-contiguous bulk async copies, full / empty barriers; as deep as shared memory allows,
//     because bytes in flight per SM are what bounds the bandwidth a streaming kernel reaches);
//   * sixteen consumer warps each own two 128-column steps of every slice for both 16-row
//     blocks of the item; activations and their per-step table are staged in shared memory
//     once per CTA, scale / zero of the next item are fetched into the registers the current
//     item has just finished with; their partial sums go to a double-buffered exchange area and
//     the warp moves on without waiting for anyone;
//   * an epilogue warp adds the sixteen partial sums and writes the outputs.  Rows whose K range
//     is spread over several items (K slices, pieces) go through the workspace: every
//     contribution is stored, the last one to arrive at the row tile's counter adds them in a
//     fixed order (deterministic) and resets the counter.  That global round trip stalls
//     nobody but the epilogue warp.
// All mbarrier waits are bounded and report PARE_ERR_TIMEOUT through the status word.

#include <type_traits>

#include "gemv_common.cuh"
#include "stage.cuh"

namespace pare {
namespace {

using namespace gemv;

constexpr int kMaxDepth = 4;           // ring slots (2..4, as many as fit)
constexpr int kMaxRows = 32;           // rows of a tile: 32, or 16 when two blocks of activation rows are in play
constexpr int kCW = 16;                // consumer warps
constexpr int kEpi = 2;                // epilogue warps
constexpr int kMaxRed = 4;             // exchange buffers at most
constexpr int kThreads = (kCW + 1 + kEpi) * 32;   // consumers + producer + epilogue warps

struct StreamPlan {
  int n_tiles;    // row tiles
  int n_slices;   // K slices
  int sps;        // 128-column steps per slice (a multiple of spw, <= 16 * spw)
  int spw;        // steps per consumer warp and slice
  int rows;       // rows per tile (16 or 32)
  int red_bufs;   // exchange buffers (1, 2 or 4; an even count is shared by two epilogue warps)
  int gs;         // CTAs per slice
  int q;          // whole items per CTA
  int n_full;     // q * gs: items of a slice handed out whole
  int P;          // pieces per left-over item (power of two <= 16), 0 if nothing is left over
  int pieces;     // left-over items * P (per slice)
  int units;      // contributions per slice: n_full + pieces
  int depth;      // ring slots
  int compact;    // M <= 2: the exchange area keeps only the two activation columns in use
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ bool wait_or_die(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  if (dead) return false;
  if (mbar_wait(bar, parity, status)) return true;
  dead = true;
  return false;
}

// Wait of a warp that is not on the critical path (producer, epilogue): sleeps between polls so that
// its polling does not compete with the consumers for issue slots and the shared-memory pipe.
__device__ __forceinline__ bool wait_relaxed(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  if (dead) return false;
#pragma unroll 1
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_test(bar, parity)) return true;
    __nanosleep(128);
  }
  if (status) atomicExch(status, PARE_ERR_TIMEOUT);
  dead = true;
  return false;
}

// The i-th work item of CTA bl of a slice: a whole 32-row tile, or first of all one piece of a left-over tile.
struct Item {
  int tile;
  int w_lo, w_hi;   // consumer warps that take part
  int unit;         // index of this contribution within the slice
};
__device__ __forceinline__ Item item_of(const StreamPlan& pl, int bl, int i) {
  Item it;
  const bool has_piece = bl < pl.pieces;
  if (has_piece && i == 0) {
    it.tile = pl.n_full + bl / pl.P;
    const int kp = bl % pl.P, wpp = kCW / pl.P;
    it.w_lo = kp * wpp;
    it.w_hi = it.w_lo + wpp;
    it.unit = pl.n_full + bl;
  } else {
    it.tile = bl + (i - (has_piece ? 1 : 0)) * pl.gs;
    it.w_lo = 0;
    it.w_hi = kCW;
    it.unit = it.tile;
  }
  return it;
}

// SPW = 128-column steps per consumer warp and slice, RB = 16-row blocks per tile, MB = blocks of 8
// activation rows (M <= 8 MB).
// PEER: the layer is a row-parallel shard of a tensor-parallel model and the epilogue warps add the ranks' partial
// outputs (peer.cuh).  A template parameter so that the single-GPU instantiations carry none of that code.
template <typename T, bool META16, int SPW, int RB, int MB, bool PROD, bool PEER>
__global__ void __launch_bounds__(kThreads, 1) w4a16_gemv_persist_kernel(const GemvParams p, const StreamPlan pl) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int R = 16 * RB;   // rows per tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int steps_total = p.K >> 7;
  const int slice = blockIdx.x / pl.gs, bl = blockIdx.x - slice * pl.gs;
  const int n_items = pl.q + (bl < pl.pieces ? 1 : 0);
  const int s0 = slice * pl.sps;                             // first 128-column step of this CTA's slice
  const int sps_this = min(pl.sps, steps_total - s0);        // even
  const int depth = pl.depth;

  const int pitch = pl.sps * 64 + 64;        // == 64 (mod 128)
  const int xstride = pl.sps * 256 + 64;
  const int red_lanes = pl.compact ? 8 : 32;                 // float4 entries per (warp, row block, activation block)
  const int red_buf = kCW * RB * MB * red_lanes * 16;        // bytes of one exchange buffer
  const int nred = pl.red_bufs;
  unsigned char* ring = smem;                                                     // [depth][32][pitch]
  unsigned char* xs = ring + depth * R * pitch;                        // [M][xstride]
  float4* tab = reinterpret_cast<float4*>(xs + (size_t)p.M * xstride);            // [sps][kTabCols] (E, SX, g, -)
  const int mcols = (p.M + 1) & ~1;   // table columns kept in shared memory: activation rows in use, rounded up to a pair
  unsigned char* red = reinterpret_cast<unsigned char*>(tab + (size_t)pl.sps * mcols);   // [2][kCW][2][red_lanes] float4
  uint32_t* zero_blk = reinterpret_cast<uint32_t*>(red + nred * red_buf);            // 256 zero bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(zero_blk + 64);                    // full[4] empty[4] red_full[2] red_empty[2]
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxDepth);
  const uint32_t rfull0 = smem_u32(bars + 2 * kMaxDepth), rempty0 = smem_u32(bars + 2 * kMaxDepth + kMaxRed);
  const uint32_t ring_u32 = smem_u32(ring), xs_u32 = smem_u32(xs), tab_u32 = smem_u32(tab), red_u32 = smem_u32(red);
  int* status = p.counters + kStatusIndex;
  bool dead = false;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kMaxDepth; ++i) {
      mbar_init(full0 + i * 8, 1);
      mbar_init(empty0 + i * 8, kCW);
    }
    for (int i = 0; i < kMaxRed; ++i) {
      mbar_init(rfull0 + i * 8, kCW);
      mbar_init(rempty0 + i * 8, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 64) zero_blk[threadIdx.x] = 0u;
  __syncthreads();
  pdl_launch_dependents();

  if (warp == kCW) {
    // ================= producer: weights never depend on the previous kernel =================
    int slot = 0, ph = 0;
    for (int i = 0; i < n_items; ++i) {
      const Item it = item_of(pl, bl, i);
      const int lo = min(it.w_lo * SPW, sps_this), hi = min(it.w_hi * SPW, sps_this);
      const int bytes = (hi - lo) * 64;
      wait_relaxed(empty0 + slot * 8, ph ^ 1, status, dead);
      if (lane == 0) mbar_expect_tx(full0 + slot * 8, R * bytes);
      __syncwarp();
      if (bytes > 0 && lane < R) {
        const int r = it.tile * R + lane;
        bulk_load(ring_u32 + (slot * R + lane) * pitch + lo * 64,
                  p.packed + (size_t)r * (p.K >> 1) + (size_t)(s0 + lo) * 64, bytes, full0 + slot * 8);
        // the item's scale / zero rows towards this SM's L1: the consumer warps read them (row-strided, one line per
        // row and array) when they reach the item, two or three items from now
        const size_t ridx = (size_t)r * p.ngroups + s0 + lo;
        if (META16) {
          prefetch_l1(p.meta_h2 + ridx);
          prefetch_l1(p.meta_h2 + ridx + (hi - lo) - 1);
        } else {
          prefetch_l1(p.scale + ridx);
          prefetch_l1(p.scale + ridx + (hi - lo) - 1);
          prefetch_l1(p.zero + ridx);
          prefetch_l1(p.zero + ridx + (hi - lo) - 1);
        }
      }
      if (++slot == depth) { slot = 0; ph ^= 1; }
    }
    return;
  }

  if (warp > kCW) {
    // ================= epilogue: sum of the consumers' partial sums, outputs =================
    // two warps, one per exchange buffer (even / odd items), so the global round trips of a
    // cross-CTA reduction have two item times to finish before they hold anything up
    pdl_wait();   // outputs, workspace partials and counters may still be in use by the previous kernel
    T* yg = reinterpret_cast<T*>(p.y);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const int n_active = sps_this / SPW;   // consumer warps with a share of this slice
    // the epilogue warps take the items in turn; their count divides the buffer count, so a buffer is always
    // served by the same warp, which therefore sees every phase of its barriers
    const int n_epi = nred >= 2 ? 2 : 1;
    const int ew = warp - kCW - 1;
    if (ew >= n_epi) return;
    // tensor-parallel row-parallel layer: the ranks' partial outputs are exchanged and added right here (peer.cuh),
    // while the consumer warps stream on
    const bool peer = PEER && peer_on(p.peer);
    const uint32_t pe = peer ? peer_epoch(p.peer) : 0u;
    bool peer_timeout = false;
    for (int i = ew; i < n_items; i += n_epi) {
      const Item it = item_of(pl, bl, i);
      const int par = i % nred, rph = (i / nred) & 1;
      wait_relaxed(rfull0 + par * 8, rph, status, dead);
      const uint32_t red_base = red_u32 + par * red_buf;
      const int w_hi = min(it.w_hi, n_active);
      // full layout: lane (gid, tig) holds rows gid, gid+8 x activation rows 2 tig, 2 tig + 1 of row block rb
      // compact layout (M <= 2): lane l < 16 holds (rb = l >> 3, gid = l & 7): rows gid, gid+8 x activation rows 0, 1
      float4 acc[RB][MB];
#pragma unroll
      for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) acc[rb][mb] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (pl.compact) {   // MB == 1
        if (lane < 8 * RB)
          for (int w = it.w_lo; w < w_hi; ++w) {
            const float4 v = lds_v4f(red_base + (w * (8 * RB) + lane) * 16);
            acc[0][0].x += v.x; acc[0][0].y += v.y; acc[0][0].z += v.z; acc[0][0].w += v.w;
          }
      } else {
        for (int w = it.w_lo; w < w_hi; ++w) {
#pragma unroll
          for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              const float4 v = lds_v4f(red_base + (((w * RB + rb) * MB + mb) * 32 + lane) * 16);
              acc[rb][mb].x += v.x; acc[rb][mb].y += v.y; acc[rb][mb].z += v.z; acc[rb][mb].w += v.w;
            }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(rempty0 + par * 8);   // the exchange buffer may be overwritten

      // (local row, activation row) of the values this lane holds: out[k], k = (rb * MB + mb) * 4 + e
      constexpr int NV = 4 * RB * MB;
      float out[NV];
#pragma unroll
      for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int k0 = (rb * MB + mb) * 4;
          out[k0] = acc[rb][mb].x; out[k0 + 1] = acc[rb][mb].y; out[k0 + 2] = acc[rb][mb].z; out[k0 + 3] = acc[rb][mb].w;
        }
      const int nvals = pl.compact ? (lane < 8 * RB ? 4 : 0) : NV;
      auto row_of = [&](int k) {
        return pl.compact ? (lane >> 3) * 16 + (lane & 7) + 8 * ((k >> 1) & 1) : (k / (4 * MB)) * 16 + gid + 8 * ((k >> 1) & 1);
      };
      auto m_of = [&](int k) { return pl.compact ? (k & 1) : ((k >> 2) % MB) * 8 + tig * 2 + (k & 1); };

      // contributions that meet in this row tile: one per K slice, P per slice for a left-over tile
      const int contrib = pl.n_slices * (it.tile >= pl.n_full ? pl.P : 1);
      const int row0 = it.tile * R;
      if (contrib == 1 && peer) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int n = row0 + row_of(k), m = m_of(k);
          if (k < nvals && m < p.M) peer_send(p.peer, pe, (size_t)m * p.N + n, out[k] + (bias ? to_float<T>(bias[n]) : 0.f));
        }
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int n = row0 + row_of(k), m = m_of(k);
          if (k < nvals && m < p.M) yg[(size_t)m * p.ldy + n] = from_float<T>(peer_recv(p.peer, pe, (size_t)m * p.N + n, peer_timeout));
        }
      } else if (contrib == 1) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int n = row0 + row_of(k), m = m_of(k);
          if (k < nvals && m < p.M) {
            float v = out[k];
            if (bias) v += to_float<T>(bias[n]);
            yg[(size_t)m * p.ldy + n] = from_float<T>(v);
          }
        }
      } else {
        float* mine = p.partial + ((size_t)slice * pl.units + it.unit) * p.M * R;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
          const int m = m_of(k);
          if (k < nvals && m < p.M) __stcg(mine + m * R + row_of(k), out[k]);
        }
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = (atomicAdd(p.counters + it.tile, 1) == contrib - 1);
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          const int n = row0 + lane;
          // contributions in a fixed order (slices, then pieces), loaded eight at a time so that the
          // loads overlap instead of each waiting for the previous sum
          const int per_slice = it.tile < pl.n_full ? 1 : pl.P;   // a power of two
          const int lg = 31 - __clz(per_slice);
          const int u0 = it.tile < pl.n_full ? it.tile : pl.n_full + (it.tile - pl.n_full) * pl.P;
          // MI activation rows x C contributions in flight at a time
          auto final_rows = [&](auto mi_tag) {
            constexpr int MI = decltype(mi_tag)::value;
            constexpr int C = MI <= 4 ? 8 : 4;   // contributions per batch: 32 loads in flight at most
            for (int m0 = 0; m0 < p.M; m0 += MI) {
              float v[MI];
#pragma unroll
              for (int mi = 0; mi < MI; ++mi) v[mi] = 0.f;
              for (int c0 = 0; c0 < contrib; c0 += C) {
                float t[MI][C];
#pragma unroll
                for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                  for (int c = 0; c < C; ++c) {
                    const int cc = c0 + c, m = m0 + mi;
                    const int sl = cc >> lg, kp = cc & (per_slice - 1);
                    t[mi][c] = (cc < contrib && m < p.M && lane < R)
                                   ? __ldcg(p.partial + (((size_t)sl * pl.units + u0 + kp) * p.M + m) * R + lane)
                                   : 0.f;
                  }
#pragma unroll
                for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                  for (int c = 0; c < C; ++c) v[mi] += t[mi][c];
              }
              if (peer) {
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                  const int m = m0 + mi;
                  if (m < p.M && lane < R) peer_send(p.peer, pe, (size_t)m * p.N + n, v[mi] + (bias ? to_float<T>(bias[n]) : 0.f));
                }
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                  const int m = m0 + mi;
                  if (m < p.M && lane < R) yg[(size_t)m * p.ldy + n] = from_float<T>(peer_recv(p.peer, pe, (size_t)m * p.N + n, peer_timeout));
                }
              } else {
#pragma unroll
                for (int mi = 0; mi < MI; ++mi) {
                  const int m = m0 + mi;
                  if (m < p.M && lane < R) {
                    float r = v[mi];
                    if (bias) r += to_float<T>(bias[n]);
                    yg[(size_t)m * p.ldy + n] = from_float<T>(r);
                  }
                }
              }
            }
          };
          if (p.M == 1) final_rows(std::integral_constant<int, 1>{});
          else if (p.M == 2) final_rows(std::integral_constant<int, 2>{});
          else if (p.M <= 4) final_rows(std::integral_constant<int, 4>{});
          else final_rows(std::integral_constant<int, 8>{});
          __syncwarp();
          if (lane == 0) p.counters[it.tile] = 0;
        }
      }
    }
    if (peer) {   // one exchanging unit per epilogue warp that runs
      const bool any_timeout = __any_sync(0xffffffffu, peer_timeout);
      if (lane == 0) peer_unit_done(p.peer, pe, gridDim.x * n_epi, any_timeout);
    }
    return;
  }

  // ================= consumers =================
  // scale / zero of this warp's two consecutive groups for rows (rb*16 + gid + 8h) of an item
  float ms[SPW][RB][2], mz[SPW][RB][2];
  const bool has_share = (warp + 1) * SPW <= sps_this;
  auto warp_active = [&](const Item& it) { return has_share && warp >= it.w_lo && warp < it.w_hi; };
  auto load_meta = [&](const Item& it) {
    const int g0 = s0 + warp * SPW;
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const size_t idx = (size_t)(it.tile * R + rb * 16 + gid + 8 * h) * p.ngroups + g0;
        if (SPW == 2) {
          if (META16) {
            const uint2 t2 = __ldg(reinterpret_cast<const uint2*>(p.meta_h2 + idx));
            const __half2 h0 = *reinterpret_cast<const __half2*>(&t2.x), h1 = *reinterpret_cast<const __half2*>(&t2.y);
            ms[0][rb][h] = __low2float(h0); mz[0][rb][h] = __high2float(h0);
            ms[SPW - 1][rb][h] = __low2float(h1); mz[SPW - 1][rb][h] = __high2float(h1);
          } else {
            const float2 a = __ldg(reinterpret_cast<const float2*>(p.scale + idx));
            const float2 c = __ldg(reinterpret_cast<const float2*>(p.zero + idx));
            ms[0][rb][h] = a.x; ms[SPW - 1][rb][h] = a.y;
            mz[0][rb][h] = c.x; mz[SPW - 1][rb][h] = c.y;
          }
        } else {
          if (META16) {
            const uint32_t t1 = __ldg(p.meta_h2 + idx);
            const __half2 h0 = *reinterpret_cast<const __half2*>(&t1);
            ms[0][rb][h] = __low2float(h0); mz[0][rb][h] = __high2float(h0);
          } else {
            ms[0][rb][h] = __ldg(p.scale + idx);
            mz[0][rb][h] = __ldg(p.zero + idx);
          }
        }
      }
  };
  Item cur = item_of(pl, bl, 0);
  bool active = n_items > 0 && warp_active(cur);
  if (active) load_meta(cur);

  uint4 norm_w[1];   // 32 half warps: one step each
  if constexpr (PROD) stage_prefetch_norm<T, 1>(p, sps_this, threadIdx.x, kCW * 32, norm_w);
  pdl_wait();  // the activations are the previous kernel's output
  if constexpr (PROD) {   // this CTA computes its activations itself (stage.cuh)
    stage_produce<T, 1>(p, s0, sps_this, xs, xstride, tab, mcols, threadIdx.x, kCW * 32, reinterpret_cast<float*>(red),
                        blockIdx.x == 0, norm_w, [] { named_sync(1, kCW * 32); });
  } else {
    const int vec_per_row = sps_this * 16;
    const unsigned char* xp = reinterpret_cast<const unsigned char*>(p.xp);
    for (int m = 0; m < p.M; ++m) {
      const uint4* src = reinterpret_cast<const uint4*>(xp + ((size_t)m * p.K + (size_t)s0 * 128) * 2);
      for (int v = threadIdx.x; v < vec_per_row; v += kCW * 32) sts_v4(xs_u32 + m * xstride + v * 16, __ldcg(src + v));
    }
    const uint4* tg = reinterpret_cast<const uint4*>(p.tabg + (size_t)s0 * kTabCols);
    // only the table columns of activation rows in use; threads whose rows are beyond them read
    // whatever follows (always inside this CTA's shared memory) and their results are discarded
    for (int i = threadIdx.x; i < sps_this * mcols; i += kCW * 32) {
      const int st = i / mcols, c = i - st * mcols;
      sts_v4(tab_u32 + i * 16, __ldcg(tg + st * kTabCols + c));
    }
  }
  named_sync(1, kCW * 32);

  // Offsets into the shared array (plain C++ loads from it compile to ld.shared and, unlike asm, leave
  // the compiler free to software-pipeline the four independent (step, row block) units of an item).
  const int w_off = gid * pitch + warp * (SPW * 64) + tig * 16;
  const int tab_off = (int)(reinterpret_cast<unsigned char*>(tab) - smem) + warp * (SPW * mcols * 16) + tig * 32;
  int x_off[MB], xstep[MB];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
    const int m = mb * 8 + gid;   // rows beyond M read a block of zeros that does not advance with the step
    x_off[mb] = (m < p.M ? (int)(xs - smem) + m * xstride + warp * (SPW * 256)
                         : (int)(reinterpret_cast<unsigned char*>(zero_blk) - smem)) + tig * 16;
    xstep[mb] = m < p.M ? 256 : 0;
  }

  int slot = 0, ph = 0, par = 0, rph = 0;
  for (int i = 0; i < n_items; ++i) {
    wait_or_die(full0 + slot * 8, ph, status, dead);
    const unsigned char* stage = smem + slot * R * pitch + w_off;
    float yacc[RB][MB][4];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int e = 0; e < 4; ++e) yacc[rb][mb][e] = 0.f;
    if (active) {   // warp-uniform; one basic block for the whole item
#pragma unroll
      for (int j = 0; j < SPW; ++j) {
        uint4 xb[MB][4];
        float4 t0[MB], t1[MB];   // (E, SX, g, -) of activation rows mb*8 + 2 tig and + 1
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
          for (int q = 0; q < 4; ++q) xb[mb][q] = *reinterpret_cast<const uint4*>(smem + x_off[mb] + j * xstep[mb] + q * 64);
          t0[mb] = *reinterpret_cast<const float4*>(smem + tab_off + j * (mcols * 16) + mb * 128);
          t1[mb] = *reinterpret_cast<const float4*>(smem + tab_off + j * (mcols * 16) + mb * 128 + 16);
        }
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
          const uint4 wa4 = *reinterpret_cast<const uint4*>(stage + rb * 16 * pitch + j * 64);
          const uint4 wb4 = *reinterpret_cast<const uint4*>(stage + (rb * 16 + 8) * pitch + j * 64);
          const uint32_t wa[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
          const uint32_t wb[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
          float d0[MB][4], d1[MB][4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t pa[4], pb[4];
            Nibbles<__half>::unpack(wa[q], pa);
            Nibbles<__half>::unpack(wb[q], pb);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
              if (q == 0) {
                mma16816_zero<__half>(d0[mb], pa[0], pb[0], pa[1], pb[1], xb[mb][q].x, xb[mb][q].y);
                mma16816_zero<__half>(d1[mb], pa[2], pb[2], pa[3], pb[3], xb[mb][q].z, xb[mb][q].w);
              } else {
                mma16816<__half>(d0[mb], pa[0], pb[0], pa[1], pb[1], xb[mb][q].x, xb[mb][q].y);
                mma16816<__half>(d1[mb], pa[2], pb[2], pa[3], pb[3], xb[mb][q].z, xb[mb][q].w);
              }
            }
          }
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
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + slot * 8);   // this warp has read all it needs from the slot
    if (++slot == depth) { slot = 0; ph ^= 1; }
    const bool was_active = active;
    if (i + 1 < n_items) {   // the registers are free again: fetch the next item's scale / zero
      cur = item_of(pl, bl, i + 1);
      active = warp_active(cur);
      if (active) load_meta(cur);
    }
    // ---- partial sums to the exchange buffer `par`; the epilogue warp takes it from there ----
    wait_or_die(rempty0 + par * 8, rph ^ 1, status, dead);
    if (was_active) {
      const uint32_t red_base = red_u32 + par * red_buf;
      if (pl.compact) {   // MB == 1
        if (tig == 0) {
#pragma unroll
          for (int rb = 0; rb < RB; ++rb)
            sts_v4f(red_base + ((warp * RB + rb) * 8 + gid) * 16, yacc[rb][0][0], yacc[rb][0][1], yacc[rb][0][2], yacc[rb][0][3]);
        }
      } else {
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
          for (int mb = 0; mb < MB; ++mb)
            sts_v4f(red_base + (((warp * RB + rb) * MB + mb) * 32 + lane) * 16, yacc[rb][mb][0], yacc[rb][mb][1], yacc[rb][mb][2],
                    yacc[rb][mb][3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(rfull0 + par * 8);
    if (++par == nred) { par = 0; rph ^= 1; }
  }
}

constexpr size_t kPersistSmemCap = 224 * 1024;   // of the 227 KB a block may opt in to
constexpr int kStepsPW = 2;   // steps per consumer warp and slice: slices of up to 4096 columns

size_t persist_smem(int M, int sps, int depth, int rows, int red_bufs) {
  const int mb = M <= 8 ? 1 : 2;
  const size_t red = (size_t)red_bufs * kCW * (rows / 16) * mb * (M <= 2 ? 8 : 32) * 16;
  return (size_t)depth * rows * (sps * 64 + 64) + (size_t)M * (sps * 256 + 64) + (size_t)sps * ((M + 1) & ~1) * sizeof(float4) + red + 256 +
         (2 * kMaxDepth + 2 * kMaxRed) * 8 + 128;
}


// Tile height and exchange buffers by the number of activation rows: 32-row tiles while one block of
// eight activation rows is enough (two exchange buffers if they fit, else one), 16-row tiles for
// nine to sixteen rows (two blocks: the activations take twice the shared memory, the tile half).
StreamPlan make_stream_plan(int M, int N, int K) {
  StreamPlan pl{};
  const int kGrid = sm_count();   // one resident CTA per SM
  const int steps = K >> 7;
  const int slice_steps = kCW * kStepsPW;
  pl.spw = kStepsPW;
  pl.rows = M <= 8 ? 32 : 16;
  pl.n_tiles = N / pl.rows;
  pl.n_slices = (steps + slice_steps - 1) / slice_steps;
  pl.sps = ((steps + pl.n_slices - 1) / pl.n_slices + 1) & ~1;   // even: K % 256 == 0 keeps every slice whole
  pl.n_slices = (steps + pl.sps - 1) / pl.sps;
  pl.gs = kGrid / pl.n_slices;
  if (pl.gs < 1) pl.gs = 1;
  pl.q = pl.n_tiles / pl.gs;
  pl.n_full = pl.q * pl.gs;
  const int r = pl.n_tiles - pl.n_full;
  if (r > 0) {
    int P = 1;
    while (P * 2 <= kCW && r * P * 2 <= pl.gs) P *= 2;
    pl.P = P;
    pl.pieces = r * P;
    if (pl.q == 0) pl.gs = pl.pieces;   // fewer tiles than CTAs: only the pieces exist
  }
  pl.units = pl.n_full + pl.pieces;
  pl.compact = M <= 2 ? 1 : 0;
  // two exchange buffers if they fit (four were measured: no gain, the consumer warps do not wait on them)
  pl.red_bufs = persist_smem(M, pl.sps, 2, pl.rows, 2) <= kPersistSmemCap ? 2 : 1;
  pl.depth = 2;
  while (pl.depth < kMaxDepth && pl.depth < pl.q + (pl.pieces ? 1 : 0) &&
         persist_smem(M, pl.sps, pl.depth + 1, pl.rows, pl.red_bufs) <= kPersistSmemCap)
    ++pl.depth;
  return pl;
}

template <typename X>
struct TypeTag {
  using type = X;
};

}  // namespace

constexpr int kPersistMinItems = 96;   // fewer items than this cannot occupy the machine: tile kernel

// Layers the persistent schedule serves: 128-column groups, whole 32-row tiles, activations that fit in
// shared memory next to the weight ring, and enough items to occupy the machine.
bool gemv_persist_supported(int M, int N, int K, int G, bool producer) {
  if (G != 128 || M > 16 || (K % 256) != 0 || (N % kMaxRows) != 0 || N <= 0) return false;
  const StreamPlan pl = make_stream_plan(M, N, K);
  if (pl.n_slices > sm_count()) return false;
  if ((long long)(N / kMaxRows) * pl.n_slices < kPersistMinItems) return false;
  // Less than two whole items per CTA is all ramp (and cross-CTA reduction where pieces are involved): such
  // layers are faster as independent tiles at M <= 4 (measured: 6144 x 4096 takes 8.1 us here, 6.4 us
  // there; 4096 x 4096 5.1 against 4.7 us) -- unless the kernel computes its own activations: 148 resident
  // CTAs normalise the row once each instead of 384 tiles doing it (the whole decode step gains 8 %).
  if (M <= 4 && pl.n_slices == 1 && pl.q < 2 && !(producer && pl.q == 1)) return false;
  if ((size_t)pl.n_tiles >= kStatusIndex) return false;
  return persist_smem(M, pl.sps, 2, pl.rows, pl.red_bufs) <= kPersistSmemCap;
}

// fp32 words of workspace behind the prepared activations: one [M][rows] block per contribution
size_t gemv_persist_partial_floats(int M, int N, int K) {
  const StreamPlan pl = make_stream_plan(M, N, K);
  return (size_t)pl.n_slices * pl.units * M * pl.rows;
}

int gemv_persist_launch(const gemv::GemvParams& p, int x_dtype, cudaStream_t stream) {
  using namespace gemv;
  const StreamPlan pl = make_stream_plan(p.M, p.N, p.K);
  const size_t smem = persist_smem(p.M, pl.sps, pl.depth, pl.rows, pl.red_bufs);
  auto launch = [&](auto kern) -> int {
    // set on every launch: the kernels share one function-pointer type, so a per-lambda flag would not do
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPersistSmemCap) != cudaSuccess)
      return PARE_ERR_CUDA;
    return launch_pdl(kern, dim3(pl.n_slices * pl.gs), dim3(kThreads), smem, stream, p, pl);
  };
  auto pick = [&](auto t_tag, auto m16_tag) -> int {
    using TT = typename decltype(t_tag)::type;
    constexpr bool M16 = decltype(m16_tag)::value;
    if (peer_on(p.peer)) {   // row-parallel shard: fp32 metadata only
      if constexpr (M16) return PARE_ERR_UNSUPPORTED;
      else {
        if (p.producer) return pl.rows == 32 ? launch(w4a16_gemv_persist_kernel<TT, false, kStepsPW, 2, 1, true, true>) : PARE_ERR_UNSUPPORTED;
        return pl.rows == 32 ? launch(w4a16_gemv_persist_kernel<TT, false, kStepsPW, 2, 1, false, true>)
                             : launch(w4a16_gemv_persist_kernel<TT, false, kStepsPW, 1, 2, false, true>);
      }
    }
    if (p.producer) return pl.rows == 32 ? launch(w4a16_gemv_persist_kernel<TT, M16, kStepsPW, 2, 1, true, false>) : PARE_ERR_UNSUPPORTED;
    return pl.rows == 32 ? launch(w4a16_gemv_persist_kernel<TT, M16, kStepsPW, 2, 1, false, false>)
                         : launch(w4a16_gemv_persist_kernel<TT, M16, kStepsPW, 1, 2, false, false>);
  };
  const bool m16 = p.meta_h2 != nullptr;
  if (x_dtype == PARE_F16) return m16 ? pick(TypeTag<__half>{}, std::true_type{}) : pick(TypeTag<__half>{}, std::false_type{});
  return m16 ? pick(TypeTag<__nv_bfloat16>{}, std::true_type{}) : pick(TypeTag<__nv_bfloat16>{}, std::false_type{});
}

}  // namespace pare
