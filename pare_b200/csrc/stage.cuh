// Producing a streaming kernel's activations inside the kernel: instead of copying prepared
// activations from global memory, a CTA computes them from what the model has at that point --
// RMSNorm of the residual stream, or the SwiGLU gate of a fused gate|up projection -- and writes
// them straight into its shared-memory operand buffers (prep.cuh gives the format).  Every CTA
// repeats the small computation (a few KB from L2); in exchange the stand-alone kernel, its
// launch and its drain disappear from the decode step.
#pragma once

#include "prep.cuh"

namespace pare {
namespace gemv {

constexpr int kStageRounds = 4;   // most steps a half warp of the staging threads takes: K <= 128 * rounds * threads / 16

// Norm weights of the steps a thread will produce: constants of the model, so they can be fetched before
// the dependency wait.  ROUNDS as in stage_produce.
template <typename T, int ROUNDS>
__device__ __forceinline__ void stage_prefetch_norm(const GemvParams& p, int nst, int tid, int nthreads, uint4 (&wv)[ROUNDS]) {
  const int hw = tid >> 4, c = tid & 15, n_hw = nthreads >> 4;
  const T* w = reinterpret_cast<const T*>(p.pc);
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const int st = hw + r * n_hw;
    wv[r] = make_uint4(0u, 0u, 0u, 0u);
    if (p.producer == PARE_PRODUCER_RMSNORM && st < nst) wv[r] = *reinterpret_cast<const uint4*>(w + st * 128 + c * 8);
  }
}

// Warp-collective over `nthreads` threads (a multiple of 32, thread index tid) that all call with
// the same arguments; sync(id) must be a barrier over exactly those threads.  Fills, for steps
// [st0, st0 + nst) of all p.M rows, the operand-order activations xs[m] (row stride xstride bytes)
// and the compact table tab[st - st0][mcols].  scratch: 2 * 32 floats of shared memory.
template <typename T, int ROUNDS, typename Sync>
__device__ __forceinline__ void stage_produce(const GemvParams& p, int st0, int nst, unsigned char* xs, int xstride, float4* tab,
                                              int mcols, int tid, int nthreads, float* scratch, bool first_cta,
                                              const uint4 (&wv)[ROUNDS], Sync sync) {
  const int hw = tid >> 4, c = tid & 15, n_hw = nthreads >> 4;
  const int nwarps = nthreads >> 5;
  const T* a = reinterpret_cast<const T*>(p.pa);
  if (p.producer == PARE_PRODUCER_RMSNORM) {
    // y = rmsnorm(a + b) * w over the whole row (the caller guarantees st0 == 0 and nst == K / 128)
    const T* b = reinterpret_cast<const T*>(p.pb);
    T* ro = reinterpret_cast<T*>(p.resid_out);
    constexpr int kMaxRounds = ROUNDS;
    for (int m = 0; m < p.M; ++m) {
      float h[kMaxRounds][8];
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxRounds; ++r) {
        const int st = hw + r * n_hw;
        if (r * n_hw >= nst) break;   // uniform over the threads
        if (st < nst) {
          const size_t off = (size_t)m * p.lda + st * 128 + c * 8;
          const uint4 av = *reinterpret_cast<const uint4*>(a + off);
          uint4 bv = make_uint4(0u, 0u, 0u, 0u);
          if (b) bv = *reinterpret_cast<const uint4*>(b + off);
          const T* ae = reinterpret_cast<const T*>(&av);
          const T* be = reinterpret_cast<const T*>(&bv);
          uint4 hv;
          T* he = reinterpret_cast<T*>(&hv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float f = to_float<T>(ae[e]);
            if (b) f += to_float<T>(be[e]);
            he[e] = from_float<T>(f);   // the residual stream is kept in T
            h[r][e] = to_float<T>(he[e]);
            ss += h[r][e] * h[r][e];
          }
          if (first_cta && ro) *reinterpret_cast<uint4*>(ro + off) = hv;
        }
      }
      ss = warp_sum(ss);
      float* sc = scratch + (m & 1) * 32;
      if ((tid & 31) == 0) sc[tid >> 5] = ss;
      sync();
      float tot = 0.f;
      for (int i = 0; i < nwarps; ++i) tot += sc[i];
      const float inv = rsqrtf(tot / (float)(nst * 128) + p.eps);
#pragma unroll
      for (int r = 0; r < kMaxRounds; ++r) {
        const int st = hw + r * n_hw;
        if (r * n_hw >= nst) break;
        const bool live = st < nst;
        float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (live) {
          const T* we = reinterpret_cast<const T*>(&wv[r]);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = h[r][e] * inv * to_float<T>(we[e]);
        }
        prep_store_step<T>(o, live, reinterpret_cast<__half*>(xs + (size_t)m * xstride) + st * 128, c,
                           tab + (size_t)st * mcols + m);
      }
    }
  } else {
    // y = silu(gate) * up, gate = a[m][k], up = a[m][K + k]; any K range
    for (int m = 0; m < p.M; ++m) {
      for (int r0 = 0; r0 < nst; r0 += n_hw) {
        const int sl = r0 + hw;   // step within the range
        const bool live = sl < nst;
        float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (live) {
          const size_t off = (size_t)m * p.lda + (size_t)(st0 + sl) * 128 + c * 8;
          const uint4 gv = *reinterpret_cast<const uint4*>(a + off);
          const uint4 uv = *reinterpret_cast<const uint4*>(a + off + p.K);
          const T* ge = reinterpret_cast<const T*>(&gv);
          const T* ue = reinterpret_cast<const T*>(&uv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float g = to_float<T>(ge[e]);
            o[e] = g / (1.f + __expf(-g)) * to_float<T>(ue[e]);
          }
        }
        prep_store_step<T>(o, live, reinterpret_cast<__half*>(xs + (size_t)m * xstride) + sl * 128, c,
                           tab + (size_t)sl * mcols + m);
      }
    }
  }
}

}  // namespace gemv
}  // namespace pare
