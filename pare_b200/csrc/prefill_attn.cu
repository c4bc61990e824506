// Prefill attention over full-precision K / V (fp16 / bf16), sm_100a: the attention of a prompt's tokens
// before the cache compresses them.  The reference leaves this to its caller
// (scaled_dot_product_attention on update()'s return, pare/kv_cache.py:183-186, 205-252); for a prompt
// that return is mostly a lossy reconstruction, so this kernel attends to the tokens as they were given.
//
//   out[b][hq][i][:] = softmax_j(q[b][hq][i] . k[b][hq / rep][j] * scale) . v[b][hq / rep][j]
//   causal: key j is visible to query i iff j <= i + (Tk - Tq)   (the queries are the newest Tq tokens)
//
// One CTA per (64-query tile, query head, batch), four warps of 16 query rows.  K / V stream through shared
// memory in 64-key tiles, two buffers, cp.async; S = Q K^T and O += P V on warp-level tensor-core steps
// (m16n8k16, fp32 accumulate) with ldmatrix operand loads; softmax statistics online in registers, so the
// score matrix never exists.  head_dim 128.
#include "common.cuh"

namespace pare {
namespace {

constexpr int kPD = 128;                 // head_dim
constexpr int kPQ = 64;                  // query rows per CTA
constexpr int kPK = 64;                  // keys per tile
constexpr int kPWarps = 4;
constexpr int kPThreads = kPWarps * 32;
constexpr int kPPitch = kPD * 2 + 16;    // bytes per staged row: 16-byte skew keeps ldmatrix conflict-free
constexpr size_t kPSmem = (size_t)(kPQ + 4 * kPK) * kPPitch;   // Q tile + two (K, V) buffers

struct PrefillParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  int64_t q_sb, q_sh, q_st;
  int64_t k_sb, k_sh, k_st;
  int64_t v_sb, v_sh, v_st;
  int64_t o_sb, o_sh, o_st;
  int B, Hq, H, rep, Tq, Tk;
  float scale_log2;    // softmax scale * log2(e)
  int causal;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;   // zero-fill rows beyond the sequence
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// 16-bit pair of (a, b) minus what the pair `packed` already holds: the second term of a two-term expansion
template <typename T>
__device__ __forceinline__ uint32_t residual2(float a, float b, uint32_t packed);
template <>
__device__ __forceinline__ uint32_t residual2<__nv_bfloat16>(float a, float b, uint32_t packed) {
  return pack2<__nv_bfloat16>(a - __uint_as_float(packed << 16), b - __uint_as_float(packed & 0xffff0000u));
}
template <>
__device__ __forceinline__ uint32_t residual2<__half>(float a, float b, uint32_t packed) {
  const __half2 h = *reinterpret_cast<const __half2*>(&packed);
  return pack2<__half>(a - __low2float(h), b - __high2float(h));
}

// rows [row0, row0 + rows) of a [T][128] tensor (row stride st elements) into a staged tile; rows >= T are zeros
template <typename T>
__device__ __forceinline__ void stage_rows(uint32_t dst, const T* src, int64_t st, int row0, int rows, int T_total) {
  for (int i = threadIdx.x; i < rows * (kPD / 8); i += kPThreads) {
    const int r = i >> 4, c = i & 15;
    const bool ok = row0 + r < T_total;
    cp_async16(dst + r * kPPitch + c * 16, src + (int64_t)(ok ? row0 + r : 0) * st + c * 8, ok);
  }
}

template <typename T>
__global__ void __launch_bounds__(kPThreads) prefill_attn_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
  const int qt = gridDim.x - 1 - blockIdx.x;   // the longest (latest) query tiles start first
  const int hq = blockIdx.y, b = blockIdx.z, h = hq / p.rep;
  const T* qg = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_sb + (int64_t)hq * p.q_sh;
  const T* kg = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_sb + (int64_t)h * p.k_sh;
  const T* vg = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_sb + (int64_t)h * p.v_sh;
  T* og = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_sb + (int64_t)hq * p.o_sh;
  const int q0 = qt * kPQ;
  const int off = p.Tk - p.Tq;                                   // key index of query 0's own token
  const int k_end = p.causal ? min(p.Tk, q0 + kPQ + off) : p.Tk;  // keys [0, k_end) can be visible to this tile
  const int n_tiles = (k_end + kPK - 1) / kPK;

  const uint32_t qs = (uint32_t)__cvta_generic_to_shared(smem);
  auto kbuf = [&](int buf) { return qs + (kPQ + buf * 2 * kPK) * kPPitch; };
  auto vbuf = [&](int buf) { return kbuf(buf) + kPK * kPPitch; };

  stage_rows<T>(qs, qg, p.q_st, q0, kPQ, p.Tq);
  stage_rows<T>(kbuf(0), kg, p.k_st, 0, kPK, p.Tk);
  stage_rows<T>(vbuf(0), vg, p.v_st, 0, kPK, p.Tk);
  cp_async_commit();

  uint32_t qf[kPD / 16][4];
  float o[kPD / 8][4];
#pragma unroll
  for (int ct = 0; ct < kPD / 8; ++ct)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[ct][e] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};   // rows gid and gid + 8 of this warp's 16
  const int row_lo = q0 + warp * 16 + gid;                      // query index of the first of them

  int buf = 0;
  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<0>();
    __syncthreads();   // tile t is in shared memory, and every warp has finished with the other buffer
    if (t + 1 < n_tiles) {
      stage_rows<T>(kbuf(buf ^ 1), kg, p.k_st, (t + 1) * kPK, kPK, p.Tk);
      stage_rows<T>(vbuf(buf ^ 1), vg, p.v_st, (t + 1) * kPK, kPK, p.Tk);
      cp_async_commit();
    }
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < kPD / 16; ++ks)
        ldsm_x4(qf[ks], qs + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kPPitch + (ks * 16 + (lane >> 4) * 8) * 2);
    }

    // ---- S = Q K^T for 16 query rows x 64 keys ----
    float s[kPK / 8][4];
#pragma unroll
    for (int nt = 0; nt < kPK / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < kPD / 16; ks += 2) {
        uint32_t kb[4];
        ldsm_x4(kb, kbuf(buf) + (nt * 8 + (lane & 7)) * kPPitch + (ks * 16 + (lane >> 3) * 8) * 2);
        mma16816<T>(s[nt], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kb[0], kb[1]);
        mma16816<T>(s[nt], qf[ks + 1][0], qf[ks + 1][1], qf[ks + 1][2], qf[ks + 1][3], kb[2], kb[3]);
      }
    }

    // ---- scale, mask, online softmax ----
    const int key0 = t * kPK;
    const bool need_mask = key0 + kPK > p.Tk || (p.causal && key0 + kPK - 1 > q0 + warp * 16 + off);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < kPK / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[nt][e] * p.scale_log2;
        if (need_mask) {
          const int key = key0 + nt * 8 + tig * 2 + (e & 1);
          const int row = row_lo + (e >> 1) * 8;
          if (key >= p.Tk || (p.causal && key > row + off)) x = -INFINITY;
        }
        s[nt][e] = x;
        mx[e >> 1] = fmaxf(mx[e >> 1], x);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_i[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;      // a row with nothing visible yet
      alpha[r] = exp2f(m_i[r] - m_use[r]);              // exp2(-inf) = 0 on the first tile
      m_i[r] = m_new;
      l_i[r] *= alpha[r];
    }
#pragma unroll
    for (int nt = 0; nt < kPK / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pe = exp2f(s[nt][e] - m_use[e >> 1]);
        s[nt][e] = pe;
        l_i[e >> 1] += pe;
      }
#pragma unroll
    for (int ct = 0; ct < kPD / 8; ++ct) {
      o[ct][0] *= alpha[0]; o[ct][1] *= alpha[0];
      o[ct][2] *= alpha[1]; o[ct][3] *= alpha[1];
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < kPK / 16; ++kk) {
      const uint32_t a0 = pack2<T>(s[2 * kk][0], s[2 * kk][1]), a1 = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      // a 16-bit probability keeps 8 (bf16) or 11 (fp16) bits; where the output is small by cancellation that shows.
      // A second operand with the rounding residuals keeps P.V at fp32-level accuracy.
      const uint32_t r0 = residual2<T>(s[2 * kk][0], s[2 * kk][1], a0), r1 = residual2<T>(s[2 * kk][2], s[2 * kk][3], a1);
      const uint32_t r2 = residual2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1], a2), r3 = residual2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3], a3);
#pragma unroll
      for (int ct = 0; ct < kPD / 8; ct += 2) {
        uint32_t vb[4];
        ldsm_x4_trans(vb, vbuf(buf) + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kPPitch + (ct * 8 + (lane >> 4) * 8) * 2);
        mma16816<T>(o[ct], a0, a1, a2, a3, vb[0], vb[1]);
        mma16816<T>(o[ct + 1], a0, a1, a2, a3, vb[2], vb[3]);
        mma16816<T>(o[ct], r0, r1, r2, r3, vb[0], vb[1]);
        mma16816<T>(o[ct + 1], r0, r1, r2, r3, vb[2], vb[3]);
      }
    }
    buf ^= 1;
  }

  // ---- normalise and store ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 1);
    l_i[r] += __shfl_xor_sync(0xffffffffu, l_i[r], 2);
  }
  const float inv0 = l_i[0] > 0.f ? 1.f / l_i[0] : 0.f, inv1 = l_i[1] > 0.f ? 1.f / l_i[1] : 0.f;
#pragma unroll
  for (int ct = 0; ct < kPD / 8; ++ct) {
    const int col = ct * 8 + tig * 2;
    if (row_lo < p.Tq) *reinterpret_cast<uint32_t*>(og + (int64_t)row_lo * p.o_st + col) = pack2<T>(o[ct][0] * inv0, o[ct][1] * inv0);
    if (row_lo + 8 < p.Tq)
      *reinterpret_cast<uint32_t*>(og + (int64_t)(row_lo + 8) * p.o_st + col) = pack2<T>(o[ct][2] * inv1, o[ct][3] * inv1);
  }
}

}  // namespace
}  // namespace pare

extern "C" int pare_prefill_attn(const void* q, const void* k, const void* v, void* out, int dtype, int64_t q_stride_b,
                                 int64_t q_stride_h, int64_t q_stride_t, int64_t k_stride_b, int64_t k_stride_h,
                                 int64_t k_stride_t, int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                                 int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t, int B, int Hq, int H,
                                 int Tq, int Tk, int D, float softmax_scale, int causal, void* stream) {
  using namespace pare;
  PARE_REQUIRE(B > 0 && Hq > 0 && H > 0 && Hq % H == 0 && Tq > 0 && Tk >= Tq, PARE_ERR_SHAPE);
  PARE_REQUIRE(D == kPD, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(dtype == PARE_F16 || dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(q && k && v && out, PARE_ERR_SHAPE);
  PARE_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), PARE_ERR_ALIGN);
  for (int64_t s : {q_stride_b, q_stride_h, q_stride_t, k_stride_b, k_stride_h, k_stride_t, v_stride_b, v_stride_h, v_stride_t,
                    out_stride_b, out_stride_h, out_stride_t})
    PARE_REQUIRE(s % 8 == 0, PARE_ERR_ALIGN);
  PARE_REQUIRE(Hq <= 65535 && B <= 65535, PARE_ERR_UNSUPPORTED);
  PrefillParams p{};
  p.q = q; p.k = k; p.v = v; p.out = out;
  p.q_sb = q_stride_b; p.q_sh = q_stride_h; p.q_st = q_stride_t;
  p.k_sb = k_stride_b; p.k_sh = k_stride_h; p.k_st = k_stride_t;
  p.v_sb = v_stride_b; p.v_sh = v_stride_h; p.v_st = v_stride_t;
  p.o_sb = out_stride_b; p.o_sh = out_stride_h; p.o_st = out_stride_t;
  p.B = B; p.Hq = Hq; p.H = H; p.rep = Hq / H; p.Tq = Tq; p.Tk = Tk;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  const dim3 grid((Tq + kPQ - 1) / kPQ, Hq, B);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto launch = [&](auto kern) -> int {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPSmem) != cudaSuccess) return PARE_ERR_CUDA;
    kern<<<grid, kPThreads, kPSmem, s>>>(p);
    return launch_status();
  };
  return dtype == PARE_F16 ? launch(prefill_attn_kernel<__half>) : launch(prefill_attn_kernel<__nv_bfloat16>);
}
