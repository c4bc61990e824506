// One-shot all-reduce of a small activation tensor over NVLink peer memory, sm_100a.
//
// Tensor-parallel decode sums two [rows x hidden] partial results per block (after the o and the
// down projection).  At decode sizes (a few KB) a library all-reduce is all latency; here every
// rank simply stores its partial into a slot of every peer's exchange buffer (plain peer stores,
// no multicast), raises a flag there, waits for the flags of its own buffer and adds the slots in
// rank order (fp32, deterministic, identical on all ranks).  One kernel launch per all-reduce.
//
// Exchange buffer of a rank (allocated by pare_peer_buffer_create, mapped into the peers with
// CUDA IPC):  [0, 4096): header -- epoch[kMaxCtas] ints, then flags[2][kMaxRanks][kMaxCtas] ints;
// [4096, ...): data[2][world][slot].  Slots and flags are double-buffered by the parity of a
// per-CTA epoch that the kernel itself advances, so a captured CUDA graph can be replayed: a rank
// can only be one call ahead of a peer (it needs the peer's flag of the current call to finish).
// The wait is bounded; a timeout sets PARE_ERR_TIMEOUT in the header's status word and the call
// returns whatever it has (the host reads the word with pare_peer_status).

#include "common.cuh"

namespace pare {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 16;
constexpr size_t kHeaderBytes = 4096;
constexpr int kStatusWord = kMaxCtas;                        // ints into the header
constexpr int kFlagBase = 64;                                // ints into the header
constexpr uint32_t kPeerSpinLimit = 1u << 24;
constexpr int kThreads = 256;

struct PeerParams {
  unsigned char* buf[kMaxRanks];
  const void* x;
  void* y;
  int64_t ldx, ldy;
  int rows, cols;
  int rank, world;
  size_t slot_bytes;
  int vec_per_cta;   // 16-byte vectors of the flattened [rows x cols] tensor per CTA
};

__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// cols % 8 == 0: a 16-byte vector never straddles a row
template <typename T>
__global__ void __launch_bounds__(kThreads) peer_allreduce_kernel(const PeerParams p) {
  pdl_launch_dependents();
  pdl_wait();   // x is the previous kernel's output
  const int c = blockIdx.x;
  int* hdr = reinterpret_cast<int*>(p.buf[p.rank]);
  const int e = hdr[c] + 1;
  const int par = e & 1;
  const int vec_per_row = p.cols >> 3;
  const int v_lo = c * p.vec_per_cta, v_hi = min(v_lo + p.vec_per_cta, p.rows * vec_per_row);
  const size_t slot_off = kHeaderBytes + ((size_t)par * p.world + p.rank) * p.slot_bytes;

  // 1) my partial into slot `rank` of every rank's buffer (own buffer included)
  const T* x = reinterpret_cast<const T*>(p.x);
  for (int v = v_lo + threadIdx.x; v < v_hi; v += kThreads) {
    const int r = v / vec_per_row, cc = (v - r * vec_per_row) * 8;
    const uint4 val = *reinterpret_cast<const uint4*>(x + (size_t)r * p.ldx + cc);
    for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.buf[q] + slot_off + (size_t)v * 16) = val;
  }
  __threadfence_system();
  __syncthreads();
  // 2) tell every rank that this CTA's share of my partial has landed, then wait for theirs
  if (threadIdx.x < p.world) {
    const int q = threadIdx.x;
    st_release_sys(reinterpret_cast<int*>(p.buf[q]) + kFlagBase + (par * kMaxRanks + p.rank) * kMaxCtas + c, e);
    const int* mine = hdr + kFlagBase + (par * kMaxRanks + q) * kMaxCtas + c;
    uint32_t i = 0;
    while (ld_acquire_sys(mine) != e) {
      if (++i >= kPeerSpinLimit) {
        atomicExch(hdr + kStatusWord, PARE_ERR_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  // 3) sum in rank order
  T* y = reinterpret_cast<T*>(p.y);
  const unsigned char* data = p.buf[p.rank] + kHeaderBytes + (size_t)par * p.world * p.slot_bytes;
  for (int v = v_lo + threadIdx.x; v < v_hi; v += kThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < p.world; ++q) {
      const uint4 val = __ldcg(reinterpret_cast<const uint4*>(data + (size_t)q * p.slot_bytes + (size_t)v * 16));
      const T* ve = reinterpret_cast<const T*>(&val);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += to_float<T>(ve[k]);
    }
    uint4 out;
    T* oe = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int k = 0; k < 8; ++k) oe[k] = from_float<T>(acc[k]);
    const int r = v / vec_per_row, cc = (v - r * vec_per_row) * 8;
    *reinterpret_cast<uint4*>(y + (size_t)r * p.ldy + cc) = out;
  }
  __syncthreads();
  if (threadIdx.x == 0) hdr[c] = e;
}

}  // namespace
}  // namespace pare

extern "C" {

// Set-up calls (these do allocate / map memory; everything else in the library does not).
int pare_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]) {
  PARE_REQUIRE(ptr && handle && bytes >= pare::kHeaderBytes + 4096, PARE_ERR_SHAPE);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return PARE_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return PARE_ERR_CUDA;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return PARE_ERR_CUDA;
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return PARE_OK;
}

int pare_peer_buffer_open(const unsigned char handle[64], void** ptr) {
  PARE_REQUIRE(ptr && handle, PARE_ERR_SHAPE);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? PARE_OK : PARE_ERR_CUDA;
}

int pare_peer_buffer_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? PARE_OK : PARE_ERR_CUDA; }
int pare_peer_buffer_destroy(void* ptr) { return cudaFree(ptr) == cudaSuccess ? PARE_OK : PARE_ERR_CUDA; }

// Status word of this rank's exchange buffer (0, or PARE_ERR_TIMEOUT after a wait ran out); synchronises the stream.
int pare_peer_status(const void* own_buffer, void* stream) {
  int v = 0;
  if (cudaMemcpyAsync(&v, reinterpret_cast<const int*>(own_buffer) + pare::kStatusWord, sizeof(int), cudaMemcpyDeviceToHost,
                      reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess)
    return PARE_ERR_CUDA;
  if (cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) return PARE_ERR_CUDA;
  return v;
}

// y[r][:] = sum over ranks of x[r][:] for a [rows x cols] tensor (cols % 8 == 0, 16-byte aligned rows) that is
// small enough for the exchange buffers: rows * cols * 2 <= (buffer_bytes - 4096) / (2 * world).  buffers: HOST
// array of `world` device pointers, buffers[rank] this rank's own buffer, the others its peers' buffers as mapped
// into this process.  Every rank must make the same sequence of calls.
int pare_peer_allreduce(const void* x, int64_t ldx, void* y, int64_t ldy, int rows, int cols, int dtype, int rank, int world,
                        void* const* buffers, size_t buffer_bytes, void* stream) {
  using namespace pare;
  PARE_REQUIRE(x && y && buffers && rows > 0 && cols > 0 && ldx >= cols && ldy >= cols, PARE_ERR_SHAPE);
  PARE_REQUIRE(world >= 2 && world <= kMaxRanks && rank >= 0 && rank < world, PARE_ERR_SHAPE);
  PARE_REQUIRE(dtype == PARE_F16 || dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(cols % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && aligned16(x) && aligned16(y), PARE_ERR_ALIGN);
  PeerParams p{};
  for (int q = 0; q < world; ++q) {
    PARE_REQUIRE(buffers[q] != nullptr, PARE_ERR_SHAPE);
    p.buf[q] = reinterpret_cast<unsigned char*>(buffers[q]);
  }
  p.slot_bytes = ((buffer_bytes - kHeaderBytes) / (2 * (size_t)world)) & ~(size_t)255;
  const size_t bytes = (size_t)rows * cols * 2;
  PARE_REQUIRE(buffer_bytes > kHeaderBytes && bytes <= p.slot_bytes, PARE_ERR_WORKSPACE);
  p.x = x; p.y = y; p.ldx = ldx; p.ldy = ldy; p.rows = rows; p.cols = cols; p.rank = rank; p.world = world;
  const int nvec = (int)(bytes / 16);
  int ctas = (nvec + 2 * kThreads - 1) / (2 * kThreads);   // two vectors per thread
  ctas = ctas < 1 ? 1 : (ctas > kMaxCtas ? kMaxCtas : ctas);
  p.vec_per_cta = (nvec + ctas - 1) / ctas;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return dtype == PARE_F16 ? launch_pdl(peer_allreduce_kernel<__half>, dim3(ctas), dim3(kThreads), 0, s, p)
                           : launch_pdl(peer_allreduce_kernel<__nv_bfloat16>, dim3(ctas), dim3(kThreads), 0, s, p);
}

}  // extern "C"
