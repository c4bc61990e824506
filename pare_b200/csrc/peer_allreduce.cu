// One-shot all-reduce of a small activation tensor over NVLink peer memory, sm_100a.
//
// Tensor-parallel decode sums two [rows x hidden] partial results per block (after the o and the
// down projection).  At decode sizes (a few KB) an all-reduce is all latency, so the protocol has no
// fence and no separate flag: every rank stores its partial into a slot of every peer's exchange
// buffer as 16-byte units {4 bytes data, epoch, 4 bytes data, epoch} (plain peer stores, no
// multicast) -- each 8-byte half carries its own validity mark and arrives atomically -- and then
// reads the slots of its own buffer, spinning (bounded) on each unit until both marks show the
// current epoch, adding the ranks' values in rank order (fp32, deterministic, the same bits on all
// ranks).  One kernel launch per all-reduce, one NVLink store latency end to end.
//
// Exchange buffer of a rank (allocated by pare_peer_buffer_create, mapped into the peers with
// CUDA IPC):  [0, 4096): header -- epoch[kMaxCtas] ints, status word; the first half of what follows:
// data[2][world][slot] (the second half serves the exchange fused into the linears' epilogues, peer.cuh).
// Slots are double-buffered by the parity of an epoch that the kernel itself advances, so a captured CUDA
// graph can be replayed.  Every call launches all kMaxCtas CTAs (those without units only advance their
// epoch word), so every CTA's word equals the number of calls made so far whatever the calls' shapes were:
// a unit's marks grow by one per call no matter which CTA owned it in which call, and a rank can only be
// one call ahead of a peer (it needs the peer's data of the current call to finish), so a slot is never
// overwritten while it is being read and a mark of an older call is never mistaken for the current one.
// A wait that runs out sets PARE_ERR_TIMEOUT in the header's status word and the call returns
// whatever it has (the host reads the word with pare_peer_status).

#include "common.cuh"
#include "peer.cuh"

namespace pare {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 16;
constexpr size_t kHeaderBytes = 4096;
constexpr int kStatusWord = kMaxCtas;                        // ints into the header
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
  int units_per_cta;   // 8-byte payload units (4 elements) of the flattened [rows x cols] tensor per CTA
};

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// cols % 4 == 0: an 8-byte unit never straddles a row
template <typename T>
__global__ void __launch_bounds__(kThreads) peer_allreduce_kernel(const PeerParams p) {
  pdl_launch_dependents();
  pdl_wait();   // x is the previous kernel's output
  const int c = blockIdx.x;
  int* hdr = reinterpret_cast<int*>(p.buf[p.rank]);
  const uint32_t e = (uint32_t)hdr[c] + 1u;
  const int par = e & 1;
  const int units_per_row = p.cols >> 2;
  const int u_lo = c * p.units_per_cta, u_hi = min(u_lo + p.units_per_cta, p.rows * units_per_row);
  const size_t slot_off = kHeaderBytes + ((size_t)par * p.world + p.rank) * p.slot_bytes;

  // 1) my partial into slot `rank` of every rank's buffer (own buffer included), each 8 bytes with the epoch
  const T* x = reinterpret_cast<const T*>(p.x);
  for (int u = u_lo + threadIdx.x; u < u_hi; u += kThreads) {
    const int r = u / units_per_row, cc = (u - r * units_per_row) * 4;
    const uint2 val = *reinterpret_cast<const uint2*>(x + (size_t)r * p.ldx + cc);
    const uint4 unit = make_uint4(val.x, e, val.y, e);
    for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.buf[q] + slot_off + (size_t)u * 16) = unit;
  }
  // 2) the ranks' partials from my own buffer, in rank order, as they arrive
  T* y = reinterpret_cast<T*>(p.y);
  const unsigned char* data = p.buf[p.rank] + kHeaderBytes + (size_t)par * p.world * p.slot_bytes;
  bool timed_out = false;
  for (int u = u_lo + threadIdx.x; u < u_hi; u += kThreads) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < p.world; ++q) {
      const unsigned char* src = data + (size_t)q * p.slot_bytes + (size_t)u * 16;
      uint4 v = ld_volatile_v4(src);
      uint32_t i = 0;
      while ((v.y != e || v.w != e) && !timed_out) {
        if (++i >= kPeerSpinLimit) timed_out = true;
        v = ld_volatile_v4(src);
      }
      const uint2 val = make_uint2(v.x, v.z);
      const T* ve = reinterpret_cast<const T*>(&val);
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[k] += to_float<T>(ve[k]);
    }
    uint2 out;
    T* oe = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int k = 0; k < 4; ++k) oe[k] = from_float<T>(acc[k]);
    const int r = u / units_per_row, cc = (u - r * units_per_row) * 4;
    *reinterpret_cast<uint2*>(y + (size_t)r * p.ldy + cc) = out;
  }
  if (timed_out) atomicExch(hdr + kStatusWord, PARE_ERR_TIMEOUT);
  __syncthreads();   // every thread has read this CTA's epoch
  if (threadIdx.x == 0) hdr[c] = (int)e;
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
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(p);
    return PARE_ERR_CUDA;
  }
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

// y[r][:] = sum over ranks of x[r][:] for a [rows x cols] tensor (cols % 4 == 0, 8-byte aligned rows) that is
// small enough for the exchange buffers: rows * cols * 4 <= (buffer_bytes - 4096) / (2 * world) (every 8 bytes of
// data travel with 8 bytes of validity marks).  buffers: HOST array of `world` device pointers, buffers[rank] this
// rank's own buffer, the others its peers' buffers as mapped into this process.  Every rank must make the same
// sequence of calls.
int pare_peer_allreduce(const void* x, int64_t ldx, void* y, int64_t ldy, int rows, int cols, int dtype, int rank, int world,
                        void* const* buffers, size_t buffer_bytes, void* stream) {
  using namespace pare;
  PARE_REQUIRE(x && y && buffers && rows > 0 && cols > 0 && ldx >= cols && ldy >= cols, PARE_ERR_SHAPE);
  PARE_REQUIRE(world >= 2 && world <= kMaxRanks && rank >= 0 && rank < world, PARE_ERR_SHAPE);
  PARE_REQUIRE(dtype == PARE_F16 || dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(cols % 4 == 0 && ldx % 4 == 0 && ldy % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 7u) == 0 &&
                   (reinterpret_cast<uintptr_t>(y) & 7u) == 0,
               PARE_ERR_ALIGN);
  PeerParams p{};
  for (int q = 0; q < world; ++q) {
    PARE_REQUIRE(buffers[q] != nullptr, PARE_ERR_SHAPE);
    p.buf[q] = reinterpret_cast<unsigned char*>(buffers[q]);
  }
  PARE_REQUIRE(buffer_bytes > kHeaderBytes + 2 * 4096, PARE_ERR_WORKSPACE);
  // this call's half of the data area (the other half belongs to the exchange fused into the linears, peer.cuh)
  p.slot_bytes = ((peer_fused_offset(buffer_bytes) - kHeaderBytes) / (2 * (size_t)world)) & ~(size_t)255;
  const size_t units = (size_t)rows * cols / 4;
  PARE_REQUIRE(units * 16 <= p.slot_bytes, PARE_ERR_WORKSPACE);
  p.x = x; p.y = y; p.ldx = ldx; p.ldy = ldy; p.rows = rows; p.cols = cols; p.rank = rank; p.world = world;
  int ctas = (int)((units + 2 * kThreads - 1) / (2 * kThreads));   // CTAs that get units: two units per thread
  ctas = ctas < 1 ? 1 : (ctas > kMaxCtas ? kMaxCtas : ctas);
  p.units_per_cta = (int)((units + ctas - 1) / ctas);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // always the full grid: the CTAs beyond `ctas` find no units and only advance their epoch word (see the header)
  return dtype == PARE_F16 ? launch_pdl(peer_allreduce_kernel<__half>, dim3(kMaxCtas), dim3(kThreads), 0, s, p)
                           : launch_pdl(peer_allreduce_kernel<__nv_bfloat16>, dim3(kMaxCtas), dim3(kThreads), 0, s, p);
}

}  // extern "C"
