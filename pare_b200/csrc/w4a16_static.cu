// pare_w4a16_forward_static: the decode-path W4A16 linear for callers that cannot allocate.
//
// The regular entry point takes a caller-allocated workspace.  Some hosts of this library have no
// way to provide one: a plugin that runs inside another runtime's callback where cudaMalloc is
// forbidden (allocation would synchronise the device or fail under that runtime's memory pool),
// or code that is only handed input and output pointers.  For them the same streaming kernel runs
// with its scratch in a fixed array that lives in this library's device image.

#include <mutex>

#include "common.cuh"
#include "gemv_common.cuh"
#include "peer.cuh"

namespace pare {
struct ProducerArgs {
  int kind;
  const void* a;
  const void* b;
  const void* c;
  void* resid_out;
  int64_t lda;
  float eps;
};
size_t gemv_workspace_bytes(int M, int N, int K, int G);
int gemv_forward(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale,
                 const float* zero, const void* meta_h2, const int32_t* col_perm, const float* input_scale,
                 const void* bias, void* y, int64_t ldy, int M, int N, int K, int G, void* workspace,
                 size_t workspace_bytes, cudaStream_t stream, const void* prepared, const ProducerArgs* prod,
                 const PeerCtx* peer = nullptr);
}  // namespace pare

namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;   // 16 MiB per GPU that loads the library, held until exit
constexpr size_t kZeroedPrefixBytes = pare::gemv::kStatusIndex * sizeof(int);  // the arrival counters of the split-K reduction (the status word after them is kept)

// Device storage.  In host code this name is only a handle for the runtime, never an address a
// kernel could use: the device address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mu;
void* g_scratch_ptr[64] = {};

// Device address of the scratch array on the current device (looked up on first use).
int static_scratch(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PARE_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return PARE_ERR_CUDA;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return PARE_OK;
}

}  // namespace

extern "C" {

size_t pare_w4a16_static_scratch_bytes(void) { return kStaticScratchBytes; }

int pare_w4a16_forward_static(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale,
                              const float* zero, const void* meta_h2, const int32_t* col_perm, const float* input_scale,
                              const void* bias, void* y, int64_t ldy, int M, int N, int K, int group_size, void* stream) {
  PARE_REQUIRE(M > 0 && N > 0 && K > 0 && group_size > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(M <= 16, PARE_ERR_UNSUPPORTED);  // the decode kernel only; larger batches need the regular entry point
  PARE_REQUIRE((K % 2) == 0 && (K % group_size) == 0 && ldx >= K && ldy >= N, PARE_ERR_SHAPE);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(x && packed && y && (meta_h2 || (scale && zero)), PARE_ERR_SHAPE);
  // the layer must fit the fixed array: reject, never overrun
  PARE_REQUIRE(pare::gemv_workspace_bytes(M, N, K, group_size) <= kStaticScratchBytes, PARE_ERR_WORKSPACE);
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != PARE_OK) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the counters are the part that must start at zero
  if (cudaMemsetAsync(scratch, 0, kZeroedPrefixBytes, s) != cudaSuccess) return PARE_ERR_CUDA;
  return pare::gemv_forward(x, x_dtype, ldx, packed, scale, zero, meta_h2, col_perm, input_scale, bias, y, ldy, M, N, K,
                            group_size, scratch, kStaticScratchBytes, s, nullptr, nullptr);
}

int pare_w4a16_static_status(void* stream) {
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != PARE_OK) return rc;
  return pare_workspace_status(scratch, stream);
}

}  // extern "C"
