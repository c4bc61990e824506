// extern "C" surface of libpare_b200: argument checks and dispatch only.
#include "peer.cuh"
#include "prep.cuh"

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
int gemv_prepare(const void* x, int x_dtype, int64_t ldx, const int32_t* col_perm, const float* input_scale, int M, int K,
                 void* prepared, cudaStream_t stream);
bool gemv_persist_supported(int M, int N, int K, int G, bool producer = false);
bool gemm_supported(int M, int K, int G, const float* scale, const float* zero);
size_t gemm_workspace_bytes(int M, int N, int K);
int gemm_forward(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale, const float* zero,
                 const int32_t* col_perm, const float* input_scale, const void* bias, void* y, int64_t ldy, int M, int N,
                 int K, int G, void* workspace, size_t workspace_bytes, cudaStream_t stream);
}  // namespace pare

namespace pare {
namespace {
// A wait that nothing ends: one thread waits on a shared-memory barrier nobody arrives at, through the same bounded
// wait the kernels use, with a caller-chosen (small) limit.  It returns after `limit` polls with the time-out recorded.
__global__ void bounded_wait_selftest_kernel(int* status, uint32_t limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    gemv::mbar_init(gemv::smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    gemv::mbar_wait_limit(gemv::smem_u32(&bar), 0, status, limit);
  }
}

int read_and_clear_status(int* word, cudaStream_t s) {
  int v = 0;
  if (cudaMemcpyAsync(&v, word, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess) return PARE_ERR_CUDA;
  if (cudaMemsetAsync(word, 0, sizeof(int), s) != cudaSuccess) return PARE_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return PARE_ERR_CUDA;
  return v;
}
}  // namespace
}  // namespace pare

extern "C" {

int pare_version(void) { return 100; }

const char* pare_status_string(int status) {
  switch (status) {
    case PARE_OK: return "ok";
    case PARE_ERR_SHAPE: return "invalid shape";
    case PARE_ERR_DTYPE: return "unsupported dtype";
    case PARE_ERR_ALIGN: return "pointer or leading dimension not 16-byte aligned";
    case PARE_ERR_WORKSPACE: return "workspace missing or too small";
    case PARE_ERR_UNSUPPORTED: return "unsupported configuration";
    case PARE_ERR_CUDA: return "CUDA runtime error at launch";
    case PARE_ERR_TIMEOUT: return "device-side wait timed out";
    default: return "unknown status";
  }
}

size_t pare_w4a16_workspace_bytes(int M, int N, int K, int group_size) {
  if (M <= 0 || N <= 0 || K <= 0 || group_size <= 0) return 0;
  const size_t a = pare::gemv_workspace_bytes(M, N, K, group_size);
  const size_t b = (M > 16 && K % 512 == 0 && group_size % 128 == 0) ? pare::gemm_workspace_bytes(M, N, K) : 0;
  return a > b ? a : b;
}

int pare_w4a16_forward(const void* x, int x_dtype, int64_t ldx, const uint8_t* packed, const float* scale,
                       const float* zero, const void* meta_h2, const int32_t* col_perm, const float* input_scale,
                       const void* bias, void* y, int64_t ldy, int M, int N, int K, int group_size,
                       void* workspace, size_t workspace_bytes, void* stream) {
  PARE_REQUIRE(M > 0 && N > 0 && K > 0 && group_size > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE((K % 2) == 0 && (K % group_size) == 0, PARE_ERR_SHAPE);
  PARE_REQUIRE(ldx >= K && ldy >= N, PARE_ERR_SHAPE);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(x && packed && y && (meta_h2 || (scale && zero)), PARE_ERR_SHAPE);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // M > 16: tensor-core tiles where they apply (measured on the 8B shapes: from 24 rows on they beat passes of 16
  // rows through the streaming kernel on every projection, at 17 rows they are within 10 % either way); otherwise,
  // and always for M <= 16, the streaming kernel in passes of at most 16 rows
  if (M > 16 && pare::gemm_supported(M, K, group_size, scale, zero))
    return pare::gemm_forward(x, x_dtype, ldx, packed, scale, zero, col_perm, input_scale, bias, y, ldy, M, N, K,
                              group_size, workspace, workspace_bytes, s);
  const size_t esz = 2;
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mc = (M - m0) < 16 ? (M - m0) : 16;
    const int rc = pare::gemv_forward(reinterpret_cast<const unsigned char*>(x) + (size_t)m0 * ldx * esz, x_dtype, ldx,
                                      packed, scale, zero, meta_h2, col_perm, input_scale, bias,
                                      reinterpret_cast<unsigned char*>(y) + (size_t)m0 * ldy * esz, ldy, mc, N, K,
                                      group_size, workspace, workspace_bytes, s, nullptr, nullptr);
    if (rc != PARE_OK) return rc;
  }
  return PARE_OK;
}

size_t pare_w4a16_prepared_bytes(int M, int K) {
  if (M <= 0 || M > 16 || K <= 0 || K % 128) return 0;
  return pare::prepared_bytes(M, K);
}

int pare_w4a16_prepare(const void* x, int x_dtype, int64_t ldx, const int32_t* col_perm, const float* input_scale, int M,
                       int K, void* prepared, void* stream) {
  PARE_REQUIRE(x && prepared && M > 0 && K > 0 && ldx >= K, PARE_ERR_SHAPE);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  return pare::gemv_prepare(x, x_dtype, ldx, col_perm, input_scale, M, K, prepared, reinterpret_cast<cudaStream_t>(stream));
}

int pare_w4a16_forward_prepared(const void* prepared, int x_dtype, const uint8_t* packed, const float* scale,
                                const float* zero, const void* meta_h2, const void* bias, void* y, int64_t ldy, int M,
                                int N, int K, int group_size, void* workspace, size_t workspace_bytes, void* stream) {
  PARE_REQUIRE(M > 0 && N > 0 && K > 0 && group_size > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE((K % 2) == 0 && (K % group_size) == 0 && ldy >= N, PARE_ERR_SHAPE);
  PARE_REQUIRE(M <= 16, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(prepared && packed && y && (meta_h2 || (scale && zero)), PARE_ERR_SHAPE);
  return pare::gemv_forward(nullptr, x_dtype, K, packed, scale, zero, meta_h2, nullptr, nullptr, bias, y, ldy, M, N, K,
                            group_size, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream), prepared, nullptr);
}

int pare_w4a16_forward_produced(int producer, const void* a, const void* b, const void* c, void* resid_out, int64_t lda,
                                float eps, int x_dtype, const uint8_t* packed, const float* scale, const float* zero,
                                const void* meta_h2, const void* bias, void* y, int64_t ldy, int M, int N, int K,
                                int group_size, void* workspace, size_t workspace_bytes, void* stream) {
  PARE_REQUIRE(M > 0 && M <= 16 && N > 0 && K > 0 && group_size > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE((K % 256) == 0 && (group_size % 128) == 0 && (K % group_size) == 0 && ldy >= N, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(a && packed && y && (meta_h2 || (scale && zero)), PARE_ERR_SHAPE);
  PARE_REQUIRE(pare::aligned16(a) && lda % 8 == 0, PARE_ERR_ALIGN);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (producer == PARE_PRODUCER_RMSNORM) {
    PARE_REQUIRE(c != nullptr && lda >= K && resid_out != a, PARE_ERR_SHAPE);
    PARE_REQUIRE(pare::aligned16(c) && (b == nullptr || pare::aligned16(b)) && (resid_out == nullptr || pare::aligned16(resid_out)),
                 PARE_ERR_ALIGN);
  } else if (producer == PARE_PRODUCER_SILU_MUL) {
    PARE_REQUIRE(lda >= 2 * (int64_t)K, PARE_ERR_SHAPE);
  } else {
    return PARE_ERR_UNSUPPORTED;
  }
  const pare::ProducerArgs prod{producer, a, b, c, resid_out, lda, eps};
  int rc = pare::gemv_forward(nullptr, x_dtype, K, packed, scale, zero, meta_h2, nullptr, nullptr, bias, y, ldy, M, N, K,
                              group_size, workspace, workspace_bytes, s, nullptr, &prod);
  if (rc != PARE_ERR_UNSUPPORTED) return rc;
  // no fused path for this shape: stand-alone glue kernel into the workspace's prepared-activation area
  // (same layout as a caller-owned prepared buffer), then the plain prepared forward
  PARE_REQUIRE(workspace && workspace_bytes >= pare_w4a16_workspace_bytes(M, N, K, group_size), PARE_ERR_WORKSPACE);
  void* prepared = reinterpret_cast<unsigned char*>(workspace) + pare::gemv::kCounterBytes;
  if (producer == PARE_PRODUCER_RMSNORM) {
    PARE_REQUIRE(lda == K, PARE_ERR_UNSUPPORTED);   // the stand-alone kernel reads dense rows
    rc = pare_rmsnorm_residual(a, b, c, resid_out, nullptr, prepared, M, K, eps, x_dtype, stream);
  } else {
    rc = pare_silu_mul(a, nullptr, prepared, M, K, lda, x_dtype, stream);
  }
  if (rc != PARE_OK) return rc;
  return pare::gemv_forward(nullptr, x_dtype, K, packed, scale, zero, meta_h2, nullptr, nullptr, bias, y, ldy, M, N, K,
                            group_size, workspace, workspace_bytes, s, prepared, nullptr);
}

namespace {
// exchange buffers of a tensor-parallel group -> the kernels' view of them
int make_peer_ctx(int rank, int world, void* const* buffers, size_t buffer_bytes, pare::PeerCtx* pc) {
  PARE_REQUIRE(buffers && world >= 2 && world <= pare::kPeerMaxRanks && rank >= 0 && rank < world, PARE_ERR_SHAPE);
  PARE_REQUIRE(buffer_bytes >= pare::kPeerHeaderBytes + 2 * 4096, PARE_ERR_WORKSPACE);
  *pc = pare::PeerCtx{};
  for (int q = 0; q < world; ++q) {
    PARE_REQUIRE(buffers[q] != nullptr, PARE_ERR_SHAPE);
    pc->buf[q] = reinterpret_cast<unsigned char*>(buffers[q]);
  }
  pc->rank = rank;
  pc->world = world;
  pc->data_off = pare::peer_fused_offset(buffer_bytes);
  pc->slot_bytes = ((buffer_bytes - pc->data_off) / (2 * (size_t)world)) & ~(size_t)255;
  PARE_REQUIRE(pc->slot_bytes > 0, PARE_ERR_WORKSPACE);
  return PARE_OK;
}
}  // namespace

int pare_w4a16_forward_prepared_allreduce(const void* prepared, int x_dtype, const uint8_t* packed, const float* scale,
                                          const float* zero, const void* meta_h2, const void* bias, void* y, int64_t ldy,
                                          int M, int N, int K, int group_size, void* workspace, size_t workspace_bytes,
                                          int rank, int world, void* const* buffers, size_t buffer_bytes, void* stream) {
  PARE_REQUIRE(M > 0 && N > 0 && K > 0 && group_size > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE((K % 2) == 0 && (K % group_size) == 0 && ldy >= N, PARE_ERR_SHAPE);
  PARE_REQUIRE(M <= 16, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(prepared && packed && y && (meta_h2 || (scale && zero)), PARE_ERR_SHAPE);
  pare::PeerCtx pc;
  const int rc = make_peer_ctx(rank, world, buffers, buffer_bytes, &pc);
  if (rc != PARE_OK) return rc;
  return pare::gemv_forward(nullptr, x_dtype, K, packed, scale, zero, meta_h2, nullptr, nullptr, bias, y, ldy, M, N, K,
                            group_size, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream), prepared, nullptr, &pc);
}

int pare_w4a16_forward_produced_allreduce(int producer, const void* a, const void* b, const void* c, void* resid_out,
                                          int64_t lda, float eps, int x_dtype, const uint8_t* packed, const float* scale,
                                          const float* zero, const void* meta_h2, const void* bias, void* y, int64_t ldy,
                                          int M, int N, int K, int group_size, void* workspace, size_t workspace_bytes,
                                          int rank, int world, void* const* buffers, size_t buffer_bytes, void* stream) {
  PARE_REQUIRE(M > 0 && M <= 16 && N > 0 && K > 0 && group_size > 0, PARE_ERR_SHAPE);
  PARE_REQUIRE((K % 256) == 0 && (group_size % 128) == 0 && (K % group_size) == 0 && ldy >= N, PARE_ERR_UNSUPPORTED);
  PARE_REQUIRE(x_dtype == PARE_F16 || x_dtype == PARE_BF16, PARE_ERR_DTYPE);
  PARE_REQUIRE(a && packed && y && (meta_h2 || (scale && zero)), PARE_ERR_SHAPE);
  PARE_REQUIRE(pare::aligned16(a) && lda % 8 == 0, PARE_ERR_ALIGN);
  if (producer == PARE_PRODUCER_RMSNORM) {
    PARE_REQUIRE(c != nullptr && lda >= K && resid_out != a, PARE_ERR_SHAPE);
    PARE_REQUIRE(pare::aligned16(c) && (b == nullptr || pare::aligned16(b)) && (resid_out == nullptr || pare::aligned16(resid_out)),
                 PARE_ERR_ALIGN);
  } else if (producer == PARE_PRODUCER_SILU_MUL) {
    PARE_REQUIRE(lda >= 2 * (int64_t)K, PARE_ERR_SHAPE);
  } else {
    return PARE_ERR_UNSUPPORTED;
  }
  pare::PeerCtx pc;
  int rc = make_peer_ctx(rank, world, buffers, buffer_bytes, &pc);
  if (rc != PARE_OK) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const pare::ProducerArgs prod{producer, a, b, c, resid_out, lda, eps};
  rc = pare::gemv_forward(nullptr, x_dtype, K, packed, scale, zero, meta_h2, nullptr, nullptr, bias, y, ldy, M, N, K,
                          group_size, workspace, workspace_bytes, s, nullptr, &prod, &pc);
  if (rc != PARE_ERR_UNSUPPORTED) return rc;
  // no fused staging for this shape: stand-alone glue kernel into the workspace's prepared-activation area, then the
  // prepared forward with the exchange in its epilogue
  PARE_REQUIRE(workspace && workspace_bytes >= pare_w4a16_workspace_bytes(M, N, K, group_size), PARE_ERR_WORKSPACE);
  void* prepared = reinterpret_cast<unsigned char*>(workspace) + pare::gemv::kCounterBytes;
  if (producer == PARE_PRODUCER_RMSNORM) {
    PARE_REQUIRE(lda == K, PARE_ERR_UNSUPPORTED);
    rc = pare_rmsnorm_residual(a, b, c, resid_out, nullptr, prepared, M, K, eps, x_dtype, stream);
  } else {
    rc = pare_silu_mul(a, nullptr, prepared, M, K, lda, x_dtype, stream);
  }
  if (rc != PARE_OK) return rc;
  return pare::gemv_forward(nullptr, x_dtype, K, packed, scale, zero, meta_h2, nullptr, nullptr, bias, y, ldy, M, N, K,
                            group_size, workspace, workspace_bytes, s, prepared, nullptr, &pc);
}

int pare_workspace_status(void* workspace, void* stream) {
  PARE_REQUIRE(workspace, PARE_ERR_WORKSPACE);
  return pare::read_and_clear_status(reinterpret_cast<int*>(workspace) + pare::gemv::kStatusIndex,
                                     reinterpret_cast<cudaStream_t>(stream));
}

int pare_selftest_bounded_wait(void* workspace, unsigned int polls, void* stream) {
  PARE_REQUIRE(workspace, PARE_ERR_WORKSPACE);
  PARE_REQUIRE(polls > 0 && polls <= 4096, PARE_ERR_SHAPE);   // a short wait by construction
  pare::bounded_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<int*>(workspace) + pare::gemv::kStatusIndex, polls);
  return cudaGetLastError() == cudaSuccess ? PARE_OK : PARE_ERR_CUDA;
}


}  // extern "C"
