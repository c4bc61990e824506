/*
 * pare_b200.h — C ABI of libpare_b200.so (CUDA, sm_100a).
 *
 * The library replaces the two run-time hot paths of the Pare quantization
 * toolkit with hand-written CUDA:
 *   - the fused INT4 dequantize-matmul behind QuantizedLinear.forward(use_kernel=True)
 *   - the KIVI quantized KV cache (quantize-on-append, dequantize, decode attention)
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host".
 *   - Every call is asynchronous on `stream` (a cudaStream_t passed as void*),
 *     allocates nothing, never synchronises the host, and can be captured in a
 *     CUDA graph.  The caller owns all buffers, including workspaces.
 *   - Return value: 0 (PARE_OK) or a PARE_ERR_* code.  Nothing throws, exits or traps.
 *   - dtype codes: 0 = float16, 1 = bfloat16, 2 = float32.
 */
#ifndef PARE_B200_H
#define PARE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  PARE_OK = 0,
  PARE_ERR_SHAPE = 1,        /* a size is zero/negative or violates a divisibility rule */
  PARE_ERR_DTYPE = 2,        /* dtype code not supported by this entry point */
  PARE_ERR_ALIGN = 3,        /* a pointer or leading dimension breaks the 16-byte rule */
  PARE_ERR_WORKSPACE = 4,    /* workspace missing or smaller than *_workspace_bytes() */
  PARE_ERR_UNSUPPORTED = 5,  /* valid request that no kernel covers */
  PARE_ERR_CUDA = 6,         /* the CUDA runtime reported an error at launch */
  PARE_ERR_TIMEOUT = 7       /* a bounded device-side wait gave up */
};

enum { PARE_F16 = 0, PARE_BF16 = 1, PARE_F32 = 2 };

/* Library version, major*10000 + minor*100 + patch. */
int pare_version(void);

/* Static, human-readable name of a status code (host pointer, never NULL). */
const char* pare_status_string(int status);

/* ------------------------------------------------------------------------
 * W4A16 fused dequantize-matmul:  Y[M,N] = X[M,K] . dequant(W)[N,K]^T (+ bias)
 *
 * Replaces pare/kernels/matmul_int4.py:183-243 (matmul_w4a16 + _w4a16_kernel),
 * called from QuantizedLinear._forward_kernel, pare/layers/linear.py:140-159.
 * Unlike the reference kernel it reads the STORAGE layout of pack_int4
 * (pare/core/pack.py:29-48) directly: packed[n][j] holds column 2j in bits 0..3
 * and column 2j+1 in bits 4..7.
 *
 *   x            [M, ldx]  x_dtype (F16 or BF16), row-major, ldx >= K
 *   packed       [N, K/2]  uint8
 *   scale, zero  [N, K/group_size] float32 — QuantizedLinear.scale / .zero with
 *                the trailing unit axis dropped; W = (q - zero) * scale
 *   meta_h2      optional [N, K/group_size] pairs of float16 (scale, zero); when
 *                non-NULL it is read INSTEAD of scale/zero (half the metadata bytes)
 *   col_perm     optional [K] int32: packed column j multiplies x[:, col_perm[j]]
 *                (columns sorted by GPTQ act-order group; NULL = identity)
 *   input_scale  optional [K] float32: x[:, k] is divided by input_scale[k]
 *                (AWQ per-input-channel scale applied at run time; NULL = none);
 *                indexed by the ORIGINAL column, before col_perm
 *   bias         optional [N] x_dtype
 *   y            [M, ldy]  x_dtype
 *   workspace    pare_w4a16_workspace_bytes() bytes, zero-filled ONCE by the caller
 *                before first use; calls leave it zero-consistent again.  Calls that
 *                share a workspace must be ordered on one stream.
 *
 * Any M >= 1.  M <= 16 runs the streaming dequant-GEMV; larger M runs the
 * tensor-core tile kernel.  Requires K % 2 == 0 and K % group_size == 0
 * (per_channel layers pass group_size = K).
 */
size_t pare_w4a16_workspace_bytes(int M, int N, int K, int group_size);

int pare_w4a16_forward(const void* x, int x_dtype, int64_t ldx,
                       const uint8_t* packed,
                       const float* scale, const float* zero, const void* meta_h2,
                       const int32_t* col_perm, const float* input_scale,
                       const void* bias,
                       void* y, int64_t ldy,
                       int M, int N, int K, int group_size,
                       void* workspace, size_t workspace_bytes,
                       void* stream);

/* Tuning override for experiments (host state, process-wide, not thread-safe):
 * row blocks of 16 per warp, K splits, prefetch depth; 0 = choose automatically. */
void pare_w4a16_set_tuning(int row_blocks, int k_splits, int prefetch);

#ifdef __cplusplus
}
#endif
#endif /* PARE_B200_H */
