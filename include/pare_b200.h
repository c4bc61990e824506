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
 *                indexed by the ORIGINAL column, before col_perm.  The division is done
 *                in fp32 and every kernel rounds the quotient to x_dtype before the
 *                product (what a caller gets who divides the activations himself).  The
 *                reference folds these scales into the weights offline
 *                (pare/schemes/awq.py:388-424) and has no run-time counterpart
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

/* Status word of a workspace.  Every wait inside the kernels (on a bulk copy, on another warp, on the CTAs of a
 * split) is bounded; one that runs out stores PARE_ERR_TIMEOUT in the workspace's status word, the kernel finishes
 * with whatever it has, and the call's result is then undefined.  pare_workspace_status synchronises `stream`,
 * returns the word (PARE_OK or PARE_ERR_TIMEOUT) and clears it; the word is sticky until read.  The same word
 * serves every entry point that takes this workspace (linear layers and decode attention).
 * pare_selftest_bounded_wait launches one thread that waits, through the kernels' own wait routine, at most
 * `polls` (<= 4096) polls on a shared-memory barrier that nothing arrives at, so the time-out path and this
 * accessor can be checked without a stuck kernel. */
int pare_workspace_status(void* workspace, void* stream);
int pare_selftest_bounded_wait(void* workspace, unsigned int polls, void* stream);

int pare_w4a16_forward(const void* x, int x_dtype, int64_t ldx,
                       const uint8_t* packed,
                       const float* scale, const float* zero, const void* meta_h2,
                       const int32_t* col_perm, const float* input_scale,
                       const void* bias,
                       void* y, int64_t ldy,
                       int M, int N, int K, int group_size,
                       void* workspace, size_t workspace_bytes,
                       void* stream);

/* ------------------------------------------------------------------------
 * Prepared activations: the M <= 16 path of pare_w4a16_forward in two halves, so that the
 * kernel which computes an activation (RMSNorm, SwiGLU, attention: below) can hand it to the
 * next linear in the order the streaming kernel consumes it, and the per-call preparation
 * launch disappears.  No counterpart in the reference (its Triton kernel reads x directly,
 * pare/kernels/matmul_int4.py:99-131).  A prepared buffer is opaque, 16-byte aligned,
 * pare_w4a16_prepared_bytes(M, K) bytes (0 if unsupported: M > 16 or K % 128 != 0), and tied to
 * the activation dtype.  pare_w4a16_prepare fills one from a plain x (applying the act-order
 * gather and the run-time input scale if given); pare_w4a16_forward_prepared is
 * pare_w4a16_forward minus x / col_perm / input_scale and needs K % 256 == 0, group % 128 == 0
 * (PARE_ERR_UNSUPPORTED otherwise: use the plain call). */
size_t pare_w4a16_prepared_bytes(int M, int K);
int pare_w4a16_prepare(const void* x, int x_dtype, int64_t ldx, const int32_t* col_perm, const float* input_scale,
                       int M, int K, void* prepared, void* stream);
int pare_w4a16_forward_prepared(const void* prepared, int x_dtype,
                                const uint8_t* packed, const float* scale, const float* zero, const void* meta_h2,
                                const void* bias, void* y, int64_t ldy, int M, int N, int K, int group_size,
                                void* workspace, size_t workspace_bytes, void* stream);

/* The same linear with its activations computed inside the streaming kernel from what a decode
 * step has at that point, so that the stand-alone RMSNorm / SwiGLU launch disappears (no
 * counterpart in the reference: model code).  M <= 16.
 *   PARE_PRODUCER_RMSNORM   x = rmsnorm(a + b) * c over the K columns; a = residual stream
 *                           [M][lda], b = delta [M][lda] or NULL, c = norm weight [K];
 *                           resid_out [M][lda] or NULL receives a + b (must not alias a)
 *   PARE_PRODUCER_SILU_MUL  x = silu(a[:, 0:K]) * a[:, K:2K]; a = fused gate|up [M][lda], lda >= 2 K
 * a, b, c, resid_out have the activation dtype, are 16-byte aligned, lda % 8 == 0.  Needs
 * K % 256 == 0 and group % 128 == 0 (PARE_ERR_UNSUPPORTED otherwise).  Cases the fused staging does
 * not cover (M > 4, a row longer than one CTA's K range) run as the stand-alone glue kernel
 * followed by pare_w4a16_forward_prepared on a part of the workspace: same result. */
enum { PARE_PRODUCER_RMSNORM = 1, PARE_PRODUCER_SILU_MUL = 2 };
int pare_w4a16_forward_produced(int producer, const void* a, const void* b, const void* c, void* resid_out,
                                int64_t lda, float eps, int x_dtype,
                                const uint8_t* packed, const float* scale, const float* zero, const void* meta_h2,
                                const void* bias, void* y, int64_t ldy, int M, int N, int K, int group_size,
                                void* workspace, size_t workspace_bytes, void* stream);


/* ------------------------------------------------------------------------
 * KIVI quantized KV cache.  Replaces the eager primitives and the cache
 * bookkeeping of pare/kv_cache.py: _quantize_keys :75-104, _quantize_values
 * :122-151, _dequantize_keys/_dequantize_values :107-119,154-156,
 * QuantizedKVCache._append_compressed/_reconstruct :294-325.
 *
 * Storage of ONE layer, owned and preallocated by the caller for `cap` tokens
 * (cap % 128 == 0); the reference grows six tensors with torch.cat instead:
 *   k_codes [B][H][cap][D*bits/8]           uint8, packed along channels (channel c of a
 *                                           token at bit c*bits of its row, little endian)
 *   k_scale, k_zero [B][H][cap/group][D]    fp32, per (token group, channel); zero = group min.
 *                                           When D % 128 == 0, channel c of a row sits at position
 *                                           (c & ~127) + ((c>>3)&3)*32 + ((c>>5)&3)*8 + (c&7): the order
 *                                           in which the decode-attention kernel reads it
 *   v_codes [B][H][cap/128][D][128*bits/8]  uint8, packed along tokens inside 128-token blocks
 *                                           (token t of the block at bit t*bits of row d)
 *   v_scale, v_zero [B][H][cap][D/v_group]  fp32, per (token, group of v_group channels): min/max over the
 *                                           group.  v_group == D (or 0) is the reference's form, one pair per
 *                                           token over all D channels; v_group == 32 is the finer grouping
 *                                           of the KIVI paper (not in the reference: _quantize_values with
 *                                           the channel axis viewed as [D/32][32])
 * bits in {2,4,8}; group in {16,32,64,128}; D % 32 == 0, D <= 256; v_group a multiple of 32 that divides D
 * (the fused attention takes v_group in {0, D, 32}).
 * Codes, scales and zeros are bit-identical to the reference's (same fp32 operation order).
 */

/* Quantize n_tokens (a multiple of group) tokens of k_src / v_src [B][H][n_tokens][D]
 * (src_dtype F16/BF16/F32, element strides stride_b/h/t, channels contiguous) and store
 * them as compressed tokens t0 .. t0+n_tokens-1 (t0 % group == 0).  pare/kv_cache.py:236-242. */
int pare_kivi_append(const void* k_src, const void* v_src, int src_dtype,
                     int64_t stride_b, int64_t stride_h, int64_t stride_t,
                     int n_tokens, int t0,
                     uint8_t* k_codes, float* k_scale, float* k_zero,
                     uint8_t* v_codes, float* v_scale, float* v_zero,
                     int B, int H, int D, int bits, int group, int v_group, int cap, void* stream);

/* Dense reconstruction code*scale+zero of compressed tokens 0..n_comp-1 into
 * out_k / out_v [B][H][>=n_comp][D] (out_dtype F16/BF16/F32, element strides given).
 * pare/kv_cache.py:315-325 (the part of update()'s return value that comes from the
 * compressed store). */
int pare_kivi_dequant(const uint8_t* k_codes, const float* k_scale, const float* k_zero,
                      const uint8_t* v_codes, const float* v_scale, const float* v_zero,
                      int B, int H, int D, int bits, int group, int v_group, int cap, int n_comp,
                      void* out_k, void* out_v, int out_dtype,
                      int64_t stride_b, int64_t stride_h, int64_t stride_t, void* stream);

/* Fused dequantize + decode attention for ONE query token per sequence:
 *   out[b][hq][:] = softmax(q[b][hq] . K^T * softmax_scale) . V   over n_comp compressed
 * tokens followed by n_res full-precision residual tokens, grouped-query sharing
 * (query head hq reads KV head hq / (Hq/H), Hq/H <= 8).  The reference has no such
 * function: a caller runs scaled_dot_product_attention on update()'s dense return
 * (pare/kv_cache.py:183-186); this call gives the same result without materialising it.
 *   q, out        [B][Hq][D] dtype F16/BF16, element strides *_stride_b / *_stride_h
 *   res_k, res_v  [B][H][n_res][D] same dtype, element strides res_stride_b/h/t (multiples of 8)
 *   new_k, new_v  NULL, or the newest token [B][H][D] (element strides new_stride_b/h, multiples
 *                 of 8, 16-byte aligned): it is attended to as window position n_res-1 AND stored
 *                 there by this call (the append of pare/kv_cache.py:229-231 for one token), so
 *                 the caller copies nothing; positions 0..n_res-2 must already be in the window
 *   rope          NULL, or D floats (16-byte aligned) cos[0..D/2) then sin[0..D/2) of the newest token's
 *                 position: q and new_k get the rotary embedding (pairs i, i + D/2:
 *                 x'[i] = x[i] cos[i] - x[i+D/2] sin[i], x'[i+D/2] = x[i+D/2] cos[i] + x[i] sin[i], rounded to
 *                 the dtype) before they are used, and new_k is stored rotated -- the step a model
 *                 takes between its q|k|v projection and the cache (not part of the reference, whose
 *                 callers hand update() keys that are already rotated)
 *   out           may be NULL when prepared_out is given
 *   prepared_out  NULL, or a pare_w4a16_prepared_bytes(B, Hq*D) buffer that receives the result as
 *                 prepared activations of the next W4A16 linear (B <= 16)
 * D == 128, bits == 4 or 2, group in {16, 32, 64, 128}, n_res <= 512, B * H < 16383.
 * Context length: the compressed tokens are cut into at most 250 splits per (batch, KV head), each
 * a run of blocks of 128 tokens; a split takes as many blocks as that bound needs, so n_comp is
 * limited only by `cap` and the workspace (beyond 64 blocks per split the planner merely stops
 * balancing waves).
 * Number range: BF16 keys and values of the residual window go to the tensor cores in their own
 * type; the probabilities are split into value + rounding residual in the window's type.  The
 * compressed path multiplies q by the key scale in fp32 and rounds the product (and the
 * probabilities times the value scale) to fp16 pairs, so |q * k_scale| and p * v_scale must stay
 * below 65504: value ranges (max - min per token) below 15 * 65504 (4-bit) -- any activations a
 * 16-bit model produces.
 * workspace: pare_kivi_attn_workspace_bytes(), zero-filled once (same contract and status word as
 * the W4A16 workspace; one buffer may serve both). */
size_t pare_kivi_attn_workspace_bytes(int B, int H, int n_comp, int n_res);

int pare_kivi_decode_attn(const void* q, int dtype, int64_t q_stride_b, int64_t q_stride_h,
                          const uint8_t* k_codes, const float* k_scale, const float* k_zero,
                          const uint8_t* v_codes, const float* v_scale, const float* v_zero,
                          int n_comp,
                          void* res_k, void* res_v,
                          int64_t res_stride_b, int64_t res_stride_h, int64_t res_stride_t, int n_res,
                          const void* new_k, const void* new_v, int64_t new_stride_b, int64_t new_stride_h,
                          const float* rope,
                          void* out, int64_t out_stride_b, int64_t out_stride_h, void* prepared_out,
                          float softmax_scale,
                          int B, int Hq, int H, int D, int bits, int group, int v_group, int cap,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Attention of Tq new tokens over Tk >= Tq full-precision keys / values (the new tokens are the last Tq of them):
 *   out[b][hq][i] = softmax_j(q[b][hq][i] . k[b][hq / (Hq/H)][j] * softmax_scale) . v[b][hq / (Hq/H)][j],
 * with causal != 0 over the keys j <= i + (Tk - Tq) only.  This is the prompt's attention BEFORE the cache
 * compresses the tokens: the reference's caller runs scaled_dot_product_attention on update()'s return
 * (pare/kv_cache.py:183-186, 205-252), which for a prompt is mostly the lossy reconstruction.
 *   q, out [B][Hq][Tq][D], k, v [B][H][Tk][D]; dtype F16/BF16; element strides per tensor (multiples of 8),
 *   channels contiguous, 16-byte aligned; D == 128.  No workspace. */
int pare_prefill_attn(const void* q, const void* k, const void* v, void* out, int dtype,
                      int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_t,
                      int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_t,
                      int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_t,
                      int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_t,
                      int B, int Hq, int H, int Tq, int Tk, int D, float softmax_scale, int causal, void* stream);

/* ------------------------------------------------------------------------
 * Decode-step glue (no counterpart in the reference library: model code around the two hot
 * kernels).  y = rmsnorm(x + delta) * weight, optionally storing x + delta; and the SwiGLU
 * gate out = silu(gate) * up over a fused [rows][2n] gate|up projection.  dtype F16/BF16.
 * prepared_out (NULL, or pare_w4a16_prepared_bytes(rows, n) bytes, rows <= 16, n % 128 == 0)
 * receives the result as prepared activations of the next W4A16 linear; y / out may then be NULL. */
int pare_rmsnorm_residual(const void* x, const void* delta, const void* weight, void* resid_out, void* y,
                          void* prepared_out, int rows, int n, float eps, int dtype, void* stream);
int pare_silu_mul(const void* gate_up, void* out, void* prepared_out, int rows, int n, int64_t ld, int dtype,
                  void* stream);

/* Rotary embedding of a prompt's q or k (model code in front of the cache, like the `rope` argument of
 * pare_kivi_decode_attn for one token): out [B][H][T][D] dense = x [B][H][T][D] (element strides stride_b/h/t,
 * channels contiguous) rotated with rows [T][D] floats, cos[0..D/2) then sin[0..D/2) per token, pairs (i, i + D/2):
 * x'[i] = x[i] cos[i] - x[i+D/2] sin[i], x'[i+D/2] = x[i+D/2] cos[i] + x[i] sin[i]; fp32 products and sum, each
 * rounded, then rounded to the dtype (F16 / BF16).  No counterpart in the reference, whose callers rotate. */
int pare_rope(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_t, void* out, const float* rows,
              int B, int H, int T, int D, int dtype, void* stream);

/* ------------------------------------------------------------------------
 * W4A16 decode linear without any caller-provided workspace.  No counterpart in the reference;
 * it exists for callers that cannot allocate device memory (code running inside another
 * runtime's callback or memory pool where cudaMalloc is forbidden or would synchronise, or code
 * that only ever receives input and output pointers).  Same arguments and results as
 * pare_w4a16_forward for M <= 16, minus the workspace: the scratch is a fixed 16 MiB array inside
 * the library's device image (every GPU that loads the library holds it until the process exits).
 *   - Layers whose scratch need (pare_w4a16_workspace_bytes) exceeds
 *     pare_w4a16_static_scratch_bytes() are rejected with PARE_ERR_WORKSPACE; M > 16 with
 *     PARE_ERR_UNSUPPORTED.
 *   - Calls nothing that allocates.  The first call on each device looks up the array's device
 *     address; make that first call outside any stream capture.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams) race; order them on one stream. */
size_t pare_w4a16_static_scratch_bytes(void);
/* status word of the array (see pare_workspace_status): synchronises `stream`, returns and clears it */
int pare_w4a16_static_status(void* stream);

int pare_w4a16_forward_static(const void* x, int x_dtype, int64_t ldx,
                              const uint8_t* packed,
                              const float* scale, const float* zero, const void* meta_h2,
                              const int32_t* col_perm, const float* input_scale,
                              const void* bias,
                              void* y, int64_t ldy,
                              int M, int N, int K, int group_size,
                              void* stream);

/* ------------------------------------------------------------------------
 * One-shot all-reduce of a small activation tensor over NVLink peer memory, for tensor-parallel
 * decode (the two partial sums per block after the row-parallel o and down projections).  No
 * counterpart in the reference, which is single-GPU.  Every rank stores its partial into every
 * peer's exchange buffer (plain peer stores; each 8 bytes travel with their own validity marks, so
 * there is no fence and no separate flag) and adds the partials from its own buffer in rank order as
 * they arrive (bounded waits): fp32, deterministic, the same bits on every rank; one launch.
 *   pare_peer_buffer_create  allocates and zeroes this rank's exchange buffer and returns its
 *                            64-byte CUDA IPC handle (to be sent to the peers by any host channel)
 *   pare_peer_buffer_open    maps a peer's buffer from its handle; _close unmaps; _destroy frees
 *   pare_peer_allreduce      y = sum over ranks of x, [rows][cols] F16/BF16, cols % 4 == 0,
 *                            rows*cols*4 <= (buffer_bytes - 4096) / 2 / (2 * world); buffers = HOST array
 *                            of `world` device pointers (own buffer at index `rank`); 2 <= world <= 8;
 *                            every rank makes the same sequence of calls; capturable in a CUDA graph
 *   pare_peer_status         0 or PARE_ERR_TIMEOUT (a wait for a peer ran out); synchronises `stream`
 * The create / open / close / destroy calls are the only ones in this library that allocate. */
int pare_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]);
int pare_peer_buffer_open(const unsigned char handle[64], void** ptr);
int pare_peer_buffer_close(void* ptr);
int pare_peer_buffer_destroy(void* ptr);
int pare_peer_status(const void* own_buffer, void* stream);
int pare_peer_allreduce(const void* x, int64_t ldx, void* y, int64_t ldy, int rows, int cols, int dtype,
                        int rank, int world, void* const* buffers, size_t buffer_bytes, void* stream);

/* Row-parallel W4A16 linears of a tensor-parallel model with the sum over the ranks INSIDE the kernel: the
 * prepared / produced forwards above (M <= 16), where the thread that finishes an output element stores its fp32
 * partial into that element's slot of every rank's exchange buffer (plain 8-byte peer stores, each with its own
 * validity mark) and adds the ranks' partials from its own buffer in rank order as they arrive (bounded waits ->
 * PARE_ERR_TIMEOUT in the buffer's status word, read with pare_peer_status).  y is the complete sum on every rank,
 * identical bits everywhere, rounded once; there is no separate all-reduce launch.  No counterpart in the reference
 * (single GPU).  buffers / buffer_bytes / rank / world as for pare_peer_allreduce (the buffers' data area is split
 * between the two calls, so both may be used on the same buffers); M * N * 8 bytes must fit a slot:
 * (buffer_bytes - 4096) / 2 / (2 * world).  Every rank makes the same sequence of calls; a bias given on several
 * ranks is added once per rank that gives it (give it on one).  PARE_ERR_UNSUPPORTED for shapes the streaming
 * kernels do not take (K % 256, group % 128): run the plain call and pare_peer_allreduce then. */
int pare_w4a16_forward_prepared_allreduce(const void* prepared, int x_dtype,
                                          const uint8_t* packed, const float* scale, const float* zero, const void* meta_h2,
                                          const void* bias, void* y, int64_t ldy, int M, int N, int K, int group_size,
                                          void* workspace, size_t workspace_bytes,
                                          int rank, int world, void* const* buffers, size_t buffer_bytes, void* stream);
int pare_w4a16_forward_produced_allreduce(int producer, const void* a, const void* b, const void* c, void* resid_out,
                                          int64_t lda, float eps, int x_dtype,
                                          const uint8_t* packed, const float* scale, const float* zero, const void* meta_h2,
                                          const void* bias, void* y, int64_t ldy, int M, int N, int K, int group_size,
                                          void* workspace, size_t workspace_bytes,
                                          int rank, int world, void* const* buffers, size_t buffer_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PARE_B200_H */
