/*
 * q8_kernels_b200 -- C ABI of the B200 (sm_100a) 8-bit DiT inference kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches asynchronously on that
 * stream, allocates nothing and never synchronises.  The return value is 0 on
 * success or a negative Q8K_ERR_* code; q8k_error_string() explains it and
 * q8k_last_error_detail() gives the message of the last failing call on the
 * calling thread.
 *
 * Each function names the entry point of the reference extension modules
 * (q8_kernels_cuda.{quantizer,ops,gemm,flash_attention}._C) it stands in for,
 * by the reference's file path and line.
 */
#ifndef Q8_KERNELS_B200_H
#define Q8_KERNELS_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define Q8K_API __attribute__((visibility("default")))
#else
#define Q8K_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- return codes ------------------------------------------------------- */
#define Q8K_OK                 0
#define Q8K_ERR_INVALID_ARG   -1   /* null pointer, bad size, bad alignment      */
#define Q8K_ERR_UNSUPPORTED   -2   /* dtype / shape combination not implemented  */
#define Q8K_ERR_WORKSPACE     -3   /* caller-provided scratch too small          */
#define Q8K_ERR_CUDA          -4   /* a CUDA runtime / driver call failed        */
#define Q8K_ERR_TOO_LARGE     -5   /* problem exceeds a fixed built-in capacity  */

/* ---- element types ------------------------------------------------------ */
#define Q8K_DT_F32   0
#define Q8K_DT_F16   1
#define Q8K_DT_BF16  2
#define Q8K_DT_E4M3  3   /* float8_e4m3fn */
#define Q8K_DT_I8    4

/* ---- device status word --------------------------------------------------
 * The tensor-core kernels (GEMM, attention) bound every mbarrier wait.  When a
 * wait gives up the kernel records  Q8K_STATUS_TIMEOUT | (site << 8)  in the
 * int32 the caller passed as `dev_status` (may be NULL), drains and exits; the
 * CUDA context stays usable.  The word is only ever written on failure, so one
 * zero-initialised int32 per device can be shared by all calls.              */
#define Q8K_STATUS_TIMEOUT  0x1

Q8K_API int         q8k_version(void);
/* Self-test of the bounded wait: one warp waits on a barrier that nothing signals, gives up after
 * `tries` (1..65536) tests and records  Q8K_STATUS_TIMEOUT | (9 << 8)  in *dev_status.  The kernel
 * returns normally and the context stays usable.  No counterpart in the reference.              */
Q8K_API int         q8k_wait_selftest(int* dev_status, unsigned tries, void* stream);
Q8K_API const char* q8k_error_string(int code);
Q8K_API const char* q8k_last_error_detail(void);

/* Per-row absmax quantizer.  x [rows, dim] (row stride x_row_stride elements)
 * -> q [rows, dim] int8 (round half away from zero) or e4m3 (RNE, overflow ->
 * NaN) and scales[rows] = absmax / QMAX.  An all-zero row gives q = 0,
 * scale = 0.  dim must be a multiple of 16.
 * Replaces tokenwise_quant: csrc/quantizer/tokenwise_quant.cpp:74-111,
 * csrc/quantizer/tokenwise_quant_cuda.cu:91-149.                              */
Q8K_API int q8k_tokenwise_quant(const void* x, int x_dtype, void* q, int q_dtype, float* scales,
                        int64_t rows, int dim, int64_t x_row_stride, void* stream);

/* Fast Walsh-Hadamard transform of every row (zero-padded to the next power of
 * two, fp32 butterflies in ascending stride order), out = cast(y * scale).
 * x bf16|e4m3, out bf16|e4m3; dim a multiple of 8, at most 16384.
 * Replaces fast_hadamard_transform:
 * csrc/fast_hadamard/fast_hadamard_transform.cpp:70-121,
 * csrc/fast_hadamard/fast_hadamard_transform_cuda.cu:42-111.                  */
Q8K_API int q8k_fast_hadamard_transform(const void* x, int x_dtype, void* out, int out_dtype,
                                int64_t rows, int dim, int64_t x_row_stride, float scale,
                                void* stream);

/* Fused producer for the linear layers: Hadamard (rounded to the input dtype,
 * as the unfused chain does) followed by the per-row quantizer, one pass over
 * x.  Bit-identical to q8k_fast_hadamard_transform + q8k_tokenwise_quant.
 * Replaces the chain in q8_kernels/functional/linear.py:30-31,143-145.        */
Q8K_API int q8k_hadamard_quant(const void* x, int x_dtype, void* q, int q_dtype, float* scales,
                       int64_t rows, int dim, int64_t x_row_stride, float scale, void* stream);

/* The whole pre-linear chain of an LTX block in one pass over x: RMS norm without affine weight,
 * adaLN modulation n*(1+s)+h with per-batch bf16 rows s, h ([rows/rows_per_mod, dim]), Hadamard
 * (times `scale`) and the per-row quantizer, with the bf16 roundings of the separate ops
 * (q8_kernels/blocks/ltx_transformer_block.py:38-39,53-54 followed by functional/linear.py:30-31).
 * x bf16 [rows, dim] contiguous, dim in (256, 8192], a multiple of 16.  Equal to the unfused chain
 * up to the fp32 summation order of the mean square (a row's 1/rms may differ by one ulp).        */
Q8K_API int q8k_norm_modulate_quant(const void* x, const void* mod_scale, const void* mod_shift, void* q, int q_dtype,
                            float* scales, int64_t rows, int dim, int64_t rows_per_mod, float scale,
                            void* stream);

/* RMS norm without eps: r = rsqrt(mean(x^2)), out = (x*r)*w (w fp32 or NULL),
 * rrms[rows] = r (may be NULL).  x, out bf16|e4m3; dim a multiple of 16.
 * Replaces rms_norm: csrc/ops/rms_norm.cpp:103-154, rms_norm_cuda.cu:100-171. */
Q8K_API int q8k_rms_norm(const void* x, int x_dtype, const float* weights, void* out, int out_dtype,
                 float* rrms, int64_t rows, int dim, void* stream);

/* Interleaved-pair rotary embedding with per-element fp32 cos/sin tables that
 * have x's shape; `freq_rows` > 0 makes the tables repeat every freq_rows rows
 * (one table shared by all batch entries), 0 means one table row per x row.
 * Replaces rope: csrc/ops/rope.cpp:96-146, rope_cuda.cu:67-106.               */
Q8K_API int q8k_rope(const void* x, int x_dtype, const float* cos_freqs, const float* sin_freqs,
             void* out, int out_dtype, int64_t rows, int dim, int64_t freq_rows, void* stream);

/* out_e4m3 = cast(float(x_e4m3) * (y + scale_add) + z); row r of x uses row
 * r / y_every of y and r / z_every of z.  (y,z) dtypes: (f32,f32), (f32,e4m3),
 * (bf16,bf16).  Replaces fma_8bit: csrc/ops/fma.cpp:72-118, fma_cuda.cu:60-98. */
Q8K_API int q8k_fma_8bit(const void* x, const void* y, int y_dtype, const void* z, int z_dtype, void* out,
                 int64_t rows, int dim, int64_t y_every, int64_t z_every, float scale_add,
                 void* stream);

/* tanh-GELU, x/out bf16|e4m3.  Replaces gelu_forward:
 * csrc/ops/gelu_act.cpp:132-172, gelu_forward_cuda.cu:72-100.                 */
Q8K_API int q8k_gelu_forward(const void* x, int x_dtype, void* out, int out_dtype, int64_t rows, int dim,
                     void* stream);

/* Training-side gradients of the row-wise ops (forward-only users never call these).  The incoming
 * gradient is read in the OUTPUT dtype, as the reference's kernels do.
 *   gelu_backward:     csrc/ops/gelu_act.cpp:84-129, gelu_backward_cuda.cu:88-100
 *   rope_backward:     csrc/ops/rope.cpp:150-199, rope_backward_cuda.cu:101-110 (freq_rows as in q8k_rope)
 *   rms_norm_backward: csrc/ops/rms_norm.cpp:157-214, rms_norm_backward_cuda.cu:135-160; x_normed is the
 *                      forward output, x_norms the per-row rsqrt it returned, weights fp32 or NULL     */
Q8K_API int q8k_gelu_backward(const void* x, int x_dtype, const void* grad_out, void* out, int out_dtype,
                      int64_t rows, int dim, void* stream);
Q8K_API int q8k_rope_backward(const void* grad_out, int grad_dtype, const float* cos_freqs, const float* sin_freqs,
                      void* out, int out_dtype, int64_t rows, int dim, int64_t freq_rows, void* stream);
Q8K_API int q8k_rms_norm_backward(const void* x_normed, int x_dtype, const float* x_norms, const void* grad_out,
                          const float* weights, void* out, int out_dtype, int64_t rows, int dim,
                          void* stream);

/* 8-bit GEMM  C[b] = act((A[b] . B[b]^T) * (sa[m]*sb[n]) + bias[n]).
 * A [bs_a, M, K], B [bs_b, N, K] K-contiguous int8 (q8k_q8_mm) or e4m3
 * (q8k_fp8_mm); bs_a == bs_b or one of them 1; sa [bs_a, M], sb [bs_b, N],
 * bias [N] fp32 or NULL; C [max(bs_a,bs_b), M, N] bf16 (RNE) or e4m3
 * (saturating).  N % 16 == 0, K % 16 == 0, all pointers 16-byte aligned.
 * Replaces q8_mm / q8_mm_bias / fp8_mm / fp8_mm_bias:
 * csrc/gemm/q8_gemm_api.cpp:40-291 and the run_* launchers declared at :27-35. */
Q8K_API int q8k_q8_mm(const void* a, const void* b, const float* bias, const float* a_scales,
              const float* b_scales, void* out, int out_dtype, int bs_a, int bs_b,
              int M, int N, int K, int fuse_gelu, int* dev_status, void* stream);
Q8K_API int q8k_fp8_mm(const void* a, const void* b, const float* bias, const float* a_scales,
               const float* b_scales, void* out, int out_dtype, int bs_a, int bs_b,
               int M, int N, int K, int fuse_gelu, int* dev_status, void* stream);

/* GEMM with the block's gated residual folded into the epilogue:
 *   out[m,n] = bf16( bf16( gate[m / rows_per_gate, n] * bf16(y[m,n]) ) + resid[m,n] ),  y = (A.B^T)*(sa*sb) + bias
 * gate (bf16, [ceil(rows/rows_per_gate), N], may be NULL for a plain residual add) and resid (bf16,
 * [batch*M, N]) follow the roundings of the separate torch ops they replace
 * (`gate_msa * attn_output + hidden_states`, q8_kernels/blocks/ltx_transformer_block.py:41,52,56),
 * so the result is bit-identical to q8_mm_bias followed by those ops.  int8 != 0 selects INT8
 * operands, else e4m3.  Output bf16 [max(bs_a,bs_b), M, N].                                        */
Q8K_API int q8k_mm_gate_residual(int int8, const void* a, const void* b, const float* bias, const float* a_scales,
                         const float* b_scales, const void* gate, const void* resid, int64_t rows_per_gate,
                         void* out, int bs_a, int bs_b, int M, int N, int K, int* dev_status, void* stream);

/* FP8 flash-attention forward, head dim 64.  q [B,H,M,64], k [B,H,N,64],
 * vt [B,H,64,ceil16(N)] e4m3 contiguous; out [B,H,M,64] e4m3 (saturating) or
 * bf16; key_lens int32 [B] valid keys per batch entry or NULL.  KV blocks are
 * visited last to first with an exact running max.
 * Replaces flash_attention: csrc/flash_attention/flash_attention.cpp:18-48 and
 * the launchers declared at :9-16.                                            */
Q8K_API int q8k_flash_attention(const void* q, const void* k, const void* vt, void* out, int out_dtype,
                        int B, int H, int M, int N, float softmax_scale, const int* key_lens,
                        int* dev_status, void* stream);

/* Same kernel with an explicit output layout: element (b, h, row, d) is written at
 * out[b*out_stride_b + h*out_stride_h + row*out_stride_s + d] (strides in elements, multiples of 16).
 * With strides (M*H*64, 64, H*64) the result lands as [B, M, H*64], which is what the attention
 * module feeds to its output projection, so the transpose copy of
 * q8_kernels/modules/attention.py:101-103 disappears.                                            */
Q8K_API int q8k_flash_attention_strided(const void* q, const void* k, const void* vt, void* out, int out_dtype,
                                int B, int H, int M, int N, int64_t out_stride_b, int64_t out_stride_h,
                                int64_t out_stride_s, float softmax_scale, const int* key_lens,
                                int* dev_status, void* stream);

/* q8k_flash_attention_strided with n_out (1..8) destinations: the finished output tile is stored, with the
 * same strides, at outs[0..n_out-1].  Destinations may be buffers of other GPUs mapped into this process
 * (q8k_ipc_open below): with attention sharded by head every rank then writes its heads straight into every
 * rank's full [B,S,H,64] buffer over NVLink and no all-gather is needed afterwards, only a barrier.  Stores
 * only: the kernel reads nothing from a peer and waits on none.  No reference counterpart (the reference is
 * single-GPU).                                                                                          */
Q8K_API int q8k_flash_attention_multi_out(const void* q, const void* k, const void* vt, void* const* outs, int n_out,
                                  int out_dtype, int B, int H, int M, int N, int64_t out_stride_b,
                                  int64_t out_stride_h, int64_t out_stride_s, float softmax_scale,
                                  const int* key_lens, int* dev_status, void* stream);

/* q8k_flash_attention_multi_out with V given as ROWS, v [B,H,N,64] e4m3 (the layout of k; no transpose, no
 * padding of the key dim): the tensor core reads the V tile as an MN-major operand.  Same arithmetic, same
 * bits as the transposed form.  This is what the attention module calls; the transposed entry points above
 * keep the reference's layout (q8_kernels/functional/flash_attention.py:40-48 builds it).                 */
Q8K_API int q8k_flash_attention_v_rows(const void* q, const void* k, const void* v, void* const* outs, int n_out,
                               int out_dtype, int B, int H, int M, int N, int64_t out_stride_b,
                               int64_t out_stride_h, int64_t out_stride_s, float softmax_scale,
                               const int* key_lens, int* dev_status, void* stream);

/* bf16 [B,H,S,64] view (element strides, last dim contiguous) -> e4m3 [B,H,S,64] contiguous, c10-style cast
 * (the `.to(float8_e4m3fn)` of q8_kernels/functional/flash_attention.py:47-48 without the transpose).     */
Q8K_API int q8k_attention_cast_rows(const void* x, void* out8, int B, int H, int S, int64_t stride_b, int64_t stride_s,
                            int64_t stride_h, void* stream);

/* Set-up helpers for peer destinations (host side, no kernel): export the CUDA IPC handle of the device
 * allocation that contains ptr plus ptr's offset in it; map such an allocation of another process into this
 * one with the calling thread's current device (peer access is enabled by the mapping) and return the
 * address of the same offset; unmap it again.                                                            */
#define Q8K_IPC_HANDLE_BYTES 64
Q8K_API int q8k_ipc_export(const void* ptr, unsigned char handle[Q8K_IPC_HANDLE_BYTES], int64_t* offset);
Q8K_API int q8k_ipc_open(const unsigned char handle[Q8K_IPC_HANDLE_BYTES], int64_t offset, void** ptr);
Q8K_API int q8k_ipc_close(void* ptr, int64_t offset);

/* Pre-pass of the attention call: from bf16 q,k,v given as strided [B,S,H,64]
 * views (strides in elements, last dim contiguous) produce q8,k8 [B,H,S,64]
 * e4m3 (Hadamard-rotated times qk_scale when apply_hadamard, else plain cast)
 * and vt [B,H,64,ceil16(S_kv)] e4m3 (transposed, zero padded).
 * Replaces the torch glue in q8_kernels/functional/flash_attention.py:30-60.  */
Q8K_API int q8k_attention_prep(const void* q, const void* k, const void* v,
                       void* q8, void* k8, void* vt8,
                       int B, int H, int S_q, int S_kv,
                       int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                       int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                       int64_t v_stride_b, int64_t v_stride_s, int64_t v_stride_h,
                       int apply_hadamard, float qk_scale, void* stream);

/* Q or K after its projection, in one pass per tensor: RMS norm over all H*64 channels with the fp32
 * weight norm_w (result rounded to bf16), optional rotary embedding with fp32 tables [S, H*64] shared
 * by the batch (rounded to bf16; pass NULL tables to skip), per-head 64-point Hadamard times qk_scale
 * when apply_hadamard, c10 e4m3 cast, output head-major [B,H,S,64].  x bf16 rows of H*64 channels with
 * row stride x_row_stride.  Replaces q_norm/k_norm + apply_rope of q8_kernels/modules/attention.py:54-68
 * and the Q/K half of the glue in functional/flash_attention.py:50-54; q8k_attention_prep_v is the V
 * half (transpose, zero pad, cast) of q8k_attention_prep on its own.                                  */
Q8K_API int q8k_qk_norm_rope_prep(const void* x, int64_t x_row_stride, const float* norm_w, const float* cos_t,
                          const float* sin_t, void* out8, int B, int S, int H, int apply_hadamard,
                          float qk_scale, void* stream);
/* The same for Q and K of one self-attention in a single launch (both [B*S, H*64] with the same row
 * stride, e.g. two column slices of one fused projection output): the rotary table rows are read once. */
Q8K_API int q8k_qk_norm_rope_prep_pair(const void* xq, const void* xk, int64_t x_row_stride, const float* norm_wq,
                               const float* norm_wk, const float* cos_t, const float* sin_t, void* outq8,
                               void* outk8, int B, int S, int H, int apply_hadamard, float qk_scale, void* stream);
/* q8k_qk_norm_rope_prep_pair plus the V of the same self-attention (a third slice of the fused projection
 * output, same row stride): V is only cast to e4m3 (the .to(float8_e4m3fn) of
 * q8_kernels/functional/flash_attention.py:48) and written as rows [B,H,S,64], the layout
 * q8k_flash_attention_v_rows reads.  One launch for everything between the QKV projection and the
 * attention kernel.  xq, norm_wq and outq8 may all be NULL: K and V only (cross-attention, where Q is
 * projected from another tensor).                                                                */
Q8K_API int q8k_qkv_prep(const void* xq, const void* xk, const void* xv, int64_t x_row_stride, const float* norm_wq,
                 const float* norm_wk, const float* cos_t, const float* sin_t, void* outq8, void* outk8,
                 void* outv8, int B, int S, int H, int apply_hadamard, float qk_scale, void* stream);
Q8K_API int q8k_attention_prep_v(const void* v, void* vt8, int B, int H, int S_kv, int64_t v_stride_b,
                         int64_t v_stride_s, int64_t v_stride_h, void* stream);

/* Whole activation side of Q8Linear / FP8Linear in one call: fused Hadamard +
 * per-token quantizer into caller-provided scratch, then the GEMM.
 * x bf16 [M,K]; w int8|e4m3 [N,K] with w_scales [N]; workspace must hold
 * q8k_linear_workspace_bytes(M,K) bytes, 256-byte aligned.
 * Replaces Q8LinearFunc.forward / FP8LinearFunc.forward:
 * q8_kernels/functional/linear.py:24-42,138-159.                              */
Q8K_API size_t q8k_linear_workspace_bytes(int M, int K);
Q8K_API int q8k_linear(const void* x, int x_dtype, const void* w, int w_dtype, const float* w_scales,
               const float* bias, void* out, int out_dtype, int M, int N, int K,
               int use_hadamard, int fuse_gelu, void* workspace, size_t workspace_bytes,
               int* dev_status, void* stream);

/* q8k_linear without any allocation on either side of the call.  No counterpart in the
 * reference: it exists for callers that cannot obtain device scratch at call time -- a plugin
 * living inside a host runtime that has reserved the whole device heap and hands a plugin nothing
 * but its input and output buffers, or a latency-critical thread for which a cudaMalloc (and the
 * device-wide synchronisation it may imply) is not acceptable.  The quantised activations and
 * their row scales go into an array compiled into the library image (16.25 MiB of device memory
 * on every GPU that loads the library, held until the process exits), so the problem is limited to
 * M*K <= Q8K_LINEAR_STATIC_MAX_MK and M <= Q8K_LINEAR_STATIC_MAX_M; larger ones are rejected with
 * Q8K_ERR_TOO_LARGE and must use q8k_linear with a workspace.  The function itself calls no
 * cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with that device current) and caches it; make that first call before any stream capture
 *     is begun on the device.  The cached address belongs to the device's primary context: it does
 *     not survive a cudaDeviceReset, and `stream` must be a stream of the device that is current
 *     when the call is made.
 *   - All calls on a device share the one array and it keeps the previous call's contents.  Every
 *     byte a call reads it has written first, so nothing needs clearing, but two calls whose
 *     kernels can overlap on the GPU (different streams without an ordering between them) race
 *     on it: serialise them on one stream or with events.
 * Arguments, dtypes, results and error codes are otherwise those of q8k_linear.                  */
#define Q8K_LINEAR_STATIC_MAX_MK (16 * 1024 * 1024)
#define Q8K_LINEAR_STATIC_MAX_M  65536
Q8K_API int q8k_linear_static(const void* x, int x_dtype, const void* w, int w_dtype, const float* w_scales,
                              const float* bias, void* out, int out_dtype, int M, int N, int K,
                              int use_hadamard, int fuse_gelu, int* dev_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q8_KERNELS_B200_H */
