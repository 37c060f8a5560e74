/*
 * llmqrt_b200 -- C ABI of the sm_100a kernels behind the quantized-linear and
 * KV-cache-attention operators.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current device unless its name ends in `_host`;
 *   - every call is asynchronous on `stream` and returns a status code at once; nothing is
 *     allocated, freed or synchronised inside (the caller owns outputs and workspaces);
 *   - matrices are row-major with an explicit leading dimension in ELEMENTS;
 *   - weights are passed as W[N, K] row-major.  The reference hands the same memory to its
 *     kernels as a "[K, N] column-major" view (stride [1, K]); the pointer is identical;
 *   - 0 = success; negative = error, message available from llmqrt_last_error().
 *
 * Citations `ref:` give the reference interface (path inside the reference project) that the
 * entry point stands in for.
 */
#ifndef LLMQRT_B200_H
#define LLMQRT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* llmqrt_stream_t; /* a cudaStream_t */

enum {
  LLMQRT_OK = 0,
  LLMQRT_ERR_INVALID = -1,     /* bad shape / alignment / dtype argument                  */
  LLMQRT_ERR_CUDA = -2,        /* a CUDA runtime or driver call failed                    */
  LLMQRT_ERR_WORKSPACE = -3,   /* workspace missing or too small                          */
  LLMQRT_ERR_UNSUPPORTED = -4  /* valid request this build does not implement             */
};

enum { /* element types */
  LLMQRT_F16 = 0,
  LLMQRT_BF16 = 1,
  LLMQRT_F32 = 2,
  LLMQRT_E4M3 = 3,
  LLMQRT_E5M2 = 4
};

/* Message of the last failing call made by this thread (never NULL). */
const char* llmqrt_last_error(void);
/* ABI version; bumped when a signature changes. */
int llmqrt_abi_version(void);
/* Number of kernels this library has launched in the process so far (all threads). */
long long llmqrt_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Workspace.  Kernels that split the reduction dimension across thread blocks keep partial
 * sums and arrival counters in caller-provided scratch.  The scratch must be at least
 * llmqrt_workspace_bytes() long, 256-byte aligned, ZERO-FILLED ONCE after allocation (kernels
 * restore the counters to zero before they finish), and must not be shared by calls that can
 * overlap on the GPU (use one per stream).
 * ---------------------------------------------------------------------------------------- */
size_t llmqrt_workspace_bytes(void);

/* ------------------------------------------------------------------------------------------
 * Activation quantizers
 * ---------------------------------------------------------------------------------------- */

/* Dynamic symmetric int8 quantization of x[M, K] (fp16 / bf16).
 * per_token != 0: one scale per row, else one scale for the whole tensor.
 *   scale = clamp(absmax, 1e-5) / 127 evaluated in x's dtype, q = clamp(rint(x / scale)).
 * Outputs: q int8 [M, K] (contiguous); scale_x in x's dtype ([M] or [1], may be NULL);
 * scale_f32 ([M] or [1], may be NULL) = float(T(scale * scale_mul)) -- pass scale_mul = the
 * weight scale to obtain the GEMM's alpha without a host round trip, or 1.0f.
 * ref: runtime/nn_models/modules/linear/linear_sq.py:44-53 (per tensor), :55-65 (per token). */
int llmqrt_quantize_int8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int per_token,
                         int8_t* q, void* scale_x, float* scale_f32, float scale_mul, void* workspace,
                         llmqrt_stream_t stream);

/* Dynamic FP8 e4m3 quantization: scale = clamp(amax, 1e-12) / 448 in x's dtype,
 * q = e4m3(clamp(x / scale, +-448)).  scale_f32 ([M] or [1]) = float(scale) * scale_mul.
 * ref: runtime/nn_models/modules/linear/linear_fp8.py:11-32 (per tensor), :40-63 (per token). */
int llmqrt_quantize_fp8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int per_token,
                        uint8_t* q, float* scale_f32, float scale_mul, void* workspace, llmqrt_stream_t stream);

/* Static FP8 quantization with a given one-element fp32 scale: q = e4m3(clamp(x / scale)).
 * ref: runtime/nn_models/modules/linear/linear_fp8.py:34-37. */
int llmqrt_quantize_fp8_static(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const float* scale,
                               uint8_t* q, llmqrt_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * W8A8 GEMMs.   acc[m, n] = sum_k a[m, k] * w[n, k]
 * Requirements: K % 16 == 0, lda % 16 == 0, ldw % 16 == 0, 16-byte aligned a and w.
 * `alpha_dev`, when not NULL, is a device fp32 scalar used instead of `alpha`.
 * `flags`: 0, or LLMQRT_GEMM_STATIC_WEIGHT when `w` is a stored weight that no kernel still
 * running or queued on `stream` writes.  With that flag the kernels may start reading `w` before
 * the kernel that precedes the call on `stream` has finished (they still wait for it before
 * touching `a`, the scales and `out`), which hides the first weight fetch behind the previous
 * kernel's tail.  Without it every operand is read only after the preceding kernel has completed,
 * so a weight quantized on the same stream right before the call is safe.
 * ---------------------------------------------------------------------------------------- */
enum { LLMQRT_GEMM_STATIC_WEIGHT = 1 };

/* int8 x int8 -> exact int32 accumulators -> out fp16 = alpha * acc + beta * bias[n].
 * bias is fp16 [N] and required, like the reference's.
 * ref: w8a8_int8_linear_bbf16_obf16_per_tensor, runtime/csrc/smoothquant/sq_gemm.cu:36-160,
 *      declared runtime/csrc/smoothquant/sq_gemm.h:12-17, bound runtime/csrc/bindings.cpp:10-11. */
int llmqrt_w8a8_int8_linear_per_tensor(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, const void* bias,
                                       float alpha, const float* alpha_dev, float beta, void* out, int64_t ldo,
                                       int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags);

/* int8 GEMM with the per-token x per-output-channel dequantization fused:
 * out = T( (float(acc) * w_scale[n]) * a_scale[m] + bias[n] ), T = out_dtype, bias optional.
 * ref: w8a8_int8_linear_bbf16_obf16_per_channel, declared runtime/csrc/smoothquant/sq_gemm.h:19-24
 *      (body commented out, sq_gemm.cu:162-278); arithmetic of
 *      dequantize_activation_w_per_channel_a_per_token, runtime/utils/quantization_utils.py:90-97. */
int llmqrt_w8a8_int8_linear_per_channel(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, const void* bias,
                                        int bias_dtype, const float* a_scale, const float* w_scale, void* out,
                                        int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace,
                                        llmqrt_stream_t stream, int flags);

/* Same operator as llmqrt_w8a8_int8_linear_per_channel for callers that cannot hand over a workspace
 * because they are not allowed, or cannot afford, to allocate device memory: plug-ins of a server
 * that owns the whole memory plan, or loops where the device-wide stall of cudaMalloc / cudaFree is
 * unacceptable.  The split-K scratch is a fixed 8 MiB + 16 KiB array inside the library's device
 * image (resident on every GPU that loads the library until the process exits); nothing is allocated
 * or freed by the call.  Limits: M <= 64, N <= 524288, and the partial sums of the chosen split must
 * fit in 8 MiB -- larger problems are rejected with LLMQRT_ERR_WORKSPACE.  The array is shared by all
 * calls: calls that can overlap on one GPU race on it.  The first call on each device resolves the
 * array's device address (cudaGetSymbolAddress) and should be made before any stream capture starts.
 * No counterpart in the reference: it exists only for such callers. */
int llmqrt_w8a8_int8_linear_per_channel_noalloc(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw,
                                                const void* bias, int bias_dtype, const float* a_scale,
                                                const float* w_scale, void* out, int out_dtype, int64_t ldo,
                                                int64_t M, int64_t N, int64_t K, llmqrt_stream_t stream);

/* Raw int32 accumulators acc[M, ldo] of the int8 GEMM (the quantity the parity gate checks bit for
 * bit); same kernels as the two entry points above with the epilogue reduced to a store. */
int llmqrt_w8a8_int8_gemm_s32(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, int32_t* acc, int64_t ldo,
                              int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags);

/* FP8 GEMM, tensor-wise scaling: out = T( alpha * acc_f32 + beta * bias[n] ), T in {bf16, fp16},
 * bias optional and of type T.  a_format = LLMQRT_E4M3 or LLMQRT_E5M2; w is e4m3.
 * ref: f8f8bf16_tensorwise (bound as cutlass_f8f8bf16_tensorwise_sm89),
 *      runtime/csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:316-334, bindings.cpp:12. */
int llmqrt_f8f8_tensorwise(const uint8_t* a, int a_format, int64_t lda, const uint8_t* w, int64_t ldw,
                           const void* bias, float alpha, const float* alpha_dev, float beta, void* out, int out_dtype,
                           int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags);

/* FP8 GEMM, row-wise scaling: out bf16 = ((acc_f32 * x_scale[m]) * w_scale[n]) + bias[n];
 * bias optional, bf16 or fp32.
 * ref: f8f8bf16_rowwise (bound as cutlass_f8f8bf16_rowwise_sm89),
 *      runtime/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:582-606, bindings.cpp:13. */
int llmqrt_f8f8bf16_rowwise(const uint8_t* a, int a_format, int64_t lda, const uint8_t* w, int64_t ldw,
                            const void* bias, int bias_dtype, const float* x_scale, const float* w_scale, void* out,
                            int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags);

/* Path selection of the W8A8 GEMMs, for tests and benchmarks: 0 = automatic (default),
 * 1 = register-operand streaming kernel only, 2 = tcgen05/TMEM kernel only.  Process-wide. */
int llmqrt_set_gemm_path(int path);

/* ------------------------------------------------------------------------------------------
 * AWQ W4A16
 * Reference storage: qweight int32 [K, N/8] and qzeros int32 [K/G, N/8], eight 4-bit values per
 * word along N with nibble i holding column 8j + {0,2,4,6,1,3,5,7}[i]; scales fp16 [K/G, N].
 * ---------------------------------------------------------------------------------------- */

/* W[K, N] fp16 = (nibble(qweight) - nibble(qzeros[k/G])) * scales[k/G].
 * ref: awq_dequantize_triton, runtime/triton_kernels/awq_kernels.py:273-320 (kernel :33-127). */
int llmqrt_awq_dequantize(const int32_t* qweight, const void* scales, const int32_t* qzeros, int64_t K, int64_t N,
                          int64_t group_size, void* out, llmqrt_stream_t stream);

/* One-time repack of a layer into the streaming layout the GEMM kernels read:
 *   wq_t  uint32 [N, K/8]  eight K-consecutive values per word, value 2p in nibble p and 2p+1 in nibble p+4;
 *   sz_t  half2  [N, K/G]  per (column, group): { scale, -(1024 + zero) } as two fp16.
 * ref: replaces the per-call unpacking of runtime/triton_kernels/awq_kernels.py:205-250. */
int llmqrt_awq_repack(const int32_t* qweight, const void* scales, const int32_t* qzeros, int64_t K, int64_t N,
                      int64_t group_size, uint32_t* wq_t, uint32_t* sz_t, llmqrt_stream_t stream);

/* C[M, N] fp16 = x[M, K] fp16 @ dequant(W) (+ bias fp16 [N], optional) on the repacked layer.
 * fp32 accumulation; K % 128 == 0 when group_size < K, N % 8 == 0.
 * ref: awq_gemm_triton, runtime/triton_kernels/awq_kernels.py:328-378 (kernel :134-267), and the
 *      dequantize + matmul branch of runtime/nn_models/modules/linear/linear_awq.py:49-53. */
int llmqrt_awq_gemm(const void* x, int64_t ldx, const uint32_t* wq_t, const uint32_t* sz_t, const void* bias,
                    void* out, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t group_size, void* workspace,
                    llmqrt_stream_t stream);

/* Dequantize the repacked layer to W^T fp16 [N, K] (K contiguous), the operand layout of the
 * tcgen05 fp16 GEMM used for large M. */
int llmqrt_awq_dequantize_t(const uint32_t* wq_t, const uint32_t* sz_t, int64_t K, int64_t N, int64_t group_size,
                            void* out, llmqrt_stream_t stream);

/* Dense 16-bit GEMM on tcgen05: out[M, N] = a[M, K] @ w[N, K]^T (+ bias[n]), fp32 accumulate,
 * a / w / out / bias all of type `dtype` (fp16 or bf16).  K % 8 == 0.
 * ref: the torch.matmul of runtime/nn_models/modules/linear/linear_awq.py:53. */
int llmqrt_gemm_16bit(const void* a, int64_t lda, const void* w, int64_t ldw, const void* bias, void* out,
                      int64_t ldo, int dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                      llmqrt_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Attention over the contiguous GQA KV cache.  dtype = fp16 or bf16 for q, k, v, caches, out.
 * Query head h reads KV head h / (Hq / Hkv).  head_dim must be 64 or 128.
 * ---------------------------------------------------------------------------------------- */

/* cache[b, cache_seqlens[b] + s] = k/v[b, s] for s < S_new.  Caches are [Bc, Smax, Hkv, d] with the
 * given batch and row strides (elements); k/v are [B, S_new, Hkv, d] contiguous.
 * ref: the in-place append of flash_attn_with_kvcache (call site
 *      runtime/nn_models/modules/nonlinear/attn.py:305-315) and WindowedCache.update_kv,
 *      runtime/nn_models/modules/nonlinear/cache.py:41-46 (cache_seqlens == NULL: write at `start_pos`). */
int llmqrt_kv_append(void* k_cache, void* v_cache, int64_t cache_batch_stride, int64_t cache_row_stride,
                     const void* k, const void* v, const int32_t* cache_seqlens, int32_t start_pos, int dtype,
                     int64_t B, int64_t S_new, int64_t Hkv, int64_t d, int64_t Smax, llmqrt_stream_t stream);

/* Decode attention: q [B, Hq, d] (one new token per sequence) attends to cache rows
 * [0, seqlens[b]) of sequence b; out [B, Hq, d] contiguous.  softcap = 0 disables logit soft-capping.
 * q_batch_stride = elements between the query rows of consecutive sequences (heads and d contiguous),
 * so q may be a slice of a fused qkv projection output.
 * out_q / out_scale (both or neither; may be NULL): additionally the per-token int8 quantization of
 * out viewed as [B, Hq * d] -- the same arithmetic as llmqrt_quantize_int8(per_token = 1) applied to
 * out, scales as fp32 -- which is the input of an int8 output projection (Hq * d <= 8192).
 * max_seqlen: upper bound of seqlens[b], at most the cache capacity; the grid and the split-KV
 * scratch are sized from it without reading seqlens back.  A sequence whose length exceeds it is
 * attended over its first max_seqlen rows only (and llmqrt_attn_decode_append writes nothing for
 * it): no access outside the cache or the scratch results.
 * ref: flash_attn_with_kvcache call site, runtime/nn_models/modules/nonlinear/attn.py:300-315;
 *      the quantization that follows it in an int8 model: quantize_activation_per_token_absmax,
 *      runtime/nn_models/modules/linear/linear_sq.py:56-65, called from
 *      SqW8A8BBF16OBF16PerChannel.forward, linear_sq.py:185. */
int llmqrt_attn_decode(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                       int64_t cache_batch_stride, int64_t cache_row_stride, const int32_t* seqlens, void* out,
                       int8_t* out_q, float* out_scale, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t d,
                       int64_t max_seqlen, float softcap, void* workspace, llmqrt_stream_t stream);

/* llmqrt_attn_decode with the work on the newest token folded in (the newest token of sequence b is
 * cache row seqlens[b] - 1, i.e. seqlens already counts it):
 *   cos_table / sin_table (fp32 [table_rows, d/2], may be NULL): rotary embedding, half-split pairing,
 *     of q -- in registers, q itself is not modified -- and of the new key, at angle row
 *     seqlens[b] - 1 (rows outside the table: no rotation and no cache write);
 *   k_new / v_new ([B, Hkv, d] with batch stride kv_batch_stride, may be NULL): the new key (rotated)
 *     and value are written into the caches at that row before the row is read.
 * One kernel instead of rotary + cache write + attention.
 * ref: flash_attn_with_kvcache(q, k_cache, v_cache, k=, v=, rotary_cos=, rotary_sin=, cache_seqlens=,
 *      rotary_interleaved=False) of the flash-attn package, whose append-and-attend form the reference
 *      calls at runtime/nn_models/modules/nonlinear/attn.py:300-315 after applying
 *      RoPE.forward (attn.py:53-87) and WindowedCache.update_kv (cache.py:41-46) itself. */
int llmqrt_attn_decode_append(const void* q, int64_t q_batch_stride, const void* k_new, const void* v_new,
                              int64_t kv_batch_stride, const float* cos_table, const float* sin_table,
                              int64_t table_rows, void* k_cache, void* v_cache, int64_t cache_batch_stride,
                              int64_t cache_row_stride, const int32_t* seqlens, void* out, int8_t* out_q,
                              float* out_scale, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t d,
                              int64_t max_seqlen, float softcap, void* workspace, llmqrt_stream_t stream);

/* Prefill attention over the new tokens: q [B, S, Hq, d], k / v [B, S, Hkv, d], out [B, S, Hq, d],
 * token stride given in elements (heads and d contiguous), causal mask optional.
 * ref: flash_attn_func call site, runtime/nn_models/modules/nonlinear/attn.py:283-298. */
int llmqrt_attn_prefill(const void* q, int64_t q_token_stride, const void* k, const void* v, int64_t kv_token_stride,
                        void* out, int64_t out_token_stride, int dtype, int64_t B, int64_t S, int64_t Hq, int64_t Hkv,
                        int64_t d, int causal, float softcap, llmqrt_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Block glue used by the decode step (each fuses what the reference runs as a chain of torch ops)
 * ---------------------------------------------------------------------------------------- */

/* y = weight * T(x32 * rsqrt(mean(x32^2) + eps)); optional residual: x <- x + residual first
 * (the sum is written back to `x_out` when not NULL).  Optional fused per-token int8 quantization
 * of y (q, scale_f32 not NULL), same arithmetic as llmqrt_quantize_int8.
 * ref: RMSNorm.forward, runtime/nn_models/modules/nonlinear/norm.py:10-16; residual adds of
 *      LlamaLikeBlock.forward, runtime/nn_models/modules/nonlinear/block.py:64-78. */
int llmqrt_rmsnorm(const void* x, const void* residual, void* x_out, const void* weight, float eps, void* y,
                   int8_t* q, float* scale_f32, int dtype, int64_t M, int64_t H, llmqrt_stream_t stream);

/* Rotary embedding (half-split pairing) of q [B, S, Hq, d] and k [B, S, Hkv, d] in place at positions
 * pos0 + s (pos_dev, when not NULL, is a device int32 scalar overriding pos0), then, when k_cache is
 * not NULL, writes the rotated k and v [B, S, Hkv, d] into the caches at rows pos + s.
 * cos_table / sin_table are fp32 [table_rows, d/2] (angle = pos * theta^(-2i/d), the real and
 * imaginary parts of the reference's freqs_cis); tokens whose position is outside the table are left
 * untouched.
 * ref: RoPE.forward, runtime/nn_models/modules/nonlinear/attn.py:53-87 (table :37-43), cache.py:41-46. */
int llmqrt_rope_kv_write(void* q, int64_t q_token_stride, void* k, const void* v, int64_t kv_token_stride,
                         void* k_cache, void* v_cache, int64_t cache_batch_stride, int64_t cache_row_stride,
                         int32_t pos0, const int32_t* pos_dev, const float* cos_table, const float* sin_table,
                         int64_t table_rows, int dtype, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t d,
                         llmqrt_stream_t stream);

/* h = silu(gate) * up for gate_up [M, 2*I] (gate in columns [0, I), up in [I, 2I)), written to `y`
 * [M, I] when not NULL, with optional fused per-token int8 quantization of h.
 * ref: the activation of the Hugging Face Qwen2MLP, down_proj(act_fn(gate_proj(x)) * up_proj(x)),
 *      which the reference passes through unchanged (mlp=module.mlp, runtime/nn_models/models/qwen2.py:153). */
int llmqrt_silu_mul(const void* gate_up, int64_t ld, void* y, int8_t* q, float* scale_f32, int dtype, int64_t M,
                    int64_t I, llmqrt_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Tensor-parallel sum of the row-parallel partial outputs (after o_proj and down_proj) over
 * peer-mapped buffers on one NVLink/NVSwitch node, one process per GPU, up to 8 ranks.
 * No counterpart in the reference, which has no tensor parallelism (its only multi-device mode is
 * layer placement, runtime/core/base.py:213-221).
 *
 * Set-up, once per process (these calls allocate and synchronize; llmqrt_comm_allreduce does not):
 *   llmqrt_comm_create        allocates this rank's buffer (capacity max_bytes per call) on the
 *                             current device;
 *   llmqrt_comm_local_handle  writes llmqrt_comm_handle_bytes() bytes identifying it; the caller
 *                             exchanges them with the other ranks by any means (an all-gather);
 *   llmqrt_comm_open_peer     maps rank `peer`'s buffer from its handle.
 * llmqrt_comm_allreduce: out[i] = sum over ranks of x[i] (fp32 accumulation in rank order, one
 * rounding; identical bits on every rank); n a multiple of 8, out may alias x.  Every rank must
 * issue the same sequence of calls with the same n.  Waits on peers are bounded (5 s, or what
 * llmqrt_comm_set_poll_limit_ms set; the limit applies to calls launched, or graphs captured,
 * afterwards): on a time-out the output is not written and a sticky status is raised, after which
 * further calls return without waiting; llmqrt_comm_status reads it (0 = healthy; synchronizes the
 * device).
 * ------------------------------------------------------------------------------------------ */
int llmqrt_comm_create(int rank, int world, int64_t max_bytes, void** comm_out);
int llmqrt_comm_handle_bytes(void);
int llmqrt_comm_local_handle(void* comm, void* handle_out);
int llmqrt_comm_open_peer(void* comm, int peer, const void* handle);
int llmqrt_comm_allreduce(void* comm, const void* x, void* out, int dtype, int64_t n, llmqrt_stream_t stream);
/* llmqrt_rmsnorm with the residual arriving as tensor-parallel partial sums: residual =
 * all-reduce(partial) exactly as llmqrt_comm_allreduce computes it (rounded to the 16-bit type), then
 * h = x + residual, RMSNorm and the optional per-token int8 quantization, in one kernel
 * (H a multiple of 8, H <= 8192, M * H * 2 bytes within the communicator's capacity).  partial may be
 * NULL when the partial sums have already been pushed by llmqrt_comm_int8_linear_per_channel. */
int llmqrt_comm_allreduce_rmsnorm(void* comm, const void* partial, const void* x, void* x_out, const void* weight,
                                  float eps, void* y, int8_t* q, float* scale_f32, int dtype, int64_t M, int64_t H,
                                  llmqrt_stream_t stream);
/* Row-parallel linear fused with the first half of that all-reduce: llmqrt_w8a8_int8_linear_per_channel
 * whose 16-bit results do not go to an output tensor but, straight from the GEMM's epilogue, over
 * NVLink into the peers' all-reduce buffers as this rank's contribution to the NEXT call.  That call
 * must be llmqrt_comm_allreduce_rmsnorm with partial = NULL, the same M and H = N, which then only
 * gathers, sums and normalises: GEMM + collective + normalisation in two kernels with no partial tensor
 * in between.  16 < M <= 128, N a multiple of 8, N <= 8192.  (No counterpart in the reference, which has
 * no tensor parallelism.) */
int llmqrt_comm_int8_linear_per_channel(void* comm, const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw,
                                        const void* bias, int bias_dtype, const float* a_scale, const float* w_scale,
                                        int out_dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                                        llmqrt_stream_t stream, int flags);
int llmqrt_comm_set_poll_limit_ms(void* comm, int32_t ms);
int llmqrt_comm_status(void* comm, int32_t* status_out);
int llmqrt_comm_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif /* LLMQRT_B200_H */
