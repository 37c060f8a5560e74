// Dynamic activation quantizers (int8 SmoothQuant, fp8 e4m3), per token or per tensor.
//
// The operators these replace are chains of torch elementwise ops on a 16-bit tensor; each op
// there computes in fp32 and rounds to the 16-bit dtype, and a division by a Python scalar is
// executed on CUDA as a multiplication by the fp32 reciprocal.  The kernels reproduce those
// roundings step by step so that the quantized integers are bit-identical.
//
// HBM-bound: one read of x for the absmax, one (L2-resident) re-read for the conversion, one
// write of q.  One thread block per token row; 128-bit loads when the row is 16-byte aligned.
#include "common.cuh"

namespace llmqrt {
namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ float row_absmax(const T* __restrict__ row, int64_t K, bool vec_ok) {
  float m = 0.f;
  if (vec_ok) {
    const uint4* p = reinterpret_cast<const uint4*>(row);
    for (int64_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
      uint4 v = p[i];
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(to_f32<T>(e[j])));
    }
  } else {
    for (int64_t i = threadIdx.x; i < K; i += blockDim.x) m = fmaxf(m, fabsf(to_f32<T>(row[i])));
  }
  return m;
}

__device__ __forceinline__ float block_max(float m) {
  __shared__ float red[kThreads / 32];
  __shared__ float result;
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0.f;
    v = warp_max(v);
    if (threadIdx.x == 0) result = v;
  }
  __syncthreads();
  return result;
}

__device__ __forceinline__ float clamp_keep_nan(float v, float lo, float hi) {
  return v != v ? v : fminf(fmaxf(v, lo), hi);
}

// scale (as fp32 value of a T number) from an absmax, following the reference op by op.
template <typename T, bool FP8>
__device__ __forceinline__ float scale_from_absmax(float amax) {
  float s = round_to<T>(fmaxf(amax, FP8 ? 1e-12f : 1e-5f));   // clamp(min=...)
  const float inv = 1.0f / (FP8 ? 448.0f : 127.0f);            // CUDA torch: x / python_scalar -> x * (1/scalar)
  return round_to<T>(__fmul_rn(s, inv));
}

template <typename T, bool FP8>
__device__ __forceinline__ uint8_t quantize_one(float x, float s) {
  float v = round_to<T>(__fdiv_rn(x, s));                      // tensor / tensor: true division, rounded to T
  if constexpr (FP8) {
    v = clamp_keep_nan(v, -448.f, 448.f);
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
  } else {
    v = rintf(v);                                              // .round(): half to even
    v = clamp_keep_nan(v, -128.f, 127.f);
    return (uint8_t)(int8_t)(int)v;
  }
}

template <typename T, bool FP8>
__device__ __forceinline__ void quantize_row(const T* __restrict__ row, uint8_t* __restrict__ qrow, int64_t K,
                                             float s, bool vec_ok) {
  if (vec_ok) {
    const uint4* p = reinterpret_cast<const uint4*>(row);
    uint2* qp = reinterpret_cast<uint2*>(qrow);
    for (int64_t i = threadIdx.x; i < K / 8; i += blockDim.x) {
      uint4 v = p[i];
      const T* e = reinterpret_cast<const T*>(&v);
      uint8_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = quantize_one<T, FP8>(to_f32<T>(e[j]), s);
      uint2 w;
      w.x = o[0] | (o[1] << 8) | (o[2] << 16) | ((uint32_t)o[3] << 24);
      w.y = o[4] | (o[5] << 8) | (o[6] << 16) | ((uint32_t)o[7] << 24);
      qp[i] = w;
    }
  } else {
    for (int64_t i = threadIdx.x; i < K; i += blockDim.x) qrow[i] = quantize_one<T, FP8>(to_f32<T>(row[i]), s);
  }
}

// Per-token: one block per row does absmax + conversion.
template <typename T, bool FP8>
__global__ void __launch_bounds__(kThreads)
quantize_per_token_kernel(const T* __restrict__ x, int64_t K, int64_t ldx, uint8_t* __restrict__ q,
                          T* __restrict__ scale_x, float* __restrict__ scale_f32, float scale_mul, bool vec_ok) {
  pdl_wait_then_trigger();
  const int64_t m = blockIdx.x;
  const T* row = x + m * ldx;
  float amax = block_max(row_absmax<T>(row, K, vec_ok));
  float s = scale_from_absmax<T, FP8>(amax);
  if (threadIdx.x == 0) {
    if (scale_x) scale_x[m] = from_f32<T>(s);
    if (scale_f32) scale_f32[m] = FP8 ? __fmul_rn(s, scale_mul) : round_to<T>(__fmul_rn(s, scale_mul));
  }
  quantize_row<T, FP8>(row, q + m * K, K, s, vec_ok);
}

// Per-tensor pass 1: absmax of the whole tensor, merged with an atomic max on the fp32 bit pattern
// (monotonic for non-negative floats).
template <typename T>
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const T* __restrict__ x, int64_t K, int64_t ldx, unsigned* __restrict__ amax_bits, bool vec_ok) {
  float amax = block_max(row_absmax<T>(x + (int64_t)blockIdx.x * ldx, K, vec_ok));
  if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(amax));
}

// Per-tensor pass 2 (also the static-scale kernel when `static_scale` is given).
template <typename T, bool FP8>
__global__ void __launch_bounds__(kThreads)
quantize_per_tensor_kernel(const T* __restrict__ x, int64_t K, int64_t ldx, uint8_t* __restrict__ q,
                           const unsigned* __restrict__ amax_bits, const float* __restrict__ static_scale,
                           T* __restrict__ scale_x, float* __restrict__ scale_f32, float scale_mul, bool vec_ok) {
  const int64_t m = blockIdx.x;
  float s = static_scale ? *static_scale : scale_from_absmax<T, FP8>(__uint_as_float(*amax_bits));
  if (m == 0 && threadIdx.x == 0) {
    if (scale_x) scale_x[0] = from_f32<T>(s);
    if (scale_f32) scale_f32[0] = FP8 ? __fmul_rn(s, scale_mul) : round_to<T>(__fmul_rn(s, scale_mul));
  }
  const T* row = x + m * ldx;
  if (static_scale) {
    // tensor(16-bit) / tensor(fp32) promotes to fp32: no intermediate 16-bit rounding.
    uint8_t* qrow = q + m * K;
    for (int64_t i = threadIdx.x; i < K; i += blockDim.x) {
      float v = clamp_keep_nan(__fdiv_rn(to_f32<T>(row[i]), s), -448.f, 448.f);
      qrow[i] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    }
  } else {
    quantize_row<T, FP8>(row, q + m * K, K, s, vec_ok);
  }
}

template <typename T, bool FP8>
int launch(const void* x, int64_t M, int64_t K, int64_t ldx, int per_token, uint8_t* q, void* scale_x,
           float* scale_f32, float scale_mul, const float* static_scale, void* workspace, cudaStream_t st) {
  const T* xp = reinterpret_cast<const T*>(x);
  const bool vec_ok = (K % 8 == 0) && (ldx % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
  if (M == 0 || K == 0) return LLMQRT_OK;
  if (static_scale) {
    quantize_per_tensor_kernel<T, FP8><<<(unsigned)M, kThreads, 0, st>>>(xp, K, ldx, q, nullptr, static_scale,
                                                                        nullptr, nullptr, 1.f, vec_ok);
    return check_launch("quantize_static");
  }
  if (per_token) {
    if (int rc = launch_chained(quantize_per_token_kernel<T, FP8>, dim3((unsigned)M), dim3(kThreads), 0, st, 1, xp, K,
                                ldx, q, reinterpret_cast<T*>(scale_x), scale_f32, scale_mul, vec_ok))
      return rc;
    return check_launch("quantize_per_token");
  }
  if (!workspace) return set_error(LLMQRT_ERR_WORKSPACE, "per-tensor quantization needs the workspace");
  unsigned* amax_bits = ws_scalars(workspace);
  LLMQRT_CUDA_OK(cudaMemsetAsync(amax_bits, 0, sizeof(unsigned), st));
  absmax_kernel<T><<<(unsigned)M, kThreads, 0, st>>>(xp, K, ldx, amax_bits, vec_ok);
  if (int rc = check_launch("absmax")) return rc;
  quantize_per_tensor_kernel<T, FP8><<<(unsigned)M, kThreads, 0, st>>>(
      xp, K, ldx, q, amax_bits, nullptr, reinterpret_cast<T*>(scale_x), scale_f32, scale_mul, vec_ok);
  return check_launch("quantize_per_tensor");
}

template <bool FP8>
int dispatch(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int per_token, uint8_t* q, void* scale_x,
             float* scale_f32, float scale_mul, const float* static_scale, void* workspace, cudaStream_t st) {
  LLMQRT_REQUIRE(M >= 0 && K >= 0 && ldx >= K, "quantize: bad shape M=%lld K=%lld ldx=%lld", (long long)M,
                 (long long)K, (long long)ldx);
  LLMQRT_REQUIRE(M < (1ll << 31), "quantize: M too large");
  if (M == 0 || K == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(x && q, "quantize: null pointer");
  if (x_dtype == LLMQRT_F16)
    return launch<__half, FP8>(x, M, K, ldx, per_token, q, scale_x, scale_f32, scale_mul, static_scale, workspace, st);
  if (x_dtype == LLMQRT_BF16)
    return launch<__nv_bfloat16, FP8>(x, M, K, ldx, per_token, q, scale_x, scale_f32, scale_mul, static_scale,
                                      workspace, st);
  return set_error(LLMQRT_ERR_INVALID, "quantize: x must be fp16 or bf16");
}

}  // namespace
}  // namespace llmqrt

extern "C" {

int llmqrt_quantize_int8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int per_token, int8_t* q,
                         void* scale_x, float* scale_f32, float scale_mul, void* workspace, llmqrt_stream_t stream) {
  return llmqrt::dispatch<false>(x, x_dtype, M, K, ldx, per_token, reinterpret_cast<uint8_t*>(q), scale_x, scale_f32,
                                 scale_mul, nullptr, workspace, (cudaStream_t)stream);
}

int llmqrt_quantize_fp8(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, int per_token, uint8_t* q,
                        float* scale_f32, float scale_mul, void* workspace, llmqrt_stream_t stream) {
  return llmqrt::dispatch<true>(x, x_dtype, M, K, ldx, per_token, q, nullptr, scale_f32, scale_mul, nullptr,
                                workspace, (cudaStream_t)stream);
}

int llmqrt_quantize_fp8_static(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ldx, const float* scale,
                               uint8_t* q, llmqrt_stream_t stream) {
  if (!scale) return llmqrt::set_error(LLMQRT_ERR_INVALID, "quantize_fp8_static: null scale");
  return llmqrt::dispatch<true>(x, x_dtype, M, K, ldx, 1, q, nullptr, nullptr, 1.f, scale, nullptr,
                                (cudaStream_t)stream);
}

}  // extern "C"
