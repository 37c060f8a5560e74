// Block glue of the decode step: RMSNorm (+ residual add, + int8 quantization), rotary embedding
// fused with the KV-cache write, SiLU(gate) * up (+ int8 quantization).  Each kernel replaces a
// chain of small torch ops and keeps their rounding points (fp32 math, one rounding to the 16-bit
// activation type after every op of the chain).  All are HBM/L2-bound row kernels: one block per
// token row, 128-bit accesses, the row staged once in shared memory.
#include "common.cuh"

namespace llmqrt {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_reduce(float v, bool is_max) {
  __shared__ float red[kThreads / 32];
  __shared__ float result;
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();                                  // protects `red`/`result` between successive calls
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : (is_max ? 0.f : 0.f);
    w = is_max ? warp_max(w) : warp_sum(w);
    if (threadIdx.x == 0) result = w;
  }
  __syncthreads();
  return result;
}

// Per-token int8 quantization of a row already rounded to T and held in shared memory; same
// arithmetic as the stand-alone quantizer (scale = T(T(max(absmax,1e-5)) * (1/127)), q = rint(T(x/scale))).
template <typename T>
__device__ __forceinline__ void quantize_row_int8(const T* __restrict__ row_s, int64_t n, float amax,
                                                  int8_t* __restrict__ q, float* __restrict__ scale_out) {
  float s = round_to<T>(fmaxf(amax, 1e-5f));
  s = round_to<T>(__fmul_rn(s, 1.0f / 127.0f));
  if (threadIdx.x == 0) *scale_out = s;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = rintf(round_to<T>(__fdiv_rn(to_f32<T>(row_s[i]), s)));
    v = v != v ? v : fminf(fmaxf(v, -128.f), 127.f);
    q[i] = (int8_t)(int)v;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual, T* __restrict__ x_out,
               const T* __restrict__ weight, float eps, T* __restrict__ y, int8_t* __restrict__ q,
               float* __restrict__ scale_f32, int64_t H) {
  extern __shared__ __align__(16) uint8_t smem[];
  T* row = reinterpret_cast<T*>(smem);
  const int64_t m = blockIdx.x;
  const T* xr = x + m * H;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_f32<T>(xr[i]);
    if (residual) v = round_to<T>(v + to_f32<T>(residual[m * H + i]));    // h = x + r in T
    T hv = from_f32<T>(v);
    if (x_out) x_out[m * H + i] = hv;
    row[i] = hv;
    ss += v * v;
  }
  ss = block_reduce(ss, false);
  const float inv = rsqrtf(ss / (float)H + eps);
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < H; i += blockDim.x) {
    const float n = round_to<T>(to_f32<T>(row[i]) * inv);                 // (x32 * inv).to(T)
    const float o = round_to<T>(to_f32<T>(weight[i]) * n);                // weight * that, in T
    const T ov = from_f32<T>(o);
    if (y) y[m * H + i] = ov;
    row[i] = ov;
    amax = fmaxf(amax, fabsf(o));
  }
  if (q) {
    amax = block_reduce(amax, true);
    quantize_row_int8<T>(row, H, amax, q + m * H, scale_f32 + m);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_mul_kernel(const T* __restrict__ gate_up, int64_t ld, T* __restrict__ y, int8_t* __restrict__ q,
                float* __restrict__ scale_f32, int64_t I) {
  extern __shared__ __align__(16) uint8_t smem[];
  T* row = reinterpret_cast<T*>(smem);
  const int64_t m = blockIdx.x;
  const T* gr = gate_up + m * ld;
  const T* ur = gr + I;
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < I; i += blockDim.x) {
    const float g = to_f32<T>(gr[i]);
    const float act = round_to<T>(g / (1.0f + expf(-g)));                 // silu in T
    const float h = round_to<T>(act * to_f32<T>(ur[i]));                  // * up, in T
    const T hv = from_f32<T>(h);
    if (y) y[m * I + i] = hv;
    if (q) row[i] = hv;
    amax = fmaxf(amax, fabsf(h));
  }
  if (q) {
    amax = block_reduce(amax, true);
    quantize_row_int8<T>(row, I, amax, q + m * I, scale_f32 + m);
  }
}

// One block per (token, head); thread i rotates the pair (i, i + d/2).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ q, int64_t q_token_stride, T* __restrict__ k,
                                     const T* __restrict__ v, int64_t kv_token_stride, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int64_t cache_batch_stride, int64_t cache_row_stride,
                                     int pos0, const int32_t* __restrict__ pos_dev, const float* __restrict__ cos_tab,
                                     const float* __restrict__ sin_tab, int table_rows, int S, int Hq, int Hkv, int d) {
  const int token = blockIdx.x, head = blockIdx.y;
  const int b = token / S, s = token - b * S;
  const int pos = (pos_dev ? *pos_dev : pos0) + s;
  const int half = d / 2, i = threadIdx.x;
  if (pos < 0 || pos >= table_rows) return;          // outside the table: leave untouched
  const float c = cos_tab[(int64_t)pos * half + i], sn = sin_tab[(int64_t)pos * half + i];
  if (head < Hq) {
    T* p = q + (int64_t)token * q_token_stride + (int64_t)head * d;
    const float a = to_f32<T>(p[i]), bb = to_f32<T>(p[i + half]);
    p[i] = from_f32<T>(a * c - bb * sn);
    p[i + half] = from_f32<T>(a * sn + bb * c);
  } else {
    const int hk = head - Hq;
    T* p = k + (int64_t)token * kv_token_stride + (int64_t)hk * d;
    const float a = to_f32<T>(p[i]), bb = to_f32<T>(p[i + half]);
    const T r0 = from_f32<T>(a * c - bb * sn), r1 = from_f32<T>(a * sn + bb * c);
    p[i] = r0;
    p[i + half] = r1;
    if (k_cache) {
      const int64_t dst = (int64_t)b * cache_batch_stride + (int64_t)pos * cache_row_stride + (int64_t)hk * d;
      const T* vp = v + (int64_t)token * kv_token_stride + (int64_t)hk * d;
      k_cache[dst + i] = r0;
      k_cache[dst + i + half] = r1;
      v_cache[dst + i] = vp[i];
      v_cache[dst + i + half] = vp[i + half];
    }
  }
}

}  // namespace
}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_rmsnorm(const void* x, const void* residual, void* x_out, const void* weight, float eps, void* y,
                   int8_t* q, float* scale_f32, int dtype, int64_t M, int64_t H, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "rmsnorm: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(M >= 0 && H > 0 && M < (1ll << 31) && H * 2 <= 200 * 1024, "rmsnorm: bad shape");
  if (M == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(x && weight && (y || q), "rmsnorm: null pointer");
  LLMQRT_REQUIRE(!q || scale_f32, "rmsnorm: quantized output needs scale_f32");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)H * 2;
#define LLMQRT_RUN(T)                                                                                              \
  do {                                                                                                             \
    auto kern = rmsnorm_kernel<T>;                                                                                 \
    if (smem > 48 * 1024)                                                                                          \
      if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem)) return rc;          \
    kern<<<(unsigned)M, kThreads, smem, st>>>(reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(residual), \
                                              reinterpret_cast<T*>(x_out), reinterpret_cast<const T*>(weight), eps,  \
                                              reinterpret_cast<T*>(y), q, scale_f32, H);                            \
  } while (0)
  if (dtype == LLMQRT_F16) LLMQRT_RUN(__half); else LLMQRT_RUN(__nv_bfloat16);
#undef LLMQRT_RUN
  return check_launch("rmsnorm");
}

int llmqrt_silu_mul(const void* gate_up, int64_t ld, void* y, int8_t* q, float* scale_f32, int dtype, int64_t M,
                    int64_t I, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "silu_mul: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(M >= 0 && I > 0 && ld >= 2 * I && M < (1ll << 31) && I * 2 <= 200 * 1024, "silu_mul: bad shape");
  if (M == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(gate_up && (y || q), "silu_mul: null pointer");
  LLMQRT_REQUIRE(!q || scale_f32, "silu_mul: quantized output needs scale_f32");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = q ? (size_t)I * 2 : 0;
#define LLMQRT_RUN(T)                                                                                        \
  do {                                                                                                       \
    auto kern = silu_mul_kernel<T>;                                                                          \
    if (smem > 48 * 1024)                                                                                    \
      if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem)) return rc;    \
    kern<<<(unsigned)M, kThreads, smem, st>>>(reinterpret_cast<const T*>(gate_up), ld, reinterpret_cast<T*>(y), q, \
                                              scale_f32, I);                                                  \
  } while (0)
  if (dtype == LLMQRT_F16) LLMQRT_RUN(__half); else LLMQRT_RUN(__nv_bfloat16);
#undef LLMQRT_RUN
  return check_launch("silu_mul");
}

int llmqrt_rope_kv_write(void* q, int64_t q_token_stride, void* k, const void* v, int64_t kv_token_stride,
                         void* k_cache, void* v_cache, int64_t cache_batch_stride, int64_t cache_row_stride,
                         int32_t pos0, const int32_t* pos_dev, const float* cos_table, const float* sin_table,
                         int64_t table_rows, int dtype, int64_t B, int64_t S, int64_t Hq, int64_t Hkv, int64_t d,
                         llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "rope: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(d > 0 && d % 2 == 0 && d <= 2048 && Hq >= 0 && Hkv >= 0 && Hq + Hkv < 65536, "rope: bad head shape");
  if (B * S == 0 || Hq + Hkv == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(cos_table && sin_table && table_rows > 0, "rope: null angle table");
  LLMQRT_REQUIRE((Hq == 0 || q) && (Hkv == 0 || k), "rope: null pointer");
  LLMQRT_REQUIRE(!k_cache || (v && v_cache), "rope: cache write needs v and v_cache");
  LLMQRT_REQUIRE(B * S < (1ll << 31), "rope: too many tokens");
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)(B * S), (unsigned)(Hq + Hkv));
#define LLMQRT_RUN(T)                                                                                               \
  rope_kv_write_kernel<T><<<grid, (unsigned)(d / 2), 0, st>>>(                                                      \
      reinterpret_cast<T*>(q), q_token_stride, reinterpret_cast<T*>(k), reinterpret_cast<const T*>(v),              \
      kv_token_stride, reinterpret_cast<T*>(k_cache), reinterpret_cast<T*>(v_cache), cache_batch_stride,           \
      cache_row_stride, pos0, pos_dev, cos_table, sin_table, (int)table_rows, (int)S, (int)Hq, (int)Hkv, (int)d)
  if (dtype == LLMQRT_F16) LLMQRT_RUN(__half); else LLMQRT_RUN(__nv_bfloat16);
#undef LLMQRT_RUN
  return check_launch("rope_kv_write");
}

}  // extern "C"
