// Shared device/host helpers for the sm_100a kernels of this library.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/llmqrt_b200.h"

namespace llmqrt {

// ----------------------------------------------------------------------------------------------
// Host-side error reporting.  No exception ever crosses the C ABI: every entry point returns a
// status code and leaves a human-readable message in a thread-local buffer.
// ----------------------------------------------------------------------------------------------
char* last_error_buffer();                      // defined in capi.cu, thread-local, 512 bytes
int set_error(int code, const char* fmt, ...);  // formats into the buffer and returns `code`

#define LLMQRT_REQUIRE(cond, ...)                                          \
  do {                                                                     \
    if (!(cond)) return ::llmqrt::set_error(LLMQRT_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define LLMQRT_CUDA_OK(expr)                                                                 \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return ::llmqrt::set_error(LLMQRT_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// Called right after every kernel launch: reports a launch error and counts the launch (capi.cu).
int check_launch(const char* what);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Workspace layout (see llmqrt_workspace_bytes): arrival counters first, partial sums after.
constexpr size_t LLMQRT_WS_COUNTER_BYTES = (size_t)64 << 10;
constexpr size_t LLMQRT_WS_PARTIAL_BYTES = (size_t)160 << 20;
constexpr int LLMQRT_WS_NUM_COUNTERS = (int)(LLMQRT_WS_COUNTER_BYTES / 4) - 64;  // last 64 words: scalars
inline int* ws_counters(void* ws) { return reinterpret_cast<int*>(ws); }
inline unsigned* ws_scalars(void* ws) { return reinterpret_cast<unsigned*>(ws) + LLMQRT_WS_NUM_COUNTERS; }
inline void* ws_partials(void* ws) { return reinterpret_cast<char*>(ws) + LLMQRT_WS_COUNTER_BYTES; }
int sm_count();  // cached multiprocessor count of the current device (capi.cu)
// Raises the dynamic shared-memory limit of kernel `func` on the current device to at least `bytes`.
// The attribute is only touched when a larger value than ever before is needed, so steady-state
// launches (and stream capture after a warm-up call) make no driver call here.
int ensure_dynamic_smem(const void* func, int bytes);

// ----------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A decode step is a chain of several hundred short kernels; with
// this launch attribute the blocks of the next kernel are scheduled, and run their set-up, while the
// previous kernel drains.  Contract: a kernel launched through launch_chained() executes pdl_wait()
// before its first access to global memory (it returns once the preceding kernel has completed and
// its writes are visible) and may call pdl_trigger() as soon as it has started.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Entry of a small kernel whose successor is typically a GEMM: it waits for its own predecessor first
// and releases its dependents right after, so the successor's blocks become resident -- and request
// their weights, which nobody in the chain writes -- while this kernel does its work.  (Releasing
// BEFORE the wait lets the successor start while the predecessor GEMM is still streaming; its early
// weight requests then compete with that GEMM's for HBM, and the step was measured slower.)
__device__ __forceinline__ void pdl_wait_then_trigger() {
  pdl_wait();
  pdl_trigger();
}
bool pdl_enabled();   // capi.cu: on unless the environment variable LLMQRT_PDL is "0"

template <typename... KArgs, typename... Args>
inline int launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, dim3 cluster,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  LLMQRT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
  return LLMQRT_OK;
}
template <typename... KArgs, typename... Args>
inline int launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster_x,
                          Args... args) {
  return launch_chained(kern, grid, block, smem, st, dim3((unsigned)(cluster_x > 1 ? cluster_x : 1), 1, 1), args...);
}

// ----------------------------------------------------------------------------------------------
// 16-bit float helpers.  T is __half or __nv_bfloat16.
// ----------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// Round an fp32 value to the 16-bit type T and widen it again (what a torch op on a
// 16-bit tensor does to its fp32 intermediate).
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

// Loads a 16-bit float of runtime dtype (LLMQRT_F16 / LLMQRT_BF16 / LLMQRT_F32) as fp32.
__device__ __forceinline__ float load_as_f32(const void* p, int64_t i, int dtype) {
  if (dtype == LLMQRT_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  if (dtype == LLMQRT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_from_f32(void* p, int64_t i, int dtype, float v) {
  if (dtype == LLMQRT_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else if (dtype == LLMQRT_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

// ----------------------------------------------------------------------------------------------
// Global-memory access.  Weights and KV rows are read exactly once per launch: bypass L1.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_16B(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Coherent 16-byte load that still skips L1 allocation (for data another kernel or this CTA wrote).
__device__ __forceinline__ uint4 ldg_cg_16B(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ----------------------------------------------------------------------------------------------
// Warp-level tensor-core MMAs (register operands).  Used by the bandwidth-bound small-M and
// decode kernels, where the weight / KV stream goes HBM -> registers -> MMA without staging.
// Fragment ownership for lane = 4*g + t (g = 0..7, t = 0..3):
//   8-bit m16n8k32:  a0=(row g, k 4t..4t+3) a1=(row g+8, same k) a2=(row g, k 16+4t..) a3=(row g+8, ..)
//                    b0=(k 4t..4t+3, col g) b1=(k 16+4t.., col g)
//   16-bit m16n8k16: a0=(row g, k 2t,2t+1) a1=(row g+8, ..) a2=(row g, k 2t+8,2t+9) a3=(row g+8, ..)
//                    b0=(k 2t,2t+1, col g) b1=(k 2t+8,2t+9, col g)
//   accumulators:    c0=(row g, col 2t) c1=(row g, col 2t+1) c2=(row g+8, col 2t) c3=(row g+8, col 2t+1)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// A (weights) is always e4m3; B (activations) is e4m3 or e5m2.
template <bool B_E5M2>
__device__ __forceinline__ void mma_f8_16832(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  if constexpr (B_E5M2) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e5m2.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// ----------------------------------------------------------------------------------------------
// GEMM epilogue shared by every W8A8 kernel (streaming, split-K fix-up and tcgen05 paths).
// ----------------------------------------------------------------------------------------------
enum EpilogueMode : int {
  EPI_RAW = 0,       // store the raw accumulator (int32 or fp32)
  EPI_TENSOR = 1,    // out = T( fma(alpha, acc, beta * bias[n]) )
  EPI_ROW_COL = 2,   // out = T( (acc * row_scale[m]) * col_scale[n] + bias[n] )
  EPI_COL_ROW = 3,   // out = T( (acc * col_scale[n]) * row_scale[m] + bias[n] )
};

struct Epilogue {
  int mode;
  int out_dtype;            // LLMQRT_F16 / LLMQRT_BF16 (ignored for EPI_RAW)
  int bias_dtype;           // dtype of `bias`
  float alpha;              // used when alpha_dev == nullptr
  float beta;
  const float* alpha_dev;   // optional device scalar overriding `alpha`
  const void* bias;         // [N] or nullptr
  const float* row_scale;   // [M] (per token)
  const float* col_scale;   // [N] (per output channel)
  void* out;                // [M, ldo]
  int64_t ldo;
};

__device__ __forceinline__ float epilogue_value(const Epilogue& e, float acc, int64_t m, int64_t n, float alpha) {
  float b = e.bias ? load_as_f32(e.bias, n, e.bias_dtype) : 0.f;
  if (e.mode == EPI_TENSOR) return __fmaf_rn(alpha, acc, __fmul_rn(e.beta, b));
  float v;
  if (e.mode == EPI_ROW_COL) v = __fmul_rn(__fmul_rn(acc, e.row_scale[m]), e.col_scale[n]);
  else v = __fmul_rn(__fmul_rn(acc, e.col_scale[n]), e.row_scale[m]);
  return e.bias ? __fadd_rn(v, b) : v;
}

template <typename AccT>
__device__ __forceinline__ void epilogue_store(const Epilogue& e, AccT acc, int64_t m, int64_t n, float alpha) {
  if (e.mode == EPI_RAW) {
    reinterpret_cast<AccT*>(e.out)[m * e.ldo + n] = acc;
  } else {
    store_from_f32(e.out, m * e.ldo + n, e.out_dtype, epilogue_value(e, static_cast<float>(acc), m, n, alpha));
  }
}

}  // namespace llmqrt
