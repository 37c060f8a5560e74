// Weight-streaming W8A8 GEMM for small M (decode): C[M, N] = A[M, K] * W[N, K]^T, int8 or fp8.
//
// Bandwidth-bound design: the weight matrix is read exactly once, HBM -> registers with 128-bit
// loads that bypass L1, and fed straight to warp-level tensor-core MMAs; the (tiny) activation
// slice sits in shared memory.  The problem is computed transposed -- weights are the 16-row MMA
// operand, tokens the 8-column operand -- so no lane is wasted on padding when M is 1..8.
//
// Lane (g, t) loads 16 consecutive K-bytes of weight rows n0+g and n0+g+8.  An MMA sums over its
// 32 k-slots in any order, so the 16 loaded bytes are used as k-slots {4t..4t+3, 16+4t..16+4t+3}
// of two consecutive MMAs, with the activation fragment taken from the same 16 bytes of the token
// row: no shuffles, no byte permutes.
//
// Grid: (ceil(N/128), S).  Each block owns 128 weight rows (16 per warp) and one K slice.  When
// S > 1 the slices' partial sums go to the workspace and the block that arrives last for a row
// panel adds them in slice order (deterministic, exact for int32) and runs the epilogue.
#include "gemm_w8a8.cuh"

#include <mutex>

namespace llmqrt {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerBlock = 128;
constexpr int kChunk = 64;      // K bytes consumed per warp step (4 lanes x 16 B per row)
constexpr int kUnroll = 4;      // chunks in flight per thread

template <int KIND> struct AccOf { using type = float; };
template <> struct AccOf<KIND_I8> { using type = int; };

template <int KIND>
__device__ __forceinline__ void mma8(typename AccOf<KIND>::type (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                     uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (KIND == KIND_I8) mma_s8_16832(c, a0, a1, a2, a3, b0, b1);
  else mma_f8_16832<KIND == KIND_F8_E5M2>(c, a0, a1, a2, a3, b0, b1);
}

__host__ __device__ inline int xs_stride_for(int kps) { return (kps % 128 == 0) ? kps + 64 : kps; }

template <int KIND, int MB>
__global__ void __launch_bounds__(kThreads)
w8a8_stream_kernel(const uint8_t* __restrict__ A, int64_t lda, const uint8_t* __restrict__ W, int64_t ldw, int M,
                   int N, int K, int kps, int num_splits, void* __restrict__ partials, int* __restrict__ counters,
                   Epilogue epi) {
  using Acc = typename AccOf<KIND>::type;
  extern __shared__ __align__(16) uint8_t xs[];
  __shared__ int s_ticket;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int k_begin = blockIdx.y * kps;
  const int k_len = min(kps, K - k_begin);          // > 0 by construction, multiple of 16
  const int stride = xs_stride_for(kps);

  // ---- stage the activation slice: rows >= M and columns >= k_len are zero ----
  {
    const int chunks = kps / 16;
    for (int i = tid; i < MB * 8 * chunks; i += kThreads) {
      const int r = i / chunks, c = i - r * chunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < M && c * 16 < k_len) v = *reinterpret_cast<const uint4*>(A + (int64_t)r * lda + k_begin + c * 16);
      *reinterpret_cast<uint4*>(xs + r * stride + c * 16) = v;
    }
  }
  __syncthreads();

  const int n0 = blockIdx.x * kRowsPerBlock + warp * 16;
  Acc acc[MB][4];
#pragma unroll
  for (int i = 0; i < MB; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;

  if (n0 < N) {
    const uint8_t* wa = W + (int64_t)min(n0 + g, N - 1) * ldw + k_begin + 16 * t;
    const uint8_t* wb = W + (int64_t)min(n0 + g + 8, N - 1) * ldw + k_begin + 16 * t;
    const uint8_t* xrow = xs + g * stride + 16 * t;
    const int my_len = k_len - 16 * t;               // this lane's 16 bytes at chunk kc are valid iff kc < my_len

    for (int kc = 0; kc < k_len; kc += kChunk * kUnroll) {
      uint4 ra[kUnroll], rb[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = kc + u * kChunk;
        if (k < my_len) {
          ra[u] = ldg_stream_16B(wa + k);
          rb[u] = ldg_stream_16B(wb + k);
        } else {
          ra[u] = make_uint4(0, 0, 0, 0);
          rb[u] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = kc + u * kChunk;
        if (k < k_len) {                              // warp-uniform
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            const uint4 x = *reinterpret_cast<const uint4*>(xrow + mb * 8 * stride + k);
            mma8<KIND>(acc[mb], ra[u].x, rb[u].x, ra[u].y, rb[u].y, x.x, x.y);
            mma8<KIND>(acc[mb], ra[u].z, rb[u].z, ra[u].w, rb[u].w, x.z, x.w);
          }
        }
      }
    }
  }

  const float alpha = epi.alpha_dev ? *epi.alpha_dev : epi.alpha;

  if (num_splits == 1) {
    if (n0 < N) {
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + g + (j >> 1) * 8, m = mb * 8 + 2 * t + (j & 1);
          if (n < N && m < M) epilogue_store<Acc>(epi, acc[mb][j], m, n, alpha);
        }
    }
    return;
  }

  // ---- split-K: publish this slice's partial sums, last arriver reduces ----
  Acc* part = reinterpret_cast<Acc*>(partials);
  if (n0 < N) {
    Acc* mine = part + (int64_t)blockIdx.y * M * N;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + g + (j >> 1) * 8, m = mb * 8 + 2 * t + (j & 1);
        if (n < N && m < M) mine[(int64_t)m * N + n] = acc[mb][j];
      }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(&counters[blockIdx.x], 1);
  __syncthreads();
  if (s_ticket != num_splits - 1) return;
  __threadfence();

  const int nb0 = blockIdx.x * kRowsPerBlock;
  if ((N & 3) == 0 && M >= 4) {
    // enough rows to keep every thread busy with vectors: four columns per thread and the slices
    // four at a time -- the loads of a thread do not depend on one another, so the fix-up costs a
    // few L2 round trips instead of one per slice and element
    constexpr int kVecs = kRowsPerBlock / 4;
    for (int i = tid; i < M * kVecs; i += kThreads) {
      const int m = i / kVecs, n = nb0 + (i % kVecs) * 4;
      if (n >= N) continue;
      Acc sum[4] = {0, 0, 0, 0};
#pragma unroll 4
      for (int s = 0; s < num_splits; ++s) {
        const uint4 p = __ldcg(reinterpret_cast<const uint4*>(part + ((int64_t)s * M + m) * N + n));
        const Acc* pv = reinterpret_cast<const Acc*>(&p);
#pragma unroll
        for (int j = 0; j < 4; ++j) sum[j] += pv[j];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) epilogue_store<Acc>(epi, sum[j], m, n + j, alpha);
    }
  } else {
    for (int i = tid; i < M * kRowsPerBlock; i += kThreads) {
      const int m = i / kRowsPerBlock, n = nb0 + (i % kRowsPerBlock);
      if (n >= N) continue;
      Acc sum = 0;
#pragma unroll 4
      for (int s = 0; s < num_splits; ++s) sum += __ldcg(part + ((int64_t)s * M + m) * N + n);
      epilogue_store<Acc>(epi, sum, m, n, alpha);
    }
  }
  if (tid == 0) counters[blockIdx.x] = 0;            // leave the workspace ready for the next call
}

template <int KIND, int MB>
int launch(const uint8_t* A, int64_t lda, const uint8_t* W, int64_t ldw, int M, int N, int K, const Epilogue& epi,
           void* workspace, cudaStream_t st) {
  const int n_blocks = (int)ceil_div(N, kRowsPerBlock);
  // K slice per block: enough blocks to cover every SM about three times, slices of at least 256
  // bytes, and an activation slice that fits in 96 KiB of shared memory.
  const int max_kps_smem = ((96 * 1024) / (MB * 8) - 64) / 64 * 64;
  int want_splits = (int)ceil_div(3 * sm_count(), n_blocks);
  if (want_splits > 16) want_splits = 16;            // the last block adds all slices: keep that tail short
  int kps = (int)ceil_div(ceil_div(K, want_splits), 64) * 64;
  if (kps < 256) kps = 256;
  if (kps > max_kps_smem) kps = max_kps_smem;
  if (kps > (int)ceil_div(K, 64) * 64) kps = (int)ceil_div(K, 64) * 64;
  int splits = (int)ceil_div(K, kps);
  const size_t acc_bytes = 4;
  while (splits > 1 && (size_t)splits * M * N * acc_bytes > LLMQRT_WS_PARTIAL_BYTES) {
    kps += 64;
    if (kps > max_kps_smem) return set_error(LLMQRT_ERR_WORKSPACE, "w8a8 stream: partial sums do not fit the workspace");
    splits = (int)ceil_div(K, kps);
  }
  if (splits > 1) {
    if (!workspace) return set_error(LLMQRT_ERR_WORKSPACE, "w8a8 stream: split-K needs the workspace");
    if (n_blocks > LLMQRT_WS_NUM_COUNTERS) return set_error(LLMQRT_ERR_INVALID, "w8a8 stream: N too large");
  }
  const size_t smem = (size_t)MB * 8 * xs_stride_for(kps);
  auto kern = w8a8_stream_kernel<KIND, MB>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem)) return rc;
  dim3 grid(n_blocks, splits);
  kern<<<grid, kThreads, smem, st>>>(A, lda, W, ldw, M, N, K, kps, splits,
                                     workspace ? ws_partials(workspace) : nullptr,
                                     workspace ? ws_counters(workspace) : nullptr, epi);
  return check_launch("w8a8_stream");
}

template <int KIND>
int launch_mb(const uint8_t* A, int64_t lda, const uint8_t* W, int64_t ldw, int M, int N, int K, const Epilogue& epi,
              void* workspace, cudaStream_t st) {
  if (M <= 8) return launch<KIND, 1>(A, lda, W, ldw, M, N, K, epi, workspace, st);
  if (M <= 16) return launch<KIND, 2>(A, lda, W, ldw, M, N, K, epi, workspace, st);
  if (M <= 32) return launch<KIND, 4>(A, lda, W, ldw, M, N, K, epi, workspace, st);
  return launch<KIND, 8>(A, lda, W, ldw, M, N, K, epi, workspace, st);
}

}  // namespace

int w8a8_gemm_stream(int kind, const uint8_t* A, int64_t lda, const uint8_t* W, int64_t ldw, int64_t M, int64_t N,
                     int64_t K, const Epilogue& epi_in, void* workspace, cudaStream_t st) {
  // Token panels of at most 64 rows; larger M re-streams the weights once per panel (the tcgen05
  // kernel is the intended path there).
  for (int64_t m0 = 0; m0 < M; m0 += 64) {
    const int mc = (int)((M - m0 < 64) ? (M - m0) : 64);
    Epilogue epi = epi_in;
    const int64_t elt = (epi.mode == EPI_RAW || epi.out_dtype == LLMQRT_F32) ? 4 : 2;
    epi.out = reinterpret_cast<char*>(epi_in.out) + m0 * epi_in.ldo * elt;
    if (epi.row_scale) epi.row_scale = epi_in.row_scale + m0;
    const uint8_t* a = A + m0 * lda;
    int rc;
    if (kind == KIND_I8) rc = launch_mb<KIND_I8>(a, lda, W, ldw, mc, (int)N, (int)K, epi, workspace, st);
    else if (kind == KIND_F8_E4M3) rc = launch_mb<KIND_F8_E4M3>(a, lda, W, ldw, mc, (int)N, (int)K, epi, workspace, st);
    else rc = launch_mb<KIND_F8_E5M2>(a, lda, W, ldw, mc, (int)N, (int)K, epi, workspace, st);
    if (rc) return rc;
  }
  return LLMQRT_OK;
}

}  // namespace llmqrt

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of the per-channel int8 linear.
//
// Some hosts give a library nothing but the tensors of the call: an inference server that carves up
// all device memory at start-up and forbids plug-ins to call cudaMalloc, or a decode loop that cannot
// afford the device-wide synchronisation a cudaMalloc / cudaFree implies.  Such a caller has no way
// to provide the split-K workspace the regular entry points expect.  This entry point therefore
// carries its own scratch: a fixed array in the library's device data segment.  It costs
// kNoAllocScratchBytes of device memory on every GPU that loads the library, for as long as the
// process lives, and it bounds the problem size (see the error message below).
//
// The array is shared by every call and keeps whatever the previous call left in it.  The arrival
// counters are therefore cleared on the stream at the start of each call; the partial sums need no
// clearing because every slot that is read has been written by the same launch.  Two calls that may
// run at the same time on one GPU (different streams without a dependency) would race on it.
//
// The device address of the array is looked up with cudaGetSymbolAddress the first time the entry
// point runs on a device (the array's name is only a host-side handle, not a pointer a kernel could
// use).  That first call should be made before any stream capture begins.
// ------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kNoAllocCounterBytes = 16 * 1024;                    // 4096 row panels of 128 outputs
constexpr size_t kNoAllocPartialBytes = (size_t)8 << 20;              // split-K partial sums
constexpr size_t kNoAllocScratchBytes = kNoAllocCounterBytes + kNoAllocPartialBytes;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of g_noalloc_scratch on the current device, resolved once per device.
int noalloc_scratch(unsigned char** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static unsigned char* table[kMaxDevices] = {nullptr};
  int dev = 0;
  LLMQRT_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return llmqrt::set_error(LLMQRT_ERR_UNSUPPORTED, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!table[dev]) {
    void* p = nullptr;
    LLMQRT_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch));      // `dev` is the current device
    table[dev] = static_cast<unsigned char*>(p);
  }
  *out = table[dev];
  return LLMQRT_OK;
}

template <int MB>
int launch_noalloc(const uint8_t* A, int64_t lda, const uint8_t* W, int64_t ldw, int M, int N, int K,
                   const llmqrt::Epilogue& epi, unsigned char* scratch, cudaStream_t st) {
  using namespace llmqrt;
  const int n_blocks = (int)ceil_div(N, kRowsPerBlock);
  if ((size_t)n_blocks * sizeof(int) > kNoAllocCounterBytes)
    return set_error(LLMQRT_ERR_WORKSPACE, "no-alloc int8 linear: N=%d exceeds the built-in scratch (max N = %d)", N,
                     (int)(kNoAllocCounterBytes / sizeof(int)) * kRowsPerBlock);
  // Same decomposition rule as the regular path, with the partial sums limited to the built-in array.
  const int max_kps_smem = ((96 * 1024) / (MB * 8) - 64) / 64 * 64;
  int want_splits = (int)ceil_div(3 * sm_count(), n_blocks);
  if (want_splits > 16) want_splits = 16;            // the last block adds all slices: keep that tail short
  int kps = (int)ceil_div(ceil_div(K, want_splits), 64) * 64;
  if (kps < 256) kps = 256;
  if (kps > max_kps_smem) kps = max_kps_smem;
  if (kps > (int)ceil_div(K, 64) * 64) kps = (int)ceil_div(K, 64) * 64;
  int splits = (int)ceil_div(K, kps);
  while (splits > 1 && (size_t)splits * M * N * 4 > kNoAllocPartialBytes) {
    kps += 64;
    if (kps > max_kps_smem)
      return set_error(LLMQRT_ERR_WORKSPACE,
                       "no-alloc int8 linear: M=%d N=%d K=%d needs more than the %zu-byte built-in scratch; "
                       "use llmqrt_w8a8_int8_linear_per_channel with a caller-provided workspace",
                       M, N, K, kNoAllocPartialBytes);
    splits = (int)ceil_div(K, kps);
  }
  int* counters = reinterpret_cast<int*>(scratch);
  void* partials = scratch + kNoAllocCounterBytes;
  if (splits > 1) LLMQRT_CUDA_OK(cudaMemsetAsync(counters, 0, (size_t)n_blocks * sizeof(int), st));
  const size_t smem = (size_t)MB * 8 * xs_stride_for(kps);
  auto kern = w8a8_stream_kernel<KIND_I8, MB>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem)) return rc;
  kern<<<dim3(n_blocks, splits), kThreads, smem, st>>>(A, lda, W, ldw, M, N, K, kps, splits, partials, counters, epi);
  return check_launch("w8a8_stream (no-alloc)");
}

}  // namespace

extern "C" int llmqrt_w8a8_int8_linear_per_channel_noalloc(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw,
                                                           const void* bias, int bias_dtype, const float* a_scale,
                                                           const float* w_scale, void* out, int out_dtype, int64_t ldo,
                                                           int64_t M, int64_t N, int64_t K, llmqrt_stream_t stream) {
  using namespace llmqrt;
  LLMQRT_REQUIRE(a && w && out && a_scale && w_scale, "no-alloc int8 linear: null pointer");
  LLMQRT_REQUIRE(M >= 0 && N > 0 && K > 0 && N < (1ll << 31) && K < (1ll << 31), "no-alloc int8 linear: bad shape");
  LLMQRT_REQUIRE(M <= 64, "no-alloc int8 linear: M=%lld exceeds the supported maximum of 64 rows", (long long)M);
  LLMQRT_REQUIRE(K % 16 == 0 && lda >= K && ldw >= K && lda % 16 == 0 && ldw % 16 == 0 && ldo >= N,
                 "no-alloc int8 linear: K and the leading dimensions must be multiples of 16 (K=%lld)", (long long)K);
  LLMQRT_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                 "no-alloc int8 linear: operands must be 16-byte aligned");
  LLMQRT_REQUIRE(out_dtype == LLMQRT_F16 || out_dtype == LLMQRT_BF16, "no-alloc int8 linear: out must be fp16/bf16");
  LLMQRT_REQUIRE(!bias || bias_dtype == LLMQRT_F16 || bias_dtype == LLMQRT_BF16 || bias_dtype == LLMQRT_F32,
                 "no-alloc int8 linear: bad bias dtype");
  if (M == 0) return LLMQRT_OK;
  unsigned char* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  Epilogue e{};
  e.mode = EPI_COL_ROW; e.out_dtype = out_dtype; e.bias_dtype = bias_dtype; e.bias = bias; e.row_scale = a_scale;
  e.col_scale = w_scale; e.out = out; e.ldo = ldo;
  const uint8_t* A8 = reinterpret_cast<const uint8_t*>(a);
  const uint8_t* W8 = reinterpret_cast<const uint8_t*>(w);
  cudaStream_t st = (cudaStream_t)stream;
  if (M <= 8) return launch_noalloc<1>(A8, lda, W8, ldw, (int)M, (int)N, (int)K, e, scratch, st);
  if (M <= 16) return launch_noalloc<2>(A8, lda, W8, ldw, (int)M, (int)N, (int)K, e, scratch, st);
  if (M <= 32) return launch_noalloc<4>(A8, lda, W8, ldw, (int)M, (int)N, (int)K, e, scratch, st);
  return launch_noalloc<8>(A8, lda, W8, ldw, (int)M, (int)N, (int)K, e, scratch, st);
}
