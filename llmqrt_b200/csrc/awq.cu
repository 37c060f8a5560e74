// AWQ W4A16: dequantization, one-time repack into a K-major streaming layout, and the
// weight-streaming dequant-GEMM for decode-sized M.
//
// Reference storage packs eight 4-bit values per int32 ALONG N with the nibble order
// {0,2,4,6,1,3,5,7}.  A tensor-core operand register must hold two K-consecutive values of one
// output column, so streaming that layout would need a transpose in registers.  The repack turns
// a layer into
//     wq_t [N, K/8]  : word (n, j) = values k = 8j..8j+7 of column n, value 2p in nibble p and value
//                      2p+1 in nibble p+4, so `(w >> 4p) & 0x000F000F | 0x64006400` is the half2
//                      {1024 + v[2p], 1024 + v[2p+1]} in one shift and one logic op;
//     sz_t [N, K/G]  : half2 { scale, -(1024 + zero) }.
// Dequantization is then  (h + (-(1024+zero))) * scale  = exactly fp16((v - zero) * scale): the
// subtraction is exact and the product is rounded once, like the reference's kernels.
//
// The decode-sized GEMM (M <= 64) is computed transposed (weights are the 16-row MMA operand, tokens the
// 8-column one), each warp owns 32 weight rows so that one activation fragment feeds two weight
// fragments, and the reduction dimension is split across blocks with a deterministic last-arriver
// fix-up.  Above 64 tokens the same entry point runs the TMA + tcgen05 GEMM kernel with the weight
// operand dequantized tile by tile into shared memory by extra warps of that kernel (gemm_tc.cu).
#include "gemm_w8a8.cuh"

namespace llmqrt {
namespace {

__device__ __forceinline__ int rev_nibble(int c) {
  // nibble index that holds logical column c of a word: inverse of {0,2,4,6,1,3,5,7}
  return ((c & 1) << 2) | (c >> 1);
}

// ---- reference layout -> W[K, N] fp16 -----------------------------------------------------------
__global__ void __launch_bounds__(256)
awq_dequantize_kernel(const uint32_t* __restrict__ qweight, const __half* __restrict__ scales,
                      const uint32_t* __restrict__ qzeros, int64_t K, int64_t NW, int64_t G, __half* __restrict__ out) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= K * NW) return;
  const int64_t k = idx / NW, j = idx - k * NW, kg = k / G;
  const uint32_t w = qweight[idx], z = qzeros[kg * NW + j];
  const uint4 sv = *reinterpret_cast<const uint4*>(scales + (kg * NW + j) * 8);
  const __half* s = reinterpret_cast<const __half*>(&sv);
  __align__(16) __half o[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int sh = 4 * rev_nibble(c);
    const int d = (int)((w >> sh) & 0xF) - (int)((z >> sh) & 0xF);
    o[c] = __float2half_rn((float)d * __half2float(s[c]));
  }
  *reinterpret_cast<uint4*>(out + (k * NW + j) * 8) = *reinterpret_cast<const uint4*>(o);
}

// ---- reference layout -> streaming layout ---------------------------------------------------------
__global__ void __launch_bounds__(256)
awq_repack_weights_kernel(const uint32_t* __restrict__ qweight, int64_t K, int64_t N, uint32_t* __restrict__ wq_t) {
  // consecutive threads take consecutive n (reads coalesce); one output word per thread
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t KW = K / 8;
  if (idx >= N * KW) return;
  const int64_t j = idx / N, n = idx - j * N;
  const int sh = 4 * rev_nibble((int)(n & 7));
  uint32_t word = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const uint32_t v = (qweight[(8 * j + e) * (N / 8) + (n >> 3)] >> sh) & 0xF;
    word |= v << (4 * (e >> 1) + 16 * (e & 1));
  }
  wq_t[n * KW + j] = word;
}

__global__ void __launch_bounds__(256)
awq_repack_scales_kernel(const __half* __restrict__ scales, const uint32_t* __restrict__ qzeros, int64_t KG, int64_t N,
                         uint32_t* __restrict__ sz_t) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * KG) return;
  const int64_t kg = idx / N, n = idx - kg * N;
  const uint32_t z = (qzeros[kg * (N / 8) + (n >> 3)] >> (4 * rev_nibble((int)(n & 7)))) & 0xF;
  const __half2 v = __halves2half2(scales[kg * N + n], __float2half_rn(-(1024.f + (float)z)));
  sz_t[n * KG + kg] = *reinterpret_cast<const uint32_t*>(&v);
}

// ---- streaming layout -> W^T[N, K] fp16 -----------------------------------------------------------
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 negz, __half2 s, uint32_t (&out)[4]) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint32_t h = ((w >> (4 * p)) & 0x000F000Fu) | 0x64006400u;
    __half2 v = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&h), negz), s);
    out[p] = *reinterpret_cast<uint32_t*>(&v);
  }
}

__global__ void __launch_bounds__(256)
awq_dequantize_t_kernel(const uint32_t* __restrict__ wq_t, const uint32_t* __restrict__ sz_t, int64_t KW, int64_t N,
                        int64_t G, __half* __restrict__ out) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * KW) return;
  const int64_t n = idx / KW, j = idx - n * KW;
  const uint32_t szv = sz_t[n * (KW * 8 / G) + (8 * j) / G];
  const __half2 sz = *reinterpret_cast<const __half2*>(&szv);
  uint32_t o[4];
  dequant_word(wq_t[idx], __half2half2(__high2half(sz)), __half2half2(__low2half(sz)), o);
  *reinterpret_cast<uint4*>(out + idx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

// ---- streaming dequant-GEMM -------------------------------------------------------------------------
constexpr int kThreads = 128;          // 4 warps
constexpr int kRowsPerWarp = 32;
constexpr int kRowsPerBlock = 128;
constexpr int kChunkK = 128;           // k-values per warp step: 4 lanes x 32 per weight row

// Activation slice in shared memory: row stride = kps*2 + 16 bytes and 16-byte chunk c stored at
// c ^ (((c >> 3) & 1) << 1), which makes the eight lanes of every 128-bit load phase hit 32 distinct banks.
__host__ __device__ inline int xs_stride_bytes(int kps) { return kps * 2 + 16; }
__device__ __forceinline__ int xs_chunk(int c) { return c ^ (((c >> 3) & 1) << 1); }

template <int MB>
__global__ void __launch_bounds__(kThreads)
awq_gemm_stream_kernel(const __half* __restrict__ X, int64_t ldx, const uint32_t* __restrict__ wq_t,
                       const uint32_t* __restrict__ sz_t, int M, int N, int K, int G, int kps, int num_splits,
                       float* __restrict__ partials, int* __restrict__ counters, Epilogue epi) {
  extern __shared__ __align__(16) uint8_t xs[];
  __shared__ int s_ticket;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int k_begin = blockIdx.y * kps;
  const int k_len = min(kps, K - k_begin);        // multiple of 32
  const int stride = xs_stride_bytes(kps);
  const int KW = K / 8, KG = K / G;

  {
    const int chunks = kps / 8;                   // 16-byte chunks (8 halves) per row
    for (int i = tid; i < MB * 8 * chunks; i += kThreads) {
      const int r = i / chunks, c = i - r * chunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < M && c * 8 < k_len) v = *reinterpret_cast<const uint4*>(X + (int64_t)r * ldx + k_begin + c * 8);
      *reinterpret_cast<uint4*>(xs + r * stride + xs_chunk(c) * 16) = v;
    }
  }
  __syncthreads();

  const int n0 = blockIdx.x * kRowsPerBlock + warp * kRowsPerWarp;
  float acc[2][MB][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int i = 0; i < MB; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[h][i][j] = 0.f;

  if (n0 < N) {
    // rows handled by this lane: n0 + 16h + g and n0 + 16h + g + 8
    int rows[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) rows[r] = min(n0 + 16 * (r >> 1) + g + 8 * (r & 1), N - 1);
    const int my_len = k_len - 32 * t;

    // The weights of step kc + 1 are requested before step kc is consumed (two register sets), so a
    // block's steps overlap their load latency instead of paying it one after the other.
    uint4 wnext[4];
    uint32_t sznext[4];
    auto fetch = [&](int kc) {
      const bool valid = kc < my_len;
      const int kk = k_begin + kc + 32 * t;       // first k of this lane's 32 values
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        if (valid) {
          wnext[r] = ldg_stream_16B(wq_t + (int64_t)rows[r] * KW + kk / 8);
          sznext[r] = __ldg(sz_t + (int64_t)rows[r] * KG + kk / G);
        } else {
          wnext[r] = make_uint4(0, 0, 0, 0);
          sznext[r] = 0;                            // scale 0: contributes nothing
        }
      }
    };
    fetch(0);
    for (int kc = 0; kc < k_len; kc += kChunkK) {
      uint4 wv[4];
      uint32_t szv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        wv[r] = wnext[r];
        szv[r] = sznext[r];
      }
      if (kc + kChunkK < k_len) fetch(kc + kChunkK);
      const uint32_t* wp[4] = {&wv[0].x, &wv[1].x, &wv[2].x, &wv[3].x};
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        uint32_t a[4][4];                           // [row][pair]
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const __half2 sz = *reinterpret_cast<const __half2*>(&szv[r]);
          dequant_word(wp[r][wi], __half2half2(__high2half(sz)), __half2half2(__low2half(sz)), a[r]);
        }
        const int c = (kc + 32 * t) / 8 + wi;       // 16-byte chunk of the activation row
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const uint4 x = *reinterpret_cast<const uint4*>(xs + (mb * 8 + g) * stride + xs_chunk(c) * 16);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            mma_16816<false>(acc[h][mb], a[2 * h][0], a[2 * h + 1][0], a[2 * h][1], a[2 * h + 1][1], x.x, x.y);
            mma_16816<false>(acc[h][mb], a[2 * h][2], a[2 * h + 1][2], a[2 * h][3], a[2 * h + 1][3], x.z, x.w);
          }
        }
      }
    }
  }

  const float alpha = 1.f;
  auto for_each_acc = [&](auto&& fn) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + 16 * h + g + (j >> 1) * 8, m = mb * 8 + 2 * t + (j & 1);
          if (n < N && m < M) fn(acc[h][mb][j], m, n);
        }
  };

  if (num_splits == 1) {
    if (n0 < N) for_each_acc([&](float v, int m, int n) { epilogue_store<float>(epi, v, m, n, alpha); });
    return;
  }
  if (n0 < N) {
    float* mine = partials + (int64_t)blockIdx.y * M * N;
    for_each_acc([&](float v, int m, int n) { mine[(int64_t)m * N + n] = v; });
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_ticket = atomicAdd(&counters[blockIdx.x], 1);
  __syncthreads();
  if (s_ticket != num_splits - 1) return;
  __threadfence();
  // N is a multiple of 8: four columns per thread, slices four at a time (independent loads, so the
  // fix-up costs a few L2 round trips instead of one per slice and element)
  const int nb0 = blockIdx.x * kRowsPerBlock;
  constexpr int kVecs = kRowsPerBlock / 4;
  if (M < 4) {                                     // too few rows to keep every thread busy with vectors
    for (int i = tid; i < M * kRowsPerBlock; i += kThreads) {
      const int m = i / kRowsPerBlock, n = nb0 + (i % kRowsPerBlock);
      if (n >= N) continue;
      float sum = 0.f;
#pragma unroll 4
      for (int s = 0; s < num_splits; ++s) sum += __ldcg(partials + ((int64_t)s * M + m) * N + n);
      epilogue_store<float>(epi, sum, m, n, alpha);
    }
    if (tid == 0) counters[blockIdx.x] = 0;
    return;
  }
  for (int i = tid; i < M * kVecs; i += kThreads) {
    const int m = i / kVecs, n = nb0 + (i % kVecs) * 4;
    if (n >= N) continue;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int s = 0; s < num_splits; ++s) {
      const float4 p = __ldcg(reinterpret_cast<const float4*>(partials + ((int64_t)s * M + m) * N + n));
      sum[0] += p.x; sum[1] += p.y; sum[2] += p.z; sum[3] += p.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) epilogue_store<float>(epi, sum[j], m, n + j, alpha);
  }
  if (tid == 0) counters[blockIdx.x] = 0;
}

template <int MB>
int launch_gemm(const __half* X, int64_t ldx, const uint32_t* wq_t, const uint32_t* sz_t, int M, int N, int K, int G,
                const Epilogue& epi, void* workspace, cudaStream_t st) {
  const int n_blocks = (int)ceil_div(N, kRowsPerBlock);
  const int max_kps_smem = ((96 * 1024) / (MB * 8) - 16) / 2 / kChunkK * kChunkK;
  // enough blocks to cover every SM about four times, but at most 16 slices: the block that arrives
  // last adds them all, and that serial tail outweighs finer slices
  int want_splits = (int)ceil_div(4 * sm_count(), n_blocks);
  if (want_splits > 16) want_splits = 16;
  int kps = (int)ceil_div(ceil_div(K, want_splits), kChunkK) * kChunkK;
  if (kps < 256) kps = 256;
  if (kps > max_kps_smem) kps = max_kps_smem;
  if (kps > (int)ceil_div(K, kChunkK) * kChunkK) kps = (int)ceil_div(K, kChunkK) * kChunkK;
  int splits = (int)ceil_div(K, kps);
  while (splits > 1 && (size_t)splits * M * N * 4 > LLMQRT_WS_PARTIAL_BYTES) {
    kps += kChunkK;
    if (kps > max_kps_smem) return set_error(LLMQRT_ERR_WORKSPACE, "awq gemm: partial sums do not fit the workspace");
    splits = (int)ceil_div(K, kps);
  }
  if (splits > 1) {
    if (!workspace) return set_error(LLMQRT_ERR_WORKSPACE, "awq gemm: split-K needs the workspace");
    if (n_blocks > LLMQRT_WS_NUM_COUNTERS) return set_error(LLMQRT_ERR_INVALID, "awq gemm: N too large");
  }
  const size_t smem = (size_t)MB * 8 * xs_stride_bytes(kps);
  auto kern = awq_gemm_stream_kernel<MB>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem)) return rc;
  kern<<<dim3(n_blocks, splits), kThreads, smem, st>>>(
      X, ldx, wq_t, sz_t, M, N, K, G, kps, splits,
      workspace ? reinterpret_cast<float*>(ws_partials(workspace)) : nullptr,
      workspace ? ws_counters(workspace) : nullptr, epi);
  return check_launch("awq_gemm_stream");
}

int check_layer(int64_t K, int64_t N, int64_t G) {
  LLMQRT_REQUIRE(K > 0 && N > 0 && G > 0, "awq: bad shape K=%lld N=%lld G=%lld", (long long)K, (long long)N, (long long)G);
  LLMQRT_REQUIRE(N % 8 == 0, "awq: N=%lld must be a multiple of 8", (long long)N);
  LLMQRT_REQUIRE(K % G == 0, "awq: K=%lld must be a multiple of the group size %lld", (long long)K, (long long)G);
  LLMQRT_REQUIRE(K < (1ll << 31) && N < (1ll << 31), "awq: dimension too large");
  return LLMQRT_OK;
}

}  // namespace
}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_awq_dequantize(const int32_t* qweight, const void* scales, const int32_t* qzeros, int64_t K, int64_t N,
                          int64_t group_size, void* out, llmqrt_stream_t stream) {
  if (int rc = check_layer(K, N, group_size)) return rc;
  LLMQRT_REQUIRE(qweight && scales && qzeros && out, "awq_dequantize: null pointer");
  const int64_t total = K * (N / 8);
  awq_dequantize_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint32_t*>(qweight), reinterpret_cast<const __half*>(scales),
      reinterpret_cast<const uint32_t*>(qzeros), K, N / 8, group_size, reinterpret_cast<__half*>(out));
  return check_launch("awq_dequantize");
}

int llmqrt_awq_repack(const int32_t* qweight, const void* scales, const int32_t* qzeros, int64_t K, int64_t N,
                      int64_t group_size, uint32_t* wq_t, uint32_t* sz_t, llmqrt_stream_t stream) {
  if (int rc = check_layer(K, N, group_size)) return rc;
  LLMQRT_REQUIRE(K % 8 == 0, "awq_repack: K=%lld must be a multiple of 8", (long long)K);
  LLMQRT_REQUIRE(qweight && scales && qzeros && wq_t && sz_t, "awq_repack: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  awq_repack_weights_kernel<<<(unsigned)ceil_div(N * (K / 8), 256), 256, 0, st>>>(
      reinterpret_cast<const uint32_t*>(qweight), K, N, wq_t);
  if (int rc = check_launch("awq_repack_weights")) return rc;
  awq_repack_scales_kernel<<<(unsigned)ceil_div(N * (K / group_size), 256), 256, 0, st>>>(
      reinterpret_cast<const __half*>(scales), reinterpret_cast<const uint32_t*>(qzeros), K / group_size, N, sz_t);
  return check_launch("awq_repack_scales");
}

int llmqrt_awq_dequantize_t(const uint32_t* wq_t, const uint32_t* sz_t, int64_t K, int64_t N, int64_t group_size,
                            void* out, llmqrt_stream_t stream) {
  if (int rc = check_layer(K, N, group_size)) return rc;
  LLMQRT_REQUIRE(K % 8 == 0 && group_size % 8 == 0, "awq_dequantize_t: K and group size must be multiples of 8");
  LLMQRT_REQUIRE(wq_t && sz_t && out, "awq_dequantize_t: null pointer");
  awq_dequantize_t_kernel<<<(unsigned)ceil_div(N * (K / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      wq_t, sz_t, K / 8, N, group_size, reinterpret_cast<__half*>(out));
  return check_launch("awq_dequantize_t");
}

int llmqrt_awq_gemm(const void* x, int64_t ldx, const uint32_t* wq_t, const uint32_t* sz_t, const void* bias,
                    void* out, int64_t ldo, int64_t M, int64_t N, int64_t K, int64_t group_size, void* workspace,
                    llmqrt_stream_t stream) {
  if (int rc = check_layer(K, N, group_size)) return rc;
  LLMQRT_REQUIRE(x && wq_t && sz_t && out, "awq_gemm: null pointer");
  LLMQRT_REQUIRE(K % 32 == 0 && group_size % 32 == 0, "awq_gemm: K and group size must be multiples of 32");   // (a thread's 32 values of a K block share one group)
  LLMQRT_REQUIRE(ldx >= K && ldx % 8 == 0 && ldo >= N, "awq_gemm: bad leading dimension");
  LLMQRT_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(wq_t) & 15) == 0,
                 "awq_gemm: operands must be 16-byte aligned");
  LLMQRT_REQUIRE(M >= 0 && M < (1ll << 31), "awq_gemm: bad M");
  Epilogue e{};
  e.mode = EPI_TENSOR; e.out_dtype = LLMQRT_F16; e.bias_dtype = LLMQRT_F16; e.alpha = 1.f; e.beta = 1.f; e.bias = bias;
  e.ldo = ldo;
  const __half* xp = reinterpret_cast<const __half*>(x);
  cudaStream_t st = (cudaStream_t)stream;
  if (M >= 1024 && workspace && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ldo % 8 == 0) {
    // A thousand tokens and more: the GEMM is compute-bound, the two-CTA fp16 kernel runs about twice
    // as fast as the kernel that dequantizes into its own shared memory (whose dequantizing warps and
    // tensor core share the SM's shared-memory bandwidth), and writing the fp16 weights out once and
    // reading them back costs a tenth of the GEMM.  The weights are expanded panel by panel into the
    // workspace (same rounding: fp16((v - z) * s)) and each panel is multiplied by the dense kernel.
    const int64_t cap_rows = (int64_t)(LLMQRT_WS_PARTIAL_BYTES / (size_t)(K * 2)) / 256 * 256;
    if (cap_rows >= 256) {
      __half* deq = reinterpret_cast<__half*>(ws_partials(workspace));
      for (int64_t n0 = 0; n0 < N; n0 += cap_rows) {
        const int64_t nc = (N - n0 < cap_rows) ? (N - n0) : cap_rows;
        awq_dequantize_t_kernel<<<(unsigned)ceil_div(nc * (K / 8), 256), 256, 0, st>>>(
            wq_t + n0 * (K / 8), sz_t + n0 * (K / group_size), K / 8, nc, group_size, deq);
        if (int rc = check_launch("awq_dequantize_t")) return rc;
        Epilogue ep = e;
        ep.out = reinterpret_cast<__half*>(out) + n0;
        ep.bias = bias ? reinterpret_cast<const __half*>(bias) + n0 : nullptr;
        if (int rc = gemm_tc(KIND_F16, x, ldx, deq, K, M, nc, K, ep, workspace, st)) return rc;
      }
      return LLMQRT_OK;
    }
  }
  if (M > 64) {
    // 64 < M < 1024: ONE kernel.  The tcgen05 GEMM runs with four extra warps that turn the
    // packed 4-bit tiles into fp16 operand tiles in shared memory (same rounding: fp16((v - z) * s)),
    // so the dequantized weights never exist in global memory.
    e.out = out;
    const AwqOperand op = {wq_t, sz_t, group_size};
    return gemm_tc(KIND_F16, x, ldx, nullptr, 0, M, N, K, e, workspace, st, false, &op);
  }
  for (int64_t m0 = 0; m0 < M; m0 += 32) {       // token panels of 32: larger M re-streams the weights per panel
    const int mc = (int)((M - m0 < 32) ? (M - m0) : 32);
    e.out = reinterpret_cast<__half*>(out) + m0 * ldo;
    const __half* xr = xp + m0 * ldx;
    int rc;
    if (mc <= 8) rc = launch_gemm<1>(xr, ldx, wq_t, sz_t, mc, (int)N, (int)K, (int)group_size, e, workspace, st);
    else if (mc <= 16) rc = launch_gemm<2>(xr, ldx, wq_t, sz_t, mc, (int)N, (int)K, (int)group_size, e, workspace, st);
    else rc = launch_gemm<4>(xr, ldx, wq_t, sz_t, mc, (int)N, (int)K, (int)group_size, e, workspace, st);
    if (rc) return rc;
  }
  return LLMQRT_OK;
}

}  // extern "C"
