// Prefill attention over the new tokens: O = softmax(mask(Q K^T / sqrt(d))) V, causal, GQA.
//
// Flash-attention style single pass: a block owns 64 query rows of one head (16 per warp), walks
// the keys in tiles of 64 that are double-buffered in shared memory with cp.async, keeps S, P and
// O in registers and never writes the score matrix.  Shared-memory rows are XOR-swizzled in
// 16-byte chunks so that cp.async stores and ldmatrix loads are conflict free.  Query tiles are
// issued heaviest first (causal tiles near the end of the sequence see the most keys).
#include "common.cuh"

namespace llmqrt {
namespace {

// 4 warps x 16 query rows, key tiles of 64 (128 rows with 8 warps was measured 30 % slower: one
// block per SM instead of three)
constexpr int kBM = 64, kBN = 64, kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;                      // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// byte offset of 16-byte chunk `c` of row `r` in a [rows][D] 16-bit tile
template <int D> __device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)(r * D * 2 + ((c ^ (r & 7)) << 4)); }

template <int D, int ROWS>
__device__ __forceinline__ void load_tile(uint32_t dst_base, const uint16_t* src, int64_t row_stride, int row0,
                                          int rows_total) {
  constexpr int CH = D / 8;                            // chunks per row
  static_assert(ROWS * CH % kThreads == 0, "tile does not divide among the threads");
#pragma unroll
  for (int i = 0; i < ROWS * CH / kThreads; ++i) {
    const int id = i * kThreads + threadIdx.x;
    const int r = id / CH, c = id % CH;
    const bool valid = row0 + r < rows_total;
    const uint16_t* p = src + (int64_t)(valid ? row0 + r : 0) * row_stride + c * 8;
    cp_async_16(dst_base + swz<D>(r, c), p, valid);
  }
}

template <bool BF16, int D>
__global__ void __launch_bounds__(kThreads)
attn_prefill_kernel(const uint16_t* __restrict__ q, int64_t q_ts, const uint16_t* __restrict__ k,
                    const uint16_t* __restrict__ v, int64_t kv_ts, uint16_t* __restrict__ out, int64_t out_ts, int S,
                    int Hq, int Hkv, int causal, float scale, float softcap) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int kTileBytes = kBN * D * 2;
  const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t sK = sQ + kBM * D * 2, sV = sK + 2 * kTileBytes;

  const int qt = gridDim.x - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (Hq / Hkv);
  const int q0 = qt * kBM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

  const uint16_t* qb = q + (int64_t)b * S * q_ts + (int64_t)hq * D;
  const uint16_t* kb = k + (int64_t)b * S * kv_ts + (int64_t)hkv * D;
  const uint16_t* vb = v + (int64_t)b * S * kv_ts + (int64_t)hkv * D;

  const int n_tiles = causal ? min((q0 + kBM + kBN - 1) / kBN, (S + kBN - 1) / kBN) : (S + kBN - 1) / kBN;

  load_tile<D, kBM>(sQ, qb, q_ts, q0, S);
  load_tile<D, kBN>(sK, kb, kv_ts, 0, S);
  load_tile<D, kBN>(sV, vb, kv_ts, 0, S);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float sl2 = scale * kLog2e;

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) {                           // prefetch the next K/V tile into the other buffer
      load_tile<D, kBN>(sK + (buf ^ 1) * kTileBytes, kb, kv_ts, (tile + 1) * kBN, S);
      load_tile<D, kBN>(sV + (buf ^ 1) * kTileBytes, vb, kv_ts, (tile + 1) * kBN, S);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    if (tile == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = 2 * ks + (lane >> 4);
        ldmatrix_x4(sQ + swz<D>(r, c), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
      }
    }

    // A key tile entirely above this warp's 16 rows is masked out completely: nothing to compute
    // (the barriers below are still reached by every warp).
    const bool skip = causal && tile * kBN > q0 + warp * 16 + 15;
    if (!skip) {
    // ---- S = Q K^T (16 x 64 per warp) ----
    float s[kBN / 8][4];
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb) {
#pragma unroll
      for (int c = 0; c < 4; ++c) s[nb][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(sK + buf * kTileBytes + swz<D>(nb * 8 + (lane & 7), 2 * ks + (lane >> 3)), b0, b1, b2, b3);
        mma_16816<BF16>(s[nb], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
        mma_16816<BF16>(s[nb], qf[ks + 1][0], qf[ks + 1][1], qf[ks + 1][2], qf[ks + 1][3], b2, b3);
      }
    }

    // ---- scale, mask, online softmax (rows g and g+8 of this warp's 16) ----
    const int key_base = tile * kBN;
    const bool need_mask = (key_base + kBN > S) || (causal && key_base + kBN > q0 + warp * 16);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float x = s[nb][c];
        if (softcap != 0.f) x = softcap * tanhf(x * scale / softcap) * kLog2e;
        else x *= sl2;
        if (need_mask) {
          const int key = key_base + nb * 8 + 2 * t + (c & 1);
          const int row = q0 + warp * 16 + g + 8 * (c >> 1);
          if (key >= S || (causal && key > row)) x = -INFINITY;
        }
        s[nb][c] = x;
        mx[c >> 1] = fmaxf(mx[c >> 1], x);
      }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      // a fully masked row keeps m = -inf; use 0 as the reference point so that exp2 yields 0, not NaN
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f(m_run[r] - m_safe);
      m_run[r] = m_new;
      mx[r] = m_safe;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < kBN / 8; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(s[nb][c] - mx[c >> 1]);
        s[nb][c] = p;
        psum[c >> 1] += p;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + psum[r];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      const uint32_t a0 = pack2<BF16>(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a1 = pack2<BF16>(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack2<BF16>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t a3 = pack2<BF16>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int db = 0; db < D / 8; db += 2) {
        uint32_t b0, b1, b2, b3;
        const int r = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = db + (lane >> 4);
        ldmatrix_x4_trans(sV + buf * kTileBytes + swz<D>(r, c), b0, b1, b2, b3);
        mma_16816<BF16>(o[db], a0, a1, a2, a3, b0, b1);
        mma_16816<BF16>(o[db + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    }
    __syncthreads();                                    // everyone is done with `buf` before it is refilled
  }

  // ---- normalise and store ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = q0 + warp * 16 + g + 8 * r;
    if (row >= S) continue;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    uint32_t* dst = reinterpret_cast<uint32_t*>(out + ((int64_t)b * S + row) * out_ts + (int64_t)hq * D);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) dst[i * 4 + t] = pack2<BF16>(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
  }
}

}  // namespace
}  // namespace llmqrt

using namespace llmqrt;

extern "C" int llmqrt_attn_prefill(const void* q, int64_t q_token_stride, const void* k, const void* v,
                                   int64_t kv_token_stride, void* out, int64_t out_token_stride, int dtype, int64_t B,
                                   int64_t S, int64_t Hq, int64_t Hkv, int64_t d, int causal, float softcap,
                                   llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "attn_prefill: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(d == 64 || d == 128, "attn_prefill: head_dim must be 64 or 128 (got %lld)", (long long)d);
  LLMQRT_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && Hq < 65536 && B < 65536 && B >= 0 && S >= 0 && S < (1 << 30),
                 "attn_prefill: bad shape");
  LLMQRT_REQUIRE(q_token_stride % 8 == 0 && kv_token_stride % 8 == 0 && out_token_stride % 2 == 0,
                 "attn_prefill: token strides must be multiples of 8 elements");
  if (B == 0 || S == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(q && k && v && out, "attn_prefill: null pointer");
  LLMQRT_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out) & 3) == 0, "attn_prefill: pointers must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid((unsigned)ceil_div(S, kBM), (unsigned)Hq, (unsigned)B);
  const float scale = 1.0f / sqrtf((float)d);
  const int smem = (kBM + 4 * kBN) * (int)d * 2;
#define LLMQRT_RUN(BF, DD)                                                                                         \
  do {                                                                                                             \
    auto kern = attn_prefill_kernel<BF, DD>;                                                                       \
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;                \
    kern<<<grid, kThreads, smem, st>>>(reinterpret_cast<const uint16_t*>(q), q_token_stride,                       \
                                       reinterpret_cast<const uint16_t*>(k), reinterpret_cast<const uint16_t*>(v), \
                                       kv_token_stride, reinterpret_cast<uint16_t*>(out), out_token_stride, (int)S, \
                                       (int)Hq, (int)Hkv, causal, scale, softcap);                                  \
  } while (0)
  const bool bf = dtype == LLMQRT_BF16;
  if (d == 128) { if (bf) LLMQRT_RUN(true, 128); else LLMQRT_RUN(false, 128); }
  else { if (bf) LLMQRT_RUN(true, 64); else LLMQRT_RUN(false, 64); }
#undef LLMQRT_RUN
  return check_launch("attn_prefill");
}
