// Block glue of the decode step: RMSNorm (+ residual add, + int8 quantization), rotary embedding
// fused with the KV-cache write, SiLU(gate) * up (+ int8 quantization).  Each kernel replaces a
// chain of small torch ops and keeps their rounding points (fp32 math, one rounding to the 16-bit
// activation type after every op of the chain).
//
// The row kernels (RMSNorm, SiLU*up) are HBM/L2-bound.  A token row is handled by a thread-block
// cluster of 1, 2, 4 or 8 CTAs, each owning a contiguous slice of the row; the row-wide reductions
// (sum of squares, absmax) are exchanged through distributed shared memory.  With the 64 rows of a
// decode step this spreads the work over every SM instead of 64 of them.  128-bit accesses whenever
// the slice is 16-byte aligned; the computed slice stays in shared memory for the quantization pass.
#include <cooperative_groups.h>
#include <cstdlib>

#include "common.cuh"
#include "peer_comm.cuh"

namespace cg = cooperative_groups;

namespace llmqrt {
namespace {

constexpr int kThreads = 256;

template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v) {
  __shared__ float red[kThreads / 32];
  __shared__ float result;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();                                  // protects `red` / `result` between successive calls
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < kThreads / 32 ? red[threadIdx.x] : 0.f;
    w = IS_MAX ? warp_max(w) : warp_sum(w);
    if (threadIdx.x == 0) result = w;
  }
  __syncthreads();
  return result;
}

// Combines the per-CTA values of a cluster in rank order (same result in every CTA).  `slot` is a
// shared-memory word of this CTA that the other CTAs of the cluster read remotely.
template <bool IS_MAX>
__device__ __forceinline__ float cluster_reduce(float block_val, float* slot, int cluster_size) {
  if (cluster_size == 1) return block_val;
  cg::cluster_group cluster = cg::this_cluster();
  if (threadIdx.x == 0) *slot = block_val;
  cluster.sync();
  float r = 0.f;
  for (int c = 0; c < cluster_size; ++c) {
    const float v = *cluster.map_shared_rank(slot, c);
    r = IS_MAX ? fmaxf(r, v) : r + v;
  }
  return r;
}

template <typename T, int U> struct Pack { T v[U]; };

template <typename T, bool VEC>
__device__ __forceinline__ void load_unit(const T* p, int64_t unit, T (&out)[VEC ? 8 : 1]) {
  if constexpr (VEC) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p + unit * 8);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = e[j];
  } else {
    out[0] = p[unit];
  }
}
template <typename T, bool VEC>
__device__ __forceinline__ void store_unit(T* p, int64_t unit, const T (&in)[VEC ? 8 : 1]) {
  if constexpr (VEC) {
    *reinterpret_cast<uint4*>(p + unit * 8) = *reinterpret_cast<const uint4*>(in);
  } else {
    p[unit] = in[0];
  }
}

// Per-token int8 quantization of a row slice already rounded to T and held in shared memory; same
// arithmetic as the stand-alone quantizer (scale = T(T(max(absmax,1e-5)) * (1/127)), q = rint(T(x/scale))).
template <typename T, bool VEC>
__device__ __forceinline__ void quantize_slice_int8(const T* __restrict__ row_s, int64_t units, float amax,
                                                    int8_t* __restrict__ q, float* __restrict__ scale_out) {
  constexpr int U = VEC ? 8 : 1;
  float s = round_to<T>(fmaxf(amax, 1e-5f));
  s = round_to<T>(__fmul_rn(s, 1.0f / 127.0f));
  if (scale_out && threadIdx.x == 0) *scale_out = s;
  for (int64_t u = threadIdx.x; u < units; u += blockDim.x) {
    T e[U];
    load_unit<T, VEC>(row_s, u, e);
    __align__(8) int8_t o[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      float v = rintf(round_to<T>(__fdiv_rn(to_f32<T>(e[j]), s)));
      v = v != v ? v : fminf(fmaxf(v, -128.f), 127.f);
      o[j] = (int8_t)(int)v;
    }
    if constexpr (VEC) *reinterpret_cast<uint2*>(q + u * 8) = *reinterpret_cast<const uint2*>(o);
    else q[u] = o[0];
  }
}

// grid = (cluster_size, M): blockIdx.x = rank in the row's cluster, blockIdx.y = row.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual, T* __restrict__ x_out,
               const T* __restrict__ weight, float eps, T* __restrict__ y, int8_t* __restrict__ q,
               float* __restrict__ scale_f32, int64_t H, int64_t slice) {
  constexpr int U = VEC ? 8 : 1;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float slot_ss, slot_amax;
  pdl_wait_then_trigger();
  T* row = reinterpret_cast<T*>(smem);
  const int cl = gridDim.x, rank = blockIdx.x;
  const int64_t m = blockIdx.y, c0 = (int64_t)rank * slice;
  const int64_t len = max((int64_t)0, min(slice, H - c0)), units = len / U;
  const int64_t off = m * H + c0;
  float ss = 0.f;
  for (int64_t u = threadIdx.x; u < units; u += blockDim.x) {
    T e[U], r[U];
    load_unit<T, VEC>(x + off, u, e);
    if (residual) load_unit<T, VEC>(residual + off, u, r);
#pragma unroll
    for (int j = 0; j < U; ++j) {
      float v = to_f32<T>(e[j]);
      if (residual) v = round_to<T>(v + to_f32<T>(r[j]));                 // h = x + r in T
      e[j] = from_f32<T>(v);
      ss += v * v;
    }
    if (x_out) store_unit<T, VEC>(x_out + off, u, e);
    store_unit<T, VEC>(row, u, e);
  }
  ss = cluster_reduce<false>(block_reduce<false>(ss), &slot_ss, cl);
  const float inv = rsqrtf(ss / (float)H + eps);
  float amax = 0.f;
  for (int64_t u = threadIdx.x; u < units; u += blockDim.x) {
    T e[U], w[U];
    load_unit<T, VEC>(row, u, e);
    load_unit<T, VEC>(weight + c0, u, w);
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const float n = round_to<T>(to_f32<T>(e[j]) * inv);                 // (x32 * inv).to(T)
      const float o = round_to<T>(to_f32<T>(w[j]) * n);                   // weight * that, in T
      e[j] = from_f32<T>(o);
      amax = fmaxf(amax, fabsf(o));
    }
    if (y) store_unit<T, VEC>(y + off, u, e);
    store_unit<T, VEC>(row, u, e);
  }
  if (q) {
    amax = cluster_reduce<true>(block_reduce<true>(amax), &slot_amax, cl);
    __syncthreads();
    quantize_slice_int8<T, VEC>(row, units, amax, q + off, rank == 0 ? scale_f32 + m : nullptr);
  }
  if (cl > 1) cg::this_cluster().sync();             // nobody leaves while its slots may still be read
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
silu_mul_kernel(const T* __restrict__ gate_up, int64_t ld, T* __restrict__ y, int8_t* __restrict__ q,
                float* __restrict__ scale_f32, int64_t I, int64_t slice) {
  constexpr int U = VEC ? 8 : 1;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float slot_amax;
  pdl_wait_then_trigger();
  T* row = reinterpret_cast<T*>(smem);
  const int cl = gridDim.x, rank = blockIdx.x;
  const int64_t m = blockIdx.y, c0 = (int64_t)rank * slice;
  const int64_t len = max((int64_t)0, min(slice, I - c0)), units = len / U;
  const T* gr = gate_up + m * ld + c0;
  const T* ur = gr + I;
  float amax = 0.f;
  for (int64_t u = threadIdx.x; u < units; u += blockDim.x) {
    T g[U], up[U];
    load_unit<T, VEC>(gr, u, g);
    load_unit<T, VEC>(ur, u, up);
#pragma unroll
    for (int j = 0; j < U; ++j) {
      const float gv = to_f32<T>(g[j]);
      const float act = round_to<T>(gv / (1.0f + expf(-gv)));             // silu in T
      const float h = round_to<T>(act * to_f32<T>(up[j]));                // * up, in T
      g[j] = from_f32<T>(h);
      amax = fmaxf(amax, fabsf(h));
    }
    if (y) store_unit<T, VEC>(y + m * I + c0, u, g);
    if (q) store_unit<T, VEC>(row, u, g);
  }
  if (q) {
    amax = cluster_reduce<true>(block_reduce<true>(amax), &slot_amax, cl);
    __syncthreads();
    quantize_slice_int8<T, VEC>(row, units, amax, q + m * I + c0, rank == 0 ? scale_f32 + m : nullptr);
  }
  if (cl > 1) cg::this_cluster().sync();
}

// Block-wide reduction for a block of any whole number of warps (up to 32).
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce_any(float v) {
  __shared__ float red[32];
  __shared__ float result;
  const int nwarps = blockDim.x >> 5;
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = (int)threadIdx.x < nwarps ? red[threadIdx.x] : 0.f;
    w = IS_MAX ? warp_max(w) : warp_sum(w);
    if (threadIdx.x == 0) result = w;
  }
  __syncthreads();
  return result;
}

// SiLU(gate) * up with the row split over the CTAs of a cluster (possibly of one) and U units of eight
// elements per thread held in registers from the load to the quantized store; the row absmax is
// reduced in the block and then across the cluster through distributed shared memory.
// grid = (cluster_size, M), blockDim.x * 8 * U >= slice; unit k of a thread is unit threadIdx.x + k * blockDim.x.
template <typename T, int U>
__global__ void __launch_bounds__(1024)
silu_mul_regs_kernel(const T* __restrict__ gate_up, int64_t ld, T* __restrict__ y, int8_t* __restrict__ q,
                     float* __restrict__ scale_f32, int64_t I, int64_t slice) {
  __shared__ float slot_amax[8];                       // slot r: the maximum found by the cluster's CTA r
  pdl_wait_then_trigger();
  const int cl = gridDim.x, rank = blockIdx.x;
  const int64_t m = blockIdx.y, c0 = (int64_t)rank * slice;
  float f[U][8];
  float amax = 0.f;
  const T* gr = gate_up + m * ld + c0;
  T g[U][8], up[U][8];
#pragma unroll
  for (int k = 0; k < U; ++k) {                        // all loads first: U independent pairs in flight
    const int64_t u = threadIdx.x + (int64_t)k * blockDim.x;
    if (u * 8 < slice) {
      load_unit<T, true>(gr, u, g[k]);
      load_unit<T, true>(gr + I, u, up[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < U; ++k) {
    const int64_t u = threadIdx.x + (int64_t)k * blockDim.x;
    if (u * 8 < slice) {
      T h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gv = to_f32<T>(g[k][j]);
        const float act = round_to<T>(gv / (1.0f + expf(-gv)));             // silu in T
        f[k][j] = round_to<T>(act * to_f32<T>(up[k][j]));                   // * up, in T
        h[j] = from_f32<T>(f[k][j]);
        amax = fmaxf(amax, fabsf(f[k][j]));
      }
      if (y) store_unit<T, true>(y + m * I + c0, u, h);
    }
  }
  if (q) {
    amax = block_reduce_any<true>(amax);
    if (cl > 1) {
      // every CTA stores its maximum into its slot in EVERY CTA of the cluster, then ONE cluster barrier
      // (release / acquire) and each CTA reads its own copy: nobody reads remote memory afterwards, so
      // there is no second barrier before leaving
      if (threadIdx.x < cl) {
        uint32_t remote;
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(&slot_amax[rank]);
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)threadIdx.x));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(amax) : "memory");
      }
      asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
      amax = 0.f;
      for (int c = 0; c < cl; ++c) amax = fmaxf(amax, slot_amax[c]);
    }
    float s = round_to<T>(fmaxf(amax, 1e-5f));
    s = round_to<T>(__fmul_rn(s, 1.0f / 127.0f));
    if (rank == 0 && threadIdx.x == 0) scale_f32[m] = s;
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int64_t u = threadIdx.x + (int64_t)k * blockDim.x;
      if (u * 8 < slice) {
        __align__(8) int8_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float v = rintf(round_to<T>(__fdiv_rn(f[k][j], s)));
          v = v != v ? v : fminf(fmaxf(v, -128.f), 127.f);
          o[j] = (int8_t)(int)v;
        }
        *reinterpret_cast<uint2*>(q + m * I + c0 + u * 8) = *reinterpret_cast<const uint2*>(o);
      }
    }
  }
}

// RMSNorm of one row held in registers, eight elements per thread (rows of up to 8192 elements, one
// block per row): `h` are the row's values already rounded to T (x, or x + residual), `on` says
// whether this thread owns a unit.  Two block reductions, no staging; optional quantized store.
template <typename T>
__device__ __forceinline__ void rmsnorm_regs_finish(bool on, float (&f)[8], int64_t m, int64_t u, int64_t H,
                                                    const T* __restrict__ weight, float eps, T* __restrict__ y,
                                                    int8_t* __restrict__ q, float* __restrict__ scale_f32) {
  const int64_t off = m * H;
  T e[8], w[8];
  float ss = 0.f;
  if (on) {
    load_unit<T, true>(weight, u, w);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_reduce_any<false>(ss);
  const float inv = rsqrtf(ss / (float)H + eps);
  float amax = 0.f;
  if (on) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float n = round_to<T>(f[j] * inv);                            // (x32 * inv).to(T)
      f[j] = round_to<T>(to_f32<T>(w[j]) * n);                            // weight * that, in T
      e[j] = from_f32<T>(f[j]);
      amax = fmaxf(amax, fabsf(f[j]));
    }
    if (y) store_unit<T, true>(y + off, u, e);
  }
  if (q) {
    amax = block_reduce_any<true>(amax);
    float s = round_to<T>(fmaxf(amax, 1e-5f));
    s = round_to<T>(__fmul_rn(s, 1.0f / 127.0f));
    if (threadIdx.x == 0) scale_f32[m] = s;
    if (on) {
      __align__(8) int8_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = rintf(round_to<T>(__fdiv_rn(f[j], s)));
        v = v != v ? v : fminf(fmaxf(v, -128.f), 127.f);
        o[j] = (int8_t)(int)v;
      }
      *reinterpret_cast<uint2*>(q + off + u * 8) = *reinterpret_cast<const uint2*>(o);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
rmsnorm_regs_kernel(const T* __restrict__ x, const T* __restrict__ residual, T* __restrict__ x_out,
                    const T* __restrict__ weight, float eps, T* __restrict__ y, int8_t* __restrict__ q,
                    float* __restrict__ scale_f32, int64_t H) {
  pdl_wait_then_trigger();
  const int64_t m = blockIdx.x, u = threadIdx.x;
  const bool on = u * 8 < H;
  const int64_t off = m * H;
  float f[8];
  if (on) {
    T e[8], r[8];
    load_unit<T, true>(x + off, u, e);
    if (residual) load_unit<T, true>(residual + off, u, r);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = to_f32<T>(e[j]);
      if (residual) v = round_to<T>(v + to_f32<T>(r[j]));                 // h = x + r in T
      e[j] = from_f32<T>(v);
      f[j] = v;
    }
    if (x_out) store_unit<T, true>(x_out + off, u, e);
  }
  rmsnorm_regs_finish<T>(on, f, m, u, H, weight, eps, y, q, scale_f32);
}

// The same, with the residual arriving as tensor-parallel partial sums: every rank pushes its row of
// `partial` to all ranks through the peer-mapped buffers, gathers the W copies, adds them in rank
// order in fp32 and rounds to T -- exactly the stand-alone all-reduce -- and goes on with
// h = x + that sum.  One kernel instead of all-reduce + RMSNorm.
// partial == nullptr: the GEMM that produced the partial sums has already pushed them from its
// epilogue (llmqrt_comm_int8_linear_per_channel), this kernel only gathers.
// MAXT bounds the block size (512 leaves 128 registers per thread: the gathered copies of eight
// ranks stay in registers).  NS >= the number of ranks (2, 4 or 8) sizes the register array of the
// gathered copies: with it fixed at 8 the kernel needed 122 registers per thread at any world size, and
// a 448-thread block then fills the register file so that no block of the GEMM that follows (or
// precedes) it in the decode chain can be resident on the same SM.
template <typename T, int MAXT, int NS>
__global__ void __launch_bounds__(MAXT)
allreduce_rmsnorm_kernel(CommDev c, const T* __restrict__ partial, const T* __restrict__ x, T* __restrict__ x_out,
                         const T* __restrict__ weight, float eps, T* __restrict__ y, int8_t* __restrict__ q,
                         float* __restrict__ scale_f32, int64_t H, int two_step) {
  pdl_wait_then_trigger();
  __shared__ unsigned s_seq;
  __shared__ int s_ok;
  const int64_t m = blockIdx.x, u = threadIdx.x;
  const bool on = u * 8 < H;
  const int64_t off = m * H;
  // Everything that does not depend on the peers is requested first: this rank's partial row, the
  // residual row and (thread 0) the call's sequence number travel to L2 at the same time.
  uint4 pv = make_uint4(0u, 0u, 0u, 0u);
  T e[8];
  const bool pushed = partial == nullptr;
  if (on) {
    if (!pushed) pv = *reinterpret_cast<const uint4*>(partial + off + u * 8);
    load_unit<T, true>(x + off, u, e);
  }
  if (threadIdx.x == 0) {
    unsigned sq;
    s_ok = comm_enter(c, &sq) ? 1 : 0;
    s_seq = sq;
  }
  __syncthreads();
  const unsigned seq = s_seq;
  const bool live = s_ok != 0;                         // false: the status is raised, the sum is skipped
  float f[8];
  if (on) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (live) {
      // Word placement (any bijection works, as every rank uses the same one): the two words of a
      // thread sit 32 words apart so that each store or poll of a warp covers 512 contiguous bytes.
      const long long words[2] = {comm_word0(m, u, (int)blockDim.x), comm_word0(m, u, (int)blockDim.x) + 32};
      // One step: every rank sends its row to every rank and all add the W copies themselves (W x the
      // payload leaves each rank).  Two steps, for many ranks: a row goes only to the rank that owns
      // it (rows are dealt out in equal runs), the owner adds the copies and sends the finished row,
      // rounded to T, to everyone (2 x the payload leaves each rank, one more hop of latency).
      const int rows_per_rank = ((int)gridDim.x + c.world - 1) / c.world;
      const int owner = two_step ? min((int)(m / rows_per_rank), c.world - 1) : c.rank;
      if (pushed) {
        // the GEMM's epilogue has sent this rank's rows (to everyone, or to their owners)
      } else if (two_step) {
        comm_push_one(c, seq, owner, c.rank, words[0], make_uint2(pv.x, pv.y));
        comm_push_one(c, seq, owner, c.rank, words[1], make_uint2(pv.z, pv.w));
      } else {
        comm_push(c, seq, words[0], make_uint2(pv.x, pv.y));
        comm_push(c, seq, words[1], make_uint2(pv.z, pv.w));
      }
      const unsigned long long t0 = comm_timer_ns();
      bool ok = true;
      if (owner == c.rank) {
        // at most four sources per round of polls: eight at once need 64 registers for the copies alone
        constexpr int NB = NS > 4 ? 4 : NS;
#pragma unroll 1
        for (int s0 = 0; s0 < c.world && ok; s0 += NB) {
          uint4 d[NB][2];
          ok = comm_gather_all<NB, 2>(c, seq, s0, min(NB, c.world - s0), words, t0, d);
          if (ok) {
#pragma unroll
            for (int s = 0; s < NB; ++s) {             // rank order: the same bits on every rank
              if (s0 + s < c.world) {
                const uint2 p0 = make_uint2(d[s][0].x, d[s][0].z), p1 = make_uint2(d[s][1].x, d[s][1].z);
                const T* e0 = reinterpret_cast<const T*>(&p0);
                const T* e1 = reinterpret_cast<const T*>(&p1);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  acc[j] += to_f32<T>(e0[j]);
                  acc[4 + j] += to_f32<T>(e1[j]);
                }
              }
            }
          }
        }
      }
      if (two_step) {
        if (owner == c.rank && ok) {
          __align__(16) T red[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) red[j] = from_f32<T>(acc[j]);
          const uint4 rv = *reinterpret_cast<const uint4*>(red);
          for (int p = 0; p < c.world; ++p) {
            comm_push_one(c, seq, p, kCommMaxWorld, words[0], make_uint2(rv.x, rv.y));
            comm_push_one(c, seq, p, kCommMaxWorld, words[1], make_uint2(rv.z, rv.w));
          }
        }
        uint4 d[1][2];
        ok = ok && comm_gather_all<1, 2>(c, seq, kCommMaxWorld, 1, words, t0, d);
        const uint2 p0 = make_uint2(d[0][0].x, d[0][0].z), p1 = make_uint2(d[0][1].x, d[0][1].z);
        const T* e0 = reinterpret_cast<const T*>(&p0);
        const T* e1 = reinterpret_cast<const T*>(&p1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[j] = ok ? to_f32<T>(e0[j]) : 0.f;
          acc[4 + j] = ok ? to_f32<T>(e1[j]) : 0.f;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float r = round_to<T>(acc[j]);                                // the all-reduced value, in T
      const float v = round_to<T>(to_f32<T>(e[j]) + r);                   // h = x + r in T
      e[j] = from_f32<T>(v);
      f[j] = v;
    }
    if (x_out) store_unit<T, true>(x_out + off, u, e);
  }
  rmsnorm_regs_finish<T>(on, f, m, u, H, weight, eps, y, q, scale_f32);
  if (threadIdx.x == 0) comm_leave(c, seq);            // after the barriers above: every thread is done with seq
}

// Cluster size for a row kernel: as many CTAs per row as needed to put about two CTAs on every SM,
// limited to 8 and to slices that stay 16-byte aligned.
int pick_cluster(int64_t M, int64_t row_len) {
  int cl = 1;
  while (cl < 8 && M * cl < 2 * sm_count() && row_len % (cl * 2 * 8) == 0 && row_len / (cl * 2) >= 256) cl *= 2;
  return cl;
}

template <typename Kern, typename... Args>
int launch_row_kernel(Kern kern, int cl, int64_t M, size_t smem, cudaStream_t st, Args... args) {
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), (int)smem)) return rc;
  return launch_chained(kern, dim3((unsigned)cl, (unsigned)M, 1), dim3(kThreads, 1, 1), smem, st, cl, args...);
}

// One block per (token, head); thread i rotates the pair (i, i + d/2).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ q, int64_t q_token_stride, T* __restrict__ k,
                                     const T* __restrict__ v, int64_t kv_token_stride, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int64_t cache_batch_stride, int64_t cache_row_stride,
                                     int pos0, const int32_t* __restrict__ pos_dev, const float* __restrict__ cos_tab,
                                     const float* __restrict__ sin_tab, int table_rows, int S, int Hq, int Hkv, int d) {
  pdl_wait();
  pdl_trigger();
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

inline bool aligned16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace llmqrt

namespace llmqrt {
// two steps from 8 ranks on (or when LLMQRT_ALLREDUCE_TWO_STEP=1 asks for it, e.g. to test on fewer)
int comm_two_step(int world) {
  static const bool force_two_step = [] {
    const char* v = getenv("LLMQRT_ALLREDUCE_TWO_STEP");
    return v != nullptr && v[0] == '1';
  }();
  return (world >= 8 || force_two_step) ? 1 : 0;
}
}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_rmsnorm(const void* x, const void* residual, void* x_out, const void* weight, float eps, void* y,
                   int8_t* q, float* scale_f32, int dtype, int64_t M, int64_t H, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "rmsnorm: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(M >= 0 && H > 0 && M < 65536ll * 32768 && H * 2 <= 200 * 1024, "rmsnorm: bad shape");
  if (M == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(x && weight && (y || q), "rmsnorm: null pointer");
  LLMQRT_REQUIRE(!q || scale_f32, "rmsnorm: quantized output needs scale_f32");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = H % 8 == 0 && aligned16(x) && aligned16(residual) && aligned16(x_out) && aligned16(weight) &&
                   aligned16(y) && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
  if (vec && H <= 8192 && M <= 0x7fffffffll) {
    // the row fits the registers of one block: one block per row, rows on gridDim.x
    const unsigned threads = (unsigned)(((H / 8) + 31) / 32 * 32);
    int rc;
#define LLMQRT_RUN(T)                                                                                             \
  rc = launch_chained(rmsnorm_regs_kernel<T>, dim3((unsigned)M, 1, 1), dim3(threads, 1, 1), 0, st, 1,               \
                      reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(residual),                          \
                      reinterpret_cast<T*>(x_out), reinterpret_cast<const T*>(weight), eps, reinterpret_cast<T*>(y), \
                      q, scale_f32, H)
    if (dtype == LLMQRT_F16) LLMQRT_RUN(__half); else LLMQRT_RUN(__nv_bfloat16);
#undef LLMQRT_RUN
    if (rc) return rc;
    return check_launch("rmsnorm");
  }
  // gridDim.y carries the row: rows beyond 65535 are launched in panels
  const int cl = vec ? pick_cluster(M, H) : 1;
  const int64_t slice = H / cl;
  const size_t smem = (size_t)slice * 2;
  for (int64_t m0 = 0; m0 < M; m0 += 65535) {
    const int64_t mc = (M - m0 < 65535) ? (M - m0) : 65535;
    const int64_t o = m0 * H;
    int rc;
#define LLMQRT_RUN(T, V)                                                                                          \
  rc = launch_row_kernel(rmsnorm_kernel<T, V>, cl, mc, smem, st, reinterpret_cast<const T*>(x) + o,                \
                         residual ? reinterpret_cast<const T*>(residual) + o : (const T*)nullptr,                  \
                         x_out ? reinterpret_cast<T*>(x_out) + o : (T*)nullptr, reinterpret_cast<const T*>(weight), \
                         eps, y ? reinterpret_cast<T*>(y) + o : (T*)nullptr, q ? q + o : (int8_t*)nullptr,          \
                         scale_f32 ? scale_f32 + m0 : (float*)nullptr, H, slice)
    if (dtype == LLMQRT_F16) { if (vec) LLMQRT_RUN(__half, true); else LLMQRT_RUN(__half, false); }
    else { if (vec) LLMQRT_RUN(__nv_bfloat16, true); else LLMQRT_RUN(__nv_bfloat16, false); }
#undef LLMQRT_RUN
    if (rc) return rc;
    if (int rc2 = check_launch("rmsnorm")) return rc2;
  }
  return LLMQRT_OK;
}

int llmqrt_comm_allreduce_rmsnorm(void* comm, const void* partial, const void* x, void* x_out, const void* weight,
                                  float eps, void* y, int8_t* q, float* scale_f32, int dtype, int64_t M, int64_t H,
                                  llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(comm != nullptr, "comm_allreduce_rmsnorm: null communicator");
  Comm* c = static_cast<Comm*>(comm);
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "comm_allreduce_rmsnorm: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(M >= 0 && M <= 0x7fffffffll && H > 0 && H % 8 == 0 && H <= 8192, "comm_allreduce_rmsnorm: need H %% 8 == 0 and H <= 8192");
  LLMQRT_REQUIRE(M * (((H / 8) + 31) / 32 * 32) * 32 <= c->dev.slot_bytes, "comm_allreduce_rmsnorm: M * H exceeds the communicator's capacity");
  if (M == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(x && weight && (y || q), "comm_allreduce_rmsnorm: null pointer");   // partial may be null: already pushed
  LLMQRT_REQUIRE(!q || scale_f32, "comm_allreduce_rmsnorm: quantized output needs scale_f32");
  LLMQRT_REQUIRE(aligned16(partial) && aligned16(x) && aligned16(x_out) && aligned16(weight) && aligned16(y) &&
                 (reinterpret_cast<uintptr_t>(q) & 7) == 0, "comm_allreduce_rmsnorm: pointers must be 16-byte aligned (q: 8)");
  for (int p = 0; p < c->dev.world; ++p)
    LLMQRT_REQUIRE(c->dev.base[p] != nullptr, "comm_allreduce_rmsnorm: peer %d has not been opened", p);
  const unsigned threads = (unsigned)comm_row_threads(H);
  const int two_step = comm_two_step(c->dev.world);
  int rc;
#define LLMQRT_RUN_NS(T, MAXT, NS)                                                                                 \
  rc = launch_chained(allreduce_rmsnorm_kernel<T, MAXT, NS>, dim3((unsigned)M, 1, 1), dim3(threads, 1, 1), 0,        \
                      (cudaStream_t)stream, 1, c->dev, reinterpret_cast<const T*>(partial),                          \
                      reinterpret_cast<const T*>(x), reinterpret_cast<T*>(x_out), reinterpret_cast<const T*>(weight), \
                      eps, reinterpret_cast<T*>(y), q, scale_f32, H, two_step)
#define LLMQRT_RUN(T, MAXT)                                       \
  do {                                                            \
    if (c->dev.world <= 2) LLMQRT_RUN_NS(T, MAXT, 2);             \
    else if (c->dev.world <= 4) LLMQRT_RUN_NS(T, MAXT, 4);        \
    else LLMQRT_RUN_NS(T, MAXT, 8);                               \
  } while (0)
  if (threads <= 512) { if (dtype == LLMQRT_F16) LLMQRT_RUN(__half, 512); else LLMQRT_RUN(__nv_bfloat16, 512); }
  else { if (dtype == LLMQRT_F16) LLMQRT_RUN(__half, 1024); else LLMQRT_RUN(__nv_bfloat16, 1024); }
#undef LLMQRT_RUN
#undef LLMQRT_RUN_NS
  if (rc) return rc;
  return check_launch("allreduce_rmsnorm");
}

int llmqrt_silu_mul(const void* gate_up, int64_t ld, void* y, int8_t* q, float* scale_f32, int dtype, int64_t M,
                    int64_t I, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "silu_mul: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(M >= 0 && I > 0 && ld >= 2 * I && M < 65536ll * 32768 && I * 2 <= 200 * 1024, "silu_mul: bad shape");
  if (M == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(gate_up && (y || q), "silu_mul: null pointer");
  LLMQRT_REQUIRE(!q || scale_f32, "silu_mul: quantized output needs scale_f32");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = I % 8 == 0 && ld % 8 == 0 && aligned16(gate_up) && aligned16(y) &&
                   (reinterpret_cast<uintptr_t>(q) & 7) == 0;
  // Register-resident variant: the smallest cluster whose slices fit one block (8 elements per
  // thread), widened while that still leaves every SM at most a few blocks and slices of >= 128 threads.
  // (Timed alone, fewer and larger blocks win -- 64 rows of 18944: two CTAs with two units per thread
  // 6.5 us against 8.5 us with four CTAs --, but inside the decode chain, where the launch and the
  // cluster set-up hide behind the preceding GEMM, the wider split is the faster one: 3.457 against
  // 3.486 ms per step.)
  int rcl = 0;
  const int upt = 1;
  if (vec && M <= 1024) {                            // (prefill-sized M: the staged kernel streams better)
    const int64_t units = I / 8;
    for (int c = 1; c <= 8; c *= 2)
      if (units % c == 0 && units / c <= 1024) { rcl = c; break; }
    while (rcl && rcl < 8 && units % (rcl * 2) == 0 && units / (rcl * 2) >= 128 && M * rcl * 2 <= 4 * sm_count()) rcl *= 2;
  }
  const int cl = rcl ? rcl : (vec ? pick_cluster(M, I) : 1);
  const int64_t slice = I / cl;
  const size_t smem = q ? (size_t)slice * 2 : 0;
  for (int64_t m0 = 0; m0 < M; m0 += 65535) {
    const int64_t mc = (M - m0 < 65535) ? (M - m0) : 65535;
    int rc;
    if (rcl) {
      const unsigned threads = (unsigned)(((slice / 8 + upt - 1) / upt + 31) / 32 * 32);
#define LLMQRT_RUN_REGS(T, U)                                                                                          \
  rc = launch_chained(silu_mul_regs_kernel<T, U>, dim3((unsigned)cl, (unsigned)mc, 1), dim3(threads, 1, 1), 0, st, cl, \
                      reinterpret_cast<const T*>(gate_up) + m0 * ld, ld,                                                \
                      y ? reinterpret_cast<T*>(y) + m0 * I : (T*)nullptr, q ? q + m0 * I : (int8_t*)nullptr,            \
                      scale_f32 ? scale_f32 + m0 : (float*)nullptr, I, slice)
#define LLMQRT_RUN_REGS_U(T)                                                                                           \
  switch (upt) {                                                                                                       \
    default: LLMQRT_RUN_REGS(T, 1); break;                                                                             \
  }
      if (dtype == LLMQRT_F16) { LLMQRT_RUN_REGS_U(__half); } else { LLMQRT_RUN_REGS_U(__nv_bfloat16); }
#undef LLMQRT_RUN_REGS_U
#undef LLMQRT_RUN_REGS
      if (rc) return rc;
      if (int rc2 = check_launch("silu_mul")) return rc2;
      continue;
    }
#define LLMQRT_RUN(T, V)                                                                                       \
  rc = launch_row_kernel(silu_mul_kernel<T, V>, cl, mc, smem, st, reinterpret_cast<const T*>(gate_up) + m0 * ld, ld, \
                         y ? reinterpret_cast<T*>(y) + m0 * I : (T*)nullptr, q ? q + m0 * I : (int8_t*)nullptr,   \
                         scale_f32 ? scale_f32 + m0 : (float*)nullptr, I, slice)
    if (dtype == LLMQRT_F16) { if (vec) LLMQRT_RUN(__half, true); else LLMQRT_RUN(__half, false); }
    else { if (vec) LLMQRT_RUN(__nv_bfloat16, true); else LLMQRT_RUN(__nv_bfloat16, false); }
#undef LLMQRT_RUN
    if (rc) return rc;
    if (int rc2 = check_launch("silu_mul")) return rc2;
  }
  return LLMQRT_OK;
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
  rc = launch_chained(rope_kv_write_kernel<T>, grid, dim3((unsigned)(d / 2)), 0, st, 1,                              \
      reinterpret_cast<T*>(q), q_token_stride, reinterpret_cast<T*>(k), reinterpret_cast<const T*>(v),              \
      kv_token_stride, reinterpret_cast<T*>(k_cache), reinterpret_cast<T*>(v_cache), cache_batch_stride,           \
      cache_row_stride, (int)pos0, pos_dev, cos_table, sin_table, (int)table_rows, (int)S, (int)Hq, (int)Hkv, (int)d)
  int rc;
  if (dtype == LLMQRT_F16) LLMQRT_RUN(__half); else LLMQRT_RUN(__nv_bfloat16);
#undef LLMQRT_RUN
  if (rc) return rc;
  return check_launch("rope_kv_write");
}

}  // extern "C"

