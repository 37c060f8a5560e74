// Decode attention over the contiguous GQA KV cache (one query token per sequence), split-KV.
//
// HBM-bound: every K and V row of every sequence is read exactly once, streamed by cp.async through
// a small per-warp ring in shared memory (three stages of 16 keys in flight per warp, no registers
// held), and consumed by warp-level MMAs whose 16-row operand is the group of query heads that share
// the KV head (GQA packing: up to 8 query heads per pass), so the arithmetic stays far below the
// memory time.  Fragments are plain 16-byte pieces of rows, no transposes:
//   S = Q K^T : the K fragment of lane (g, t) is 16 contiguous bytes of key row g; Q is pre-loaded
//               with the same head_dim permutation.
//   O += P V  : the V fragment needs two keys per register; two 16-byte loads (keys 2t, 2t+1) are
//               interleaved with one byte-permute per register.  The MMA's n index is mapped to
//               head_dim so that every load is a contiguous 128-byte row segment.
// Grid (splits, Hkv, B); each block walks `chunk` keys with 4 warps (16 keys per warp step), merges
// its warps through shared memory and writes either the final output (single split) or an
// unnormalised partial (max, sum, O) that a small combine kernel reduces; the combine kernel can also
// emit the per-token int8 quantization of the result, which is what an int8 output projection reads.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"

namespace llmqrt {
namespace {

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kRing = 3;            // cp.async stages per warp (2 measured slower: too few bytes in flight)

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds_16B(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
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

// Merges the split partials of sequence b (all heads) into `out` and, with out_q, quantizes the merged
// token row to int8 with a per-token scale -- the arithmetic of the stand-alone per-token quantizer
// applied to the 16-bit result.  Called by every thread of a block; `row_s` (shared, Hq * D 16-bit
// words, needed only with out_q) and `red` (shared, 32 floats) are scratch.
template <bool BF16, int D>
__device__ __forceinline__ void merge_sequence(int b, int n_splits, uint16_t* __restrict__ out, int Hq, int max_splits,
                                               const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                               int8_t* __restrict__ out_q, float* __restrict__ out_scale,
                                               uint16_t* row_s, float* red) {
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  const int units = Hq * D / 8;
  uint16_t* orow = out + (int64_t)b * Hq * D;
  float amax = 0.f;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    __align__(16) T e[8];
    if (n_splits <= 1) {
      *reinterpret_cast<uint4*>(e) = __ldcg(reinterpret_cast<const uint4*>(orow + u * 8));
    } else {
      const int hq = (u * 8) / D, dd = (u * 8) % D;
      const int64_t base = ((int64_t)b * Hq + hq) * max_splits;
      // one pass with a running maximum (splits in index order): the loads of successive splits do
      // not depend on one another, so several are in flight at a time
      float M = -INFINITY, lsum = 0.f, osum[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) osum[j] = 0.f;
#pragma unroll 4
      for (int s = 0; s < n_splits; ++s) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + (base + s) * 2));
        const float4 a = __ldcg(reinterpret_cast<const float4*>(part_o + (base + s) * D + dd));
        const float4 c = __ldcg(reinterpret_cast<const float4*>(part_o + (base + s) * D + dd + 4));
        const float Mn = fmaxf(M, ml.x);
        const float keep = M > -INFINITY ? exp2f(M - Mn) : 0.f;
        const float f = ml.x > -INFINITY ? exp2f(ml.x - Mn) : 0.f;
        M = Mn;
        lsum = lsum * keep + ml.y * f;
        osum[0] = osum[0] * keep + a.x * f; osum[1] = osum[1] * keep + a.y * f;
        osum[2] = osum[2] * keep + a.z * f; osum[3] = osum[3] * keep + a.w * f;
        osum[4] = osum[4] * keep + c.x * f; osum[5] = osum[5] * keep + c.y * f;
        osum[6] = osum[6] * keep + c.z * f; osum[7] = osum[7] * keep + c.w * f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(lsum > 0.f ? osum[j] / lsum : 0.f);
      *reinterpret_cast<uint4*>(orow + u * 8) = *reinterpret_cast<const uint4*>(e);
    }
    if (out_q) {
      *reinterpret_cast<uint4*>(row_s + u * 8) = *reinterpret_cast<const uint4*>(e);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(to_f32<T>(e[j])));
    }
  }
  if (!out_q) return;
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) amax = fmaxf(amax, red[w]);
  float s = round_to<T>(fmaxf(amax, 1e-5f));
  s = round_to<T>(__fmul_rn(s, 1.0f / 127.0f));
  if (threadIdx.x == 0) out_scale[b] = s;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    __align__(16) T e[8];
    *reinterpret_cast<uint4*>(e) = *reinterpret_cast<const uint4*>(row_s + u * 8);
    __align__(8) int8_t o8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v = rintf(round_to<T>(__fdiv_rn(to_f32<T>(e[j]), s)));
      v = v != v ? v : fminf(fmaxf(v, -128.f), 127.f);
      o8[j] = (int8_t)(int)v;
    }
    *reinterpret_cast<uint2*>(out_q + (int64_t)b * Hq * D + u * 8) = *reinterpret_cast<const uint2*>(o8);
  }
}

// Optional work folded into the attention kernel for the newest token of every sequence (row
// seqlens[b] - 1 of the cache): rotary embedding of q (cos_tab / sin_tab: fp32 [table_rows, D/2],
// half-split pairing, angle row = the token's cache row) and, with k_new / v_new, rotation of the new
// key and the write of key and value into the cache before the block that covers that row reads it.
struct DecodeAppend {
  const uint16_t* k_new;             // [B, Hkv, D] with batch stride kv_batch_stride, or null
  const uint16_t* v_new;
  long long kv_batch_stride;
  const float* cos_tab;              // null: no rotation
  const float* sin_tab;
  int table_rows;
};

template <bool BF16> __device__ __forceinline__ float bits_to_f32(uint16_t h) {
  if constexpr (BF16) return __uint_as_float((uint32_t)h << 16);
  else return __half2float(__ushort_as_half(h));
}
template <bool BF16> __device__ __forceinline__ uint16_t f32_to_bits(float f) {
  if constexpr (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
  else return __half_as_ushort(__float2half_rn(f));
}

template <bool BF16, int D>
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const uint16_t* __restrict__ q, int64_t q_batch_stride, const uint16_t* __restrict__ k_cache,
                   const uint16_t* __restrict__ v_cache, int64_t cache_batch_stride, int64_t cache_row_stride,
                   const int32_t* __restrict__ seqlens, uint16_t* __restrict__ out, int Hq, int Hkv, int chunk,
                   int max_splits, int max_len, float scale, float softcap, float* __restrict__ part_o,
                   float* __restrict__ part_ml, DecodeAppend ap, int8_t* __restrict__ out_q,
                   float* __restrict__ out_scale, int q_cluster) {
  constexpr int NJ = D / 32;          // 16-byte K chunks per lane (quad covers 64 B per step)
  constexpr int NH = D / 64;          // 16-byte V chunks per lane (8 lanes cover 128 B per step)
  pdl_wait();
  pdl_trigger();
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int rep = Hq / Hkv;
  // A length beyond the bound the grid and the partial slots were sized for (the host's max_seqlen,
  // at most the cache capacity) is clamped: the sequence is attended over its first max_len rows and
  // nothing is appended, so neither the cache nor a neighbour's partial slots are touched.
  const int L_raw = seqlens[b];
  const int L = min(L_raw, max_len);
  const int key_begin = split * chunk;
  if (key_begin >= L && !(L == 0 && split == 0)) return;
  const int key_end = min(L, key_begin + chunk);
  const int n_splits = L == 0 ? 1 : (L + chunk - 1) / chunk;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;

  // ---- Q fragments: head row g (zero when g >= rep), same chunk order as the K loads ----
  uint32_t qf[NJ][4];
  {
    const uint16_t* qrow = q + (int64_t)b * q_batch_stride + (int64_t)(hkv * rep + g) * D;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (g < rep) v = *reinterpret_cast<const uint4*>(qrow + 8 * (4 * j + t));
      qf[j][0] = v.x; qf[j][1] = v.y; qf[j][2] = v.z; qf[j][3] = v.w;
    }
  }

  // ---- newest token: rotate q in registers; the block that covers its cache row writes K and V ----
  const int pos = L - 1;
  const bool rotate = ap.cos_tab != nullptr && pos >= 0 && pos < ap.table_rows;
  if (rotate) {
    // chunk 4j+t pairs with chunk 4(j + NJ/2)+t: element i with i + D/2, both held by this thread
    const float* cr = ap.cos_tab + (int64_t)pos * (D / 2);
    const float* sr = ap.sin_tab + (int64_t)pos * (D / 2);
#pragma unroll
    for (int j = 0; j < NJ / 2; ++j) {
      const int i0 = 8 * (4 * j + t);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float2 cs = *reinterpret_cast<const float2*>(cr + i0 + 2 * w);
        const float2 sn = *reinterpret_cast<const float2*>(sr + i0 + 2 * w);
        const uint32_t lo = qf[j][w], hi = qf[j + NJ / 2][w];
        const float a0 = bits_to_f32<BF16>((uint16_t)(lo & 0xffffu)), a1 = bits_to_f32<BF16>((uint16_t)(lo >> 16));
        const float b0 = bits_to_f32<BF16>((uint16_t)(hi & 0xffffu)), b1 = bits_to_f32<BF16>((uint16_t)(hi >> 16));
        qf[j][w] = (uint32_t)f32_to_bits<BF16>(a0 * cs.x - b0 * sn.x) |
                   ((uint32_t)f32_to_bits<BF16>(a1 * cs.y - b1 * sn.y) << 16);
        qf[j + NJ / 2][w] = (uint32_t)f32_to_bits<BF16>(a0 * sn.x + b0 * cs.x) |
                            ((uint32_t)f32_to_bits<BF16>(a1 * sn.y + b1 * cs.y) << 16);
      }
    }
  }
  // (block-uniform condition; like the stand-alone rotary kernel, a position outside the table
  // leaves the cache untouched)
  if (ap.k_new != nullptr && L_raw <= max_len && pos >= key_begin && pos < key_end &&
      (ap.cos_tab == nullptr || rotate)) {
    const int64_t src = (int64_t)b * ap.kv_batch_stride + (int64_t)hkv * D;
    const int64_t dst = (int64_t)b * cache_batch_stride + (int64_t)pos * cache_row_stride + (int64_t)hkv * D;
    uint16_t* kc = const_cast<uint16_t*>(k_cache);
    uint16_t* vc = const_cast<uint16_t*>(v_cache);
    if (tid < D / 2) {
      const float a = bits_to_f32<BF16>(ap.k_new[src + tid]), bb = bits_to_f32<BF16>(ap.k_new[src + tid + D / 2]);
      float c = 1.f, sn = 0.f;
      if (rotate) {
        c = ap.cos_tab[(int64_t)pos * (D / 2) + tid];
        sn = ap.sin_tab[(int64_t)pos * (D / 2) + tid];
      }
      kc[dst + tid] = rotate ? f32_to_bits<BF16>(a * c - bb * sn) : ap.k_new[src + tid];
      kc[dst + tid + D / 2] = rotate ? f32_to_bits<BF16>(a * sn + bb * c) : ap.k_new[src + tid + D / 2];
    } else if (tid < D / 2 + D / 8) {
      const int i = (tid - D / 2) * 8;
      *reinterpret_cast<uint4*>(vc + dst + i) = *reinterpret_cast<const uint4*>(ap.v_new + src + i);
    }
    __syncthreads();                               // the row is in place before any warp of the block fetches it
  }

  float o[NH][8][4];
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[h][e][c] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;      // row g: running max (log2 domain) and this lane's partial sum

  const uint16_t* kb = k_cache + (int64_t)b * cache_batch_stride + (int64_t)hkv * D;
  const uint16_t* vb = v_cache + (int64_t)b * cache_batch_stride + (int64_t)hkv * D;
  const float sl2 = scale * kLog2e;

  // Each warp streams its keys through a private ring of kRing stages in shared memory filled with
  // cp.async (16 keys x (K row + V row) per stage), so several stages are in flight per warp without
  // holding registers.  16-byte chunks are XOR-swizzled per row so that the fragment loads below
  // (K: chunks 4j+t of rows g, g+1; V: chunk g+8h of rows 2t, 2t+2, ...) are bank-conflict free.
  constexpr int ROWB = D * 2;                    // bytes of one K (or V) row of this head
  constexpr int CPR = ROWB / 16;                 // 16-byte chunks per row
  constexpr int STAGEB = 2 * 16 * ROWB;          // K tile + V tile
  extern __shared__ __align__(16) uint8_t ring_all[];
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(ring_all) + (uint32_t)(warp * kRing * STAGEB);
  auto issue_stage = [&](int key0, int stage) {
    if (key0 < key_end) {
      const uint32_t base = ring + (uint32_t)(stage * STAGEB);
#pragma unroll
      for (int i = 0; i < 16 * CPR / 32; ++i) {
        const int id = i * 32 + lane, r = id / CPR, c = id % CPR;
        const int64_t row_off = (int64_t)min(key0 + r, key_end - 1) * cache_row_stride + c * 8;   // clamped rows are masked
        cp_async_16(base + (uint32_t)(r * ROWB + ((c ^ ((r & 1) << 2)) << 4)), kb + row_off);
        cp_async_16(base + (uint32_t)(16 * ROWB + r * ROWB + ((c ^ (((r >> 1) & 3) << 1)) << 4)), vb + row_off);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");          // always commit: group counting stays uniform
  };
  const int first_key = key_begin + warp * 16;
#pragma unroll
  for (int s = 0; s < kRing - 1; ++s) issue_stage(first_key + s * kWarps * 16, s);

  int it = 0;
  for (int key0 = first_key; key0 < key_end; key0 += kWarps * 16, ++it) {
    issue_stage(key0 + (kRing - 1) * kWarps * 16, (it + kRing - 1) % kRing);
    asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");
    __syncwarp();
    const uint32_t st_base = ring + (uint32_t)((it % kRing) * STAGEB);
    uint4 kf[2][NJ];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      const int r = 8 * nb + g;
#pragma unroll
      for (int j = 0; j < NJ; ++j) kf[nb][j] = lds_16B(st_base + (uint32_t)(r * ROWB + (((4 * j + t) ^ ((r & 1) << 2)) << 4)));
    }
    uint4 vf[4][NH];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int r = 2 * t + (s & 1) + 8 * (s >> 1);
#pragma unroll
      for (int h = 0; h < NH; ++h)
        vf[s][h] = lds_16B(st_base + (uint32_t)(16 * ROWB + r * ROWB + (((g + 8 * h) ^ (((r >> 1) & 3) << 1)) << 4)));
    }
    __syncwarp();                                  // every lane has its fragments: the stage may be refilled

    // ---- S = Q K^T for 16 keys ----
    float s_acc[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int c = 0; c < 4; ++c) s_acc[nb][c] = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        mma_16816<BF16>(s_acc[nb], qf[j][0], 0u, qf[j][1], 0u, kf[nb][j].x, kf[nb][j].y);
        mma_16816<BF16>(s_acc[nb], qf[j][2], 0u, qf[j][3], 0u, kf[nb][j].z, kf[nb][j].w);
      }
    }

    // ---- online softmax for head row g (this lane: keys 8nb + 2t, 8nb + 2t + 1) ----
    float p[2][2];
    float mx = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float s = s_acc[nb][c];
        if (softcap != 0.f) s = softcap * tanhf(s * scale / softcap) * kLog2e;
        else s *= sl2;
        if (key0 + 8 * nb + 2 * t + c >= key_end) s = -INFINITY;
        p[nb][c] = s;
        mx = fmaxf(mx, s);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);                        // finite: key0 < key_end
    const float corr = exp2f(m_run - m_new);
    m_run = m_new;
    float psum = 0.f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        p[nb][c] = exp2f(p[nb][c] - m_new);
        psum += p[nb][c];
      }
    l_run = l_run * corr + psum;
#pragma unroll
    for (int h = 0; h < NH; ++h)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[h][e][0] *= corr;
        o[h][e][1] *= corr;
      }
    const uint32_t pa0 = pack2<BF16>(p[0][0], p[0][1]);          // key slots 2t, 2t+1
    const uint32_t pa2 = pack2<BF16>(p[1][0], p[1][1]);          // key slots 2t+8, 2t+9

    // ---- O += P V ----
#pragma unroll
    for (int h = 0; h < NH; ++h) {
      const uint32_t* v0 = &vf[0][h].x;
      const uint32_t* v1 = &vf[1][h].x;
      const uint32_t* v2 = &vf[2][h].x;
      const uint32_t* v3 = &vf[3][h].x;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(v0[e >> 1], v1[e >> 1], sel);
        const uint32_t b1 = __byte_perm(v2[e >> 1], v3[e >> 1], sel);
        mma_16816<BF16>(o[h][e], pa0, 0u, pa2, 0u, b0, b1);
      }
    }
  }

  // ---- merge the warps of this block ----
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                 // all rings are idle: reuse them for the merge
  float (*sm_o)[8][D] = reinterpret_cast<float (*)[8][D]>(ring_all);
  __shared__ float sm_m[kWarps][8];
  __shared__ float sm_l[kWarps][8];
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (t == 0) {
    sm_m[warp][g] = m_run;
    sm_l[warp][g] = l_run;
  }
#pragma unroll
  for (int h = 0; h < NH; ++h)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      sm_o[warp][g][8 * (2 * t + 8 * h) + e] = o[h][e][0];
      sm_o[warp][g][8 * (2 * t + 1 + 8 * h) + e] = o[h][e][1];
    }
  __syncthreads();

  // out_q (only passed without splits, when the blocks of the sequence's KV heads -- this one alone, or
  // the q_cluster CTAs of this thread-block cluster -- hold the WHOLE token row between them): the
  // per-token int8 quantization of the row is done right here and the merge kernel is not launched.
  // The row's absolute maximum is the one thing the blocks exchange, through distributed shared memory.
  using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
  // (scratch behind the merge tile inside the idle rings: static shared memory would push two
  // resident blocks over the next carve-out step and cost L1)
  uint16_t* row_bits = reinterpret_cast<uint16_t*>(ring_all + kWarps * 8 * D * 4);
  float* red_amax = reinterpret_cast<float*>(ring_all + kWarps * 8 * D * 4 + 8 * D * 2);
  float amax = 0.f;
  for (int i = tid; i < rep * D; i += kThreads) {
    const int hd = i / D, dd = i - hd * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, sm_m[w][hd]);
    float lsum = 0.f, osum = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float f = exp2f(sm_m[w][hd] - M);
        lsum += sm_l[w][hd] * f;
        osum += sm_o[w][hd][dd] * f;
      }
    }
    const int hq = hkv * rep + hd;
    if (n_splits == 1) {
      const float r = lsum > 0.f ? osum / lsum : 0.f;
      uint16_t bits;
      if constexpr (BF16) { __nv_bfloat16 hv = __float2bfloat16_rn(r); bits = *reinterpret_cast<uint16_t*>(&hv); }
      else { __half hv = __float2half_rn(r); bits = *reinterpret_cast<uint16_t*>(&hv); }
      out[((int64_t)b * Hq + hq) * D + dd] = bits;
      if (out_q) {
        row_bits[i] = bits;
        amax = fmaxf(amax, fabsf(bits_to_f32<BF16>(bits)));
      }
    } else {
      const int64_t slot = ((int64_t)b * Hq + hq) * max_splits + split;
      part_o[slot * D + dd] = osum;
      if (dd == 0) {
        part_ml[slot * 2] = M;
        part_ml[slot * 2 + 1] = lsum;
      }
    }
  }
  if (out_q) {                                       // block-uniform; the arithmetic of the stand-alone per-token quantizer
    amax = warp_max(amax);
    if (lane == 0) red_amax[warp] = amax;
    __syncthreads();
    amax = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) amax = fmaxf(amax, red_amax[w]);
    if (q_cluster > 1) {
      // every CTA leaves its maximum in its own scratch (its rings are idle by now; a peer's may not
      // be, so nothing is written remotely), one cluster barrier, then every thread reads the peers'
      // values through distributed shared memory.  A second barrier keeps each CTA's shared memory
      // alive until all peers have read it: arrive right after the reads, wait after the stores below.
      if (tid == 0) red_amax[kWarps] = amax;
      asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
      const uint32_t local = (uint32_t)__cvta_generic_to_shared(&red_amax[kWarps]);
      for (int r = 0; r < q_cluster; ++r) {
        uint32_t remote;
        float v;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)r));
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
        amax = fmaxf(amax, v);
      }
      asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    }
    float sc = round_to<T>(fmaxf(amax, 1e-5f));
    sc = round_to<T>(__fmul_rn(sc, 1.0f / 127.0f));
    if (tid == 0 && hkv == 0) out_scale[b] = sc;
    for (int i = tid; i < rep * D; i += kThreads) {
      float v = rintf(round_to<T>(__fdiv_rn(bits_to_f32<BF16>(row_bits[i]), sc)));
      v = v != v ? v : fminf(fmaxf(v, -128.f), 127.f);
      out_q[((int64_t)b * Hq + hkv * rep) * D + i] = (int8_t)(int)v;     // this block's heads of the token row
    }
    if (q_cluster > 1) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
  }
}

// Merge of the splits, one block per sequence.  Dynamic shared memory: Hq * D 16-bit words when out_q
// is given.  (Letting the last block of a sequence do this inside the main kernel, counted off with
// an atomic per block, was measured slower: the round trip of the atomic holds every block's shared
// memory for about a microsecond and the last merges form a serial tail.)
template <bool BF16, int D>
__global__ void __launch_bounds__(1024)
attn_decode_combine_kernel(const int32_t* __restrict__ seqlens, uint16_t* __restrict__ out, int Hq, int chunk,
                           int max_splits, int max_len, const float* __restrict__ part_o,
                           const float* __restrict__ part_ml,
                           int8_t* __restrict__ out_q, float* __restrict__ out_scale) {
  extern __shared__ __align__(16) uint8_t row_raw[];
  __shared__ float red[32];
  pdl_wait_then_trigger();
  const int b = blockIdx.x;
  const int L = min(seqlens[b], max_len);          // same clamp as the main kernel
  const int n_splits = (L + chunk - 1) / chunk;
  if (n_splits <= 1 && !out_q) return;             // the main kernel already wrote the result
  merge_sequence<BF16, D>(b, n_splits, out, Hq, max_splits, part_o, part_ml, out_q, out_scale,
                          reinterpret_cast<uint16_t*>(row_raw), red);
}

__global__ void kv_append_kernel(uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, int64_t batch_stride16,
                                 int64_t row_stride16, const uint4* __restrict__ k, const uint4* __restrict__ v,
                                 const int32_t* __restrict__ seqlens, int start_pos, int S_new, int row16, int Smax) {
  // one block per (b, s); row16 = Hkv * d / 8 sixteen-byte units per token
  const int s = blockIdx.x, b = blockIdx.y;
  const int pos = (seqlens ? seqlens[b] : start_pos) + s;
  if (pos < 0 || pos >= Smax) return;              // never write outside the cache
  const int64_t src = ((int64_t)b * S_new + s) * row16;
  const int64_t dst = (int64_t)b * batch_stride16 + (int64_t)pos * row_stride16;
  for (int i = threadIdx.x; i < row16; i += blockDim.x) {
    k_cache[dst + i] = k[src + i];
    v_cache[dst + i] = v[src + i];
  }
}

// Quantization inside the attention kernel is used unless the environment variable
// LLMQRT_ATTN_FUSED_QUANT is "0" (then the merge kernel quantizes).
bool quant_fused_enabled() {
  static const bool on = [] {
    const char* v = getenv("LLMQRT_ATTN_FUSED_QUANT");
    return !(v && v[0] == '0');
  }();
  return on;
}

template <bool BF16, int D>
int launch_decode(const void* q, int64_t qbs, const void* kc, const void* vc, int64_t bs, int64_t rs,
                  const int32_t* seqlens, void* out, int8_t* out_q, float* out_scale, int B, int Hq, int Hkv,
                  int max_seqlen, float softcap, void* workspace, cudaStream_t st, const DecodeAppend& ap) {
  // Keys per block: the smallest power of two for which all blocks are resident at once (two fit an
  // SM), i.e. as many blocks as one wave takes and no second wave -- a block costs about 3 us beyond
  // its keys (first loads, merge of its warps), so waves of short blocks lose to one wave of long
  // ones (batch 64 x 4 KV heads x 1100 keys: 35 us with 256-key blocks, 26 us unsplit).
  int chunk = 64;
  {
    const int64_t slots = 2 * (int64_t)sm_count();
    while (chunk < max_seqlen && (int64_t)B * Hkv * ceil_div(max_seqlen, chunk) > slots) chunk *= 2;
    // Longer blocks than about a thousand keys stop paying: with ragged lengths the longest sequence
    // then runs alone at the end (32 sequences of 512..8192 keys: 59 us at 1024, 65 us at 4096).
    if (chunk > 1024 && max_seqlen > 2048) chunk = 1024;
    // Two splits per sequence when the unsplit blocks alone would cover most of the SMs: not worth the
    // merge kernel (batch 64 x 2 KV heads x 1150 keys: 16.0 us unsplit, 21.3 us as 2 x 1024 keys + merge;
    // batch 64 x 1 KV head: 15.0 us unsplit against 14.3 us in three splits, left alone).
    if (max_seqlen <= 2048 && ceil_div(max_seqlen, chunk) == 2 && (int64_t)B * Hkv * 4 >= 3 * (int64_t)sm_count()) chunk *= 2;
  }
  static const int forced_chunk = [] {               // LLMQRT_ATTN_CHUNK=<power of two>: keys per block, for A/B runs
    const char* env = getenv("LLMQRT_ATTN_CHUNK");
    const int v = env ? atoi(env) : 0;
    return (v >= 16 && (v & (v - 1)) == 0) ? v : 0;
  }();
  if (forced_chunk) chunk = forced_chunk;
  int max_splits = (int)ceil_div(max_seqlen > 0 ? max_seqlen : 1, chunk);
  while (max_splits > 1 && (size_t)B * Hq * max_splits * (D + 2) * 4 > LLMQRT_WS_PARTIAL_BYTES) {
    chunk *= 2;
    max_splits = (int)ceil_div(max_seqlen, chunk);
  }
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (max_splits > 1) {
    if (!workspace) return set_error(LLMQRT_ERR_WORKSPACE, "attn_decode: split-KV needs the workspace");
    part_o = reinterpret_cast<float*>(ws_partials(workspace));
    part_ml = part_o + (size_t)B * Hq * max_splits * D;
  }
  const float scale = 1.0f / sqrtf((float)D);
  constexpr int smem = kWarps * kRing * 2 * 16 * D * 2;           // per-warp rings; also holds the 16 KiB merge tile
  static_assert(smem >= kWarps * 8 * D * 4 + 8 * D * 2 + kWarps * 4 + 4, "ring too small for the merge tile and the quantization scratch");
  auto kern = attn_decode_kernel<BF16, D>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  // No splits: the attention blocks of a sequence produce the whole token row and quantize it
  // themselves -- one kernel less per layer.
  // Several KV heads: the blocks of one sequence form a thread-block cluster (at most 8 CTAs) and
  // exchange the row maximum through distributed shared memory.
  const bool quant_in_kernel = out_q != nullptr && Hkv <= 8 && max_splits == 1 && Hq / Hkv <= 8 && quant_fused_enabled();
  const int q_cluster = quant_in_kernel ? Hkv : 1;
  const bool need_merge = max_splits > 1 || (out_q != nullptr && !quant_in_kernel);
  if (int rc = launch_chained(kern, dim3(max_splits, Hkv, B), dim3(kThreads), smem, st, dim3(1, (unsigned)q_cluster, 1),
                              reinterpret_cast<const uint16_t*>(q), qbs, reinterpret_cast<const uint16_t*>(kc),
                              reinterpret_cast<const uint16_t*>(vc), bs, rs, seqlens, reinterpret_cast<uint16_t*>(out),
                              Hq, Hkv, chunk, max_splits, max_seqlen, scale, softcap, part_o, part_ml, ap,
                              quant_in_kernel ? out_q : (int8_t*)nullptr, quant_in_kernel ? out_scale : (float*)nullptr,
                              q_cluster))
    return rc;
  if (int rc = check_launch("attn_decode")) return rc;
  if (need_merge) {
    const int units = Hq * D / 8;
    const int threads = units >= 1024 ? 1024 : (units + 31) / 32 * 32;
    const size_t row_smem = out_q ? (size_t)Hq * D * 2 : 0;
    if (int rc = launch_chained(attn_decode_combine_kernel<BF16, D>, dim3(B), dim3(threads), row_smem, st, 1, seqlens,
                                reinterpret_cast<uint16_t*>(out), Hq, chunk, max_splits, max_seqlen,
                                static_cast<const float*>(part_o), static_cast<const float*>(part_ml), out_q,
                                out_scale))
      return rc;
    return check_launch("attn_decode_combine");
  }
  return LLMQRT_OK;
}

}  // namespace
}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_kv_append(void* k_cache, void* v_cache, int64_t cache_batch_stride, int64_t cache_row_stride, const void* k,
                     const void* v, const int32_t* cache_seqlens, int32_t start_pos, int dtype, int64_t B,
                     int64_t S_new, int64_t Hkv, int64_t d, int64_t Smax, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "kv_append: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(B >= 0 && S_new >= 0 && Hkv > 0 && d > 0 && (Hkv * d) % 8 == 0, "kv_append: bad shape");
  LLMQRT_REQUIRE(cache_batch_stride % 8 == 0 && cache_row_stride % 8 == 0, "kv_append: strides must be multiples of 8");
  if (B == 0 || S_new == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(k_cache && v_cache && k && v, "kv_append: null pointer");
  LLMQRT_REQUIRE(((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
                   reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0,
                 "kv_append: pointers must be 16-byte aligned");
  const int row16 = (int)(Hkv * d / 8);
  kv_append_kernel<<<dim3((unsigned)S_new, (unsigned)B), row16 < 256 ? row16 : 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<uint4*>(k_cache), reinterpret_cast<uint4*>(v_cache), cache_batch_stride / 8,
      cache_row_stride / 8, reinterpret_cast<const uint4*>(k), reinterpret_cast<const uint4*>(v), cache_seqlens,
      start_pos, (int)S_new, row16, (int)Smax);
  return check_launch("kv_append");
}

static int attn_decode_entry(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                             int64_t cache_batch_stride, int64_t cache_row_stride, const int32_t* seqlens, void* out,
                             int8_t* out_q, float* out_scale, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t d,
                             int64_t max_seqlen, float softcap, void* workspace, llmqrt_stream_t stream,
                             const DecodeAppend& ap) {
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "attn_decode: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(d == 64 || d == 128, "attn_decode: head_dim must be 64 or 128 (got %lld)", (long long)d);
  LLMQRT_REQUIRE(Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= 8, "attn_decode: need Hq %% Hkv == 0 and at most 8 query heads per KV head");
  LLMQRT_REQUIRE(B >= 0 && B < 65536 && Hkv < 65536 && max_seqlen >= 0, "attn_decode: bad shape");
  LLMQRT_REQUIRE(cache_batch_stride % 8 == 0 && cache_row_stride % 8 == 0, "attn_decode: cache strides must be multiples of 8");
  LLMQRT_REQUIRE(q_batch_stride >= Hq * d && q_batch_stride % 8 == 0, "attn_decode: q_batch_stride must be a multiple of 8 and at least Hq * d");
  LLMQRT_REQUIRE(!out_q || (out_scale && Hq * d <= 8192), "attn_decode: quantized output needs out_scale and Hq * d <= 8192");
  if (B == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(q && k_cache && v_cache && seqlens && out, "attn_decode: null pointer");
  LLMQRT_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) |
                   reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(out_q) & 7) == 0, "attn_decode: pointers must be 16-byte aligned (out_q: 8)");
  cudaStream_t st = (cudaStream_t)stream;
  const bool bf = dtype == LLMQRT_BF16;
#define LLMQRT_GO(BF, DD)                                                                                          \
  return launch_decode<BF, DD>(q, q_batch_stride, k_cache, v_cache, cache_batch_stride, cache_row_stride, seqlens, \
                               out, out_q, out_scale, (int)B, (int)Hq, (int)Hkv, (int)max_seqlen, softcap,         \
                               workspace, st, ap)
  if (d == 128) { if (bf) LLMQRT_GO(true, 128); else LLMQRT_GO(false, 128); }
  if (bf) LLMQRT_GO(true, 64); else LLMQRT_GO(false, 64);
#undef LLMQRT_GO
}

int llmqrt_attn_decode(const void* q, int64_t q_batch_stride, const void* k_cache, const void* v_cache,
                       int64_t cache_batch_stride, int64_t cache_row_stride, const int32_t* seqlens, void* out,
                       int8_t* out_q, float* out_scale, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t d,
                       int64_t max_seqlen, float softcap, void* workspace, llmqrt_stream_t stream) {
  const DecodeAppend none = {nullptr, nullptr, 0, nullptr, nullptr, 0};
  return attn_decode_entry(q, q_batch_stride, k_cache, v_cache, cache_batch_stride, cache_row_stride, seqlens, out,
                           out_q, out_scale, dtype, B, Hq, Hkv, d, max_seqlen, softcap, workspace, stream, none);
}

int llmqrt_attn_decode_append(const void* q, int64_t q_batch_stride, const void* k_new, const void* v_new,
                              int64_t kv_batch_stride, const float* cos_table, const float* sin_table,
                              int64_t table_rows, void* k_cache, void* v_cache, int64_t cache_batch_stride,
                              int64_t cache_row_stride, const int32_t* seqlens, void* out, int8_t* out_q,
                              float* out_scale, int dtype, int64_t B, int64_t Hq, int64_t Hkv, int64_t d,
                              int64_t max_seqlen, float softcap, void* workspace, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE((k_new == nullptr) == (v_new == nullptr), "attn_decode_append: k_new and v_new go together");
  LLMQRT_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attn_decode_append: cos and sin tables go together");
  LLMQRT_REQUIRE(!k_new || (kv_batch_stride >= Hkv * d && kv_batch_stride % 8 == 0 &&
                            ((reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new)) & 15) == 0),
                 "attn_decode_append: k_new / v_new must be 16-byte aligned with a batch stride that is a multiple of 8");
  LLMQRT_REQUIRE(!cos_table || (table_rows > 0 && table_rows <= 0x7fffffffll &&
                                ((reinterpret_cast<uintptr_t>(cos_table) | reinterpret_cast<uintptr_t>(sin_table)) & 7) == 0),
                 "attn_decode_append: rotary tables must be 8-byte aligned fp32 [table_rows, d/2]");
  const DecodeAppend ap = {static_cast<const uint16_t*>(k_new), static_cast<const uint16_t*>(v_new),
                           (long long)kv_batch_stride, cos_table, sin_table, (int)table_rows};
  return attn_decode_entry(q, q_batch_stride, k_cache, v_cache, cache_batch_stride, cache_row_stride, seqlens, out,
                           out_q, out_scale, dtype, B, Hq, Hkv, d, max_seqlen, softcap, workspace, stream, ap);
}

}  // extern "C"

