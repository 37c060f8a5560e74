// Prefill attention over the new tokens on the 5th-generation tensor cores:
//     O = softmax(mask(Q K^T / sqrt(d))) V,  causal or not, GQA (query head h reads KV head h / (Hq/Hkv)).
//
// One CTA owns 256 consecutive query rows of one head as two 128-row tiles.  Roles (384 threads):
//   warps 0-3 / 4-7  one softmax group per query tile, one thread per query row;
//   warp 8           TMA producer: the two Q tiles once, then K and V tiles of 128 keys through a ring;
//   warp 9           owns tensor memory and issues every tcgen05.mma (one elected lane, warp-uniform loop);
//   warps 10-11      none: they complete the third warpgroup, which hands most of its registers to
//                    the softmax groups (setmaxnreg), whose threads hold a whole 128-wide row of S.
// Per key tile j and query tile w:
//   S_w = Q_w K_j^T    tcgen05.mma kind::f16, both operands K-major in shared memory (TMA, 128-byte
//                      swizzle), 128 x 128 fp32 accumulator in tensor memory;
//   softmax            the row's thread reads the whole S row with tcgen05.ld, keeps the reference
//                      maximum and the sum in registers and writes P as packed 16-bit pairs back into
//                      tensor memory over the first half of S (tcgen05.st);
//   O_w += P V_j       tcgen05.mma with P as the tensor-memory operand and V as an MN-major
//                      shared-memory operand (V tiles are stored [key][d], d contiguous), accumulating
//                      over the key tiles in a 128 x d fp32 accumulator in tensor memory.
// The exponentials of a row are taken relative to a reference maximum that is only moved when the
// row's true maximum has grown by more than 2^8 since (P then stays below 256, exact enough in 16
// bits and far from overflow): moving it means scaling the row of O in tensor memory (a tcgen05.ld /
// tcgen05.st round trip), which with this rule happens in the first tiles of a row and hardly ever
// afterwards.  The tensor pipe alternates between the two query tiles: while one group runs its
// softmax, the pipe multiplies for the other.
//
// Tensor memory (512 columns): S_0 | S_1 | O_0 | O_1, 128 columns each (O uses d).  P_w aliases the
// first 64 columns of S_w; the MMAs of one CTA execute in issue order, and S_w(j+1) is only issued
// after P_w(j) V_j, so the alias is never overwritten while it is being read, and S_w(j+1) complete
// implies P_w(j) V_j complete, so O_w is at rest whenever its group touches it.
//
// Every wait on an mbarrier is bounded; when one runs out the block raises a flag, every role
// leaves its loop, outstanding copies are drained, tensor memory is freed and a status word is set.
// No multicast: every CTA fetches its own tiles.
#include "tc_primitives.cuh"

#include <mutex>

namespace llmqrt {
namespace {

constexpr int kThreads = 384;
constexpr int kRows = 128;              // query rows per softmax group / keys per tile
constexpr int kSubBytes = 128 * 128;    // one 64-element-wide sub-tile: 128 rows x 128 bytes
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillParams {
  int S, Hq, Hkv, causal;
  float scale, softcap;
  uint16_t* out;
  long long out_ts;                     // elements between the output rows of consecutive tokens
  uint32_t idesc_s, idesc_pv;
  unsigned* status;                     // set to 1 if a bounded wait ran out (may be null)
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tensor_map, uint32_t bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst_smem), "l"(tensor_map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Shared-memory descriptor of an MN-major operand stored as rows of 128 bytes (64 16-bit values of the
// M/N dimension per row, one row per K index) with the 128-byte swizzle: the eight 16-byte units of a
// row are contiguous, consecutive K rows are 128 bytes apart, groups of eight K rows `sbo` bytes apart
// and consecutive 64-value chunks of the M/N dimension `lbo` bytes apart.
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
  const uint32_t hi = (sbo >> 4) | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (packed 16-bit pairs).
__device__ __forceinline__ void mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns, registers -> tensor memory.
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

// K and V tiles travel through rings of their own: a K tile is free as soon as both S products that
// read it have retired, long before the V tile of the same keys, so its slot can be refilled a whole
// key tile earlier.  With 128-wide heads shared memory holds two Q tiles, three K and two V tiles.
template <int D> constexpr int k_stages() { return D == 128 ? 3 : 4; }
template <int D> constexpr int v_stages() { return D == 128 ? 2 : 4; }
template <int D> constexpr int tile_bytes() { return (D / 64) * kSubBytes; }
template <int D> constexpr int smem_bytes() { return (2 + k_stages<D>() + v_stages<D>()) * tile_bytes<D>() + 1024; }

template <bool BF16, int D>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, PrefillParams prm) {
  constexpr int kSub = D / 64;
  constexpr int kTile = tile_bytes<D>();
  constexpr int kKS = k_stages<D>(), kVS = v_stages<D>();
  constexpr uint32_t kColS = 0, kColO = 256;           // tensor-memory columns: S_w at 128 w, O_w at 256 + 128 w

  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;                                  // [2][kTile]
  uint8_t* sK = base + 2 * kTile;                      // [kKS][kTile]
  uint8_t* sV = sK + kKS * kTile;                      // [kVS][kTile]
  __shared__ __align__(8) uint64_t bar_q;
  __shared__ __align__(8) uint64_t bar_k_full[kKS];
  __shared__ __align__(8) uint64_t bar_k_empty[kKS];
  __shared__ __align__(8) uint64_t bar_v_full[kVS];
  __shared__ __align__(8) uint64_t bar_v_empty[kVS];
  __shared__ __align__(8) uint64_t bar_s_full[2];      // S_w(j) complete (MMA commit)
  __shared__ __align__(8) uint64_t bar_p_ready[2];     // P_w(j) written, O_w rescaled if need be (128 arrivals)
  __shared__ __align__(8) uint64_t bar_o_full[2];      // O_w complete after the last key tile (MMA commit)
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &abort_flag;

  // heaviest query tiles first: with a causal mask the last rows see the most keys
  const int pair = (int)gridDim.x - 1 - (int)blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (prm.Hq / prm.Hkv);
  const int S = prm.S;
  const int q0 = pair * 2 * kRows;
  const int kv_tiles = (S + kRows - 1) / kRows;
  int n_tiles[2];                                      // key tiles each query tile attends to
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int qb = q0 + w * kRows;
    n_tiles[w] = qb >= S ? 0 : (prm.causal ? min(qb / kRows + 1, kv_tiles) : kv_tiles);
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc::mbar_init(tc::smem_u32(&bar_q), 1);
    for (int s = 0; s < kKS; ++s) {
      tc::mbar_init(tc::smem_u32(&bar_k_full[s]), 1);
      tc::mbar_init(tc::smem_u32(&bar_k_empty[s]), 1);
    }
    for (int s = 0; s < kVS; ++s) {
      tc::mbar_init(tc::smem_u32(&bar_v_full[s]), 1);
      tc::mbar_init(tc::smem_u32(&bar_v_empty[s]), 1);
    }
    for (int w = 0; w < 2; ++w) {
      tc::mbar_init(tc::smem_u32(&bar_s_full[w]), 1);
      tc::mbar_init(tc::smem_u32(&bar_p_ready[w]), kRows);
      tc::mbar_init(tc::smem_u32(&bar_o_full[w]), 1);
    }
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&tm_q);
    tc::tma_prefetch_descriptor(&tm_k);
    tc::tma_prefetch_descriptor(&tm_v);
  }
  if (warp == 9) {
    tc::tmem_alloc(tc::smem_u32(&tmem_base_slot), 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  // Register budget per warpgroup (8 x 216 + 4 x 72 registers per lane fit the SM's file): each role
  // branch starts by shrinking or growing its warpgroup's share.
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 8) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      const int nq = (n_tiles[0] > 0) + (n_tiles[1] > 0);
      tc::mbar_arrive_expect_tx(tc::smem_u32(&bar_q), (uint32_t)(nq * kTile));
      for (int w = 0; w < 2; ++w)
        if (n_tiles[w] > 0)
          for (int sub = 0; sub < kSub; ++sub)
            tma_load_3d(tc::smem_u32(sQ + w * kTile + sub * kSubBytes), &tm_q, tc::smem_u32(&bar_q), hq * D + sub * 64,
                        q0 + w * kRows, b);
      bool ok = true;
      // K runs up to two tiles ahead of V (its ring is deeper and its slots come free earlier)
      int kj = 0, vj = 0;
      while (ok && (kj < n_max || vj < n_max)) {
        if (kj < n_max && (kj <= vj + 2 || vj >= n_max)) {
          const int st = kj % kKS;
          const uint32_t ph = (uint32_t)(kj / kKS) & 1u;
          if (!tc::mbar_wait(tc::smem_u32(&bar_k_empty[st]), ph ^ 1u, abort)) { ok = false; break; }
          const uint32_t full = tc::smem_u32(&bar_k_full[st]);
          tc::mbar_arrive_expect_tx(full, kTile);
          for (int sub = 0; sub < kSub; ++sub)
            tma_load_3d(tc::smem_u32(sK + st * kTile + sub * kSubBytes), &tm_k, full, hkv * D + sub * 64, kj * kRows, b);
          ++kj;
        } else {
          const int st = vj % kVS;
          const uint32_t ph = (uint32_t)(vj / kVS) & 1u;
          if (!tc::mbar_wait(tc::smem_u32(&bar_v_empty[st]), ph ^ 1u, abort)) { ok = false; break; }
          const uint32_t full = tc::smem_u32(&bar_v_full[st]);
          tc::mbar_arrive_expect_tx(full, kTile);
          for (int sub = 0; sub < kSub; ++sub)
            tma_load_3d(tc::smem_u32(sV + st * kTile + sub * kSubBytes), &tm_v, full, hkv * D + sub * 64, vj * kRows, b);
          ++vj;
        }
      }
      if (!ok) {
        // drain: wait (bounded) for the copies still in flight so that none lands after the block left
        const uint64_t t0 = tc::global_timer_ns();
        while (!tc::mbar_try_wait(tc::smem_u32(&bar_q), 0u) && tc::global_timer_ns() - t0 < tc::kWaitLimitNs) {}
        for (int i = max(0, kj - kKS); i < kj; ++i)
          while (!tc::mbar_try_wait(tc::smem_u32(&bar_k_full[i % kKS]), (uint32_t)(i / kKS) & 1u) &&
                 tc::global_timer_ns() - t0 < tc::kWaitLimitNs) {}
        for (int i = max(0, vj - kVS); i < vj; ++i)
          while (!tc::mbar_try_wait(tc::smem_u32(&bar_v_full[i % kVS]), (uint32_t)(i / kVS) & 1u) &&
                 tc::global_timer_ns() - t0 < tc::kWaitLimitNs) {}
      }
    }
  } else if (warp == 9) {
    // ------------------------------- MMA issuer ---------------------------------
    // The whole warp runs the loop; only the tcgen05 instructions themselves are issued by one elected lane.
    if (n_max > 0) {
      bool ok = tc::mbar_wait_warp(tc::smem_u32(&bar_q), 0u, abort);
      // S_w = Q_w K^T: both operands K-major; D / 16 instructions of K = 16
      auto issue_s = [&](int w, int st) {
        const uint32_t qa = tc::smem_u32(sQ + w * kTile), ka = tc::smem_u32(sK + st * kTile);
        const uint32_t d_tmem = tmem_base + kColS + (uint32_t)(w * 128);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (uint32_t)((ks / 4) * kSubBytes + (ks % 4) * 32);
          const uint64_t da = tc::smem_desc_k_major_sw128(qa + off), db = tc::smem_desc_k_major_sw128(ka + off);
          if (tc::elect_one()) tc::mma_ss<tc::MMA_F16>(d_tmem, da, db, prm.idesc_s, ks > 0 ? 1u : 0u);
        }
        if (tc::elect_one()) tc::mma_commit(tc::smem_u32(&bar_s_full[w]));
      };
      // O_w = P_w V: P from tensor memory (8 packed columns per 16 keys), V MN-major (16 key rows per step)
      auto issue_pv = [&](int w, int st, int j) {
        const uint32_t va = tc::smem_u32(sV + st * kTile);
        const uint32_t d_tmem = tmem_base + kColO + (uint32_t)(w * 128), a_tmem = tmem_base + kColS + (uint32_t)(w * 128);
#pragma unroll
        for (int t = 0; t < kRows / 16; ++t) {
          const uint64_t db = smem_desc_mn_major_sw128(va + (uint32_t)(t * 16 * 128), kSubBytes, 1024);
          if (tc::elect_one()) mma_ts_f16(d_tmem, a_tmem + (uint32_t)(t * 8), db, prm.idesc_pv, (j > 0 || t > 0) ? 1u : 0u);
        }
        if (j == n_tiles[w] - 1 && tc::elect_one()) tc::mma_commit(tc::smem_u32(&bar_o_full[w]));   // last tile: O complete
      };
      // the last query tile that reads key tile t (the second one sees at least as many tiles as the
      // first, unless it lies beyond the sequence altogether)
      auto last_user = [&](int t) { return t < n_tiles[1] ? 1 : 0; };
      if (ok) ok = tc::mbar_wait_warp(tc::smem_u32(&bar_k_full[0]), 0u, abort);
      if (ok) {
        tc::fence_after_sync();
        for (int w = 0; w < 2; ++w)
          if (n_tiles[w] > 0) issue_s(w, 0);
        if (tc::elect_one()) tc::mma_commit(tc::smem_u32(&bar_k_empty[0]));
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int vs = j % kVS, ks1 = (j + 1) % kKS;
        const uint32_t vph = (uint32_t)(j / kVS) & 1u, kph1 = (uint32_t)((j + 1) / kKS) & 1u;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j >= n_tiles[w]) continue;
          if (!tc::mbar_wait_warp(tc::smem_u32(&bar_p_ready[w]), (uint32_t)j & 1u, abort)) { ok = false; break; }
          if (!tc::mbar_wait_warp(tc::smem_u32(&bar_v_full[vs]), vph, abort)) { ok = false; break; }
          tc::fence_after_sync();
          issue_pv(w, vs, j);
          if (w == last_user(j) && tc::elect_one()) tc::mma_commit(tc::smem_u32(&bar_v_empty[vs]));      // V_j free once these retire
          if (j + 1 < n_tiles[w]) {
            if (!tc::mbar_wait_warp(tc::smem_u32(&bar_k_full[ks1]), kph1, abort)) { ok = false; break; }
            issue_s(w, ks1);
            if (w == last_user(j + 1) && tc::elect_one()) tc::mma_commit(tc::smem_u32(&bar_k_empty[ks1]));   // K_{j+1} likewise
          }
        }
      }
    }
  }
  } else {
    // ------------------------------- softmax groups ------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int w = warp >> 2;                           // query tile of this group
    const int quad = warp & 3;                         // tensor-memory lane quadrant of this warp
    const int r = quad * 32 + lane;                    // row of the tile handled by this thread
    const int row = q0 + w * kRows + r;                // query position
    const int n = n_tiles[w];
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + kColS + (uint32_t)(w * 128);
    const uint32_t t_o = tmem_base + lane_addr + kColO + (uint32_t)(w * 128);
    const float sl = prm.scale * kLog2e;
    const bool capped = prm.softcap != 0.f;
    float m_ref = -INFINITY, l_run = 0.f;              // reference maximum of the exponentials, running sum
    bool ok = true;

    for (int j = 0; j < n; ++j) {
      // every thread of the group must take the same path: OR the failure over the group's 128 threads
      const bool failed = !tc::mbar_wait(tc::smem_u32(&bar_s_full[w]), (uint32_t)j & 1u, abort);
      if (tc::named_barrier_or(1 + w, kRows, failed)) { ok = false; break; }
      tc::fence_after_sync();
      const int key0 = j * kRows;
      // keys this row may see in this tile: [key0, key0 + limit)
      int limit = S - key0;
      if (prm.causal) limit = min(limit, row - key0 + 1);
      const bool need_mask = limit < kRows;            // (limit >= 1 for every row < S: key 0 of the row's first tile)

      // the whole row of S: four loads in flight, one wait
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc::tmem_ld_32x32(t_s + (uint32_t)(c * 32), v[c]);
      tc::tmem_ld_wait();

      // row maximum: eight independent chains (a single chain of 128 dependent maxima is pure latency)
      float mxs[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mxs[i] = -INFINITY;
      if (capped || need_mask) {                        // soft cap and mask applied in place (diagonal / last tile)
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = __uint_as_float(v[c][i]);
            if (capped) x = prm.softcap * tanhf(x * prm.scale / prm.softcap) / prm.scale;
            if (need_mask && c * 32 + i >= limit) x = -INFINITY;
            v[c][i] = __float_as_uint(x);
            mxs[i & 7] = fmaxf(mxs[i & 7], x);
          }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(v[c][i]));
      }
      const float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                             fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      // Move the reference only when the maximum has outgrown it by more than 2^8 (always on the first
      // tile).  tcgen05.ld / st are warp-wide, so the decision is taken per warp; a lane of a moving warp
      // moves to its own exact maximum.
      const bool grow = (mx - m_ref) * sl > 8.f;       // m_ref = -inf: true unless the row sees no key at all
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float corr = m_new == m_ref ? 1.f : fast_exp2((m_ref - m_safe) * sl);     // m_ref = -inf: 0
        m_ref = m_new;
        l_run *= corr;
        if (j > 0) {                                    // O holds the tiles before this one: scale its row
#pragma unroll 1
          for (int c = 0; c < D / 16; ++c) {            // (a rare path: short, rolled, few registers)
            uint32_t ov[16];
            tmem_ld_32x16(t_o + (uint32_t)(c * 16), ov);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
            tmem_st_32x16(t_o + (uint32_t)(c * 16), ov);
          }
        }
      }
      const float neg_ms = m_ref == -INFINITY ? 0.f : -m_ref * sl;

      // P = exp2(s * sl - m * sl), row sum, packed 16-bit pairs into the first half of S
      float ps[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) ps[i] = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[c][i]), sl, neg_ms));       // masked: exp2(-inf) = 0
          const float p1 = fast_exp2(fmaf(__uint_as_float(v[c][i + 1]), sl, neg_ms));
          ps[i & 7] += p0;
          ps[(i & 7) + 1] += p1;
          pk[i / 2] = pack2<BF16>(p0, p1);
        }
        tmem_st_32x16(t_s + (uint32_t)(c * 16), pk);
      }
      const float psum = ((ps[0] + ps[1]) + (ps[2] + ps[3])) + ((ps[4] + ps[5]) + (ps[6] + ps[7]));
      l_run += psum;
      tmem_st_wait();
      tc::fence_before_sync();
      tc::mbar_arrive(tc::smem_u32(&bar_p_ready[w]));
    }

    if (ok && n > 0) {
      const bool f3 = !tc::mbar_wait(tc::smem_u32(&bar_o_full[w]), 0u, abort);
      if (!tc::named_barrier_or(1 + w, kRows, f3)) {
        tc::fence_after_sync();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint4* dst = reinterpret_cast<uint4*>(prm.out + ((long long)b * S + row) * prm.out_ts + (long long)hq * D);
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t ov[32];
          tc::tmem_ld_32x32(t_o + (uint32_t)(c * 32), ov);
          tc::tmem_ld_wait();
          if (row < S) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[c * 4 + i] = make_uint4(
                  pack2<BF16>(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv),
                  pack2<BF16>(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv),
                  pack2<BF16>(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv),
                  pack2<BF16>(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv));
          }
        }
      }
    }
  }

  // ------------------------------- teardown ---------------------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && abort_flag && prm.status) *prm.status = 1u;
}

// ---- host side -------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [B, S, H * d] 16-bit tensor with `ts` elements between tokens; box = 64 elements x 128 tokens of one
// sequence (tokens beyond S read as zero, never the next sequence's).
int make_token_map(CUtensorMap* map, const void* base, int64_t B, int64_t S, int64_t width, int64_t ts) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return set_error(LLMQRT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)width, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[2] = {(cuuint64_t)(ts * 2), (cuuint64_t)(S * ts * 2)};
  cuuint32_t box[3] = {64, (cuuint32_t)kRows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LLMQRT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LLMQRT_OK;
}

template <bool BF16, int D>
int launch_prefill(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, PrefillParams prm, int64_t B,
                   cudaStream_t st) {
  auto kern = attn_prefill_tc_kernel<BF16, D>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes<D>())) return rc;
  const uint32_t fmt = BF16 ? 1u : 0u;
  prm.idesc_s = tc::instr_desc(1, fmt, fmt, kRows, kRows);
  prm.idesc_pv = tc::instr_desc(1, fmt, fmt, kRows, D) | (1u << 16);       // bit 16: B operand is MN-major
  const dim3 grid((unsigned)ceil_div(prm.S, 2 * kRows), (unsigned)prm.Hq, (unsigned)B);
  kern<<<grid, kThreads, smem_bytes<D>(), st>>>(tq, tk, tv, prm);
  return check_launch("attn_prefill");
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
  LLMQRT_REQUIRE(q_token_stride % 8 == 0 && kv_token_stride % 8 == 0 && out_token_stride % 8 == 0 &&
                 q_token_stride >= Hq * d && kv_token_stride >= Hkv * d && out_token_stride >= Hq * d,
                 "attn_prefill: token strides must cover a token and be multiples of 8 elements");
  if (B == 0 || S == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(q && k && v && out, "attn_prefill: null pointer");
  LLMQRT_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                   reinterpret_cast<uintptr_t>(out)) & 15) == 0, "attn_prefill: pointers must be 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tq, tk, tv;
  if (int rc = make_token_map(&tq, q, B, S, Hq * d, q_token_stride)) return rc;
  if (int rc = make_token_map(&tk, k, B, S, Hkv * d, kv_token_stride)) return rc;
  if (int rc = make_token_map(&tv, v, B, S, Hkv * d, kv_token_stride)) return rc;
  PrefillParams prm{};
  prm.S = (int)S; prm.Hq = (int)Hq; prm.Hkv = (int)Hkv; prm.causal = causal;
  prm.scale = 1.0f / sqrtf((float)d);
  prm.softcap = softcap;
  prm.out = reinterpret_cast<uint16_t*>(out);
  prm.out_ts = out_token_stride;
  prm.status = nullptr;
  const bool bf = dtype == LLMQRT_BF16;
  if (d == 128) return bf ? launch_prefill<true, 128>(tq, tk, tv, prm, B, st) : launch_prefill<false, 128>(tq, tk, tv, prm, B, st);
  return bf ? launch_prefill<true, 64>(tq, tk, tv, prm, B, st) : launch_prefill<false, 64>(tq, tk, tv, prm, B, st);
}

