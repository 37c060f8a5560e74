// Dense GEMM on the 5th-generation tensor cores:  D[i, j] = sum_k P[i, k] * Q[j, k]
// for int8 (exact int32), fp8 e4m3/e5m2 and fp16/bf16 (fp32) operands, both K-major.
//
//   TMA (SWIZZLE_128B, 128-byte rows)  ->  shared-memory ring  ->  tcgen05.mma (M=128, N=BN)
//   ->  accumulator in tensor memory (double buffered)  ->  tcgen05.ld  ->  fused epilogue.
//
// P is the operand whose rows become the 128 TMEM lanes, Q the one whose rows become TMEM columns.
// For prefill-sized M the tokens are P and the weights Q.  For decode-sized M the roles are swapped
// (weights are P, the few tokens are Q with BN = 32/64/128), so the tile is never mostly padding and
// the kernel is a pure weight streamer; the reduction dimension is then split across thread blocks
// to occupy every SM, with partial sums in the workspace and a last-arriver fix-up.
//
// Warp roles (192 threads): warp 0 lane 0 issues TMA; warp 1 owns tensor memory and its lane 0
// issues the MMAs; warps 2-5 run the epilogue (TMEM lane quadrant = warp id % 4).  All waits on
// mbarriers are bounded; a time-out raises a block-wide abort flag and a status word in the
// workspace, every role drains and the block frees its tensor memory before returning.
//
// No thread-block clusters and no multicast: every CTA fetches its own tiles.
#include "gemm_w8a8.cuh"
#include "tc_primitives.cuh"

#include <mutex>
#include <type_traits>

namespace llmqrt {
namespace {

constexpr int kThreads = 192;
constexpr int kBM = 128;           // rows of P per tile (UMMA M)
constexpr int kRowBytes = 128;     // bytes of K per stage row (one swizzle span)
constexpr int kSmemBudget = 200 * 1024;

struct TcParams {
  int rows_p, rows_q;              // extents of P and Q (M/N or N/M)
  int k_blocks;                    // ceil(K bytes / 128)
  int tiles_p, tiles_q, splits, kb_per_split;
  int swap;                        // 0: P = tokens (i -> m, j -> n); 1: P = weights (i -> n, j -> m)
  int M, N;
  uint32_t idesc;
  void* partials;
  int* counters;
  unsigned* status;                // set to 1 if a bounded wait ran out
  Epilogue epi;
};

template <int BN> constexpr int stage_bytes() { return (kBM + BN) * kRowBytes; }
template <int BN> constexpr int num_stages() {
  int s = (kSmemBudget - 1024) / stage_bytes<BN>();
  return s > 8 ? 8 : s;
}
template <int BN> constexpr uint32_t tmem_cols() { return 2 * BN < 32 ? 32 : 2 * BN; }

template <typename AccT> __device__ __forceinline__ AccT acc_from_bits(uint32_t b);
template <> __device__ __forceinline__ int acc_from_bits<int>(uint32_t b) { return (int)b; }
template <> __device__ __forceinline__ float acc_from_bits<float>(uint32_t b) { return __uint_as_float(b); }

__device__ __forceinline__ uint32_t pack16(float a, float b, int dtype) {
  if (dtype == LLMQRT_F16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int KIND, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_q, TcParams prm) {
  using AccT = typename std::conditional<KIND == tc::MMA_I8, int, float>::type;
  constexpr int kStages = num_stages<BN>();
  constexpr int kStageBytes = stage_bytes<BN>();
  constexpr uint32_t kTmemCols = tmem_cols<BN>();

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern and the descriptors assume.
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int s_ticket;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &abort_flag;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(tc::smem_u32(&bar_full[s]), 1);
      tc::mbar_init(tc::smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(tc::smem_u32(&bar_acc_full[b]), 1);
      tc::mbar_init(tc::smem_u32(&bar_acc_empty[b]), 128);
    }
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&tm_p);
    tc::tma_prefetch_descriptor(&tm_q);
  }
  if (warp == 1) {
    tc::tmem_alloc(tc::smem_u32(&tmem_base_slot), kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  const int num_work = prm.tiles_p * prm.tiles_q * prm.splits;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;                 // loads issued in total (for draining on abort)
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int split = w % prm.splits;
        const int tile = w / prm.splits;
        const int tq = tile % prm.tiles_q, tp = tile / prm.tiles_q;
        const int kb0 = split * prm.kb_per_split;
        const int kb1 = min(kb0 + prm.kb_per_split, prm.k_blocks);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc::mbar_wait(tc::smem_u32(&bar_empty[stage]), phase ^ 1u, abort)) { ok = false; break; }
          const uint32_t full = tc::smem_u32(&bar_full[stage]);
          uint8_t* sp = tiles + stage * kStageBytes;
          tc::mbar_arrive_expect_tx(full, kStageBytes);
          // x coordinate in ELEMENTS of the tensor map's type; the maps are built on bytes for the
          // 8-bit kinds and on 16-bit elements for fp16/bf16.
          const int x = kb * (KIND == tc::MMA_F16 ? kRowBytes / 2 : kRowBytes);
          tc::tma_load_2d(tc::smem_u32(sp), &tm_p, full, x, tp * kBM);
          tc::tma_load_2d(tc::smem_u32(sp + kBM * kRowBytes), &tm_q, full, x, tq * BN);
          ++issued;
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Drain: every load that was issued completes on its full barrier; wait for the most recent
        // `min(issued, kStages)` of them (bounded) so that no copy is in flight when the block exits.
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < min(issued, kStages); ++i) {
          if (--s < 0) { s = kStages - 1; ph ^= 1u; }
          const uint64_t t0 = tc::global_timer_ns();
          while (!tc::mbar_try_wait(tc::smem_u32(&bar_full[s]), ph) &&
                 tc::global_timer_ns() - t0 < tc::kWaitLimitNs) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int split = w % prm.splits;
        const int kb0 = split * prm.kb_per_split;
        const int kb1 = min(kb0 + prm.kb_per_split, prm.k_blocks);
        if (!tc::mbar_wait(tc::smem_u32(&bar_acc_empty[buf]), acc_phase[buf] ^ 1u, abort)) { ok = false; break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!tc::mbar_wait(tc::smem_u32(&bar_full[stage]), phase, abort)) { ok = false; break; }
          tc::fence_after_sync();
          const uint32_t sp = tc::smem_u32(tiles + stage * kStageBytes);
          const uint64_t dp = tc::smem_desc_k_major_sw128(sp);
          const uint64_t dq = tc::smem_desc_k_major_sw128(sp + kBM * kRowBytes);
#pragma unroll
          for (int j = 0; j < kRowBytes / 32; ++j) {
            // 32 bytes of K per instruction (32 8-bit or 16 16-bit elements): +2 in the >>4 address field.
            tc::mma_ss<KIND>(d_tmem, dp + (uint64_t)(2 * j), dq + (uint64_t)(2 * j), prm.idesc,
                             (kb > kb0 || j > 0) ? 1u : 0u);
          }
          tc::mma_commit(tc::smem_u32(&bar_empty[stage]));      // frees the stage once the MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc::mma_commit(tc::smem_u32(&bar_acc_full[buf]));        // accumulator complete
        acc_phase[buf] ^= 1u;
        buf ^= 1;
      }
    }
  } else {
    // ------------------------------- epilogue -----------------------------------
    const int quad = warp & 3;                         // TMEM lane quadrant this warp may read
    const int et = quad * 32 + lane;                   // row of the tile handled by this thread
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    const Epilogue& epi = prm.epi;
    const float alpha = epi.alpha_dev ? *epi.alpha_dev : epi.alpha;
    AccT* part = reinterpret_cast<AccT*>(prm.partials);

    for (int w = blockIdx.x; w < num_work; w += gridDim.x) {
      const int split = w % prm.splits;
      const int tile = w / prm.splits;
      const int tq = tile % prm.tiles_q, tp = tile / prm.tiles_q;
      // The four epilogue warps must agree on leaving the loop: OR the failure over all 128 threads.
      const bool failed = !tc::mbar_wait(tc::smem_u32(&bar_acc_full[buf]), acc_phase[buf], abort);
      if (tc::named_barrier_or(2, 128, failed)) break;
      tc::fence_after_sync();
      acc_phase[buf] ^= 1u;

      const int i = tp * kBM + et;                     // global row of P
      const bool row_ok = i < prm.rows_p;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);

#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tc::tmem_ld_32x32(taddr + (uint32_t)c0, r);
        tc::tmem_ld_wait();
        const int j0 = tq * BN + c0;                   // global row of Q for r[0]
        if (j0 >= prm.rows_q) continue;                // warp-uniform
        if (prm.splits > 1) {
          // partial sums, layout [split][M][N]
          AccT* mine = part + (int64_t)split * prm.M * prm.N;
          if (row_ok) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const int j = j0 + jj;
              if (j < prm.rows_q) {
                const int64_t m = prm.swap ? j : i, n = prm.swap ? i : j;
                mine[m * prm.N + n] = acc_from_bits<AccT>(r[jj]);
              }
            }
          }
        } else if (prm.swap) {
          // lane -> n (contiguous in memory), jj -> m: coalesced 16-bit stores across the warp
          if (row_ok) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const int j = j0 + jj;
              if (j < prm.rows_q) epilogue_store<AccT>(epi, acc_from_bits<AccT>(r[jj]), j, i, alpha);
            }
          }
        } else if (row_ok) {
          // thread -> m, jj -> 32 consecutive n: vector stores when aligned
          const bool vec = epi.mode != EPI_RAW && epi.out_dtype != LLMQRT_F32 && j0 + 32 <= prm.rows_q &&
                           (epi.ldo % 8 == 0) && ((reinterpret_cast<uintptr_t>(epi.out) & 15) == 0);
          if (vec) {
            uint32_t packed[16];
#pragma unroll
            for (int jj = 0; jj < 32; jj += 2) {
              const float v0 = epilogue_value(epi, (float)acc_from_bits<AccT>(r[jj]), i, j0 + jj, alpha);
              const float v1 = epilogue_value(epi, (float)acc_from_bits<AccT>(r[jj + 1]), i, j0 + jj + 1, alpha);
              packed[jj / 2] = pack16(v0, v1, epi.out_dtype);
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(epi.out) + (int64_t)i * epi.ldo + j0);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4)
              dst[q4] = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const int j = j0 + jj;
              if (j < prm.rows_q) epilogue_store<AccT>(epi, acc_from_bits<AccT>(r[jj]), i, j, alpha);
            }
          }
        }
      }
      // accumulator buffer may be overwritten by the next-but-one tile
      tc::fence_before_sync();
      tc::mbar_arrive(tc::smem_u32(&bar_acc_empty[buf]));
      buf ^= 1;

      if (prm.splits > 1) {
        // last arriver of this tile sums the slices in order and applies the epilogue
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) s_ticket = atomicAdd(&prm.counters[tile], 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = s_ticket == prm.splits - 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");   // s_ticket may be rewritten after this point
        if (last) {
          __threadfence();
          if (row_ok) {
            for (int jj = 0; jj < BN; ++jj) {
              const int j = tq * BN + jj;
              if (j >= prm.rows_q) break;
              const int64_t m = prm.swap ? j : i, n = prm.swap ? i : j;
              AccT sum = 0;
              for (int s = 0; s < prm.splits; ++s) sum += __ldcg(part + ((int64_t)s * prm.M + m) * prm.N + n);
              epilogue_store<AccT>(epi, sum, m, n, alpha);
            }
          }
          if (threadIdx.x == 64) prm.counters[tile] = 0;
        }
      }
    }
  }

  // ------------------------------- teardown ---------------------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem_base, kTmemCols);
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

// 2-D K-major operand [rows, K] with `ld` elements between rows; box = 128 bytes x box_rows.
int make_operand_map(CUtensorMap* map, const void* base, int elt_bytes, int64_t rows, int64_t K, int64_t ld,
                     int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return set_error(LLMQRT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld * elt_bytes)};
  cuuint32_t box[2] = {(cuuint32_t)(kRowBytes / elt_bytes), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, elt_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LLMQRT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LLMQRT_OK;
}

template <int KIND, int BN>
int launch(const CUtensorMap& tm_p, const CUtensorMap& tm_q, const TcParams& prm, int grid, cudaStream_t st) {
  constexpr int smem = num_stages<BN>() * stage_bytes<BN>() + 1024;
  auto kern = gemm_tc_kernel<KIND, BN>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem)) return rc;
  kern<<<grid, kThreads, smem, st>>>(tm_p, tm_q, prm);
  return check_launch("gemm_tc");
}

template <int KIND>
int launch_bn(int bn, const CUtensorMap& tm_p, const CUtensorMap& tm_q, const TcParams& prm, int grid,
              cudaStream_t st) {
  switch (bn) {
    case 32: return launch<KIND, 32>(tm_p, tm_q, prm, grid, st);
    case 64: return launch<KIND, 64>(tm_p, tm_q, prm, grid, st);
    case 128: return launch<KIND, 128>(tm_p, tm_q, prm, grid, st);
    default: return launch<KIND, 256>(tm_p, tm_q, prm, grid, st);
  }
}

}  // namespace

int gemm_tc(int kind, const void* A, int64_t lda, const void* W, int64_t ldw, int64_t M, int64_t N, int64_t K,
            const Epilogue& epi, void* workspace, cudaStream_t st) {
  const int elt = (kind == KIND_F16 || kind == KIND_BF16) ? 2 : 1;
  LLMQRT_REQUIRE((K * elt) % 16 == 0 && (lda * elt) % 16 == 0 && (ldw * elt) % 16 == 0,
                 "tcgen05 gemm: K and leading dimensions must cover multiples of 16 bytes");
  LLMQRT_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0,
                 "tcgen05 gemm: operands must be 16-byte aligned");

  TcParams prm{};
  prm.M = (int)M;
  prm.N = (int)N;
  prm.epi = epi;
  prm.swap = M <= 128 ? 1 : 0;
  int bn;
  if (prm.swap) bn = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  else bn = N <= 128 ? 128 : 256;
  prm.rows_p = prm.swap ? (int)N : (int)M;
  prm.rows_q = prm.swap ? (int)M : (int)N;
  prm.k_blocks = (int)ceil_div(K * elt, kRowBytes);
  prm.tiles_p = (int)ceil_div(prm.rows_p, kBM);
  prm.tiles_q = (int)ceil_div(prm.rows_q, bn);

  const int sms = sm_count();
  const int tiles = prm.tiles_p * prm.tiles_q;
  int splits = 1;
  if (tiles < sms && workspace) {
    splits = sms / tiles;
    const int max_by_k = prm.k_blocks / 4 > 0 ? prm.k_blocks / 4 : 1;      // at least 4 K blocks per slice
    if (splits > max_by_k) splits = max_by_k;
    while (splits > 1 && (size_t)splits * M * N * 4 > LLMQRT_WS_PARTIAL_BYTES) --splits;
    if (tiles > LLMQRT_WS_NUM_COUNTERS) splits = 1;
  }
  prm.kb_per_split = (int)ceil_div(prm.k_blocks, splits);
  prm.splits = (int)ceil_div(prm.k_blocks, prm.kb_per_split);               // no empty slice
  prm.partials = workspace ? ws_partials(workspace) : nullptr;
  prm.counters = workspace ? ws_counters(workspace) : nullptr;
  prm.status = workspace ? ws_scalars(workspace) + 1 : nullptr;

  // A/B formats of the instruction follow P/Q.
  uint32_t fmt_act = 0, fmt_w = 0, c_fmt = 1;
  int mk = tc::MMA_F8;
  if (kind == KIND_I8) { mk = tc::MMA_I8; fmt_act = fmt_w = 1; c_fmt = 2; }
  else if (kind == KIND_F8_E5M2) { fmt_act = 1; }
  else if (kind == KIND_F16) { mk = tc::MMA_F16; }
  else if (kind == KIND_BF16) { mk = tc::MMA_F16; fmt_act = fmt_w = 1; }
  prm.idesc = tc::instr_desc(c_fmt, prm.swap ? fmt_w : fmt_act, prm.swap ? fmt_act : fmt_w, kBM, (uint32_t)bn);

  CUtensorMap tm_p, tm_q;
  const void* p_base = prm.swap ? W : A;
  const void* q_base = prm.swap ? A : W;
  if (int rc = make_operand_map(&tm_p, p_base, elt, prm.rows_p, K, prm.swap ? ldw : lda, kBM)) return rc;
  if (int rc = make_operand_map(&tm_q, q_base, elt, prm.rows_q, K, prm.swap ? lda : ldw, bn)) return rc;

  const int work = tiles * prm.splits;
  const int grid = work < sms ? work : sms;
  if (mk == tc::MMA_I8) return launch_bn<tc::MMA_I8>(bn, tm_p, tm_q, prm, grid, st);
  if (mk == tc::MMA_F8) return launch_bn<tc::MMA_F8>(bn, tm_p, tm_q, prm, grid, st);
  return launch_bn<tc::MMA_F16>(bn, tm_p, tm_q, prm, grid, st);
}

}  // namespace llmqrt
