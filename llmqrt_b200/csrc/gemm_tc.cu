// Dense GEMM on the 5th-generation tensor cores:  D[i, j] = sum_k P[i, k] * Q[j, k]
// for int8 (exact int32), fp8 e4m3/e5m2 and fp16/bf16 (fp32) operands, both K-major.
//
//   TMA (SWIZZLE_128B, 128-byte rows)  ->  shared-memory ring  ->  tcgen05.mma (M=128, N=BN)
//   ->  accumulator in tensor memory (double buffered)  ->  tcgen05.ld  ->  fused epilogue.
//
// P is the operand whose rows become the 128 TMEM lanes, Q the one whose rows become TMEM columns.
// For prefill-sized M the tokens are P and the weights Q.  For decode-sized M the roles are swapped
// (weights are P, the few tokens are Q with BN = 32/64/128), so the tile is never mostly padding and
// the kernel is a pure weight streamer.
//
// Split-K for skinny problems: when there are fewer tiles than SMs, the reduction dimension of a tile
// is divided among the 2 to 8 CTAs of a thread-block CLUSTER.  Each CTA accumulates its K range in
// tensor memory, then the cluster reduce-scatters through distributed shared memory: CTA r owns
// about BN/S accumulator columns (whole groups of eight), every CTA bulk-copies its slice of those columns into r's shared memory
// after one cluster barrier, r adds the S contributions in rank order (deterministic) and runs the
// epilogue; peers are released by remote mbarrier arrivals instead of a second cluster barrier.  No
// global scratch, no atomics, no second kernel.
//
// Launched with programmatic dependent launch: when the caller declares the weights static (constants
// of the model), the block's first ring of WEIGHT tiles is requested before griddepcontrol.wait and
// only the activation tiles after it; otherwise every tile waits.
//
// Warp roles (192 threads): warp 0 lane 0 issues TMA; warp 1 owns tensor memory and its lane 0
// issues the MMAs; warps 2-5 run the epilogue (TMEM lane quadrant = warp id % 4).  All waits on
// mbarriers are bounded; a time-out raises a block-wide abort flag and a status word in the
// workspace, every role drains and the block frees its tensor memory before returning.
//
// Epilogue: accumulators go TMEM -> registers, the scales / bias are applied there (the per-column
// ones come from a small shared-memory vector loaded once per tile), the 16-bit results are staged in
// shared memory and leave for global memory as 16-byte vectors that are contiguous across lanes.
//
// No multicast anywhere: every CTA fetches its own tiles with plain TMA loads.
//
// Two relatives of this kernel live further down: gemm_tc_pair_kernel, the two-CTA (cta_group::2) form
// for prefill-sized M, and the PUSH instantiation of this one, whose epilogue delivers the output rows of
// a row-parallel layer straight into the other GPUs' all-reduce buffers.
#include "gemm_w8a8.cuh"
#include "peer_comm.cuh"
#include "tc_primitives.cuh"

#include <map>
#include <mutex>
#include <type_traits>

namespace llmqrt {
namespace {

constexpr int kThreads = 192;
constexpr int kAwqWarps = 8;                  // warps that dequantize the 4-bit weight tiles (two per scheduler)
constexpr int kThreadsAwq = kThreads + kAwqWarps * 32;
constexpr int kBM = 128;           // rows of P per tile (UMMA M)
constexpr int kRowBytes = 128;     // bytes of K per stage row (one swizzle span)
constexpr int kSmemBudget = 226 * 1024;   // of the 227 KiB a block may use
constexpr int kChunk = 32;         // accumulator columns handled per epilogue step
constexpr int kEpiStageBytes = 18 * 1024;  // staging tile for one chunk (worst case 128 x 32 x 4 B + padding)

struct TcParams {
  int rows_p, rows_q;              // extents of P and Q (M/N or N/M)
  int k_blocks;                    // ceil(K bytes / 128)
  int tiles_p, tiles_q, splits;    // splits == cluster size along K (1 .. 8)
  int swap;                        // 0: P = tokens (i -> m, j -> n); 1: P = weights (i -> n, j -> m)
  int early_w;                     // weight tiles of the first ring may be requested before the dependency wait
  int M, N;
  uint32_t idesc;
  unsigned* status;                // set to 1 if a bounded wait ran out
  Epilogue epi;
  // AWQ mode: the weight operand is not fetched by TMA but produced in shared memory by four extra
  // warps from the packed 4-bit layer (wq_t [N, K/8] words of eight K-consecutive values, sz_t
  // [N, K/G] half2 {scale, -(1024 + zero)}, see awq.cu)
  const uint32_t* awq_w;
  const uint32_t* awq_sz;
  int awq_kw, awq_kg, awq_g;       // K / 8, K / G, G
  // Row-parallel output under tensor parallelism: instead of going to `out`, the 16-bit results are
  // stored as the tagged words of the NEXT all-reduce call into the peers' buffers (peer_comm.cuh);
  // the row kernel that consumes the sum then only gathers.
  int store32;                     // two-CTA kernel: output rows are 32-byte aligned, 256-bit stores may be used
  int comm_on, comm_threads, comm_two_step;
  CommDev comm;
};

template <int BN> constexpr int stage_bytes() { return (kBM + BN) * kRowBytes; }
template <int BN> constexpr int num_stages() {
  // The decode-sized tiles (BN <= 128) leave about 28 KiB of the SM's shared memory unclaimed, so that
  // blocks of the small kernel that precedes the GEMM in a chain can share the SM with a GEMM block
  // that has been launched early and is streaming its first weights.
  constexpr int budget = BN > 128 ? kSmemBudget : 200 * 1024;
  int s = (budget - 1024 - kEpiStageBytes) / stage_bytes<BN>();
  return s > 8 ? 8 : s;
}
template <int BN> constexpr int smem_bytes() { return num_stages<BN>() * stage_bytes<BN>() + kEpiStageBytes + 1024; }
// AWQ mode (always with the weights as the 128-lane operand): every stage also holds the PACKED 4-bit
// weight tile (32 bytes = 64 values of K per row, 128 rows) that TMA delivers and the dequantizing warps
// expand into the stage's fp16 weight tile.  The output is 16-bit and transposed through a 32 x 128
// staging tile, so the staging area is half the general one -- which buys the 256-token tile a fourth
// pipeline stage.
constexpr int kPackedRowBytes = 32;
constexpr int kPackedBytes = kBM * kPackedRowBytes;
constexpr int kEpiStageBytesAwq = 9 * 1024;            // kChunk rows x (128 x 2 B + 16 B pad)
template <int BN> constexpr int num_stages_awq() {
  constexpr int budget = BN > 128 ? kSmemBudget : 200 * 1024;
  int s = (budget - 1024 - kEpiStageBytesAwq) / (stage_bytes<BN>() + kPackedBytes);
  return s > 8 ? 8 : s;
}
template <int BN> constexpr int smem_bytes_awq() {
  return num_stages_awq<BN>() * (stage_bytes<BN>() + kPackedBytes) + kEpiStageBytesAwq + 1024;
}
template <int BN, bool AWQ> constexpr int smem_bytes_of() { return AWQ ? smem_bytes_awq<BN>() : smem_bytes<BN>(); }
template <int BN> constexpr uint32_t tmem_cols() { return 2 * BN < 32 ? 32 : 2 * BN; }

template <typename AccT> __device__ __forceinline__ AccT acc_from_bits(uint32_t b);
template <> __device__ __forceinline__ int acc_from_bits<int>(uint32_t b) { return (int)b; }
template <> __device__ __forceinline__ float acc_from_bits<float>(uint32_t b) { return __uint_as_float(b); }
template <typename AccT> __device__ __forceinline__ uint32_t acc_to_bits(AccT v);
template <> __device__ __forceinline__ uint32_t acc_to_bits<int>(int v) { return (uint32_t)v; }
template <> __device__ __forceinline__ uint32_t acc_to_bits<float>(float v) { return __float_as_uint(v); }

__device__ __forceinline__ uint32_t pack16(float a, float b, int dtype) {
  if (dtype == LLMQRT_F16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// Bulk asynchronous copy of `bytes` from this CTA's shared memory to the same offsets' counterpart in
// CTA `cta_rank` of the cluster; completion is counted (complete_tx) on that CTA's mbarrier.
// dst_local / bar_local are addresses in THIS CTA's window; mapa translates them to the peer's.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_local, uint32_t src_local, uint32_t bytes,
                                                 uint32_t bar_local, uint32_t cta_rank) {
  uint32_t dst, bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(dst_local), "r"(cta_rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(bar_local), "r"(cta_rank));
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "r"(src_local), "r"(bytes), "r"(bar)
               : "memory");
}
// One arrival on the mbarrier at the same shared-memory offset in CTA `cta_rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_local, uint32_t cta_rank) {
  uint32_t bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(bar_local), "r"(cta_rank));
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Split mode: the BN accumulator columns are dealt out to the S CTAs of the cluster in groups of eight,
// as evenly as S allows (S need not divide BN / 8: a cluster of three owns 24 + 24 + 16 of 64 columns).
__device__ __forceinline__ int split_col_begin(int owner, int bn, int S) { return (owner * (bn / 8) / S) * 8; }

// ---- epilogue --------------------------------------------------------------------------------------
// Arithmetic of one output element.  `var` is the scale that changes with the accumulator column
// (Q side), `fix` the one that belongs to the thread's row (P side); `var_first` says which of the two
// the operator multiplies first (row scale first for the fp8 row-wise op, channel scale first for the
// int8 per-channel op).
struct EpiConsts {
  int mode;
  bool var_first, has_bias;
  float alpha, fix_scale, fix_bias;
};

__device__ __forceinline__ float epi_value(const EpiConsts& c, float acc, float var_scale, float var_bias, bool swap) {
  const float bias = swap ? c.fix_bias : var_bias;
  if (c.mode == EPI_TENSOR) return __fmaf_rn(c.alpha, acc, bias);        // bias already multiplied by beta
  const float s1 = c.var_first ? var_scale : c.fix_scale, s2 = c.var_first ? c.fix_scale : var_scale;
  const float v = __fmul_rn(__fmul_rn(acc, s1), s2);
  return c.has_bias ? __fadd_rn(v, bias) : v;
}

// Per-tile set-up: the Q-side scale / bias vectors go to shared memory, the P-side ones to registers.
__device__ __forceinline__ EpiConsts epi_setup(const TcParams& prm, float alpha, int i, int j_base, int ncols_q,
                                               int t, float* q_scale, float* q_bias) {
  const Epilogue& e = prm.epi;
  const bool scaled = e.mode == EPI_ROW_COL || e.mode == EPI_COL_ROW;
  const float bmul = e.mode == EPI_TENSOR ? e.beta : 1.f;
  for (int c = t; c < ncols_q; c += 128) {
    const int j = j_base + c;
    float s = 1.f, b = 0.f;
    if (j < prm.rows_q) {
      if (scaled) s = prm.swap ? e.row_scale[j] : e.col_scale[j];
      if (!prm.swap && e.bias && e.mode != EPI_RAW) b = __fmul_rn(bmul, load_as_f32(e.bias, j, e.bias_dtype));
    }
    q_scale[c] = s;
    q_bias[c] = b;
  }
  EpiConsts c;
  c.mode = e.mode;
  c.alpha = alpha;
  c.has_bias = e.bias != nullptr;
  c.var_first = (e.mode == EPI_ROW_COL) == (prm.swap != 0);
  c.fix_scale = 1.f;
  c.fix_bias = 0.f;
  if (i < prm.rows_p) {
    if (scaled) c.fix_scale = prm.swap ? e.col_scale[i] : e.row_scale[i];
    if (prm.swap && e.bias && e.mode != EPI_RAW) c.fix_bias = __fmul_rn(bmul, load_as_f32(e.bias, i, e.bias_dtype));
  }
  return c;
}

// Staging-tile geometry.  es = bytes per output element (2, or 4 for raw / fp32 output).
//   normal: [128 rows][kChunk cols] with a 16-byte pad per row; swap: [kChunk rows (m)][128 cols (n)] + pad.
__device__ __forceinline__ int stage_pitch(bool swap, int es) { return (swap ? kBM : kChunk) * es + 16; }

// Phase 1, eight accumulator columns at a time (kept short: this code runs cold, see the header):
// apply the epilogue to r[0..8) = row `et`, columns c .. c+7 of the current chunk (q_scale / q_bias
// already point at column c) and park the results in the staging tile.
template <typename AccT>
__device__ __forceinline__ void epi_stage_group8(const TcParams& prm, const EpiConsts& ec, const uint32_t (&r)[8],
                                                 const float* q_scale, const float* q_bias, int c, int et,
                                                 uint8_t* stage) {
  const Epilogue& e = prm.epi;
  const bool raw = e.mode == EPI_RAW, swap = prm.swap != 0;
  const int es = (raw || e.out_dtype == LLMQRT_F32) ? 4 : 2;
  const int pitch = stage_pitch(swap, es);
  uint32_t w[8];
  if (raw) {
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) w[jj] = r[jj];
  } else {
    const float4 s0 = *reinterpret_cast<const float4*>(q_scale), s1 = *reinterpret_cast<const float4*>(q_scale + 4);
    const float4 b0 = *reinterpret_cast<const float4*>(q_bias), b1 = *reinterpret_cast<const float4*>(q_bias + 4);
    const float qs[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const float qb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int jj = 0; jj < 8; ++jj)
      w[jj] = __float_as_uint(epi_value(ec, (float)acc_from_bits<AccT>(r[jj]), qs[jj], qb[jj], swap));
  }
  if (swap) {
    // element jj goes to staged row c + jj, column et: scalar stores, contiguous across lanes
    if (es == 4) {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) *reinterpret_cast<uint32_t*>(stage + (c + jj) * pitch + et * 4) = w[jj];
    } else {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj)
        *reinterpret_cast<uint16_t*>(stage + (c + jj) * pitch + et * 2) =
            (uint16_t)pack16(__uint_as_float(w[jj]), 0.f, e.out_dtype);
    }
  } else if (es == 4) {
    uint4* dst = reinterpret_cast<uint4*>(stage + et * pitch + c * 4);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    *reinterpret_cast<uint4*>(stage + et * pitch + c * 2) =
        make_uint4(pack16(__uint_as_float(w[0]), __uint_as_float(w[1]), e.out_dtype),
                   pack16(__uint_as_float(w[2]), __uint_as_float(w[3]), e.out_dtype),
                   pack16(__uint_as_float(w[4]), __uint_as_float(w[5]), e.out_dtype),
                   pack16(__uint_as_float(w[6]), __uint_as_float(w[7]), e.out_dtype));
  }
}

// The same for the case every decode step runs four times per layer -- swapped roles, scaled epilogue,
// 16-bit output -- with the run-time choices of the general version (mode, order of the two scales,
// bias, output type) made once per group instead of once per element: the epilogue of a narrow GEMM
// is a short single pass per block, bound by its instruction count.
template <typename AccT, bool BF16, bool VAR_FIRST, bool HAS_BIAS>
__device__ __forceinline__ void epi_stage_group8_swap16(const EpiConsts& ec, const uint32_t (&r)[8],
                                                        const float* q_scale, int c, int et, uint8_t* stage) {
  constexpr int pitch = kBM * 2 + 16;                  // stage_pitch(swap = true, es = 2)
  const float4 s0 = *reinterpret_cast<const float4*>(q_scale), s1 = *reinterpret_cast<const float4*>(q_scale + 4);
  const float qs[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  uint8_t* p = stage + c * pitch + et * 2;             // element jj goes to staged row c + jj, column et
#pragma unroll
  for (int jj = 0; jj < 8; ++jj) {
    const float acc = (float)acc_from_bits<AccT>(r[jj]);
    float v = VAR_FIRST ? __fmul_rn(__fmul_rn(acc, qs[jj]), ec.fix_scale) : __fmul_rn(__fmul_rn(acc, ec.fix_scale), qs[jj]);
    if (HAS_BIAS) v = __fadd_rn(v, ec.fix_bias);       // swapped roles: the bias belongs to this lane's channel
    uint16_t bits;
    if constexpr (BF16) bits = __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else bits = __half_as_ushort(__float2half_rn(v));
    *reinterpret_cast<uint16_t*>(p + jj * pitch) = bits;
  }
}

template <typename AccT>
__device__ __forceinline__ void epi_stage_group8_any(const TcParams& prm, const EpiConsts& ec, const uint32_t (&r)[8],
                                                     const float* q_scale, const float* q_bias, int c, int et,
                                                     uint8_t* stage) {
  const Epilogue& e = prm.epi;
  if (prm.swap && (e.mode == EPI_ROW_COL || e.mode == EPI_COL_ROW) && e.out_dtype != LLMQRT_F32) {
    const int sel = (e.out_dtype == LLMQRT_BF16 ? 4 : 0) | (ec.var_first ? 2 : 0) | (ec.has_bias ? 1 : 0);
    switch (sel) {
      case 0: return epi_stage_group8_swap16<AccT, false, false, false>(ec, r, q_scale, c, et, stage);
      case 1: return epi_stage_group8_swap16<AccT, false, false, true>(ec, r, q_scale, c, et, stage);
      case 2: return epi_stage_group8_swap16<AccT, false, true, false>(ec, r, q_scale, c, et, stage);
      case 3: return epi_stage_group8_swap16<AccT, false, true, true>(ec, r, q_scale, c, et, stage);
      case 4: return epi_stage_group8_swap16<AccT, true, false, false>(ec, r, q_scale, c, et, stage);
      case 5: return epi_stage_group8_swap16<AccT, true, false, true>(ec, r, q_scale, c, et, stage);
      case 6: return epi_stage_group8_swap16<AccT, true, true, false>(ec, r, q_scale, c, et, stage);
      default: return epi_stage_group8_swap16<AccT, true, true, true>(ec, r, q_scale, c, et, stage);
    }
  }
  epi_stage_group8<AccT>(prm, ec, r, q_scale, q_bias, c, et, stage);
}

// Phase 2: staged block D[i0 .. i0+128, j0 .. j0+ncols) -> global memory, 16 bytes per thread and step.
template <bool PUSH = false>
__device__ __forceinline__ void epi_drain_chunk(const TcParams& prm, const uint8_t* stage, int ncols, int i0, int j0,
                                                int t, unsigned comm_seq = 0u, bool comm_live = false) {
  const Epilogue& e = prm.epi;
  if constexpr (PUSH) {
    // (swapped roles, 16-bit output, N a multiple of 8: checked on the host) a staged row is one token m
    // with 128 channels; a 16-byte vector is unit u = n / 8 of the token's row and becomes two tagged words
    if (!comm_live) return;                            // the communicator's status is raised: the consumer skips the sum
    const CommDev& c = prm.comm;
    const int rows_per_rank = (prm.M + c.world - 1) / c.world;
#pragma unroll 1
    for (int idx = t; idx < ncols * (kBM / 8); idx += 128) {
      const int sr = idx / (kBM / 8), sv = idx - sr * (kBM / 8);
      const int m = j0 + sr, n = i0 + sv * 8;
      if (m >= prm.M || n >= prm.N) continue;
      const uint4 val = *reinterpret_cast<const uint4*>(stage + sr * stage_pitch(true, 2) + sv * 16);
      const long long w0 = comm_word0(m, n >> 3, prm.comm_threads);
      if (prm.comm_two_step) {
        const int owner = min(m / rows_per_rank, c.world - 1);
        comm_push_one(c, comm_seq, owner, c.rank, w0, make_uint2(val.x, val.y));
        comm_push_one(c, comm_seq, owner, c.rank, w0 + 32, make_uint2(val.z, val.w));
      } else {
#pragma unroll 1
        for (int p = 0; p < c.world; ++p) {            // (rolled: this path must stay light on registers)
          comm_push_one(c, comm_seq, p, c.rank, w0, make_uint2(val.x, val.y));
          comm_push_one(c, comm_seq, p, c.rank, w0 + 32, make_uint2(val.z, val.w));
        }
      }
    }
    return;
  }
  const int es = (e.mode == EPI_RAW || e.out_dtype == LLMQRT_F32) ? 4 : 2;
  const int per = 16 / es;                             // elements per 16-byte vector
  const int pitch = stage_pitch(prm.swap != 0, es);
  uint8_t* out = reinterpret_cast<uint8_t*>(e.out);
  const bool base_ok = (reinterpret_cast<uintptr_t>(e.out) & 15) == 0 && (e.ldo % per) == 0;
  // staged rows x vectors per staged row; in swap mode a staged row is one m with 128 n
  const int srows = prm.swap ? ncols : kBM;
  const int vec_per_row = (prm.swap ? kBM : kChunk) / per;
  const int row_limit = prm.M, col_limit = prm.N;
#pragma unroll 1
  for (int idx = t; idx < srows * vec_per_row; idx += 128) {
    const int sr = idx / vec_per_row, sv = idx - sr * vec_per_row;
    const int m = prm.swap ? j0 + sr : i0 + sr;
    const int n = (prm.swap ? i0 : j0) + sv * per;
    const int n_end = prm.swap ? col_limit : min(col_limit, j0 + ncols);
    if (m >= row_limit || n >= n_end) continue;
    const uint4 val = *reinterpret_cast<const uint4*>(stage + sr * pitch + sv * 16);
    uint8_t* dst = out + ((int64_t)m * e.ldo + n) * es;
    if (base_ok && n + per <= n_end && (n % per) == 0) {
      *reinterpret_cast<uint4*>(dst) = val;
    } else {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(&val);
      for (int k = 0; k < per && n + k < n_end; ++k)
        for (int b = 0; b < es; ++b) dst[k * es + b] = src[k * es + b];
    }
  }
}

// PUSH: the output rows go into the peers' all-reduce buffers (a kernel of its own: the pushing
// epilogue needs 114 registers per thread against 67, and the register budget of a decode GEMM decides
// whether its blocks can become resident, and fetch their first weights, beside the blocks of the
// kernel before it -- with the push compiled into the common kernel the decode step lost 3.7 %).
template <int KIND, int BN, bool AWQ = false, bool PUSH = false>
__global__ void __launch_bounds__(AWQ ? kThreadsAwq : kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_p, const __grid_constant__ CUtensorMap tm_q,
               const __grid_constant__ CUtensorMap tm_w, TcParams prm) {
  static_assert(!AWQ || KIND == tc::MMA_F16, "the 4-bit weights dequantize to fp16");
  using AccT = typename std::conditional<KIND == tc::MMA_I8, int, float>::type;
  constexpr int kStages = AWQ ? num_stages_awq<BN>() : num_stages<BN>();
  constexpr int kStageBytes = stage_bytes<BN>();
  constexpr int kPkBytes = kPackedBytes;
  constexpr uint32_t kTmemCols = tmem_cols<BN>();
  constexpr int kBurst = kStages >= 8 ? 4 : (kStages >= 4 ? 2 : 1);  static_assert(BN > 128 || kStages * kStageBytes >= (2 * BN + 64) * kBM * 4, "ring too small for the reduce buffers");
  static_assert(kStages >= 3, "pipeline too shallow");

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern and the descriptors assume.
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage = tiles + kStages * kStageBytes;      // epilogue staging tile
  uint8_t* packed = stage + (AWQ ? kEpiStageBytesAwq : kEpiStageBytes);   // AWQ: [kStages][kPkBytes] packed weight tiles
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_pk[AWQ ? kStages : 1];   // AWQ: packed weight tile of the stage has landed
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ __align__(8) uint64_t bar_reduce;         // split mode: counts the bytes of the incoming slices
  __shared__ __align__(8) uint64_t bar_release;        // split mode: one arrival per peer that has received its slice
  __shared__ __align__(16) float q_scale[BN];
  __shared__ __align__(16) float q_bias[BN];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int cluster_abort;                        // split mode: set in every CTA of the cluster by one that failed
  __shared__ unsigned comm_seq_s;                      // push mode: the all-reduce call's sequence number ...
  __shared__ int comm_live_s;                          // ... and whether the communicator is healthy

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &abort_flag;
  const uint32_t abort_u32 = tc::smem_u32(&abort_flag);
  const int S = prm.splits;
  const int my_split = S > 1 ? (int)cluster_ctarank() : 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    cluster_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(tc::smem_u32(&bar_full[s]), AWQ ? 1 + kAwqWarps : 1);   // AWQ: + one arrival per dequantizing warp
      tc::mbar_init(tc::smem_u32(&bar_empty[s]), 1);
      if (AWQ) tc::mbar_init(tc::smem_u32(&bar_pk[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(tc::smem_u32(&bar_acc_full[b]), 1);
      tc::mbar_init(tc::smem_u32(&bar_acc_empty[b]), 128);
    }
    tc::mbar_init(tc::smem_u32(&bar_reduce), 1);
    tc::mbar_init(tc::smem_u32(&bar_release), (uint32_t)S);
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
  // Everything above touched only shared and tensor memory; from here on global memory is read.
  // The producer thread waits later: it first requests weight tiles, which the preceding kernel of
  // the stream does not write.
  if (threadIdx.x != 0) {
    pdl_wait();
    pdl_trigger();
  }
  if constexpr (PUSH) {
    if (threadIdx.x == 64) {                           // read by the epilogue warps after their first barrier
      unsigned sq;
      comm_live_s = comm_enter(prm.comm, &sq) ? 1 : 0;
      comm_seq_s = sq;
    }
  }

  // Work items: split mode -> exactly one tile per cluster (grid = tiles * S, non persistent);
  // otherwise a persistent walk over the tiles.
  const int num_tiles = prm.tiles_p * prm.tiles_q;
  const int first_tile = S > 1 ? (int)(blockIdx.x / S) : (int)blockIdx.x;
  const int tile_step = S > 1 ? num_tiles : (int)gridDim.x;      // split mode: one iteration
  // K range of this CTA (balanced, never empty because k_blocks >= 2 * S)
  const int kb_begin = (int)((int64_t)my_split * prm.k_blocks / S);
  const int kb_count = (int)((int64_t)(my_split + 1) * prm.k_blocks / S) - kb_begin;
  EpiConsts ec_split = {};           // split mode: set by the epilogue warps before they wait for the MMAs

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      int stage_i = 0;
      uint32_t phase = 0;
      bool ok = true;
      int issued = 0;
      // x coordinate in ELEMENTS of the tensor map's type; the maps are built on bytes for the
      // 8-bit kinds and on 16-bit elements for fp16/bf16.
      constexpr int kXPerBlock = KIND == tc::MMA_F16 ? kRowBytes / 2 : kRowBytes;
      // The weight operand is a constant of the model, so the first ring-full of weight tiles of the
      // first work item is requested BEFORE waiting for the preceding kernel of the stream; the
      // activation tiles of the same stages follow after the wait and complete the same barriers.
      // On a programmatic launch this streams up to a ring of weights per SM while the preceding
      // kernel is still running.  Only when the caller declared W a stored weight: a matrix that the
      // preceding kernel has just produced (a weight quantized on the fly, an AWQ layer dequantized
      // for a large M) must be waited for like the activations.
      const bool early_w = prm.early_w != 0;
      // AWQ: only the activation tile arrives by TMA (the weight tile is written by the dequantizing warps)
      const bool tma_p = !(AWQ && prm.swap != 0), tma_q = !(AWQ && prm.swap == 0);
      const uint32_t tx_bytes = AWQ ? (uint32_t)((prm.swap ? BN : kBM) * kRowBytes) : (uint32_t)kStageBytes;
      const uint32_t pk_bytes = (uint32_t)kPackedBytes;
      if (!early_w) {
        pdl_wait();
        pdl_trigger();
      }
      const int pre = first_tile < num_tiles ? min(kStages, kb_count) : 0;
      for (int phase_w = 1; phase_w >= 0; --phase_w) {     // 1: weights, 0: activations
        const int tq = first_tile % prm.tiles_q, tp = first_tile / prm.tiles_q;
        const int rot = pre ? (tp * 5 + tq * 3) % kb_count : 0;
        const bool load_p = (prm.swap != 0) == (phase_w != 0);
        for (int g = 0; g < pre; ++g) {
          int kr = g + rot;
          if (kr >= kb_count) kr -= kb_count;
          const int x = (kb_begin + kr) * kXPerBlock;
          const uint32_t full = tc::smem_u32(&bar_full[g]);
          uint8_t* sp = tiles + g * kStageBytes;
          if (phase_w) tc::mbar_arrive_expect_tx(full, tx_bytes);
          if (AWQ && phase_w) {                        // packed 4-bit tile: words 8 kb .. 8 kb + 7 of the tile's weight rows
            const uint32_t pk = tc::smem_u32(&bar_pk[g]);
            tc::mbar_arrive_expect_tx(pk, pk_bytes);
            tc::tma_load_2d(tc::smem_u32(packed + g * kPkBytes), &tm_w, pk, (kb_begin + kr) * 8, tp * kBM);
          }
          if (load_p) { if (tma_p) tc::tma_load_2d(tc::smem_u32(sp), &tm_p, full, x, tp * kBM); }
          else if (tma_q) tc::tma_load_2d(tc::smem_u32(sp + kBM * kRowBytes), &tm_q, full, x, tq * BN);
        }
        if (phase_w && early_w) {
          // (Prefetching further weight tiles into L2 here was measured to slow the kernel down: the
          // ring already keeps more bytes in flight than HBM needs, and the activation loads then
          // queue behind the prefetches.)
          pdl_wait();
          pdl_trigger();
        }
      }
      issued = pre;
      if (pre == kStages) phase = 1; else stage_i = pre;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        const int tq = tile % prm.tiles_q, tp = tile / prm.tiles_q;
        // Blocks start at different K offsets so that they do not all pull the same activation rows
        // out of L2 at the same moment; the accumulation order per tile stays fixed.
        const int rot = (tp * 5 + tq * 3) % kb_count;
        // K blocks are issued in bursts of kBurst consecutive blocks: the same weight rows are then
        // requested at consecutive 128-byte offsets within nanoseconds, which the DRAM controller can
        // serve from open pages (a lone 128-byte piece per row and visit is the worst case for HBM).
        for (int it0 = tile == first_tile ? pre : 0; it0 < kb_count && ok; it0 += kBurst) {
          const int nb = min(kBurst, kb_count - it0);
          int s_w = stage_i;
          uint32_t ph_w = phase;
          for (int g = 0; g < nb; ++g) {               // wait until all slots of the burst are free
            tc::mbar_wait_or_flag(tc::smem_u32(&bar_empty[s_w]), ph_w ^ 1u, abort_u32);
            if (++s_w == kStages) { s_w = 0; ph_w ^= 1u; }
          }
          if (*abort) { ok = false; break; }           // a wait ran out (here or in another role)
          for (int g = 0; g < nb; ++g) {
            int kr = it0 + g + rot;
            if (kr >= kb_count) kr -= kb_count;
            const int kb = kb_begin + kr;
            const uint32_t full = tc::smem_u32(&bar_full[stage_i]);
            uint8_t* sp = tiles + stage_i * kStageBytes;
            tc::mbar_arrive_expect_tx(full, tx_bytes);
            const int x = kb * kXPerBlock;
            if (AWQ) {
              const uint32_t pk = tc::smem_u32(&bar_pk[stage_i]);
              tc::mbar_arrive_expect_tx(pk, pk_bytes);
              tc::tma_load_2d(tc::smem_u32(packed + stage_i * kPkBytes), &tm_w, pk, kb * 8, tp * kBM);
            }
            if (tma_p) tc::tma_load_2d(tc::smem_u32(sp), &tm_p, full, x, tp * kBM);
            if (tma_q) tc::tma_load_2d(tc::smem_u32(sp + kBM * kRowBytes), &tm_q, full, x, tq * BN);
            ++issued;
            if (++stage_i == kStages) { stage_i = 0; phase ^= 1u; }
          }
        }
      }
      if (!ok) {
        // Drain: every load that was issued completes on its full barrier; wait (bounded) for the most
        // recent min(issued, kStages) of them so that no copy is in flight when the block exits.
        int s = stage_i;
        uint32_t ph = phase;
        for (int i = 0; i < min(issued, kStages); ++i) {
          if (--s < 0) { s = kStages - 1; ph ^= 1u; }
          const uint64_t t0 = tc::global_timer_ns();
          while (!tc::mbar_try_wait(tc::smem_u32(&bar_full[s]), ph) &&
                 tc::global_timer_ns() - t0 < tc::kWaitLimitNs) {}
          if (AWQ)
            while (!tc::mbar_try_wait(tc::smem_u32(&bar_pk[s]), ph) && tc::global_timer_ns() - t0 < tc::kWaitLimitNs) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------
    if (lane == 0) {
      int stage_i = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        if (!tc::mbar_wait(tc::smem_u32(&bar_acc_empty[buf]), acc_phase[buf] ^ 1u, abort)) { ok = false; break; }
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int it = 0; it < kb_count; ++it) {
          // No result and no tcgen05 fence here: the tiles were written by TMA, whose completion on
          // the barrier orders them before MMAs issued after the wait; the flag is checked per tile.
          tc::mbar_wait_or_flag(tc::smem_u32(&bar_full[stage_i]), phase, abort_u32);
          const uint32_t sp = tc::smem_u32(tiles + stage_i * kStageBytes);
          const uint64_t dp = tc::smem_desc_k_major_sw128(sp);
          const uint64_t dq = tc::smem_desc_k_major_sw128(sp + kBM * kRowBytes);
#pragma unroll
          for (int j = 0; j < kRowBytes / 32; ++j) {
            // 32 bytes of K per instruction (32 8-bit or 16 16-bit elements): +2 in the >>4 address field.
            tc::mma_ss<KIND>(d_tmem, dp + (uint64_t)(2 * j), dq + (uint64_t)(2 * j), prm.idesc,
                             (it > 0 || j > 0) ? 1u : 0u);
          }
          tc::mma_commit(tc::smem_u32(&bar_empty[stage_i]));    // frees the stage once the MMAs retire
          if (++stage_i == kStages) { stage_i = 0; phase ^= 1u; }
        }
        if (*abort) { ok = false; break; }
        tc::mma_commit(tc::smem_u32(&bar_acc_full[buf]));        // accumulator complete
        acc_phase[buf] ^= 1u;
        buf ^= 1;
      }
    }
  } else if (AWQ && warp >= 6) {
    // ------------------------------- AWQ weight producer -------------------------
    // 256 threads expand the packed 4-bit tile of every stage (delivered by TMA: 32 bytes = 64 values
    // of K per weight row, 128 rows) into the stage's fp16 weight tile: a thread owns half a row --
    // four packed words (eight values of K each) -> four 16-byte chunks of fp16, stored at the
    // 128-byte-swizzle positions a TMA load of fp16 weights would have used, then made visible to the
    // tensor core (async proxy) before the warp's arrival.  Two warps share a
    // scheduler so that one's arithmetic hides the other's latencies.  The {scale, zero} pair of the
    // row's quantization group is the only thing read from global memory here, kDepth blocks ahead.
    constexpr int kDepth = 4;
    const int t = (int)threadIdx.x - 6 * 32;
    const int rr = t & (kBM - 1);                      // my row of the 128-row weight tile
    const int j0 = 4 * (t >> 7);                       // my four of the row's eight words
    // prefetch cursor of the scale / zero pairs: walks the (tile, K block) sequence kDepth blocks ahead
    int pf_tile = first_tile, pf_it = 0, pf_rot = 0;
    const uint32_t* pf_z = nullptr;                    // my row's scale-zero pairs in the cursor's tile
    auto pf_enter_tile = [&]() {
      pf_z = nullptr;
      if (pf_tile >= num_tiles) return;
      const int tq = pf_tile % prm.tiles_q, tp = pf_tile / prm.tiles_q;
      pf_rot = (tp * 5 + tq * 3) % kb_count;           // the TMA producer's K rotation
      const int n = tp * kBM + rr;
      if (n < prm.N) pf_z = prm.awq_sz + (int64_t)n * prm.awq_kg;
    };
    uint32_t szv[kDepth];                              // {scale, -(1024 + zero)} of my 32 values (groups of >= 32 values)
    auto fetch = [&](uint32_t& z) {
      z = 0u;                                          // scale 0: rows outside the matrix and values beyond K dequantize to 0
      if (pf_z != nullptr) {
        int kr = pf_it + pf_rot;
        if (kr >= kb_count) kr -= kb_count;
        const int wi = (kb_begin + kr) * 8 + j0;       // my first word of this K block
        if (wi < prm.awq_kw) z = __ldg(pf_z + (wi * 8) / prm.awq_g);
      }
      if (++pf_it == kb_count) {                       // advance the cursor
        pf_it = 0;
        pf_tile += tile_step;
        pf_enter_tile();
      }
    };
    pf_enter_tile();
#pragma unroll
    for (int d = 0; d < kDepth; ++d) fetch(szv[d]);
    const int my_tiles = first_tile < num_tiles ? (num_tiles - first_tile + tile_step - 1) / tile_step : 0;
    const int total = my_tiles * kb_count;             // K blocks this CTA consumes, in ring order
    int stage_i = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int q0 = 0; q0 < total && ok; q0 += kDepth) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        if (q0 + d >= total || !ok) continue;
        // the packed tile has landed; the TMA thread requested it only after the stage's previous
        // contents had been consumed, so the fp16 tile may be overwritten as well
        tc::mbar_wait_or_flag(tc::smem_u32(&bar_pk[stage_i]), phase, abort_u32);
        if (*abort) { ok = false; continue; }
        {
          const uint4 a = *reinterpret_cast<const uint4*>(packed + stage_i * kPkBytes + rr * kPackedRowBytes + j0 * 4);
          uint4* dst = reinterpret_cast<uint4*>(tiles + stage_i * kStageBytes + rr * kRowBytes);
          const uint32_t words[4] = {a.x, a.y, a.z, a.w};
          const __half2 sz = *reinterpret_cast<const __half2*>(&szv[d]);
          const __half2 negz = __half2half2(__high2half(sz)), sc = __half2half2(__low2half(sz));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t o[4];
#pragma unroll
            for (int p4 = 0; p4 < 4; ++p4) {
              uint32_t h = ((words[j] >> (4 * p4)) & 0x000F000Fu) | 0x64006400u;         // {1024 + v[2p], 1024 + v[2p+1]}
              const __half2 v2 = __hmul2(__hadd2(*reinterpret_cast<__half2*>(&h), negz), sc);
              o[p4] = *reinterpret_cast<const uint32_t*>(&v2);
            }
            dst[(j0 + j) ^ (rr & 7)] = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(tc::smem_u32(&bar_full[stage_i]));
        if (++stage_i == kStages) { stage_i = 0; phase ^= 1u; }
        fetch(szv[d]);                                 // refill the slot for kDepth blocks ahead
      }
    }
  } else {
    // ------------------------------- epilogue -----------------------------------
    const int quad = warp & 3;                         // TMEM lane quadrant this warp may read
    const int et = quad * 32 + lane;                   // row of the tile handled by this thread
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    const float alpha = prm.epi.alpha_dev ? *prm.epi.alpha_dev : prm.epi.alpha;

    for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
      const int tq = tile % prm.tiles_q, tp = tile / prm.tiles_q;
      EpiConsts ec;
      if (S == 1) {
        epi_barrier();                                 // previous tile no longer reads q_scale / q_bias
        ec = epi_setup(prm, alpha, tp * kBM + et, tq * BN, BN, et, q_scale, q_bias);
      } else {
        // split mode: the scales of the columns this CTA owns, fetched while the MMAs still run
        const int col0 = split_col_begin(my_split, BN, S), cpo = split_col_begin(my_split + 1, BN, S) - col0;
        ec_split = epi_setup(prm, alpha, tp * kBM + et, tq * BN + col0, cpo, et, q_scale, q_bias);
      }
      // The four epilogue warps must agree on leaving the loop: OR the failure over all 128 threads.
      const bool failed = !tc::mbar_wait(tc::smem_u32(&bar_acc_full[buf]), acc_phase[buf], abort);
      if (tc::named_barrier_or(2, 128, failed)) break;
      tc::fence_after_sync();
      acc_phase[buf] ^= 1u;
      if (S > 1) break;                                // split mode: the reduce-scatter below takes over

      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kChunk) {
        const int j0 = tq * BN + c0;                   // global row of Q of the first column of the chunk
        if (j0 >= prm.rows_q) break;
        epi_barrier();                                 // staging tile drained by everyone
#pragma unroll 1
        for (int c = 0; c < kChunk; c += 8) {
          uint32_t r[8];
          tc::tmem_ld_32x8(taddr + (uint32_t)(c0 + c), r);
          tc::tmem_ld_wait();
          epi_stage_group8_any<AccT>(prm, ec, r, q_scale + c0 + c, q_bias + c0 + c, c, et, stage);
        }
        epi_barrier();
        epi_drain_chunk<PUSH>(prm, stage, min(kChunk, prm.rows_q - j0), tp * kBM, j0, et, PUSH ? comm_seq_s : 0u, PUSH && comm_live_s != 0);
      }
      // accumulator buffer may be overwritten by the next-but-one tile
      tc::fence_before_sync();
      tc::mbar_arrive(tc::smem_u32(&bar_acc_empty[buf]));
      buf ^= 1;
    }
  }

  // ------------------------------- cluster reduce-scatter (split mode) --------------------------
  if constexpr (BN <= 128) {
  if (S > 1) {
    // The pipeline ring is dead once a CTA's MMAs have retired.  It is reused as
    //   recv = ring[0, S * cpo_max * 512)   [source rank][owned column][128 rows] 32-bit words
    //   send = behind it, BN * 512 bytes    [accumulator column][128 rows]
    // Each CTA parks its accumulator in `send`, and after a cluster barrier (every ring dead) one
    // thread pushes slice o of `send` into `recv` of CTA o with a bulk shared->shared copy that
    // completes on o's `bar_reduce`.
    const int col0 = split_col_begin(my_split, BN, S);                 // accumulator columns owned by this CTA:
    const int cpo = split_col_begin(my_split + 1, BN, S) - col0;        // [col0, col0 + cpo)
    const uint32_t slice_bytes = (uint32_t)cpo * kBM * 4;              // what every CTA sends to this one
    const int cpo_max = ((BN / 8 + S - 1) / S) * 8;
    uint32_t* send = reinterpret_cast<uint32_t*>(tiles + S * cpo_max * kBM * 4);
    const bool own_healthy = abort_flag == 0;          // own MMAs finished (epilogue warps waited for them)
    const int quad = warp & 3, et = quad * 32 + lane;
    const bool epi_warp = warp >= 2 && warp < 6;       // (AWQ mode has more warps behind them)
    const int tq = first_tile % prm.tiles_q, tp = first_tile / prm.tiles_q;
    const EpiConsts& ec = ec_split;                    // q_scale / q_bias cover only the columns this CTA owns
    if (epi_warp && own_healthy) {
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
      // 32 columns per round trip to tensor memory (four loads in flight before the wait): the
      // wait, not the data volume, is what each round costs
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[4][8];
#pragma unroll
        for (int q = 0; q < 4; ++q) tc::tmem_ld_32x8(taddr + (uint32_t)(c0 + 8 * q), r[q]);
        tc::tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) send[(c0 + 8 * q + jj) * kBM + et] = r[q][jj];
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> bulk-copy reads
      if (threadIdx.x == 64) tc::mbar_arrive_expect_tx(tc::smem_u32(&bar_reduce), slice_bytes * (uint32_t)S);
    }
    // A CTA whose waits ran out tells every CTA of the cluster before the barrier, and then ALL of
    // them skip the exchange: nobody copies into, or arrives on a barrier of, a CTA that may have left.
    if (!own_healthy && threadIdx.x == 64) {
      for (int o = 0; o < S; ++o) {
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(tc::smem_u32(&cluster_abort)), "r"(o));
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(1u) : "memory");
      }
    }
    // Cluster barrier: every ring is dead, every `send` is complete, every `bar_reduce` is armed,
    // every failure flag has landed (release / acquire).
    __syncwarp();
    cluster_sync_all();
    const bool healthy = own_healthy && *reinterpret_cast<volatile int*>(&cluster_abort) == 0;
    if (!healthy && threadIdx.x == 64) abort_flag = 1;                 // reported through the status word at exit
    if (threadIdx.x == 64 && healthy) {
      for (int o = 0; o < S; ++o) {                   // owner o receives its columns of my accumulator
        const int ob = split_col_begin(o, BN, S);
        const uint32_t obytes = (uint32_t)(split_col_begin(o + 1, BN, S) - ob) * kBM * 4;
        bulk_copy_to_cta(tc::smem_u32(tiles) + (uint32_t)my_split * obytes, tc::smem_u32(send) + (uint32_t)ob * kBM * 4,
                         obytes, tc::smem_u32(&bar_reduce), (uint32_t)o);
      }
    }
    // Once every slice addressed to this CTA has landed, the peers' `send` buffers are no longer
    // being read on its behalf: tell each of them.  A CTA leaves once all S owners have said so, which
    // by then happened during its own epilogue -- no cluster barrier at the end.  Done by the otherwise
    // idle producer thread, which waits for the slices on its own: the remote arrivals take a few
    // hundred ns each and would hold up the epilogue warps.
    if (threadIdx.x == 0 && healthy && tc::mbar_wait(tc::smem_u32(&bar_reduce), 0u, abort)) {
      for (int o = 0; o < S; ++o) mbar_arrive_remote(tc::smem_u32(&bar_release), (uint32_t)o);
    }
    bool reduce_ok = false;
    if (epi_warp) {
      const bool failed = !healthy || !tc::mbar_wait(tc::smem_u32(&bar_reduce), 0u, abort);
      reduce_ok = !tc::named_barrier_or(2, 128, failed);
    }
    if (epi_warp && reduce_ok) {
      const AccT* rbuf = reinterpret_cast<const AccT*>(tiles);
#pragma unroll 1
      for (int c0 = 0; c0 < cpo; c0 += kChunk) {
        const int j0 = tq * BN + col0 + c0;
        if (j0 >= prm.rows_q) break;
        const int ncols = min(min(kChunk, cpo - c0), prm.rows_q - j0);
        epi_barrier();
#pragma unroll 1
        for (int c = 0; c < min(kChunk, cpo - c0); c += 8) {
          AccT sum[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) sum[jj] = 0;
#pragma unroll 1
          for (int s = 0; s < S; ++s) {                // rank order: deterministic
            const AccT* src = rbuf + (s * cpo + c0 + c) * kBM + et;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) sum[jj] += src[jj * kBM];
          }
          uint32_t r[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) r[jj] = acc_to_bits<AccT>(sum[jj]);
          epi_stage_group8_any<AccT>(prm, ec, r, q_scale + c0 + c, q_bias + c0 + c, c, et, stage);
        }
        epi_barrier();
        epi_drain_chunk<PUSH>(prm, stage, ncols, tp * kBM, j0, et, PUSH ? comm_seq_s : 0u, PUSH && comm_live_s != 0);
      }
    }
    // Nobody leaves while a peer may still be copying out of its `send` buffer (bounded: a peer that
    // failed never reports, and the block then gives up with the abort flag raised).
    if (threadIdx.x == 64 && healthy) tc::mbar_wait(tc::smem_u32(&bar_release), 0u, abort);
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


// ---- two-CTA kernel for prefill-sized problems -------------------------------------------------
// Tokens are the 128-lane operand.  The two CTAs of a cluster compute one 256 x 256 output tile with
// tcgen05.mma.cta_group::2 (M = 256, N = 256): each CTA stages ITS 128 token rows and ITS 128 of the
// tile's 256 weight rows, 32 KiB per K block of 128 bytes instead of the 48 KiB a lone CTA needs for a
// 128 x 256 tile, and each MMA reads 8 KiB instead of 12 KiB of a CTA's shared memory per 128 x 256 x 32
// multiply -- the shared-memory operand feed, not the tensor pipe, is what bounds the single-CTA form.
// Each CTA's tensor memory receives its 128 accumulator rows (2 x 256 columns, double buffered).
//   producer (warp 0, both CTAs): TMA loads whose bytes are counted on the LEADER's `full` barrier
//   MMA issuer (warp 1, leader only): 4 MMAs per stage, commits fan out to both CTAs' barriers
//   epilogue (warps 2-9, both CTAs): TMEM -> registers -> scales / bias -> global memory, 64 or 128
//     contiguous bytes per thread and step straight from registers (a staged TMA store was measured
//     three times slower with one staging tile: its completion latency of a few microseconds
//     serialises the chunks, and shared memory has no room for a deeper staging ring next to six stages)
constexpr int kPairBN = 256;
constexpr int kPairHalfB = kPairBN / 2;
constexpr int kPairStageBytes = (kBM + kPairHalfB) * kRowBytes;         // 32 KiB
constexpr int kPairStages = 6;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024;
constexpr uint32_t kPairTmemCols = 2 * kPairBN;
constexpr int kPairThreads = 64 + 256;                                 // producer warp, MMA warp, eight epilogue warps
__device__ __forceinline__ void pair_epi_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// 32 bytes from registers to global memory in one instruction (the address must be 32-byte aligned): half
// the store instructions, and every lane writes a whole 32-byte sector.
__device__ __forceinline__ void st_global_256(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t e,
                                              uint32_t f, uint32_t g, uint32_t h) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d), "r"(e),
               "r"(f), "r"(g), "r"(h) : "memory");
}

// Tile order: the weight tiles are walked in groups of kPairGroup; inside a group the token tile
// changes fastest.  The clusters that run at the same time then share a few weight tiles and a few
// token tiles, and a weight group (8 x 256 rows) stays in L2 until every token tile has used it -- with
// the weight tile changing fastest instead, a weight matrix larger than L2 (gate_up of Qwen2-7B: 136 MB)
// is streamed from HBM once per token tile.
constexpr int kPairGroup = 8;
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_p, int tiles_q, int& tp, int& tq) {
  const int per_group = tiles_p * kPairGroup;
  const int group = tile / per_group, within = tile - group * per_group;
  const int gw = min(kPairGroup, tiles_q - group * kPairGroup);         // weight tiles in this group
  tp = within / gw;
  tq = group * kPairGroup + within - tp * gw;
}

template <int KIND>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, TcParams prm) {
  using AccT = typename std::conditional<KIND == tc::MMA_I8, int, float>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar_full[kPairStages];      // used in the leader only
  __shared__ __align__(8) uint64_t bar_empty[kPairStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];           // used in the leader only: one arrival per CTA
  __shared__ __align__(16) float q_scale[kPairBN];
  __shared__ __align__(16) float q_bias[kPairBN];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &abort_flag;
  const uint32_t abort_u32 = tc::smem_u32(&abort_flag);
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kPairStages; ++s) {
      tc::mbar_init(tc::smem_u32(&bar_full[s]), 1);
      tc::mbar_init(tc::smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(tc::smem_u32(&bar_acc_full[b]), 1);
      tc::mbar_init(tc::smem_u32(&bar_acc_empty[b]), 2);
    }
    tc::mbar_fence_init();
    tc::tma_prefetch_descriptor(&tm_a);
    tc::tma_prefetch_descriptor(&tm_w);
  }
  if (warp == 1) {
    tc::tmem_alloc_pair(tc::smem_u32(&tmem_base_slot), kPairTmemCols);
    tc::tmem_relinquish_pair();
  }
  tc::fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                  // both CTAs' barriers exist before anything signals them
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();
  pdl_trigger();

  const int num_tiles = prm.tiles_p * prm.tiles_q;     // in units of 256 x 256
  const int first_tile = (int)(blockIdx.x >> 1), tile_step = (int)(gridDim.x >> 1);
  const int kb_count = prm.k_blocks;

  if (warp == 0) {
    if (lane == 0) {
      constexpr int kXPerBlock = KIND == tc::MMA_F16 ? kRowBytes / 2 : kRowBytes;
      const uint32_t full0 = tc::cluster_addr(tc::smem_u32(&bar_full[0]), 0u);   // the leader's barriers
      int stage_i = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        int tp, tq;
        pair_tile_coords(tile, prm.tiles_p, prm.tiles_q, tp, tq);
        const int row_a = tp * 2 * kBM + (int)rank * kBM, row_w = tq * kPairBN + (int)rank * kPairHalfB;
        for (int it = 0; it < kb_count; ++it) {
          tc::mbar_wait_or_flag(tc::smem_u32(&bar_empty[stage_i]), phase ^ 1u, abort_u32);
          if (leader) tc::mbar_arrive_expect_tx(tc::smem_u32(&bar_full[stage_i]), 2u * kPairStageBytes);
          const uint32_t full = full0 + (uint32_t)stage_i * 8u;
          const uint32_t sp = tc::smem_u32(tiles + stage_i * kPairStageBytes);
          tc::tma_load_2d_pair(sp, &tm_a, full, it * kXPerBlock, row_a);
          tc::tma_load_2d_pair(sp + kBM * kRowBytes, &tm_w, full, it * kXPerBlock, row_w);
          if (++stage_i == kPairStages) { stage_i = 0; phase ^= 1u; }
        }
        if (*abort) ok = false;
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      int stage_i = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
        if (!tc::mbar_wait(tc::smem_u32(&bar_acc_empty[buf]), acc_phase[buf] ^ 1u, abort)) break;
        tc::fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kPairBN);
        for (int it = 0; it < kb_count; ++it) {
          tc::mbar_wait_or_flag(tc::smem_u32(&bar_full[stage_i]), phase, abort_u32);
          const uint32_t sp = tc::smem_u32(tiles + stage_i * kPairStageBytes);
          const uint64_t da = tc::smem_desc_k_major_sw128(sp);
          const uint64_t db = tc::smem_desc_k_major_sw128(sp + kBM * kRowBytes);
#pragma unroll
          for (int j = 0; j < kRowBytes / 32; ++j)
            tc::mma_ss_pair<KIND>(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), prm.idesc,
                                  (it > 0 || j > 0) ? 1u : 0u);
          tc::mma_commit_pair(tc::smem_u32(&bar_empty[stage_i]));      // frees the stage in both CTAs
          if (++stage_i == kPairStages) { stage_i = 0; phase ^= 1u; }
        }
        if (*abort) break;
        tc::mma_commit_pair(tc::smem_u32(&bar_acc_full[buf]));          // accumulators complete in both CTAs
        acc_phase[buf] ^= 1u;
        buf ^= 1;
      }
    }
  } else {
    // Eight warps: two per tensor-memory lane quadrant, each taking one half (128) of the tile's columns.
    // One warp per scheduler does not hide its own latencies, and the epilogue of a 128 x 256 tile must
    // finish within the main loop of the next (K = 3584: 11 us) or the tensor pipe waits for it.
    const int quad = warp & 3, et = quad * 32 + lane;
    const int half = (warp - 2) >> 2;                                   // which 128 columns
    const int te = (int)threadIdx.x - 64;                               // 0 .. 255
    const bool issuer = threadIdx.x == 64;
    const Epilogue& e = prm.epi;
    const bool raw = e.mode == EPI_RAW, tensor = e.mode == EPI_TENSOR;
    const bool scaled = e.mode == EPI_ROW_COL || e.mode == EPI_COL_ROW;
    const bool wide = raw || e.out_dtype == LLMQRT_F32;                 // 4-byte outputs
    const bool bf16 = e.out_dtype == LLMQRT_BF16;
    const bool has_bias = e.bias != nullptr;
    const bool col_first = e.mode == EPI_COL_ROW;                       // (acc * col_scale) * row_scale
    const int es = wide ? 4 : 2;
    const float alpha = e.alpha_dev ? *e.alpha_dev : e.alpha;
    const float bmul = tensor ? e.beta : 1.f;
    const uint32_t acc_empty0 = tc::cluster_addr(tc::smem_u32(&bar_acc_empty[0]), 0u);
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step) {
      int tp, tq;
        pair_tile_coords(tile, prm.tiles_p, prm.tiles_q, tp, tq);
      const int row = tp * 2 * kBM + (int)rank * kBM + et;
      const bool row_ok = row < prm.M;
      pair_epi_barrier();                              // previous tile no longer reads q_scale / q_bias
      {
        const int j = tq * kPairBN + te;               // one column's scale and bias per thread
        float sc = 1.f, bi = 0.f;
        if (j < prm.N) {
          if (scaled) sc = e.col_scale[j];
          if (has_bias && !raw) bi = __fmul_rn(bmul, load_as_f32(e.bias, j, e.bias_dtype));
        }
        q_scale[te] = sc;
        q_bias[te] = bi;
      }
      const float rs = (scaled && row_ok) ? e.row_scale[row] : 1.f;
      const bool failed = !tc::mbar_wait(tc::smem_u32(&bar_acc_full[buf]), acc_phase[buf], abort);
      if (tc::named_barrier_or(2, 256, failed)) break;
      tc::fence_after_sync();
      acc_phase[buf] ^= 1u;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * kPairBN + half * 128);
      const int ncols = min(128, prm.N - tq * kPairBN - half * 128);    // my columns inside the matrix (may be <= 0)
      uint8_t* orow = reinterpret_cast<uint8_t*>(e.out) + ((int64_t)row * e.ldo + (int64_t)tq * kPairBN + half * 128) * es;
      // 32 accumulator columns per step; the load of the next step is issued before this step's
      // arithmetic and stores so that its latency is hidden.  A thread owns 32 consecutive outputs of
      // one row (64 or 128 contiguous bytes) and writes them straight from registers: fire-and-forget
      // stores, nothing to wait for, the accumulator buffer is free as soon as the last load is back.
      uint32_t r[2][32];
      if (ncols > 0) tc::tmem_ld_32x32(taddr, r[0]);
#pragma unroll 1
      for (int c0 = 0; c0 < ncols; c0 += 64) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int c = c0 + 32 * h;
          if (c >= ncols) break;
          tc::tmem_ld_wait();
          if (c + 32 < ncols) tc::tmem_ld_32x32(taddr + (uint32_t)(c + 32), r[h ^ 1]);
          uint32_t (&v)[32] = r[h];
          // the operator's arithmetic, its run-time choices made once per 32 columns
          if (!raw) {
            const float4* qs4 = reinterpret_cast<const float4*>(q_scale + half * 128 + c);
            const float4* qb4 = reinterpret_cast<const float4*>(q_bias + half * 128 + c);
            float f[32];
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) f[jj] = (float)acc_from_bits<AccT>(v[jj]);
            if (tensor) {                              // fma(alpha, acc, beta * bias)
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const float4 b = qb4[k];
                f[4 * k] = __fmaf_rn(alpha, f[4 * k], b.x); f[4 * k + 1] = __fmaf_rn(alpha, f[4 * k + 1], b.y);
                f[4 * k + 2] = __fmaf_rn(alpha, f[4 * k + 2], b.z); f[4 * k + 3] = __fmaf_rn(alpha, f[4 * k + 3], b.w);
              }
            } else {
              if (col_first) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  const float4 q = qs4[k];
                  f[4 * k] = __fmul_rn(__fmul_rn(f[4 * k], q.x), rs); f[4 * k + 1] = __fmul_rn(__fmul_rn(f[4 * k + 1], q.y), rs);
                  f[4 * k + 2] = __fmul_rn(__fmul_rn(f[4 * k + 2], q.z), rs); f[4 * k + 3] = __fmul_rn(__fmul_rn(f[4 * k + 3], q.w), rs);
                }
              } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  const float4 q = qs4[k];
                  f[4 * k] = __fmul_rn(__fmul_rn(f[4 * k], rs), q.x); f[4 * k + 1] = __fmul_rn(__fmul_rn(f[4 * k + 1], rs), q.y);
                  f[4 * k + 2] = __fmul_rn(__fmul_rn(f[4 * k + 2], rs), q.z); f[4 * k + 3] = __fmul_rn(__fmul_rn(f[4 * k + 3], rs), q.w);
                }
              }
              if (has_bias) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  const float4 b = qb4[k];
                  f[4 * k] = __fadd_rn(f[4 * k], b.x); f[4 * k + 1] = __fadd_rn(f[4 * k + 1], b.y);
                  f[4 * k + 2] = __fadd_rn(f[4 * k + 2], b.z); f[4 * k + 3] = __fadd_rn(f[4 * k + 3], b.w);
                }
              }
            }
            if (wide) {
#pragma unroll
              for (int jj = 0; jj < 32; ++jj) v[jj] = __float_as_uint(f[jj]);
            } else if (bf16) {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                __nv_bfloat162 p2 = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
                v[k] = *reinterpret_cast<uint32_t*>(&p2);
              }
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k) {
                __half2 p2 = __floats2half2_rn(f[2 * k], f[2 * k + 1]);
                v[k] = *reinterpret_cast<uint32_t*>(&p2);
              }
            }
          }
          if (row_ok) {
            if (wide) {                                // v[0..32): 32-bit outputs
              if (c + 32 <= ncols && prm.store32) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                  st_global_256(orow + c * 4 + 32 * k, v[8 * k], v[8 * k + 1], v[8 * k + 2], v[8 * k + 3], v[8 * k + 4],
                                v[8 * k + 5], v[8 * k + 6], v[8 * k + 7]);
              } else if (c + 32 <= ncols) {
#pragma unroll
                for (int k = 0; k < 8; ++k)
                  reinterpret_cast<uint4*>(orow + c * 4)[k] = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
              } else {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj)
                  if (c + jj < ncols) reinterpret_cast<uint32_t*>(orow + c * 4)[jj] = v[jj];
              }
            } else {                                   // v[0..16): pairs of 16-bit outputs
              if (c + 32 <= ncols && prm.store32) {
#pragma unroll
                for (int k = 0; k < 2; ++k)
                  st_global_256(orow + c * 2 + 32 * k, v[8 * k], v[8 * k + 1], v[8 * k + 2], v[8 * k + 3], v[8 * k + 4],
                                v[8 * k + 5], v[8 * k + 6], v[8 * k + 7]);
              } else if (c + 32 <= ncols) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                  reinterpret_cast<uint4*>(orow + c * 2)[k] = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
              } else {
#pragma unroll
                for (int jj = 0; jj < 32; ++jj)
                  if (c + jj < ncols) reinterpret_cast<uint16_t*>(orow + c * 2)[jj] = (uint16_t)(v[jj >> 1] >> (16 * (jj & 1)));
              }
            }
          }
        }
      }
      // every thread's tensor-memory reads are done: the buffer may be overwritten
      tc::fence_before_sync();
      pair_epi_barrier();
      if (issuer) tc::mbar_arrive_cluster(acc_empty0 + (uint32_t)buf * 8u);
      buf ^= 1;
    }
  }

  // ------------------------------- teardown ---------------------------------------
  tc::fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    // a wait ran out: give copies that may still be in flight towards either CTA time to land
    const uint64_t t0 = tc::global_timer_ns();
    while (tc::global_timer_ns() - t0 < 100000ull) __nanosleep(1000);
  }
  cluster_sync_all();                                  // nobody leaves while its peer may still signal it
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc_pair(tmem_base, kPairTmemCols);
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

// Packed 4-bit weights as a 2-D uint32 matrix [rows, words] (row-major); box = 8 words x box_rows, no swizzle.
int make_packed_map(CUtensorMap* map, const void* base, int64_t rows, int64_t words, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return set_error(LLMQRT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)words, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(words * 4)};
  cuuint32_t box[2] = {8, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(LLMQRT_ERR_CUDA, "cuTensorMapEncodeTiled (packed weights) failed with code %d", (int)r);
  return LLMQRT_OK;
}

template <int KIND, int BN, bool AWQ = false>
cudaLaunchConfig_t make_config(int grid, int cluster, cudaStream_t st, cudaLaunchAttribute* attr) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(AWQ ? kThreadsAwq : kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes_of<BN, AWQ>();
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (pdl_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  return cfg;
}

// How many clusters of `cluster` CTAs of this kernel can be resident at once (cached per device).
template <int KIND, int BN, bool AWQ = false, bool PUSH = false>
int max_active_clusters(int cluster) {
  static std::mutex mu;
  static std::map<std::pair<int, int>, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find({dev, cluster});
  if (it != cache.end()) return it->second;
  auto kern = gemm_tc_kernel<KIND, BN, AWQ, PUSH>;
  int n = 0;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes_of<BN, AWQ>()) == LLMQRT_OK) {
    cudaLaunchAttribute attr[2];
    cudaLaunchConfig_t cfg = make_config<KIND, BN, AWQ>(cluster, cluster, nullptr, attr);
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
  }
  cache[{dev, cluster}] = n;
  return n;
}

template <int KIND, int BN, bool AWQ = false, bool PUSH = false>
int launch(const CUtensorMap& tm_p, const CUtensorMap& tm_q, const CUtensorMap& tm_w, TcParams prm, cudaStream_t st) {
  auto kern = gemm_tc_kernel<KIND, BN, AWQ, PUSH>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_bytes_of<BN, AWQ>())) return rc;
  const int sms = sm_count();
  const int tiles = prm.tiles_p * prm.tiles_q;
  int splits = 1;
  if (BN <= 128 && tiles < sms) {
    // Pick the cluster size (1, 2, 4, 8) with the smallest estimated time: waves of co-resident
    // clusters x (K blocks per CTA + a fixed per-CTA cost of about eight K blocks for pipeline fill,
    // reduce-scatter and epilogue).
    const float fixed = 8.f;
    float best = (float)ceil_div(tiles, sms) * ((float)prm.k_blocks + fixed);
    for (int s = 2; s <= 8; ++s) {                     // (any size: 36 tiles fit as clusters of three, not of four)
      if (prm.k_blocks < 2 * s || BN / 8 < s) continue;
      const int active = max_active_clusters<KIND, BN, AWQ, PUSH>(s);
      if (active <= 0) continue;
      const float t = (float)ceil_div(tiles, active) * ((float)prm.k_blocks / s + fixed);
      if (t < best) { best = t; splits = s; }
    }
  }
  prm.splits = splits;
  const int grid = splits > 1 ? tiles * splits : (tiles < sms ? tiles : sms);
  cudaLaunchAttribute attr[2];
  cudaLaunchConfig_t cfg = make_config<KIND, BN, AWQ>(grid, splits, st, attr);
  LLMQRT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tm_p, tm_q, tm_w, prm));
  return check_launch("gemm_tc");
}

// Clusters of two CTAs of the pair kernel that can be resident at once (cached per device).
template <int KIND>
int pair_max_clusters() {
  static std::mutex mu;
  static std::map<int, int> cache;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(dev);
  if (it != cache.end()) return it->second;
  auto kern = gemm_tc_pair_kernel<KIND>;
  int n = 0;
  if (ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kPairSmemBytes) == LLMQRT_OK) {
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
  }
  cache[dev] = n;
  return n;
}

template <int KIND>
int launch_pair(const CUtensorMap& tm_a, const CUtensorMap& tm_w, const TcParams& prm, cudaStream_t st) {
  auto kern = gemm_tc_pair_kernel<KIND>;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kPairSmemBytes)) return rc;
  int clusters = pair_max_clusters<KIND>();
  if (clusters <= 0) return set_error(LLMQRT_ERR_CUDA, "tcgen05 pair gemm: no cluster of two CTAs fits on this device");
  const int tiles = prm.tiles_p * prm.tiles_q;
  if (clusters > tiles) clusters = tiles;
  cudaLaunchAttribute attr[2];
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (pdl_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  LLMQRT_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_w, prm));
  return check_launch("gemm_tc_pair");
}

template <int KIND, bool AWQ = false>
int launch_bn(int bn, const CUtensorMap& tm_p, const CUtensorMap& tm_q, const CUtensorMap& tm_w, const TcParams& prm,
              cudaStream_t st) {
  switch (bn) {
    case 32: return launch<KIND, 32, AWQ>(tm_p, tm_q, tm_w, prm, st);
    case 64: return launch<KIND, 64, AWQ>(tm_p, tm_q, tm_w, prm, st);
    case 128: return launch<KIND, 128, AWQ>(tm_p, tm_q, tm_w, prm, st);
    default: return launch<KIND, 256, AWQ>(tm_p, tm_q, tm_w, prm, st);
  }
}

// The two-CTA kernel is used unless the environment variable LLMQRT_GEMM_PAIR is "0".
bool pair_enabled() {
  static const bool on = [] {
    const char* v = getenv("LLMQRT_GEMM_PAIR");
    return !(v && v[0] == '0');
  }();
  return on;
}

}  // namespace

int gemm_tc(int kind, const void* A, int64_t lda, const void* W, int64_t ldw, int64_t M, int64_t N, int64_t K,
            const Epilogue& epi, void* workspace, cudaStream_t st, bool static_w, const AwqOperand* awq,
            const CommPush* push) {
  const int elt = (kind == KIND_F16 || kind == KIND_BF16) ? 2 : 1;
  if (awq) {                                           // W is produced in shared memory from the packed layer
    LLMQRT_REQUIRE(kind == KIND_F16 && awq->wq_t && awq->sz_t && awq->G > 0 && K % 32 == 0 && K % awq->G == 0 &&
                   awq->G % 32 == 0 && (reinterpret_cast<uintptr_t>(awq->wq_t) & 15) == 0,
                   "tcgen05 awq gemm: fp16 activations, K and group size multiples of 32, 16-byte aligned packed weights");
    W = A;                                             // placeholder for the unused tensor map
    ldw = lda;
    static_w = false;
  }
  LLMQRT_REQUIRE((K * elt) % 16 == 0 && (lda * elt) % 16 == 0 && (ldw * elt) % 16 == 0,
                 "tcgen05 gemm: K and leading dimensions must cover multiples of 16 bytes");
  LLMQRT_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0,
                 "tcgen05 gemm: operands must be 16-byte aligned");

  // A mid-sized M with a narrow N has only a handful of 128 x 256 tiles, and that schedule has no
  // split-K: most SMs would idle (M = 256, N = 1536, K = 8960: 12 tiles).  Such problems run through
  // the small-M schedule instead -- weights as the 128-lane operand, tokens in panels of 128 as the
  // column operand, cluster split-K -- as ONE launch whose grid covers every (weight tile, token
  // panel) pair; neighbouring clusters share a weight tile, so the panels after the first read it
  // from L2.
  bool panels = false;
  if (M > 128 && M <= 1024) {
    const int64_t tiles = ceil_div(M, (int64_t)kBM) * ceil_div(N, (int64_t)(N <= 128 ? 128 : 256));
    panels = tiles * 4 <= sm_count();
  }

  TcParams prm{};
  prm.M = (int)M;
  prm.N = (int)N;
  prm.epi = epi;
  prm.early_w = static_w ? 1 : 0;
  prm.swap = (M <= 128 || panels) ? 1 : 0;
  int bn;
  if (prm.swap) bn = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  else bn = N <= 128 ? 128 : 256;
  if (awq && !prm.swap) {
    // AWQ with many tokens: the weights stay the 128-lane operand and the tokens come in tiles of 256.
    // A dequantized weight tile (the expensive operand: it is produced by arithmetic, not by a copy)
    // then serves 256 tokens instead of 128, halving the dequantization work per multiply; and the
    // dequantizing warps only ever see 128-row weight tiles.
    prm.swap = 1;
    bn = 256;
  }
  if (push) {
    LLMQRT_REQUIRE(prm.swap && !awq && epi.mode != EPI_RAW && epi.out_dtype != LLMQRT_F32 && N % 8 == 0 &&
                   N / 8 <= push->threads,
                   "tcgen05 gemm: output push needs the small-M schedule, a 16-bit output and N a multiple of 8");
    prm.comm_on = 1;
    prm.comm_threads = push->threads;
    prm.comm_two_step = push->two_step;
    prm.comm = push->dev;
  }
  prm.rows_p = prm.swap ? (int)N : (int)M;
  prm.rows_q = prm.swap ? (int)M : (int)N;
  prm.k_blocks = (int)ceil_div(K * elt, kRowBytes);
  prm.tiles_p = (int)ceil_div(prm.rows_p, kBM);
  prm.tiles_q = (int)ceil_div(prm.rows_q, bn);
  prm.status = workspace ? ws_scalars(workspace) + 1 : nullptr;

  // A/B formats of the instruction follow P/Q.
  uint32_t fmt_act = 0, fmt_w = 0, c_fmt = 1;
  int mk = tc::MMA_F8;
  if (kind == KIND_I8) { mk = tc::MMA_I8; fmt_act = fmt_w = 1; c_fmt = 2; }
  else if (kind == KIND_F8_E5M2) { fmt_act = 1; }
  else if (kind == KIND_F16) { mk = tc::MMA_F16; }
  else if (kind == KIND_BF16) { mk = tc::MMA_F16; fmt_act = fmt_w = 1; }

  // Prefill-sized problems whose 256-row pair tiles waste no more rows than 128-row tiles would: the
  // two-CTA kernel.  Its vector stores need a 16-byte aligned output with a 16-byte multiple row pitch.
  {
    const int es = (epi.mode == EPI_RAW || epi.out_dtype == LLMQRT_F32) ? 4 : 2;
    const bool out_ok = (reinterpret_cast<uintptr_t>(epi.out) & 15) == 0 && (epi.ldo * es) % 16 == 0;
    const bool rows_ok = M >= 2048 || ceil_div(M, (int64_t)256) * 256 == ceil_div(M, (int64_t)128) * 128;
    if (!awq && !prm.swap && bn == 256 && M >= 512 && rows_ok && out_ok && pair_enabled()) {
      prm.tiles_p = (int)ceil_div(M, (int64_t)(2 * kBM));
      prm.tiles_q = (int)ceil_div(N, (int64_t)kPairBN);
      prm.idesc = tc::instr_desc(c_fmt, fmt_act, fmt_w, 2 * kBM, kPairBN);
      prm.store32 = ((reinterpret_cast<uintptr_t>(epi.out) & 31) == 0 && (epi.ldo * es) % 32 == 0) ? 1 : 0;
      CUtensorMap tm_a, tm_w;
      if (int rc = make_operand_map(&tm_a, A, elt, M, K, lda, kBM)) return rc;
      if (int rc = make_operand_map(&tm_w, W, elt, N, K, ldw, kPairHalfB)) return rc;
      if (mk == tc::MMA_I8) return launch_pair<tc::MMA_I8>(tm_a, tm_w, prm, st);
      if (mk == tc::MMA_F8) return launch_pair<tc::MMA_F8>(tm_a, tm_w, prm, st);
      return launch_pair<tc::MMA_F16>(tm_a, tm_w, prm, st);
    }
  }
  prm.idesc = tc::instr_desc(c_fmt, prm.swap ? fmt_w : fmt_act, prm.swap ? fmt_act : fmt_w, kBM, (uint32_t)bn);

  CUtensorMap tm_p, tm_q;
  const void* p_base = prm.swap ? W : A;
  const void* q_base = prm.swap ? A : W;
  if (int rc = make_operand_map(&tm_p, p_base, elt, prm.rows_p, K, prm.swap ? ldw : lda, kBM)) return rc;
  if (int rc = make_operand_map(&tm_q, q_base, elt, prm.rows_q, K, prm.swap ? lda : ldw, bn)) return rc;

  if (awq) {
    prm.awq_w = awq->wq_t;
    prm.awq_sz = awq->sz_t;
    prm.awq_kw = (int)(K / 8);
    prm.awq_kg = (int)(K / awq->G);
    prm.awq_g = (int)awq->G;
    // packed words as a 2-D uint32 matrix [N, K / 8]; box = the 8 words of a K block x the tile's weight rows
    CUtensorMap tm_w;
    if (int rc = make_packed_map(&tm_w, awq->wq_t, N, K / 8, kBM)) return rc;
    return launch_bn<tc::MMA_F16, true>(bn, tm_p, tm_q, tm_w, prm, st);
  }
  if (push) {                                          // (int8, weights as the 128-lane operand: checked above)
    LLMQRT_REQUIRE(mk == tc::MMA_I8, "tcgen05 gemm: the output push is built for the int8 kind");
    switch (bn) {
      case 32: return launch<tc::MMA_I8, 32, false, true>(tm_p, tm_q, tm_p, prm, st);
      case 64: return launch<tc::MMA_I8, 64, false, true>(tm_p, tm_q, tm_p, prm, st);
      default: return launch<tc::MMA_I8, 128, false, true>(tm_p, tm_q, tm_p, prm, st);
    }
  }
  if (mk == tc::MMA_I8) return launch_bn<tc::MMA_I8>(bn, tm_p, tm_q, tm_p, prm, st);
  if (mk == tc::MMA_F8) return launch_bn<tc::MMA_F8>(bn, tm_p, tm_q, tm_p, prm, st);
  return launch_bn<tc::MMA_F16>(bn, tm_p, tm_q, tm_p, prm, st);
}

}  // namespace llmqrt

