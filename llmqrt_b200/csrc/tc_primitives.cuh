// Thin inline-PTX wrappers for the Blackwell (sm_100a) asynchronous machinery used by the dense
// GEMM kernel: mbarriers with bounded waits, TMA tiled loads (never multicast), tensor-memory
// allocation, tcgen05.mma / commit / ld, and the 64-bit shared-memory matrix descriptor.
#pragma once
#include "common.cuh"

namespace llmqrt {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `kWaitLimitNs`, or as soon as another thread of the block has
// raised `*abort`.  On a time-out it raises `*abort` itself.  Returns true when the phase completed.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
  // One probe first: a counted retry loop gets unrolled into a chain of predicated probes, and a
  // barrier that is already complete then pays the latency of every one of them.
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort = 1;
        return false;
      }
    }
  }
}

// The same bounded wait for the per-stage waits of the pipeline, where the single thread that issues
// the copies or the MMAs pays for every dependent instruction: no result is returned (a conditional
// exit from the issuing loop costs more than the probe itself).  On a time-out, or when another
// thread has raised the flag, the 32-bit flag at shared address `abort_smem` is set / left set and
// the caller, which checks the flag once per tile or burst, carries on until then with whatever the
// stage holds.
__device__ __forceinline__ void mbar_wait_or_flag(uint32_t bar, uint32_t parity, uint32_t abort_smem) {
  asm volatile(
      "{\n\t.reg .pred P1, P2;\n\t.reg .u32 c;\n\t.reg .u64 t0, t1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%0], %1;\n\t"
      "@P1 bra W_DONE;\n\t"
      "mov.u64 t0, %%globaltimer;\n\t"
      "W_LOOP:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%0], %1;\n\t"
      "@P1 bra W_DONE;\n\t"
      "ld.volatile.shared.u32 c, [%2];\n\t"
      "setp.ne.u32 P2, c, 0;\n\t"
      "@P2 bra W_DONE;\n\t"
      "mov.u64 t1, %%globaltimer;\n\t"
      "sub.u64 t1, t1, t0;\n\t"
      "setp.lt.u64 P2, t1, %3;\n\t"
      "@P2 bra W_LOOP;\n\t"
      "mov.u32 c, 1;\n\t"
      "st.volatile.shared.u32 [%2], c;\n\t"
      "W_DONE:\n\t}"
      ::"r"(bar), "r"(parity), "r"(abort_smem), "l"(kWaitLimitNs)
      : "memory");
}

// One lane of a fully converged warp.  The issuing warp runs its loop with all 32 lanes and guards only
// the asynchronous instruction itself with this: the operands (descriptors, addresses) are then
// computed in warp-uniform code, where the compiler can keep them in uniform registers -- computed
// under `if (lane == 0)` they have to be moved there one by one for every instruction issued.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
// Bounded wait executed by every lane of a converged warp; the result is warp-uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort));
}

// Named barrier over `nthreads` threads that also ORs a predicate across them (uniform result).
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(id), "r"(nthreads)
      : "memory");
  return r != 0;
}

// ---- TMA: 2-D tiled load, global -> this CTA's shared memory, completion on an mbarrier ------
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tensor_map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(tensor_map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const void* tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------
// Whole-warp operations (.sync.aligned): every lane of the calling warp must execute them.
__device__ __forceinline__ void tmem_alloc(uint32_t result_slot_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives columns [c, c+32) of
// TMEM lane (lane_base + i).  The warp may only address the lane quadrant 32 * (warp_id % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Same with 8 columns per thread.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- tcgen05.mma ----------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes long and stored with
// the 128-byte swizzle (what a TMA load with SWIZZLE_128B and a 128-byte inner box produces):
//   bits  0-13  start address >> 4          bits 16-29  leading byte offset >> 4 (1: unused here)
//   bits 32-45  stride byte offset >> 4 = 64 (8 rows x 128 B between row groups)
//   bits 46-47  descriptor version = 1       bits 61-63  layout = 2 (SWIZZLE_128B)
// Stepping along K inside the 128-byte row adds the byte offset to the start address.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_addr) {
  const uint32_t lo = ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
  const uint32_t hi = 64u | (1u << 14) | (2u << 29);
  return ((uint64_t)hi << 32) | lo;
}

// Instruction descriptor (dense, K-major A and B, no negation):
//   bits 4-5 accumulator format (1 = F32, 2 = S32); bits 7-9 A format; bits 10-12 B format;
//   bits 17-22 N >> 3; bits 24-28 M >> 4.
// Formats: kind::i8 1 = signed; kind::f8f6f4 0 = e4m3, 1 = e5m2; kind::f16 0 = fp16, 1 = bf16.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m,
                                                  uint32_t n) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

enum MmaKind : int { MMA_I8 = 0, MMA_F8 = 1, MMA_F16 = 2 };

// D[tmem] (+)= A[smem] * B[smem]^T, issued by a single thread.
template <int KIND>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  if constexpr (KIND == MMA_I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else if constexpr (KIND == MMA_F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  }
}

// Makes `bar` receive one arrival once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}


// ---- two-CTA form (cta_group::2) --------------------------------------------------------------
// The two CTAs of a thread-block cluster of size 2 act as one tensor-core unit: an MMA issued by one
// thread of the even ("leader") CTA multiplies a 256-row A (128 rows from each CTA's shared memory) by
// a B whose N rows are split between the two shared memories, and each CTA's tensor memory receives
// its 128 accumulator rows.  Every CTA therefore stages only half of B.
// Allocation / deallocation: one warp of EACH CTA executes these (same shared-memory slot offset).
__device__ __forceinline__ void tmem_alloc_pair(uint32_t result_slot_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
// Address of the same shared-memory offset in CTA `cta_rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local_smem, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem), "r"(cta_rank));
  return r;
}
// TMA load into THIS CTA's shared memory whose completion bytes are counted on an mbarrier that may
// live in the peer CTA of the pair (`bar_cluster` is a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tensor_map, uint32_t bar_cluster, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst_smem), "l"(tensor_map), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
template <int KIND>
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  if constexpr (KIND == MMA_I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else if constexpr (KIND == MMA_F8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
// One arrival on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once every MMA
// issued so far by this thread has finished (a signal fanned out to two barriers, not a data copy).
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// One arrival (release at cluster scope) on an mbarrier given by its shared::cluster address.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

}  // namespace tc
}  // namespace llmqrt
