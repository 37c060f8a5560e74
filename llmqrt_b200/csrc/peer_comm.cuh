// Peer-mapped buffers of the tensor-parallel all-reduce: layout, device helpers and the host-side
// communicator object shared by the kernels that push to and gather from them.
//
// Every rank owns one buffer, allocated once and mapped into every other rank's process through CUDA
// IPC.  After a small control area it holds, per call parity p and source rank s (plus one more
// slot per parity for rows that arrive already reduced, see the two-step variant in glue.cu), a slot
// of 16-byte words
//     { data[0:4 bytes], seq, data[4:8 bytes], seq }
// -- eight payload bytes (four 16-bit values), each half tagged with the sequence number of the call
// that wrote it, so a word proves its own arrival and no fence, flag or barrier separates the data
// from its notification.  In one call every rank stores its tagged words into slot (p, me) of EVERY
// rank's buffer and then polls its OWN rank's slots (p, s) for all s until both tags carry the
// call's sequence number.
// Two parities: a rank can run at most one call ahead of a peer (it cannot finish call k+1 before
// that peer has pushed for k+1, which the peer does after finishing call k), so call k+1 never
// overwrites words a peer still reads for call k, and a stale word always carries an older tag.
// The sequence number of the last completed call lives in the buffer; a call uses the next one and
// the block that finishes last publishes it (every block has used it by then), so a call can be
// replayed from a CUDA graph.
// Polls are bounded (5 s unless the host sets another limit): on a time-out the sticky status word of
// the buffer is raised and later calls return without waiting.
#pragma once
#include "common.cuh"

namespace llmqrt {

constexpr int kCommMaxWorld = 8;
constexpr int kCommSlots = kCommMaxWorld + 1;   // per parity: one slot per source rank + one for reduced rows
constexpr size_t kCommCtrlBytes = 4096;                              // {sequence, status, ticket}
constexpr unsigned long long kCommPollLimitNs = 5000000000ull;       // default bound of a poll: 5 s

struct CommDev {                         // passed to kernels by value
  unsigned char* base[kCommMaxWorld];    // every rank's buffer as mapped in this process; [rank] is the local one
  int rank, world;
  long long slot_bytes;                  // capacity of one slot (tagged words: twice the payload)
  unsigned long long poll_limit_ns;      // bound of a poll
};

// What a row-parallel GEMM needs to deliver its output rows as the pushes of the next call (the row
// kernel that consumes the sum then only gathers): the word of element 8u .. 8u+7 of row m depends on
// the block size of that row kernel, and both must agree on one step or two.
struct CommPush {
  CommDev dev;
  int threads;                           // block size of the consuming row kernel (comm_row_threads)
  int two_step;
};
inline int comm_row_threads(int64_t H) { return (int)(((H / 8) + 31) / 32 * 32); }
int comm_two_step(int world);            // glue.cu: two steps from 8 ranks on, or when the environment forces it
// Word indices of unit u (elements 8u .. 8u+7) of row m: the two words of a unit sit 32 words apart so
// that each store or poll of a warp covers 512 contiguous bytes.  (Any bijection works, as every
// rank and both kernels use this one.)
__host__ __device__ __forceinline__ long long comm_word0(long long m, long long u, int threads) {
  return m * (2 * (long long)threads) + (u >> 5) * 64 + (u & 31);
}

struct Comm {                            // what the opaque handle of the C ABI points to
  CommDev dev;
  int device;
  bool opened[kCommMaxWorld];
};

__device__ __forceinline__ uint4* comm_slot(unsigned char* base, long long slot_bytes, int parity, int src) {
  return reinterpret_cast<uint4*>(base + kCommCtrlBytes + ((size_t)parity * kCommSlots + src) * (size_t)slot_bytes);
}
__device__ __forceinline__ void comm_st_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 comm_ld_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long comm_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Sequence numbers run 1, 2, ..., 0xFFFFFFFE, 1, ...: never 0 (the tag of a buffer that was never
// written) and with alternating parity across the wrap (0xFFFFFFFE is even, 1 is odd).
__device__ __forceinline__ unsigned comm_next_seq(unsigned s) { return s >= 0xFFFFFFFEu ? 1u : s + 1u; }

// Start of a call, ONE thread per block: reads the call's sequence number (one more than the last
// completed call's) and whether the sticky status is raised (the caller then neither pushes nor
// polls).  Nothing is written here, so the block's first stores do not wait for an atomic.
__device__ __forceinline__ bool comm_enter(const CommDev& c, unsigned* seq) {
  const unsigned* ctrl = reinterpret_cast<const unsigned*>(c.base[c.rank]);   // [0] sequence, [1] status, [2] ticket
  const unsigned last = *reinterpret_cast<const volatile unsigned*>(ctrl);
  const unsigned bad = *reinterpret_cast<const volatile unsigned*>(ctrl + 1);
  *seq = comm_next_seq(last);
  return bad == 0u;
}

// End of a call, ONE thread per block, after the block's last use of the sequence number: the block
// that draws the last ticket publishes the number as completed.  The next call on this rank is
// ordered after this kernel by the stream, so it reads the advanced number; a CUDA graph replays.
__device__ __forceinline__ void comm_leave(const CommDev& c, unsigned seq) {
  unsigned* ctrl = reinterpret_cast<unsigned*>(c.base[c.rank]);
  __threadfence();
  if (atomicAdd(ctrl + 2, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) {
    ctrl[2] = 0u;
    *reinterpret_cast<volatile unsigned*>(ctrl) = seq;
  }
}

// Stores one tagged word (eight payload bytes) into slot (parity of seq, me) of every rank.
__device__ __forceinline__ void comm_push(const CommDev& c, unsigned seq, long long word, uint2 payload) {
  const uint4 tagged = make_uint4(payload.x, seq, payload.y, seq);
  for (int p = 0; p < c.world; ++p) comm_st_v4(comm_slot(c.base[p], c.slot_bytes, (int)(seq & 1u), c.rank) + word, tagged);
}

// Stores one tagged word into slot `slot` of rank `dst` only.
__device__ __forceinline__ void comm_push_one(const CommDev& c, unsigned seq, int dst, int slot, long long word,
                                              uint2 payload) {
  comm_st_v4(comm_slot(c.base[dst], c.slot_bytes, (int)(seq & 1u), slot) + word,
             make_uint4(payload.x, seq, payload.y, seq));
}

// Polls word `word` of source rank s in the local buffer until it carries `seq`.  Returns false (and
// raises the status) when the wait ran out or another thread has already given up.
__device__ __forceinline__ bool comm_gather(const CommDev& c, unsigned seq, int s, long long word,
                                            unsigned long long t0, uint2* payload) {
  volatile unsigned* status = reinterpret_cast<unsigned*>(c.base[c.rank]) + 1;
  const uint4* src = comm_slot(c.base[c.rank], c.slot_bytes, (int)(seq & 1u), s) + word;
  uint4 v = comm_ld_v4(src);
  for (unsigned it = 1; v.y != seq || v.w != seq; ++it) {
    if ((it & 255u) == 0u && (*status != 0u || comm_timer_ns() - t0 > c.poll_limit_ns)) {
      *status = 1u;
      return false;
    }
    v = comm_ld_v4(src);
  }
  *payload = make_uint2(v.x, v.z);
  return true;
}

// The same for NW words of each of the slots first_slot .. first_slot + nslots - 1 (nslots <= NS) at
// once: all loads of a round are issued before any tag is looked at, so a round costs one trip to L2
// however many sources there are (polling them one after the other costs one trip each even when
// every word has long arrived).  words[j] are the word indices; on success v[i][j] holds the tagged
// word of slot first_slot + i, word j: payload in .x and .z.
template <int NS, int NW>
__device__ __forceinline__ bool comm_gather_all(const CommDev& c, unsigned seq, int first_slot, int nslots,
                                                const long long (&words)[NW], unsigned long long t0,
                                                uint4 (&v)[NS][NW]) {
  volatile unsigned* status = reinterpret_cast<unsigned*>(c.base[c.rank]) + 1;
  const uint4* slot0 = comm_slot(c.base[c.rank], c.slot_bytes, (int)(seq & 1u), first_slot);
  const long long slot_words = c.slot_bytes / 16;
  unsigned pending = 0u;                              // bit (i * NW + j): word not yet seen
#pragma unroll
  for (int i = 0; i < NS; ++i)
    if (i < nslots) pending |= ((1u << NW) - 1u) << (i * NW);
  for (unsigned it = 1; pending != 0u; ++it) {
#pragma unroll
    for (int i = 0; i < NS; ++i)
#pragma unroll
      for (int j = 0; j < NW; ++j)
        if (pending >> (i * NW + j) & 1u) v[i][j] = comm_ld_v4(slot0 + i * slot_words + words[j]);
#pragma unroll
    for (int i = 0; i < NS; ++i)
#pragma unroll
      for (int j = 0; j < NW; ++j)
        if ((pending >> (i * NW + j) & 1u) && v[i][j].y == seq && v[i][j].w == seq) pending &= ~(1u << (i * NW + j));
    if (pending != 0u && (it & 63u) == 0u && (*status != 0u || comm_timer_ns() - t0 > c.poll_limit_ns)) {
      *status = 1u;
      return false;
    }
  }
  return true;
}

}  // namespace llmqrt
