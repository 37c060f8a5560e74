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
// The sequence number lives in the buffer and is advanced once per call by the block that draws the
// last ticket (after every block has read it), so a call can be replayed from a CUDA graph.
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

// Start of a call, ONE thread per block: returns the call's sequence number, or 0 when the status
// word is raised (the caller then neither pushes nor polls).  The block that draws the last ticket
// knows that every block has read the old number and advances it.
__device__ __forceinline__ unsigned comm_enter(const CommDev& c) {
  unsigned* ctrl = reinterpret_cast<unsigned*>(c.base[c.rank]);          // [0] sequence, [1] status, [2] ticket
  const unsigned seq = *reinterpret_cast<volatile unsigned*>(ctrl) + 1u;
  const bool bad = *reinterpret_cast<volatile unsigned*>(ctrl + 1) != 0u;
  __threadfence();                                                       // the reads above before the ticket below
  if (atomicAdd(ctrl + 2, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) {
    ctrl[2] = 0u;
    *reinterpret_cast<volatile unsigned*>(ctrl) = seq;
  }
  return bad ? 0u : seq;
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

}  // namespace llmqrt
