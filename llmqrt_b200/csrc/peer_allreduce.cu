// One-shot sum all-reduce of 16-bit activations over peer-mapped buffers (NVLink / NVSwitch), for the
// row-parallel partial outputs of a tensor-parallel decode step (a few hundred KB per call, latency
// bound: a library all-reduce costs several times the wire time at this size).
//
// Every rank owns one buffer, allocated once and mapped into every other rank's process through CUDA
// IPC.  A buffer holds, per call parity p and source rank s, a slot of 16-byte words
//     { data[0:4 bytes], seq, data[4:8 bytes], seq }
// -- eight payload bytes (four 16-bit values), each half tagged with the sequence number of the call
// that wrote it, so a word proves its own arrival and no fence, flag or barrier separates the data
// from its notification.  One call, identical on every rank (same length, same grid):
//   push   : every thread tags its words of the local vector with the call's sequence number and
//            stores them into slot (p, me) of EVERY rank's buffer (the peers' addresses are ordinary
//            global pointers; 16-byte volatile stores).
//   gather : the same thread polls its OWN rank's slots (p, s) for all s until both tags of its
//            word carry the sequence number, adds the W copies in rank order in fp32 (same order on
//            every rank, so all ranks get identical bits), rounds once and writes the local output.
//            The poll is bounded (5 s): on a time-out the thread raises the buffer's sticky status
//            word and stops; later calls see the status and return at once.
// Two parities: a rank can run at most one call ahead of a peer (it cannot finish call k+1 before
// that peer has pushed for k+1, which the peer does after finishing call k), so call k+1 never
// overwrites words a peer still reads for call k, and a stale word always carries an older tag.
// The sequence number lives in the buffer and is advanced once per call by the block that draws the
// last ticket (after every block has read it), so the kernel can be replayed from a CUDA graph.
//
// No multicast, no TMA, no atomics on peer memory: only stores to, and polls of, plain memory.
#include <cstring>
#include <new>

#include "common.cuh"

namespace llmqrt {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kArThreads = 256;
constexpr int kMaxBlocks = 296;
constexpr size_t kCtrlBytes = 4096;                              // {sequence, status, ticket}
constexpr unsigned long long kPollLimitNs = 5000000000ull;       // 5 s

struct CommDev {                     // passed to the kernel by value
  unsigned char* base[kMaxWorld];    // every rank's buffer as mapped in this process; [rank] is the local one
  int rank, world;
  long long slot_bytes;              // capacity of one slot (tagged words: twice the payload)
};

struct Comm {
  CommDev dev;
  int device;
  bool opened[kMaxWorld];
};

__device__ __forceinline__ uint4* slot_ptr(unsigned char* base, long long slot_bytes, int parity, int src) {
  return reinterpret_cast<uint4*>(base + kCtrlBytes + ((size_t)parity * kMaxWorld + src) * (size_t)slot_bytes);
}
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// x / out are viewed as 8-byte words (four 16-bit values each).
template <typename T>
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_kernel(CommDev c, const uint2* __restrict__ x, uint2* __restrict__ out, long long nword) {
  pdl_wait();
  pdl_trigger();
  unsigned char* me = c.base[c.rank];
  unsigned* ctrl = reinterpret_cast<unsigned*>(me);                    // [0] sequence, [1] status, [2] ticket
  volatile unsigned* status = ctrl + 1;
  __shared__ unsigned s_seq;
  __shared__ int s_bad;
  if (threadIdx.x == 0) {
    const unsigned seq0 = *reinterpret_cast<volatile unsigned*>(ctrl) + 1u;
    s_seq = seq0;
    s_bad = *status != 0u;
    __threadfence();                                                   // the read above before the ticket below
    // Whoever draws the last ticket knows that every block has read the old sequence number.
    if (atomicAdd(ctrl + 2, 1u) == gridDim.x - 1) {
      ctrl[2] = 0u;
      *reinterpret_cast<volatile unsigned*>(ctrl) = seq0;
    }
  }
  __syncthreads();
  if (s_bad) return;
  const unsigned seq = s_seq;
  const int parity = (int)(seq & 1u);
  const long long stride = (long long)gridDim.x * kArThreads;
  const long long w0 = (long long)blockIdx.x * kArThreads + threadIdx.x;

  for (long long w = w0; w < nword; w += stride) {
    const uint2 d = x[w];
    const uint4 tagged = make_uint4(d.x, seq, d.y, seq);
    for (int p = 0; p < c.world; ++p) st_volatile_v4(slot_ptr(c.base[p], c.slot_bytes, parity, c.rank) + w, tagged);
  }

  const unsigned long long t0 = timer_ns();
  for (long long w = w0; w < nword; w += stride) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < c.world; ++s) {
      const uint4* src = slot_ptr(me, c.slot_bytes, parity, s) + w;
      uint4 v = ld_volatile_v4(src);
      for (unsigned it = 1; v.y != seq || v.w != seq; ++it) {
        if ((it & 255u) == 0u && (*status != 0u || timer_ns() - t0 > kPollLimitNs)) {
          *status = 1u;
          return;
        }
        v = ld_volatile_v4(src);
      }
      const uint2 d = make_uint2(v.x, v.z);
      const T* e = reinterpret_cast<const T*>(&d);
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += to_f32<T>(e[j]);
    }
    __align__(8) T r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = from_f32<T>(acc[j]);
    out[w] = *reinterpret_cast<const uint2*>(r);
  }
}

}  // namespace
}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_comm_create(int rank, int world, int64_t max_bytes, void** comm_out) {
  LLMQRT_REQUIRE(comm_out != nullptr, "comm_create: null output");
  LLMQRT_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "comm_create: need 0 <= rank < world <= %d", kMaxWorld);
  LLMQRT_REQUIRE(max_bytes > 0 && max_bytes <= ((int64_t)1 << 28), "comm_create: max_bytes must be in (0, 256 MiB]");
  Comm* c = new (std::nothrow) Comm();
  LLMQRT_REQUIRE(c != nullptr, "comm_create: out of host memory");
  for (int i = 0; i < kMaxWorld; ++i) { c->dev.base[i] = nullptr; c->opened[i] = false; }
  c->dev.rank = rank;
  c->dev.world = world;
  c->dev.slot_bytes = 2 * ((max_bytes + 255) / 256 * 256);            // tagged words: twice the payload
  const size_t total = kCtrlBytes + (size_t)2 * kMaxWorld * (size_t)c->dev.slot_bytes;
  void* p = nullptr;
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc(&p, total);                     // set-up allocation; calls allocate nothing
  if (e == cudaSuccess) e = cudaMemset(p, 0, total);                   // tag 0 everywhere: older than any call
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    delete c;
    return set_error(LLMQRT_ERR_CUDA, "comm_create: %s", cudaGetErrorString(e));
  }
  c->dev.base[rank] = static_cast<unsigned char*>(p);
  *comm_out = c;
  return LLMQRT_OK;
}

int llmqrt_comm_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

int llmqrt_comm_local_handle(void* comm, void* handle_out) {
  LLMQRT_REQUIRE(comm && handle_out, "comm_local_handle: null pointer");
  Comm* c = static_cast<Comm*>(comm);
  cudaIpcMemHandle_t h;
  LLMQRT_CUDA_OK(cudaIpcGetMemHandle(&h, c->dev.base[c->dev.rank]));
  memcpy(handle_out, &h, sizeof(h));
  return LLMQRT_OK;
}

int llmqrt_comm_open_peer(void* comm, int peer, const void* handle) {
  LLMQRT_REQUIRE(comm && handle, "comm_open_peer: null pointer");
  Comm* c = static_cast<Comm*>(comm);
  LLMQRT_REQUIRE(peer >= 0 && peer < c->dev.world && peer != c->dev.rank, "comm_open_peer: bad peer rank %d", peer);
  LLMQRT_REQUIRE(!c->opened[peer], "comm_open_peer: peer %d already opened", peer);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  LLMQRT_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  c->dev.base[peer] = static_cast<unsigned char*>(p);
  c->opened[peer] = true;
  return LLMQRT_OK;
}

int llmqrt_comm_allreduce(void* comm, const void* x, void* out, int dtype, int64_t n, llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(comm != nullptr, "comm_allreduce: null communicator");
  Comm* c = static_cast<Comm*>(comm);
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "comm_allreduce: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(n >= 0 && n % 8 == 0 && n * 4 <= c->dev.slot_bytes, "comm_allreduce: n must be a multiple of 8 with n * 2 <= %lld bytes", (long long)(c->dev.slot_bytes / 2));
  if (n == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE(x && out && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0, "comm_allreduce: pointers must be non-null and 16-byte aligned");
  for (int p = 0; p < c->dev.world; ++p)
    LLMQRT_REQUIRE(c->dev.base[p] != nullptr, "comm_allreduce: peer %d has not been opened", p);
  const long long nword = n / 4;
  long long blocks = (nword + kArThreads - 1) / kArThreads;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  int rc;
  if (dtype == LLMQRT_F16)
    rc = launch_chained(peer_allreduce_kernel<__half>, dim3((unsigned)blocks), dim3(kArThreads), 0, (cudaStream_t)stream, 1,
                        c->dev, static_cast<const uint2*>(x), static_cast<uint2*>(out), nword);
  else
    rc = launch_chained(peer_allreduce_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(kArThreads), 0,
                        (cudaStream_t)stream, 1, c->dev, static_cast<const uint2*>(x), static_cast<uint2*>(out), nword);
  if (rc) return rc;
  return check_launch("peer_allreduce");
}

int llmqrt_comm_status(void* comm, int32_t* status_out) {
  LLMQRT_REQUIRE(comm && status_out, "comm_status: null pointer");
  Comm* c = static_cast<Comm*>(comm);
  unsigned s = 0;
  LLMQRT_CUDA_OK(cudaMemcpy(&s, c->dev.base[c->dev.rank] + 4, 4, cudaMemcpyDeviceToHost));
  *status_out = (int32_t)s;
  return LLMQRT_OK;
}

int llmqrt_comm_destroy(void* comm) {
  if (!comm) return LLMQRT_OK;
  Comm* c = static_cast<Comm*>(comm);
  for (int p = 0; p < c->dev.world; ++p)
    if (c->opened[p]) cudaIpcCloseMemHandle(c->dev.base[p]);
  cudaFree(c->dev.base[c->dev.rank]);
  delete c;
  return LLMQRT_OK;
}

}  // extern "C"
