// One-shot sum all-reduce of 16-bit activations over peer-mapped buffers (NVLink / NVSwitch), for the
// row-parallel partial outputs of a tensor-parallel decode step (a few hundred KB per call, latency
// bound: a library all-reduce costs several times the wire time at this size), and the set-up of the
// communicator.  Protocol and buffer layout: peer_comm.cuh.
//   push   : every thread tags its words of the local vector and stores them into every rank's
//            buffer (the peers' addresses are ordinary global pointers);
//   gather : the same thread polls its own rank's slots until its word has arrived from every rank,
//            adds the W copies in rank order in fp32 (same order on every rank, so all ranks get
//            identical bits), rounds once and writes the local output.
// No multicast, no TMA, no atomics on peer memory: only stores to, and polls of, plain memory.
#include <cstring>
#include <new>

#include "peer_comm.cuh"

namespace llmqrt {
namespace {

constexpr int kArThreads = 256;
constexpr int kMaxBlocks = 296;

// x / out are viewed as 8-byte words (four 16-bit values each).
template <typename T>
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_kernel(CommDev c, const uint2* __restrict__ x, uint2* __restrict__ out, long long nword) {
  pdl_wait();
  pdl_trigger();
  __shared__ unsigned s_seq;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    unsigned seq;
    s_ok = comm_enter(c, &seq) ? 1 : 0;
    s_seq = seq;
  }
  __syncthreads();
  const unsigned seq = s_seq;
  if (s_ok) {                                                          // else: status raised by an earlier call
    const long long stride = (long long)gridDim.x * kArThreads;
    const long long w0 = (long long)blockIdx.x * kArThreads + threadIdx.x;
    for (long long w = w0; w < nword; w += stride) comm_push(c, seq, w, x[w]);
    const unsigned long long t0 = comm_timer_ns();
    for (long long w = w0; w < nword; w += stride) {
      uint4 d[kCommMaxWorld][1];
      const long long words[1] = {w};
      if (!comm_gather_all<kCommMaxWorld, 1>(c, seq, 0, c.world, words, t0, d)) break;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < kCommMaxWorld; ++s) {                        // rank order: identical bits everywhere
        if (s < c.world) {
          const uint2 pl = make_uint2(d[s][0].x, d[s][0].z);
          const T* e = reinterpret_cast<const T*>(&pl);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] += to_f32<T>(e[j]);
        }
      }
      __align__(8) T r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = from_f32<T>(acc[j]);
      out[w] = *reinterpret_cast<const uint2*>(r);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) comm_leave(c, seq);
}

}  // namespace
}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_comm_create(int rank, int world, int64_t max_bytes, void** comm_out) {
  LLMQRT_REQUIRE(comm_out != nullptr, "comm_create: null output");
  LLMQRT_REQUIRE(world >= 1 && world <= kCommMaxWorld && rank >= 0 && rank < world, "comm_create: need 0 <= rank < world <= %d", kCommMaxWorld);
  LLMQRT_REQUIRE(max_bytes > 0 && max_bytes <= ((int64_t)1 << 28), "comm_create: max_bytes must be in (0, 256 MiB]");
  Comm* c = new (std::nothrow) Comm();
  LLMQRT_REQUIRE(c != nullptr, "comm_create: out of host memory");
  for (int i = 0; i < kCommMaxWorld; ++i) { c->dev.base[i] = nullptr; c->opened[i] = false; }
  c->dev.rank = rank;
  c->dev.world = world;
  c->dev.poll_limit_ns = kCommPollLimitNs;
  c->dev.slot_bytes = 2 * ((max_bytes + 255) / 256 * 256);            // tagged words: twice the payload
  const size_t total = kCommCtrlBytes + (size_t)2 * kCommSlots * (size_t)c->dev.slot_bytes;
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

int llmqrt_comm_set_poll_limit_ms(void* comm, int32_t ms) {
  LLMQRT_REQUIRE(comm != nullptr && ms > 0, "comm_set_poll_limit_ms: need a communicator and a positive limit");
  static_cast<Comm*>(comm)->dev.poll_limit_ns = (unsigned long long)ms * 1000000ull;
  return LLMQRT_OK;
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
