// Internal interface between the W8A8 entry points and the two GEMM back ends.
#pragma once
#include "common.cuh"
#include "peer_comm.cuh"

namespace llmqrt {

enum GemmKind : int {
  KIND_I8 = 0,        // int8 x int8 -> int32
  KIND_F8_E4M3 = 1,   // e4m3 activations x e4m3 weights -> fp32
  KIND_F8_E5M2 = 2,   // e5m2 activations x e4m3 weights -> fp32
  KIND_F16 = 3,       // fp16 x fp16 -> fp32   (tcgen05 back end only)
  KIND_BF16 = 4       // bf16 x bf16 -> fp32   (tcgen05 back end only)
};

// Register-operand streaming kernel (gemm_stream.cu): any M, tuned for M <= 16.
int w8a8_gemm_stream(int kind, const uint8_t* A, int64_t lda, const uint8_t* W, int64_t ldw, int64_t M, int64_t N,
                     int64_t K, const Epilogue& epi, void* workspace, cudaStream_t st);

// TMA + tcgen05/TMEM kernel (gemm_tc.cu): any M; lda/ldw in elements.  static_w: W is a stored weight
// that nothing queued on the stream writes, so its first tiles may be requested before the
// preceding kernel of the stream has completed.
// awq != nullptr (kind KIND_F16): W / ldw are ignored and the weight operand is dequantized on the fly,
// tile by tile, from the repacked 4-bit layer (layouts: awq.cu) by extra warps of the same kernel.
struct AwqOperand {
  const uint32_t* wq_t;   // [N, K/8]
  const uint32_t* sz_t;   // [N, K/G]
  int64_t G;
};
int gemm_tc(int kind, const void* A, int64_t lda, const void* W, int64_t ldw, int64_t M, int64_t N, int64_t K,
            const Epilogue& epi, void* workspace, cudaStream_t st, bool static_w = false,
            const AwqOperand* awq = nullptr, const CommPush* push = nullptr);
// push != nullptr (decode-sized M only): the results do not go to epi.out but, as the tagged words of
// the next all-reduce call, into the peers' buffers; llmqrt_comm_allreduce_rmsnorm with a null
// `partial` completes the call.

// Path selection shared by all entry points (0 auto, 1 streaming, 2 tcgen05).
int gemm_path();

}  // namespace llmqrt
