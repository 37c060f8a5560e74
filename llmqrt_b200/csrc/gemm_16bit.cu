// Dense fp16 / bf16 GEMM entry point (tcgen05 back end with a plain "+ bias" epilogue).
#include "gemm_w8a8.cuh"

using namespace llmqrt;

extern "C" int llmqrt_gemm_16bit(const void* a, int64_t lda, const void* w, int64_t ldw, const void* bias, void* out,
                                 int64_t ldo, int dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                                 llmqrt_stream_t stream) {
  LLMQRT_REQUIRE(a && w && out, "gemm_16bit: null pointer");
  LLMQRT_REQUIRE(dtype == LLMQRT_F16 || dtype == LLMQRT_BF16, "gemm_16bit: dtype must be fp16 or bf16");
  LLMQRT_REQUIRE(M >= 0 && N > 0 && K > 0 && K % 8 == 0, "gemm_16bit: bad shape M=%lld N=%lld K=%lld", (long long)M,
                 (long long)N, (long long)K);
  LLMQRT_REQUIRE(lda >= K && ldw >= K && ldo >= N && lda % 8 == 0 && ldw % 8 == 0, "gemm_16bit: bad leading dimension");
  if (M == 0) return LLMQRT_OK;
  // out = 1 * acc + 1 * bias
  Epilogue e{};
  e.mode = EPI_TENSOR; e.out_dtype = dtype; e.bias_dtype = dtype; e.alpha = 1.f; e.beta = 1.f; e.bias = bias;
  e.out = out; e.ldo = ldo;
  return gemm_tc(dtype == LLMQRT_F16 ? KIND_F16 : KIND_BF16, a, lda, w, ldw, M, N, K, e, workspace,
                 (cudaStream_t)stream);
}
