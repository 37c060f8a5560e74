// C-ABI entry points of the W8A8 GEMMs: argument validation, epilogue set-up, back-end choice.
#include "gemm_w8a8.cuh"

#include <atomic>

namespace llmqrt {
namespace {

std::atomic<int> g_path{0};

// M at or below which the register-operand streaming kernel is used; above it the weights are
// streamed by TMA into shared memory and multiplied by tcgen05 with the tokens as the N operand.
constexpr int64_t kStreamMaxM = 16;

int check_common(const void* a, int64_t lda, const void* w, int64_t ldw, const void* out, int64_t ldo, int64_t M,
                 int64_t N, int64_t K) {
  LLMQRT_REQUIRE(a && w && out, "w8a8 gemm: null pointer");
  LLMQRT_REQUIRE(M >= 0 && N > 0 && K > 0, "w8a8 gemm: bad shape M=%lld N=%lld K=%lld", (long long)M, (long long)N,
                 (long long)K);
  LLMQRT_REQUIRE(N < (1ll << 31) && K < (1ll << 31) && M < (1ll << 31), "w8a8 gemm: dimension too large");
  LLMQRT_REQUIRE(K % 16 == 0, "w8a8 gemm: K=%lld must be a multiple of 16", (long long)K);
  LLMQRT_REQUIRE(lda >= K && ldw >= K && lda % 16 == 0 && ldw % 16 == 0,
                 "w8a8 gemm: lda=%lld / ldw=%lld must be >= K and multiples of 16", (long long)lda, (long long)ldw);
  LLMQRT_REQUIRE(ldo >= N, "w8a8 gemm: ldo=%lld < N", (long long)ldo);
  LLMQRT_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                 "w8a8 gemm: operands must be 16-byte aligned");
  return LLMQRT_OK;
}

int run(int kind, const void* a, int64_t lda, const void* w, int64_t ldw, int64_t M, int64_t N, int64_t K,
        const Epilogue& epi, void* workspace, cudaStream_t st, int flags) {
  if (M == 0) return LLMQRT_OK;
  LLMQRT_REQUIRE((flags & ~LLMQRT_GEMM_STATIC_WEIGHT) == 0, "w8a8 gemm: unknown flags 0x%x", flags);
  const int path = g_path.load();
  const bool stream = path == 1 || (path == 0 && M <= kStreamMaxM);
  if (stream)
    return w8a8_gemm_stream(kind, reinterpret_cast<const uint8_t*>(a), lda, reinterpret_cast<const uint8_t*>(w), ldw,
                            M, N, K, epi, workspace, st);
  return gemm_tc(kind, a, lda, w, ldw, M, N, K, epi, workspace, st, (flags & LLMQRT_GEMM_STATIC_WEIGHT) != 0);
}

int f8_kind(int a_format) {
  if (a_format == LLMQRT_E4M3) return KIND_F8_E4M3;
  if (a_format == LLMQRT_E5M2) return KIND_F8_E5M2;
  return -1;
}

}  // namespace

int gemm_path() { return g_path.load(); }

}  // namespace llmqrt

using namespace llmqrt;

extern "C" {

int llmqrt_set_gemm_path(int path) {
  if (path < 0 || path > 2) return set_error(LLMQRT_ERR_INVALID, "gemm path must be 0, 1 or 2");
  g_path.store(path);
  return LLMQRT_OK;
}

int llmqrt_w8a8_int8_linear_per_tensor(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, const void* bias,
                                       float alpha, const float* alpha_dev, float beta, void* out, int64_t ldo,
                                       int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags) {
  if (int rc = check_common(a, lda, w, ldw, out, ldo, M, N, K)) return rc;
  LLMQRT_REQUIRE(bias, "int8 per-tensor linear: bias is required (pass zeros for none)");
  Epilogue e{};
  e.mode = EPI_TENSOR; e.out_dtype = LLMQRT_F16; e.bias_dtype = LLMQRT_F16; e.alpha = alpha; e.beta = beta;
  e.alpha_dev = alpha_dev; e.bias = bias; e.out = out; e.ldo = ldo;
  return run(KIND_I8, a, lda, w, ldw, M, N, K, e, workspace, (cudaStream_t)stream, flags);
}

int llmqrt_w8a8_int8_linear_per_channel(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, const void* bias,
                                        int bias_dtype, const float* a_scale, const float* w_scale, void* out,
                                        int out_dtype, int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace,
                                        llmqrt_stream_t stream, int flags) {
  if (int rc = check_common(a, lda, w, ldw, out, ldo, M, N, K)) return rc;
  LLMQRT_REQUIRE(a_scale && w_scale, "int8 per-channel linear: null scale");
  LLMQRT_REQUIRE(out_dtype == LLMQRT_F16 || out_dtype == LLMQRT_BF16, "int8 per-channel linear: out must be fp16/bf16");
  LLMQRT_REQUIRE(!bias || bias_dtype == LLMQRT_F16 || bias_dtype == LLMQRT_BF16 || bias_dtype == LLMQRT_F32,
                 "int8 per-channel linear: bad bias dtype");
  Epilogue e{};
  e.mode = EPI_COL_ROW; e.out_dtype = out_dtype; e.bias_dtype = bias_dtype; e.bias = bias; e.row_scale = a_scale;
  e.col_scale = w_scale; e.out = out; e.ldo = ldo;
  return run(KIND_I8, a, lda, w, ldw, M, N, K, e, workspace, (cudaStream_t)stream, flags);
}

int llmqrt_comm_int8_linear_per_channel(void* comm, const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw,
                                        const void* bias, int bias_dtype, const float* a_scale, const float* w_scale,
                                        int out_dtype, int64_t M, int64_t N, int64_t K, void* workspace,
                                        llmqrt_stream_t stream, int flags) {
  LLMQRT_REQUIRE(comm != nullptr, "comm int8 linear: null communicator");
  Comm* c = static_cast<Comm*>(comm);
  if (int rc = check_common(a, lda, w, ldw, a, N, M, N, K)) return rc;       // (no output tensor: `a` stands in)
  LLMQRT_REQUIRE(a_scale && w_scale, "comm int8 linear: null scale");
  LLMQRT_REQUIRE(out_dtype == LLMQRT_F16 || out_dtype == LLMQRT_BF16, "comm int8 linear: dtype must be fp16/bf16");
  LLMQRT_REQUIRE(!bias || bias_dtype == LLMQRT_F16 || bias_dtype == LLMQRT_BF16 || bias_dtype == LLMQRT_F32,
                 "comm int8 linear: bad bias dtype");
  LLMQRT_REQUIRE((flags & ~LLMQRT_GEMM_STATIC_WEIGHT) == 0, "comm int8 linear: unknown flags 0x%x", flags);
  LLMQRT_REQUIRE(M > kStreamMaxM && M <= 128, "comm int8 linear: M = %lld is outside (16, 128], the range of the "
                 "schedule whose epilogue pushes", (long long)M);
  LLMQRT_REQUIRE(N % 8 == 0 && N <= 8192, "comm int8 linear: N must be a multiple of 8 and at most 8192");
  CommPush push;
  push.dev = c->dev;
  push.threads = comm_row_threads(N);
  push.two_step = comm_two_step(c->dev.world);
  LLMQRT_REQUIRE(M * push.threads * 32 <= c->dev.slot_bytes, "comm int8 linear: M * N exceeds the communicator's capacity");
  for (int p = 0; p < c->dev.world; ++p)
    LLMQRT_REQUIRE(c->dev.base[p] != nullptr, "comm int8 linear: peer %d has not been opened", p);
  Epilogue e{};
  e.mode = EPI_COL_ROW; e.out_dtype = out_dtype; e.bias_dtype = bias_dtype; e.bias = bias; e.row_scale = a_scale;
  e.col_scale = w_scale; e.out = nullptr; e.ldo = N;
  return gemm_tc(KIND_I8, a, lda, w, ldw, M, N, K, e, workspace, (cudaStream_t)stream,
                 (flags & LLMQRT_GEMM_STATIC_WEIGHT) != 0, nullptr, &push);
}

int llmqrt_w8a8_int8_gemm_s32(const int8_t* a, int64_t lda, const int8_t* w, int64_t ldw, int32_t* acc, int64_t ldo,
                              int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags) {
  if (int rc = check_common(a, lda, w, ldw, acc, ldo, M, N, K)) return rc;
  Epilogue e{};
  e.mode = EPI_RAW; e.out_dtype = LLMQRT_F32; e.out = acc; e.ldo = ldo;
  return run(KIND_I8, a, lda, w, ldw, M, N, K, e, workspace, (cudaStream_t)stream, flags);
}

int llmqrt_f8f8_tensorwise(const uint8_t* a, int a_format, int64_t lda, const uint8_t* w, int64_t ldw,
                           const void* bias, float alpha, const float* alpha_dev, float beta, void* out, int out_dtype,
                           int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags) {
  if (int rc = check_common(a, lda, w, ldw, out, ldo, M, N, K)) return rc;
  const int kind = f8_kind(a_format);
  LLMQRT_REQUIRE(kind >= 0, "fp8 tensorwise: activations must be e4m3 or e5m2");
  LLMQRT_REQUIRE(out_dtype == LLMQRT_F16 || out_dtype == LLMQRT_BF16, "fp8 tensorwise: out must be fp16/bf16");
  Epilogue e{};
  e.mode = EPI_TENSOR; e.out_dtype = out_dtype; e.bias_dtype = out_dtype; e.alpha = alpha; e.beta = beta;
  e.alpha_dev = alpha_dev; e.bias = bias; e.out = out; e.ldo = ldo;
  return run(kind, a, lda, w, ldw, M, N, K, e, workspace, (cudaStream_t)stream, flags);
}

int llmqrt_f8f8bf16_rowwise(const uint8_t* a, int a_format, int64_t lda, const uint8_t* w, int64_t ldw,
                            const void* bias, int bias_dtype, const float* x_scale, const float* w_scale, void* out,
                            int64_t ldo, int64_t M, int64_t N, int64_t K, void* workspace, llmqrt_stream_t stream, int flags) {
  if (int rc = check_common(a, lda, w, ldw, out, ldo, M, N, K)) return rc;
  const int kind = f8_kind(a_format);
  LLMQRT_REQUIRE(kind >= 0, "fp8 rowwise: activations must be e4m3 or e5m2");
  LLMQRT_REQUIRE(x_scale && w_scale, "fp8 rowwise: null scale");
  LLMQRT_REQUIRE(!bias || bias_dtype == LLMQRT_BF16 || bias_dtype == LLMQRT_F32, "fp8 rowwise: bias must be bf16 or fp32");
  Epilogue e{};
  e.mode = EPI_ROW_COL; e.out_dtype = LLMQRT_BF16; e.bias_dtype = bias_dtype; e.bias = bias; e.row_scale = x_scale;
  e.col_scale = w_scale; e.out = out; e.ldo = ldo;
  return run(kind, a, lda, w, ldw, M, N, K, e, workspace, (cudaStream_t)stream, flags);
}

}  // extern "C"
