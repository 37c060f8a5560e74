// TEMPORARY: placeholders for entry points that are still being written.
#include "common.cuh"
using namespace llmqrt;
#define STUB(name, ...) int name(__VA_ARGS__) { return set_error(LLMQRT_ERR_UNSUPPORTED, #name " not built yet"); }
extern "C" {
STUB(llmqrt_kv_append, void*, void*, int64_t, int64_t, const void*, const void*, const int32_t*, int32_t, int, int64_t, int64_t, int64_t, int64_t, int64_t, llmqrt_stream_t)
STUB(llmqrt_attn_decode, const void*, const void*, const void*, int64_t, int64_t, const int32_t*, void*, int, int64_t, int64_t, int64_t, int64_t, int64_t, float, void*, llmqrt_stream_t)
STUB(llmqrt_attn_prefill, const void*, int64_t, const void*, const void*, int64_t, void*, int64_t, int, int64_t, int64_t, int64_t, int64_t, int64_t, int, float, llmqrt_stream_t)
STUB(llmqrt_rmsnorm, const void*, const void*, void*, const void*, float, void*, int8_t*, float*, int, int64_t, int64_t, llmqrt_stream_t)
STUB(llmqrt_rope_kv_write, void*, int64_t, void*, const void*, int64_t, void*, void*, int64_t, int64_t, int32_t, const int32_t*, float, int, int64_t, int64_t, int64_t, int64_t, int64_t, llmqrt_stream_t)
STUB(llmqrt_silu_mul, const void*, int64_t, void*, int8_t*, float*, int, int64_t, int64_t, llmqrt_stream_t)
}
