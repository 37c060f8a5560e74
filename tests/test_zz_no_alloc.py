"""The allocation-free int8 linear entry point, called through the C ABI.

Some callers may not allocate device memory at all (a serving process that owns the whole memory plan
and forbids its plug-ins to call cudaMalloc, or a loop that cannot take the device-wide stall an
allocation causes), so they cannot supply the split-K workspace.  For them the library keeps a fixed
scratch array of its own.  This test drives that entry point with raw pointers, twice in a row and
with different shapes so that the second call sees the first call's leftovers in the shared scratch,
and requires the same bits as the regular entry point (the arithmetic is integer-exact up to the
fused fp32 epilogue, which is evaluated in the same order).  The file name makes pytest collect it
after every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed, with_bias, out_dtype):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).cuda()
    w = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8).cuda()
    a_scale = (torch.rand(M, generator=g) * 1e-2 + 1e-4).cuda()
    w_scale = (torch.rand(N, generator=g) * 1e-3 + 1e-5).cuda()
    bias = torch.randn(N, generator=g).to(out_dtype).cuda() if with_bias else None
    return a, w, bias, a_scale, w_scale


def _noalloc(a, w, bias, a_scale, w_scale, out_dtype):
    from llmqrt_b200 import _lib as L
    M, K = a.shape
    N = w.shape[0]
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)       # outputs stay the caller's business
    L.call("llmqrt_w8a8_int8_linear_per_channel_noalloc", L.ptr(a), a.stride(0), L.ptr(w), w.stride(0), L.ptr(bias),
           L.dtype_code(bias.dtype) if bias is not None else L.F16, L.ptr(a_scale), L.ptr(w_scale), L.ptr(out),
           L.dtype_code(out_dtype), N, M, N, K, L.stream(a.device))
    return out


def test_no_alloc_entry_matches_regular_entry_twice_in_a_row():
    from llmqrt_b200 import _lib as L
    from llmqrt_b200 import ops
    cases = [(16, 4864, 896, 0, False, torch.float16),        # split over K: partial sums + counters in the scratch
             (7, 1000, 3584, 1, True, torch.bfloat16),        # different shape on top of the leftovers
             (16, 4864, 896, 0, False, torch.float16),        # and the first one again
             (64, 3584, 3584, 2, True, torch.bfloat16)]
    L.set_gemm_path(1)            # the regular entry point on the same streaming kernel
    try:
        for M, N, K, seed, with_bias, dt in cases:
            a, w, bias, a_s, w_s = _case(M, N, K, seed, with_bias, dt)
            want = ops.int8_linear_per_channel(a, w, bias, a_s, w_s, dt)
            got = _noalloc(a, w, bias, a_s, w_s, dt)
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (M, N, K)
    finally:
        L.set_gemm_path(0)
    # and against the default dispatch (tcgen05 above 16 rows): still the same bits
    a, w, bias, a_s, w_s = _case(64, 3584, 3584, 2, True, torch.bfloat16)
    got = _noalloc(a, w, bias, a_s, w_s, torch.bfloat16)
    assert torch.equal(got.view(torch.int16),
                       ops.int8_linear_per_channel(a, w, bias, a_s, w_s, torch.bfloat16).view(torch.int16))
    # and directly against the CPU oracle of the operator (same fp32 op order: identical bits)
    from oracle import gemm as og
    want = og.int8_linear_per_channel(a.cpu(), w.cpu(), bias.cpu(), a_s.cpu(), w_s.cpu(), torch.bfloat16)
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


def test_no_alloc_entry_rejects_what_does_not_fit():
    a, w, bias, a_s, w_s = _case(64, 37888, 18944, 3, False, torch.bfloat16)
    with pytest.raises(RuntimeError, match="built-in scratch"):
        _noalloc(a, w, bias, a_s, w_s, torch.bfloat16)
    a, w, bias, a_s, w_s = _case(65, 256, 256, 4, False, torch.bfloat16)
    with pytest.raises(RuntimeError, match="maximum of 64 rows"):
        _noalloc(a, w, bias, a_s, w_s, torch.bfloat16)
