"""Parity of the CUDA quantizers and W8A8 GEMMs (through the C ABI) against the CPU oracle."""
import pytest
import torch

from tests.util import bits_equal, load_golden, rel_fro, ulp_mismatch_fraction

pytestmark = pytest.mark.gpu

PATHS = {"stream": 1, "tcgen05": 2}


@pytest.fixture(scope="module")
def ops():
    from llmqrt_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def _auto_path():
    yield
    from llmqrt_b200 import _lib
    _lib.set_gemm_path(0)
    assert _lib.kernel_status(torch.device("cuda:0")) == 0, "a kernel reported a bounded-wait time-out"


def _outlier_x(M, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[: max(1, K // 100)]] *= 20.0
    return x.to(dtype)


# ------------------------------------------------------------------ quantizers
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("per_token", [True, False])
def test_quantize_int8_matches_oracle_and_torch_cuda(ops, dtype, per_token):
    from oracle import quant as oq
    x = _outlier_x(16, 896, dtype, 0)
    x[3] = 0
    q_ref, s_ref = oq.quantize_int8(x, per_token, scalar_div="reciprocal")
    q, s, s32 = ops.quantize_int8(x.cuda(), per_token, scale_mul=0.5)
    assert torch.equal(q.cpu(), q_ref)
    assert bits_equal(s.cpu(), s_ref)
    assert torch.equal(s32.cpu(), (s_ref.float().reshape(-1) * 0.5).to(dtype).float())
    # the same chain of torch ops the reference executes, on this GPU (linear_sq.py:44-65)
    xc = x.cuda()
    sc = xc.abs().max(dim=-1, keepdim=True).values if per_token else xc.abs().max()
    sc = sc.clamp(min=1e-5).div(127)
    qc = xc.div(sc).round().clamp(-128, 127).to(torch.int8)
    assert torch.equal(q, qc) and bits_equal(s.reshape(-1), sc.reshape(-1))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("per_token", [True, False])
def test_quantize_fp8_matches_oracle_and_torch_cuda(ops, dtype, per_token):
    from oracle import quant as oq
    x = _outlier_x(16, 896, dtype, 2)
    q_ref, s_ref = oq.quantize_fp8(x, per_token, scalar_div="reciprocal")
    q, s = ops.quantize_fp8(x.cuda(), per_token)
    assert bits_equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu().reshape(-1), s_ref.reshape(-1))
    xc = x.cuda()                                        # linear_fp8.py:11-63 on this GPU
    amax = xc.abs().amax(dim=-1, keepdim=True) if per_token else xc.abs().amax()
    sc = amax.clamp(min=1e-12) / 448.0
    qc = (xc / sc).clamp(min=-448.0, max=448.0).to(torch.float8_e4m3fn)
    assert bits_equal(q, qc) and torch.equal(s.reshape(-1), sc.float().reshape(-1))


def test_quantize_fp8_static_matches_golden(ops):
    for tag in ("f16", "bf16"):
        g = load_golden(f"fp8_quant_{tag}")
        q = ops.quantize_fp8_static(g["x"].cuda(), g["s_static"].cuda())
        assert bits_equal(q.cpu(), g["q_static"])


def test_quantize_odd_shapes(ops):
    from oracle import quant as oq
    for M, K in ((1, 8), (3, 1000), (5, 24), (2, 18944)):
        x = _outlier_x(M, K, torch.float16, M * K)
        q_ref, _ = oq.quantize_int8(x, True, scalar_div="reciprocal")
        q, _, _ = ops.quantize_int8(x.cuda(), True)
        assert torch.equal(q.cpu(), q_ref), (M, K)
    assert ops.quantize_int8(torch.empty(0, 64, dtype=torch.float16, device="cuda"), True)[0].shape == (0, 64)


# ------------------------------------------------------------------ int8 GEMM: exact accumulators
INT8_SHAPES = [
    # (M, N, K)
    (16, 4864, 896),      # SmoothQuant headline shape
    (1, 896, 896), (7, 128, 896), (16, 896, 4864), (64, 4864, 896),
    (1, 8, 16), (3, 130, 48), (17, 1000, 208), (33, 72, 1040), (64, 3584, 3584),
    (128, 512, 1024), (200, 384, 512), (1024, 896, 896), (300, 1000, 4864),
    # per-rank shards of the Qwen2-7B linears at tensor-parallel 4 and 8 (batch 64): narrow N, short
    # or ragged K (2368 = 18.5 blocks of 128 bytes), and the 128-row panel schedule (M = 256, few tiles)
    (64, 768, 3584), (64, 3584, 384), (64, 4736, 3584), (64, 3584, 2368), (64, 3584, 896), (256, 1536, 2368),
]


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("M,N,K", INT8_SHAPES)
def test_int8_accumulators_bit_exact(ops, path, M, N, K):
    from llmqrt_b200 import _lib
    from oracle import gemm as og
    g = torch.Generator().manual_seed(M * 131 + N * 7 + K)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    _lib.set_gemm_path(PATHS[path])
    acc = ops.int8_gemm_s32(a.cuda(), w.cuda())
    assert torch.equal(acc.cpu(), og.int8_accumulate(a, w))


# Prefill-sized M: the four Qwen2-0.5B linears at M = 4096, and one Qwen2-7B shape at M = 16384 (the
# token count of a 16 x 1024 prefill chunk, 128 x 256 tiles, persistent schedule).  The fp64 oracle is
# evaluated on a few hundred sampled rows so that it stays a matter of seconds.
# The shapes after the first five aim at the two-CTA (256 x 256 tile) kernel: a token count that is
# no multiple of 256, an N that ends inside a tile, a ragged K, the smallest M that takes this kernel,
# and an output whose row pitch is no multiple of 16 bytes (which must fall back to the one-CTA kernel).
@pytest.mark.parametrize("M,N,K", [(4096, 896, 896), (4096, 128, 896), (4096, 4864, 896), (4096, 896, 4864),
                                   (16384, 4608, 3584), (2300, 1000, 528), (1024, 4864, 896), (2048, 1001, 256),
                                   (2049, 264, 3584)])
def test_int8_accumulators_bit_exact_prefill_sizes(ops, M, N, K):
    from oracle import gemm as og
    g = torch.Generator().manual_seed(M + N * 3 + K)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    acc = ops.int8_gemm_s32(a.cuda(), w.cuda()).cpu()
    rows = torch.cat([torch.tensor([0, 127, 128, 255, 256, M - 129, M - 1]), torch.randperm(M, generator=g)[:249]])
    assert torch.equal(acc[rows], og.int8_accumulate(a[rows], w))


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(2304, 1000, 896), (4096, 4608, 3584)])
def test_int8_epilogues_prefill_sizes(ops, out_dtype, M, N, K):
    # per-token x per-channel (bit-identical to the oracle's fp32 op order) and per-tensor epilogues of
    # the kernel that serves M >= 1024, ragged edges included
    from oracle import gemm as og
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    a_scale = torch.rand(M, generator=g) * 0.02 + 0.001
    w_scale = torch.rand(N, generator=g) * 0.01 + 0.0005
    bias = torch.randn(N, generator=g).to(out_dtype)
    rows = torch.cat([torch.tensor([0, 127, 128, 255, 256, M - 1]), torch.randperm(M, generator=g)[:122]])
    y = ops.int8_linear_per_channel(a.cuda(), w.cuda(), bias.cuda(), a_scale.cuda(), w_scale.cuda(), out_dtype)
    y_ref = og.int8_linear_per_channel(a[rows], w, bias, a_scale[rows], w_scale, out_dtype)
    assert bits_equal(y.cpu()[rows], y_ref)
    if out_dtype == torch.float16:
        yt = ops.int8_linear_per_tensor(a.cuda(), w.cuda(), bias.cuda(), 1e-4, 1.0)
        yt_ref = og.int8_linear_per_tensor(a[rows], w, bias, 1e-4, 1.0)
        frac, dist = ulp_mismatch_fraction(yt.cpu()[rows], yt_ref)
        assert dist <= 1 and frac < 1e-3


@pytest.mark.parametrize("path", list(PATHS))
def test_int8_gemm_is_repeatable_with_split_k(ops, path):
    # split-K partials live in a shared workspace whose counters must return to zero
    from llmqrt_b200 import _lib
    from oracle import gemm as og
    g = torch.Generator().manual_seed(5)
    a = torch.randint(-128, 128, (16, 3584), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (512, 3584), generator=g, dtype=torch.int8)
    ref = og.int8_accumulate(a, w)
    _lib.set_gemm_path(PATHS[path])
    for _ in range(3):
        assert torch.equal(ops.int8_gemm_s32(a.cuda(), w.cuda()).cpu(), ref)


@pytest.mark.parametrize("path", list(PATHS))
def test_int8_per_tensor_epilogue(ops, path):
    # shapes and construction of the reference unit test runtime/unittest/test_sq_linear.py:7-34
    from llmqrt_b200 import _lib
    from oracle import gemm as og
    g = torch.Generator().manual_seed(0)
    B, M, N = 128, 512, 1024
    w = torch.randint(-128, 127, (N, M), generator=g, dtype=torch.int8)
    x = torch.randint(-128, 127, (B, M), generator=g, dtype=torch.int8)
    bias = torch.randn(N, generator=g).to(torch.float16)
    alpha, input_scale = 0.00334, 0.002
    y_gt = torch.nn.functional.linear(x.to(torch.float16) * input_scale, w.to(torch.float16) * alpha, bias)
    _lib.set_gemm_path(PATHS[path])
    y = ops.int8_linear_per_tensor(x.cuda(), w.cuda(), bias.cuda(), alpha * input_scale, 1.0)
    assert torch.allclose(y_gt, y.cpu(), atol=0.1)                      # the reference's own tolerance
    y_or = og.int8_linear_per_tensor(x, w, bias, alpha * input_scale, 1.0)
    frac, dist = ulp_mismatch_fraction(y.cpu(), y_or)
    assert dist <= 1 and frac < 1e-3                                      # fma vs fp64-emulated fma
    # alpha passed as a device scalar, as the reference's callers do
    y2 = ops.int8_linear_per_tensor(x.cuda(), w.cuda(), bias.cuda(),
                                    torch.tensor(alpha * input_scale, device="cuda"), 1.0)
    assert bits_equal(y, y2)


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("out_dtype", [torch.float16, torch.bfloat16])
def test_int8_per_channel_smoothquant_config(ops, path, out_dtype):
    # X[16,896] N(0,1) with 1% outlier channels x20, W[4864,896] N(0,0.02), alpha=0.5 smoothing, seed 0
    from llmqrt_b200 import _lib
    from oracle import gemm as og
    from oracle import quant as oq
    g = torch.Generator().manual_seed(0)
    x = _outlier_x(16, 896, torch.float16, 0).float()
    w = torch.randn(4864, 896, generator=g) * 0.02
    s = (x.abs().amax(0).clamp_min(1e-5).sqrt() / w.abs().amax(0).clamp_min(1e-5).sqrt())
    xs, ws = (x / s).to(torch.float16), (w * s).to(torch.float16)
    wq, w_scale = oq.quantize_weight_int8_per_channel(ws)
    xq_ref, a_scale_ref = oq.quantize_int8(xs, per_token=True)
    xq, a_scale, a_scale32 = ops.quantize_int8(xs.cuda(), per_token=True)
    assert torch.equal(xq.cpu(), xq_ref)
    _lib.set_gemm_path(PATHS[path])
    y = ops.int8_linear_per_channel(xq, wq.cuda(), None, a_scale32, w_scale.cuda(), out_dtype)
    y_ref = og.int8_linear_per_channel(xq_ref, wq, None, a_scale_ref.float(), w_scale.float(), out_dtype)
    assert bits_equal(y.cpu(), y_ref)                                     # same fp32 op order: exact
    assert rel_fro(y, x @ w.t()) < 0.05                                   # and a sane quantized linear


# ------------------------------------------------------------------ fp8 GEMM
FP8_SHAPES = [(N, K) for (N, K) in ((896, 896), (128, 896), (4864, 896), (896, 4864))]


@pytest.mark.parametrize("path", list(PATHS))
@pytest.mark.parametrize("M", [1, 16, 64, 1024])
@pytest.mark.parametrize("N,K", FP8_SHAPES)
def test_fp8_rowwise_sweep(ops, path, M, N, K):
    from llmqrt_b200 import _lib
    from oracle import gemm as og
    from oracle import quant as oq
    if path == "stream" and M > 64:
        pytest.skip("the streaming kernel is not the path for prefill-sized M")
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    wq, w_scale = oq.quantize_weight_fp8_per_channel(w)
    xq, x_scale = oq.quantize_fp8(x, per_token=True)
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if N in (896, 128) else None
    _lib.set_gemm_path(PATHS[path])
    y = ops.fp8_linear_rowwise(xq.cuda(), wq.cuda(), None if bias is None else bias.cuda(), x_scale.cuda(),
                               w_scale.reshape(1, -1).cuda())
    y_ref = og.fp8_linear_rowwise(xq, wq, bias, x_scale, w_scale.reshape(1, -1))
    assert rel_fro(y, y_ref) < 1e-2


@pytest.mark.parametrize("N,K", FP8_SHAPES)
def test_fp8_rowwise_m4096(ops, N, K):
    # the largest M of the FP8 sweep configuration; epilogue order of
    # runtime/csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:193-245
    from oracle import gemm as og
    from oracle import quant as oq
    M = 4096
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    wq, w_scale = oq.quantize_weight_fp8_per_channel(w)
    xq, x_scale = oq.quantize_fp8(x, per_token=True)
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if N in (896, 128) else None
    y = ops.fp8_linear_rowwise(xq.cuda(), wq.cuda(), None if bias is None else bias.cuda(), x_scale.cuda(),
                               w_scale.reshape(1, -1).cuda())
    rows = torch.cat([torch.tensor([0, 127, 128, M - 1]), torch.randperm(M, generator=g)[:508]])
    y_ref = og.fp8_linear_rowwise(xq[rows], wq, bias, x_scale[rows], w_scale.reshape(1, -1))
    assert rel_fro(y[rows.cuda()], y_ref) < 1e-2
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("M", [64, 256, 4096])
def test_weight_quantized_right_before_the_gemm(ops, M):
    # Without LLMQRT_GEMM_STATIC_WEIGHT the GEMM must not read W before the kernel in front of it on
    # the stream has finished: here that kernel is the library's own quantizer producing W.
    from oracle import gemm as og
    g = torch.Generator().manual_seed(M)
    N, K = 1024, 2048
    x = torch.randn(M, K, generator=g).to(torch.float16).cuda()
    w = torch.randn(N, K, generator=g).to(torch.float16).cuda()
    for _ in range(3):
        wq_stale = torch.zeros(N, K, dtype=torch.int8, device="cuda")     # what an early read would see
        xq, _, _ = ops.quantize_int8(x, per_token=True)
        wq, _, _ = ops.quantize_int8(w, per_token=True)
        acc = ops.int8_gemm_s32(xq, wq)
        del wq_stale
        assert torch.equal(acc.cpu(), og.int8_accumulate(xq.cpu(), wq.cpu()))


@pytest.mark.parametrize("path", list(PATHS))
def test_fp8_reference_unit_test_procedures(ops, path):
    # runtime/unittest/test_fp8_rowwise_linear.py:5-52 and test_fp8_tensorwise_linear.py:5-50
    from llmqrt_b200 import _lib
    from oracle import gemm as og
    torch.manual_seed(42)
    a = torch.randn(128, 256, dtype=torch.bfloat16).to(torch.float8_e4m3fn)
    b = torch.randn(512, 256, dtype=torch.bfloat16).to(torch.float8_e4m3fn)
    scale_a, scale_b = torch.rand(128, 1), torch.rand(1, 512)
    _lib.set_gemm_path(PATHS[path])
    y = ops.fp8_linear_rowwise(a.cuda(), b.cuda(), None, scale_a.cuda(), scale_b.cuda())
    ref = og.fp8_linear_rowwise(a, b, None, scale_a, scale_b)
    assert torch.allclose(y.cpu().float(), ref.float(), atol=0.25) and rel_fro(y, ref) < 1e-2
    try:                                                   # the reference test's own ground truth
        ref_mm = torch._scaled_mm(a.cuda(), b.cuda().t(), scale_a=scale_a.cuda(), scale_b=scale_b.cuda(),
                                  out_dtype=torch.bfloat16, use_fast_accum=True)
    except Exception:                                      # not every torch build has row-wise _scaled_mm
        ref_mm = None
    if ref_mm is not None:
        assert torch.allclose(y.float(), ref_mm.float(), atol=0.25)
    bias = torch.randn(512, dtype=torch.bfloat16)
    for dt in (torch.bfloat16, torch.float16):
        y = ops.fp8_linear_tensorwise(a.cuda(), b.cuda(), bias.to(dt).cuda(), 0.5 * 1.2, 1.0, dt)
        ref = og.fp8_linear_tensorwise(a, b, bias.to(dt), 0.5 * 1.2, 1.0, dt)
        assert torch.allclose(y.cpu().float(), ref.float(), atol=0.25) and rel_fro(y, ref) < 1e-2
    y = ops.fp8_linear_tensorwise(a.to(torch.float32).to(torch.float8_e5m2).cuda(), b.cuda(), None, 0.6, 1.0,
                                  torch.bfloat16)
    ref = og.fp8_linear_tensorwise(a.to(torch.float32).to(torch.float8_e5m2), b, None, 0.6, 1.0, torch.bfloat16)
    assert rel_fro(y, ref) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (100, 1536, 1536), (2048, 2048, 1536), (300, 136, 8960),
                                   (2100, 1160, 1000)])
def test_gemm_16bit_tcgen05(ops, dtype, M, N, K):
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    bias = torch.randn(N, generator=g).to(dtype)
    y = ops.gemm_16bit(a.cuda(), w.cuda(), bias.cuda())
    ref = (a.double() @ w.double().t() + bias.double()).to(dtype)
    assert rel_fro(y, ref) < 2e-3


def test_gemm_rejects_bad_arguments(ops):
    a = torch.zeros(4, 24, dtype=torch.int8, device="cuda")
    w = torch.zeros(8, 24, dtype=torch.int8, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.int8_gemm_s32(a, w)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.int8_gemm_s32(a.cpu(), w.cpu())
