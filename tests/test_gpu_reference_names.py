"""The kernels reached through the reference's own module names, called the way its unit tests call them.

install_reference_aliases() registers `runtime.sq_fp8_kernels` and
`runtime.triton_kernels.awq_kernels`; the three procedures below follow runtime/unittest/
test_sq_linear.py:7-34, test_fp8_rowwise_linear.py:5-52 and test_fp8_tensorwise_linear.py:5-50 line by
line (positional arguments, weight passed as the column-major [K, N] view, same seeds and tolerances).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _aliases():
    import llmqrt_b200
    llmqrt_b200.install_reference_aliases()


@torch.no_grad()
def test_sq_linear_procedure():
    from runtime.sq_fp8_kernels import w8a8_int8_linear_bbf16_obf16_per_tensor
    torch.manual_seed(0)
    B, M, N = 128, 512, 1024
    weight = torch.randint(-128, 127, (N, M), dtype=torch.int8)
    weight_t = weight.t()
    bias = torch.randn(N, dtype=torch.float16)
    x = torch.randint(-128, 127, (B, M), dtype=torch.int8)
    alpha, beta = 0.00334, 1
    input_scale = 0.002
    xx = x.to(torch.float16) * input_scale
    linear = torch.nn.Linear(N, M, bias=True)
    linear.weight.data = weight.to(torch.float16) * alpha
    linear.bias.data = bias.to(torch.float16) * beta
    alpha *= input_scale
    y_gt = linear(xx)
    for _ in range(20):
        y = w8a8_int8_linear_bbf16_obf16_per_tensor(x.cuda(), weight_t.cuda(), bias.cuda(), alpha, beta)
    assert y.dtype == torch.float16 and tuple(y.shape) == (B, N)
    assert torch.allclose(y_gt, y.cpu(), atol=0.1)


def _scaled_mm(a, b, scale_a, scale_b):
    """The reference tests' ground truth; falls back to the fp32 formula where this torch build has no
    such _scaled_mm variant."""
    try:
        return torch._scaled_mm(a, b, scale_a=scale_a, scale_b=scale_b, out_dtype=torch.bfloat16,
                                use_fast_accum=True).to(torch.bfloat16).cpu()
    except Exception:
        return ((a.float() @ b.float()) * scale_a.float() * scale_b.float()).to(torch.bfloat16).cpu()


def test_fp8_rowwise_procedure():
    from runtime.sq_fp8_kernels import cutlass_f8f8bf16_rowwise_sm89
    torch.manual_seed(42)
    a = torch.randn(128, 256, dtype=torch.bfloat16, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(512, 256, dtype=torch.bfloat16, device="cuda").to(torch.float8_e4m3fn)
    b = b.t()
    scale_a = torch.rand(a.shape[0], 1, dtype=torch.float32, device="cuda")
    scale_b = torch.rand(1, b.shape[1], dtype=torch.float32, device="cuda")
    bias = None
    output = cutlass_f8f8bf16_rowwise_sm89(a, b, bias, scale_a, scale_b, True).cpu()
    ref_output = _scaled_mm(a, b, scale_a, scale_b)
    assert output.dtype == torch.bfloat16 and tuple(output.shape) == (128, 512)
    assert torch.allclose(output, ref_output, atol=0.25)


def test_fp8_tensorwise_procedure():
    from runtime.sq_fp8_kernels import cutlass_f8f8bf16_tensorwise_sm89
    torch.manual_seed(42)
    a = torch.randn(128, 256, dtype=torch.bfloat16, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(512, 256, dtype=torch.bfloat16, device="cuda").to(torch.float8_e4m3fn)
    b = b.t()
    scale_a = torch.tensor(0.5, dtype=torch.float32, device="cuda")
    scale_b = torch.tensor(1.2, dtype=torch.float32, device="cuda")
    bias = torch.randn(b.shape[1], dtype=torch.bfloat16, device="cuda")
    alpha = scale_a * scale_b
    beta = 1
    output = cutlass_f8f8bf16_tensorwise_sm89(a, b, bias, alpha, beta, "bfloat16").cpu()
    ref_output = _scaled_mm(a, b, scale_a, scale_b)
    ref_output += bias.cpu().reshape(1, -1)
    assert output.dtype == torch.bfloat16 and tuple(output.shape) == (128, 512)
    assert torch.allclose(output, ref_output, atol=0.25)


def test_awq_kernels_by_reference_name():
    from runtime.triton_kernels.awq_kernels import awq_dequantize_triton, awq_gemm_triton
    from oracle import awq as oawq
    qw, qz, sc = oawq.random_layer(256, 128, 128, seed=1)
    x = torch.randn(4, 256, generator=torch.Generator().manual_seed(2)).half()
    w = awq_dequantize_triton(qw.cuda(), sc.cuda(), qz.cuda())
    assert torch.equal(w.cpu(), oawq.dequantize(qw, qz, sc, 128))
    y = awq_gemm_triton(x.cuda(), qw.cuda(), sc.cuda(), qz.cuda(), 8)
    ref = oawq.gemm(x, qw, qz, sc, 128)
    assert float((y.cpu().double() - ref.double()).norm() / ref.double().norm()) < 1e-2
