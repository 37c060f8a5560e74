"""Parity of the AWQ W4A16 kernels against the CPU oracle and the reference-generated fixtures."""
import pytest
import torch

from tests.util import bits_equal, load_golden, rel_fro

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from llmqrt_b200 import ops as _ops
    return _ops


def test_dequantize_matches_reference_fixture(ops):
    g = load_golden("awq_small")
    w = ops.awq_dequantize(g["qweight"].cuda(), g["scales"].cuda(), g["qzeros"].cuda())
    assert bits_equal(w.cpu(), g["w_dequant"]) and bits_equal(w.cpu(), g["w_dequant_triton"])


def test_gemm_matches_reference_triton_fixture(ops):
    g = load_golden("awq_small")
    packed = ops.AwqPacked(g["qweight"].cuda(), g["scales"].cuda(), g["qzeros"].cuda())
    y = ops.awq_gemm(g["x"].cuda(), packed)
    assert rel_fro(y, g["y_gemm_triton"]) < 2e-3


@pytest.mark.parametrize("K,N,G", [(1536, 2048, 128), (8960, 1536, 128), (256, 64, 32), (512, 72, 64), (384, 136, 384)])
def test_repack_and_dequantize_bit_exact(ops, K, N, G):
    from oracle import awq as oa
    qw, qz, sc = oa.random_layer(K, N, G, seed=K + N)
    w_ref = oa.dequantize(qw, qz, sc, G)
    assert bits_equal(ops.awq_dequantize(qw.cuda(), sc.cuda(), qz.cuda()).cpu(), w_ref)
    packed = ops.AwqPacked(qw.cuda(), sc.cuda(), qz.cuda())
    assert (packed.wq_t.cpu().numpy().view("uint32") == oa.repack_k_major(qw)).all()
    assert bits_equal(ops.awq_dequantize_t(packed).cpu(), w_ref.t().contiguous())


AWQ_SHAPES = [(2048, 1536), (1536, 1536), (8960, 1536), (1536, 8960)]      # (N, K): qkv, o, gate/up, down


@pytest.mark.parametrize("M", [1, 16, 256, 2048])
@pytest.mark.parametrize("N,K", AWQ_SHAPES)
def test_gemm_sweep(ops, M, N, K):
    from oracle import awq as oa
    if M == 2048 and N * K > 8960 * 1536 - 1 and K == 8960:
        pass
    qw, qz, sc = oa.random_layer(K, N, 128, seed=N + K + M)
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).to(torch.float16)
    bias = torch.randn(N, generator=g).to(torch.float16) if N == 2048 else None
    packed = ops.AwqPacked(qw.cuda(), sc.cuda(), qz.cuda())
    y = ops.awq_gemm(x.cuda(), packed, None if bias is None else bias.cuda())
    w = oa.dequantize(qw, qz, sc, 128).double()
    ref = x.double() @ w
    if bias is not None:
        ref = ref + bias.double()
    assert rel_fro(y, ref.to(torch.float16)) < 1e-2


def test_gemm_many_tokens_weight_panels(ops):
    # from 1024 tokens on the weights are expanded panel by panel into the workspace and multiplied by the dense
    # fp16 kernel: a layer whose fp16 form (9600 x 8960 x 2 B = 172 MB) exceeds one 160 MB panel takes two
    from oracle import awq as oa
    K, N, G, M = 8960, 9600, 128, 1024
    qw, qz, sc = oa.random_layer(K, N, G, seed=11)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K, generator=g).to(torch.float16)
    bias = torch.randn(N, generator=g).to(torch.float16)
    packed = ops.AwqPacked(qw.cuda(), sc.cuda(), qz.cuda())
    y = ops.awq_gemm(x.cuda(), packed, bias.cuda()).cpu()
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 511, 512, 1000, M - 1])
    w = oa.dequantize(qw, qz, sc, G).float()
    ref = (x[rows].float() @ w).double() + bias.double()
    assert rel_fro(y[rows], ref.to(torch.float16)) < 1e-2
    assert torch.isfinite(y.float()).all()


# up to 64 tokens: the weight-streaming kernel; above: the tcgen05 kernel that dequantizes the weight
# tiles in shared memory (K = 416 ends in half a 64-value block, N = 200 in a partial tile, groups of 32)
@pytest.mark.parametrize("M", [3, 9, 17, 33, 64, 65, 100, 300, 1100])
def test_gemm_ragged_shapes(ops, M):
    from oracle import awq as oa
    K, N, G = 416, 200, 32
    qw, qz, sc = oa.random_layer(K, N, G, seed=M)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.float16)
    packed = ops.AwqPacked(qw.cuda(), sc.cuda(), qz.cuda())
    y = ops.awq_gemm(x.cuda(), packed)
    assert rel_fro(y, oa.gemm(x, qw, qz, sc, G)) < 2e-3
    y2 = ops.awq_gemm(x.cuda(), packed)
    assert bits_equal(y, y2)                       # fixed reduction order: repeatable
