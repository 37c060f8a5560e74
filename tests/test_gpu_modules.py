"""The reference-facing modules (linear layers, fused attention block) against oracle compositions."""
import pytest
import torch

from tests.util import max_abs, rel_fro

pytestmark = pytest.mark.gpu


def _linear(i, o, bias, seed):
    g = torch.Generator().manual_seed(seed)
    lin = torch.nn.Linear(i, o, bias=bias)
    lin.weight.data = torch.randn(o, i, generator=g) * 0.05
    if bias:
        lin.bias.data = torch.randn(o, generator=g) * 0.1
    return lin.cuda()


@pytest.mark.parametrize("method", ["sq", "fp8_dynamic_quant", "fp8_static_quant", "awq"])
def test_method_registry_layers_run_and_approximate_the_dense_layer(method):
    from llmqrt_b200.linear import get_concrete_linear_module
    cls = get_concrete_linear_module(method)
    lin = _linear(256, 384, True, 1)
    dt = torch.float16 if method in ("sq", "awq") else torch.bfloat16
    if method == "awq":
        G = 128
        w = lin.weight.data
        wg = w.view(384, 256 // G, G)
        scales = ((wg.amax(-1) - wg.amin(-1)).clamp_min(1e-5) / 15)                 # [N, K/G]
        zeros = torch.round(-wg.amin(-1) / scales).clamp(0, 15)
        layer = cls.from_linear(lin, 4, G, init_only=False, scales=scales.t().contiguous(),
                                zeros=zeros.t().contiguous())
    else:
        layer = cls.from_linear(lin, 8, 0, init_only=False, dtype=dt)
        if method == "fp8_static_quant":
            layer.input_scale.data.fill_(4.0 / 448)
    x = torch.randn(2, 5, 256, generator=torch.Generator().manual_seed(2)).to(dt).cuda()
    y = layer(x)
    ref = torch.nn.functional.linear(x.float(), lin.weight.data, lin.bias.data)
    assert y.shape == (2, 5, 384) and y.dtype == dt
    assert rel_fro(y, ref) < (0.12 if method == "awq" else 0.06)
    assert layer(x[:0]).shape == (0, 5, 384)


def test_sq_per_channel_module_matches_oracle():
    from llmqrt_b200.linear import SqW8A8BBF16OBF16PerChannel
    from oracle import gemm as og
    from oracle import quant as oq
    lin = _linear(896, 512, True, 3)
    layer = SqW8A8BBF16OBF16PerChannel.from_linear(lin, 8, 0, init_only=False, dtype=torch.bfloat16)
    x = torch.randn(16, 896, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    y = layer(x.cuda())
    xq, xs = oq.quantize_int8(x, per_token=True)
    ref = og.int8_linear_per_channel(xq, layer.qweight.cpu(), layer.bias.cpu(), xs.float(), layer.weight_scale.cpu(),
                                     torch.bfloat16)
    assert torch.equal(y.cpu().view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("double_append", [False, True])
def test_fused_attention_block_prefill_then_decode(double_append):
    from llmqrt_b200.linear import SqW8A8BBF16OBF16PerChannel
    from llmqrt_b200.nonlinear import QuantAttentionFused
    from oracle import attention as oa
    hidden, H, Hkv, d, B, S, maxlen = 256, 4, 2, 64, 2, 11, 32
    dt = torch.float16
    mk = lambda i, o, b, s: SqW8A8BBF16OBF16PerChannel.from_linear(_linear(i, o, b, s), 8, 0, init_only=False, dtype=dt)
    q_proj, k_proj, v_proj, o_proj = mk(hidden, H * d, True, 5), mk(hidden, Hkv * d, True, 6), mk(hidden, Hkv * d, True, 7), \
        mk(H * d, hidden, False, 8)
    attn = QuantAttentionFused(hidden, H, Hkv, None, o_proj, "cuda:0", q_proj=q_proj, k_proj=k_proj, v_proj=v_proj,
                               max_seq_len=maxlen, rope_theta=1e6)
    attn.REFERENCE_DOUBLE_APPEND = double_append
    g = torch.Generator().manual_seed(9)
    x0 = torch.randn(B, S, hidden, generator=g).to(dt).cuda()
    x1 = torch.randn(B, 1, hidden, generator=g).to(dt).cuda()
    out0, w0, _ = attn(x0)
    out1, w1, _ = attn(x1)
    assert attn.start_pos == S + 1 and out1.shape == (B, 1, hidden)

    # oracle composition from the module's own projections (the linears are checked elsewhere)
    def proj(x, n):
        return q_proj(x).view(B, n, H, d).cpu(), k_proj(x).view(B, n, Hkv, d).cpu(), v_proj(x).view(B, n, Hkv, d).cpu()
    q, k, v = proj(x0, S)
    q, k = oa.rope_apply(q, 0, 1e6, maxlen), oa.rope_apply(k, 0, 1e6, maxlen)
    kc, vc = torch.zeros(B, maxlen, Hkv, d, dtype=dt), torch.zeros(B, maxlen, Hkv, d, dtype=dt)
    oa.cache_update(kc, vc, k, v, 0)
    assert max_abs(w0.view(B, S, H, d), oa.attention_prefill(q, k, v)) < 2e-3
    q1, k1, v1 = proj(x1, 1)
    q1, k1 = oa.rope_apply(q1, S, 1e6, maxlen), oa.rope_apply(k1, S, 1e6, maxlen)
    oa.cache_update(kc, vc, k1, v1, S)
    lens = torch.full((B,), S + 1, dtype=torch.int32)
    if double_append:       # the reference's call pattern: the op appends the same K/V again at S + 1
        ref1 = oa.attention_decode_kvcache(q1, kc, vc, k1, v1, lens)
    else:
        ref1 = oa.attention_decode_kvcache(q1, kc, vc, None, None, lens)
    assert max_abs(w1.view(B, 1, H, d), ref1) < 2e-3
    assert torch.equal(attn.cache.k[:, :S + 1].cpu().view(torch.int16), kc[:, :S + 1].view(torch.int16))


# ------------------------------------------------------------------ q/k/v and gate/up fusion
def _quant_layers(method, shapes, K, seed):
    """One quantized layer per (out_features, bias) in `shapes`, all reading K input channels."""
    from llmqrt_b200.linear import FP8DynamicLinear, SqW8A8BBF16OBF16PerChannel, SqW8A8BBF16OBF16PerTensor, WQLinear_GEMM
    layers = []
    for i, (n, bias) in enumerate(shapes):
        lin = _linear(K, n, bias, seed + i)
        if method == "sq_channel":
            layers.append(SqW8A8BBF16OBF16PerChannel.from_linear(lin, 8, 0, init_only=False, dtype=torch.bfloat16))
        elif method == "sq_tensor":
            layers.append(SqW8A8BBF16OBF16PerTensor.from_linear(lin, 8, 0, init_only=False, dtype=torch.float16))
        elif method == "fp8_token":
            layers.append(FP8DynamicLinear.from_linear(lin, 8, 0, init_only=False, dtype=torch.bfloat16, per_tensor=False))
        elif method == "fp8_tensor":
            layers.append(FP8DynamicLinear.from_linear(lin, 8, 0, init_only=False, dtype=torch.bfloat16, per_tensor=True))
        else:
            G = 128
            wg = lin.weight.data.view(n, K // G, G)
            scales = ((wg.amax(-1) - wg.amin(-1)).clamp_min(1e-5) / 15)
            zeros = torch.round(-wg.amin(-1) / scales).clamp(0, 15)
            layers.append(WQLinear_GEMM.from_linear(lin, 4, G, init_only=False, scales=scales.t().contiguous(),
                                                    zeros=zeros.t().contiguous()))
    return layers


@pytest.mark.parametrize("method", ["sq_channel", "fp8_token", "awq"])
@pytest.mark.parametrize("tokens", [7, 200])
def test_fuse_qkv_equals_separate_projections(method, tokens):
    # ref fused_utils.py:43-104 fuses AWQ only; the schemes with run-time activation scales fuse here too
    from llmqrt_b200.fused_utils import fuse_qkv
    from tests.util import bits_equal
    K = 256
    q, k, v = _quant_layers(method, [(512, True), (128, True), (128, True)], K, 20)
    dt = torch.float16 if method == "awq" else torch.bfloat16
    x = torch.randn(1, tokens, K, generator=torch.Generator().manual_seed(5)).to(dt).cuda()
    want = torch.cat([q(x), k(x), v(x)], dim=-1)
    fused = fuse_qkv(torch.nn.ModuleList([q, k, v]), q, k, v)
    assert not isinstance(fused, tuple) and fused.out_features == 768
    got = fused(x)
    if method == "sq_channel":
        assert bits_equal(got, want)              # exact integer accumulators, same fp32 epilogue per column
    else:
        assert rel_fro(got, want) < 2e-3          # fp32 sums may be split over K differently for another N


@pytest.mark.parametrize("method", ["sq_tensor", "fp8_tensor"])
def test_fuse_qkv_leaves_per_tensor_schemes_alone(method):
    # q, k and v carry different per-tensor scales: like the reference (fused_utils.py:47-56) they stay separate
    from llmqrt_b200.fused_utils import fuse_qkv
    q, k, v = _quant_layers(method, [(256, True), (128, True), (128, True)], 256, 30)
    out = fuse_qkv(torch.nn.ModuleList([q, k, v]), q, k, v)
    assert isinstance(out, tuple) and out[0] is q and out[1] is k and out[2] is v


@pytest.mark.parametrize("method", ["sq_channel", "awq"])
def test_fused_gate_up_mlp(method):
    from llmqrt_b200.fused_utils import FusedGateUpMLP
    K, I = 256, 512
    gate, up = _quant_layers(method, [(I, False), (I, False)], K, 40)
    down = _quant_layers(method, [(K, False)], I, 50)[0]
    dt = torch.float16 if method == "awq" else torch.bfloat16
    x = torch.randn(3, 4, K, generator=torch.Generator().manual_seed(6)).to(dt).cuda()
    want = down(torch.nn.functional.silu(gate(x)) * up(x))
    got = FusedGateUpMLP(gate, up, down)(x)
    assert got.shape == want.shape and rel_fro(got, want) < 1e-2
