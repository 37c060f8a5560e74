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
