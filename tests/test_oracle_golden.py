"""The CPU oracle against fixtures produced by the reference's own code (tests/golden)."""
import torch

from oracle import attention as oattn
from oracle import awq as oawq
from oracle import gemm as ogemm
from oracle import quant as oquant
from tests.util import bits_equal, load_golden, rel_fro


def test_int8_quantizers_match_reference():
    for tag in ("f16", "bf16"):
        g = load_golden(f"sq_quant_{tag}")
        q, s = oquant.quantize_int8(g["x"], per_token=True, scalar_div="true")
        assert torch.equal(q, g["q_token"]) and bits_equal(s, g["s_token"])
        q, s = oquant.quantize_int8(g["x"], per_token=False, scalar_div="true")
        assert torch.equal(q, g["q_tensor"]) and bits_equal(s.reshape(1), g["s_tensor"])


def test_int8_quantizer_reciprocal_mode_is_close():
    g = load_golden("sq_quant_f16")
    q, _ = oquant.quantize_int8(g["x"], per_token=True, scalar_div="reciprocal")
    assert (q.int() - g["q_token"].int()).abs().max() <= 1


def test_fp8_quantizers_match_reference():
    for tag in ("f16", "bf16"):
        g = load_golden(f"fp8_quant_{tag}")
        q, s = oquant.quantize_fp8(g["x"], per_token=True, scalar_div="true")
        assert bits_equal(q, g["q_token"]) and torch.equal(s, g["s_token"])
        q, s = oquant.quantize_fp8(g["x"], per_token=False, scalar_div="true")
        assert bits_equal(q, g["q_tensor"]) and torch.equal(s.reshape(1), g["s_tensor"])
        q = oquant.quantize_fp8_static(g["x"], g["s_static"])
        assert bits_equal(q, g["q_static"])


def test_per_token_per_channel_dequant_matches_reference():
    for tag, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        g = load_golden(f"sq_dequant_{tag}")
        y = ogemm.dequant_per_token_per_channel(g["acc"], g["w_scale"], g["a_scale"], None, dt)
        assert bits_equal(y, g["y"])


def test_fp8_rowwise_close_to_reference_fallback():
    # The reference's CPU fallback dequantizes to bf16 first, so it only agrees
    # with the fp32-epilogue kernel formula to bf16 rounding noise.
    g = load_golden("fp8_fallback_linear")
    y = ogemm.fp8_linear_rowwise(g["xq"], g["wq"], g["bias"], g["xs"], g["ws"].reshape(1, -1))
    assert rel_fro(y, g["y"]) < 1e-2


def test_awq_unpack_and_dequant_match_reference():
    g = load_golden("awq_small")
    assert torch.equal(oawq.unpack_cols(g["qweight"]), g["iweight"])
    assert torch.equal(oawq.unpack_cols(g["qzeros"]), g["izeros"])
    w = oawq.dequantize(g["qweight"], g["qzeros"], g["scales"], g["group_size"])
    assert bits_equal(w, g["w_dequant"])
    assert bits_equal(w, g["w_dequant_triton"])
    assert torch.equal(oawq.pack_cols(g["iweight"]), g["qweight"])


def test_awq_gemm_close_to_reference_triton():
    g = load_golden("awq_small")
    y = oawq.gemm(g["x"], g["qweight"], g["qzeros"], g["scales"], g["group_size"])
    assert rel_fro(y, g["y_gemm_triton"]) < 2e-3


def test_awq_k_major_repack_roundtrip():
    qw, _, _ = oawq.random_layer(64, 32, 32, seed=9)
    rp = oawq.repack_k_major(qw)
    w = oawq.unpack_cols(qw).numpy()
    for p in range(4):
        lo = (rp >> (4 * p)) & 0xF
        hi = (rp >> (4 * p + 16)) & 0xF
        assert (lo == w.T.reshape(32, 8, 8)[:, :, 2 * p]).all()
        assert (hi == w.T.reshape(32, 8, 8)[:, :, 2 * p + 1]).all()


def test_glue_matches_reference():
    for tag in ("f16", "bf16"):
        g = load_golden(f"glue_{tag}")
        assert bits_equal(oattn.rmsnorm(g["norm_x"], g["norm_w"], 1e-6), g["norm_y"])
        oq = oattn.rope_apply(g["rope_q"], 5, 1e6, 32)
        ok = oattn.rope_apply(g["rope_k"], 5, 1e6, 32)
        assert bits_equal(oq, g["rope_oq"]) and bits_equal(ok, g["rope_ok"])
        kc = torch.zeros_like(g["cache_k"])
        vc = torch.zeros_like(g["cache_v"])
        oattn.cache_update(kc, vc, ok, g["cache_v_in"], 5)
        assert bits_equal(kc, g["cache_k"]) and bits_equal(vc, g["cache_v"])


def test_int8_unit_test_procedure():
    # Shapes and construction of the reference's runtime/unittest/test_sq_linear.py:7-34
    # (CPU fp16 dequantize-then-linear as ground truth, atol 0.1).
    g = torch.Generator().manual_seed(0)
    B, M, N = 128, 512, 1024
    w = torch.randint(-128, 127, (N, M), generator=g, dtype=torch.int8)
    x = torch.randint(-128, 127, (B, M), generator=g, dtype=torch.int8)
    bias = torch.randn(N, generator=g).to(torch.float16)
    alpha, input_scale = 0.00334, 0.002
    y_gt = torch.nn.functional.linear(x.to(torch.float16) * input_scale, w.to(torch.float16) * alpha, bias)
    y = ogemm.int8_linear_per_tensor(x, w, bias, alpha * input_scale, 1.0)
    assert torch.allclose(y_gt, y, atol=0.1)


def test_attention_decode_equals_prefill_last_row():
    g = torch.Generator().manual_seed(1)
    B, S, Hq, Hkv, d = 2, 9, 4, 2, 16
    q = torch.randn(B, S, Hq, d, generator=g)
    k = torch.randn(B, S, Hkv, d, generator=g)
    v = torch.randn(B, S, Hkv, d, generator=g)
    full = oattn.attention_prefill(q, k, v)
    kc = torch.zeros(B, 12, Hkv, d)
    vc = torch.zeros(B, 12, Hkv, d)
    kc[:, : S - 1] = k[:, : S - 1]
    vc[:, : S - 1] = v[:, : S - 1]
    lens = torch.full((B,), S - 1, dtype=torch.int32)
    dec = oattn.attention_decode_kvcache(q[:, -1:], kc, vc, k[:, -1:], v[:, -1:], lens)
    assert torch.allclose(dec, full[:, -1:], atol=1e-6)
    assert torch.equal(kc[:, S - 1], k[:, S - 1])
