"""Pins the attention oracle, and the kernels, to the flash-attn package the reference calls.

The reference's attention arithmetic is not in its tree: runtime/nn_models/modules/nonlinear/attn.py
imports flash_attn_func / flash_attn_with_kvcache from the pip package flash-attn (line 11) and calls
them at lines 290-298 (prefill) and 305-315 (decode) with exactly the keyword sets used below.  Where
that package is installed and runs on this GPU, its outputs are the reference's outputs: the oracle
and the CUDA kernels must both agree with them.  Where it cannot run, the tests skip with the
package's own message as the reason.
"""
import pytest
import torch

from tests.util import bits_equal, max_abs

pytestmark = pytest.mark.gpu

TOL_F16 = 2e-3        # max abs, the tolerance of the attention parity gate
TOL_BF16 = 1.6e-2     # bf16 outputs carry 8 mantissa bits


def _flash_attn():
    try:
        import flash_attn
        from flash_attn import flash_attn_func, flash_attn_with_kvcache
    except Exception as e:                                  # not installed / binary does not load
        pytest.skip(f"flash_attn cannot be imported: {type(e).__name__}: {e}")
    try:                                                    # one tiny call decides whether it runs on this GPU
        t = torch.randn(1, 16, 2, 64, device="cuda", dtype=torch.float16)
        flash_attn_func(t, t, t, causal=True)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"flash_attn {getattr(flash_attn, '__version__', '?')} does not run on this GPU: "
                    f"{type(e).__name__}: {str(e)[:300]}")
    return flash_attn_func, flash_attn_with_kvcache


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,S,Hq,Hkv,d", [(2, 64, 4, 2, 128), (1, 200, 14, 2, 64), (2, 515, 28, 4, 128),
                                          (1, 2048, 28, 4, 128)])
def test_prefill_oracle_and_kernel_match_flash_attn(dtype, B, S, Hq, Hkv, d):
    fa_func, _ = _flash_attn()
    from llmqrt_b200.attention import flash_attn_func
    from oracle import attention as oa
    g = torch.Generator().manual_seed(S + Hq)
    q = torch.randn(B, S, Hq, d, generator=g).to(dtype)
    k = torch.randn(B, S, Hkv, d, generator=g).to(dtype)
    v = torch.randn(B, S, Hkv, d, generator=g).to(dtype)
    # keyword set of attn.py:290-298 (softcap 0.0: the reference's default for Qwen2)
    ref = fa_func(q.cuda(), k.cuda(), v.cuda(), causal=True, softcap=0.0)
    tol = TOL_F16 if dtype == torch.float16 else TOL_BF16
    out = flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=True, softcap=0.0)
    assert max_abs(out, ref) < tol                          # kernel == the reference's implementation
    if S <= 515:                                            # the O(S^2) fp64 oracle on the smaller cases
        assert max_abs(oa.attention_prefill(q, k, v, causal=True), ref) < tol      # oracle == the same


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Hq,Hkv,d,Smax,lens", [
    (4, 28, 4, 128, 600, [1, 17, 300, 599]),
    (3, 14, 2, 64, 260, [64, 255, 256]),
    (8, 28, 4, 128, 4200, [512, 4199, 1000, 2048, 3333, 777, 4096, 1]),
])
def test_decode_oracle_and_kernel_match_flash_attn(dtype, B, Hq, Hkv, d, Smax, lens):
    _, fa_kvcache = _flash_attn()
    from llmqrt_b200.attention import flash_attn_with_kvcache
    from oracle import attention as oa
    g = torch.Generator().manual_seed(B * Hq + d)
    kc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype)
    vc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype)
    q = torch.randn(B, 1, Hq, d, generator=g).to(dtype)
    kn = torch.randn(B, 1, Hkv, d, generator=g).to(dtype)
    vn = torch.randn(B, 1, Hkv, d, generator=g).to(dtype)
    seqlens = torch.tensor(lens, dtype=torch.int32)
    # keyword set of attn.py:305-315
    kc_f, vc_f = kc.cuda(), vc.cuda()
    ref = fa_kvcache(q=q.cuda(), k=kn.cuda(), k_cache=kc_f, v=vn.cuda(), v_cache=vc_f,
                     cache_seqlens=seqlens.cuda(), causal=True, softcap=0.0)
    kc_o, vc_o = kc.cuda(), vc.cuda()
    out = flash_attn_with_kvcache(q=q.cuda(), k=kn.cuda(), k_cache=kc_o, v=vn.cuda(), v_cache=vc_o,
                                  cache_seqlens=seqlens.cuda(), causal=True, softcap=0.0)
    tol = TOL_F16 if dtype == torch.float16 else TOL_BF16
    assert max_abs(out, ref) < tol
    assert bits_equal(kc_o, kc_f) and bits_equal(vc_o, vc_f)              # the same in-place append
    kc_c, vc_c = kc.clone(), vc.clone()
    want = oa.attention_decode_kvcache(q, kc_c, vc_c, kn, vn, seqlens)
    assert max_abs(want, ref) < tol
    assert bits_equal(kc_c, kc_f.cpu()) and bits_equal(vc_c, vc_f.cpu())
