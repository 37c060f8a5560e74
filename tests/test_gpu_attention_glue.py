"""Parity of the attention and block-glue kernels against the CPU oracle and reference fixtures."""
import pytest
import torch

from tests.util import bits_equal, load_golden, max_abs, ulp_mismatch_fraction

pytestmark = pytest.mark.gpu

ATTN_TOL = 2e-3       # max abs error allowed on attention outputs


def _qkv(B, S, Hq, Hkv, d, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, S, Hq, d, generator=g).to(dtype), torch.randn(B, S, Hkv, d, generator=g).to(dtype),
            torch.randn(B, S, Hkv, d, generator=g).to(dtype))


# ------------------------------------------------------------------ prefill
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,S,Hq,Hkv,d", [(2, 64, 4, 2, 128), (1, 200, 14, 2, 64), (2, 129, 7, 1, 128),
                                          (1, 1, 4, 4, 64), (1, 515, 28, 4, 128)])
def test_prefill_causal(dtype, B, S, Hq, Hkv, d):
    from llmqrt_b200.attention import flash_attn_func
    from oracle import attention as oa
    q, k, v = _qkv(B, S, Hq, Hkv, d, dtype, S + Hq)
    out = flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=True)
    ref = oa.attention_prefill(q, k, v, causal=True)
    tol = ATTN_TOL if dtype == torch.float16 else 1.6e-2      # bf16 output has 8 mantissa bits
    assert max_abs(out, ref) < tol


def test_prefill_noncausal_softcap_and_strided_inputs():
    from llmqrt_b200.attention import flash_attn_func
    from oracle import attention as oa
    B, S, Hq, Hkv, d = 2, 96, 8, 2, 64
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * d, generator=g).to(torch.float16)       # fused projection output
    q = qkv[..., : Hq * d].reshape(B, S, Hq, d)
    k = qkv[..., Hq * d: (Hq + Hkv) * d].reshape(B, S, Hkv, d)
    v = qkv[..., (Hq + Hkv) * d:].reshape(B, S, Hkv, d)
    qc, kc, vc = (t.cuda() for t in (qkv[..., : Hq * d], qkv[..., Hq * d: (Hq + Hkv) * d], qkv[..., (Hq + Hkv) * d:]))
    qkv_c = qkv.cuda()
    qv = qkv_c[..., : Hq * d].view(B, S, Hq, d)
    kv = qkv_c[..., Hq * d: (Hq + Hkv) * d].view(B, S, Hkv, d)
    vv = qkv_c[..., (Hq + Hkv) * d:].view(B, S, Hkv, d)
    for causal, softcap in ((False, 0.0), (True, 30.0)):
        out = flash_attn_func(qv, kv, vv, causal=causal, softcap=softcap)
        ref = oa.attention_prefill(q, k, v, causal=causal, softcap=softcap)
        assert max_abs(out, ref) < ATTN_TOL


def test_prefill_full_size_properties():
    # batch 4 x 2048 tokens, 28/4 heads, head_dim 128: row 0 of every head attends only to key 0
    # (output == v[0]), and a causal run restricted to a prefix equals the prefix of the full run.
    from llmqrt_b200.attention import flash_attn_func
    B, S, Hq, Hkv, d = 4, 2048, 28, 4, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(B, S, Hq, d, generator=g, device="cuda", dtype=torch.float16)
    k = torch.randn(B, S, Hkv, d, generator=g, device="cuda", dtype=torch.float16)
    v = torch.randn(B, S, Hkv, d, generator=g, device="cuda", dtype=torch.float16)
    out = flash_attn_func(q, k, v, causal=True)
    assert torch.isfinite(out.float()).all()
    assert max_abs(out[:, 0], v[:, 0].repeat_interleave(Hq // Hkv, dim=1)) < 1e-3
    part = flash_attn_func(q[:, :300].contiguous(), k[:, :300].contiguous(), v[:, :300].contiguous(), causal=True)
    assert max_abs(out[:, :300], part) < 1e-3


def test_prefill_full_size_against_oracle():
    # batch 4 x 2048 tokens, 28/4 heads, head_dim 128, causal: sampled (batch, head, query row) triples,
    # among them the rows around the tile boundaries and the last one, against the fp64 oracle
    from llmqrt_b200.attention import flash_attn_func
    from oracle import attention as oa
    B, S, Hq, Hkv, d = 4, 2048, 28, 4, 128
    g = torch.Generator().manual_seed(4)
    q = torch.randn(B, S, Hq, d, generator=g).to(torch.float16)
    k = torch.randn(B, S, Hkv, d, generator=g).to(torch.float16)
    v = torch.randn(B, S, Hkv, d, generator=g).to(torch.float16)
    out = flash_attn_func(q.cuda(), k.cuda(), v.cuda(), causal=True).cpu()
    rows = [0, 1, 63, 64, 127, 128, 129, 255, 256, 1023, 1024, 2046, 2047] + \
        torch.randint(0, S, (19,), generator=g).tolist()
    worst = 0.0
    for b in range(B):
        for h in (0, 6, 7, 13, 27):
            hk = h // (Hq // Hkv)
            for r in rows:
                ref = oa.attention_prefill(q[b:b + 1, r:r + 1, h:h + 1], k[b:b + 1, :r + 1, hk:hk + 1],
                                           v[b:b + 1, :r + 1, hk:hk + 1], causal=True)
                worst = max(worst, max_abs(out[b, r, h], ref[0, 0, 0]))
    assert worst < ATTN_TOL


# ------------------------------------------------------------------ decode
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,Hq,Hkv,d,Smax,lens", [
    (4, 28, 4, 128, 600, [1, 17, 300, 599]),
    (3, 14, 2, 64, 260, [64, 255, 256]),
    (2, 8, 1, 128, 128, [5, 127]),
    (2, 4, 4, 64, 40, [0, 33]),
])
def test_decode_with_append(dtype, B, Hq, Hkv, d, Smax, lens):
    from llmqrt_b200.attention import flash_attn_with_kvcache
    from oracle import attention as oa
    g = torch.Generator().manual_seed(B * Hq + d)
    kc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype)
    vc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype)
    q = torch.randn(B, 1, Hq, d, generator=g).to(dtype)
    kn = torch.randn(B, 1, Hkv, d, generator=g).to(dtype)
    vn = torch.randn(B, 1, Hkv, d, generator=g).to(dtype)
    seqlens = torch.tensor(lens, dtype=torch.int32)
    kc_g, vc_g = kc.cuda(), vc.cuda()
    out = flash_attn_with_kvcache(q.cuda(), kc_g, vc_g, k=kn.cuda(), v=vn.cuda(), cache_seqlens=seqlens.cuda(),
                                  causal=True)
    ref = oa.attention_decode_kvcache(q, kc, vc, kn, vn, seqlens)           # also appends into kc / vc
    tol = ATTN_TOL if dtype == torch.float16 else 1.6e-2
    assert max_abs(out, ref) < tol
    assert bits_equal(kc_g.cpu(), kc) and bits_equal(vc_g.cpu(), vc)       # in-place append, nothing else touched


def test_decode_config_shape_long_contexts():
    # batch 32, 28/4 heads, head_dim 128, context lengths uniform in [512, 8192]; every sequence is
    # checked against the oracle
    from llmqrt_b200.attention import attn_decode
    from oracle import attention as oa
    B, Hq, Hkv, d, Smax = 32, 28, 4, 128, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn(B, Smax, Hkv, d, generator=g, device="cuda", dtype=torch.float16)
    vc = torch.randn(B, Smax, Hkv, d, generator=g, device="cuda", dtype=torch.float16)
    q = torch.randn(B, Hq, d, generator=g, device="cuda", dtype=torch.float16)
    lens = torch.randint(512, 8193, (B,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    out = attn_decode(q, kc, vc, lens.cuda(), Smax)
    assert torch.isfinite(out.float()).all()
    for b in range(B):
        L_b = int(lens[b])
        ref = oa.attention_decode_kvcache(q[b:b + 1].cpu().unsqueeze(1), kc[b:b + 1, :L_b].cpu(), vc[b:b + 1, :L_b].cpu(),
                                          None, None, lens[b:b + 1])
        assert max_abs(out[b], ref[0, 0]) < ATTN_TOL, b
    out2 = attn_decode(q, kc, vc, lens.cuda(), Smax)
    assert bits_equal(out, out2)                                            # fixed combine order: repeatable


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("lens", [[700, 1, 0, 513, 256], [40, 7, 64, 1, 33]])      # several KV splits / a single one
def test_decode_strided_q_and_fused_quantization(dtype, lens):
    # q read in place from a fused qkv row; the int8 row and scale must be exactly what the per-token
    # quantizer makes of the 16-bit output
    from llmqrt_b200.attention import attn_decode
    from oracle import quant as oq
    B, Hq, Hkv, d = len(lens), 28, 4, 128
    Smax = max(lens)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * d, generator=g).to(dtype).cuda()
    kc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype).cuda()
    seqlens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    q_view = qkv.view(B, Hq + 2 * Hkv, d)[:, :Hq]
    assert not q_view.is_contiguous()
    plain = attn_decode(q_view.contiguous(), kc, vc, seqlens, Smax)
    out, out_q, scale = attn_decode(q_view, kc, vc, seqlens, Smax, quantize=True)
    assert bits_equal(out, plain)
    q_ref, s_ref = oq.quantize_int8(out.reshape(B, Hq * d).cpu(), per_token=True)
    assert torch.equal(out_q.cpu(), q_ref) and torch.equal(scale.cpu(), s_ref.float().reshape(-1))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,d,lens,Smax", [(28, 4, 128, [1100, 1, 300, 513], 1200), (14, 2, 64, [64, 7, 33], 64),
                                                 (3, 1, 128, [5000, 4097], 5100)])
def test_decode_with_rotary_and_append_in_kernel(dtype, Hq, Hkv, d, lens, Smax):
    # rotary + cache write folded into the attention kernel == rope_kv_write kernel, then attention
    from llmqrt_b200 import glue
    from llmqrt_b200.attention import attn_decode, flash_attn_with_kvcache
    B = len(lens)
    g = torch.Generator().manual_seed(21)
    qkv = torch.randn(B, (Hq + 2 * Hkv) * d, generator=g).to(dtype).cuda()
    kc0 = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype).cuda()
    vc0 = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype).cuda()
    seqlens = torch.tensor(lens, dtype=torch.int32, device="cuda")                 # lengths INCLUDING the new token
    cos, sin = glue.rope_tables(d, Smax, 1e6, "cuda")
    rows = qkv.view(B, Hq + 2 * Hkv, d)
    # reference chain, one sequence at a time (the stand-alone rotary kernel takes one position per call)
    kc_ref, vc_ref = kc0.clone(), vc0.clone()
    q_rot = torch.empty(B, Hq, d, dtype=dtype, device="cuda")
    for b, L_b in enumerate(lens):
        r = rows[b:b + 1].unsqueeze(1).clone()                                     # [1, 1, heads, d]
        q1, k1, v1 = r[:, :, :Hq], r[:, :, Hq:Hq + Hkv], r[:, :, Hq + Hkv:]
        glue.rope_kv_write(q1, k1, v1, cos, sin, pos0=L_b - 1, k_cache=kc_ref[b:b + 1], v_cache=vc_ref[b:b + 1])
        q_rot[b] = q1[0, 0]
    want = attn_decode(q_rot, kc_ref, vc_ref, seqlens, Smax)
    kc, vc = kc0.clone(), vc0.clone()
    got, got_q, got_s = attn_decode(rows[:, :Hq], kc, vc, seqlens, Smax, quantize=True, k_new=rows[:, Hq:Hq + Hkv],
                                    v_new=rows[:, Hq + Hkv:], cos=cos, sin=sin)
    assert bits_equal(kc, kc_ref) and bits_equal(vc, vc_ref)                       # same rotation arithmetic, same rows
    assert bits_equal(got, want)
    # the flash-attn spelling of the same call: cache_seqlens are the lengths BEFORE the append
    kc2, vc2 = kc0.clone(), vc0.clone()
    out2 = flash_attn_with_kvcache(rows[:, :Hq].unsqueeze(1), kc2, vc2, k=rows[:, Hq:Hq + Hkv].unsqueeze(1),
                                   v=rows[:, Hq + Hkv:].unsqueeze(1), rotary_cos=cos, rotary_sin=sin,
                                   cache_seqlens=seqlens - 1, rotary_interleaved=False, max_seqlen_k=Smax)
    assert bits_equal(out2[:, 0], got) and bits_equal(kc2, kc)


def test_decode_append_on_a_full_cache_writes_nothing():
    # cache_seqlens == capacity: there is no row left for the new token.  The kernels clamp: nothing is
    # written (the guard rows behind the cache stay intact) and the sequence attends over the full cache.
    from llmqrt_b200.attention import attn_decode, flash_attn_with_kvcache
    B, Hq, Hkv, d, cap = 2, 8, 2, 128, 96
    g = torch.Generator().manual_seed(13)
    big_k = torch.randn(B + 1, cap, Hkv, d, generator=g).half().cuda()     # sequence b + 1 guards sequence b
    big_v = torch.randn(B + 1, cap, Hkv, d, generator=g).half().cuda()
    kc, vc = big_k[:B], big_v[:B]
    k0, v0 = big_k.clone(), big_v.clone()
    q = torch.randn(B, 1, Hq, d, generator=g).half().cuda()
    kn = torch.randn(B, 1, Hkv, d, generator=g).half().cuda()
    vn = torch.randn(B, 1, Hkv, d, generator=g).half().cuda()
    cos = torch.ones(cap, d // 2, device="cuda")
    sin = torch.zeros(cap, d // 2, device="cuda")
    full = torch.full((B,), cap, dtype=torch.int32, device="cuda")
    for rotary in (False, True):
        kw = dict(rotary_cos=cos, rotary_sin=sin, rotary_interleaved=False) if rotary else {}
        out = flash_attn_with_kvcache(q, kc, vc, k=kn, v=vn, cache_seqlens=full, causal=True, **kw)
        torch.cuda.synchronize()
        assert bits_equal(big_k, k0) and bits_equal(big_v, v0)
        want = attn_decode(q[:, 0], kc, vc, full, cap)
        assert max_abs(out[:, 0], want) < ATTN_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,lens,Smax", [(4, 1, [1100, 1, 300, 0, 513], 1200), (3, 1, [40, 7, 64], 64),
                                               (7, 1, [200, 199], 256), (4, 1, [5000, 4097], 5100),
                                               (28, 4, [1100, 1, 300, 0, 513, 77], 1200), (14, 2, [64, 3], 64),
                                               (16, 8, [130, 129, 1], 256), (28, 4, [5000, 4097], 5100),
                                               (6, 3, [70, 33, 128], 128), (14, 7, [200], 256),      # clusters of 3 and 7 blocks
                                               # enough sequences that two splits give way to one block per KV head
                                               (14, 2, [1100] * 60 + [1, 0, 513, 77], 1200)])
def test_decode_fused_quantization(dtype, Hq, Hkv, lens, Smax):
    # an unsplit sequence is quantized by the attention kernel itself (one block with one KV head -- a
    # tensor-parallel rank of 4 or 8 --, a thread-block cluster of the KV heads' blocks otherwise), a split
    # one by the merge kernel; both must be the per-token quantizer's bits
    from llmqrt_b200.attention import attn_decode
    from oracle import quant as oq
    B, d = len(lens), 128
    g = torch.Generator().manual_seed(Hq)
    q = torch.randn(B, Hq, d, generator=g).to(dtype).cuda()
    kc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(B, Smax, Hkv, d, generator=g).to(dtype).cuda()
    seqlens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    plain = attn_decode(q, kc, vc, seqlens, Smax)
    out, out_q, scale = attn_decode(q, kc, vc, seqlens, Smax, quantize=True)
    assert bits_equal(out, plain)
    q_ref, s_ref = oq.quantize_int8(out.reshape(B, Hq * d).cpu(), per_token=True)
    assert torch.equal(out_q.cpu(), q_ref) and torch.equal(scale.cpu(), s_ref.float().reshape(-1))


def test_decode_quantization_single_split_without_workspace():
    # short caches need no split partials, hence no workspace; the merge kernel still quantizes the rows
    from llmqrt_b200 import _lib as L
    from llmqrt_b200.attention import attn_decode
    from oracle import quant as oq
    B, Hq, Hkv, d, Smax = 3, 28, 4, 128, 64
    g = torch.Generator().manual_seed(9)
    q = torch.randn(B, Hq, d, generator=g).half().cuda()
    kc = torch.randn(B, Smax, Hkv, d, generator=g).half().cuda()
    vc = torch.randn(B, Smax, Hkv, d, generator=g).half().cuda()
    seqlens = torch.tensor([64, 3, 17], dtype=torch.int32, device="cuda")
    ref = attn_decode(q, kc, vc, seqlens, Smax)
    out = torch.empty_like(q)
    out_q = torch.empty(B, Hq * d, dtype=torch.int8, device="cuda")
    scale = torch.empty(B, dtype=torch.float32, device="cuda")
    L.call("llmqrt_attn_decode", L.ptr(q), Hq * d, L.ptr(kc), L.ptr(vc), kc.stride(0), kc.stride(1), L.ptr(seqlens),
           L.ptr(out), L.ptr(out_q), L.ptr(scale), L.dtype_code(q.dtype), B, Hq, Hkv, d, Smax, 0.0, None,
           L.stream(q.device))
    assert bits_equal(out, ref)
    q_ref, s_ref = oq.quantize_int8(out.reshape(B, Hq * d).cpu(), per_token=True)
    assert torch.equal(out_q.cpu(), q_ref) and torch.equal(scale.cpu(), s_ref.float().reshape(-1))


def test_decode_equals_last_row_of_prefill():
    from llmqrt_b200.attention import attn_decode, flash_attn_func
    B, S, Hq, Hkv, d = 2, 333, 28, 4, 128
    q, k, v = (t.cuda() for t in _qkv(B, S, Hq, Hkv, d, torch.float16, 11))
    full = flash_attn_func(q, k, v, causal=True)
    lens = torch.full((B,), S, dtype=torch.int32, device="cuda")
    dec = attn_decode(q[:, -1].contiguous(), k, v, lens, S)
    assert max_abs(dec, full[:, -1]) < 1e-3


# ------------------------------------------------------------------ glue
@pytest.mark.parametrize("tag", ["f16", "bf16"])
def test_rmsnorm_and_rope_match_reference_fixture(tag):
    from llmqrt_b200 import glue
    g = load_golden(f"glue_{tag}")
    y, _, _, _ = glue.rmsnorm(g["norm_x"].cuda(), g["norm_w"].cuda(), 1e-6)
    frac, dist = ulp_mismatch_fraction(y.cpu(), g["norm_y"])
    assert dist <= 1 and frac < 0.02          # fp32 reduction order differs from torch's: at most 1 ulp
    cos, sin = glue.rope_tables(64, 32, 1e6, "cuda")
    q, k = g["rope_q"].cuda(), g["rope_k"].cuda()
    kc = torch.zeros(2, 16, 2, 64, dtype=q.dtype, device="cuda")
    vc = torch.zeros_like(kc)
    v = g["cache_v_in"].to(q.dtype).cuda()
    glue.rope_kv_write(q, k, v, cos, sin, pos0=5, k_cache=kc, v_cache=vc)
    for got, want in ((q, g["rope_oq"]), (k, g["rope_ok"])):
        frac, dist = ulp_mismatch_fraction(got.cpu(), want)
        assert dist <= 1 and frac < 0.01      # fused multiply-add contraction of the complex product
    assert bits_equal(kc[:, 5:8].cpu(), k.cpu()) and bits_equal(vc[:, 5:8].cpu(), v.cpu())
    assert float(kc[:, :5].abs().max()) == 0 and float(kc[:, 8:].abs().max()) == 0
    # position taken from a device scalar
    q2, k2 = g["rope_q"].cuda(), g["rope_k"].cuda()
    glue.rope_kv_write(q2, k2, None, cos, sin, pos0=0, pos_dev=torch.tensor([5], dtype=torch.int32, device="cuda"))
    assert bits_equal(q2, q) and bits_equal(k2, k)


# 3584 and 8192: one block per row with the row in registers; 16384: cluster of blocks per row;
# 1001: scalar accesses
@pytest.mark.parametrize("H", [3584, 8192, 16384, 1001])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rmsnorm_residual_and_fused_quant(dtype, H):
    from llmqrt_b200 import glue
    from oracle import attention as oa
    from oracle import quant as oq
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, H, generator=g).to(dtype)
    r = torch.randn(5, H, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    y, h, q, s = glue.rmsnorm(x.cuda(), w.cuda(), 1e-6, residual=r.cuda(), quantize=True)
    h_ref = x + r
    assert bits_equal(h.cpu(), h_ref)
    frac, dist = ulp_mismatch_fraction(y.cpu(), oa.rmsnorm(h_ref, w, 1e-6))
    # a 1-ulp (fp32) difference of the row's 1/rms moves a few elements across a rounding boundary
    # of x*inv; the product with a weight above 1 can then land 2 ulp away
    assert dist <= 2 and frac < 0.02
    q_ref, s_ref = oq.quantize_int8(y.cpu(), per_token=True)              # quantizer applied to the kernel's own y
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.float().reshape(-1))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
# 18944, 9472, 2368: cluster of blocks with the slice in registers; 66056: slices staged in shared
# memory; 1001: scalar accesses
@pytest.mark.parametrize("I", [18944, 9472, 2368, 66056, 1001])
def test_silu_mul_and_fused_quant(dtype, I):
    from llmqrt_b200 import glue
    from oracle import quant as oq
    g = torch.Generator().manual_seed(2)
    gu = torch.randn(6, 2 * I, generator=g).to(dtype)
    h, q, s = glue.silu_mul(gu.cuda(), quantize=True)
    gate, up = gu[:, :I], gu[:, I:]
    ref = torch.nn.functional.silu(gate) * up
    frac, dist = ulp_mismatch_fraction(h.cpu(), ref)
    assert dist <= 1 and frac < 0.01          # expf on the GPU vs the CPU's exp
    q_ref, s_ref = oq.quantize_int8(h.cpu(), per_token=True)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref.float().reshape(-1))
