"""CPU-only tests: C-ABI exports, host-side tensor-parallel logic (gloo, world size 2), oracle TP emulation."""
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    import ctypes
    from llmqrt_b200 import _lib
    header = open(os.path.join(ROOT, "include", "llmqrt_b200.h")).read()
    declared = set(re.findall(r"\b(llmqrt_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/llmqrt_b200.h but not exported"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    assert _lib._lib.llmqrt_abi_version() == _lib.ABI_VERSION
    assert _lib.WORKSPACE_BYTES > 64 * 1024


def test_product_path_refuses_cpu_tensors():
    import pytest
    from llmqrt_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.int8_gemm_s32(torch.zeros(4, 16, dtype=torch.int8), torch.zeros(8, 16, dtype=torch.int8))


def test_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "llmqrt_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, re.M), f
                assert "tests.golden" not in src and "_work/" not in src, f


def test_reference_module_names_resolve_to_this_package():
    # runtime/csrc/bindings.cpp:7-14 is imported as runtime.sq_fp8_kernels (linear_sq.py:14,
    # linear_fp8.py:7-8); the AWQ kernels as runtime.triton_kernels.awq_kernels (linear_awq.py:14)
    code = ("import llmqrt_b200, sys; names = llmqrt_b200.install_reference_aliases(); "
            "from runtime.sq_fp8_kernels import w8a8_int8_linear_bbf16_obf16_per_tensor, "
            "cutlass_f8f8bf16_tensorwise_sm89, cutlass_f8f8bf16_rowwise_sm89; "
            "from runtime.triton_kernels.awq_kernels import awq_gemm_triton, awq_dequantize_triton; "
            "import runtime.sq_fp8_kernels as m; import llmqrt_b200.sq_fp8_kernels as ours; "
            "assert m is ours and 'runtime.sq_fp8_kernels' in names; "
            "assert awq_gemm_triton.__module__ == 'llmqrt_b200.triton_kernels.awq_kernels'; print('ok')")
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert p.returncode == 0 and p.stdout.strip().endswith("ok"), p.stdout + p.stderr


def test_head_assignment_partitions_heads():
    from llmqrt_b200.tp import head_assignment
    for hq, hkv in ((28, 4), (14, 2), (12, 2), (32, 8)):
        rep = hq // hkv
        for tp in (1, 2, 4, 8):
            if not (hkv % tp == 0 or (tp % hkv == 0 and tp // hkv <= rep)):
                continue
            seen = []
            for r in range(tp):
                q, kv = head_assignment(hq, hkv, tp, r)
                assert q and kv and all(h // rep in kv for h in q)          # every q head next to its KV head
                assert len(q) % len(kv) == 0 and len(q) // len(kv) <= 8
                seen += q
            assert sorted(seen) == list(range(hq))                           # each query head exactly once
    q, kv = head_assignment(28, 4, 8, 0)
    assert (q, kv) == ([0, 1, 2, 3], [0])
    q, kv = head_assignment(28, 4, 8, 1)
    assert (q, kv) == ([4, 5, 6], [0])


def test_gpu_worker_models_divide_among_their_ranks():
    # the model shapes tests/tp_worker.py builds at each world size must be shardable there (a 4 / 2-head
    # model cannot be spread over 8 ranks: more ranks per KV head than query heads in its group)
    from llmqrt_b200.tp import head_assignment
    src = open(os.path.join(ROOT, "tests", "tp_worker.py")).read()
    m = re.search(r"num_heads=(\d+),\s*num_kv_heads=(\d+)", src)
    assert m, "tp_worker.py no longer spells out its 8-rank model"
    big = (int(m.group(1)), int(m.group(2)))
    for world, (hq, hkv) in ((2, (4, 2)), (4, (4, 2)), (8, big)):
        seen = []
        for r in range(world):
            q, kv = head_assignment(hq, hkv, world, r)
            assert q and kv
            seen += q
        assert sorted(seen) == list(range(hq))
    with pytest.raises(ValueError):
        head_assignment(4, 2, 8, 0)


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from llmqrt_b200.tp import allreduce_sum, greedy_select
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
g = torch.Generator().manual_seed(7)
logits = torch.randn(5, 64, generator=g)
logits[0, 40] = logits[0, 3] = 9.0                      # tie across shards: lowest token id must win
shard = logits[:, rank * 32:(rank + 1) * 32]
val, idx = shard.max(dim=-1)
tok = greedy_select(val, idx + rank * 32, 2)
assert torch.equal(tok, logits.argmax(dim=-1)), (tok, logits.argmax(dim=-1))
x = torch.full((3, 4), float(rank + 1))
assert torch.equal(allreduce_sum(x, 2), torch.full((3, 4), 3.0))
dist.destroy_process_group()
print("ok", rank)
"""


def test_greedy_select_and_allreduce_world_size_2_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29600 + os.getpid() % 300)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs


def test_oracle_tensor_parallel_emulation_matches_single_rank():
    # Row-parallel partial sums with per-rank activation scales must stay close to the unsharded model.
    from llmqrt_b200.tp import head_assignment, rows_of_heads
    from oracle.qwen2 import Qwen2Oracle

    class Cfg:
        hidden, head_dim, rms_eps, rope_theta, dtype = 64, 16, 1e-6, 1e6, torch.bfloat16
    Hq, Hkv, I, V, d = 4, 2, 96, 128, 16
    g = torch.Generator().manual_seed(0)

    def rnd(*shape):
        return (torch.randn(*shape, generator=g) * 0.05).to(torch.bfloat16)

    def quant(w):
        s = (w.float().abs().amax(1, keepdim=True) / 127).clamp_min(1e-8)
        return torch.round(w.float() / s).clamp(-128, 127).to(torch.int8), s.reshape(-1)

    full = dict(wq=rnd(Hq * d, 64), wk=rnd(Hkv * d, 64), wv=rnd(Hkv * d, 64), bq=rnd(Hq * d), bk=rnd(Hkv * d),
                bv=rnd(Hkv * d), wo=rnd(64, Hq * d), wg=rnd(I, 64), wu=rnd(I, 64), wd=rnd(64, I))
    embed, lm_head = rnd(V, 64) * 10, rnd(V, 64)

    def shards(tp):
        out = []
        for r in range(tp):
            qh, kh = head_assignment(Hq, Hkv, tp, r)
            qr, kr = rows_of_heads(qh, d), rows_of_heads(kh, d)
            i0, i1 = r * I // tp, (r + 1) * I // tp
            wqkv, sqkv = quant(torch.cat([full["wq"][qr], full["wk"][kr], full["wv"][kr]]))
            wo, so = quant(full["wo"][:, qr])
            wgu, sgu = quant(torch.cat([full["wg"][i0:i1], full["wu"][i0:i1]]))
            wd, sd = quant(full["wd"][:, i0:i1])
            layer = dict(ln1=torch.ones(64, dtype=torch.bfloat16), ln2=torch.ones(64, dtype=torch.bfloat16), wqkv=wqkv,
                         sqkv=sqkv, bqkv=torch.cat([full["bq"][qr], full["bk"][kr], full["bv"][kr]]), wo=wo, so=so,
                         wgu=wgu, sgu=sgu, wd=wd, sd=sd)
            out.append(dict(hq=len(qh), hkv=len(kh), embed=embed, norm_f=torch.ones(64, dtype=torch.bfloat16),
                            lm_head=lm_head[r * V // tp:(r + 1) * V // tp], layers=[layer]))
        return out

    toks = torch.randint(0, V, (2, 5), generator=g)
    l1 = Qwen2Oracle(Cfg, shards(1), 2, 8).forward(toks).float()
    l2 = Qwen2Oracle(Cfg, shards(2), 2, 8).forward(toks).float()
    assert l1.shape == l2.shape == (2, V)
    assert float((l1 - l2).norm() / l1.norm()) < 0.05


# ---------------------------------------------------------------------------------------------
# state-dict sharding (column / row tensor parallelism of loaded quantized layers)
# ---------------------------------------------------------------------------------------------
def test_split_points_respect_units():
    from llmqrt_b200.tp import split_points
    assert split_points(18944, 8, 128) == [0, 2432, 4864, 7296, 9728, 12032, 14336, 16640, 18944]   # 148 groups: 19 x 4 + 18 x 4
    assert split_points(18944, 8, 16)[1] == 2368
    assert split_points(96, 2, 16) == [0, 48, 96]
    import pytest
    with pytest.raises(ValueError):
        split_points(100, 2, 16)


def test_shard_linear_state_awq_blocks_and_errors():
    import pytest
    from llmqrt_b200.tp import shard_linear_state
    from oracle import awq as oa
    K, N, G = 256, 64, 64
    qw, qz, sc = oa.random_layer(K, N, G, seed=3)
    st = {"qweight": qw, "qzeros": qz, "scales": sc, "bias": torch.arange(N, dtype=torch.float16)}
    w = oa.dequantize(qw, qz, sc, G)                                     # [K, N]
    col = shard_linear_state(st, "awq", "column", (16, 48))
    assert torch.equal(oa.dequantize(col["qweight"], col["qzeros"], col["scales"], G), w[:, 16:48])
    assert torch.equal(col["bias"], st["bias"][16:48])
    heads = list(range(8, 16)) + list(range(40, 48))                     # two separate aligned runs of 8 columns
    col2 = shard_linear_state(st, "awq", "column", heads)
    assert torch.equal(oa.dequantize(col2["qweight"], col2["qzeros"], col2["scales"], G), w[:, heads])
    row = shard_linear_state(st, "awq", "row", (64, 192), keep_bias=False)
    assert torch.equal(oa.dequantize(row["qweight"], row["qzeros"], row["scales"], G), w[64:192])
    assert float(row["bias"].abs().max()) == 0
    with pytest.raises(ValueError, match="whole"):
        shard_linear_state(st, "awq", "column", (4, 36))                 # cuts through a packed word
    with pytest.raises(ValueError, match="whole"):
        shard_linear_state(st, "awq", "row", (32, 160))                  # cuts through a quantization group


_SHARD_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from llmqrt_b200.tp import shard_decoder_layer, head_assignment
from oracle import awq as oa, gemm as og, quant as oq
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + sys.argv[2], rank=int(sys.argv[3]), world_size=2)
rank, tp = dist.get_rank(), 2
H, Hq, Hkv, d, I, G = 128, 4, 2, 32, 256, 64
g = torch.Generator().manual_seed(11)                                    # the same full checkpoint on every rank
x = torch.randn(6, H, generator=g).to(torch.float16)

def linear_sq(st, a):                                                    # per-token x per-channel int8 linear (CPU oracle)
    aq, a_s = oq.quantize_int8(a, per_token=True)
    return og.int8_linear_per_channel(aq, st["qweight"], st.get("bias"), a_s.float(), st["weight_scale"].float(), torch.float16)

def linear_awq(st, a):
    y = oa.gemm(a, st["qweight"], st["qzeros"], st["scales"], G)
    return y if st.get("bias") is None else (y.float() + st["bias"].float()).to(torch.float16)

def make_sq(n, k, bias):
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.float16)
    q, s = oq.quantize_weight_int8_per_channel(w)
    st = {"qweight": q, "weight_scale": s.float().reshape(-1)}
    if bias: st["bias"] = (torch.randn(n, generator=g) * 0.1).to(torch.float16)
    return st

def make_awq(n, k, bias):
    qw, qz, sc = oa.random_layer(k, n, G, seed=int(torch.randint(0, 1 << 30, (1,), generator=g)))
    st = {"qweight": qw, "qzeros": qz, "scales": sc}
    if bias: st["bias"] = (torch.randn(n, generator=g) * 0.1).to(torch.float16)
    return st

for method, make, lin, tol in (("sq", make_sq, linear_sq, 3e-2), ("awq", make_awq, linear_awq, 3e-3)):
    full = {"q_proj": make(Hq * d, H, True), "k_proj": make(Hkv * d, H, True), "v_proj": make(Hkv * d, H, True),
            "o_proj": make(H, Hq * d, False), "gate_proj": make(I, H, False), "up_proj": make(I, H, False),
            "down_proj": make(H, I, True)}
    mine = shard_decoder_layer(full, method, Hq, Hkv, d, tp, rank)
    # column-parallel outputs are slices of the full outputs, bit for bit
    qh, kh = head_assignment(Hq, Hkv, tp, rank)
    q_full, q_mine = lin(full["q_proj"], x), lin(mine["q_proj"], x)
    assert torch.equal(q_mine, q_full.view(6, Hq, d)[:, qh].reshape(6, -1)), method
    # attention stand-in: this rank's q rows go through o_proj (row-parallel), then the MLP
    o_part = lin(mine["o_proj"], q_mine).float()
    dist.all_reduce(o_part)                                              # sum of the ranks' 16-bit partial outputs
    o_full = lin(full["o_proj"], q_full).float()
    err = float((o_part - o_full).norm() / o_full.norm())
    assert err < tol, (method, "o_proj", err)
    h = o_full.to(torch.float16)
    act = lambda st: (torch.nn.functional.silu(lin(st["gate_proj"], h).float()) * lin(st["up_proj"], h).float()).to(torch.float16)
    d_part = lin(mine["down_proj"], act(mine)).float()
    dist.all_reduce(d_part)
    d_full = lin(full["down_proj"], act(full)).float()
    err = float((d_part - d_full).norm() / d_full.norm())
    assert err < tol, (method, "down_proj", err)                         # (the bias is added once: kept on rank 0 only)
dist.destroy_process_group()
print("ok", rank)
"""


def test_shard_decoder_layer_world_size_2_gloo(tmp_path):
    script = tmp_path / "shard_worker.py"
    script.write_text(_SHARD_WORKER)
    port = str(29100 + os.getpid() % 300)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, port, str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
