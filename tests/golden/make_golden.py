"""Generate the golden fixtures in this directory from the reference's own code.

Run once, in a container where the reference checkout is mounted:

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

It executes, on the CPU, the parts of the reference that are importable
without its CUDA extension, on small seeded inputs, and stores inputs and
outputs as .npz files next to this script.  Code that lives in modules which
cannot be imported as a whole (they pull in the missing extension or the
`accelerate` package) is obtained by parsing the file and executing only the
named function / class definitions; nothing is copied into this repository.

16-bit floats are stored as their raw uint16 bit patterns (suffix `_bits`
with a sibling `_dtype` entry), fp8 as raw uint8.
"""
from __future__ import annotations

import ast
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_defs(path: str, names: list[str], extra_globals: dict | None = None) -> dict:
    """Execute only the top-level defs/classes called `names` from a source file."""
    tree = ast.parse(open(path).read())
    body = [n for n in tree.body
            if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    assert len(body) == len(names), (path, names)
    ns = {"torch": torch, "nn": torch.nn, "Tuple": tuple, "Optional": object}
    ns.update(extra_globals or {})
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return ns


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def save(name: str, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            if v.dtype in (torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2):
                out[k + "_bits"] = bits(v)
                out[k + "_dtype"] = np.array(str(v.dtype))
            else:
                out[k] = v.numpy()
        else:
            out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: getattr(v, "shape", None) for k, v in out.items()})


def outlier_activations(M, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    cols = torch.randperm(K, generator=g)[: max(1, K // 100)]
    x[:, cols] *= 20.0
    return x.to(dtype)


def main(ref_root: str):
    sys.path.insert(0, ref_root)
    rt = os.path.join(ref_root, "runtime")

    # ---- SmoothQuant int8 quantizers: linear_sq.py:44-65 -------------------------------
    sq = load_defs(os.path.join(rt, "nn_models/modules/linear/linear_sq.py"),
                   ["quantize_activation_per_tensor_absmax", "quantize_activation_per_token_absmax"])
    for dt, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        x = outlier_activations(16, 896, dt, seed=0)
        x[3] = 0                                   # exercises the clamp(min=1e-5) branch
        x[5, :8] = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, -3.5], dtype=dt) * x[5].abs().max() / 127
        q_t, s_t = sq["quantize_activation_per_tensor_absmax"](x.clone())
        q_k, s_k = sq["quantize_activation_per_token_absmax"](x.clone())
        save(f"sq_quant_{tag}", x=x, q_tensor=q_t, s_tensor=s_t.reshape(1), q_token=q_k, s_token=s_k)

    # ---- per-token x per-channel dequant: quantization_utils.py:90-97 ----------------
    from runtime.utils import quantization_utils as qu
    g = torch.Generator().manual_seed(1)
    acc = torch.randint(-(2 ** 20), 2 ** 20, (16, 256), generator=g, dtype=torch.int32)
    w_s = (torch.rand(256, generator=g) * 1e-3).to(torch.float16)
    for dt, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        a_s = (torch.rand(16, 1, generator=g) * 1e-2).to(dt)
        y = qu.dequantize_activation_w_per_channel_a_per_token(acc.clone(), w_s, a_s)
        save(f"sq_dequant_{tag}", acc=acc, w_scale=w_s, a_scale=a_s, y=y)

    # ---- FP8 quantizers + dequantize-then-matmul fallback: linear_fp8.py:11-101 -------
    f8 = load_defs(os.path.join(rt, "nn_models/modules/linear/linear_fp8.py"),
                   ["per_tensor_quantize", "static_per_tensor_quantize", "per_token_quantize", "fp8_gemm"])
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16")):
        x = outlier_activations(16, 896, dt, seed=2)
        q_t, s_t = f8["per_tensor_quantize"](x.clone())
        q_k, s_k = f8["per_token_quantize"](x.clone())
        s_static = torch.tensor([0.037], dtype=torch.float32)
        q_s = f8["static_per_tensor_quantize"](x.clone(), s_static)
        save(f"fp8_quant_{tag}", x=x, q_tensor=q_t, s_tensor=s_t.reshape(1), q_token=q_k, s_token=s_k,
             s_static=s_static, q_static=q_s)
    g = torch.Generator().manual_seed(3)
    xq, xs = f8["per_token_quantize"](torch.randn(16, 128, generator=g).to(torch.bfloat16))
    wq, ws = f8["per_token_quantize"]((torch.randn(64, 128, generator=g) * 0.02).to(torch.bfloat16))
    bias = torch.randn(64, generator=g).to(torch.bfloat16)
    # the fallback multiplies A by A_scale without a cast, so the scale must already be 16-bit
    y = f8["fp8_gemm"](xq, xs.to(torch.bfloat16), wq, ws, bias, torch.bfloat16)
    save("fp8_fallback_linear", xq=xq, xs=xs, wq=wq, ws=ws, bias=bias, y=y)

    # ---- AWQ: packing_utils.py + Triton kernels under the interpreter ------------------
    from runtime.utils import packing_utils as pu
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), ".."))
    from oracle import awq as oawq
    K, N, G, M = 256, 64, 128, 4
    qweight, qzeros, scales = oawq.random_layer(K, N, G, seed=4)
    w_ref = pu.dequantize_gemm(qweight, qzeros, scales, 4, G)
    iw, iz = pu.unpack_awq(qweight, qzeros, 4)
    iw, iz = pu.reverse_awq_order(iw, iz, 4)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).to(torch.float16)
    arrays = dict(qweight=qweight, qzeros=qzeros, scales=scales, w_dequant=w_ref,
                  iweight=(iw & 0xF).to(torch.int32), izeros=(iz & 0xF).to(torch.int32), x=x,
                  group_size=G)
    try:
        from runtime.triton_kernels import awq_kernels as ak
        import triton
        out = torch.empty(K, N, dtype=torch.float16)
        ak.awq_dequantize_kernel[(triton.cdiv(N // 8, 32), triton.cdiv(K, 32))](
            qweight, scales, qzeros, G, out, N // 8, K, BLOCK_SIZE_X=32, BLOCK_SIZE_Y=32)
        arrays["w_dequant_triton"] = out
        c = torch.zeros(M, N, dtype=torch.float16)
        ak.awq_gemm_kernel[(triton.cdiv(M, 32) * triton.cdiv(N, 32), 8)](
            x, qweight, c, qzeros, scales, M, N, K, G,
            BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=32, SPLIT_K=8)
        arrays["y_gemm_triton"] = c
    except Exception as e:                                    # pragma: no cover
        print("triton interpreter unavailable:", repr(e))
    save("awq_small", **arrays)

    # ---- RMSNorm / RoPE / WindowedCache -------------------------------------------------
    from runtime.nn_models.modules.nonlinear.norm import RMSNorm
    from runtime.nn_models.modules.nonlinear.cache import WindowedCache
    rope_ns = load_defs(os.path.join(rt, "nn_models/modules/nonlinear/attn.py"), ["RoPE"])
    g = torch.Generator().manual_seed(6)
    for dt, tag in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        x = torch.randn(2, 3, 128, generator=g).to(dt)
        w = (1 + 0.1 * torch.randn(128, generator=g)).to(dt)
        y = RMSNorm(w, eps=1e-6)(x)
        rope = rope_ns["RoPE"](64, 32, "cpu", 1e6)
        xq = torch.randn(2, 3, 4, 64, generator=g).to(dt)
        xk = torch.randn(2, 3, 2, 64, generator=g).to(dt)
        oq, ok = rope.forward(xq, xk, start_pos=5, seqlen=3)
        cache = WindowedCache(2, 4, 2, 64, 16, "cpu")
        xv = torch.randn(2, 3, 2, 64, generator=g).to(torch.float16)
        cache.update_kv(values_store=xv, keys_store=ok.to(torch.float16), batch_size=2, start_pos=5, seqlen=3)
        save(f"glue_{tag}", norm_x=x, norm_w=w, norm_y=y, rope_q=xq, rope_k=xk, rope_oq=oq, rope_ok=ok,
             cache_v_in=xv, cache_k=cache.k, cache_v=cache.v)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
