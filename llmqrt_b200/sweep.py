"""Shape sweep of the quantized GEMMs and the attention kernels against their rooflines.

    python -m llmqrt_b200.sweep [--what int8,fp8,awq,attn] [--reps 20] [--hbm GB/s] [--bf16 TFLOP/s]

Times every operator shape of the stated configurations on the current GPU: seeded synthetic inputs,
each shape replayed from a CUDA graph that rotates over enough distinct weight (or KV) buffers to
exceed L2, CUDA events around the replays.  Prints one line per shape: time, algorithmic GB/s and
TOP/s, the lower bound max(bytes / HBM, flops / pipe) and the fraction of it that was reached.

Peaks default to the pool's measured copy bandwidth and cuBLAS bf16 rate (the 8-bit pipes are taken
as twice the bf16 figure, their nominal ratio); pass the box's own numbers to override.

Configurations (shapes of the checkpoints the reference's examples quantize):
  int8 : SmoothQuant per-token x per-channel, X[16, 896] . W[4864, 896]^T, plus the Qwen2-7B decode
         shapes at M = 64 and the same at M = 4096;
  fp8  : e4m3 row-wise, all Qwen2-0.5B linears, M in {1, 16, 64, 1024, 4096};
  awq  : W4A16 group 128, Qwen2-1.5B linears (fused qkv, o, gate, fused gate_up, down), M in {1, 16, 256, 2048};
  attn : Qwen2-7B heads (28 / 4, d = 128): decode batch 32 with context lengths uniform in
         [512, 8192]; causal prefill 4 x 2048.
"""
from __future__ import annotations

import argparse
import math

import torch

L2_BYTES = 126 << 20


def _time_graph(body, reps: int) -> float:
    """Seconds per replay of `body` captured in a CUDA graph."""
    body()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3 / reps


def _copies(nbytes: int) -> int:
    """Distinct buffers to rotate over so that the working set exceeds L2 (at least 2, at most 64)."""
    return max(2, min(64, math.ceil(1.5 * L2_BYTES / max(nbytes, 1))))


def _report(tag, M, N, K, secs, nbytes, flops, hbm, pipe):
    bound = max(nbytes / hbm, flops / pipe)
    which = "hbm" if nbytes / hbm >= flops / pipe else "pipe"
    print(f"{tag:22s} M={M:5d} N={N:6d} K={K:6d}  {secs * 1e6:9.2f} us  {nbytes / secs / 1e9:8.1f} GB/s  "
          f"{flops / secs / 1e12:8.2f} TOP/s  bound {bound * 1e6:8.2f} us ({which})  frac {bound / secs:5.3f}")


def sweep_int8(reps, hbm, pipe8):
    from . import ops
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    shapes = [("sq qwen2-0.5b gate", 16, 4864, 896)]
    for M in (64, 4096):
        shapes += [(f"sq 7b qkv", M, 4608, 3584), ("sq 7b o", M, 3584, 3584), ("sq 7b gate_up", M, 37888, 3584),
                   ("sq 7b down", M, 3584, 18944)]
    for tag, M, N, K in shapes:
        n = _copies(N * K)
        ws = [torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8) for _ in range(n)]
        a = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
        sa = torch.rand(M, generator=g, device=dev) * 1e-2
        sw = torch.rand(N, generator=g, device=dev) * 1e-2
        secs = _time_graph(lambda: [ops.int8_linear_per_channel(a, w, None, sa, sw, torch.bfloat16) for w in ws], reps) / n
        _report(tag, M, N, K, secs, M * K + N * K + 2 * M * N + 4 * (M + N), 2 * M * N * K, hbm, pipe8)


def sweep_fp8(reps, hbm, pipe8):
    from . import ops
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    for tag, N, K in (("fp8 q/o", 896, 896), ("fp8 k/v", 128, 896), ("fp8 gate/up", 4864, 896), ("fp8 down", 896, 4864)):
        for M in (1, 16, 64, 1024, 4096):
            n = _copies(N * K)
            ws = [(torch.randn(N, K, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn) for _ in range(n)]
            a = torch.randn(M, K, generator=g, device=dev).to(torch.float8_e4m3fn)
            sa = torch.rand(M, 1, generator=g, device=dev) * 1e-2
            sw = torch.rand(1, N, generator=g, device=dev) * 1e-2
            secs = _time_graph(lambda: [ops.fp8_linear_rowwise(a, w, None, sa, sw) for w in ws], reps) / n
            _report(tag, M, N, K, secs, M * K + N * K + 2 * M * N + 4 * (M + N), 2 * M * N * K, hbm, pipe8)


def _awq_layer(N, K, G, gen, dev):
    """Random AWQ layer in the reference's storage layout (nibbles uniform, scales ~ U(0.001, 0.02)):
    (qweight [K, N/8], scales [K/G, N], qzeros [K/G, N/8])."""
    qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), generator=gen, device=dev, dtype=torch.int32)
    qzeros = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // G, N // 8), generator=gen, device=dev, dtype=torch.int32)
    scales = (torch.rand(K // G, N, generator=gen, device=dev) * 0.019 + 0.001).half()
    return qweight, scales, qzeros


def sweep_awq(reps, hbm, pipe16):
    from . import ops
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    G = 128
    for tag, N, K in (("awq qkv", 2048, 1536), ("awq o", 1536, 1536), ("awq gate", 8960, 1536),
                      ("awq gate_up", 17920, 1536), ("awq down", 1536, 8960)):
        for M in (1, 16, 256, 2048):
            wbytes = K * N // 2 + (K // G) * N * 2 + (K // G) * N // 2
            n = _copies(wbytes)
            layers = [ops.AwqPacked(*_awq_layer(N, K, G, g, dev)) for _ in range(n)]
            x = torch.randn(M, K, generator=g, device=dev).half()
            secs = _time_graph(lambda: [ops.awq_gemm(x, p) for p in layers], reps) / n
            _report(tag, M, N, K, secs, 2 * M * K + wbytes + 2 * M * N, 2 * M * N * K, hbm, pipe16)


def sweep_attn(reps, hbm, pipe16):
    from .attention import attn_decode, flash_attn_func
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    B, Hq, Hkv, d, Smax = 32, 28, 4, 128, 8192
    lens = torch.randint(512, 8193, (B,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    kc = torch.randn(B, Smax, Hkv, d, generator=g, device=dev, dtype=torch.float16)     # 268 MB each: beyond L2
    vc = torch.randn(B, Smax, Hkv, d, generator=g, device=dev, dtype=torch.float16)
    q = torch.randn(B, Hq, d, generator=g, device=dev, dtype=torch.float16)
    ld = lens.to(dev)
    secs = _time_graph(lambda: attn_decode(q, kc, vc, ld, Smax), reps)
    ctx = int(lens.sum())
    nbytes = ctx * Hkv * d * 2 * 2 + 2 * B * Hq * d * 2
    _report("attn decode b32", B, ctx // B, d, secs, nbytes, 4 * ctx * Hq * d, hbm, pipe16)
    del kc, vc
    Bp, S = 4, 2048
    qs = [torch.randn(Bp, S, Hq, d, generator=g, device=dev, dtype=torch.float16) for _ in range(2)]
    ks = [torch.randn(Bp, S, Hkv, d, generator=g, device=dev, dtype=torch.float16) for _ in range(2)]
    vs = [torch.randn(Bp, S, Hkv, d, generator=g, device=dev, dtype=torch.float16) for _ in range(2)]
    secs = _time_graph(lambda: [flash_attn_func(a, b, c, causal=True) for a, b, c in zip(qs, ks, vs)], reps) / 2
    _report("attn prefill 4x2048", Bp * S, S, d, secs, Bp * S * (2 * Hq + 2 * Hkv) * d * 2, 4 * Bp * Hq * S * S * d // 2,
            hbm, pipe16)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--what", default="int8,fp8,awq,attn")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--hbm", type=float, default=6545.0, help="HBM bandwidth peak, GB/s")
    ap.add_argument("--bf16", type=float, default=1641.6, help="dense bf16 tensor peak, TFLOP/s")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("llmqrt_b200.sweep needs a CUDA device")
    hbm, pipe16 = args.hbm * 1e9, args.bf16 * 1e12
    print(f"peaks: HBM {args.hbm:.0f} GB/s, 16-bit pipe {args.bf16:.1f} TFLOP/s, 8-bit pipes {2 * args.bf16:.1f} TOP/s")
    for what in args.what.split(","):
        {"int8": lambda: sweep_int8(args.reps, hbm, 2 * pipe16), "fp8": lambda: sweep_fp8(args.reps, hbm, 2 * pipe16),
         "awq": lambda: sweep_awq(args.reps, hbm, pipe16), "attn": lambda: sweep_attn(args.reps, hbm, pipe16)}[what]()


if __name__ == "__main__":
    main()
