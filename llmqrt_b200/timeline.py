"""In-situ kernel timeline of one replayed decode step of the Qwen2-7B int8 decoder (1 GPU).

Needs a library built with the timeline marks compiled in:

    LLMQRT_NVCC_FLAGS=-DLLMQRT_TIMELINE python llmqrt_b200/build.py --force
    python -m llmqrt_b200.timeline [--batch 64] [--prompt-len 1024] [--layers 28]
    python llmqrt_b200/build.py --force            # back to the product build

Block 0 of every instrumented kernel records global-timer marks ("enter" at kernel entry, "ready"
right after the dependency wait; the tcgen05 GEMM also its pipeline stages).  A kernel's duration
inside the CUDA-graph replay is taken from its own "ready" mark to the next kernel's, which includes
the hand-over between the two.  No profiler is involved; the marks cost the marking thread a few
hundred ns each (the GEMM's are SM-clock readings parked in shared memory and cost next to nothing).
"""
from __future__ import annotations

import argparse
import collections
import ctypes

import numpy as np
import torch

NAMES = {1: "gemm.enter", 2: "gemm.ready", 3: "gemm.done", 4: "gemm.prev_last_block_done",
         10: "rms.enter", 11: "rms.ready", 20: "silu.enter", 21: "silu.ready", 30: "rope.enter", 31: "rope.ready",
         40: "attn.enter", 41: "attn.ready", 50: "merge.enter", 51: "merge.ready",
         52: "g.start", 53: "g.setup_done", 54: "g.first_stage_full", 55: "g.mmas_issued", 56: "g.accumulator_full",
         57: "g.tail_done", 58: "g.block_synced", 59: "g.partial_parked", 60: "g.slices_sent", 61: "g.slices_landed",
         62: "g.epilogue_done"}
LAYER_PATTERN = ["rmsnorm_1", "qkv_gemm", "attention", "merge+quant", "o_gemm", "rmsnorm_2", "gate_up_gemm",
                 "silu_mul", "down_gemm"]


def _dump(lib, reset: bool):
    events = []
    for unit in ("gemm", "glue", "attn"):
        try:
            fn = getattr(lib, "llmqrt_timeline_" + unit)
        except AttributeError:
            raise SystemExit("this library was built without -DLLMQRT_TIMELINE (see the module docstring)") from None
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        buf = np.zeros(1 << 15, dtype=np.uint64)
        n = fn(buf.ctypes.data, buf.size, int(reset))
        if n < 0:
            raise SystemExit("reading the timeline buffer failed")
        events += [(int(v) & ~0x3f, int(v) & 0x3f) for v in buf[:n]]
    return sorted(events)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--show-layer", type=int, default=2, help="layer whose raw marks are listed")
    args = ap.parse_args()
    from . import _lib
    from .qwen2 import Qwen2Config, Qwen2Decoder
    dev = torch.device("cuda:0")
    cfg = Qwen2Config.qwen2_7b()
    cfg.num_layers = args.layers
    model = Qwen2Decoder(cfg, dev, batch=args.batch, max_seq_len=args.prompt_len + 40, tp=1, rank=0, group=None, seed=0)
    prompt = torch.randint(0, cfg.vocab, (args.batch, args.prompt_len), generator=torch.Generator().manual_seed(0)).to(dev)
    tok = model.prefill(prompt).clone()
    for _ in range(6):
        tok = model.decode_step(tok)
    torch.cuda.synchronize()
    _dump(_lib._lib, True)
    model.decode_step(tok)
    torch.cuda.synchronize()
    ev = _dump(_lib._lib, True)
    ev = [e for e in ev if e[1] != 4 or e[0] >= min(t for t, i in ev if i != 4)]   # drop the previous step's last-block mark
    t0 = ev[0][0]
    print(f"{len(ev)} marks over {(ev[-1][0] - t0) / 1e3:.1f} us (one decode step, batch {args.batch}, context {args.prompt_len + 7})")
    ready = [(t, NAMES[i]) for t, i in ev if NAMES.get(i, "").endswith("ready")]
    per = collections.defaultdict(list)
    n_layer_kernels = len(LAYER_PATTERN) * cfg.num_layers
    for k in range(min(n_layer_kernels, len(ready) - 1)):
        per[LAYER_PATTERN[k % len(LAYER_PATTERN)]].append((ready[k + 1][0] - ready[k][0]) / 1e3)
    total = 0.0
    print("kernel (ready -> next kernel's ready), mean over the layers:")
    for name in LAYER_PATTERN:
        v = per[name]
        if v:
            print(f"  {name:14s} {np.mean(v):7.2f} us   (min {np.min(v):6.2f}, max {np.max(v):6.2f}, n={len(v)})")
            total += float(np.mean(v))
    print(f"  sum per layer  {total:7.2f} us")
    rest = ready[n_layer_kernels:]
    if len(rest) > 1:
        print("after the layers:", ", ".join(f"{n.split('.')[0]} {(rest[k + 1][0] - rest[k][0]) / 1e3:.1f} us"
                                            for k, (_, n) in enumerate(rest[:-1])))
    starts = [k for k, (_, i) in enumerate(ev) if i == 11]
    lo = 2 * args.show_layer
    if lo + 2 < len(starts):
        print(f"marks of layer {args.show_layer} (us from the start of the step):")
        for t, i in ev[starts[lo]:starts[lo + 2]]:
            print(f"  {(t - t0) / 1e3:9.2f}  {NAMES.get(i, str(i))}")


if __name__ == "__main__":
    main()
