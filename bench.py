"""Benchmark driver: random-init Qwen2-7B SmoothQuant int8 W8A8 greedy decode, batch 64, 1024-token
prompts, tensor parallel over N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

A "step" is one decode step of the whole batch (one new token per sequence).  Prints ONE JSON line
(rank 0).  `value` is generated tokens per second with the token ids resident on the device (the step
is a replayed CUDA graph); `e2e` is the same loop driven through Qwen2Decoder.decode_step_host with
pinned host buffers (ids copied to the device and sampled ids copied back every step).  `roofline`
times the dominant kernel -- the int8 GEMM behind the four linears of every layer -- over all layers'
weights (3.8 GB at one GPU, far larger than L2), in a CUDA graph, with CUDA events.

--impl reference times the reference's own CPU path for this workload (torch dequantize-then-matmul for
the seven linears of a decoder layer plus a torch decode attention) on the host cores; each step is one
layer sample and the reported step time is layers x mean + lm_head.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "qwen2_7b_w8a8_decode_tokens_per_s"
UNIT = "tokens/s"
BATCH, PROMPT, GEN = 64, 1024, 256


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=GEN)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--prompt-len", type=int, default=PROMPT)
    ap.add_argument("--layers", type=int, default=28, help="decoder layers (28 = Qwen2-7B; fewer is NOT the benchmark)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def workload_config(args, n):
    return {"workload": "Qwen2-7B int8 W8A8 (per-token x per-channel) greedy decode, random-init weights, "
                        f"batch {args.batch}, prompt {args.prompt_len}, one token per sequence per step",
            "layers": args.layers, "hidden": 3584, "intermediate": 18944, "heads": "28/4", "vocab": 152064,
            "batch": args.batch, "prompt_len": args.prompt_len, "parallelism": f"tp{n}",
            "l2": "every step streams all weights (7.6 GB / tp) and the KV cache: inputs far larger than L2"}


# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML every 20 ms while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz, self._stop, self._t = [], set(), None, threading.Event(), None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = torch.cuda.get_device_properties(device_index).uuid
                self.h = pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{uuid}".encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._t is not None:
            self._t.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def measured_peak_hbm():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ----------------------------------------------------------------------------------------------
def gemm_bytes(M, N, K, bias):
    return M * K + N * K + 2 * M * N + 4 * (M + N) + (2 * N if bias else 0)


def gemm_roofline_pass(model, batch, torch):
    """Average duration of the int8 GEMM kernel over the four linears of all layers (distinct weights)."""
    from llmqrt_b200 import ops
    dev, dt = model.device, model.cfg.dtype
    d = model.cfg.head_dim
    g = torch.Generator(device=dev).manual_seed(1)
    acts = {}
    for K in (model.cfg.hidden, model.hq * d, model.inter_local):
        acts[K] = (torch.randint(-127, 128, (batch, K), generator=g, device=dev, dtype=torch.int8),
                   torch.rand(batch, generator=g, device=dev) * 1e-2)

    names = {"qkv": ("wqkv", "sqkv", "bqkv"), "o": ("wo", "so", None), "gate_up": ("wgu", "sgu", None),
             "down": ("wd", "sd", None)}

    def timed(which):
        def body():
            for L_ in model.layers:
                for nm in which:
                    wn, sn, bn = names[nm]
                    w = getattr(L_, wn)
                    xq, xs = acts[w.shape[1]]
                    ops.int8_linear_per_channel(xq, w, getattr(L_, bn) if bn else None, xs, getattr(L_, sn), dt)
        body()
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            body()
        graph.replay()
        torch.cuda.synchronize(dev)
        reps = 5
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / 1e3 / reps

    L0 = model.layers[0]
    nlay = len(model.layers)
    per_shape = {}
    for nm, (wn, _, bn) in names.items():
        N, K = getattr(L0, wn).shape
        secs = timed([nm]) / nlay
        b = gemm_bytes(batch, N, K, bn is not None)
        per_shape[nm] = {"N": N, "K": K, "us": secs * 1e6, "gbs": b / secs / 1e9}
    secs_all = timed(list(names))                       # the four GEMMs of every layer, in model order
    nbytes = sum(gemm_bytes(batch, *getattr(L0, wn).shape, bn is not None) for wn, _, bn in names.values()) * nlay
    launches = 4 * nlay
    return nbytes / launches, secs_all / launches, per_shape


def attn_roofline_pass(model, batch, ctx, torch):
    """Average duration of decode attention over all layers' caches at context `ctx`."""
    from llmqrt_b200 import attention
    dev, dt, d = model.device, model.cfg.dtype, model.cfg.head_dim
    q = torch.randn(batch, model.hq, d, device=dev, dtype=dt)
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)

    def body():
        for L_ in model.layers:
            attention.attn_decode(q, L_.k_cache, L_.v_cache, lens, ctx)

    body()
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    graph.replay()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(dev)
    secs = e0.elapsed_time(e1) / 1e3 / 5 / len(model.layers)
    nbytes = batch * ctx * model.hkv * d * 2 * 2 + 2 * batch * model.hq * d * 2
    return nbytes, secs


def cpu_baseline_sample(args, budget_s=12.0):
    import torch
    from oracle import reference_cpu as rc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    layer = rc.Qwen2LayerSample(3584, 18944, 28, 4, 128, args.batch, args.prompt_len)
    layer.step()
    times = []
    t0 = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t0 < budget_s and len(times) < 64):
        times.append(layer.step())
    t_head = rc.time_lm_head(3584, 152064, args.batch)
    step_s = args.layers * statistics.mean(times) + t_head
    return {"value": args.batch / step_s, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{len(times)} runs of one decoder layer (7 int8 linears as torch dequantize-then-matmul in "
                      f"bf16 + torch decode attention at context {args.prompt_len}), step = {args.layers} x mean + "
                      "one lm_head matmul; the reference ships no CPU attention"}, step_s


# ----------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import reference_cpu as rc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    layer = rc.Qwen2LayerSample(3584, 18944, 28, 4, 128, args.batch, args.prompt_len)
    for _ in range(max(1, min(args.warmup, 3))):
        layer.step()
    times = [layer.step() for _ in range(args.steps)]
    t_head = rc.time_lm_head(3584, 152064, args.batch)
    step_s = args.layers * statistics.mean(times) + t_head
    value = args.batch / step_s
    sample = (f"each of the {args.steps} steps = one decoder layer on the CPU (7 int8 linears as torch "
              f"dequantize-then-matmul in bf16 + torch decode attention at context {args.prompt_len}); reported step "
              f"= {args.layers} x mean layer time + one lm_head matmul")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD

    from llmqrt_b200 import _lib
    from llmqrt_b200.qwen2 import Qwen2Config, Qwen2Decoder
    cfg = Qwen2Config.qwen2_7b()
    cfg.num_layers = args.layers
    K, W, B = args.steps, max(args.warmup, 3), args.batch
    max_len = args.prompt_len + W + K + 2
    model = Qwen2Decoder(cfg, dev, batch=B, max_seq_len=max_len, tp=world, rank=rank, group=group, seed=0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    prompt = torch.randint(0, cfg.vocab, (B, args.prompt_len), generator=torch.Generator().manual_seed(0)).to(dev)
    first = model.prefill(prompt).clone()

    # ---- device-resident loop -----------------------------------------------------------------
    tok = first
    launches0 = _lib.launch_count()
    tok = model.decode_step(tok)                      # captures the graph (one eager warm-up + capture)
    launches_per_step = (_lib.launch_count() - launches0) // 2
    for _ in range(W - 1):
        tok = model.decode_step(tok)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record()
        for _ in range(K):
            tok = model.decode_step(tok)
        e1.record()
        barrier()
    elapsed = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    secs = float(elapsed.item())

    # ---- host-buffer loop through the public API ----------------------------------------------
    model.reset_position(args.prompt_len)
    h_in = first.cpu().pin_memory()
    h_out = torch.empty_like(h_in).pin_memory()
    for _ in range(W):
        model.decode_step_host(h_in, h_out)
        h_in, h_out = h_out, h_in
    barrier()
    e0.record()
    for _ in range(K):
        model.decode_step_host(h_in, h_out)
        h_in, h_out = h_out, h_in
    e1.record()
    barrier()
    elapsed = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    secs_e2e = float(elapsed.item())

    # ---- dominant kernel --------------------------------------------------------------------------
    bytes_per_launch, secs_per_launch, gemm_shapes = gemm_roofline_pass(model, B, torch)
    attn_bytes, attn_secs = attn_roofline_pass(model, B, args.prompt_len + W + K // 2, torch)
    peak, peak_kind = measured_peak_hbm()
    achieved = bytes_per_launch / secs_per_launch / 1e9
    status = _lib.kernel_status(dev)
    if status != 0:
        raise SystemExit("a kernel reported a bounded-wait time-out; the numbers are invalid")

    if rank == 0:
        ctx_mid = args.prompt_len + W + K // 2
        kv_bytes = B * ctx_mid * model.hkv * cfg.head_dim * 2 * 2 * cfg.num_layers
        step_bytes = model.weight_bytes() + kv_bytes
        line = {
            "metric": METRIC, "value": B * K / secs, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic", "config": workload_config(args, world),
            "clocks": clocks.summary(),
            "e2e": {"value": B * K / secs_e2e, "unit": UNIT, "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
            "gpu_launches": launches_per_step * K,
            "roofline": {"bound": "hbm", "kernel": "gemm_tc_kernel<int8> (TMA + tcgen05, weights as the M operand)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})",
                         # dram read + write per launch, averaged over the four linears of a layer, from the ncu
                         # capture summarised in profiles/gemm_tc_int8_decode_ncu_full.md (1 GPU, batch 64)
                         "traffic": 60.0e6 if (world == 1 and B == 64) else None,
                         "bytes_per_launch": bytes_per_launch, "us_per_launch": secs_per_launch * 1e6},
            "extras": {"launches_per_step": launches_per_step, "int8_gemm_by_shape": gemm_shapes,
                       "step_hbm_gbs": step_bytes / (secs / K) / 1e9, "step_hbm_frac": step_bytes / (secs / K) / 1e9 / peak,
                       "attn_decode_gbs": attn_bytes / attn_secs / 1e9, "attn_decode_frac": attn_bytes / attn_secs / 1e9 / peak,
                       "attn_decode_us": attn_secs * 1e6},
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline_sample(args)
        print(json.dumps(line))
    if world > 1:
        # Tearing the NCCL communicator down while CUDA graphs that captured its collectives are alive
        # blocks for ever; everything is measured and printed, so leave without the orderly shutdown.
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
