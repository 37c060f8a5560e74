"""Benchmark driver: random-init Qwen2-7B SmoothQuant int8 W8A8 greedy decode, batch 64, 1024-token
prompts, tensor parallel over N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --sweep [int8,fp8,awq,attn]      # one JSON line per operator shape (1 GPU)

A "step" is one decode step of the whole batch (one new token per sequence).  Prints ONE JSON line
(rank 0).  `value` is generated tokens per second with the token ids resident on the device (the step
is a replayed CUDA graph); `e2e` is the same loop driven through Qwen2Decoder.decode_step_host with
pinned host buffers (ids copied to the device and sampled ids copied back every step).  `roofline`
times the dominant kernel -- the int8 GEMM behind the four linears of every layer -- over all layers'
weights (3.8 GB at one GPU, far larger than L2), in a CUDA graph, with CUDA events.
Both loops are timed as BLOCKS repetitions of exactly K steps (each block restarts at the end of the
prompt, so every block does the same work) and the median block is reported: one block of a short
run is a few tens of milliseconds, too little to trust on its own.

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
BLOCKS = 5                      # timed repetitions of the K-step region; the median is reported


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
    ap.add_argument("--sweep", nargs="?", const="int8,fp8,awq,attn", default=None,
                    help="time every operator shape of the other configurations against its bound instead "
                         "(comma list of int8, fp8, awq, attn, attn_decode, attn_prefill)")
    ap.add_argument("--reps", type=int, default=20, help="graph replays per shape of --sweep")
    ap.add_argument("--no-pipe-peaks", action="store_true",
                    help="--sweep: skip the library GEMMs that measure the tensor-pipe rates (use the recorded bf16 "
                         "rate and twice that for the 8-bit kinds); keeps a profiler run short")
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
                    ops.int8_linear_per_channel(xq, w, getattr(L_, bn) if bn else None, xs, getattr(L_, sn), dt, True)
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
    max_len = args.prompt_len + W + K + 4
    model = Qwen2Decoder(cfg, dev, batch=B, max_seq_len=max_len, tp=world, rank=rank, group=group, seed=0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    prompt = torch.randint(0, cfg.vocab, (B, args.prompt_len), generator=torch.Generator().manual_seed(0)).to(dev)
    first = model.prefill(prompt).clone()

    def timed_blocks(step_fn):
        """BLOCKS x (rewind to the end of the prompt, W warm-up steps, exactly K timed steps); per block the
        device time of the K steps, max over ranks.  Returns the list of block times in seconds."""
        out = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(BLOCKS):
            model.reset_position(args.prompt_len)
            for _ in range(W):
                step_fn()
            barrier()
            e0.record()
            for _ in range(K):
                step_fn()
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out.append(float(t.item()))
        return out

    # ---- device-resident loop -----------------------------------------------------------------
    state = {"tok": first}
    launches0 = _lib.launch_count()
    state["tok"] = model.decode_step(state["tok"])      # captures the graph (one eager warm-up + capture)
    launches_per_step = (_lib.launch_count() - launches0) // 2

    def dev_step():
        state["tok"] = model.decode_step(state["tok"])

    # Untimed ramp: a run of only a few steps would otherwise be measured while the GPU is still leaving
    # its idle clocks (a 2-step run read 3x slower on every kernel).  A fixed number of steps (the same
    # on every rank: the steps contain collectives), about 0.4 s on one GPU.
    for _ in range(16):
        model.reset_position(args.prompt_len)
        for _ in range(8):
            dev_step()
    torch.cuda.synchronize(dev)

    with ClockSampler(local) as clocks:
        block_secs = timed_blocks(dev_step)
    secs = statistics.median(block_secs)

    # ---- host-buffer loop through the public API ----------------------------------------------
    host = {"in": first.cpu().pin_memory()}
    host["out"] = torch.empty_like(host["in"]).pin_memory()

    def host_step():
        model.decode_step_host(host["in"], host["out"])
        host["in"], host["out"] = host["out"], host["in"]

    block_secs_e2e = timed_blocks(host_step)
    secs_e2e = statistics.median(block_secs_e2e)

    # ---- the run is only valid if no bounded wait ran out and all ranks decoded the same tokens ----
    problems = []
    if _lib.kernel_status(dev) != 0:
        problems.append("a kernel reported a bounded-wait time-out")
    if model.comm is not None:
        try:
            model.comm.check()
        except RuntimeError as e:
            problems.append(str(e))
    last_ids = host["in"].to(dev)                       # ids sampled by the last step, as this rank saw them
    if world > 1:
        ids = [torch.empty_like(last_ids) for _ in range(world)]
        dist.all_gather(ids, last_ids)
        if any(not torch.equal(ids[0], t) for t in ids[1:]):
            problems.append("the ranks sampled different token ids")
        bad = torch.tensor([1 if problems else 0], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()) and not problems:
            problems.append("another rank reported a failure")
    if problems:
        print(f"rank {rank}: INVALID RUN: " + "; ".join(problems), file=sys.stderr, flush=True)
        sys.stdout.flush()
        os._exit(3)

    # ---- dominant kernel --------------------------------------------------------------------------
    bytes_per_launch, secs_per_launch, gemm_shapes = gemm_roofline_pass(model, B, torch)
    attn_bytes, attn_secs = attn_roofline_pass(model, B, args.prompt_len + W + K // 2, torch)
    peak, peak_kind = measured_peak_hbm()
    achieved = bytes_per_launch / secs_per_launch / 1e9
    if _lib.kernel_status(dev) != 0:
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
                         "traffic": 60.0e6 if (world == 1 and B == 64 and args.layers == 28) else None,
                         "traffic_source": ("recorded constant, not measured by this run: dram__bytes_read.sum + "
                                            "dram__bytes_write.sum per launch from one ncu capture of this kernel at this "
                                            "configuration (1 GPU, batch 64), averaged over the four linears of a layer"
                                            if (world == 1 and B == 64 and args.layers == 28) else None),
                         "bytes_per_launch": bytes_per_launch, "us_per_launch": secs_per_launch * 1e6},
            "extras": {"launches_per_step": launches_per_step, "int8_gemm_by_shape": gemm_shapes,
                       "timing": f"median of {BLOCKS} blocks of {K} steps, each block rewound to the end of the prompt",
                       "block_ms_per_step": [t / K * 1e3 for t in block_secs],
                       "block_ms_per_step_e2e": [t / K * 1e3 for t in block_secs_e2e],
                       "checked": "no bounded-wait time-out; peer all-reduce status clean; identical ids on all ranks",
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


# ----------------------------------------------------------------------------------------------
# --sweep: every operator shape of the micro-benchmark configurations against its bound
# ----------------------------------------------------------------------------------------------
L2_BYTES = 126 << 20


def _time_graph(torch, body, reps):
    """Seconds per replay of `body` captured in a CUDA graph (CUDA events around `reps` replays)."""
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


def _copies(nbytes):
    """Distinct buffers to rotate over so that the working set exceeds L2 (at least 2, at most 64)."""
    import math
    return max(2, min(64, math.ceil(1.5 * L2_BYTES / max(nbytes, 1))))


def measure_pipe_peaks(torch):
    """Dense tensor-pipe rates of this GPU measured the way MEASURED_PEAKS.json measures bf16: the
    library GEMM at 8192^3, best of 10.  Used only as roofline denominators of the sweep."""
    dev = torch.device("cuda")
    n = 8192
    out = {}

    def best(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / 1e3)
        return 2 * n ** 3 / min(ts)

    a16 = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
    b16 = torch.randn(n, n, device=dev, dtype=torch.bfloat16)
    out["bf16"] = best(lambda: torch.matmul(a16, b16.t()))
    try:
        a8, b8 = a16.to(torch.float8_e4m3fn), b16.to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        out["fp8"] = best(lambda: torch._scaled_mm(a8, b8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
    except Exception:
        out["fp8"] = None
    try:
        ai = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        bi = torch.randint(-127, 128, (n, n), device=dev, dtype=torch.int8)
        out["int8"] = best(lambda: torch._int_mm(ai, bi.t()))
    except Exception:
        out["int8"] = None
    return out


def run_sweep(args):
    """One JSON line per operator shape: time, algorithmic GB/s and TOP/s, bound = max(bytes / HBM,
    flops / pipe), frac = bound / time.  Every shape is replayed from a CUDA graph that rotates over
    enough distinct weight (or KV) buffers to exceed L2."""
    import torch
    from llmqrt_b200 import _lib, ops
    from llmqrt_b200.attention import attn_decode, flash_attn_func
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --sweep needs a CUDA device")
    dev = torch.device("cuda")
    hbm_gbs, peak_kind = measured_peak_hbm()
    hbm = hbm_gbs * 1e9
    pipes = measure_pipe_peaks(torch) if not args.no_pipe_peaks else {"bf16": None, "fp8": None, "int8": None}
    if pipes["bf16"] is None:                           # not measured here: the pool's recorded cuBLAS bf16 rate
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                pipes["bf16"] = float(json.load(f)["bf16_tflops"]) * 1e12
        except Exception:
            pipes["bf16"] = 1590e12
    pipe16 = pipes["bf16"]
    pipe_f8 = pipes["fp8"] or 2 * pipe16
    pipe_i8 = pipes["int8"] or 2 * pipe16
    print(json.dumps({"sweep": "peaks", "hbm_gbs": hbm_gbs, "hbm_source": peak_kind,
                      "pipe_tflops_measured_here": {k: (v / 1e12 if v else None) for k, v in pipes.items()},
                      "note": "pipes = library GEMM at 8192^3, best of 10; a kind the library refuses falls back "
                              "to twice the bf16 figure"}), flush=True)
    reps = args.reps

    def report(tag, M, N, K, secs, nbytes, flops, pipe, **extra):
        bound = max(nbytes / hbm, flops / pipe)
        print(json.dumps({"sweep": tag, "M": M, "N": N, "K": K, "us": secs * 1e6, "gbs": nbytes / secs / 1e9,
                          "tops": flops / secs / 1e12, "bound_us": bound * 1e6,
                          "bound": "hbm" if nbytes / hbm >= flops / pipe else "pipe", "frac": bound / secs, **extra}),
              flush=True)

    what = args.sweep.split(",")
    if "int8" in what:
        g = torch.Generator(device=dev).manual_seed(0)
        shapes = [("sq qwen2-0.5b gate", 16, 4864, 896)]
        for M in (64, 4096):
            shapes += [("sq 7b qkv", M, 4608, 3584), ("sq 7b o", M, 3584, 3584), ("sq 7b gate_up", M, 37888, 3584),
                       ("sq 7b down", M, 3584, 18944)]
        for tag, M, N, K in shapes:
            n = _copies(N * K)
            ws = [torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8) for _ in range(n)]
            a = torch.randint(-127, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
            sa = torch.rand(M, generator=g, device=dev) * 1e-2
            sw = torch.rand(N, generator=g, device=dev) * 1e-2
            secs = _time_graph(torch, lambda: [ops.int8_linear_per_channel(a, w, None, sa, sw, torch.bfloat16, True)
                                               for w in ws], reps) / n
            report(tag, M, N, K, secs, gemm_bytes(M, N, K, False), 2 * M * N * K, pipe_i8)
            if M == 16:                                  # the allocation-free entry point on the same shape
                out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

                def noalloc():
                    for w in ws:
                        _lib.call("llmqrt_w8a8_int8_linear_per_channel_noalloc", _lib.ptr(a), a.stride(0), _lib.ptr(w),
                                  w.stride(0), None, _lib.F16, _lib.ptr(sa), _lib.ptr(sw), _lib.ptr(out), _lib.BF16, N,
                                  M, N, K, _lib.stream(dev))
                noalloc()                                # resolves the scratch address before any capture
                secs = _time_graph(torch, noalloc, reps) / n
                report(tag + " (no-alloc entry)", M, N, K, secs, gemm_bytes(M, N, K, False), 2 * M * N * K, pipe_i8)
            del ws
    if "fp8" in what:
        g = torch.Generator(device=dev).manual_seed(1)
        for tag, N, K in (("fp8 q/o", 896, 896), ("fp8 k/v", 128, 896), ("fp8 gate/up", 4864, 896), ("fp8 down", 896, 4864)):
            for M in (1, 16, 64, 1024, 4096):
                n = _copies(N * K)
                ws = [(torch.randn(N, K, generator=g, device=dev) * 0.5).to(torch.float8_e4m3fn) for _ in range(n)]
                a = torch.randn(M, K, generator=g, device=dev).to(torch.float8_e4m3fn)
                sa = torch.rand(M, 1, generator=g, device=dev) * 1e-2
                sw = torch.rand(1, N, generator=g, device=dev) * 1e-2
                secs = _time_graph(torch, lambda: [ops.fp8_linear_rowwise(a, w, None, sa, sw, True) for w in ws], reps) / n
                report(tag, M, N, K, secs, gemm_bytes(M, N, K, False), 2 * M * N * K, pipe_f8)
    if "awq" in what:
        g = torch.Generator(device=dev).manual_seed(2)
        G = 128
        for tag, N, K in (("awq qkv", 2048, 1536), ("awq o", 1536, 1536), ("awq gate", 8960, 1536),
                          ("awq gate_up", 17920, 1536), ("awq down", 1536, 8960)):
            for M in (1, 16, 256, 2048):
                wbytes = K * N // 2 + (K // G) * N * 2 + (K // G) * N // 2
                n = _copies(wbytes)
                layers = []
                for _ in range(n):                       # nibbles uniform, scales ~ U(0.001, 0.02)
                    qweight = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), generator=g, device=dev, dtype=torch.int32)
                    qzeros = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // G, N // 8), generator=g, device=dev, dtype=torch.int32)
                    scales = (torch.rand(K // G, N, generator=g, device=dev) * 0.019 + 0.001).half()
                    layers.append(ops.AwqPacked(qweight, scales, qzeros))
                x = torch.randn(M, K, generator=g, device=dev).half()
                secs = _time_graph(torch, lambda: [ops.awq_gemm(x, p) for p in layers], reps) / n
                report(tag, M, N, K, secs, 2 * M * K + wbytes + 2 * M * N, 2 * M * N * K, pipe16)
    Hq, Hkv, d = 28, 4, 128
    if "attn" in what or "attn_decode" in what:
        g = torch.Generator(device=dev).manual_seed(3)
        B, Smax = 32, 8192
        lens = torch.randint(512, 8193, (B,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
        kc = torch.randn(B, Smax, Hkv, d, generator=g, device=dev, dtype=torch.float16)     # 268 MB each: beyond L2
        vc = torch.randn(B, Smax, Hkv, d, generator=g, device=dev, dtype=torch.float16)
        q = torch.randn(B, Hq, d, generator=g, device=dev, dtype=torch.float16)
        ld = lens.to(dev)
        secs = _time_graph(torch, lambda: attn_decode(q, kc, vc, ld, Smax), reps)
        ctx = int(lens.sum())
        report("attn decode b32 ctx U[512,8192]", B, ctx // B, d, secs, ctx * Hkv * d * 2 * 2 + 2 * B * Hq * d * 2,
               4 * ctx * Hq * d, pipe16)
        del kc, vc
    if "attn" in what or "attn_prefill" in what:
        g = torch.Generator(device=dev).manual_seed(4)
        Bp, S = 4, 2048
        qs = [torch.randn(Bp, S, Hq, d, generator=g, device=dev, dtype=torch.float16) for _ in range(2)]
        ks = [torch.randn(Bp, S, Hkv, d, generator=g, device=dev, dtype=torch.float16) for _ in range(2)]
        vs = [torch.randn(Bp, S, Hkv, d, generator=g, device=dev, dtype=torch.float16) for _ in range(2)]
        secs = _time_graph(torch, lambda: [flash_attn_func(a, b, c, causal=True) for a, b, c in zip(qs, ks, vs)], reps) / 2
        report("attn prefill 4x2048 causal", Bp * S, S, d, secs, Bp * S * (2 * Hq + 2 * Hkv) * d * 2,
               4 * Bp * Hq * S * S * d // 2, pipe16)
    if _lib.kernel_status(dev) != 0:
        raise SystemExit("a kernel reported a bounded-wait time-out; the sweep is invalid")


if __name__ == "__main__":
    a = parse_args()
    if a.sweep is not None:
        run_sweep(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
