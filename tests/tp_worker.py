"""Worker of the tensor-parallel GPU test: one process per GPU, launched by torch.distributed.run.

Builds the tiny decoder with tp = world size, runs prefill and a few CUDA-graph decode steps, gathers
every rank's weight shard on rank 0 and compares the logits with the CPU oracle's emulation of the
same sharding (per-rank activation scales, 16-bit partial sums added in rank order).
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    # ---- the peer-buffer all-reduce alone: exact fp32 rank-order sums, back-to-back calls ----
    from llmqrt_b200.tp import PeerAllreduce
    comm = PeerAllreduce(dev, rank, world, 1 << 20, dist.group.WORLD)
    for dtype in (torch.float16, torch.bfloat16):
        for n in (8, 4096, 229376, 524288):
            xs = []
            for rep in range(3):                                     # three calls in flight: both parities reused
                g = torch.Generator().manual_seed(1000 * rank + n + rep)
                xs.append(torch.randn(n, generator=g).to(dtype).to(dev))
            wants = []
            for x in xs:
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                acc = torch.zeros(n, dtype=torch.float32, device=dev)
                for p in parts:
                    acc += p.float()
                wants.append(acc.to(dtype))
            gots = [comm.allreduce(x.clone()) for x in xs]
            ok &= all(torch.equal(gv, w) for gv, w in zip(gots, wants))
    # ---- all-reduce fused into the RMSNorm that consumes it == all-reduce, then RMSNorm ----
    from llmqrt_b200 import glue
    for dtype in (torch.float16, torch.bfloat16):
        for M, H in ((5, 3584), (64, 3584), (3, 256)):
            g = torch.Generator().manual_seed(77 + M)
            x = torch.randn(M, H, generator=g).to(dtype).to(dev)                       # same on every rank
            w = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype).to(dev)
            part = torch.randn(M, H, generator=torch.Generator().manual_seed(500 + rank)).to(dtype).to(dev)
            want = glue.rmsnorm(x, w, 1e-6, residual=comm.allreduce(part.clone()), quantize=True)
            got = glue.rmsnorm(x, w, 1e-6, residual=part.clone(), quantize=True, comm=comm)
            ok &= all(torch.equal(a, b) for a, b in zip(got, want))
    # ---- row-parallel int8 linear that sends its partial sums from the GEMM's epilogue == the same linear
    #      writing a tensor that the fused kernel then pushes (identical bits), three calls back to back ----
    from llmqrt_b200 import ops
    for dtype in (torch.float16, torch.bfloat16):
        for M, N, K in ((64, 3584, 4736), (64, 3584, 256), (17, 1000, 512), (128, 256, 2048)):
            g = torch.Generator().manual_seed(31 * M + N + K)
            x = torch.randn(M, N, generator=g).to(dtype).to(dev)                       # same on every rank
            wn = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype).to(dev)
            gr = torch.Generator().manual_seed(9000 + rank)                            # this rank's shard
            a = torch.randint(-128, 128, (M, K), generator=gr, dtype=torch.int8).to(dev)
            w = torch.randint(-128, 128, (N, K), generator=gr, dtype=torch.int8).to(dev)
            a_s = (torch.rand(M, generator=gr) * 1e-2 + 1e-3).to(dev)
            w_s = (torch.rand(N, generator=gr) * 1e-2 + 1e-3).to(dev)
            assert comm.push_ok(M, N)
            for rep in range(3):
                part = ops.int8_linear_per_channel(a, w, None, a_s, w_s, dtype)
                want = glue.rmsnorm(x, wn, 1e-6, residual=part, quantize=True, comm=comm)
                token = comm.linear_push(a, w, None, a_s, w_s, dtype)
                got = glue.rmsnorm(x, wn, 1e-6, residual=token, quantize=True, comm=comm)
                ok &= all(torch.equal(p, q) for p, q in zip(got, want))
    comm.check()
    if not ok:
        print(f"rank {rank}: peer all-reduce mismatch")

    # ---- a peer that does not deliver: the bounded wait runs out, the kernel returns, the status is raised ----
    # The failure is made on the host (the last rank skips the call); nothing waits on that rank's GPU.
    lame = PeerAllreduce(dev, rank, world, 4096, dist.group.WORLD)
    lame.set_poll_limit_ms(200)
    t = torch.ones(1024, dtype=torch.float16, device=dev)
    if rank != world - 1:
        lame.allreduce(t)
        torch.cuda.synchronize(dev)                              # returns after ~0.2 s, context intact
        try:
            lame.check()
            ok = False
            print(f"rank {rank}: the missing peer went unnoticed")
        except RuntimeError:
            pass
        lame.allreduce(t)                                        # sticky status: returns without waiting
        torch.cuda.synchronize(dev)
    else:
        lame.check()                                             # the rank that skipped has seen no time-out
    dist.barrier()

    from llmqrt_b200.qwen2 import Qwen2Config, Qwen2Decoder
    # 4 query / 2 KV heads divide among up to 4 ranks; 8 ranks get 12 query / 4 KV heads: every KV head on
    # two ranks, its three query heads split 2 + 1 (the uneven case of Qwen2-7B's 28 / 4 heads on 8 ranks)
    cfg = Qwen2Config.tiny() if world <= 4 else Qwen2Config(num_layers=2, hidden=256, intermediate=512, num_heads=12,
                                                            num_kv_heads=4, head_dim=64, vocab=1024)
    B, S, steps, max_len = 3, 21, 3, 48
    model = Qwen2Decoder(cfg, dev, batch=B, max_seq_len=max_len, tp=world, rank=rank, group=dist.group.WORLD, seed=5)
    prompt = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(0))
    nxt = model.prefill(prompt.to(dev))
    logits, fed = [model.last_logits.clone()], []
    for _ in range(steps):
        fed.append(nxt.clone().cpu())
        nxt = model.decode_step(nxt).clone()
        logits.append(model.last_logits.clone())
    # full-vocabulary logits: concatenate the vocabulary shards of all ranks
    full = []
    for lg in logits:
        parts = [torch.empty_like(lg) for _ in range(world)]
        dist.all_gather(parts, lg.contiguous())
        full.append(torch.cat(parts, dim=1).cpu())
    shards = [None] * world
    dist.gather_object(model.export_shard(), shards if rank == 0 else None, dst=0)
    if model.comm is not None:
        model.comm.check()
    if rank == 0:
        from oracle.qwen2 import Qwen2Oracle
        orc = Qwen2Oracle(cfg, shards, B, max_len)
        want = [orc.forward(prompt)] + [orc.forward(t.reshape(-1, 1)) for t in fed]
        for got, w in zip(full, want):
            err = float((got.double() - w.double()).norm() / w.double().norm())
            print("rel_fro", err)
            ok &= err < 2e-2
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)             # every rank's own checks count
    dist.barrier()
    torch.cuda.synchronize(dev)
    code = 0 if int(flag.item()) == 1 else 1
    # destroy_process_group() blocks while CUDA graphs holding captured NCCL collectives are alive
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


if __name__ == "__main__":
    main()
