"""GPT-2-medium under DistributedDataParallel: tokens/s and peak memory.

    python benchmarks/gpt2_ddp.py --gpus 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29521 benchmarks/gpt2_ddp.py --gpus 8 --mode fused

24 layers, d=1024, 16 heads, MLP 4096, vocab 50257, learned positions, sequence
1024, micro-batch 8 per GPU, bf16 parameters (``cast_model``), FlashAdamW with
24-bit master weights, synthetic uniform token ids, random init N(0, 0.02).

Modes: ``fused`` (this library: per-bucket all-reduce fused with the update over
NVLink peer memory), ``plain`` (this library's optimizer after stock NCCL DDP),
``reference`` (the reference optimizer from ``baseline/_ref`` after stock NCCL DDP).
Device-timed with CUDA events, barrier + synchronize on both sides, max over ranks.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import warnings

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--mode", default="fused", choices=["fused", "plain", "reference"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--comm-ctas", type=int, default=0, help="fused: grid cap of the all-reduce + update kernel")
    ap.add_argument("--multicast", action="store_true", help="fused: NVSwitch multimem.ld_reduce")
    ap.add_argument("--two-shot", default="auto", choices=["auto", "on", "off"],
                    help="fused: reduce + broadcast then local step for large buckets (auto: more than 2 GPUs)")
    args = ap.parse_args()
    if args.mode == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

    import torch
    import torch.distributed as dist
    from torch.nn.parallel import DistributedDataParallel as DDP

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, "launch with torch.distributed.run for --gpus > 1"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    spec = importlib.util.spec_from_file_location("_bench_gpt2", os.path.join(ROOT, "flashoptim_b200", "models", "gpt2.py"))
    gpt2 = importlib.util.module_from_spec(spec)
    sys.modules["_bench_gpt2"] = gpt2
    spec.loader.exec_module(gpt2)
    if args.mode == "reference":
        import flashoptim as lib
    else:
        import flashoptim_b200 as lib

    cfg = gpt2.GPT2Config.medium(n_layer=args.layers, max_seq_len=args.seq_len)
    with torch.device(dev):
        model = gpt2.GPT2(cfg)
    model.init_weights(0.02, seed=0)
    lib.cast_model(model, dtype=torch.bfloat16)
    n_params = sum(p.numel() for p in model.parameters())
    ddp = DDP(model, device_ids=[local_rank], gradient_as_bucket_view=True)
    warnings.simplefilter("ignore")
    opt = lib.FlashAdamW(ddp.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01, master_weight_bits=24)
    state = None
    if args.mode == "fused":
        from flashoptim_b200.parallel import fuse_ddp_allreduce

        state = fuse_ddp_allreduce(ddp, opt, use_multicast=args.multicast, max_ctas=args.comm_ctas,
                                   two_shot={"auto": None, "on": True, "off": False}[args.two_shot])

    b, s = args.micro_batch, args.seq_len
    g = torch.Generator().manual_seed(99 + rank)
    toks = torch.randint(0, cfg.vocab_size, (args.warmup + args.steps, b, s + 1), generator=g).to(dev)

    def step(i):
        loss = ddp(toks[i, :, :-1], toks[i, :, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if state is not None:
        state.check()
    torch.cuda.reset_peak_memory_stats()
    # read-only NVML sampler, loaded by file path so the reference mode imports nothing of this package
    tspec = importlib.util.spec_from_file_location(
        "_bench_timing", os.path.join(ROOT, "flashoptim_b200", "utils", "timing.py"))
    timing = importlib.util.module_from_spec(tspec)
    sys.modules["_bench_timing"] = timing
    tspec.loader.exec_module(timing)
    sampler = timing.ClockSampler(local_rank)
    dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(args.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps, torch.cuda.max_memory_allocated() / 2**30], device=dev,
                     dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, gib = t.tolist()
    if state is not None:
        state.check()
    if rank == 0:
        print(json.dumps({
            "bench": "gpt2-medium ddp", "mode": args.mode, "n_gpus": world, "n_params": n_params,
            "micro_batch": b, "seq_len": s, "ms_per_step": round(ms, 3),
            "tokens_per_s": round(world * b * s / (ms * 1e-3), 1), "peak_gib_per_gpu": round(gib, 2),
            "loss": float(loss), "steps": args.steps, "warmup": args.warmup,
            "buckets_fused_per_step": (state.buckets_fused // (args.steps + args.warmup)) if state else 0,
            "buckets_two_shot_per_step": (state.buckets_two_shot // (args.steps + args.warmup)) if state else 0,
            "clocks": sampler.summary(),
        }), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
