"""The CPU configuration: MLP 784 -> 256 -> ReLU -> 10 in bf16 with FlashAdamW (24-bit master
weights, 8-bit states) against fp32 ``torch.optim.AdamW``, 200 steps, then a checkpoint round
trip; alone or as DistributedDataParallel over gloo.

    python benchmarks/mlp_cpu.py
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29641 benchmarks/mlp_cpu.py

Inputs x ~ N(0, 1) of shape [64, 784] (each rank takes its slice under DDP), labels uniform in
[0, 10), seed 0.  Prints one JSON line: first / last loss of both optimizers, the normalised
mean squared error and correlation of the two loss curves, the largest state difference
after a save / load cycle, optimizer-state bytes per parameter, and host milliseconds per step.
The reference cannot run this configuration: its quantised states and master-weight split
need CUDA (``flashoptim/optimizers.py:484-493``).
"""

from __future__ import annotations

import copy
import json
import os
import sys
import time
import warnings

import torch
import torch.distributed as dist
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from flashoptim_b200 import FlashAdamW, cast_model  # noqa: E402
from flashoptim_b200.models import make_mlp  # noqa: E402
from flashoptim_b200.optim.state import MaybeQuantizedTensor  # noqa: E402

STEPS = 200


def main() -> None:
    warnings.simplefilter("ignore")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29641")
        dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 784, generator=g)
    y = torch.randint(0, 10, (64,), generator=g)
    per = 64 // world
    xs, ys = x[rank * per:(rank + 1) * per], y[rank * per:(rank + 1) * per]

    base = make_mlp()
    narrow = copy.deepcopy(base)
    cast_model(narrow, torch.bfloat16)
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP

        base, narrow = DDP(base), DDP(narrow)
    ref_opt = torch.optim.AdamW(base.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01)
    opt = FlashAdamW(narrow.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01, master_weight_bits=24)

    def run(model, optimizer, dtype, steps):
        losses, t0 = [], time.perf_counter()
        for _ in range(steps):
            loss = nn.functional.cross_entropy(model(xs.to(dtype)).float(), ys)
            loss.backward()
            optimizer.step()
            optimizer.zero_grad()
            losses.append(float(loss.detach()))
        return losses, (time.perf_counter() - t0) * 1e3 / steps

    ref_losses, ref_ms = run(base, ref_opt, torch.float32, STEPS)
    losses, ms = run(narrow, opt, torch.bfloat16, STEPS)

    # checkpoint: save, load into a fresh optimizer, compare every state tensor
    sd = copy.deepcopy(opt.state_dict())
    fresh = FlashAdamW(narrow.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01, master_weight_bits=24)
    fresh.load_state_dict(sd)
    worst, state_bytes, n_params = 0.0, 0, 0
    for p in narrow.parameters():
        n_params += p.numel()
        for key, a in opt.state[p].items():
            b = fresh.state[p][key]
            if isinstance(a, MaybeQuantizedTensor):
                state_bytes += sum(t.numel() * t.element_size() for t in (a.quantized, a.scales))
                a, b = a.materialize(), b.materialize()
            elif a.dim() > 0:
                state_bytes += a.numel() * a.element_size()
            worst = max(worst, float((a.float() - b.float()).abs().max()))

    a, b = torch.tensor(ref_losses), torch.tensor(losses)
    out = {
        "bench": "MLP 784-256-10 on CPU, FlashAdamW-24 (bf16) vs torch.optim.AdamW (fp32)",
        "world_size": world, "backend": "gloo" if world > 1 else None, "steps": STEPS,
        "loss_fp32_adamw": [round(ref_losses[0], 4), round(ref_losses[-1], 5)],
        "loss_flash_adamw": [round(losses[0], 4), round(losses[-1], 5)],
        "loss_curve_nmse": float(((a - b) ** 2).mean() / (a ** 2).mean()),
        "loss_curve_correlation": float(torch.corrcoef(torch.stack([a, b]))[0, 1]),
        "state_dict_round_trip_max_abs_diff": worst,
        "optimizer_state_bytes_per_param": round(state_bytes / n_params, 4),
        "ms_per_step": {"fp32_adamw": round(ref_ms, 3), "flash_adamw_cpu_path": round(ms, 3)},
    }
    if world > 1:
        # replicas must agree bit for bit
        flat = torch.cat([p.detach().float().flatten() for p in narrow.parameters()])
        hi, lo = flat.clone(), flat.clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        out["replicas_bit_identical"] = bool(torch.equal(hi, lo))
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
