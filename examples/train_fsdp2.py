"""FSDP2 training of a small Llama-style decoder with ``FlashAdamW``.

    # CPU, two gloo ranks (plain path: FSDP2's collectives + optimizer.step())
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29611 examples/train_fsdp2.py --device cpu
    # GPUs of one NVLink node: reduce-scatter fused with the sharded update, and the updated
    # parameters pushed into every rank's all-gather buffer by the same kernel
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29611 examples/train_fsdp2.py --fused --push-params

Each rank trains on its own slice of a synthetic next-token task (a fixed random bigram
table, so the loss has somewhere to go), prints the loss, then saves and reloads a sharded
optimizer checkpoint through ``torch.distributed.checkpoint`` and checks that training
continues from the same state.  The reference documents the same FSDP2 and DCP usage
(``README.md:212-288`` there) without an example script.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict, set_optimizer_state_dict
from torch.distributed.fsdp import fully_shard

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from flashoptim_b200 import FlashAdamW, cast_model, enable_gradient_release  # noqa: E402
from flashoptim_b200.models.llama import Llama, LlamaConfig  # noqa: E402


def batches(rank: int, steps: int, batch: int, seq: int, vocab: int, device):
    table = torch.randint(0, vocab, (vocab,), generator=torch.Generator().manual_seed(0))
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(steps):
        first = torch.randint(0, vocab, (batch, 1), generator=g)
        toks = [first]
        for _ in range(seq):
            toks.append(table[toks[-1]])
        t = torch.cat(toks, dim=1).to(device)
        yield t[:, :-1], t[:, 1:]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu", choices=["cuda", "cpu"])
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--lr", type=float, default=3e-3)
    ap.add_argument("--master-weight-bits", type=int, default=24, choices=[24, 32])
    ap.add_argument("--compress-state-dict", action="store_true")
    ap.add_argument("--gradient-release", action="store_true")
    ap.add_argument("--fused", action="store_true", help="CUDA: fuse the reduce-scatter with the update")
    ap.add_argument("--push-params", action="store_true", help="with --fused: all-gather on write")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29611")
    if args.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        device = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo", rank=rank, world_size=world)

    cfg = LlamaConfig.tiny()
    model = Llama(cfg).to(device)
    model.init_weights()
    cast_model(model, torch.bfloat16)
    for layer in model.layers:
        fully_shard(layer)
    fully_shard(model)
    opt = FlashAdamW(model.parameters(), lr=args.lr, weight_decay=0.01, master_weight_bits=args.master_weight_bits,
                     compress_state_dict=args.compress_state_dict)
    fused = None
    if args.fused and args.device == "cuda":
        from flashoptim_b200.parallel import enable_fused_fsdp, tuned_options

        # kernel, grid cap and load path that measured best for this number of GPUs; the
        # all-gather on write costs an unsharded copy of the parameters and is opt-in here
        opts = tuned_options(world)
        opts.pop("own_all_gather", None), opts.pop("all_gather_copy_engine", None)
        fused = enable_fused_fsdp(model, opt, push_params=args.push_params, **opts)
    if args.gradient_release:
        enable_gradient_release(model, opt)

    def step(x, y) -> float:
        loss = model(x, y)
        loss.backward()
        opt.step()       # no-ops under gradient release; skips what the fused kernel updated
        opt.zero_grad()
        return float(loss.detach())

    losses = [step(x, y) for x, y in batches(rank, args.steps, 8, 64, cfg.vocab_size, device)]
    if fused is not None:
        fused.check()
    if rank == 0:
        print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f} over {args.steps} steps on {world} rank(s)"
              + (f"; fused reduce-scatters {fused.fused_calls}, all-gathers without data movement "
                 f"{fused.ag_eliminated}" if fused is not None else ""))

    # sharded optimizer checkpoint: save, scramble, load, compare
    folder = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(folder, src=0)
    osd = get_optimizer_state_dict(model, opt)
    dcp.save({"optimizer": osd}, checkpoint_id=folder[0])
    before = {k: {kk: (vv.to_local().clone() if hasattr(vv, "to_local") else vv.clone()) for kk, vv in v.items()}
              for k, v in osd["state"].items()}
    for x, y in batches(rank + 50, 2, 8, 64, cfg.vocab_size, device):
        step(x, y)       # moves the state away from the checkpoint
    template = get_optimizer_state_dict(model, opt)
    dcp.load({"optimizer": template}, checkpoint_id=folder[0])
    set_optimizer_state_dict(model, opt, template)
    after = get_optimizer_state_dict(model, opt)["state"]
    worst = 0.0
    for k, v in before.items():
        for kk, want in v.items():
            got = after[k][kk]
            got = got.to_local() if hasattr(got, "to_local") else got
            if want.numel():
                worst = max(worst, float((got.float().cpu() - want.float().cpu()).abs().max()))
    if rank == 0:
        print(f"checkpoint round trip: largest state difference {worst:.2e}")
    dist.barrier()
    dist.destroy_process_group()
    if losses[-1] >= losses[0] or worst >= 1e-2:
        raise SystemExit(f"rank {rank}: loss {losses[0]:.3f} -> {losses[-1]:.3f}, state difference {worst:.2e}")


if __name__ == "__main__":
    main()
