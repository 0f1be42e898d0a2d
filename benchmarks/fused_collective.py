"""Reduce-scatter fused with the sharded AdamW update vs NCCL reduce-scatter + local step.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29531 benchmarks/fused_collective.py --gpus 8

One FSDP2-style parameter group: ``--numel`` bf16 gradient elements per rank laid
out ``[world, shard]`` in a symmetric buffer (default 218 103 808 = one Llama-3-8B
layer).  Rank r reduces row r of every rank and updates its shard (AdamW, 24-bit
master weights, 8-bit states).  Timed on the device with CUDA events, max over
ranks; every iteration touches far more than the 126 MB L2.

``fused_peer_loads`` / ``fused_multimem`` are the register-path kernels, ``fused_staged`` the
bulk-copy staged kernel (``cp.async.bulk`` from the peers' memory into shared memory);
``--ctas 0,32,64`` times every fused variant at those grid caps (``name@cap``).
The ``*_push`` variants also store the updated bf16 shard into every rank's parameter buffer
(all-gather on write); their baseline is ``nccl_then_step_then_all_gather``.

Roofline of the fused kernel = the slower of
  * NVLink: bytes per direction per GPU / 770 GB/s (measured peer-copy rate).  With peer
    loads a rank receives (world-1) rows of shard*2 bytes and serves as many to its
    peers.  With multimem.ld_reduce the switch adds, so a rank receives one reduced row,
    but its memory is still read once for every other rank's row: (world-1)*shard*2 bytes
    leave each GPU either way, and that direction is the bound;
  * HBM: shard * (12.25 + 2) bytes (update traffic + this rank's own row) / measured copy
    bandwidth.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--numel", type=int, default=218103808)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ctas", default="0", help="comma-separated grid caps to time every fused variant at (0: none)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from flashoptim_b200.ops.quant import quantize
    from flashoptim_b200.ops.step import (
        AdamHyper, SegmentTable, launch_adam, launch_adam_peer, make_rows,
    )
    from flashoptim_b200.parallel.symm import ParamPush, PeerGradients, PeerGroup
    from flashoptim_b200.utils.timing import ClockSampler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29535")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    n = args.numel // (world * 2048) * (world * 2048)
    shard = n // world
    peers = PeerGroup(timeout_s=30.0, use_multicast=True)
    buf = peers.allocate(n * 2)
    ready, done = peers.new_channels()
    grads = buf.view(0, n, torch.bfloat16)
    grads.normal_(0, 1e-3)
    p = torch.empty(shard, dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
    ecc = torch.zeros(shard, dtype=torch.int8, device=dev)
    m, ms = quantize(torch.zeros(shard, device=dev))
    v, vs = quantize(torch.zeros(shard, device=dev), signed=False, sqrt=True, softsign=False)
    rs_out = torch.empty(shard, dtype=torch.bfloat16, device=dev)
    table_peer, table_local = SegmentTable(dev), SegmentTable(dev)
    rows_peer = make_rows([p], [None], [ecc], [m], [ms], [v], [vs])
    rows_peer[:, 1] = rank * shard * 2
    rows_local = make_rows([p], [rs_out], [ecc], [m], [ms], [v], [vs])

    def hyper(step, scale):
        return AdamHyper(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=1e-6, step=step,
                         decoupled=True, grad_scale=scale)

    # all-gather on write: the kernel also stores its new bf16 shard into row `rank` of a second
    # [world, shard] buffer on every rank (what FSDP2 would otherwise all-gather)
    push_target = ParamPush(peers.allocate(n * 2), peers.new_channel())

    results = {}
    ag_out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    caps = [int(c) for c in args.ctas.split(",")]
    names = []
    for base in ("fused_peer_loads", "fused_staged", "fused_multimem", "fused_peer_loads_push", "fused_staged_push",
                 "fused_staged_push_mc", "fused_multimem_push"):
        names += [f"{base}@{c}" if c else base for c in caps]
    names += ["nccl_then_step", "nccl_then_step_then_all_gather"]
    sampler = ClockSampler(local_rank)
    sampler.start()
    for name in names:
        kind, _, cap = name.partition("@")
        use_mc = "multimem" in kind
        if (use_mc or kind.endswith("_mc")) and not buf.multicast_ptr:
            continue
        pg = PeerGradients(peers, buf, ready, done, grad_scale=1.0 / world)
        pg.push = push_target if "_push" in kind else None
        peers.use_multicast = use_mc
        peers.push_multicast = use_mc or kind.endswith("_mc")
        peers.variant = 1 if "staged" in kind else 0
        peers.max_ctas = int(cap) if cap else 0
        pg.epoch = results.get("_epoch", 0)
        step = [0]

        def run():
            step[0] += 1
            if name.startswith("nccl"):
                dist.reduce_scatter_tensor(rs_out, grads, op=dist.ReduceOp.AVG)
                launch_adam(table_local, rows_local, torch.bfloat16, 1, True, hyper(step[0], 1.0))
                if kind.endswith("all_gather"):
                    dist.all_gather_into_tensor(ag_out, p)
            else:
                launch_adam_peer(table_peer, rows_peer, torch.bfloat16, 1, True, hyper(step[0], 1.0 / world),
                                 pg.next_args())

        for _ in range(args.warmup):
            run()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            run()
        e1.record()
        torch.cuda.synchronize()
        peers.check_status()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[name] = float(t.item())
        results["_epoch"] = pg.epoch
        dist.barrier()

    sampler.stop()
    if rank == 0:
        peak_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        hbm = float(json.load(open(peak_path))["hbm_gbs"]) if os.path.exists(peak_path) else 6650.0
        link = 770.0
        out = {"bench": "fused reduce-scatter + AdamW-24", "n_gpus": world, "grad_elems_per_rank": n,
               "shard_elems": shard}
        hbm_ms = shard * 14.25 / (hbm * 1e9) * 1e3
        for name, ms_ in results.items():
            if name.startswith("_"):
                continue
            rec = {"ms": round(ms_, 4)}
            if not name.startswith("nccl"):
                kind = name.partition("@")[0]
                pulls = "multimem" not in kind  # peer loads and bulk copies fetch every rank's row
                stores_mc = "multimem" in kind or kind.endswith("_mc")
                inbound = shard * 2 * ((world - 1) if pulls else (1 if world > 1 else 0))
                outbound = shard * 2 * (world - 1)
                if "_push" in kind:
                    # the new shard goes to the other world-1 ranks (peer stores: that many copies
                    # leave this GPU; multimem.st: one copy leaves and the switch replicates it),
                    # and world-1 shards arrive either way
                    inbound += shard * 2 * (world - 1)
                    outbound += shard * 2 * ((world - 1) if not stores_mc else (1 if world > 1 else 0))
                link_ms = max(inbound, outbound) / (link * 1e9) * 1e3
                roof = max(link_ms, hbm_ms)
                rec.update({"nvlink_inbound_MB": round(inbound / 1e6, 1),
                            "nvlink_outbound_MB": round(outbound / 1e6, 1), "roofline_ms": round(roof, 4),
                            "bound": "nvlink" if link_ms > hbm_ms else "hbm",
                            "frac_of_roofline": round(roof / ms_, 3)})
            out[name] = rec
        out["clocks"] = sampler.summary()
        print(json.dumps(out), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
