"""The reduce-scatter + AdamW kernels on ONE GPU with emulated ranks (for Nsight Compute).

    python benchmarks/peer_kernel_emulated.py --world 8 --variant staged --shard-elems 16777216

``world`` gradient buffers of ``shard-elems`` bf16 elements each live on this GPU and play the
ranks' rows; the flags that the other ranks would publish are written by the host beforehand, so
the kernel of "rank 0" never waits (kernels of different ranks never have to run at the same
time here).  What this measures is the kernel's instruction and memory behaviour — registers,
issue utilisation, bytes per element — with NVLink replaced by local HBM: the link latency and
bandwidth that bound the real kernel are NOT represented, so the times printed here are not
collective times (those come from ``benchmarks/fused_collective.py`` on real ranks).
Defaults: 8 x 32 MB of gradients + 172 MB of state, beyond the 126 MB L2 and far below a few GB.
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
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--variant", default="register", choices=["register", "staged"])
    ap.add_argument("--shard-elems", type=int, default=1 << 24)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--push", action="store_true", help="also store the new parameters into every rank's buffer")
    args = ap.parse_args()

    import torch

    from flashoptim_b200.ops.quant import quantize
    from flashoptim_b200.ops.step import AdamHyper, SegmentTable, launch_adam_peer, make_rows
    from flashoptim_b200.parallel.symm import PeerGroup, SymmBuffer

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w, n = args.world, args.shard_elems // 2048 * 2048
    bufs = [torch.empty(n * 2, dtype=torch.uint8, device=dev) for _ in range(w)]
    for b in bufs:
        b.view(torch.bfloat16).normal_(0, 1e-3)
    # flags far ahead of every epoch used below: every other rank has always "arrived" already
    pads = [torch.full((64 * 8,), 1 << 30, dtype=torch.int32, device=dev) for _ in range(w)]
    pushed = [torch.empty(n * 2, dtype=torch.uint8, device=dev) for _ in range(w)] if args.push else []
    group = PeerGroup(group=None, timeout_s=5.0)
    group.world, group.rank = w, 0
    group.variant = 1 if args.variant == "staged" else 0
    group.max_ctas = args.ctas
    p = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_(0, 0.02)
    ecc = torch.zeros(n, dtype=torch.int8, device=dev)
    m, ms = quantize(torch.zeros(n, device=dev))
    v, vs = quantize(torch.zeros(n, device=dev), signed=False, sqrt=True, softsign=False)
    rows = make_rows([p], [None], [ecc], [m], [ms], [v], [vs])
    rows[:, 1] = 0
    table = SegmentTable(dev)
    buf = SymmBuffer(bufs[0], [b.data_ptr() for b in bufs], 0)
    epoch = [0]

    def run():
        epoch[0] += 1
        a = group.comm_args(buf, epoch[0], 0, 1, pads=[q.data_ptr() for q in pads])
        if args.push:
            a.push = 1
            for r in range(w):
                a.param_out[r] = pushed[r].data_ptr()
            a.push_epoch, a.pushed_channel = epoch[0], 2
        h = AdamHyper(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=1e-6, step=epoch[0], decoupled=True,
                      grad_scale=1.0 / w)
        launch_adam_peer(table, rows, torch.bfloat16, 1, True, h, a)

    for _ in range(args.warmup):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    group.check_status()
    nbytes = n * (2 * w + 12.25 + (2 * w if args.push else 0))
    ms_ = sorted(times)[len(times) // 2]
    print(json.dumps({"bench": "reduce-scatter + AdamW-24 kernel, emulated ranks on one GPU", "world": w,
                      "variant": args.variant, "ctas": args.ctas, "shard_elems": n, "push": args.push,
                      "ms": round(ms_, 4), "local_bytes": nbytes, "local_GBps": round(nbytes / ms_ / 1e6, 1),
                      "note": "every 'remote' row is local HBM here: not a collective time"}), flush=True)


if __name__ == "__main__":
    main()
