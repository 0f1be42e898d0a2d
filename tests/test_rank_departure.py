"""A rank that leaves between steps: the survivors' next fused step must not hang.  Its
device-side wait for the missing rank runs out, the kernel returns, and the host raises
``CommTimeoutError`` naming that rank.  The leaver exits with nothing in flight; NVLS is
off and the peer kernels use plain peer loads (no multicast mapping is created)."""

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _worker(rank, world):
    import os

    # PyTorch's symmetric-memory allocator binds buffers to an NVSwitch multicast object when
    # it can; this test wants none (set before the first symmetric allocation of the process)
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    from flashoptim_b200.ops.quant import quantize
    from flashoptim_b200.ops.step import AdamHyper, SegmentTable, launch_adam_peer, make_rows
    from flashoptim_b200.parallel.symm import CommTimeoutError, PeerGradients, PeerGroup

    dev = torch.device("cuda", rank)
    errors = []
    peers = PeerGroup(timeout_s=1.0, use_multicast=False)
    n = 1 << 16
    buf = peers.allocate(n * 2)
    ready, done = peers.new_channels()
    pg = PeerGradients(peers, buf, ready, done, grad_scale=1.0 / world)
    buf.view(0, n, torch.bfloat16).fill_(1e-3)
    p = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    m, ms = quantize(torch.zeros(n, device=dev))
    v, vs = quantize(torch.zeros(n, device=dev), signed=False, sqrt=True, softsign=False)
    rows = make_rows([p], [None], [None], [m], [ms], [v], [vs])
    rows[:, 1] = 0
    table = SegmentTable(dev)
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True,
                  grad_scale=1.0 / world)
    # step 1: everybody takes part
    launch_adam_peer(table, rows, torch.bfloat16, 0, True, h, pg.next_args())
    peers.check_status()
    if float(p.float().abs().sum()) == 0:
        errors.append(f"rank {rank}: first step did nothing")
    torch.cuda.synchronize()
    dist.barrier()
    # between steps rank 1 stops taking part (it keeps its mappings alive until the others
    # have seen the timeout, so nobody reads unmapped memory)
    snapshot = p.clone()
    if rank != 1:
        h.step = 2
        launch_adam_peer(table, rows, torch.bfloat16, 0, True, h, pg.next_args())
        try:
            peers.check_status()
            errors.append(f"rank {rank}: step with a missing rank did not report a timeout")
        except CommTimeoutError as e:
            if "missing rank 1" not in str(e):
                errors.append(f"rank {rank}: wrong diagnosis: {e}")
        if not torch.equal(snapshot, p):
            errors.append(f"rank {rank}: parameters changed although the step timed out")
        # the context still works
        if float((p.float() * 2).sum()) != float(p.float().sum()) * 2:
            errors.append(f"rank {rank}: device unusable after the timeout")
    dist.barrier()
    return errors


def test_survivors_report_missing_rank():
    run_distributed(_worker, world_size=2, backend="nccl")
