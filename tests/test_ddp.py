"""DistributedDataParallel (modelled on the reference's ``test/test_ddp.py``): a DDP run on
two ranks against a single-process run on the concatenated batch, weights compared every
step and bit-equality across ranks.  CPU ranks over gloo; the same body on two GPUs over NCCL."""

import warnings

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from flashoptim_b200 import FlashAdamW, FlashLion, FlashSGD, cast_model, enable_gradient_release

from dist_utils import run_distributed
from helpers import check_similar, get_tolerances

CONFIGS = [  # dtype, master_weight_bits, quantize
    (torch.float32, None, False), (torch.float32, None, True),
    (torch.bfloat16, 24, True), (torch.bfloat16, 32, True),
]
OPTS = [
    ("adamw", FlashAdamW, dict(lr=5e-4, weight_decay=1e-2)),
    ("lion", FlashLion, dict(lr=5e-4, weight_decay=1e-2)),
    ("sgd", FlashSGD, dict(lr=5e-2, momentum=0.9)),
]


def _net(dtype, device):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(10, 16), nn.ReLU(), nn.Linear(16, 5)).to(device)
    if dtype != torch.float32:
        cast_model(m, dtype)
    return m


def _worker(rank, world, use_cuda):
    from torch.nn.parallel import DistributedDataParallel as DDP

    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    errors = []
    g = torch.Generator().manual_seed(123)
    data = [(torch.randn(world * 8, 10, generator=g), torch.randint(0, 5, (world * 8,), generator=g))
            for _ in range(6)]
    for oname, cls, kw in OPTS:
        for accumulate in (False, True):
            for dtype, mwb, quantize in CONFIGS:
                tag = f"{oname} acc={accumulate} {dtype} mwb={mwb} q={quantize}"
                with warnings.catch_warnings():
                    warnings.simplefilter("ignore")
                    single = _net(dtype, device)
                    ddp = DDP(_net(dtype, device), device_ids=[rank] if use_cuda else None)
                    o1 = cls(single.parameters(), master_weight_bits=mwb, quantize=quantize, **kw)
                    o2 = cls(ddp.parameters(), master_weight_bits=mwb, quantize=quantize, **kw)
                tol = get_tolerances(dtype, quantize)
                for step, (x, y) in enumerate(data):
                    x, y = x.to(device=device, dtype=dtype), y.to(device)
                    xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
                    nn.functional.cross_entropy(single(x).float(), y).backward()
                    if accumulate and step % 2 == 0:
                        # both runs keep this micro-batch's gradient and step after the next one;
                        # the all-reduce of the next backward averages the accumulated sum
                        with ddp.no_sync():
                            nn.functional.cross_entropy(ddp(xs).float(), ys).backward()
                        continue
                    nn.functional.cross_entropy(ddp(xs).float(), ys).backward()
                    o1.step(); o1.zero_grad(); o2.step(); o2.zero_grad()
                    for (n1, p1), (n2, p2) in zip(single.named_parameters(), ddp.module.named_parameters()):
                        errors += check_similar(p2.detach(), p1.detach(), tol, f"{tag} step {step} {n1}")
                    for p in ddp.parameters():  # replicas must agree exactly
                        hi, lo = p.detach().float().clone(), p.detach().float().clone()
                        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                        if not torch.equal(hi, lo):
                            errors.append(f"{tag} step {step}: replicas diverged")
                sd = o2.get_fp32_model_state_dict(ddp)  # unwraps .module
                if set(sd) != set(single.state_dict()):
                    errors.append(f"{tag}: fp32 export keys {sorted(sd)}")
    # gradient release is refused for DDP
    ddp = DDP(_net(torch.float32, device), device_ids=[rank] if use_cuda else None)
    opt = FlashAdamW(ddp.parameters(), lr=1e-3, master_weight_bits=None)
    try:
        enable_gradient_release(ddp, opt)
        errors.append("enable_gradient_release accepted a DDP model")
    except TypeError:
        pass
    return errors


def test_ddp_gloo_two_ranks():
    run_distributed(_worker, world_size=2, backend="gloo", args=(False,))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_ddp_nccl_two_gpus():
    run_distributed(_worker, world_size=2, backend="nccl", args=(True,))
