"""Two real GPUs: the peer kernels over NVLink symmetric memory, the fused DDP hook and
the fused FSDP2 reduce-scatter against their NCCL counterparts.  Workers never fault a
GPU: every device-side wait is bounded and reported through a status word."""

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from dist_utils import run_distributed
from helpers import check_similar, get_tolerances

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _net(device, dtype=torch.bfloat16, d=64):
    from flashoptim_b200 import cast_model

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d), nn.LayerNorm(d), nn.Linear(d, 16)).to(device)
    cast_model(m, dtype)
    return m


def _batches(world, d=64, steps=5):
    g = torch.Generator().manual_seed(11)
    return [(torch.randn(world * 8, d, generator=g), torch.randint(0, 16, (world * 8,), generator=g))
            for _ in range(steps)]


def _peer_kernel_worker(rank, world, use_multicast):
    from flashoptim_b200.ops import oracle
    from flashoptim_b200.ops.quant import compute_ecc_bits, quantize
    from flashoptim_b200.ops.step import AdamHyper, SegmentTable, launch_adam_peer, make_rows
    from flashoptim_b200.parallel.symm import PeerGradients, PeerGroup

    errors = []
    dev = torch.device("cuda", rank)
    peers = PeerGroup(timeout_s=5.0, use_multicast=use_multicast)
    n = 1 << 20
    buf = peers.allocate(n * 2)
    if use_multicast and not buf.multicast_ptr:
        return []  # no NVSwitch multicast on this machine: nothing to test
    ready, done = peers.new_channels()
    pg = PeerGradients(peers, buf, ready, done, grad_scale=1.0 / world)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    mine = torch.randn(n, device=dev, generator=g) * 1e-3
    buf.view(0, n, torch.bfloat16).copy_(mine)
    # every rank builds the same state
    gs = torch.Generator(device=dev).manual_seed(7)
    p32 = torch.randn(n, device=dev, generator=gs) * 0.02
    p = p32.to(torch.bfloat16)
    ecc = compute_ecc_bits(p32, p, master_bytewidth=3)
    m, ms = quantize(torch.randn(n, device=dev, generator=gs) * 1e-3)
    v, vs = quantize((torch.randn(n, device=dev, generator=gs) * 1e-3).square(), signed=False, sqrt=True,
                     softsign=False)
    # NCCL reference for the mean gradient
    gsum = buf.view(0, n, torch.bfloat16).float()
    dist.all_reduce(gsum)
    gmean = (gsum / world).cpu()
    p_old = oracle.ecc_decode_ref(p.cpu(), ecc.cpu())
    want_p, want_m, want_v = oracle.adam_math(
        p_old, gmean, oracle.dequantize_ref(m.cpu(), ms.cpu()),
        oracle.dequantize_ref(v.cpu(), vs.cpu(), signed=False, sqrt=True, softsign=False),
        lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, decoupled=True, step=1)
    rows = make_rows([p], [None], [ecc], [m], [ms], [v], [vs])
    rows[:, 1] = 0
    out = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    pg.grad_out = out
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, step=1, decoupled=True,
                  grad_scale=1.0 / world)
    torch.cuda.synchronize()
    dist.barrier()
    launch_adam_peer(SegmentTable(dev), rows, torch.bfloat16, 1, True, h, pg.next_args())
    peers.check_status()
    rec = oracle.ecc_decode_ref(p.cpu(), ecc.cpu())
    half_ulp = torch.exp2(oracle.ecc_log_scale(p.cpu()).float())
    # multimem.ld_reduce hands back the switch's fp32 sum narrowed to bf16 (observed: up to one
    # bf16 ULP, 2^-7 relative, from the exact sum).  Adam's step is at most linear in the
    # gradient, so allow that fraction (with margin) of the step taken.
    g_tol = (2 ** -6 * (want_p - p_old).abs() + 1e-3 * 2 ** -6 * gmean.abs() /
             ((want_v / (1 - 0.999)).sqrt() + 1e-8)) if use_multicast else 0
    bound = half_ulp * 0.75 / 127 + 4e-6 * (want_p - p_old).abs() + 4e-7 * want_p.abs() + 1e-10 + g_tol
    diff = (rec - want_p).abs()
    bad = diff > bound
    if bad.any():
        i = int((diff / bound).argmax())
        errors.append(f"rank {rank} mc={use_multicast}: {int(bad.sum())} params off, worst x{float((diff / bound).max()):.1f} "
                      f"at {i}: got {float(rec[i])} want {float(want_p[i])} old {float(p_old[i])} g {float(gmean[i])} "
                      f"handed-back g {float(out[i])}")
    if not torch.allclose(out.float().cpu(), gmean, rtol=2 ** -6 if use_multicast else 2 ** -7, atol=1e-8):
        errors.append(f"rank {rank} mc={use_multicast}: averaged gradient hand-back is off")
    # replicas bit-identical
    for t in (p, ecc, m, v):
        hi, lo = t.float().clone(), t.float().clone()
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        if not torch.equal(hi, lo):
            errors.append(f"rank {rank} mc={use_multicast}: replicas differ")
            break
    # second use of the buffer: producers wait for done(epoch) first
    pg.wait_done()
    buf.view(0, n, torch.bfloat16).copy_(mine * 2)
    h.step = 2
    launch_adam_peer(SegmentTable(dev), rows, torch.bfloat16, 1, True, h, pg.next_args())
    peers.check_status()
    dist.barrier()
    return errors


def test_peer_adam_kernel_two_gpus_p2p():
    run_distributed(_peer_kernel_worker, world_size=2, backend="nccl", args=(False,))


def test_peer_adam_kernel_two_gpus_multimem():
    run_distributed(_peer_kernel_worker, world_size=2, backend="nccl", args=(True,))


def _ddp_worker(rank, world, two_shot=False):
    from torch.nn.parallel import DistributedDataParallel as DDP

    from flashoptim_b200 import FlashAdamW, FlashLion
    from flashoptim_b200.parallel import fuse_ddp_allreduce

    dev = torch.device("cuda", rank)
    errors = []
    for cls, kw in ((FlashAdamW, dict(lr=5e-4, weight_decay=1e-2)), (FlashLion, dict(lr=2e-4))):
        plain = DDP(_net(dev), device_ids=[rank])
        fused = DDP(_net(dev), device_ids=[rank], gradient_as_bucket_view=True, bucket_cap_mb=0.05)
        o1 = cls(plain.parameters(), **kw)
        o2 = cls(fused.parameters(), **kw)
        state = fuse_ddp_allreduce(fused, o2, two_shot=two_shot, two_shot_min_bytes=1024)
        tol = get_tolerances(torch.bfloat16, True)
        for step, (x, y) in enumerate(_batches(world)):
            xs = x[rank * 8:(rank + 1) * 8].to(dev, torch.bfloat16)
            ys = y[rank * 8:(rank + 1) * 8].to(dev)
            accumulate = step == 1
            for model, opt in ((plain, o1), (fused, o2)):
                if accumulate:
                    with model.no_sync():
                        nn.functional.cross_entropy(model(xs).float(), ys).backward()
                else:
                    nn.functional.cross_entropy(model(xs).float(), ys).backward()
                    opt.step()
                    opt.zero_grad()
            if accumulate:
                continue
            state.check()
            for (n1, p1), (_, p2) in zip(plain.module.named_parameters(), fused.module.named_parameters()):
                errors += check_similar(p2.detach(), p1.detach(), tol, f"{cls.__name__} step {step} {n1}")
            for p in fused.parameters():
                hi, lo = p.detach().float().clone(), p.detach().float().clone()
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                if not torch.equal(hi, lo):
                    errors.append(f"{cls.__name__} step {step}: fused replicas diverged")
                    break
        if state.buckets_fused < 4:
            errors.append(f"{cls.__name__}: only {state.buckets_fused} buckets went through the fused hook")
        if two_shot and state.buckets_two_shot < 4:
            errors.append(f"{cls.__name__}: only {state.buckets_two_shot} buckets took the two-shot route")
    return errors


def test_fused_ddp_matches_nccl_ddp():
    run_distributed(_ddp_worker, world_size=2, backend="nccl")


def test_fused_ddp_two_shot_matches_nccl_ddp():
    run_distributed(_ddp_worker, world_size=2, backend="nccl", args=(True,))


def _fsdp_worker(rank, world):
    from torch.distributed.fsdp import fully_shard

    from flashoptim_b200 import FlashAdamW, FlashLion, enable_gradient_release
    from flashoptim_b200.parallel import enable_fused_fsdp

    dev = torch.device("cuda", rank)
    errors = []

    def shard(m):
        for layer in m:
            if isinstance(layer, nn.Linear):
                fully_shard(layer)
        fully_shard(m)
        return m

    for cls, kw in ((FlashAdamW, dict(lr=5e-4, weight_decay=1e-2)), (FlashLion, dict(lr=2e-4))):
        for release in (False, True):
            plain, fused = shard(_net(dev)), shard(_net(dev))
            o1 = cls(plain.parameters(), **kw)
            o2 = cls(fused.parameters(), **kw)
            own_ag = release  # half of the cases also use the library's all-gather kernel
            state = enable_fused_fsdp(fused, o2, own_all_gather=own_ag)
            if release:
                enable_gradient_release(plain, o1)
                enable_gradient_release(fused, o2)
            tol = get_tolerances(torch.bfloat16, True)
            for step, (x, y) in enumerate(_batches(world)):
                xs = x[rank * 8:(rank + 1) * 8].to(dev, torch.bfloat16)
                ys = y[rank * 8:(rank + 1) * 8].to(dev)
                for model, opt in ((plain, o1), (fused, o2)):
                    nn.functional.cross_entropy(model(xs).float(), ys).backward()
                    if not release:
                        opt.step()
                        opt.zero_grad()
                state.check()
                for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                    errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                            f"{cls.__name__} release={release} step {step} {n1}")
            if state.fused_calls < 5 or state.fallbacks:
                errors.append(f"{cls.__name__} release={release}: fused {state.fused_calls}, fallbacks {state.fallbacks}")
            if own_ag and state.ag_calls < 5:
                errors.append(f"{cls.__name__}: own all-gather ran {state.ag_calls} times, fell back {state.ag_fallbacks}")
    return errors


def test_fused_fsdp_matches_nccl_fsdp():
    run_distributed(_fsdp_worker, world_size=2, backend="nccl")


def _fsdp_push_worker(rank, world):
    from torch.distributed.fsdp import fully_shard

    from flashoptim_b200 import FlashAdamW, enable_gradient_release
    from flashoptim_b200.parallel import enable_fused_fsdp

    dev = torch.device("cuda", rank)
    errors = []

    def shard(m):
        for layer in m:
            if isinstance(layer, nn.Linear):
                fully_shard(layer)
        fully_shard(m)
        return m

    for release in (False, True):
        plain, fused = shard(_net(dev)), shard(_net(dev))
        o1 = FlashAdamW(plain.parameters(), lr=5e-4, weight_decay=1e-2)
        o2 = FlashAdamW(fused.parameters(), lr=5e-4, weight_decay=1e-2)
        state = enable_fused_fsdp(fused, o2, push_params=True)
        if release:
            enable_gradient_release(plain, o1)
            enable_gradient_release(fused, o2)
        tol = get_tolerances(torch.bfloat16, True)
        for step, (x, y) in enumerate(_batches(world)):
            xs = x[rank * 8:(rank + 1) * 8].to(dev, torch.bfloat16)
            ys = y[rank * 8:(rank + 1) * 8].to(dev)
            losses = []
            for model, opt in ((plain, o1), (fused, o2)):
                loss = nn.functional.cross_entropy(model(xs).float(), ys)
                loss.backward()
                losses.append(float(loss))
                if not release:
                    opt.step()
                    opt.zero_grad()
            state.check()
            if abs(losses[0] - losses[1]) > 2e-2 * max(1.0, abs(losses[0])):
                errors.append(f"release={release} step {step}: loss {losses[1]} vs {losses[0]}")
            for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                        f"push release={release} step {step} {n1}")
            # what the next all-gathers hand to FSDP2: every rank's shards, bit for bit
            for gi, gather in enumerate(state.gathers):
                if not gather.is_current():
                    errors.append(f"release={release} step {step}: group {gi} was not pushed")
                    continue
                t = gather.target
                state.peers.wait(state.peers.comm_args(t.buf, t.epoch, t.channel, t.channel), t.channel)
                mine = torch.cat([fp._sharded_param_data.view(-1) for fp in gather.rs.fsdp_params])
                want = torch.empty(world * mine.numel(), dtype=mine.dtype, device=dev)
                dist.all_gather_into_tensor(want, mine)
                got = t.buf.view(0, want.numel(), want.dtype)
                if not torch.equal(got.view(torch.int16), want.view(torch.int16)):
                    bad = int((got.view(torch.int16) != want.view(torch.int16)).sum())
                    errors.append(f"release={release} step {step}: group {gi}: {bad} pushed elements differ")
            state.check()
        if state.fallbacks or state.ag_eliminated < 8:
            errors.append(f"release={release}: rs fallbacks {state.fallbacks}, all-gathers without data movement "
                          f"{state.ag_eliminated}, with NCCL {state.ag_fallbacks}")
        # a local update (no push) must send the next all-gather back to NCCL
        before = state.ag_fallbacks
        if not release:
            for p in fused.parameters():
                p.grad = torch.zeros_like(p)
            o2.step()
            o2.zero_grad()
            if any(g.is_current() for g in state.gathers):
                errors.append("a local step left pushed parameters marked current")
            with torch.no_grad():
                fused(xs)
            if state.ag_fallbacks == before:
                errors.append("all-gather after a local step did not move data")
            state.check()
    return errors


def test_fused_fsdp_param_push_replaces_all_gather():
    run_distributed(_fsdp_push_worker, world_size=2, backend="nccl")
