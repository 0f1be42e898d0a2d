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


def _peer_kernel_worker(rank, world, mode):
    """``mode``: "p2p" (peer loads, register path), "multimem" (multimem.ld_reduce, four units
    per thread) or "staged" (bulk copies of the peers' chunks into shared memory)."""
    from flashoptim_b200.ops import oracle
    from flashoptim_b200.ops.quant import compute_ecc_bits, quantize
    from flashoptim_b200.ops.step import AdamHyper, SegmentTable, launch_adam_peer, make_rows
    from flashoptim_b200.parallel.symm import PeerGradients, PeerGroup

    use_multicast = mode == "multimem"
    errors = []
    dev = torch.device("cuda", rank)
    peers = PeerGroup(timeout_s=5.0, use_multicast=use_multicast, variant=1 if mode == "staged" else 0)
    # a large aligned tensor, one with a ragged tail, one smaller than a quantisation group
    sizes = [1 << 20, 50257, 33]
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (n + 7) // 8 * 8 * 2
    buf = peers.allocate(total)
    if use_multicast and not buf.multicast_ptr:
        return []  # no NVSwitch multicast on this machine: nothing to test
    ready, done = peers.new_channels()
    pg = PeerGradients(peers, buf, ready, done, grad_scale=1.0 / world)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    mine = torch.randn(total // 2, device=dev, generator=g) * 1e-3
    flat = buf.view(0, total // 2, torch.bfloat16)
    flat.copy_(mine)
    # NCCL reference for the mean gradient
    gsum = flat.float()
    dist.all_reduce(gsum)
    gmean_all = (gsum / world).cpu()
    # every rank builds the same state
    gs = torch.Generator(device=dev).manual_seed(7)
    states, wants, olds, gmeans = [], [], [], []
    for n, off in zip(sizes, offs):
        p32 = torch.randn(n, device=dev, generator=gs) * 0.02
        p = p32.to(torch.bfloat16)
        ecc = compute_ecc_bits(p32, p, master_bytewidth=3)
        m, ms = quantize(torch.randn(n, device=dev, generator=gs) * 1e-3)
        v, vs = quantize((torch.randn(n, device=dev, generator=gs) * 1e-3).square(), signed=False, sqrt=True,
                         softsign=False)
        states.append([p, ecc, m, ms, v, vs])
        gmean = gmean_all[off // 2: off // 2 + n]
        p_old = oracle.ecc_decode_ref(p.cpu(), ecc.cpu())
        wants.append(oracle.adam_math(
            p_old, gmean, oracle.dequantize_ref(m.cpu(), ms.cpu()),
            oracle.dequantize_ref(v.cpu(), vs.cpu(), signed=False, sqrt=True, softsign=False),
            lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, decoupled=True, step=1))
        olds.append(p_old)
        gmeans.append(gmean)
    cols = list(zip(*states))
    rows = make_rows(cols[0], [None] * len(sizes), cols[1], cols[2], cols[3], cols[4], cols[5])
    rows[:, 1] = offs
    out = torch.zeros(total // 2, dtype=torch.bfloat16, device=dev)
    pg.grad_out = out
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, step=1, decoupled=True,
                  grad_scale=1.0 / world)
    table = SegmentTable(dev)
    torch.cuda.synchronize()
    dist.barrier()
    launch_adam_peer(table, rows, torch.bfloat16, 1, True, h, pg.next_args())
    peers.check_status()
    for i, (st, (want_p, _, want_v), p_old, gmean, n, off) in enumerate(zip(states, wants, olds, gmeans, sizes, offs)):
        p, ecc = st[0], st[1]
        rec = oracle.ecc_decode_ref(p.cpu(), ecc.cpu())
        half_ulp = torch.exp2(oracle.ecc_log_scale(p.cpu()).float())
        # multimem.ld_reduce hands back the switch's fp32 sum narrowed to bf16 (observed: up to one
        # bf16 ULP, 2^-7 relative, from the exact sum).  Adam's step is at most linear in the
        # gradient, so allow that fraction (with margin) of the step taken.  Tails and unaligned
        # tensors go through peer loads in every mode, so the allowance is an upper bound there.
        g_tol = (2 ** -6 * (want_p - p_old).abs() + 1e-3 * 2 ** -6 * gmean.abs() /
                 ((want_v / (1 - 0.999)).sqrt() + 1e-8)) if use_multicast else 0
        bound = half_ulp * 0.75 / 127 + 4e-6 * (want_p - p_old).abs() + 4e-7 * want_p.abs() + 1e-10 + g_tol
        diff = (rec - want_p).abs()
        bad = diff > bound
        if bad.any():
            k = int((diff / bound).argmax())
            errors.append(f"rank {rank} {mode} tensor {i}: {int(bad.sum())} params off, worst "
                          f"x{float((diff / bound).max()):.1f} at {k}: got {float(rec[k])} want {float(want_p[k])} "
                          f"old {float(p_old[k])} g {float(gmean[k])} handed-back g {float(out[off // 2 + k])}")
        back = out[off // 2: off // 2 + n].float().cpu()
        if not torch.allclose(back, gmean, rtol=2 ** -6 if use_multicast else 2 ** -7, atol=1e-8):
            k = int((back - gmean).abs().argmax())
            errors.append(f"rank {rank} {mode} tensor {i}: averaged gradient hand-back is off at {k}: "
                          f"{float(back[k])} vs {float(gmean[k])}")
    # replicas bit-identical
    for i, st in enumerate(states):
        for name, t in zip(("param", "ecc", "exp_avg", "exp_avg_sq"), (st[0], st[1], st[2], st[4])):
            hi, lo = t.float().clone(), t.float().clone()
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            if not torch.equal(hi, lo):
                errors.append(f"rank {rank} {mode} tensor {i}: replicas differ in {name} "
                              f"({int((hi != lo).sum())} elements)")
                break
    # second use of the buffer: producers wait for done(epoch) first
    pg.wait_done()
    flat.copy_(mine * 2)
    h.step = 2
    launch_adam_peer(table, rows, torch.bfloat16, 1, True, h, pg.next_args())
    peers.check_status()
    dist.barrier()
    return errors


def test_peer_adam_kernel_two_gpus_p2p():
    run_distributed(_peer_kernel_worker, world_size=2, backend="nccl", args=("p2p",))


def test_peer_adam_kernel_two_gpus_multimem():
    run_distributed(_peer_kernel_worker, world_size=2, backend="nccl", args=("multimem",))


def test_peer_adam_kernel_two_gpus_staged():
    run_distributed(_peer_kernel_worker, world_size=2, backend="nccl", args=("staged",))


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


def _fsdp_worker(rank, world, staged=False, ag_copy_engine=False):
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
            own_ag = own_ag or ag_copy_engine
            state = enable_fused_fsdp(fused, o2, own_all_gather=own_ag, staged=staged, max_ctas=2 if staged else 0,
                                      all_gather_copy_engine=ag_copy_engine)
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


def test_fused_fsdp_copy_engine_all_gather():
    """FSDP2's parameter all-gather as copy-engine pulls between two flag kernels."""
    run_distributed(_fsdp_worker, world_size=2, backend="nccl", args=(False, True))


def test_fused_fsdp_staged_kernels_match_nccl_fsdp():
    run_distributed(_fsdp_worker, world_size=2, backend="nccl", args=(True,))


def _fsdp_accum_worker(rank, world):
    """Gradient accumulation through the fused reduce-scatter: micro-batches run with
    ``set_requires_gradient_sync(False)`` and only the last one reduces, which is then the
    optimizer update (what the reference tests against a single-process run,
    test/test_fsdp2.py:95-115, 444-455; here against FSDP2 on NCCL with the same schedule)."""
    from torch.distributed.fsdp import fully_shard

    from flashoptim_b200 import FlashAdamW
    from flashoptim_b200.parallel import enable_fused_fsdp

    dev = torch.device("cuda", rank)
    errors = []

    def shard(m):
        for layer in m:
            if isinstance(layer, nn.Linear):
                fully_shard(layer)
        fully_shard(m)
        return m

    for staged in (False, True):
        plain, fused = shard(_net(dev)), shard(_net(dev))
        o1 = FlashAdamW(plain.parameters(), lr=5e-4, weight_decay=1e-2)
        o2 = FlashAdamW(fused.parameters(), lr=5e-4, weight_decay=1e-2)
        state = enable_fused_fsdp(fused, o2, staged=staged, push_params=True)
        tol = get_tolerances(torch.bfloat16, True)
        batches = _batches(world, steps=6)
        for step in range(3):
            for micro in range(2):
                x, y = batches[2 * step + micro]
                xs = x[rank * 8:(rank + 1) * 8].to(dev, torch.bfloat16)
                ys = y[rank * 8:(rank + 1) * 8].to(dev)
                last = micro == 1
                for model in (plain, fused):
                    model.set_requires_gradient_sync(last)
                    (nn.functional.cross_entropy(model(xs).float(), ys) / 2).backward()
            for opt in (o1, o2):
                opt.step()
                opt.zero_grad()
            state.check()
            for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                        f"accumulation staged={staged} step {step} {n1}")
        if state.fused_calls < 3 * 4 or state.fallbacks:
            errors.append(f"accumulation staged={staged}: fused {state.fused_calls}, fallbacks {state.fallbacks}")
    return errors


def test_fused_fsdp_gradient_accumulation():
    run_distributed(_fsdp_accum_worker, world_size=2, backend="nccl")


def _fsdp_push_worker(rank, world, staged=False, transport="kernel"):
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
        # staged: gradients by bulk copies from the peers, parameters pushed with multimem.st
        state = enable_fused_fsdp(fused, o2, push_params=True, staged=staged,
                                  push_multicast=True if (staged and transport == "kernel") else None,
                                  transport=transport)
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


def test_fused_fsdp_param_push_from_staged_kernels():
    run_distributed(_fsdp_push_worker, world_size=2, backend="nccl", args=(True,))


def test_fused_fsdp_copy_engine_transport():
    """Gradient rows and parameter pushes cross NVLink in copy-engine copies; the update kernels
    (register path, then staged) read local memory.  Same checks as the in-kernel transport:
    training agrees with FSDP2 on NCCL and the pushed buffers equal an NCCL all-gather."""
    run_distributed(_fsdp_push_worker, world_size=2, backend="nccl", args=(False, "copy_engine"))
    run_distributed(_fsdp_push_worker, world_size=2, backend="nccl", args=(True, "copy_engine"))
