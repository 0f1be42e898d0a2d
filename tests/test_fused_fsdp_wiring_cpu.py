"""FSDP2 wiring of the fused reduce-scatter and of the all-gather on write, on two gloo
ranks: the NVLink group and the two kernels are replaced by stand-ins that do the same
thing with gloo collectives, so that FSDP2 itself drives ``allocate()`` / ``__call__()``,
the buffers, the validity bookkeeping and the fall-backs exactly as on GPUs."""

import warnings

import torch
import torch.distributed as dist
import torch.nn as nn

from dist_utils import run_distributed
from helpers import check_similar, get_tolerances


class _FakePeers:
    """Stands in for ``PeerGroup``: ordinary host tensors as "symmetric" buffers; waits are
    no-ops because the stand-in kernels below are blocking gloo collectives."""

    def __init__(self, group=None, device=None, timeout_s=2.0, use_multicast=True, max_ctas=0,
                 push_multicast=None, variant=0):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device("cpu")
        self.use_multicast = False
        self._next_channel = 0
        self.waits = 0

    def allocate(self, nbytes, zero=False):
        from flashoptim_b200.parallel.symm import SymmBuffer

        t = torch.zeros((int(nbytes) + 255) // 256 * 256, dtype=torch.uint8)
        return SymmBuffer(t, [t.data_ptr()] * self.world, 0)

    def new_channel(self):
        self._next_channel += 1
        return self._next_channel - 1

    def new_channels(self):
        self._next_channel += 2
        return self._next_channel - 2, self._next_channel - 1

    def comm_args(self, buf, epoch, ready, done, grad_out=None, grad_out_sub=0):
        from flashoptim_b200.ops import native

        a = native.FoCommArgs()
        a.world, a.rank, a.epoch = self.world, self.rank, epoch
        return a

    def wait(self, args, channel):
        self.waits += 1

    def check_status(self):
        pass


def _fake_step_from_peers(opt, params, slot):
    """What the fused kernel does, with gloo: average the ranks' [world, row] gradient
    matrices, hand row `rank` back, update the shards, and (all-gather on write) leave every
    rank's new shards in every rank's parameter buffer."""
    from torch.distributed.tensor import DTensor

    from flashoptim_b200.optim.base import local_tensor

    peers = slot.group
    locals_ = [local_tensor(p) for p in params]
    dtype = locals_[0].dtype
    esize = locals_[0].element_size()
    row_bytes = slot.grad_out.numel() * esize
    full = slot.buf.view(0, peers.world * slot.grad_out.numel(), dtype).float()
    dist.all_reduce(full, group=peers.group)
    mine = (full.view(peers.world, -1)[peers.rank] / peers.world).to(dtype)
    slot.grad_out.copy_(mine)
    slot.next_args()  # one launch: advances the epochs as the real path does
    for p, pl in zip(params, locals_):
        off = (slot.offsets[id(pl)] - slot.grad_out_sub) // esize
        g = mine[off:off + pl.numel()].view(pl.shape)
        p.grad = (DTensor.from_local(g, p.device_mesh, p.placements, run_check=False, shape=p.shape, stride=p.stride())
                  if hasattr(p, "device_mesh") else g)
    index_of = {id(p): gi for gi, g in enumerate(opt.param_groups) for p in g["params"]}
    for p in params:
        opt._step_group([p], opt.param_groups[index_of[id(p)]], index_of[id(p)])
        opt._peer_stepped.add(id(p))
    if slot.push is not None:
        out = slot.push.buf.view(0, peers.world * slot.grad_out.numel(), dtype)
        shard = torch.zeros(slot.grad_out.numel(), dtype=dtype)
        for pl in locals_:
            off = (slot.offsets[id(pl)] - slot.grad_out_sub) // esize
            shard[off:off + pl.numel()] = pl.reshape(-1)
        dist.all_gather_into_tensor(out, shard, group=peers.group)
    assert row_bytes * peers.rank == slot.grad_out_sub


def _net():
    from flashoptim_b200 import cast_model

    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 16), nn.LayerNorm(16), nn.Linear(16, 8))
    cast_model(m, torch.bfloat16)
    return m


def _worker(rank, world):
    from torch.distributed.fsdp import fully_shard

    import flashoptim_b200.parallel.fsdp as fsdp_mod
    from flashoptim_b200 import FlashAdamW, enable_gradient_release
    from flashoptim_b200.optim.base import FlashOptimizer

    errors = []
    fsdp_mod.PeerGroup = _FakePeers
    real_local_listeners = []

    def shard(m, reshard=True):
        for layer in m:
            if isinstance(layer, nn.Linear):
                fully_shard(layer, reshard_after_forward=reshard)
        fully_shard(m, reshard_after_forward=reshard)
        return m

    g = torch.Generator().manual_seed(3)
    data = [(torch.randn(world * 4, 16, generator=g), torch.randint(0, 8, (world * 4,), generator=g))
            for _ in range(4)]
    for push, release, reshard in ((False, False, True), (True, False, True), (True, True, True),
                                   (True, False, False)):
        tag = f"push={push} release={release} reshard={reshard}"
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            plain, fused = shard(_net(), reshard), shard(_net(), reshard)
            o1 = FlashAdamW(plain.parameters(), lr=5e-4)
            o2 = FlashAdamW(fused.parameters(), lr=5e-4)
        o2.step_from_peers = lambda params, slot, _o=o2: _fake_step_from_peers(_o, params, slot)
        state = fsdp_mod.enable_fused_fsdp(fused, o2, push_params=push)
        if release:
            enable_gradient_release(plain, o1)
            enable_gradient_release(fused, o2)
        tol = get_tolerances(torch.bfloat16, True)
        for step, (x, y) in enumerate(data):
            xs, ys = x[rank * 4:(rank + 1) * 4].bfloat16(), y[rank * 4:(rank + 1) * 4]
            for model, opt in ((plain, o1), (fused, o2)):
                nn.functional.cross_entropy(model(xs).float(), ys).backward()
                if not release:
                    opt.step()
                    opt.zero_grad()
            for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                        f"{tag} step {step} {n1}")
            if push and not all(gather.is_current() for gather in state.gathers):
                errors.append(f"{tag} step {step}: a group is not marked current after its push")
        if state.fallbacks or state.fused_calls != 4 * len(data):
            errors.append(f"{tag}: {state.fused_calls} fused reduce-scatters, {state.fallbacks} fall-backs")
        if push:
            # first step: nothing pushed yet -> NCCL-style all-gathers; later steps: flag waits only
            if state.ag_eliminated < 4 * (len(data) - 1) or state.ag_fallbacks > 8:
                errors.append(f"{tag}: {state.ag_eliminated} all-gathers without data movement, "
                              f"{state.ag_fallbacks} with")
            if not release:
                before = state.ag_fallbacks
                for p in fused.parameters():
                    p.grad = torch.zeros_like(p)
                o2.step()  # a local update: the pushed copies are stale now
                o2.zero_grad()
                if any(gather.is_current() for gather in state.gathers):
                    errors.append(f"{tag}: a local step left pushed parameters marked current")
                with torch.no_grad():
                    fused(xs)
                if state.ag_fallbacks == before:
                    errors.append(f"{tag}: the all-gather after a local step moved no data")
        elif state.ag_eliminated or state.gathers:
            errors.append(f"{tag}: all-gathers were touched without push_params")
        # remove(): the next step runs on FSDP2's own collectives and still matches
        if not release:
            calls = (state.fused_calls, state.ag_eliminated)
            state.remove()
            x, y = data[0]
            xs, ys = x[rank * 4:(rank + 1) * 4].bfloat16(), y[rank * 4:(rank + 1) * 4]
            for model, opt in ((plain, o1), (fused, o2)):
                nn.functional.cross_entropy(model(xs).float(), ys).backward()
                opt.step()
                opt.zero_grad()
            if (state.fused_calls, state.ag_eliminated) != calls:
                errors.append(f"{tag}: the fused path still ran after remove()")
            if not push:  # (with push the fused model took one extra local step above)
                for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                    errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                            f"{tag} after remove {n1}")
    # gradient accumulation: only the last micro-batch synchronises, and that reduce-scatter is the update
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        plain, fused = shard(_net()), shard(_net())
        o1 = FlashAdamW(plain.parameters(), lr=5e-4)
        o2 = FlashAdamW(fused.parameters(), lr=5e-4)
    o2.step_from_peers = lambda params, slot, _o=o2: _fake_step_from_peers(_o, params, slot)
    state = fsdp_mod.enable_fused_fsdp(fused, o2, push_params=True)
    for step in range(2):
        for micro, (x, y) in enumerate(data[:2]):
            xs, ys = x[rank * 4:(rank + 1) * 4].bfloat16(), y[rank * 4:(rank + 1) * 4]
            for model in (plain, fused):
                model.set_requires_gradient_sync(micro == 1)
                nn.functional.cross_entropy(model(xs).float(), ys).backward()
        for opt in (o1, o2):
            opt.step()
            opt.zero_grad()
        for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
            errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(),
                                    get_tolerances(torch.bfloat16, True), f"accumulation step {step} {n1}")
    if state.fused_calls != 8 or state.fallbacks:
        errors.append(f"accumulation: {state.fused_calls} fused reduce-scatters, {state.fallbacks} fall-backs")

    # a user's all-reduce hook post-processes the reduce-scatter output: leave those groups alone
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        hooked = shard(_net())
        o3 = FlashAdamW(hooked.parameters(), lr=5e-4)
    o3.step_from_peers = lambda params, slot: errors.append("fused update ran although an all-reduce hook is set")
    state = fsdp_mod.enable_fused_fsdp(hooked, o3)
    for pg in (m._get_fsdp_state()._fsdp_param_group for m in hooked.modules() if hasattr(m, "_get_fsdp_state")):
        if pg is not None:
            pg._all_reduce_hook = lambda t: None
    x, y = data[0]
    nn.functional.cross_entropy(hooked(x[rank * 4:(rank + 1) * 4].bfloat16()).float(), y[rank * 4:(rank + 1) * 4]).backward()
    o3.step()
    if state.fused_calls or not state.fallbacks:
        errors.append(f"hooked groups: fused {state.fused_calls}, fall-backs {state.fallbacks}")
    return errors


def test_fused_fsdp_wiring_on_gloo():
    run_distributed(_worker, world_size=2, backend="gloo")
