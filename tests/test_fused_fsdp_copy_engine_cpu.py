"""Host-side logic of the copy-engine paths of the fused FSDP2 integration, on two and three gloo ranks.

``FusedReduceScatter._pull_rows`` / ``_finish_copy_engine`` and the copy-engine branch of
``PeerAllGather`` compute source and destination addresses in the ranks' symmetric buffers
(rows, slots, the push offset) and issue one copy per peer between a barrier and a flag
signal.  Here the NVLink group is replaced by a stand-in with a made-up address space
(rank and buffer number in the high bits of every "pointer") whose ``copy()`` performs the
transfer that those addresses describe over gloo, so that wrong offsets, rows or sizes show up as
wrong parameters.  FSDP2 itself drives ``allocate()`` / ``__call__()`` as on GPUs.
"""

import ctypes
import warnings

import torch
import torch.distributed as dist
import torch.nn as nn

from dist_utils import run_distributed
from helpers import check_similar, get_tolerances
from test_fused_fsdp_wiring_cpu import _FakePeers, _fake_step_from_peers

_RANK_SHIFT, _BUF_SHIFT = 48, 32


class _AddressedPeers(_FakePeers):
    """``_FakePeers`` whose buffers have distinguishable per-rank addresses and whose copies,
    barriers and signals are executed over gloo (every rank calls them in the same order)."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.buffers = []
        self.copies = 0
        self.barriers = 0
        self.signals = 0

    def allocate(self, nbytes, zero=False):
        from flashoptim_b200.parallel.symm import SymmBuffer

        t = torch.zeros((int(nbytes) + 255) // 256 * 256, dtype=torch.uint8)
        k = len(self.buffers)
        self.buffers.append(t)
        return SymmBuffer(t, [((p + 1) << _RANK_SHIFT) | (k << _BUF_SHIFT) for p in range(self.world)], 0)

    def _decode(self, addr):
        """(rank, local address) of a made-up or a real pointer."""
        if addr >> _RANK_SHIFT == 0:
            return self.rank, addr  # an ordinary host pointer of this process
        rank = (addr >> _RANK_SHIFT) - 1
        k = (addr >> _BUF_SHIFT) & 0xFFFF
        off = addr & ((1 << _BUF_SHIFT) - 1)
        assert off < self.buffers[k].numel(), f"offset {off} outside buffer {k}"
        return rank, ("buf", k, off)

    def _local_ptr(self, where, nbytes):
        if isinstance(where, tuple):
            _, k, off = where
            assert off + nbytes <= self.buffers[k].numel(), "copy runs past the end of a symmetric buffer"
            return self.buffers[k].data_ptr() + off
        return where

    def barrier(self, args):
        self.barriers += 1
        dist.barrier(self.group)

    def signal(self, args, channel):
        self.signals += 1

    def copy(self, dst, src, nbytes):
        self.copies += 1
        (drank, dwhere), (srank, swhere) = self._decode(dst), self._decode(src)
        assert drank == self.rank or srank == self.rank, "a copy between two other ranks"
        request = None
        if srank != self.rank:
            request = ("read", srank, swhere, nbytes)
        elif drank != self.rank:
            payload = ctypes.string_at(self._local_ptr(swhere, nbytes), nbytes)
            request = ("write", drank, dwhere, payload)
        else:
            ctypes.memmove(self._local_ptr(dwhere, nbytes), self._local_ptr(swhere, nbytes), nbytes)
        requests = [None] * self.world
        dist.all_gather_object(requests, request, group=self.group)
        replies = {}
        for q, req in enumerate(requests):
            if req is None or req[1] != self.rank:
                continue
            if req[0] == "read":
                replies[q] = ctypes.string_at(self._local_ptr(req[2], req[3]), req[3])
            else:
                ctypes.memmove(self._local_ptr(req[2], len(req[3])), req[3], len(req[3]))
        all_replies = [None] * self.world
        dist.all_gather_object(all_replies, replies, group=self.group)
        if request is not None and request[0] == "read":
            data = all_replies[srank][self.rank]
            assert len(data) == nbytes
            ctypes.memmove(self._local_ptr(dwhere, nbytes), data, nbytes)


def _fake_step_local_rows(opt, params, slot):
    """What the step kernel does under the copy-engine transport: the other ranks' rows are
    already in the local staging matrix; average them with this rank's own row, update the
    shards, and (push) leave the new shards in this rank's own copy of the push buffer only."""
    from torch.distributed.tensor import DTensor

    from flashoptim_b200.optim.base import local_tensor

    peers = slot.group
    w, r = peers.world, peers.rank
    staging, row_bytes = slot.local_rows
    locals_ = [local_tensor(p) for p in params]
    dtype, esize = locals_[0].dtype, locals_[0].element_size()
    n_row = slot.grad_out.numel()
    assert row_bytes == n_row * esize and slot.grad_out_sub == r * row_bytes
    total = torch.zeros(n_row, dtype=torch.float32)
    for p in range(w):
        if p == r:
            total += slot.buf.view(r * row_bytes, n_row, dtype).float()
        else:
            raw = bytearray(ctypes.string_at(staging + p * row_bytes, row_bytes))
            total += torch.frombuffer(raw, dtype=dtype).float()
    mine = (total / w).to(dtype)
    slot.grad_out.copy_(mine)
    epoch = slot.epoch
    slot.next_args()
    assert slot.epoch == epoch, "the copy-engine transport advances the epochs itself"
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
        own = slot.push.buf.view(r * row_bytes + slot.push.delta, n_row, dtype)
        for pl in locals_:
            off = (slot.offsets[id(pl)] - slot.grad_out_sub) // esize
            own[off:off + pl.numel()] = pl.reshape(-1)


def _net(world):
    """Layer sizes that give every rank a 16-byte multiple per group (the copy-engine all-gather's
    condition), except the last Linear, whose 8 output rows also shard unevenly over 3 ranks."""
    from flashoptim_b200 import cast_model

    torch.manual_seed(0)
    d = 8 * world
    m = nn.Sequential(nn.Linear(d, 2 * d), nn.GELU(), nn.Linear(2 * d, d), nn.LayerNorm(d), nn.Linear(d, 8))
    cast_model(m, torch.bfloat16)
    return m


def _worker(rank, world):
    from torch.distributed.fsdp import fully_shard

    import flashoptim_b200.parallel.fsdp as fsdp_mod
    from flashoptim_b200 import FlashAdamW

    errors = []
    fsdp_mod.PeerGroup = _AddressedPeers

    def shard(m):
        for layer in m:
            if isinstance(layer, nn.Linear):
                fully_shard(layer)
        fully_shard(m)
        return m

    def step_fn(opt):
        def run(params, slot):
            if slot.local_rows is not None:
                _fake_step_local_rows(opt, params, slot)
            else:
                _fake_step_from_peers(opt, params, slot)
        return run

    g = torch.Generator().manual_seed(5)
    data = [(torch.randn(world * 4, 8 * world, generator=g), torch.randint(0, 8, (world * 4,), generator=g))
            for _ in range(4)]
    tol = get_tolerances(torch.bfloat16, True)
    configs = [
        ("copy-engine all-gather", dict(own_all_gather=True, all_gather_copy_engine=True)),
        ("copy-engine transport", dict(transport="copy_engine")),
        ("copy-engine transport + push", dict(transport="copy_engine", push_params=True)),
        ("copy-engine transport + copy-engine all-gather",
         dict(transport="copy_engine", own_all_gather=True, all_gather_copy_engine=True)),
    ]
    for tag, kwargs in configs:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            plain, fused = shard(_net(world)), shard(_net(world))
            o1 = FlashAdamW(plain.parameters(), lr=5e-4)
            o2 = FlashAdamW(fused.parameters(), lr=5e-4)
        o2.step_from_peers = step_fn(o2)
        state = fsdp_mod.enable_fused_fsdp(fused, o2, **kwargs)
        peers = state.peers
        for step, (x, y) in enumerate(data):
            xs, ys = x[rank * 4:(rank + 1) * 4].bfloat16(), y[rank * 4:(rank + 1) * 4]
            for model, opt in ((plain, o1), (fused, o2)):
                nn.functional.cross_entropy(model(xs).float(), ys).backward()
                opt.step()
                opt.zero_grad()
            for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                        f"{tag} step {step} {n1}")
        n_groups = 4
        if state.fallbacks or state.fused_calls != n_groups * len(data):
            errors.append(f"{tag}: {state.fused_calls} fused reduce-scatters, {state.fallbacks} fall-backs")
        ce_transport = kwargs.get("transport") == "copy_engine"
        if kwargs.get("all_gather_copy_engine"):
            # the last Linear's shard is not a multiple of 16 bytes per rank: NCCL-style fall-back
            if state.ag_calls == 0 or state.ag_fallbacks == 0:
                errors.append(f"{tag}: {state.ag_calls} copy-engine all-gathers, {state.ag_fallbacks} fall-backs")
        if kwargs.get("push_params"):
            if state.ag_eliminated < n_groups * (len(data) - 1):
                errors.append(f"{tag}: only {state.ag_eliminated} all-gathers were served by pushes")
            if not all(gather.is_current() for gather in state.gathers):
                errors.append(f"{tag}: a group is not marked current after its push")
        expect_copies = 0
        if ce_transport:
            expect_copies += (world - 1) * state.fused_calls * (2 if kwargs.get("push_params") else 1)
        expect_copies += (world - 1) * state.ag_calls
        if peers.copies != expect_copies:
            errors.append(f"{tag}: {peers.copies} copies, expected {expect_copies}")
        expect_barriers = (state.fused_calls if ce_transport else 0) + state.ag_calls
        if peers.barriers != expect_barriers:
            errors.append(f"{tag}: {peers.barriers} barriers, expected {expect_barriers}")
        state.remove()

    # switching the all-gather between steps (what a comparison run does): push -> copy engines
    # -> FSDP2's own -> push again; the parameters must follow the plain model throughout and
    # each mode must be the one that serves the all-gathers
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        plain, fused = shard(_net(world)), shard(_net(world))
        o1 = FlashAdamW(plain.parameters(), lr=5e-4)
        o2 = FlashAdamW(fused.parameters(), lr=5e-4)
    o2.step_from_peers = step_fn(o2)
    state = fsdp_mod.enable_fused_fsdp(fused, o2, push_params=True, own_all_gather=True, all_gather_copy_engine=True)
    if state.all_gather_mode != "push":
        errors.append(f"mode after enabling with push_params: {state.all_gather_mode}")
    for mode in ("push", "pull", "nccl", "push"):
        state.set_all_gather_mode(mode)
        if any(gather.is_current() for gather in state.gathers):
            errors.append(f"mode {mode}: a push buffer is still marked current right after the switch")
        before = (state.ag_eliminated, state.ag_calls, state.ag_fallbacks)
        for step, (x, y) in enumerate(data[:3]):
            xs, ys = x[rank * 4:(rank + 1) * 4].bfloat16(), y[rank * 4:(rank + 1) * 4]
            for model, opt in ((plain, o1), (fused, o2)):
                nn.functional.cross_entropy(model(xs).float(), ys).backward()
                opt.step()
                opt.zero_grad()
            for (n1, p1), (_, p2) in zip(plain.named_parameters(), fused.named_parameters()):
                errors += check_similar(p2.detach().full_tensor(), p1.detach().full_tensor(), tol,
                                        f"mode {mode} step {step} {n1}")
        eliminated, pulled, fell_back = (a - b for a, b in
                                         zip((state.ag_eliminated, state.ag_calls, state.ag_fallbacks), before))
        if mode == "push" and (eliminated < 4 * 2 or pulled):
            errors.append(f"mode push: {eliminated} all-gathers served by pushes, {pulled} by copies")
        if mode == "pull" and (eliminated or not pulled):
            errors.append(f"mode pull: {eliminated} all-gathers served by pushes, {pulled} by copies")
        if mode == "nccl" and (eliminated or pulled):
            errors.append(f"mode nccl: {eliminated} all-gathers served by pushes, {pulled} by copies")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        bare = shard(_net(world))
        o3 = FlashAdamW(bare.parameters(), lr=5e-4)
    bare_state = fsdp_mod.enable_fused_fsdp(bare, o3)  # neither push buffers nor an all-gather pool
    for mode in ("push", "pull"):
        try:
            bare_state.set_all_gather_mode(mode)
            errors.append(f"mode {mode} was accepted although its buffers were never allocated")
        except ValueError:
            pass
    return errors


import pytest


@pytest.mark.parametrize("world_size", [2, 3])
def test_copy_engine_paths_on_gloo(world_size):
    """Three ranks: uneven (padded) shards and a ring of more than one peer per rank."""
    run_distributed(_worker, world_size=world_size, backend="gloo")
