"""FSDP2 (``fully_shard``) with the gradient reduce-scatter fused into the sharded update.

``enable_fused_fsdp(model, optimizer)`` installs a custom reduce-scatter
communicator on every FSDP module (``FSDPModule.set_custom_reduce_scatter``).
FSDP2 lays a parameter group's unsharded gradients out as a ``[world, shard]``
matrix; that matrix is allocated inside a symmetric NVLink buffer, and when
FSDP2 asks for the reduce-scatter, rank ``r`` launches ONE kernel that reads row
``r`` of every rank, averages in fp32 and applies the optimizer update to its
shards of the group's parameters in the same pass.  The averaged shard is also
written to FSDP2's reduce-scatter output so that ``param.grad`` stays meaningful.
The kernel runs on FSDP2's reduce-scatter stream, overlapped with backward
compute, exactly where the reference's gradient-release hook would have run its
per-tensor update after NCCL finished (``flashoptim/optimizers.py:3040-3047``).

With ``push_params=True`` the same kernel also stores every freshly updated bf16/fp16
parameter unit into a per-group symmetric buffer on every rank ("all-gather on write",
NVLink peer stores or one ``multimem.st``).  That buffer is what FSDP2 is handed as its
all-gather output, so the parameter all-gathers of the following forward and backward
passes move no data: they wait for the ranks' "pushed" flags and return
(:class:`PushedAllGather`).  The price is one unsharded copy of the parameters per rank.

Where that copy is too much, ``own_all_gather=True, all_gather_copy_engine=True`` keeps FSDP2's
all-gather but performs it with ``cudaMemcpyAsync`` pulls between two one-CTA flag kernels
(:class:`PeerAllGather`): the copy engines move the bytes and no SM is taken from the GEMMs that
the all-gather overlaps, which is where NCCL's all-gather costs a training step most.
:func:`tuned_options` returns the combination that measured best for a given number of GPUs.

Parameters updated this way are skipped once by the next ``step()`` /
``step_param()``, so the usual training loop and gradient release keep working.
Groups the kernel cannot serve (non-default divide factors, a reduce dtype
different from the parameters, shards along a non-zero dimension, parameters
without gradients) fall back to NCCL for that call.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import native
from ..optim.base import FlashOptimizer, local_tensor
from .symm import ParamPush, PeerGradients, PeerGroup

try:  # torch >= 2.8
    from torch.distributed.fsdp import FSDPModule
    from torch.distributed.fsdp._fully_shard._fsdp_api import AllGather, ReduceScatter
except Exception:  # pragma: no cover
    FSDPModule = None  # type: ignore[assignment]
    ReduceScatter = object  # type: ignore[assignment,misc]
    AllGather = object  # type: ignore[assignment,misc]


class _Pool:
    """Round-robin pool of symmetric reduce-scatter input buffers shared by all groups."""

    def __init__(self, peers: PeerGroup, nbytes: int, depth: int):
        self.slots = []
        for i in range(depth):
            buf = peers.allocate(nbytes)
            ready, done = peers.new_channels()
            self.slots.append(PeerGradients(peers, buf, ready, done, grad_scale=1.0 / peers.world, key=i))
        self._next = 0

    def take(self) -> PeerGradients:
        s = self.slots[self._next]
        self._next = (self._next + 1) % len(self.slots)
        return s


def _every_rank_has_rows(sharded_param: torch.Tensor, world: int) -> bool:
    """FSDP2 gives rank r rows [r * c, (r + 1) * c) of dimension 0 with c = ceil(rows / world);
    a rank whose range is empty would launch fewer kernels for the group than its peers, and
    the launches of all ranks pair up through their epochs."""
    rows = sharded_param.shape[0] if sharded_param.dim() > 0 else 1  # DTensor: the global shape
    chunk = -(-rows // world)
    return (world - 1) * chunk < rows


class FusedReduceScatter(ReduceScatter):  # type: ignore[misc,valid-type]
    def __init__(self, ctx: "FusedFSDPState", fsdp_params: list, param_group=None) -> None:
        self.ctx = ctx
        self.fsdp_params = fsdp_params
        self.param_group = param_group  # FSDP2's group object (for settings that can change later)
        self._slot: Optional[PeerGradients] = None
        self.gather: Optional["PushedAllGather"] = None  # receives the updated parameters
        # the group that backward reduces last has no GEMM left to share the GPU with:
        # its kernel ignores the grid cap
        self.full_grid = False
        w = ctx.peers.world
        self.row_numels = [fp.padded_sharded_param_size.numel() for fp in fsdp_params]
        self.input_numel = w * sum(self.row_numels)
        self.dtype = fsdp_params[0].sharded_param.dtype
        owned = {id(p) for g in ctx.optimizer.param_groups for p in g["params"]}
        self.supported = all(
            fp.sharded_param.dtype == self.dtype and getattr(fp.fsdp_placement, "dim", 0) == 0
            and not fp.offload_to_cpu and id(fp.sharded_param) in owned and fp.sharded_param.requires_grad
            and _every_rank_has_rows(fp.sharded_param, w)
            for fp in fsdp_params
        )

    # FSDP2 calls allocate() for the reduce-scatter input (on the compute stream, right
    # before it packs the gradients) and then for the output (on the reduce-scatter stream).
    def allocate(self, size, *, dtype, device):
        numel = int(size[0])
        esize = torch.empty((), dtype=dtype).element_size()
        # a user's all-reduce hook post-processes the reduce-scatter output: the update must wait for it
        hooked = getattr(self.param_group, "_all_reduce_hook", None) is not None
        if (self.ctx.enabled and self.supported and not hooked and numel == self.input_numel
                and dtype == self.dtype and numel * esize <= self.ctx.pool_bytes):
            slot = self.ctx.pool.take()
            slot.wait_done()  # every rank is done reading this buffer's previous contents
            self._slot = slot
            return slot.buf.view(0, numel, dtype)
        return torch.empty(*size, dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, op, async_op=False):
        slot, self._slot = self._slot, None
        fused = (
            slot is not None
            and input_tensor.data_ptr() == slot.buf.tensor.data_ptr()
            and op == dist.ReduceOp.AVG
            and not async_op
        )
        if not fused:
            self.ctx.fallbacks += 1
            if self.gather is not None:
                self.gather.invalidate()  # the parameters will change without a push
            return dist.reduce_scatter_tensor(output=output_tensor, input=input_tensor, group=group, op=op,
                                              async_op=async_op)
        peers = self.ctx.peers
        esize = input_tensor.element_size()
        row_bytes = sum(self.row_numels) * esize
        base = peers.rank * row_bytes
        offsets, off = {}, 0
        for fp, n in zip(self.fsdp_params, self.row_numels):
            offsets[id(local_tensor(fp.sharded_param))] = base + off
            off += n * esize
        slot.offsets = offsets
        slot.grad_out, slot.grad_out_sub = output_tensor, base
        # the all-gather output of this group has the reduce-scatter input's layout (rank r's
        # padded shards at r * row_bytes), so a parameter lands at its gradient's offset
        slot.push = self.gather.target if (self.gather is not None and esize == self.gather.esize
                                           and self.ctx.push_enabled) else None
        slot.max_ctas = 0 if self.full_grid else None
        copy_engine = self.ctx.transport == "copy_engine"
        try:
            if copy_engine:
                self._pull_rows(slot, row_bytes)
            self.ctx.optimizer.step_from_peers([fp.sharded_param for fp in self.fsdp_params], slot)
            if copy_engine:
                self._finish_copy_engine(slot, row_bytes)
        finally:
            pushed, slot.push, slot.max_ctas, slot.local_rows = slot.push is not None, None, None, None
        if self.gather is not None:
            if pushed:
                self.gather.mark_pushed()
            else:
                self.gather.invalidate()
        self.ctx.fused_calls += 1
        return None

    # ---- copy-engine transport: the bytes cross NVLink in cudaMemcpyAsync copies (no SM), the
    # update kernel reads local memory only and runs at HBM speed
    def _pull_rows(self, slot: PeerGradients, row_bytes: int) -> None:
        """Barrier, then copy row ``rank`` of every other rank's gradient matrix into the local
        staging matrix; the step kernels are pointed at it."""
        peers = self.ctx.peers
        w, r = peers.world, peers.rank
        slot.epoch += 1
        args = peers.comm_args(slot.buf, slot.epoch, slot.ready_channel, slot.done_channel)
        peers.barrier(args)
        staging = self.ctx.staging.data_ptr()
        for i in range(1, w):
            p = (r + i) % w  # every rank starts with a different peer: no link is asked twice at once
            peers.copy(staging + p * row_bytes, slot.buf.ptrs[p] + r * row_bytes, row_bytes)
        slot.local_rows = (staging, row_bytes)
        if slot.push is not None:
            slot.push.epoch += 1

    def _finish_copy_engine(self, slot: PeerGradients, row_bytes: int) -> None:
        """After the update: tell the ranks that their gradient buffers are free again, copy
        this rank's fresh parameter row into every other rank's all-gather buffer and publish it."""
        peers = self.ctx.peers
        w, r = peers.world, peers.rank
        args = peers.comm_args(slot.buf, slot.epoch, slot.ready_channel, slot.done_channel)
        peers.signal(args, slot.done_channel)
        t = slot.push
        if t is not None:
            mine = t.buf.ptrs[r] + r * row_bytes + t.delta
            for i in range(1, w):
                p = (r + i) % w
                peers.copy(t.buf.ptrs[p] + r * row_bytes + t.delta, mine, row_bytes)
            peers.signal(peers.comm_args(t.buf, t.epoch, t.channel, t.channel), t.channel)


class PeerAllGather(AllGather):  # type: ignore[misc,valid-type]
    """FSDP2's parameter all-gather done by this library's pull kernel.

    FSDP2 allocates the ``[world, shard]`` all-gather output through :meth:`allocate`
    (here: a symmetric buffer from a small pool), copies its own shards into slot
    ``rank`` and calls the communicator; every rank then pulls slot ``s`` from rank
    ``s`` over NVLink with plain 16-byte peer loads (``fo_allgather_peer``) or, with
    ``ctx.ag_copy_engine``, with one ``cudaMemcpyAsync`` per peer between two one-CTA flag
    kernels: the copy engines then move the bytes and no SM is taken from the GEMMs that the
    all-gather overlaps.  Calls whose slot size is not a multiple of 16 bytes, or that are
    larger than the pool's buffers, use NCCL.
    """

    def __init__(self, ctx: "FusedFSDPState") -> None:
        self.ctx = ctx
        self._slot: Optional[PeerGradients] = None

    def allocate(self, size, *, dtype, device):
        numel = int(size[0])
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        w = self.ctx.peers.world
        if nbytes <= self.ctx.ag_pool_bytes and (nbytes // w) % 16 == 0 and nbytes % w == 0:
            slot = self.ctx.ag_pool.take()
            slot.wait_done()  # peers have pulled my slot's previous contents
            self._slot = slot
            return slot.buf.view(0, numel, dtype)
        self._slot = None
        return torch.empty(*size, dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, async_op=False):
        slot, self._slot = self._slot, None
        if slot is None or output_tensor.data_ptr() != slot.buf.tensor.data_ptr() or async_op:
            self.ctx.ag_fallbacks += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)
        slot_bytes = input_tensor.numel() * input_tensor.element_size()
        peers = self.ctx.peers
        if self.ctx.ag_copy_engine:
            w, r = peers.world, peers.rank
            slot.epoch += 1
            args = peers.comm_args(slot.buf, slot.epoch, slot.ready_channel, slot.done_channel)
            peers.barrier(args)  # every rank's shards are in its own slot
            for i in range(1, w):
                s = (r + i) % w  # every rank starts with a different peer
                peers.copy(slot.buf.ptrs[r] + s * slot_bytes, slot.buf.ptrs[s] + s * slot_bytes, slot_bytes)
            peers.signal(args, slot.done_channel)  # my reads of the peers' slots are complete
        else:
            args = slot.next_args()
            rc = native.load().fo_allgather_peer(slot_bytes, ctypes.byref(args), native.stream_ptr(peers.device))
            native.check(rc, "fo_allgather_peer")
        self.ctx.ag_calls += 1
        return None


class PushedAllGather(AllGather):  # type: ignore[misc,valid-type]
    """FSDP2's parameter all-gather of one group, served by the step kernel's pushes.

    The group's all-gather output lives in one persistent symmetric buffer.  While it is
    *current* (the last change of the group's sharded parameters was a fused update that
    pushed them, on every rank) an all-gather only enqueues a bounded wait for the ranks'
    "pushed" flags; otherwise (first use, after a checkpoint load, after an update that did
    not go through the fused kernel) it is an NCCL all-gather into the same buffer.  The
    sharded tensors' version counters reveal in-place changes made by anything else.
    Every rank must reach the same verdict, which holds when all ranks run the same program.
    """

    def __init__(self, ctx: "FusedFSDPState", rs: FusedReduceScatter) -> None:
        self.ctx = ctx
        self.rs = rs
        self.esize = torch.empty((), dtype=rs.dtype).element_size()
        self.numel = rs.input_numel
        self.supported = rs.supported
        self.target: Optional[ParamPush] = None
        if self.supported:
            buf = ctx.peers.allocate(self.numel * self.esize)
            self.target = ParamPush(buf, ctx.peers.new_channel())
        self._current = False
        self._versions: list[int] = []

    def _param_versions(self) -> list[int]:
        return [local_tensor(fp.sharded_param)._version for fp in self.rs.fsdp_params]

    def mark_pushed(self) -> None:
        self._current = True
        self._versions = self._param_versions()

    def invalidate(self) -> None:
        self._current = False

    def is_current(self) -> bool:
        return self._current and self._versions == self._param_versions()

    def allocate(self, size, *, dtype, device):
        if self.target is not None and int(size[0]) == self.numel and dtype == self.rs.dtype:
            return self.target.buf.view(0, self.numel, dtype)
        return torch.empty(*size, dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, async_op=False):
        t = self.target
        mine = t is not None and output_tensor.data_ptr() == t.buf.tensor.data_ptr() and not async_op
        if mine and self.is_current():
            peers = self.ctx.peers
            args = peers.comm_args(t.buf, t.epoch, t.channel, t.channel)
            peers.wait(args, t.channel)
            self.ctx.ag_eliminated += 1
            return None
        self.ctx.ag_fallbacks += 1
        return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)


def oversized_mask(sizes: list[int]) -> list[bool]:
    """Which groups are more than twice the size of the typical (median) group: a model's
    embedding + output head beside its transformer layers."""
    typical = sorted(sizes)[len(sizes) // 2]
    return [n > 2 * typical for n in sizes]


def select_push_groups(sizes: list[int], budget_bytes: Optional[int]) -> list[bool]:
    """Which groups get a persistent all-gather buffer: all supported ones (size > 0) without
    a budget, else in module order as long as their buffers fit into ``budget_bytes`` (the
    buffers together hold an unsharded copy of those groups' parameters on every rank)."""
    out, used = [], 0
    for n in sizes:
        take = n > 0 and (budget_bytes is None or used + n <= budget_bytes)
        if take:
            used += n
        out.append(take)
    return out


class UnsupportedFSDPInternals(RuntimeError):
    """The installed PyTorch does not have the FSDP2 internals this module reads."""


# FSDP2 attributes outside its public API that the fused path depends on.  They are checked
# once, by name, before anything is installed; a PyTorch release that renames one makes
# enable_fused_fsdp() warn and leave the model on FSDP2's own (NCCL) collectives.
_PARAM_GROUP_ATTRS = ("fsdp_params", "device", "_reduce_scatter_process_group", "_all_reduce_hook", "_is_hsdp")
_FSDP_PARAM_ATTRS = ("sharded_param", "padded_sharded_param_size", "fsdp_placement", "offload_to_cpu")


def _fsdp_param_groups(model: nn.Module) -> list:
    """``(module, FSDPParamGroup)`` of every fully_shard-ed module that owns parameters."""
    if FSDPModule is None:
        raise UnsupportedFSDPInternals("torch.distributed.fsdp.FSDPModule with custom collectives needs torch >= 2.8")
    modules = [m for m in model.modules() if isinstance(m, FSDPModule)]
    if not modules:
        raise ValueError("model has no fully_shard-ed modules")
    for name in ("set_custom_reduce_scatter", "set_custom_all_gather", "_get_fsdp_state"):
        if not hasattr(modules[0], name):
            raise UnsupportedFSDPInternals(f"FSDPModule.{name} is missing in torch {torch.__version__}")
    groups = []
    for m in modules:
        state = m._get_fsdp_state()
        if not hasattr(state, "_fsdp_param_group"):
            raise UnsupportedFSDPInternals(f"FSDPState._fsdp_param_group is missing in torch {torch.__version__}")
        pg = state._fsdp_param_group
        if pg is None or not getattr(pg, "fsdp_params", None):
            continue
        missing = [a for a in _PARAM_GROUP_ATTRS if not hasattr(pg, a)]
        missing += [a for a in _FSDP_PARAM_ATTRS if not hasattr(pg.fsdp_params[0], a)]
        if missing:
            raise UnsupportedFSDPInternals(
                f"FSDP2 internals {missing} are missing in torch {torch.__version__}")
        groups.append((m, pg))
    return groups


class FusedFSDPState:
    def __init__(self, model: nn.Module, optimizer: FlashOptimizer, group, timeout_s, use_multicast, depth,
                 max_ctas=0, own_all_gather=False, push_params=False, push_budget_bytes=None,
                 last_group_full_grid=True, staged=False, push_multicast=None, transport="kernel",
                 all_gather_copy_engine=False, oversized_groups="nccl"):
        if oversized_groups not in ("nccl", "fused"):
            raise ValueError(f"oversized_groups must be 'nccl' or 'fused', got {oversized_groups!r}")
        self.optimizer = optimizer
        self.ag_copy_engine = bool(all_gather_copy_engine)  # own_all_gather: copy engines, not the pull kernel
        if transport not in ("kernel", "copy_engine"):
            raise ValueError(f"transport must be 'kernel' or 'copy_engine', got {transport!r}")
        self.transport = transport  # may be switched between steps (for comparisons)
        self.enabled = True        # False: every reduce-scatter goes to NCCL (for comparisons)
        self.push_enabled = True   # False: updates stop pushing, all-gathers go back to NCCL
        groups = _fsdp_param_groups(model)
        if not groups:
            raise ValueError("no FSDP parameter groups found")
        if any(pg._is_hsdp for _, pg in groups):
            # FSDP2 all-reduces the reduce-scatter output across replicas afterwards; an update
            # inside the reduce-scatter would use a gradient that is averaged over one replica only
            raise ValueError("the fused FSDP2 path does not support HSDP (replicate x shard) meshes; "
                             "use fully_shard with optimizer.step() there")
        mesh_group = groups[0][1]._reduce_scatter_process_group
        self.peers = PeerGroup(group or mesh_group, device=groups[0][1].device, timeout_s=timeout_s,
                               use_multicast=use_multicast, max_ctas=max_ctas, push_multicast=push_multicast,
                               variant=1 if staged else 0)
        self.fused_calls = 0
        self.fallbacks = 0
        self.comms = []
        sizes = []
        for m, pg in groups:
            comm = FusedReduceScatter(self, list(pg.fsdp_params), pg)
            sizes.append(comm.input_numel * torch.empty((), dtype=comm.dtype).element_size())
            self.comms.append((m, comm))
        # The symmetric buffers are pools sized by the largest group they serve.  A group much
        # larger than the typical one (a model's embedding + output head beside its layers)
        # would multiply every pool buffer: with oversized_groups="nccl" such a group keeps
        # FSDP2's own collectives (it is reduced last and gathered first, where nothing overlaps
        # anyway) and the pools stay at the size of a layer.
        self.oversized = oversized_mask(sizes) if oversized_groups == "nccl" else [False] * len(sizes)
        for (m, comm), big in zip(self.comms, self.oversized):
            if big:
                comm.supported = False
        need = max([n for n, big in zip(sizes, self.oversized) if not big] or [0])
        # modules() lists the outermost module first; its group holds what the model applies
        # first and is therefore the one whose gradients backward completes last
        if last_group_full_grid and len(self.comms) > 1 and not self.oversized[0]:
            self.comms[0][1].full_grid = True
        self.pool_bytes = need
        self.pool = _Pool(self.peers, need, depth)
        self._staging: Optional[torch.Tensor] = None
        self.ag_calls = 0
        self.ag_fallbacks = 0
        self.ag_eliminated = 0
        self.gathers: list[PushedAllGather] = []
        # every symmetric allocation comes first and the communicators are installed last, so
        # that a failed allocation leaves the model on FSDP2's own collectives
        self._push_installs: list[tuple[nn.Module, object]] = []
        self._pull_installs: list[tuple[nn.Module, object]] = []
        self._listener = None
        if push_params:
            by_param = {}
            chosen = select_push_groups(
                [comm.input_numel * torch.empty((), dtype=comm.dtype).element_size() if comm.supported else 0
                 for _, comm in self.comms], push_budget_bytes)
            for (m, comm), take in zip(self.comms, chosen):
                if not take:
                    continue  # this group keeps FSDP2's own all-gather
                gather = PushedAllGather(self, comm)
                comm.gather = gather
                self.gathers.append(gather)
                self._push_installs.append((m, gather))
                for fp in comm.fsdp_params:
                    by_param[id(fp.sharded_param)] = gather

            def on_local_update(params, _by_param=by_param):
                for p in params:
                    g = _by_param.get(id(p))
                    if g is not None:
                        g.invalidate()

            optimizer._local_update_listeners.append(on_local_update)
            self._listener = on_local_update
        if own_all_gather:
            # the all-gather output of a group is as large as its reduce-scatter input;
            # three buffers: one being copied out, one prefetched, one spare
            self.ag_pool_bytes = need
            self.ag_pool = _Pool(self.peers, need, 3)
            self._pull_installs = [(m, PeerAllGather(self)) for (m, _), big in zip(groups, self.oversized) if not big]
        for m, comm in self.comms:
            m.set_custom_reduce_scatter(comm)
        self._installs: list[tuple[nn.Module, object]] = []
        self.all_gather_mode = "nccl"
        self.set_all_gather_mode("push" if push_params else ("pull" if own_all_gather else "nccl"))

    def set_all_gather_mode(self, mode: str) -> None:
        """Which parameter all-gather FSDP2 uses from now on (collective: every rank, between
        steps): ``"push"`` (all-gather on write; groups without a push buffer use this library's
        all-gather where that was set up, else NCCL),
        ``"pull"`` (this library's all-gather: pull kernel or copy engines) or ``"nccl"``.
        Only modes whose buffers were allocated at construction are available."""
        from torch.distributed.fsdp._fully_shard._fsdp_collectives import DefaultAllGather

        if mode not in ("push", "pull", "nccl"):
            raise ValueError(f"unknown all-gather mode {mode!r}")
        if (mode == "push" and not self._push_installs) or (mode == "pull" and not self._pull_installs):
            raise ValueError(f"all-gather mode {mode!r} was not set up when the fused path was enabled")
        for m, _ in self._installs:
            m.set_custom_all_gather(DefaultAllGather())
        installs = {"push": list(self._push_installs), "pull": list(self._pull_installs), "nccl": []}[mode]
        if mode == "push":
            # groups that got no push buffer (memory budget): this library's all-gather if it was
            # set up, else FSDP2's
            pushed = {id(m) for m, _ in installs}
            installs += [(m, g) for m, g in self._pull_installs if id(m) not in pushed]
        self._installs = installs
        for m, gather in self._installs:
            m.set_custom_all_gather(gather)
        for g in self.gathers:
            g.invalidate()  # whatever the buffers hold now was not necessarily put there by a push
        self.push_enabled = mode == "push"
        self.all_gather_mode = mode

    @property
    def staging(self) -> torch.Tensor:
        """Copy-engine transport: the local ``[world, row]`` matrix that the peers' gradient rows
        are copied into (allocated on first use; one buffer serves every group because copies
        and kernels of consecutive groups are ordered on the reduce-scatter stream)."""
        if self._staging is None:
            self._staging = torch.empty(self.pool_bytes, dtype=torch.uint8, device=self.peers.device)
        return self._staging

    def remove(self) -> None:
        """Hand the model back to FSDP2's own collectives (collective: call on every rank,
        between steps).  The symmetric buffers live until this object is dropped."""
        from torch.distributed.fsdp._fully_shard._fsdp_collectives import DefaultAllGather, DefaultReduceScatter

        for m, _ in self.comms:
            m.set_custom_reduce_scatter(DefaultReduceScatter())
        for m, _ in self._installs:
            m.set_custom_all_gather(DefaultAllGather())
        self._installs = []
        if self._listener is not None and self._listener in self.optimizer._local_update_listeners:
            self.optimizer._local_update_listeners.remove(self._listener)
        self._listener = None

    def check(self) -> None:
        """Synchronise and raise if a device-side wait for another rank timed out."""
        self.peers.check_status()

    def poll(self) -> None:
        """Non-blocking form of :meth:`check` (reports a timeout one or two calls late)."""
        self.peers.poll_status()


def tuned_options(world_size: int, unsharded_param_bytes: int = 0, push_budget_bytes: int = 0) -> dict:
    """Keyword arguments for :func:`enable_fused_fsdp` that measured best for Llama-3-8B / 70B
    training steps on 2, 4 and 8 B200s of one NVSwitch node (every path timed in one process with
    ``bench.py --sweep``).

    * Two ranks: the kernel is bound by its own arithmetic and HBM traffic, not by the link; the
      bulk-copy staged kernel on the whole GPU finishes soonest, parameters are pushed with one
      store per rank.
    * More ranks: NVLink-bound.  ``multimem.ld_reduce`` lets the switch add the ranks' copies,
      four units per thread are in flight, and 64 (3-4 ranks) or 48 (5-8 ranks) CTAs keep the
      links busy while the other SMs stay with backward's GEMMs; ``multimem.st`` for pushes.
    * Parameter all-gather: by the copy engines (``own_all_gather`` + ``all_gather_copy_engine``:
      no SM, three group-sized buffers, so peak memory stays where FSDP2's own is).  The
      all-gather on write (``push_params``) is 1-2 % faster still but keeps an unsharded copy
      of the parameters on every GPU (16 GB for 8 B parameters); it is proposed only when that
      copy, ``unsharded_param_bytes``, fits the ``push_budget_bytes`` the caller grants."""
    if world_size <= 2:
        opts = dict(use_multicast=False, staged=True, max_ctas=0, push_multicast=False)
    else:
        opts = dict(use_multicast=True, staged=False, max_ctas=64 if world_size <= 4 else 48, push_multicast=True)
    if 0 < unsharded_param_bytes <= push_budget_bytes:
        opts["push_params"] = True
    else:
        opts.update(own_all_gather=True, all_gather_copy_engine=True)
    return opts


def enable_fused_fsdp(
    model: nn.Module,
    optimizer: FlashOptimizer,
    *,
    group: Optional[dist.ProcessGroup] = None,
    timeout_s: float = 5.0,
    use_multicast: bool = False,
    depth: int = 2,
    max_ctas: int = 0,
    own_all_gather: bool = False,
    push_params: bool = False,
    push_budget_bytes: Optional[int] = None,
    last_group_full_grid: bool = True,
    staged: bool = False,
    push_multicast: Optional[bool] = None,
    transport: str = "kernel",
    all_gather_copy_engine: bool = False,
    oversized_groups: str = "nccl",
) -> Optional[FusedFSDPState]:
    """Fuse FSDP2's gradient reduce-scatter with ``optimizer``'s sharded update.

    Collective: call on every rank after ``fully_shard`` and after constructing the
    optimizer.  Returns the state object (``.fused_calls`` / ``.fallbacks`` count what
    happened; ``.check()`` raises if a device-side wait timed out), or ``None`` when the
    data-parallel group has a single rank (FSDP2 then performs no reduce-scatter).
    Like gradient release, this updates parameters during backward, so it excludes loss
    scaling with ``torch.amp.GradScaler`` and global gradient clipping (both need all
    gradients before any update).
    Every reduce-scatter then IS the optimizer update of that backward pass: accumulate
    gradients with ``model.set_requires_gradient_sync(False)`` on all but the last
    micro-batch (a second synchronised backward before ``step()`` raises).
    ``depth`` symmetric buffers of the largest group's gradient size are kept.
    ``max_ctas`` caps the kernel's grid: the reduce-scatter is NVLink-bound, so a few
    dozen CTAs keep the links busy while the SMs stay with backward's GEMMs.  With
    ``last_group_full_grid`` the outermost module's group, which backward reduces last with no
    GEMM left to overlap, ignores the cap.
    ``use_multicast`` fetches each unit with one ``multimem.ld_reduce`` (the NVSwitch
    adds the ranks' copies and returns the sum narrowed to the gradient dtype, 1/world
    of the inbound traffic of peer loads) instead of ``world`` peer loads summed in fp32.
    ``staged`` (peer loads only) runs the bulk-copy staged kernels: a producer thread per CTA
    streams the ranks' gradient chunks through shared memory with ``cp.async.bulk``, so two or
    three dozen CTAs (``max_ctas``) saturate NVLink.  ``push_multicast`` chooses ``multimem.st``
    for the parameter push independently of how gradients are fetched (default: as
    ``use_multicast``).
    ``transport="copy_engine"`` moves the bytes differently: after a one-CTA barrier the other
    ranks' gradient rows are fetched with ``cudaMemcpyAsync`` (the copy engines drive NVLink, no
    SM takes part), the update kernel then reads only local memory at HBM speed, and the fresh
    parameters go to the peers' all-gather buffers in further copy-engine copies.  It costs one
    more pass of the gradients through HBM and one local ``[world, shard]`` staging buffer, and
    leaves every SM to backward's GEMMs while the links are busy.
    ``oversized_groups="nccl"`` (default) leaves a parameter group that is more than twice the
    size of the typical one (an embedding + output head beside transformer layers) to FSDP2's own
    collectives, so that the pooled symmetric buffers have the size of a layer; ``"fused"`` serves
    it too and sizes every pool buffer for it.
    ``own_all_gather`` also replaces FSDP2's parameter all-gather by this library's own over
    symmetric buffers (:class:`PeerAllGather`): a pull kernel, or with ``all_gather_copy_engine``
    one ``cudaMemcpyAsync`` per peer, which takes no SM from the GEMMs it overlaps and costs
    three group-sized buffers instead of an unsharded copy of the model.
    ``push_params`` instead removes that all-gather: the update kernel stores the new
    parameters into every rank's all-gather buffer (:class:`PushedAllGather`); costs one
    unsharded copy of the parameters per rank (``.ag_eliminated`` counts the all-gathers
    that moved no data).  ``push_budget_bytes`` bounds that copy: groups get a buffer in
    module order while they fit, the others keep FSDP2's all-gather (Llama-3-70B's 140 GB
    of bf16 parameters do not fit beside the training state of a 180 GB GPU).
    """
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return None
    state, error = None, None
    try:
        state = FusedFSDPState(model, optimizer, group, timeout_s, use_multicast, depth, max_ctas, own_all_gather,
                               push_params, push_budget_bytes, last_group_full_grid, staged, push_multicast, transport,
                               all_gather_copy_engine, oversized_groups)
    except UnsupportedFSDPInternals as e:
        # same PyTorch on every rank, so every rank lands here together, before any collective
        import warnings

        warnings.warn(f"fused FSDP2 collectives are not available ({e}); the model stays on FSDP2's own "
                      "NCCL collectives and optimizer.step()", stacklevel=2)
        return None
    except (ValueError, TypeError):
        raise  # wrong use, raised before any collective and identically on every rank
    except Exception as e:  # e.g. an allocation that failed on this rank only
        error = e
    # all ranks or none: a rank that stayed on NCCL would never answer the others' kernels
    device = next(model.parameters()).device
    ok = torch.tensor([0 if state is None else 1], dtype=torch.int32, device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        if state is not None:
            state.remove()
        raise RuntimeError("the fused FSDP2 path could not be set up on every rank") from error
    return state
