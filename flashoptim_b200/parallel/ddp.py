"""DistributedDataParallel with the bucket all-reduce fused into the optimizer update.

``fuse_ddp_allreduce(ddp_model, optimizer)`` registers a DDP communication hook.
When a gradient bucket is ready the hook copies it into this rank's slice of a
symmetric NVLink arena and, on a side stream, launches one kernel that reads
the matching slice of every rank, averages in fp32 in rank order (all replicas
therefore compute bit-identical values) and applies the optimizer update to the
bucket's parameters and replicated states in the same pass (one-shot).  NCCL is
not involved; the averaged gradient never exists in HBM unless
``write_back=True``.  With more than two ranks large buckets go two-shot: a
reduce + broadcast kernel assembles the averaged bucket in every rank's arena
(each slice is computed once, so replicas still agree bit for bit) and a local
multi-tensor step consumes it.

The reference cannot step inside a DDP hook at all (it rejects gradient release
for DDP, ``flashoptim/optimizers.py:3111-3123``): PyTorch's reducer owns the
bucket and an update there serialises its pipeline.  Here the update runs on
its own stream from a private copy of the bucket, and ``optimizer.step()``
afterwards only skips the parameters that were already updated and joins the
side stream.  Plain DDP (no hook) with ``optimizer.step()`` keeps working.

Gradient accumulation with ``no_sync()`` is transparent: DDP does not call the
hook on unsynchronised backwards and the bucket later holds the accumulated sum.

What it buys, measured (GPT-2 medium, 8 sequences of 1024 per GPU, B200): the fused hook is a
correctness-complete alternative, NOT a speed-up.  It ran within 1 % of NCCL all-reduce followed
by this library's multi-tensor step (50.0 vs 49.3 ms per step on 2 GPUs, 50.4 vs 49.4 on 4,
50.7 vs 50.2 on 8) and 5 % ahead of the reference optimizer on stock DDP (52.8 ms on 4 GPUs).  DDP's reducer owns its buckets, so every
bucket is first copied into the symmetric arena (one more pass of all gradients through HBM),
and a replicated update is HBM-bound on every rank whatever the collective does.  The fused
FSDP2 path (``enable_fused_fsdp``), where each rank updates only its shard, is where fusing
pays.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel as DDP

from ..ops import native
from ..optim.base import FlashOptimizer
from .symm import PeerGradients, PeerGroup


class ArenaLayout:
    """Where each gradient bucket of a backward pass goes in the symmetric arena, and what the
    host has to wait for before the pass overwrites anything.

    Buckets are laid out one after the other in the order DDP hands them over.  DDP rebuilds
    its buckets after the first iteration, so a region of this pass may overlap several regions
    of the previous one at other offsets.  The protection therefore does not look at offsets:
    before the FIRST bucket of a pass is copied in, the stream waits until every rank has
    published "done" for the LAST kernel of the previous pass.  Epochs grow by one per kernel
    and a rank's kernels run in order on its side stream, so that one wait covers every region
    under any layout (and the second half of the arena, which only those kernels' peers write).
    """

    def __init__(self, half_bytes: int):
        self.half = half_bytes
        self.cursor = 0

    def place(self, bucket_index: int, nbytes: int, last_epoch: int) -> tuple[int, int]:
        """Returns ``(offset, epoch)``: the bucket's byte offset, and the epoch whose "done" flags
        must be awaited first (0: nothing to wait for)."""
        wait_epoch = 0
        if bucket_index == 0:
            self.cursor = 0
            wait_epoch = last_epoch
        off = self.cursor
        self.cursor += (nbytes + 255) // 256 * 256
        if self.cursor > self.half:
            raise RuntimeError("gradient buckets exceed the symmetric arena")
        return off, wait_epoch


class FusedDDPState:
    def __init__(
        self,
        ddp_model: DDP,
        optimizer: FlashOptimizer,
        group: Optional[dist.ProcessGroup] = None,
        timeout_s: float = 5.0,
        use_multicast: bool = False,
        write_back: bool = False,
        max_ctas: int = 0,
        two_shot_min_bytes: int = 1 << 20,
        two_shot: Optional[bool] = None,
    ):
        params = [p for p in ddp_model.parameters() if p.requires_grad]
        if not params:
            raise ValueError("model has no trainable parameters")
        if any(not p.is_cuda for p in params):
            raise ValueError("the fused DDP path needs CUDA parameters")
        self.optimizer = optimizer
        self.write_back = write_back
        self.peers = PeerGroup(group, device=params[0].device, timeout_s=timeout_s, use_multicast=use_multicast,
                               max_ctas=max_ctas)
        # every bucket gets a 256-byte aligned slice; one slice per parameter is the worst case
        total = sum(p.numel() * p.element_size() for p in params) + 256 * (len(params) + 1)
        # one-shot buckets use the first half (raw gradients); two-shot buckets also use the
        # same offset in the second half, where the averaged gradients are assembled
        self.half = (total + 255) // 256 * 256
        self.two_shot = (self.peers.world > 2) if two_shot is None else bool(two_shot)
        self.two_shot_min_bytes = two_shot_min_bytes
        self.arena = self.peers.allocate(self.half * (2 if self.two_shot else 1))
        ready, done = self.peers.new_channels()
        self.grads = PeerGradients(self.peers, self.arena, ready, done, grad_scale=1.0 / self.peers.world, key=id(self))
        self.side = torch.cuda.Stream(device=params[0].device)
        self.layout = ArenaLayout(self.half)
        self.buckets_fused = 0
        self.buckets_two_shot = 0
        optimizer._post_step_callbacks.append(self._join)

    def _join(self) -> None:
        torch.cuda.current_stream().wait_stream(self.side)

    def hook(self, _state, bucket):  # no annotations: DDP compares them to the classes themselves
        buf = bucket.buffer()
        nbytes = buf.numel() * buf.element_size()
        off, wait_epoch = self.layout.place(bucket.index(), nbytes, self.grads.epoch)
        cur = torch.cuda.current_stream()
        # peers must have finished reading what the arena held in the previous pass
        if wait_epoch and self.peers.world > 1:
            args = self.peers.comm_args(self.arena, wait_epoch, self.grads.ready_channel, self.grads.done_channel)
            self.peers.wait(args, self.grads.done_channel)
        self.arena.view(off, buf.numel(), buf.dtype).copy_(buf)
        self.side.wait_event(cur.record_event())
        params = bucket.parameters()
        base = buf.data_ptr()
        self.grads.offsets = {id(p): off + (g.data_ptr() - base) for p, g in zip(params, bucket.gradients())}
        if self.two_shot and nbytes >= self.two_shot_min_bytes:
            # two-shot: each rank averages 1/world of the bucket and stores it into every
            # rank's second half; after all "done" flags the whole averaged bucket is local
            # and one local multi-tensor step consumes it.  Per GPU this moves 2(W-1)/W of the
            # bucket over NVLink instead of W-1 times the bucket.
            with torch.cuda.stream(self.side):
                args = self.grads.next_args()
                rc = native.load().fo_reduce_bcast_peer(
                    buf.numel(), off, self.half + off, native.DTYPE_CODE[buf.dtype], 1.0 / self.peers.world,
                    ctypes.byref(args), native.stream_ptr(self.peers.device))
                native.check(rc, "fo_reduce_bcast_peer")
                self.peers.wait(args, self.grads.done_channel)
                reduced = self.arena.view(self.half + off, buf.numel(), buf.dtype)
                views = [reduced[(g.data_ptr() - base) // buf.element_size():][:g.numel()]
                         for g in bucket.gradients()]
                self.optimizer.step_with_grads(list(params), views)
            self.buckets_fused += 1
            self.buckets_two_shot += 1
            fut2: torch.futures.Future = torch.futures.Future()
            fut2.set_result(buf)
            return fut2
        if self.write_back:
            self.grads.grad_out, self.grads.grad_out_sub = buf, off
        with torch.cuda.stream(self.side):
            self.optimizer.step_from_peers(list(params), self.grads)
        self.buckets_fused += 1
        fut: torch.futures.Future = torch.futures.Future()
        fut.set_result(buf)
        return fut

    def check(self) -> None:
        """Synchronise and raise if a device-side wait for another rank timed out."""
        self.peers.check_status()

    def poll(self) -> None:
        """Non-blocking form of :meth:`check` (reports a timeout one or two calls late)."""
        self.peers.poll_status()


def fuse_ddp_allreduce(
    ddp_model: DDP,
    optimizer: FlashOptimizer,
    *,
    group: Optional[dist.ProcessGroup] = None,
    timeout_s: float = 5.0,
    use_multicast: bool = False,
    write_back: bool = False,
    max_ctas: int = 0,
    two_shot_min_bytes: int = 1 << 20,
    two_shot: Optional[bool] = None,
) -> FusedDDPState:
    """Fuse DDP's per-bucket gradient all-reduce with ``optimizer``'s update.

    Measured on 2 and 8 B200s this is about 1 % slower than leaving the all-reduce to NCCL and
    calling ``optimizer.step()`` (see the module docstring): use it for its properties
    (bit-identical replicas by construction, no NCCL in the gradient path), not for speed.

    Collective: call on every rank, after constructing ``ddp_model`` (with
    ``gradient_as_bucket_view=True``) and ``optimizer``.  Keep calling
    ``optimizer.step()`` / ``zero_grad()`` as usual: parameters updated by the hook
    are skipped there.  ``write_back=True`` also stores the averaged gradient back
    into the bucket (needed only if something else reads ``p.grad``).
    Like gradient release, the hook updates parameters during backward, so it excludes
    ``torch.amp.GradScaler`` and global gradient clipping.
    ``use_multicast`` fetches through NVSwitch ``multimem.ld_reduce``; the default
    uses peer loads in rank order, which guarantees bit-identical replicas.
    With more than two ranks, buckets of at least ``two_shot_min_bytes`` take the two-shot
    route (reduce 1/world of the bucket, store it to every rank, then one local step);
    smaller ones the one-shot kernel (``two_shot`` forces the choice).
    """
    if not isinstance(ddp_model, DDP):
        raise TypeError("fuse_ddp_allreduce expects a DistributedDataParallel model")
    state, error = None, None
    try:
        state = FusedDDPState(ddp_model, optimizer, group, timeout_s, use_multicast, write_back, max_ctas,
                              two_shot_min_bytes, two_shot)
    except (ValueError, TypeError):
        raise  # wrong use: the same on every rank, raised before any collective
    except Exception as e:  # e.g. an allocation that failed on this rank only
        error = e
    # all ranks or none (and before the hook is registered: DDP cannot unregister one)
    ok = torch.tensor([0 if state is None else 1], dtype=torch.int32, device=next(ddp_model.parameters()).device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if int(ok.item()) == 0:
        raise RuntimeError("the fused DDP path could not be set up on every rank") from error
    ddp_model.register_comm_hook(state, state.hook)
    return state
