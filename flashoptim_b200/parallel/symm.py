"""Symmetric NVLink buffers and the flag protocol of the peer kernels.

A :class:`PeerGroup` is the set of GPUs of one node that map each other's
buffers (allocation and handle exchange through
``torch.distributed._symmetric_memory``; all data movement is done by this
library's kernels).  It owns

* a *signal pad*: ``channels x 8`` uint32 flags per rank, written by peers with
  release stores and read with acquire loads, carrying monotonically growing
  epochs;
* a 4-word local *status* tensor where a kernel records a wait that ran out;
* any number of :class:`SymmBuffer` allocations.

A step kernel can also push the parameters it has just updated into a second
symmetric buffer of every rank (:class:`ParamPush`), publishing a third flag
("pushed") when done: the all-gather of the next forward pass then only waits.

Ordering protocol for a buffer with channels (ready, done) and epoch ``e``:
a consumer kernel publishes ``ready = e`` ("my copy of the buffer is written",
true by stream order), waits until every rank has published it, reads all
copies, and finally publishes ``done = e``.  Before a rank overwrites its copy
again it waits (``wait_done``) until every rank has published ``done = e``.

With ``world_size == 1`` no symmetric allocation is needed and ordinary tensors
are used, which also lets one process emulate several ranks for tests by
passing explicit buffer lists.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import native

CHANNELS = 256


class CommTimeoutError(RuntimeError):
    """A device-side wait for another rank's flag ran out of time."""


class SymmBuffer:
    """``nbytes`` of device memory mapped on every rank of a :class:`PeerGroup`."""

    def __init__(self, tensor: torch.Tensor, ptrs: Sequence[int], multicast_ptr: int, handle=None):
        self.tensor = tensor          # this rank's copy, flat uint8
        self.ptrs = list(ptrs)        # address of every rank's copy in this process
        self.multicast_ptr = multicast_ptr
        self._handle = handle         # keeps the mapping alive

    @property
    def nbytes(self) -> int:
        return self.tensor.numel()

    def view(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """This rank's copy, ``numel`` elements of ``dtype`` starting ``offset`` bytes in."""
        size = numel * torch.empty((), dtype=dtype).element_size()
        return self.tensor[offset:offset + size].view(dtype)


class PeerGroup:
    def __init__(
        self,
        group: Optional[dist.ProcessGroup] = None,
        device: Optional[torch.device] = None,
        timeout_s: float = 2.0,
        use_multicast: bool = True,
        max_ctas: int = 0,
        push_multicast: Optional[bool] = None,
        variant: int = 0,
    ):
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        if self.world > native.FO_MAX_PEERS:
            raise ValueError(f"at most {native.FO_MAX_PEERS} ranks (one NVSwitch node) are supported")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.timeout_ns = int(timeout_s * 1e9)
        # gradients through multimem.ld_reduce (NVSwitch adds the ranks' copies) instead of peer loads
        self.use_multicast = use_multicast
        # parameter pushes through multimem.st (one store, replicated by the switch) instead of
        # one store per rank; None: as use_multicast
        self.push_multicast = use_multicast if push_multicast is None else push_multicast
        # 1: bulk-copy staged step kernels where they apply (peer loads, 8-bit states, bf16/fp16)
        self.variant = variant
        self.max_ctas = max_ctas  # grid cap of the peer kernels (0: fill the GPU)
        # bytes of symmetric memory handed out so far; PyTorch's caching-allocator statistics
        # (torch.cuda.max_memory_allocated) do not see these allocations
        self.symmetric_bytes = 0
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._pad = self.allocate(CHANNELS * native.FO_MAX_PEERS * 4, zero=True)
        self._next_channel = 0

    # ------------------------------------------------------------------ allocation
    def allocate(self, nbytes: int, zero: bool = False) -> SymmBuffer:
        """Collective: every rank must call with the same size, in the same order."""
        nbytes = (int(nbytes) + 255) // 256 * 256
        self.symmetric_bytes += nbytes
        if self.world == 1:
            t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            if zero:
                t.zero_()
            return SymmBuffer(t, [t.data_ptr()], 0)
        import torch.distributed._symmetric_memory as symm_mem

        t = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        if zero:
            t.zero_()
        hdl = symm_mem.rendezvous(t, group=self.group)
        # the mapping is recorded whenever the machine has one; use_multicast / push_multicast
        # decide per launch whether a kernel gets it
        mc = int(hdl.multicast_ptr) if hdl.has_multicast_support else 0
        buf = SymmBuffer(t, [int(p) for p in hdl.buffer_ptrs], mc, hdl)
        if zero:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        return buf

    def new_channel(self) -> int:
        """One fresh channel; same sequence on every rank."""
        if self._next_channel + 1 > CHANNELS:
            raise RuntimeError("out of signal channels")
        c = self._next_channel
        self._next_channel += 1
        return c

    def new_channels(self) -> tuple[int, int]:
        """A fresh (ready, done) channel pair; same sequence on every rank."""
        if self._next_channel + 2 > CHANNELS:
            raise RuntimeError("out of signal channels")
        c = self._next_channel
        self._next_channel += 2
        return c, c + 1

    # ------------------------------------------------------------------ kernel arguments
    def comm_args(
        self,
        buf: SymmBuffer,
        epoch: int,
        ready_channel: int,
        done_channel: int,
        grad_out: Optional[torch.Tensor] = None,
        grad_out_sub: int = 0,
        multicast: Optional[bool] = None,
        pads: Optional[Sequence[int]] = None,
        ptrs: Optional[Sequence[int]] = None,
        world: Optional[int] = None,
        rank: Optional[int] = None,
    ) -> native.FoCommArgs:
        a = native.FoCommArgs()
        ptrs = list(ptrs if ptrs is not None else buf.ptrs)
        pads = list(pads if pads is not None else self._pad.ptrs)
        w = world if world is not None else self.world
        for r in range(w):
            a.grad[r] = ptrs[r]
            a.pad[r] = pads[r]
        use_mc = self.use_multicast if multicast is None else multicast
        a.multicast = buf.multicast_ptr if (use_mc and buf.multicast_ptr) else None
        a.status = self.status.data_ptr()
        a.grad_out = grad_out.data_ptr() if grad_out is not None else None
        a.grad_out_sub = grad_out_sub
        a.timeout_ns = self.timeout_ns
        a.epoch = epoch & 0xFFFFFFFF
        a.world = w
        a.rank = rank if rank is not None else self.rank
        a.ready_channel = ready_channel
        a.done_channel = done_channel
        a.max_ctas = self.max_ctas
        a.variant = self.variant
        return a

    # ------------------------------------------------------------------ flags
    def wait(self, args: native.FoCommArgs, channel: int) -> None:
        """Enqueue (current stream) a bounded wait until every rank's ``channel`` flag reached ``args.epoch``."""
        native.check(native.load().fo_comm_wait(ctypes.byref(args), channel, native.stream_ptr(self.device)),
                     "fo_comm_wait")

    def signal(self, args: native.FoCommArgs, channel: int) -> None:
        native.check(native.load().fo_comm_signal(ctypes.byref(args), channel, native.stream_ptr(self.device)),
                     "fo_comm_signal")

    def barrier(self, args: native.FoCommArgs) -> None:
        """Enqueue a one-CTA kernel that publishes ``args.epoch`` on the ready channel and waits
        (bounded) for every rank's."""
        native.check(native.load().fo_comm_barrier(ctypes.byref(args), native.stream_ptr(self.device)),
                     "fo_comm_barrier")

    def copy(self, dst_ptr: int, src_ptr: int, nbytes: int) -> None:
        """Enqueue a device-to-device copy between two mapped addresses (either may be another
        rank's symmetric buffer): the driver's copy engines move the bytes, no SM does."""
        native.check(native.load().fo_memcpy_async(dst_ptr, src_ptr, nbytes, native.stream_ptr(self.device)),
                     "fo_memcpy_async")

    def poll_status(self) -> None:
        """Like :meth:`check_status` but never waits for the device: each call inspects the copy
        of the status words that the previous call requested (if that copy has arrived) and
        requests a fresh one on the current stream.  A wait that ran out is therefore reported
        one or two calls late; meant to be called once per training step."""
        pending = getattr(self, "_poll", None)
        if pending is not None:
            host, event = pending
            if event is None or event.query():
                self._poll = None
                st = host.tolist()
                if st[0] != 0:
                    # only the two report words: the CTA counters behind them belong to kernels
                    # that may be in flight
                    self.status[:2].zero_()
                    raise CommTimeoutError(
                        f"rank {self.rank}: wait on channel mask {st[0]:#x} timed out (missing rank {st[1] - 1})"
                    )
        if getattr(self, "_poll", None) is None:
            if self.status.is_cuda:
                if getattr(self, "_poll_host", None) is None:
                    self._poll_host = torch.empty(4, dtype=torch.int32).pin_memory()
                self._poll_host.copy_(self.status, non_blocking=True)
                event = torch.cuda.Event()
                event.record()
                self._poll = (self._poll_host, event)
            else:
                self._poll = (self.status.clone(), None)

    def check_status(self) -> None:
        """Synchronise and raise :class:`CommTimeoutError` if any device-side wait ran out."""
        torch.cuda.synchronize(self.device)
        st = self.status.tolist()
        if st[0] != 0:
            self.status.zero_()
            raise CommTimeoutError(
                f"rank {self.rank}: wait on channel mask {st[0]:#x} timed out (missing rank {st[1] - 1})"
            )


@dataclass
class ParamPush:
    """Target of the step kernels' all-gather on write: every rank's copy of ``buf`` receives
    the updated parameters at (gradient byte offset + ``delta``); ``epoch`` counts the
    launches that pushed and is what the ``channel`` flags carry."""

    buf: SymmBuffer
    channel: int
    delta: int = 0
    epoch: int = 0


@dataclass
class PeerGradients:
    """What an optimizer needs to step straight from the ranks' symmetric gradient buffers."""

    group: PeerGroup
    buf: SymmBuffer
    ready_channel: int
    done_channel: int
    offsets: dict[int, int] = field(default_factory=dict)  # id(local param tensor) -> byte offset
    grad_scale: float = 1.0
    grad_out: Optional[torch.Tensor] = None
    grad_out_sub: int = 0
    key: int = 0
    epoch: int = 0  # last epoch used on this buffer
    push: Optional[ParamPush] = None  # step kernels also send the new parameters there
    max_ctas: Optional[int] = None  # grid cap of the next launch (None: the group's)
    # Copy-engine transport: the other ranks' rows were copied into this local [world, row_bytes]
    # buffer beforehand (its address, and the size of a row), so the step kernels read local
    # memory, synchronise with nobody and publish nothing; next_args() then leaves the epochs alone
    local_rows: Optional[tuple[int, int]] = None

    def next_args(self) -> native.FoCommArgs:
        staged_locally = self.local_rows is not None
        if not staged_locally:
            self.epoch += 1
        a = self.group.comm_args(
            self.buf, self.epoch, self.ready_channel, self.done_channel, self.grad_out, self.grad_out_sub
        )
        if self.max_ctas is not None:
            a.max_ctas = self.max_ctas
        if staged_locally:
            base, row_bytes = self.local_rows
            for r in range(a.world):
                if r != a.rank:  # the kernel adds (rank * row_bytes + offset in the row) to every base
                    a.grad[r] = base + (r - a.rank) * row_bytes
            a.multicast = None
            a.flags = native.FO_COMM_NO_BARRIER | native.FO_COMM_NO_SIGNAL | native.FO_COMM_PUSH_LOCAL
        if self.push is not None:
            t = self.push
            if not staged_locally:
                t.epoch += 1
            a.push = 1
            for r in range(a.world):
                a.param_out[r] = t.buf.ptrs[r]
            a.param_out_mc = (t.buf.multicast_ptr
                              if (getattr(self.group, "push_multicast", False) and t.buf.multicast_ptr) else None)
            a.param_out_delta = t.delta
            a.push_epoch = t.epoch & 0xFFFFFFFF
            a.pushed_channel = t.channel
        return a

    def wait_done(self) -> None:
        """Current stream waits until every rank has finished reading the buffer's last use."""
        if self.epoch == 0 or self.group.world == 1:
            return
        args = self.group.comm_args(self.buf, self.epoch, self.ready_channel, self.done_channel)
        self.group.wait(args, self.done_channel)
