"""Launch wrappers of the fused multi-tensor optimizer steps.

A launch takes a list of "segments" (one per tensor: parameter, gradient,
correction codes, state tensors, length) and updates all of them with one
kernel.  Up to 16 segments travel inside the kernel parameters; longer lists
live in a small device-resident table that is re-uploaded only when one of the
addresses changed since the previous step (with PyTorch's caching allocator
gradients come back at the same addresses step after step, so in steady state
nothing is uploaded).  The reference launches one Triton kernel per tensor
(``flashoptim/optimizers.py:1535-1579``, ``:2203-2251``).
"""

from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import native

SEG_WORDS = 8  # int64 words per segment: p, g, ecc, s0, s0s, s1, s1s, n

_launches = 0

# FLASHOPTIM_B200_NVTX=1 brackets every fused launch with an NVTX range named after the
# kernel family, so that a timeline shows which update (and which collective) ran where.
_NVTX = os.environ.get("FLASHOPTIM_B200_NVTX", "0") not in ("", "0")


def _launch(name: str, fn, *args) -> int:
    if not _NVTX:
        return fn(*args)
    torch.cuda.nvtx.range_push(name)
    try:
        return fn(*args)
    finally:
        torch.cuda.nvtx.range_pop()


def launch_count() -> int:
    """Number of fused step kernels launched by this process so far."""
    return _launches


class StepKernelError(RuntimeError):
    """A bounded wait inside a step kernel ran out (the update of that launch is incomplete)."""


_status: dict[int, torch.Tensor] = {}


def _ensure_status(device: torch.device) -> None:
    """Give the kernels of ``device`` a word to report a wait that ran out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        with torch.cuda.device(idx):
            native.check(native.load().fo_set_step_status(t.data_ptr()), "fo_set_step_status")
        _status[idx] = t


def check_kernel_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise :class:`StepKernelError` if a step kernel reported a timeout."""
    for idx, t in list(_status.items()):
        if device is not None and device.index not in (None, idx):
            continue
        code = int(t.item())
        if code:
            t.zero_()
            raise StepKernelError(f"cuda:{idx}: step kernel wait timed out (code {code})")


_polls: dict[int, tuple[torch.Tensor, "torch.cuda.Event"]] = {}
_poll_hosts: dict[int, torch.Tensor] = {}  # one pinned word per device, reused by every poll


def poll_kernel_status() -> None:
    """Non-blocking form of :func:`check_kernel_status`, meant to be called once per step.

    Each call looks at the copy of the status word that the previous call requested (if that
    copy has arrived) and requests a fresh one on the current stream, so the host never waits
    for the device.  A bounded wait that ran out inside a step kernel (the warps concerned
    skipped their chunks, i.e. part of that update is missing) therefore raises
    :class:`StepKernelError` one or two calls late.  Call :func:`check_kernel_status` where the
    answer must be current, e.g. before a checkpoint is written."""
    for idx, t in list(_status.items()):
        pending = _polls.get(idx)
        if pending is not None:
            host, event = pending
            if not event.query():
                continue  # still in flight: ask again next time
            del _polls[idx]
            code = int(host.item())
            if code:
                t.zero_()
                raise StepKernelError(f"cuda:{idx}: step kernel wait timed out (code {code})")
        with torch.cuda.device(idx):
            host = _poll_hosts.get(idx)
            if host is None:
                host = _poll_hosts[idx] = torch.empty(1, dtype=torch.int32).pin_memory()
            host.copy_(t, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        _polls[idx] = (host, event)


def set_step_variant(variant: int) -> None:
    """0: register-path kernels only; 1 (default): bulk-copy staged kernels where they apply."""
    native.load().fo_set_step_variant(int(variant))


def set_staged_rounds(rounds: int) -> int:
    """Tuning knob of the staged kernels: their grid is the resident CTAs times up to ``rounds``
    (1..1024; large launches only).  Returns the previous value."""
    lib = native.load()
    old = int(lib.fo_get_staged_rounds())
    lib.fo_set_staged_rounds(int(rounds))
    return old



@dataclass
class AdamHyper:
    lr: float
    beta1: float
    beta2: float
    eps: float
    weight_decay: float  # folded: wd*lr (decoupled) or wd (coupled)
    step: int
    decoupled: bool
    grad_scale: float = 1.0

    def to_c(self) -> native.FoAdamHyper:
        from .oracle import bias_corrections

        rbc1, rbc2 = bias_corrections(self.beta1, self.beta2, self.step)
        decay = 1.0 - self.weight_decay if self.decoupled else 1.0
        return native.FoAdamHyper(
            self.lr, self.beta1, self.beta2, self.eps, 1.0 - self.beta1, 1.0 - self.beta2,
            self.weight_decay, decay, rbc1, math.sqrt(rbc2), self.grad_scale, int(self.decoupled),
        )


@dataclass
class MomentumHyper:
    lr: float
    mom_coef: float
    update_coef: float
    weight_decay: float
    lion: bool = False
    nesterov: bool = False
    decoupled: bool = False
    grad_scale: float = 1.0

    def to_c(self) -> native.FoMomentumHyper:
        decay = 1.0 - self.weight_decay if (self.decoupled or self.lion) else 1.0
        return native.FoMomentumHyper(
            self.lr, self.mom_coef, self.update_coef, 1.0 - self.mom_coef, 1.0 - self.update_coef,
            self.weight_decay, decay, self.grad_scale, int(self.lion), int(self.nesterov),
            int(self.decoupled),
        )


class SegmentTable:
    """Host image + (for long lists) device copy of one launch's segment table."""

    def __init__(self, device: torch.device):
        self.device = device
        self._host: Optional[np.ndarray] = None       # [n_seg, 8] int64, last uploaded image
        self._chunks: Optional[np.ndarray] = None     # [n_seg + 1] int32
        self._dev: Optional[torch.Tensor] = None      # uint8 device buffer: segs then chunk_begin
        self._chunk = 0                               # chunk size the prefix was built for
        self.uploads = 0

    @staticmethod
    def chunk_prefix(numels: np.ndarray, chunk: int) -> np.ndarray:
        cb = np.zeros(len(numels) + 1, dtype=np.int64)
        np.cumsum((numels + chunk - 1) // chunk, out=cb[1:])
        if cb[-1] >= 2**31:
            raise ValueError("too many elements for one multi-tensor launch")
        return cb.astype(np.int32)

    def prepare(
        self, rows: np.ndarray, chunk: Optional[int] = None, force_device: bool = False
    ) -> tuple[int, int, int, int, int]:
        """``rows``: [n_seg, 8] int64.  Returns (segs_ptr, chunks_ptr, n_seg, total_chunks, on_device).

        ``chunk`` is the number of elements one CTA iteration of the target kernel covers
        (default: the local step kernels'); ``force_device`` keeps even short tables on
        the device (the peer kernels read their table from device memory only).
        """
        n_seg = rows.shape[0]
        chunk = chunk or native.chunk_elems()
        same_shape = self._host is not None and self._host.shape == rows.shape
        if not same_shape or chunk != self._chunk or not np.array_equal(self._host[:, 7], rows[:, 7]):
            self._chunks = self.chunk_prefix(rows[:, 7], chunk)
            self._chunk = chunk
            changed = True
        else:
            changed = not np.array_equal(self._host, rows)
        total = int(self._chunks[-1])
        if n_seg <= native.FO_MAX_INLINE_SEGS and not force_device:
            self._host = rows
            return rows.ctypes.data, self._chunks.ctypes.data, n_seg, total, 0
        if changed or self._dev is None:
            seg_bytes = n_seg * SEG_WORDS * 8
            img = np.empty(seg_bytes + (n_seg + 1) * 4, dtype=np.uint8)
            img[:seg_bytes] = rows.reshape(-1).view(np.uint8)
            img[seg_bytes:] = self._chunks.view(np.uint8)
            staged = torch.from_numpy(img).pin_memory()
            if self._dev is None or self._dev.numel() != img.size:
                self._dev = torch.empty(img.size, dtype=torch.uint8, device=self.device)
            self._dev.copy_(staged, non_blocking=True)
            self._host = rows.copy()
            self.uploads += 1
        base = self._dev.data_ptr()
        return base, base + n_seg * SEG_WORDS * 8, n_seg, total, 1


def launch_adam(
    table: SegmentTable,
    rows: np.ndarray,
    dtype: torch.dtype,
    err_bytes: int,
    quantized: bool,
    hyper: AdamHyper,
) -> None:
    """One fused Adam/AdamW step over every segment of ``rows`` on the current stream."""
    if rows.shape[0] == 0:
        return
    lib = native.load()
    _ensure_status(table.device)
    segs, chunks, n_seg, total, on_dev = table.prepare(rows)
    h = hyper.to_c()
    with torch.cuda.device(table.device):
        rc = _launch(
            "fo_adam_step", lib.fo_adam_step,
            segs, chunks, n_seg, total, on_dev, native.DTYPE_CODE[dtype], err_bytes, int(quantized),
            ctypes.byref(h), native.stream_ptr(table.device),
        )
    native.check(rc, "fo_adam_step")
    global _launches
    _launches += 1


def launch_momentum(
    table: SegmentTable,
    rows: np.ndarray,
    dtype: torch.dtype,
    err_bytes: int,
    state_mode: int,
    hyper: MomentumHyper,
) -> None:
    """One fused Lion / SGD / SGDW step over every segment of ``rows``."""
    if rows.shape[0] == 0:
        return
    lib = native.load()
    _ensure_status(table.device)
    segs, chunks, n_seg, total, on_dev = table.prepare(rows)
    h = hyper.to_c()
    with torch.cuda.device(table.device):
        rc = _launch(
            "fo_momentum_step", lib.fo_momentum_step,
            segs, chunks, n_seg, total, on_dev, native.DTYPE_CODE[dtype], err_bytes, state_mode,
            ctypes.byref(h), native.stream_ptr(table.device),
        )
    native.check(rc, "fo_momentum_step")
    global _launches
    _launches += 1


def launch_adam_peer(
    table: SegmentTable,
    rows: np.ndarray,
    dtype: torch.dtype,
    err_bytes: int,
    quantized: bool,
    hyper: AdamHyper,
    comm: "native.FoCommArgs",
) -> None:
    """Adam/AdamW step whose gradients are averaged from every rank's symmetric buffer
    inside the kernel; ``rows[:, 1]`` holds byte offsets into those buffers."""
    if rows.shape[0] == 0:
        return
    lib = native.load()
    chunk = lib.fo_comm_step_chunk_elems(ctypes.byref(comm), native.DTYPE_CODE[dtype], int(quantized))
    segs, chunks, n_seg, total, _ = table.prepare(rows, chunk=chunk, force_device=True)
    h = hyper.to_c()
    with torch.cuda.device(table.device):
        rc = _launch(
            "fo_adam_step_peer", lib.fo_adam_step_peer,
            segs, chunks, n_seg, total, native.DTYPE_CODE[dtype], err_bytes, int(quantized),
            ctypes.byref(h), ctypes.byref(comm), native.stream_ptr(table.device),
        )
    native.check(rc, "fo_adam_step_peer")
    global _launches
    _launches += 1


def launch_momentum_peer(
    table: SegmentTable,
    rows: np.ndarray,
    dtype: torch.dtype,
    err_bytes: int,
    state_mode: int,
    hyper: MomentumHyper,
    comm: "native.FoCommArgs",
) -> None:
    """Lion / SGD / SGDW counterpart of :func:`launch_adam_peer`."""
    if rows.shape[0] == 0:
        return
    lib = native.load()
    chunk = lib.fo_comm_step_chunk_elems(ctypes.byref(comm), native.DTYPE_CODE[dtype],
                                         int(state_mode == native.FO_STATE_Q8))
    segs, chunks, n_seg, total, _ = table.prepare(rows, chunk=chunk, force_device=True)
    h = hyper.to_c()
    with torch.cuda.device(table.device):
        rc = _launch(
            "fo_momentum_step_peer", lib.fo_momentum_step_peer,
            segs, chunks, n_seg, total, native.DTYPE_CODE[dtype], err_bytes, state_mode,
            ctypes.byref(h), ctypes.byref(comm), native.stream_ptr(table.device),
        )
    native.check(rc, "fo_momentum_step_peer")
    global _launches
    _launches += 1


def make_rows(
    params: Sequence[torch.Tensor],
    grads: Sequence[torch.Tensor],
    eccs: Sequence[Optional[torch.Tensor]],
    s0: Sequence[Optional[torch.Tensor]],
    s0s: Sequence[Optional[torch.Tensor]],
    s1: Sequence[Optional[torch.Tensor]],
    s1s: Sequence[Optional[torch.Tensor]],
) -> np.ndarray:
    """Pack tensor addresses into the [n_seg, 8] int64 image the kernels read."""
    n = len(params)
    rows = np.zeros((n, SEG_WORDS), dtype=np.int64)
    if n == 0:
        return rows

    def ptrs(ts):
        return [0 if t is None else t.data_ptr() for t in ts]

    rows[:, 0] = ptrs(params)
    rows[:, 1] = ptrs(grads)
    rows[:, 2] = ptrs(eccs)
    rows[:, 3] = ptrs(s0)
    rows[:, 4] = ptrs(s0s)
    rows[:, 5] = ptrs(s1)
    rows[:, 6] = ptrs(s1s)
    rows[:, 7] = [p.numel() for p in params]
    return rows
