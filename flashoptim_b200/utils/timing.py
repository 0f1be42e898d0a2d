"""Device timing, NVTX ranges and roofline arithmetic.

The reference has no tracing or timing of its own (its only timing is a
wall-clock loop in ``test/test_optimizers.py:681-690``).  These helpers time on
the device with CUDA events, take the maximum over ranks, and express a fused
update as a fraction of the measured copy bandwidth.
"""

from __future__ import annotations

import contextlib
import json
import os
from dataclasses import dataclass
from typing import Callable, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    """``torch.cuda.nvtx`` range that is a no-op without CUDA."""
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def time_on_device(fn: Callable[[], None], iters: int = 10, warmup: int = 3, group=None) -> float:
    """Milliseconds per call of ``fn``: CUDA events on the current stream after
    ``warmup`` calls, synchronised on both sides, maximum over the ranks of ``group``."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        ms = float(t.item())
    return ms


def step_bytes_per_element(n_states: int, err_bytes: int, param_bytes: int = 2, quantized: bool = True) -> float:
    """HBM bytes one fused update moves per element: param + grad read, param written,
    every state read and written (8-bit codes + one fp16 scale per 32 elements when
    quantised, else the param dtype), correction codes read and written."""
    state = (1 + 2 / 32) if quantized else param_bytes
    return 3 * param_bytes + 2 * n_states * state + 2 * err_bytes


@dataclass
class Roofline:
    hbm_gbs: float
    source: str  # "measured" | "fallback"

    @classmethod
    def load(cls, repo_root: Optional[str] = None) -> "Roofline":
        root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        path = os.path.join(root, "MEASURED_PEAKS.json")
        if os.path.exists(path):
            return cls(float(json.load(open(path))["hbm_gbs"]), "measured")
        return cls(6650.0, "fallback")

    def fraction(self, n_elements: int, bytes_per_element: float, ms: float) -> float:
        return n_elements * bytes_per_element / (ms * 1e-3) / 1e9 / self.hbm_gbs
