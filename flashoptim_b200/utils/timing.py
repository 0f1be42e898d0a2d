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
import statistics
import threading
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


FALLBACK_HBM_GBS = 6650.0  # an earlier copy-bandwidth measurement on B200, used when none is given


@dataclass
class Roofline:
    hbm_gbs: float
    source: str  # "measured" | "fallback"

    @classmethod
    def load(cls, peaks_file: Optional[str] = None) -> "Roofline":
        """Copy bandwidth from a JSON file with an ``hbm_gbs`` entry (``peaks_file``, else the
        file named by the environment variable ``FLASHOPTIM_B200_PEAKS``); without one the
        fallback figure, labelled as such."""
        path = peaks_file or os.environ.get("FLASHOPTIM_B200_PEAKS")
        if path and os.path.exists(path):
            with open(path) as f:
                return cls(float(json.load(f)["hbm_gbs"]), "measured")
        return cls(FALLBACK_HBM_GBS, "fallback")

    def fraction(self, n_elements: int, bytes_per_element: float, ms: float) -> float:
        return n_elements * bytes_per_element / (ms * 1e-3) / 1e9 / self.hbm_gbs


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML every 200 ms from a
    background thread.  Read-only: no clock, power or mode setting is ever changed."""

    def __init__(self, index: int):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }
