"""ctypes binding of ``libflashoptim_b200.so`` (the hand-written sm_100a kernels).

The library speaks a plain C ABI (``csrc/fo_api.h``): raw device pointers, a
stream handle, ``cudaError_t`` return codes.  Nothing here falls back to
PyTorch: if the library cannot be loaded on a CUDA machine the call raises.
It takes the place of the reference's Triton launch wrappers
(``flashoptim/optimizers.py:1535-1583``, ``:2203-2252``, ``:2446-2540``, ``:2835-2974``).
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, Structure, c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .. import build as _build

FO_BF16, FO_FP16, FO_FP32 = 0, 1, 2
FO_STATE_NONE, FO_STATE_Q8, FO_STATE_FULL = 0, 1, 2
FO_MAX_INLINE_SEGS = 16

DTYPE_CODE = {torch.bfloat16: FO_BF16, torch.float16: FO_FP16, torch.float32: FO_FP32}


class FoSeg(Structure):
    _fields_ = [
        ("p", c_void_p),
        ("g", c_void_p),
        ("ecc", c_void_p),
        ("s0", c_void_p),
        ("s0s", c_void_p),
        ("s1", c_void_p),
        ("s1s", c_void_p),
        ("n", c_int64),
    ]


class FoAdamHyper(Structure):
    _fields_ = [
        ("lr", c_float),
        ("beta1", c_float),
        ("beta2", c_float),
        ("eps", c_float),
        ("one_minus_beta1", c_float),
        ("one_minus_beta2", c_float),
        ("weight_decay", c_float),
        ("decay", c_float),
        ("rbc1", c_float),
        ("sqrt_rbc2", c_float),
        ("grad_scale", c_float),
        ("decoupled", c_int),
    ]


class FoMomentumHyper(Structure):
    _fields_ = [
        ("lr", c_float),
        ("mom_coef", c_float),
        ("update_coef", c_float),
        ("one_minus_mom_coef", c_float),
        ("one_minus_update_coef", c_float),
        ("weight_decay", c_float),
        ("decay", c_float),
        ("grad_scale", c_float),
        ("lion", c_int),
        ("nesterov", c_int),
        ("decoupled", c_int),
    ]


FO_MAX_PEERS = 8


class FoCommArgs(Structure):
    _fields_ = [
        ("grad", c_void_p * FO_MAX_PEERS),
        ("multicast", c_void_p),
        ("pad", c_void_p * FO_MAX_PEERS),
        ("status", c_void_p),
        ("grad_out", c_void_p),
        ("grad_out_sub", c_int64),
        ("timeout_ns", ctypes.c_uint64),
        ("epoch", ctypes.c_uint32),
        ("world", c_int),
        ("rank", c_int),
        ("ready_channel", c_int),
        ("done_channel", c_int),
        ("max_ctas", c_int),
        ("push", c_int),
        ("param_out", c_void_p * FO_MAX_PEERS),
        ("param_out_mc", c_void_p),
        ("param_out_delta", c_int64),
        ("push_epoch", ctypes.c_uint32),
        ("pushed_channel", c_int),
        ("variant", c_int),
        ("flags", c_int),
    ]


FO_COMM_NO_BARRIER, FO_COMM_NO_SIGNAL, FO_COMM_PUSH_LOCAL = 1, 2, 4


class NativeError(RuntimeError):
    """A kernel launch of libflashoptim_b200.so returned a CUDA error code."""


_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


def _declare(lib: ctypes.CDLL) -> None:
    lib.fo_chunk_elems.restype = c_int
    lib.fo_chunk_elems.argtypes = []
    lib.fo_step_grid.restype = c_int
    lib.fo_step_grid.argtypes = [c_int]
    lib.fo_set_staged_rounds.restype = None
    lib.fo_set_staged_rounds.argtypes = [c_int]
    lib.fo_get_staged_rounds.restype = c_int
    lib.fo_get_staged_rounds.argtypes = []
    lib.fo_set_step_variant.restype = None
    lib.fo_set_step_variant.argtypes = [c_int]
    lib.fo_get_step_variant.restype = c_int
    lib.fo_get_step_variant.argtypes = []
    lib.fo_set_step_status.restype = c_int
    lib.fo_set_step_status.argtypes = [c_void_p]
    lib.fo_adam_step.restype = c_int
    lib.fo_adam_step.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(FoAdamHyper), c_void_p,
    ]
    lib.fo_momentum_step.restype = c_int
    lib.fo_momentum_step.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(FoMomentumHyper), c_void_p,
    ]
    lib.fo_quantize.restype = c_int
    lib.fo_quantize.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
    lib.fo_dequantize.restype = c_int
    lib.fo_dequantize.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
    lib.fo_ecc_decode.restype = c_int
    lib.fo_ecc_decode.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p]
    lib.fo_ecc_encode.restype = c_int
    lib.fo_ecc_encode.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int64, c_void_p]
    lib.fo_maxabs.restype = c_int
    lib.fo_maxabs.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_void_p]
    lib.fo_comm_step_chunk_elems.restype = c_int
    lib.fo_comm_step_chunk_elems.argtypes = [POINTER(FoCommArgs), c_int, c_int]
    lib.fo_adam_step_peer.restype = c_int
    lib.fo_adam_step_peer.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, POINTER(FoAdamHyper), POINTER(FoCommArgs),
        c_void_p,
    ]
    lib.fo_momentum_step_peer.restype = c_int
    lib.fo_momentum_step_peer.argtypes = [
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, POINTER(FoMomentumHyper),
        POINTER(FoCommArgs), c_void_p,
    ]
    lib.fo_reduce_peer.restype = c_int
    lib.fo_reduce_peer.argtypes = [c_int64, c_int64, c_void_p, c_int, c_float, POINTER(FoCommArgs), c_void_p]
    lib.fo_reduce_bcast_peer.restype = c_int
    lib.fo_reduce_bcast_peer.argtypes = [c_int64, c_int64, c_int64, c_int, c_float, POINTER(FoCommArgs), c_void_p]
    lib.fo_allgather_peer.restype = c_int
    lib.fo_allgather_peer.argtypes = [c_int64, POINTER(FoCommArgs), c_void_p]
    lib.fo_adam_step_noalloc.restype = c_int
    lib.fo_adam_step_noalloc.argtypes = [c_void_p, c_int, c_int, c_int, c_int, POINTER(FoAdamHyper), c_void_p]
    lib.fo_probe_fast_ecc_split.restype = c_int
    lib.fo_probe_fast_ecc_split.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p]
    lib.fo_probe_fast_ecc_merge.restype = c_int
    lib.fo_probe_fast_ecc_merge.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p]
    lib.fo_comm_signal.restype = c_int
    lib.fo_comm_signal.argtypes = [POINTER(FoCommArgs), c_int, c_void_p]
    lib.fo_comm_wait.restype = c_int
    lib.fo_comm_wait.argtypes = [POINTER(FoCommArgs), c_int, c_void_p]
    lib.fo_comm_barrier.restype = c_int
    lib.fo_comm_barrier.argtypes = [POINTER(FoCommArgs), c_void_p]
    lib.fo_memcpy_async.restype = c_int
    lib.fo_memcpy_async.argtypes = [c_void_p, c_void_p, c_int64, c_void_p]


def load(path: Optional[str] = None) -> ctypes.CDLL:
    """Load (building first if sources changed and nvcc is present) the library."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    with _lock:
        if _lib is not None and path is None:
            return _lib
        if path is None:
            if not _build.is_current():
                if _build.find_nvcc() is not None:
                    _build.build()
                elif not _build.LIB_PATH.exists():
                    raise NativeError(
                        f"{_build.LIB_PATH} is missing and nvcc is not available to build it; "
                        "run `python -m flashoptim_b200.build` on a machine with CUDA 12.8+"
                    )
            target = str(_build.LIB_PATH)
        else:
            target = path
        lib = ctypes.CDLL(target)
        _declare(lib)
        if path is None:
            _lib = lib
        return lib


def is_available() -> bool:
    """True when a CUDA device is present (the native path is then mandatory)."""
    return torch.cuda.is_available()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with CUDA error {rc}")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def chunk_elems() -> int:
    return load().fo_chunk_elems()
