"""Helpers shared by the algorithm classes: eager write-back and fused row packing.

The reference reaches its kernels per tensor through ``_fused_momentum_step`` /
``_fused_adam_step`` (``flashoptim/optimizers.py:1535-1583``, ``:2203-2252``) and writes the eager
result back in ``_do_step`` (``:1280-1345``, ``:1414-1511``, ``:1876-1978``); here the tensors of a
whole step are packed into one address table first.
"""

from __future__ import annotations

from typing import Any, Optional

import numpy as np
import torch

from ..ops import native
from ..ops.quant import compute_ecc_bits
from ..ops.step import SEG_WORDS

GROUP = 32  # elements per quantisation group (one fp16 scale each)


def write_back(
    param: torch.Tensor, p32: torch.Tensor, errors: Optional[torch.Tensor], master_bytewidth: int
) -> None:
    """Eager path: round the fp32 master into ``param`` and refresh its correction codes."""
    param.copy_(p32.to(param.dtype))
    if errors is not None:
        errors.copy_(compute_ecc_bits(p32, param, master_bytewidth=master_bytewidth))


def err_bytes_of(state: dict[str, Any]) -> int:
    e = state.get("error_bits")
    return 0 if e is None else e.element_size()


def pack_rows(
    items: list[tuple[torch.Tensor, Any, dict[str, Any]]], state_keys: tuple[str, ...]
) -> np.ndarray:
    """[n, 8] int64 segment image (see ``csrc/fo_api.h``: p, g, ecc, s0, s0s, s1, s1s, n).

    The gradient entry of an item is a tensor (local steps) or an ``int`` byte offset
    into the ranks' symmetric gradient buffers (steps fused with the collective).

    The kernels trust this table, so every extent is checked here: a state, correction or
    gradient tensor of the wrong length (say, from a checkpoint of another model) raises
    instead of being read or written out of bounds.
    """
    rows = np.zeros((len(items), SEG_WORDS), dtype=np.int64)
    for i, (p, g, st) in enumerate(items):
        r = rows[i]
        n = p.numel()
        r[0] = p.data_ptr()
        if isinstance(g, int):
            r[1] = g
        else:
            if g.numel() != n or g.dtype != p.dtype:
                raise ValueError(f"gradient of {g.numel()} {g.dtype} elements for a parameter of {n} {p.dtype}")
            r[1] = g.data_ptr()
        e = st.get("error_bits")
        if e is not None:
            if e.numel() != n:
                raise ValueError(f"error_bits holds {e.numel()} codes for a parameter of {n} elements")
            r[2] = e.data_ptr()
        for k, key in enumerate(state_keys):
            s = st[key]
            if s.is_quantized():
                q, sc = s.quantized, s.scales
                if q.numel() != n or sc.numel() != (n + GROUP - 1) // GROUP:
                    raise ValueError(
                        f"state {key!r}: {q.numel()} codes and {sc.numel()} scales for a parameter of {n} "
                        f"elements (expected {n} and {(n + GROUP - 1) // GROUP})")
                r[3 + 2 * k] = q.data_ptr()
                r[4 + 2 * k] = sc.data_ptr()
            else:
                d = s.data
                if d.numel() != n or d.dtype != p.dtype:
                    raise ValueError(f"state {key!r}: {d.numel()} {d.dtype} elements for a parameter of {n} {p.dtype}")
                r[3 + 2 * k] = d.data_ptr()
        r[7] = n
    return rows


def state_mode(st: dict[str, Any], key: Optional[str]) -> int:
    if key is None or key not in st:
        return native.FO_STATE_NONE
    return native.FO_STATE_Q8 if st[key].is_quantized() else native.FO_STATE_FULL
