"""Helpers shared by the algorithm classes: eager write-back and fused row packing."""

from __future__ import annotations

from typing import Any, Optional

import numpy as np
import torch

from ..ops import native
from ..ops.quant import compute_ecc_bits
from ..ops.step import SEG_WORDS


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
    """
    rows = np.zeros((len(items), SEG_WORDS), dtype=np.int64)
    for i, (p, g, st) in enumerate(items):
        r = rows[i]
        r[0] = p.data_ptr()
        r[1] = g if isinstance(g, int) else g.data_ptr()
        e = st.get("error_bits")
        if e is not None:
            r[2] = e.data_ptr()
        for k, key in enumerate(state_keys):
            s = st[key]
            if s.is_quantized():
                r[3 + 2 * k] = s.quantized.data_ptr()
                r[4 + 2 * k] = s.scales.data_ptr()
            else:
                r[3 + 2 * k] = s.data.data_ptr()
        r[7] = p.numel()
    return rows


def state_mode(st: dict[str, Any], key: Optional[str]) -> int:
    if key is None or key not in st:
        return native.FO_STATE_NONE
    return native.FO_STATE_Q8 if st[key].is_quantized() else native.FO_STATE_FULL
