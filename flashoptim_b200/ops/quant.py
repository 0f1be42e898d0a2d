"""Group quantisation and master-weight split as tensor-in / tensor-out functions.

CUDA tensors go to the sm_100a kernels of ``libflashoptim_b200.so``; CPU
tensors go to the PyTorch formulation in :mod:`flashoptim_b200.ops.oracle`.
Both produce identical bits.  API parity with the reference:
``quantize`` / ``dequantize`` (``flashoptim/optimizers.py:2446-2538``),
``reconstruct_fp32_param`` (``:2835-2892``), ``compute_ecc_bits`` (``:2895-2970``).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import native, oracle
from .oracle import GROUP_SIZE, MANTISSA_BITS


def _require_group32(group_size: int) -> None:
    if group_size != GROUP_SIZE:
        raise ValueError(f"only group_size={GROUP_SIZE} is supported, got {group_size}")


def quantize(
    x_float: torch.Tensor,
    out_int8: Optional[torch.Tensor] = None,
    out_scales: Optional[torch.Tensor] = None,
    signed: bool = True,
    group_size: int = GROUP_SIZE,
    sqrt: bool = False,
    softsign: bool = True,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Quantise a float tensor to grouped 8-bit codes and fp16 per-group scales.

    Returns ``(codes, scales)``: ``codes`` has ``x_float``'s shape and dtype
    int8 (``signed``) or uint8; ``scales`` is 1-D fp16 with one entry per 32
    consecutive elements of the flattened input.
    """
    _require_group32(group_size)
    n = x_float.numel()
    q_dtype = torch.int8 if signed else torch.uint8
    if out_int8 is None:
        out_int8 = torch.empty(x_float.shape, dtype=q_dtype, device=x_float.device)
    if out_scales is None:
        out_scales = torch.empty(oracle.num_groups(n), dtype=torch.float16, device=x_float.device)
    if n == 0:
        return out_int8, out_scales
    if x_float.is_cuda:
        x = x_float.detach()
        if x.dtype not in native.DTYPE_CODE:
            x = x.to(torch.float32)
        x = x.contiguous()
        if not out_int8.is_contiguous():
            raise ValueError("out_int8 must be contiguous")
        lib = native.load()
        with torch.cuda.device(x.device):
            rc = lib.fo_quantize(
                x.data_ptr(), native.DTYPE_CODE[x.dtype], out_int8.data_ptr(), out_scales.data_ptr(),
                n, int(signed), int(sqrt), int(softsign), native.stream_ptr(x.device),
            )
        native.check(rc, "fo_quantize")
    else:
        q, s = oracle.quantize_ref(x_float, signed=signed, sqrt=sqrt, softsign=softsign)
        out_int8.copy_(q)
        out_scales.copy_(s)
    return out_int8, out_scales


def dequantize(
    in_int8: torch.Tensor,
    in_scales: torch.Tensor,
    out_float: Optional[torch.Tensor] = None,
    signed: bool = True,
    group_size: int = GROUP_SIZE,
    sqrt: bool = False,
    softsign: bool = True,
) -> torch.Tensor:
    """Inverse of :func:`quantize`; returns an fp32 tensor of ``in_int8``'s shape."""
    _require_group32(group_size)
    n = in_int8.numel()
    if out_float is None:
        out_float = torch.empty(in_int8.shape, dtype=torch.float32, device=in_int8.device)
    if n == 0:
        return out_float
    if in_int8.is_cuda:
        q = in_int8.contiguous()
        s = in_scales.contiguous()
        if out_float.dtype != torch.float32 or not out_float.is_contiguous():
            raise ValueError("out_float must be a contiguous float32 tensor")
        lib = native.load()
        with torch.cuda.device(q.device):
            rc = lib.fo_dequantize(
                q.data_ptr(), s.data_ptr(), out_float.data_ptr(), n, int(signed), int(sqrt),
                int(softsign), native.stream_ptr(q.device),
            )
        native.check(rc, "fo_dequantize")
    else:
        out_float.copy_(oracle.dequantize_ref(in_int8, in_scales, signed=signed, sqrt=sqrt, softsign=softsign))
    return out_float


def reconstruct_fp32_param(param: torch.Tensor, error_bits: torch.Tensor) -> torch.Tensor:
    """fp32 master weight from a bf16/fp16 parameter and its correction codes."""
    if param.dtype == torch.float32:
        raise ValueError(
            "param is already fp32; ECC reconstruction is only meaningful for "
            f"narrow dtypes (bf16, fp16). Got {param.dtype}."
        )
    if param.dtype not in MANTISSA_BITS:
        raise ValueError(
            f"Unsupported param dtype {param.dtype}; expected one of {list(MANTISSA_BITS)}."
        )
    if error_bits.dtype not in (torch.int8, torch.int16):
        raise ValueError(f"error_bits must be int8 or int16, got {error_bits.dtype}.")
    if param.is_cuda:
        w = param.detach().contiguous()
        e = error_bits.contiguous()
        out = torch.empty(param.shape, dtype=torch.float32, device=param.device)
        if w.numel():
            lib = native.load()
            with torch.cuda.device(w.device):
                rc = lib.fo_ecc_decode(
                    w.data_ptr(), native.DTYPE_CODE[w.dtype], e.data_ptr(), e.element_size(),
                    out.data_ptr(), w.numel(), native.stream_ptr(w.device),
                )
            native.check(rc, "fo_ecc_decode")
        return out
    return oracle.ecc_decode_ref(param.detach(), error_bits)


def compute_ecc_bits(
    fp32_param: torch.Tensor, narrow_param: torch.Tensor, master_bytewidth: int = 4
) -> torch.Tensor:
    """Correction codes (int8 for 24-bit, int16 for 32-bit masters) of ``fp32_param``
    against its narrow rounding ``narrow_param``.  Inverse of
    :func:`reconstruct_fp32_param`."""
    if fp32_param.dtype != torch.float32:
        raise ValueError(f"fp32_param must be float32, got {fp32_param.dtype}.")
    if narrow_param.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError(f"narrow_param must be bf16 or fp16, got {narrow_param.dtype}.")
    err_bytes = master_bytewidth - narrow_param.element_size()
    if err_bytes not in (1, 2):
        raise ValueError(
            f"Unsupported dtype combination: master_bytewidth={master_bytewidth} to "
            f"{narrow_param.dtype} ({narrow_param.element_size()} bytes). "
            f"Error byte width {err_bytes} must be 1 or 2."
        )
    if narrow_param.is_cuda:
        x = fp32_param.detach().to(narrow_param.device).contiguous()
        w = narrow_param.detach().contiguous()
        out = torch.empty(
            narrow_param.shape, dtype=torch.int8 if err_bytes == 1 else torch.int16, device=w.device
        )
        if w.numel():
            lib = native.load()
            with torch.cuda.device(w.device):
                rc = lib.fo_ecc_encode(
                    x.data_ptr(), w.data_ptr(), native.DTYPE_CODE[w.dtype], out.data_ptr(), err_bytes,
                    w.numel(), native.stream_ptr(w.device),
                )
            native.check(rc, "fo_ecc_encode")
        return out
    return oracle.ecc_encode_ref(fp32_param.detach(), narrow_param.detach(), err_bytes)


def maxabs(x: torch.Tensor) -> float:
    """``max |x|`` as a Python float (one device synchronisation on CUDA)."""
    if x.numel() == 0:
        return 0.0
    if x.is_cuda and x.dtype in native.DTYPE_CODE:
        xc = x.detach().contiguous()
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
        lib = native.load()
        with torch.cuda.device(xc.device):
            rc = lib.fo_maxabs(
                xc.data_ptr(), native.DTYPE_CODE[xc.dtype], xc.numel(), out.data_ptr(),
                native.stream_ptr(xc.device),
            )
        native.check(rc, "fo_maxabs")
        return float(out.item())
    return float(x.detach().abs().max().item())
