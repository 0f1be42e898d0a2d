"""Device-agnostic numerics: the written-down specification of every format.

Everything here is plain PyTorch in fp32 with IEEE operations, one rounding per
operation, so it runs on CPU (the execution path when no GPU is present) and
serves as the oracle the sm_100a kernels are tested against.

Formats (parity with the reference: ``flashoptim/optimizers.py:2610-2676`` for
the group quantiser, ``:2541-2607`` for its inverse, ``:2682-2776`` for the
error-correction split of a master weight):

* Group quantisation. The flattened tensor is cut into groups of 32 consecutive
  elements (the tail group is zero padded). Per group: ``absmax`` in fp32,
  clamped to 1e-12; ``n = x / absmax``; optional compander ``t = 2n / (1+|n|)``;
  ``q = floor(t * MAX + 0.5)`` with ``MAX`` 127 (int8) or 255 (uint8); the scale
  that is stored is ``float16(absmax)``.  ``sqrt=True`` stores ``sqrt(x)``.
* Error correction. For a narrow value ``w`` (bf16 / fp16) with mantissa width
  ``M`` and unbiased exponent ``E`` (subnormals use the smallest normal
  exponent) the half-ULP is ``2**ls`` with ``ls = E - M - 1``.  The correction
  code is ``round_half_away(clamp((x - w) / 2**ls, -1, 1) * S)`` with ``S`` 127
  (int8) or 32767 (int16), and ``x ~= w + code / S * 2**ls``.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

GROUP_SIZE = 32

DTYPE_WIDTHS = {
    torch.int8: 1,
    torch.uint8: 1,
    torch.int16: 2,
    torch.float16: 2,
    torch.bfloat16: 2,
    torch.float32: 4,
}
EXPONENT_BITS = {torch.float16: 5, torch.bfloat16: 8, torch.float32: 8}
MANTISSA_BITS = {torch.float16: 10, torch.bfloat16: 7, torch.float32: 23}
EXPONENT_BIAS = {torch.float16: 15, torch.bfloat16: 127, torch.float32: 127}


# --------------------------------------------------------------------------- quantisation


def num_groups(numel: int, group_size: int = GROUP_SIZE) -> int:
    return (numel + group_size - 1) // group_size


def quantize_ref(
    x: torch.Tensor,
    signed: bool = True,
    sqrt: bool = False,
    softsign: bool = True,
    group_size: int = GROUP_SIZE,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Group-quantise ``x`` to int8/uint8 codes (shape of ``x``) + fp16 scales."""
    n = x.numel()
    out_dtype = torch.int8 if signed else torch.uint8
    qmax = 127.0 if signed else 255.0
    ng = num_groups(n, group_size)
    if n == 0:
        return (
            torch.empty(x.shape, dtype=out_dtype, device=x.device),
            torch.empty(0, dtype=torch.float16, device=x.device),
        )
    x32 = x.detach().reshape(-1).to(torch.float32)
    if sqrt:
        x32 = x32.sqrt()
    pad = ng * group_size - n
    if pad:
        x32 = torch.nn.functional.pad(x32, (0, pad))
    g = x32.view(ng, group_size)
    absmax = g.abs().amax(dim=1).clamp_min(1e-12)
    t = g / absmax[:, None]
    if softsign:
        t = (t * 2.0) / (t.abs() + 1.0)
    q = torch.floor(t * qmax + 0.5)
    q = q.reshape(-1)[:n].to(torch.int16).to(out_dtype).reshape(x.shape)
    return q, absmax.to(torch.float16)


def dequantize_ref(
    q: torch.Tensor,
    scales: torch.Tensor,
    signed: bool = True,
    sqrt: bool = False,
    softsign: bool = True,
    group_size: int = GROUP_SIZE,
) -> torch.Tensor:
    """Inverse of :func:`quantize_ref`; returns fp32 of ``q``'s shape."""
    n = q.numel()
    if n == 0:
        return torch.empty(q.shape, dtype=torch.float32, device=q.device)
    qmax = 127.0 if signed else 255.0
    ng = num_groups(n, group_size)
    t = q.reshape(-1).to(torch.float32)
    pad = ng * group_size - n
    if pad:
        t = torch.nn.functional.pad(t, (0, pad))
    t = t.view(ng, group_size) / qmax
    if softsign:
        t = t / (2.0 - t.abs())
    x = t * scales.reshape(-1).to(torch.float32)[:, None]
    if sqrt:
        x = x * x
    return x.reshape(-1)[:n].reshape(q.shape)


# --------------------------------------------------------------------------- error correction


def _pow2(e: torch.Tensor) -> torch.Tensor:
    """Exact fp32 ``2**e`` for int32 ``e`` in [-126, 127], built from the bits."""
    return ((e.to(torch.int32) + 127) << 23).view(torch.float32)


def ecc_log_scale(narrow: torch.Tensor) -> torch.Tensor:
    """int32 ``log2`` of half an ULP of every element of a bf16/fp16 tensor."""
    dt = narrow.dtype
    m = MANTISSA_BITS[dt]
    bias = EXPONENT_BIAS[dt]
    bits = narrow.contiguous().view(torch.int16).to(torch.int32) & 0x7FFF
    field = bits >> m
    e = torch.where(field == 0, torch.full_like(field, 1 - bias), field - bias)
    return e - m - 1


def ecc_encode_ref(
    x_f32: torch.Tensor, narrow: torch.Tensor, err_bytes: int
) -> torch.Tensor:
    """Correction codes (int8 for ``err_bytes`` 1, int16 for 2) of ``x_f32 - narrow``."""
    smax = 127.0 if err_bytes == 1 else 32767.0
    out_dtype = torch.int8 if err_bytes == 1 else torch.int16
    e = x_f32.to(torch.float32) - narrow.to(torch.float32)
    neg = -ecc_log_scale(narrow)
    h = torch.div(neg, 2, rounding_mode="floor")
    e_norm = (e * _pow2(h)) * _pow2(neg - h)
    scaled = e_norm.clamp(-1.0, 1.0) * smax
    r = torch.copysign(torch.floor(scaled.abs() + 0.5), scaled)
    return r.to(torch.int32).to(out_dtype)


def ecc_decode_ref(narrow: torch.Tensor, ecc: torch.Tensor) -> torch.Tensor:
    """fp32 master value rebuilt from a narrow tensor and its correction codes."""
    smax = 127.0 if ecc.element_size() == 1 else 32767.0
    ls = ecc_log_scale(narrow)
    h = torch.div(ls, 2, rounding_mode="floor")
    corr = ecc.to(torch.float32) / smax
    e = (corr * _pow2(h)) * _pow2(ls - h)
    return narrow.to(torch.float32) + e


def read_param_fp32(param: torch.Tensor, ecc: Optional[torch.Tensor]) -> torch.Tensor:
    if ecc is not None:
        return ecc_decode_ref(param, ecc)
    return param.to(torch.float32)


# --------------------------------------------------------------------------- update rules (fp32)


def bias_corrections(beta1: float, beta2: float, step: int) -> tuple[float, float]:
    """Reciprocal Adam bias corrections, evaluated in double on the host."""
    return 1.0 / (1.0 - beta1**step), 1.0 / (1.0 - beta2**step)


def adam_math(
    p: torch.Tensor,
    g: torch.Tensor,
    m: torch.Tensor,
    v: torch.Tensor,
    *,
    lr: float,
    beta1: float,
    beta2: float,
    eps: float,
    weight_decay: float,
    decoupled: bool,
    step: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One Adam/AdamW update on fp32 tensors; returns new ``(p, m, v)``.

    ``weight_decay`` is the scalar already folded by the caller: ``wd*lr`` (or
    ``wd*lr/initial_lr``) when decoupled, raw ``wd`` when coupled
    (reference ``flashoptim/optimizers.py:1894-1898``, kernel ``:2310-2375``).
    """
    if not decoupled and weight_decay != 0.0:
        g = g + p * weight_decay
    m = m * beta1 + g * (1.0 - beta1)
    v = v * beta2 + (g * g) * (1.0 - beta2)
    if decoupled and weight_decay != 0.0:
        p = p * (1.0 - weight_decay)
    rbc1, rbc2 = bias_corrections(beta1, beta2, step)
    denom = (v * rbc2).sqrt() + eps
    p = p - ((m * rbc1) * lr) / denom
    return p, m, v


def momentum_math(
    p: torch.Tensor,
    g: torch.Tensor,
    m: Optional[torch.Tensor],
    *,
    lr: float,
    mom_coef: float,
    update_coef: float,
    weight_decay: float,
    decoupled: bool,
    nesterov: bool,
    lion: bool,
) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
    """One Lion / SGD / SGDW update on fp32 tensors; returns new ``(p, m)``.

    Lion: ``mom_coef`` is beta2 and ``update_coef`` is beta1.  SGD:
    ``mom_coef`` is the momentum and ``update_coef`` is ``1 - dampening``;
    ``m is None`` means momentum-free SGD
    (reference ``flashoptim/optimizers.py:1639-1683`` and ``:1447-1465``).
    """
    if lion:
        assert m is not None
        u = torch.sign(m * update_coef + g * (1.0 - update_coef))
        m = m * mom_coef + g * (1.0 - mom_coef)
        p = p * (1.0 - weight_decay) - u * lr
        return p, m
    if not decoupled and weight_decay != 0.0:
        g = g + p * weight_decay
    if m is None:
        if decoupled and weight_decay != 0.0:
            p = p * (1.0 - weight_decay)
        return p - g * lr, None
    m = m * mom_coef + g * update_coef
    if decoupled and weight_decay != 0.0:
        p = p * (1.0 - weight_decay)
    if nesterov:
        p = p - (g + m * mom_coef) * lr
    else:
        p = p - m * lr
    return p, m


# --------------------------------------------------------------------------- numerics check


def log2_min_expressible_step(
    dtype: torch.dtype, maxabs: float, master_bytewidth: int
) -> float:
    """log2 of the smallest step that still moves a value of magnitude ``maxabs``.

    A step has to exceed 0.49 ULP of the effective master format, which keeps
    the sign and exponent bits of ``dtype`` and widens the mantissa to
    ``max(width(dtype), master_bytewidth)`` bytes
    (reference ``flashoptim/optimizers.py:291-314``).
    """
    master_bits = max(DTYPE_WIDTHS[dtype], master_bytewidth) * 8
    mant = master_bits - 1 - EXPONENT_BITS[dtype] + math.log2(0.49)
    return math.floor(math.log2(maxabs)) - mant
