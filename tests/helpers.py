"""Metrics and tolerances shared by the tests (modelled on the reference's
``test/test_utils.py:247-366``)."""

from __future__ import annotations

import dataclasses

import torch


def nmse(truth: torch.Tensor, approx: torch.Tensor) -> float:
    d = truth.double() - approx.double()
    return float((d * d).mean() / (truth.double() * truth.double()).mean().clamp_min(1e-300))


def cossim(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.flatten().double()
    b = b.flatten().double()
    return float(torch.dot(a, b) / (a.norm() * b.norm()).clamp_min(1e-300))


@dataclasses.dataclass
class Tolerances:
    rtol: float
    atol: float
    min_cossim: float
    max_nmse: float


def get_tolerances(dtype: torch.dtype, quantized: bool) -> Tolerances:
    if quantized:
        if dtype in (torch.bfloat16, torch.float16):
            return Tolerances(1.5e-2, 2e-3, 0.9999, 1e-3)
        return Tolerances(5e-4, 5e-4, 0.99999, 1e-5)
    if dtype in (torch.bfloat16, torch.float16):
        return Tolerances(2e-3, 2e-4, 0.9999, 1e-3)
    return Tolerances(5e-6, 2e-7, 0.99999, 1e-8)


def check_similar(a: torch.Tensor, b: torch.Tensor, tol: Tolerances, name: str = "") -> list[str]:
    errs = []
    a32, b32 = a.float(), b.float()
    if not torch.allclose(a32, b32, rtol=tol.rtol, atol=tol.atol):
        errs.append(f"{name}: not close, max abs diff {(a32 - b32).abs().max().item():.3e}")
    if a.numel() >= 16:
        cs = cossim(a32, b32)
        if cs < tol.min_cossim:
            errs.append(f"{name}: cossim {cs:.6f} < {tol.min_cossim}")
    nm = nmse(a32, b32)
    if nm > tol.max_nmse:
        errs.append(f"{name}: nmse {nm:.2e} > {tol.max_nmse}")
    return errs


def fp32_with_exponent(exponent_field: int, sign: int, mantissas: torch.Tensor) -> torch.Tensor:
    """fp32 values with the given sign bit, biased exponent field (0 = subnormals) and
    23-bit mantissas (an int32 tensor)."""
    bits = mantissas.to(torch.int64) | (exponent_field << 23) | (sign << 31)
    bits = torch.where(bits >= 2**31, bits - 2**32, bits)
    return bits.to(torch.int32).view(torch.float32)


def ecc_invariant_violations(x: torch.Tensor, dtype: torch.dtype, encode, decode, half_ulp_of) -> dict[str, int]:
    """Counts, over the fp32 values ``x``, how often the master-weight split breaks one of
    its invariants (the checks of the reference's ``test/test_ecc_invariants.py``, stated
    on errors in fp32).  ``encode(x, w, master_bytewidth)`` and ``decode(w, codes)`` are the
    implementation under test; ``half_ulp_of(w)`` is half the spacing of ``dtype`` at ``w``."""
    w = x.to(dtype)
    finite = torch.isfinite(w.float())
    x, w = x[finite], w[finite]
    if x.numel() == 0:
        return {}
    base_err = (w.float() - x).abs()
    e8, e16 = encode(x, w, 3), encode(x, w, 4)
    r8, r16 = decode(w, e8), decode(w, e16)
    err8, err16 = (r8 - x).abs(), (r16 - x).abs()
    # one fp32 rounding of the reconstructed value
    ulp32 = torch.exp2(torch.floor(torch.log2(x.abs().clamp_min(2.0**-126))) - 23)
    half_ulp = half_ulp_of(w)
    exact = w.float() == x
    out = {
        "8-bit correction hurts": int((err8 > base_err + ulp32).sum()),
        # the 16-bit grid does not refine the 8-bit one (32767 / 127 is not an integer), so where
        # fp32 resolves finer than a 16-bit code step the wider code may lose by half its own step
        "16-bit worse than 8-bit": int((err16 > err8 + ulp32 + half_ulp * (0.5 / 32767)).sum()),
        "8-bit residual too large": int((err8 > half_ulp * (0.5 / 127 * 1.01) + ulp32).sum()),
        "16-bit residual too large": int((err16 > half_ulp * (0.5 / 32767 * 1.01) + ulp32).sum()),
        "exact value got a correction": int((e8[exact] != 0).sum() + (e16[exact] != 0).sum()),
        "code out of range": int((e8.to(torch.int32).abs() > 127).sum() + (e16.to(torch.int32).abs() > 32767).sum()),
        "non-finite reconstruction": int((~torch.isfinite(r8)).sum() + (~torch.isfinite(r16)).sum()),
    }
    return {k: v for k, v in out.items() if v}
