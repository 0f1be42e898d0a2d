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
