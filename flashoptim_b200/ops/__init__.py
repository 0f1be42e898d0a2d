"""Numerics (oracle), native kernel bindings and launch wrappers."""

from .quant import compute_ecc_bits, dequantize, maxabs, quantize, reconstruct_fp32_param

__all__ = ["quantize", "dequantize", "reconstruct_fp32_param", "compute_ecc_bits", "maxabs"]
