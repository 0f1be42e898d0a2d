"""Optimizer-state container that is either 8-bit group-quantised or plain.

Parity: ``QuantizedTensorSpec`` (``flashoptim/optimizers.py:70-82``) and
``_MaybeQuantizedTensor`` (``:103-285``).  Differences from the reference, on
purpose: quantisation also works for CPU tensors (through the PyTorch
formulation of the same recipe), so a CPU-only machine can run, save and load
quantised state.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops.quant import dequantize, quantize


@dataclass(frozen=True)
class QuantizedTensorSpec:
    """How one state variable is quantised: sign, sqrt domain, compander."""

    signed: bool = True
    sqrt: bool = False
    softsign: bool = True

    def __post_init__(self) -> None:
        for name in ("signed", "sqrt", "softsign"):
            v = getattr(self, name)
            if not isinstance(v, bool):
                raise ValueError(f"{name} must be bool; got {type(v)}")


class MaybeQuantizedTensor:
    """A state tensor held as (codes, scales) or as a plain tensor in ``storage_dtype``.

    ``state_dict`` / ``load_state_dict`` speak both checkpoint flavours: the
    plain key (a bf16 tensor, loadable by stock optimizers) and the compressed
    pair ``"<name>::quantized"`` + ``"<name>::scales"``.
    """

    __slots__ = ("_data", "_quantized", "_scales", "_try_quantize", "_signed", "_sqrt", "_softsign",
                 "_storage_dtype")

    def __init__(
        self,
        data: Optional[torch.Tensor],
        try_quantize: bool = True,
        signed: bool = True,
        sqrt: bool = False,
        softsign: bool = True,
        storage_dtype: torch.dtype = torch.float32,
    ):
        self._data: Optional[torch.Tensor] = None
        self._quantized: Optional[torch.Tensor] = None
        self._scales: Optional[torch.Tensor] = None
        self._try_quantize = bool(try_quantize)
        self._signed = signed
        self._sqrt = sqrt
        self._softsign = softsign
        self._storage_dtype = storage_dtype
        if data is not None:
            self.set_data(data)

    @classmethod
    def zeros(
        cls,
        like: torch.Tensor,
        try_quantize: bool = True,
        signed: bool = True,
        sqrt: bool = False,
        softsign: bool = True,
        storage_dtype: torch.dtype = torch.float32,
    ) -> "MaybeQuantizedTensor":
        """An all-zero state shaped like ``like`` without running the quantiser: the codes of
        zeros are zeros, and the scale of an all-zero group, ``float16(max(0, 1e-12))``, is zero
        as well, so two memsets give exactly what ``set_data(zeros)`` would."""
        obj = cls(None, try_quantize=try_quantize, signed=signed, sqrt=sqrt, softsign=softsign,
                  storage_dtype=storage_dtype)
        if obj._try_quantize:
            obj._quantized = torch.zeros(like.shape, dtype=torch.int8 if signed else torch.uint8, device=like.device)
            obj._scales = torch.zeros((like.numel() + 31) // 32, dtype=torch.float16, device=like.device)
        else:
            obj._data = torch.zeros(like.shape, dtype=storage_dtype, device=like.device)
        return obj

    # ------------------------------------------------------------------ accessors
    @property
    def data(self) -> torch.Tensor:
        assert self._data is not None
        return self._data

    @property
    def quantized(self) -> torch.Tensor:
        assert self._quantized is not None
        return self._quantized

    @property
    def scales(self) -> torch.Tensor:
        assert self._scales is not None
        return self._scales

    @property
    def spec(self) -> QuantizedTensorSpec:
        return QuantizedTensorSpec(self._signed, self._sqrt, self._softsign)

    def is_quantized(self) -> bool:
        return self._data is None

    @property
    def is_cuda(self) -> bool:
        return self.kernel_tensor.is_cuda

    @property
    def shape(self) -> tuple[int, ...]:
        return tuple(self.kernel_tensor.shape)

    def numel(self) -> int:
        return self.kernel_tensor.numel()

    @property
    def kernel_tensor(self) -> torch.Tensor:
        """The tensor a kernel reads: the codes when quantised, else the data."""
        return self.quantized if self.is_quantized() else self.data

    @property
    def kernel_scales_or_self(self) -> torch.Tensor:
        """The fp16 scales when quantised, else the data tensor as a placeholder."""
        return self.scales if self.is_quantized() else self.data

    def __repr__(self) -> str:
        return (
            f"{self.__class__.__name__} quantized={self.is_quantized()} "
            f"signed={self._signed} shape={self.shape}"
        )

    # ------------------------------------------------------------------ data movement
    def set_data(self, data: torch.Tensor) -> None:
        if self._try_quantize:
            self._data = None
            self._quantized, self._scales = quantize(
                data, signed=self._signed, sqrt=self._sqrt, softsign=self._softsign
            )
        else:
            self._data = data.to(dtype=self._storage_dtype)
            self._quantized = None
            self._scales = None

    def materialize(self) -> torch.Tensor:
        """fp32 values when quantised, else the stored tensor itself."""
        if not self.is_quantized():
            return self.data
        return dequantize(
            self.quantized, self.scales, signed=self._signed, sqrt=self._sqrt, softsign=self._softsign
        )

    # ------------------------------------------------------------------ checkpoint flavours
    @staticmethod
    def _quantized_vals_key(name: str) -> str:
        return f"{name}::quantized"

    @staticmethod
    def _quantized_scales_key(name: str) -> str:
        return f"{name}::scales"

    def state_dict(self, name: str, allow_quantized: bool = False) -> dict[str, torch.Tensor]:
        if self.is_quantized() and allow_quantized:
            return {
                self._quantized_vals_key(name): self.quantized,
                self._quantized_scales_key(name): self.scales,
            }
        return {name: self.materialize().to(dtype=torch.bfloat16)}

    def load_state_dict(self, d: dict[str, torch.Tensor], name: str) -> None:
        d = {k: v for k, v in d.items() if k == name or k.startswith(f"{name}::")}
        if name in d:
            if len(d) != 1:
                raise ValueError(
                    f"a checkpoint holds either '{name}' or its compressed pair, not both; found "
                    f"{sorted(d.keys())}"
                )
            self.set_data(d[name])
            return
        code_dtype = torch.int8 if self._signed else torch.uint8
        self._data = None
        self._quantized = d[self._quantized_vals_key(name)].to(dtype=code_dtype).contiguous()
        self._scales = d[self._quantized_scales_key(name)].to(dtype=torch.float16).contiguous()

    @classmethod
    def from_state_dict(
        cls,
        d: dict[str, torch.Tensor],
        name: str,
        try_quantize: bool = True,
        signed: bool = True,
        sqrt: bool = False,
        softsign: bool = True,
        storage_dtype: torch.dtype = torch.float32,
    ) -> "MaybeQuantizedTensor":
        obj = cls(None, try_quantize=try_quantize, signed=signed, sqrt=sqrt, softsign=softsign,
                  storage_dtype=storage_dtype)
        obj.load_state_dict(d, name)
        return obj
