"""Optimizer classes."""

from .adam import FlashAdam, FlashAdamW
from .base import FlashOptimizer, NumericsError
from .lion import FlashLion
from .sgd import FlashSGD, FlashSGDW
from .state import MaybeQuantizedTensor, QuantizedTensorSpec

__all__ = [
    "FlashOptimizer", "NumericsError", "FlashAdam", "FlashAdamW", "FlashLion", "FlashSGD",
    "FlashSGDW", "MaybeQuantizedTensor", "QuantizedTensorSpec",
]
