"""flashoptim_b200: memory-efficient optimizers written for NVIDIA B200 (sm_100a).

Drop-in ``torch.optim.Optimizer`` classes with 8-bit group-quantised states,
24/32-bit master weights kept as bf16/fp16 parameters plus int8/int16
error-correction codes, gradient release, and compressed checkpoints.  The
public names mirror ``flashoptim/__init__.py:3-33`` of the reference.
"""

from .ops.quant import compute_ecc_bits, dequantize, quantize, reconstruct_fp32_param
from .optim import FlashAdam, FlashAdamW, FlashLion, FlashOptimizer, FlashSGD, FlashSGDW, NumericsError
from .utils import GradientReleaseHandle, cast_model, enable_gradient_release

__version__ = "0.1.0"

_OPTIMIZERS = ("FlashOptimizer", "FlashSGD", "FlashSGDW", "FlashAdam", "FlashAdamW", "FlashLion", "NumericsError")
_MODEL_UTILITIES = ("cast_model", "enable_gradient_release", "GradientReleaseHandle")
_TENSOR_FUNCTIONS = ("quantize", "dequantize", "compute_ecc_bits", "reconstruct_fp32_param")
__all__ = [*_OPTIMIZERS, *_MODEL_UTILITIES, *_TENSOR_FUNCTIONS]
