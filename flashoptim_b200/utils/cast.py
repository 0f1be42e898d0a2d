"""``cast_model``: put a model's parameters and float buffers into a narrow dtype.

Parity: ``flashoptim/optimizers.py:2035-2200``.
"""

from __future__ import annotations

from fnmatch import fnmatch
from typing import Any, Optional, Sequence, Union

import torch
import torch.nn as nn

LayerSpec = Union[str, nn.Module]

# Norms that keep running statistics stay in fp32 under ``selective=True``;
# LayerNorm / RMSNorm / GroupNorm reduce in fp32 inside their kernels and are cast.
_STATEFUL_NORMS = (
    nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.SyncBatchNorm,
    nn.InstanceNorm1d, nn.InstanceNorm2d, nn.InstanceNorm3d,
)


def _matches(name: str, module: nn.Module, specs: Sequence[LayerSpec]) -> bool:
    for spec in specs:
        if isinstance(spec, nn.Module):
            if module is spec:
                return True
        elif fnmatch(name, spec):
            return True
    return False


def _inputs_to_fp32(module: nn.Module, args: tuple[Any, ...]) -> tuple[Any, ...]:
    return tuple(
        a.to(torch.float32) if isinstance(a, torch.Tensor) and a.is_floating_point() else a
        for a in args
    )


def _make_output_recast(dtype: torch.dtype):
    def recast(module: nn.Module, inputs: tuple[Any, ...], output: Any) -> Any:
        def conv(o):
            return o.to(dtype) if isinstance(o, torch.Tensor) and o.is_floating_point() else o

        if isinstance(output, torch.Tensor):
            return conv(output)
        if isinstance(output, tuple):
            return tuple(conv(o) for o in output)
        return output

    return recast


def cast_model(
    model: nn.Module,
    dtype: torch.dtype = torch.bfloat16,
    selective: bool = True,
    full_precision_layers: Optional[list[LayerSpec]] = None,
    full_precision_recast_layers: Optional[list[LayerSpec]] = None,
) -> None:
    """Cast parameters and floating-point buffers of ``model`` to ``dtype`` in place.

    Args:
        model: module to convert.
        dtype: target dtype (default bf16).
        selective: keep BatchNorm / InstanceNorm modules (running statistics) in fp32.
        full_precision_layers: modules kept in fp32 whose *output stays fp32*
            (e.g. ``"lm_head"``); matched by ``fnmatch`` on the full dotted module
            name (``"head"`` matches only a top-level ``head``; use ``"*.head"`` for
            nested ones) or by module identity.  Their floating positional
            inputs are cast to fp32 by a forward pre-hook.
        full_precision_recast_layers: same, plus a forward hook that casts
            tensor / tuple outputs back to ``dtype`` (layers in the middle of a
            narrow-precision network).

    Tied parameters stay tied; integer buffers are untouched.
    """
    keep = list(full_precision_layers or [])
    recast = list(full_precision_recast_layers or [])
    specs = keep + recast

    fp32_params: set[str] = set()
    fp32_buffers: set[str] = set()
    if specs:
        for mod_name, mod in model.named_modules():
            if _matches(mod_name, mod, specs):
                prefix = f"{mod_name}." if mod_name else ""
                fp32_params.update(prefix + n for n, _ in mod.named_parameters())
                fp32_buffers.update(prefix + n for n, _ in mod.named_buffers())

    name_of_param = {p: n for n, p in model.named_parameters()}
    name_of_buffer = {b: n for n, b in model.named_buffers()}

    # Tensors that alias each other (tied weights: one Parameter reachable from two modules,
    # or two Parameters over one storage) are found BEFORE anything is converted, while every
    # storage is still alive and an address therefore identifies it.  Looking addresses up
    # during the conversion would not be safe: a converted tensor may be placed where an
    # already released fp32 tensor used to live.  (The reference keys a map by ``data_ptr()``
    # while it converts, ``flashoptim/optimizers.py:2145-2185``.)
    aliases: dict[Any, list[torch.Tensor]] = {}
    visited: set[int] = set()

    def collect(t: torch.Tensor) -> None:
        if id(t) in visited:
            return
        visited.add(id(t))
        if t.device.type == "meta" or t.numel() == 0:
            key: Any = ("object", id(t))  # no storage to compare
        else:
            key = (t.data_ptr(), tuple(t.shape), tuple(t.stride()), t.dtype, str(t.device))
        aliases.setdefault(key, []).append(t)

    for module in model.modules():
        if selective and isinstance(module, _STATEFUL_NORMS):
            continue
        for param in module.parameters(recurse=False):
            if name_of_param.get(param, "") not in fp32_params:
                collect(param)
        for buf in module.buffers(recurse=False):
            if name_of_buffer.get(buf, "") not in fp32_buffers and buf.is_floating_point():
                collect(buf)

    for group in aliases.values():
        cast = group[0].data.to(dtype=dtype)
        for t in group:
            t.data = cast

    if specs:
        for name, module in model.named_modules():
            is_keep = _matches(name, module, keep)
            is_recast = _matches(name, module, recast)
            if (is_keep or is_recast) and not getattr(module, "_has_fp32_input_hook", False):
                module.register_forward_pre_hook(_inputs_to_fp32)
                if is_recast:
                    module.register_forward_hook(_make_output_recast(dtype))
                module._has_fp32_input_hook = True
