"""Gradient release: update each parameter the moment its gradient is complete
and free the gradient right away, so a whole model's gradients never coexist.

Parity: ``flashoptim/optimizers.py:2998-3138``.
"""

from __future__ import annotations

import weakref
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from ..optim.base import FlashOptimizer

PreStep = Callable[[torch.Tensor, dict[str, Any]], bool]


@dataclass
class GradientReleaseHandle:
    """Returned by :func:`enable_gradient_release`; ``remove()`` detaches the hooks
    and gives ``step()`` / ``zero_grad()`` their normal meaning back."""

    _hooks: list
    _optimizer: FlashOptimizer

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        self._optimizer._gradient_release = False

    @property
    def active(self) -> bool:
        return len(self._hooks) > 0


def _make_hook(p: torch.Tensor, group: dict[str, Any], optimizer: FlashOptimizer,
               pre_step: Optional[PreStep]) -> Callable[[torch.Tensor], None]:
    weak_opt = weakref.ref(optimizer)

    def hook(_p: torch.Tensor) -> None:
        opt = weak_opt()
        if opt is None or p.grad is None:
            return
        if pre_step is not None and not pre_step(p, group):
            return
        opt.step_param(p, group)
        p.grad = None

    return hook


def enable_gradient_release(
    model: torch.nn.Module,
    optimizer: FlashOptimizer,
    *,
    grad_scaler: Optional["torch.amp.GradScaler"] = None,
    pre_step: Optional[PreStep] = None,
) -> GradientReleaseHandle:
    """Step every parameter from a post-accumulate-grad hook and drop its gradient.

    While active, ``optimizer.step()`` and ``optimizer.zero_grad()`` warn and do
    nothing.  Works on a single GPU and under FSDP2 (``fully_shard``), where the
    hook fires after the reduce-scatter of each parameter group, on FSDP's
    reduce-scatter stream.  Incompatible with gradient accumulation, global
    gradient clipping and ``GradScaler``.

    Args:
        model: module whose parameters ``optimizer`` owns.
        optimizer: a :class:`FlashOptimizer`.
        grad_scaler: reserved; anything but ``None`` raises ``NotImplementedError``.
        pre_step: ``(param, group) -> bool``; returning False skips that update
            (the gradient is then kept).

    Raises:
        TypeError: ``model`` is wrapped in DDP or FSDP1.
        NotImplementedError: ``grad_scaler`` was given.
    """
    if grad_scaler is not None:
        raise NotImplementedError(
            "gradient release cannot be combined with a GradScaler: the scaler decides whether to "
            "skip a step only after it has seen every gradient, and by then the hooks have updated "
            "the parameters. Pass grad_scaler=None (bf16 training needs no loss scaling)."
        )
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP1
    from torch.nn.parallel import DistributedDataParallel as DDP

    if isinstance(model, FSDP1):
        raise TypeError(
            "the model is wrapped in FullyShardedDataParallel (FSDP1), whose flat parameters give "
            "gradient hooks nothing to attach to; shard it with FSDP2 (torch.distributed.fsdp."
            "fully_shard) to use gradient release."
        )
    if isinstance(model, DDP):
        # The reducer copies its bucket back into p.grad after the comm hook's future
        # resolves and no Python hook runs after that, so the gradient cannot be freed.
        raise TypeError(
            "the model is wrapped in DistributedDataParallel: its reducer writes the averaged bucket "
            "back into p.grad after every Python hook has run, so a gradient cannot be consumed and "
            "freed during backward. Use optimizer.step() with DDP, or fuse_ddp_allreduce()."
        )

    group_of = {id(p): g for g in optimizer.param_groups for p in g["params"]}
    hooks: list = []
    # model.parameters() de-duplicates tied weights, and a post-accumulate hook fires once
    # per backward after every contribution has been summed, so tied weights step once.
    for p in model.parameters():
        if not p.requires_grad:
            continue
        hooks.append(
            p.register_post_accumulate_grad_hook(_make_hook(p, group_of[id(p)], optimizer, pre_step))
        )
    optimizer._gradient_release = True
    return GradientReleaseHandle(_hooks=hooks, _optimizer=optimizer)
