"""FlashSGD / FlashSGDW (parity: ``flashoptim/optimizers.py:1348-1511``, ``:1722-1778``)."""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Iterable, Literal, Optional

import torch

from ..ops import native, oracle
from ..ops.step import MomentumHyper, launch_momentum, launch_momentum_peer
from ._common import err_bytes_of, pack_rows, state_mode, write_back
from .base import FlashOptimizer
from .state import QuantizedTensorSpec


class FlashSGD(FlashOptimizer):
    """SGD with momentum / dampening / Nesterov and L2 regularisation.

    ``m = momentum*m + (1-dampening)*g`` starting from ``m = 0`` (so with
    dampening the first step differs from ``torch.optim.SGD``, which seeds the
    buffer with the raw gradient).  The state ``momentum_buffer`` exists only
    when some group has ``momentum > 0``.  Momentum-free SGD also runs as one
    fused kernel here (the reference handles it in eager PyTorch,
    ``flashoptim/optimizers.py:1447-1465``).
    """

    def __init__(
        self,
        params: Iterable[torch.Tensor],
        lr: float = 0.001,
        momentum: float = 0.0,
        dampening: float = 0.0,
        weight_decay: float = 0.0,
        nesterov: bool = False,
        quantize: bool = True,
        compress_state_dict: bool = False,
        master_weight_bits: Optional[Literal[24, 32]] = 24,
        check_numerics: bool = False,
        fused: bool = True,
    ):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        self._nesterov = nesterov
        self._decoupled = False
        self._decouple_lr = False
        super().__init__(
            params,
            lr=lr,
            defaults={"lr": lr, "momentum": momentum, "dampening": dampening, "weight_decay": weight_decay},
            quantize=quantize,
            compress_state_dict=compress_state_dict,
            master_weight_bits=master_weight_bits,
            check_numerics=check_numerics,
            fused=fused,
        )

    def _quantized_state_spec(self) -> dict[str, QuantizedTensorSpec]:
        if any(g["momentum"] > 0.0 for g in self.param_groups):
            return {"momentum_buffer": QuantizedTensorSpec(signed=True)}
        return {}

    def _hyper(self, hparams: dict[str, Any]) -> MomentumHyper:
        wd = hparams["weight_decay"]
        if self._decoupled:
            wd *= hparams["lr"] / hparams["initial_lr"] if self._decouple_lr else hparams["lr"]
        return MomentumHyper(
            lr=hparams["lr"],
            mom_coef=hparams["momentum"],
            update_coef=1.0 - hparams["dampening"],
            weight_decay=wd,
            lion=False,
            nesterov=self._nesterov,
            decoupled=self._decoupled,
        )

    def _eager_step(self, param, grad, errors, param_state, hparams) -> None:
        h = self._hyper(hparams)
        use_mom = h.mom_coef != 0.0
        m_state = param_state["momentum_buffer"] if use_mom else None
        p32, m32 = oracle.momentum_math(
            oracle.read_param_fp32(param, errors),
            grad.to(torch.float32),
            m_state.materialize().to(torch.float32) if use_mom else None,
            lr=h.lr, mom_coef=h.mom_coef, update_coef=h.update_coef, weight_decay=h.weight_decay,
            decoupled=h.decoupled, nesterov=h.nesterov, lion=False,
        )
        write_back(param, p32, errors, hparams["master_bytewidth"])
        if use_mom:
            m_state.set_data(m32)

    def _fused_step(self, items, hparams, group_index, peer=None) -> None:
        h = self._hyper(hparams)
        key_name = "momentum_buffer" if h.mom_coef != 0.0 else None
        buckets: dict[Any, list] = defaultdict(list)
        for it in items:
            p, _, st = it
            buckets[(p.device, p.dtype, err_bytes_of(st), state_mode(st, key_name))].append(it)
        for (device, dtype, err, mode), bucket in buckets.items():
            keys = ("momentum_buffer",) if mode != native.FO_STATE_NONE else ()
            rows = pack_rows(bucket, keys)
            if peer is None:
                table = self._table((group_index, device, dtype, err, mode, len(bucket)), device)
                launch_momentum(table, rows, dtype, err, mode, h)
            else:
                h.grad_scale = peer.grad_scale
                table = self._table(("peer", peer.key, group_index, dtype, err, mode, len(bucket)), device)
                launch_momentum_peer(table, rows, dtype, err, mode, h, peer.next_args())


class FlashSGDW(FlashSGD):
    """SGD with decoupled weight decay: ``p *= 1 - lr*wd`` (``1 - wd*lr/initial_lr``
    with ``decouple_lr``) instead of adding ``wd*p`` to the gradient."""

    def __init__(
        self,
        params: Iterable[torch.Tensor],
        lr: float = 0.001,
        momentum: float = 0.0,
        dampening: float = 0.0,
        weight_decay: float = 0.0,
        nesterov: bool = False,
        decouple_lr: bool = False,
        quantize: bool = True,
        compress_state_dict: bool = False,
        master_weight_bits: Optional[Literal[24, 32]] = 24,
        check_numerics: bool = False,
        fused: bool = True,
    ):
        super().__init__(
            params,
            lr=lr,
            momentum=momentum,
            dampening=dampening,
            weight_decay=weight_decay,
            nesterov=nesterov,
            quantize=quantize,
            compress_state_dict=compress_state_dict,
            master_weight_bits=master_weight_bits,
            check_numerics=check_numerics,
            fused=fused,
        )
        self._decoupled = True
        self._decouple_lr = decouple_lr
