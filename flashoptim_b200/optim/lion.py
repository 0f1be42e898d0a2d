"""FlashLion (parity: ``flashoptim/optimizers.py:1209-1342``)."""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Iterable, Literal, Optional

import torch

from ..ops import oracle
from ..ops.step import MomentumHyper, launch_momentum, launch_momentum_peer
from ._common import err_bytes_of, pack_rows, state_mode, write_back
from .base import FlashOptimizer
from .state import QuantizedTensorSpec


class FlashLion(FlashOptimizer):
    """Lion with decoupled weight decay; one int8 companded state ``exp_avg``.

    ``u = sign(beta1*m + (1-beta1)*g); m = beta2*m + (1-beta2)*g;
    p = p*(1 - lr*wd) - lr*u`` (``wd*lr/initial_lr`` with ``decouple_lr``).
    """

    def __init__(
        self,
        params: Iterable[torch.Tensor],
        lr: float = 1e-3,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 0,
        decouple_lr: bool = False,
        quantize: bool = True,
        compress_state_dict: bool = False,
        master_weight_bits: Optional[Literal[24, 32]] = 24,
        check_numerics: bool = False,
        fused: bool = True,
    ):
        if not 0.0 <= betas[0] <= 1.0:
            raise ValueError(f"Invalid beta parameter at index 0: {betas[0]}")
        if not 0.0 <= betas[1] <= 1.0:
            raise ValueError(f"Invalid beta parameter at index 1: {betas[1]}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        self._decouple_lr = decouple_lr
        super().__init__(
            params,
            lr=lr,
            defaults={"betas": betas, "weight_decay": weight_decay},
            quantize=quantize,
            compress_state_dict=compress_state_dict,
            master_weight_bits=master_weight_bits,
            check_numerics=check_numerics,
            fused=fused,
        )

    def _quantized_state_spec(self) -> dict[str, QuantizedTensorSpec]:
        return {"exp_avg": QuantizedTensorSpec(signed=True)}

    def _hyper(self, hparams: dict[str, Any]) -> MomentumHyper:
        wd = hparams["weight_decay"]
        wd *= hparams["lr"] / hparams["initial_lr"] if self._decouple_lr else hparams["lr"]
        return MomentumHyper(
            lr=hparams["lr"],
            mom_coef=hparams["betas"][1],
            update_coef=hparams["betas"][0],
            weight_decay=wd,
            lion=True,
        )

    def _eager_step(self, param, grad, errors, param_state, hparams) -> None:
        if errors is not None and errors.dtype not in (torch.int8, torch.int16):
            raise ValueError("Errors needs to be int8 or int16")
        h = self._hyper(hparams)
        m_state = param_state["exp_avg"]
        p32, m32 = oracle.momentum_math(
            oracle.read_param_fp32(param, errors),
            grad.to(torch.float32),
            m_state.materialize().to(torch.float32),
            lr=h.lr, mom_coef=h.mom_coef, update_coef=h.update_coef, weight_decay=h.weight_decay,
            decoupled=True, nesterov=False, lion=True,
        )
        write_back(param, p32, errors, hparams["master_bytewidth"])
        m_state.set_data(m32)

    def _fused_step(self, items, hparams, group_index, peer=None) -> None:
        buckets: dict[Any, list] = defaultdict(list)
        for it in items:
            p, _, st = it
            buckets[(p.device, p.dtype, err_bytes_of(st), state_mode(st, "exp_avg"))].append(it)
        h = self._hyper(hparams)
        for (device, dtype, err, mode), bucket in buckets.items():
            rows = pack_rows(bucket, ("exp_avg",))
            if peer is None:
                table = self._table((group_index, device, dtype, err, mode, len(bucket)), device)
                launch_momentum(table, rows, dtype, err, mode, h)
            else:
                h.grad_scale = peer.grad_scale
                table = self._table(("peer", peer.key, group_index, dtype, err, mode, len(bucket)), device)
                launch_momentum_peer(table, rows, dtype, err, mode, h, peer.next_args())
