"""FlashAdam / FlashAdamW (parity: ``flashoptim/optimizers.py:1784-2032``)."""

from __future__ import annotations

from collections import defaultdict
from typing import Any, Iterable, Literal, Optional

import torch

from ..ops import oracle
from ..ops.step import AdamHyper, launch_adam, launch_adam_peer
from ._common import err_bytes_of, pack_rows, write_back
from .base import FlashOptimizer
from .state import QuantizedTensorSpec


class FlashAdam(FlashOptimizer):
    """Adam with L2 regularisation folded into the gradient (``torch.optim.Adam``
    semantics).  States: ``exp_avg`` (int8, companded) and ``exp_avg_sq`` (uint8,
    stored as its square root), ``step`` (CPU fp32 scalar tensor per parameter).

    Args:
        lr, betas, eps, weight_decay: as ``torch.optim.Adam``.
        quantize, compress_state_dict, master_weight_bits, check_numerics, fused:
            see :class:`FlashOptimizer`.
    """

    def __init__(
        self,
        params: Iterable[torch.Tensor],
        lr: float = 1e-3,
        betas: tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 0.0,
        quantize: bool = True,
        compress_state_dict: bool = False,
        master_weight_bits: Optional[Literal[24, 32]] = 24,
        check_numerics: bool = False,
        fused: bool = True,
    ):
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= betas[0] <= 1.0:
            raise ValueError(f"Invalid beta parameter at index 0: {betas[0]}")
        if not 0.0 <= betas[1] <= 1.0:
            raise ValueError(f"Invalid beta parameter at index 1: {betas[1]}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        self._decoupled = False
        self._decouple_lr = False
        super().__init__(
            params,
            lr=lr,
            defaults={"betas": betas, "weight_decay": weight_decay, "eps": eps},
            quantize=quantize,
            compress_state_dict=compress_state_dict,
            master_weight_bits=master_weight_bits,
            check_numerics=check_numerics,
            fused=fused,
        )

    def _quantized_state_spec(self) -> dict[str, QuantizedTensorSpec]:
        return {
            "exp_avg": QuantizedTensorSpec(signed=True, softsign=True),
            "exp_avg_sq": QuantizedTensorSpec(signed=False, sqrt=True, softsign=False),
        }

    def _ensure_state_initialized(self, p: torch.Tensor, hparams: dict[str, Any]) -> None:
        super()._ensure_state_initialized(p, hparams)
        state = self.state[p]
        if "step" not in state:
            # CPU fp32 scalar like torch's own optimizers write to checkpoints
            state["step"] = torch.tensor(0, dtype=torch.float32, device="cpu")

    def _min_step_size_relative_to_lr(self) -> float:
        # |m|/sqrt(v) has no lower bound; assume steps shrink to a tenth of lr
        return 0.1

    def _pre_step(self, param_state: dict[str, Any]) -> None:
        param_state["step"] += 1

    def _pre_step_many(self, param_states: list[dict[str, Any]]) -> None:
        # one call for hundreds of CPU scalars instead of one dispatcher trip each
        torch._foreach_add_([st["step"] for st in param_states], 1.0)

    def _folded_weight_decay(self, hparams: dict[str, Any]) -> float:
        wd = hparams["weight_decay"]
        if self._decoupled:
            wd *= hparams["lr"] / hparams["initial_lr"] if self._decouple_lr else hparams["lr"]
        return wd

    def _eager_step(self, param, grad, errors, param_state, hparams) -> None:
        m_state, v_state = param_state["exp_avg"], param_state["exp_avg_sq"]
        p32, m32, v32 = oracle.adam_math(
            oracle.read_param_fp32(param, errors),
            grad.to(torch.float32),
            m_state.materialize().to(torch.float32),
            v_state.materialize().to(torch.float32),
            lr=hparams["lr"],
            beta1=hparams["betas"][0],
            beta2=hparams["betas"][1],
            eps=hparams["eps"],
            weight_decay=self._folded_weight_decay(hparams),
            decoupled=self._decoupled,
            step=int(param_state["step"].item()),
        )
        write_back(param, p32, errors, hparams["master_bytewidth"])
        m_state.set_data(m32)
        v_state.set_data(v32)

    def _fused_step(self, items, hparams, group_index, peer=None) -> None:
        buckets: dict[Any, list] = defaultdict(list)
        steps = torch.stack([it[2]["step"] for it in items]).tolist() if len(items) > 1 else [
            items[0][2]["step"].item()]
        for it, step in zip(items, steps):
            p, _, st = it
            key = (p.device, p.dtype, err_bytes_of(st), st["exp_avg"].is_quantized(), int(step))
            buckets[key].append(it)
        for key, bucket in buckets.items():
            device, dtype, err, quantized, step = key
            hyper = AdamHyper(
                lr=hparams["lr"],
                beta1=hparams["betas"][0],
                beta2=hparams["betas"][1],
                eps=hparams["eps"],
                weight_decay=self._folded_weight_decay(hparams),
                step=step,
                decoupled=self._decoupled,
            )
            rows = pack_rows(bucket, ("exp_avg", "exp_avg_sq"))
            if peer is None:
                table = self._table((group_index, device, dtype, err, quantized, len(bucket)), device)
                launch_adam(table, rows, dtype, err, quantized, hyper)
            else:
                hyper.grad_scale = peer.grad_scale
                table = self._table(("peer", peer.key, group_index, dtype, err, quantized, len(bucket)), device)
                launch_adam_peer(table, rows, dtype, err, quantized, hyper, peer.next_args())


class FlashAdamW(FlashAdam):
    """AdamW: ``p *= 1 - lr*wd`` (or ``1 - wd*lr/initial_lr`` with ``decouple_lr``)
    applied to the parameter, not the gradient.  Equivalent to
    ``torch.optim.AdamW`` for the same ``lr`` / ``weight_decay``.
    """

    def __init__(
        self,
        params: Iterable[torch.Tensor],
        lr: float = 1e-3,
        betas: tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 1e-2,
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
            betas=betas,
            eps=eps,
            weight_decay=weight_decay,
            quantize=quantize,
            compress_state_dict=compress_state_dict,
            master_weight_bits=master_weight_bits,
            check_numerics=check_numerics,
            fused=fused,
        )
        self._decoupled = True
        self._decouple_lr = decouple_lr
