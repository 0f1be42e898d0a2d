"""``FlashOptimizer``: the runtime shared by every optimizer of this library.

What it provides (parity with ``flashoptim/optimizers.py:317-1203``):

* 8-bit group-quantised optimizer states (``quantize=True``),
* master weights wider than the parameters through int8/int16 error-correction
  codes kept in ``state[p]["error_bits"]`` (``master_weight_bits`` 24 / 32),
* a checkpoint format that stock PyTorch optimizers can read
  (bf16 moments) or a compressed one (``compress_state_dict=True``: int8 codes
  + fp16 scales), both readable by the reference and vice versa,
* per-parameter stepping (``step_param``) for gradient release,
* DTensor (FSDP2) parameters: kernels and state work on the local shard, state
  is re-wrapped as DTensors for ``torch.distributed.checkpoint``.

What differs by design:

* ``step()`` is one kernel launch per (parameter group, dtype/ECC/quantisation
  combination) instead of one per tensor: all tensors of a bucket are described
  by a segment table and updated by a persistent multi-tensor sm_100a kernel.
* Without a GPU everything still works: CPU tensors take the PyTorch
  formulation of the same numerics (the reference raises
  ``NotImplementedError``, ``flashoptim/optimizers.py:484-493``).
* Checkpoints reload without a detour through the parameter dtype: moments,
  codes and fp16 scales are shielded from ``torch.optim.Optimizer.load_state_dict``'s
  cast, so the compressed flavour round-trips bit-exactly.
"""

from __future__ import annotations

import abc
import math
import os
import warnings
from typing import Any, Callable, Iterable, Literal, Optional, cast

import torch
import torch.nn as nn

from ..ops import oracle
from ..ops.quant import compute_ecc_bits, maxabs, reconstruct_fp32_param
from ..ops.step import SegmentTable, poll_kernel_status
from .state import MaybeQuantizedTensor, QuantizedTensorSpec

_VALID_MASTER_WEIGHT_BITS = (None, 24, 32)
_BITS_TO_BYTES = {None: 0, 24: 3, 32: 4}


class NumericsError(RuntimeError):
    """The learning rate is too small to move the largest weights at the
    current parameter dtype and master-weight width."""


class _Shielded:
    """Carries a tensor through ``Optimizer.load_state_dict`` untouched.

    The base class casts every state tensor to the parameter dtype
    (``torch/optim/optimizer.py``, ``_process_value_according_to_param_policy``),
    which would round fp16 scales to bf16.  Non-tensor values pass through.
    """

    __slots__ = ("tensor",)

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor


def local_tensor(t: torch.Tensor) -> torch.Tensor:
    """The local shard of a DTensor (shares storage), or ``t`` itself."""
    lt = getattr(t, "_local_tensor", None)
    if lt is not None:
        return lt
    if hasattr(t, "to_local"):
        return t.to_local()
    return t


class FlashOptimizer(torch.optim.Optimizer, abc.ABC):
    """Base class: quantised states, ECC master weights, fused multi-tensor steps.

    Args:
        params: iterable of parameters or param-group dicts.
        lr: learning rate.
        quantize: keep optimizer states as int8/uint8 codes + one fp16 scale
            per 32 elements (8.5 bits per element instead of 32).
        compress_state_dict: write the codes and scales to ``state_dict()``
            instead of bf16 tensors.  Requires ``quantize=True``.
        master_weight_bits: 24 or 32 adds an int8 / int16 correction tensor per
            bf16/fp16 parameter so updates accumulate at that precision; None
            trains at the parameter precision.
        check_numerics: raise :class:`NumericsError` when ``lr`` cannot move the
            largest weight of a tensor (uses a cached ``max|w|``; refresh with
            :meth:`recompute_param_stats`).
        fused: CUDA parameters are updated by the fused sm_100a kernels.  With
            ``fused=False`` the arithmetic runs as eager PyTorch ops (debugging).

    Raises:
        ValueError: invalid hyper-parameters, or ``master_weight_bits`` set while
            every parameter is fp32 (no effect; override with the environment
            variable ``FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS``).
    """

    def __init__(
        self,
        params: Iterable[torch.Tensor],
        lr: float = 1e-3,
        quantize: bool = True,
        compress_state_dict: bool = False,
        master_weight_bits: Optional[Literal[24, 32]] = 24,
        check_numerics: bool = False,
        fused: bool = True,
        defaults: Optional[dict[str, Any]] = None,
    ):
        if compress_state_dict and not quantize:
            raise ValueError("compress_state_dict=True requires quantize=True")
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if master_weight_bits not in _VALID_MASTER_WEIGHT_BITS:
            raise ValueError(
                f"Master weight bits {master_weight_bits} invalid; must be one of "
                f"{_VALID_MASTER_WEIGHT_BITS}"
            )
        master_bytewidth = _BITS_TO_BYTES[master_weight_bits]
        self._fused = fused
        self._quantize = quantize
        self._master_bytewidth = master_bytewidth
        self._compress_state_dict = compress_state_dict
        self._check_numerics = check_numerics
        self._gradient_release = False
        # per-parameter data that must not reach state_dict(), keyed by id(param)
        self._transient_state: dict[int, dict[str, Any]] = {}
        # device segment tables of the fused launches, keyed by bucket
        self._tables: dict[Any, SegmentTable] = {}
        # parameters already updated during this backward by a kernel fused with the
        # gradient collective (see flashoptim_b200.parallel); the next step()/step_param()
        # skips them once
        self._peer_stepped: set[int] = set()
        self._post_step_callbacks: list[Callable[[], None]] = []
        # called with the parameters that a local (not collective-fused) update changed
        self._local_update_listeners: list[Callable[[list[torch.Tensor]], None]] = []

        defaults = dict(defaults or {})
        defaults.update({"lr": lr, "master_bytewidth": master_bytewidth, "quantize": quantize})
        super().__init__(params, defaults=defaults)

        all_params = [p for g in self.param_groups for p in g["params"]]
        if master_weight_bits is not None and not os.environ.get(
            "FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS"
        ):
            if all(p.dtype == torch.float32 for p in all_params):
                raise ValueError(
                    f"every parameter is float32, so master_weight_bits={master_weight_bits} would add "
                    "nothing: correction codes exist only for bf16/fp16 parameters. Pass "
                    "master_weight_bits=None (or set FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS=1 "
                    "to construct the optimizer anyway)."
                )
        if master_weight_bits is None and any(p.dtype != torch.float32 for p in all_params):
            warnings.warn(
                "bf16/fp16 parameters are being trained without master weights "
                "(master_weight_bits=None): every update is rounded to the parameter dtype and small "
                "updates are lost. master_weight_bits=24 adds one byte per parameter and keeps them.",
                stacklevel=3,
            )

    def add_param_group(self, param_group: dict[str, Any]) -> None:
        # initial_lr is each group's own learning rate at creation (the reference
        # stamps the constructor's lr on every group, flashoptim/optimizers.py:502-509,
        # which skews decouple_lr for groups with their own lr)
        super().add_param_group(param_group)
        group = self.param_groups[-1]
        group.setdefault("initial_lr", group["lr"])

    # ------------------------------------------------------------------ introspection
    def __repr__(self) -> str:
        lines = [f"{self.__class__.__name__} (", "FlashOptim Config"]
        cfg = {
            "fused": self._fused,
            "quantize": self._quantize,
            "master_bytewidth": self._master_bytewidth,
            "compress_state_dict": self._compress_state_dict,
            "check_numerics": self._check_numerics,
            "gradient_release": self._gradient_release,
        }
        lines += [f"    {k}: {v}" for k, v in cfg.items()]
        for i, group in enumerate(self.param_groups):
            lines += ["", f"Parameter Group {i}"]
            lines += [f"    {k}: {group[k]}" for k in sorted(group) if k != "params"]
        return "\n".join(lines) + "\n)"

    # ------------------------------------------------------------------ subclass hooks
    @abc.abstractmethod
    def _quantized_state_spec(self) -> dict[str, QuantizedTensorSpec]:
        """Names and quantisation recipes of the per-parameter state tensors."""

    @abc.abstractmethod
    def _eager_step(
        self,
        param: torch.Tensor,
        grad: torch.Tensor,
        errors: Optional[torch.Tensor],
        param_state: dict[str, Any],
        hparams: dict[str, Any],
    ) -> None:
        """Update one (local) tensor with eager PyTorch ops (CPU, ``fused=False``)."""

    @abc.abstractmethod
    def _fused_step(
        self,
        items: list[tuple[torch.Tensor, Any, dict[str, Any]]],
        hparams: dict[str, Any],
        group_index: int,
        peer: Any = None,
    ) -> None:
        """Update a list of (local param, local grad, state) on CUDA with fused kernels.

        With ``peer`` (a :class:`flashoptim_b200.parallel.symm.PeerGradients`) the
        gradient entries are byte offsets into the ranks' symmetric buffers and the
        kernels average them over NVLink while updating."""

    def _initial_value_for_state_var(self, param: torch.Tensor, key: str) -> torch.Tensor:
        del key
        return torch.zeros_like(param)

    def _min_step_size_relative_to_lr(self) -> float:
        return 1.0  # sign-based updates (Lion) move every weight by lr

    def _pre_step(self, param_state: dict[str, Any]) -> None:
        """Called once per parameter right before it is updated."""

    def _pre_step_many(self, param_states: list[dict[str, Any]]) -> None:
        """Same for all parameters of one fused launch (override to batch the work)."""
        for st in param_states:
            self._pre_step(st)

    # ------------------------------------------------------------------ DTensor helpers
    @staticmethod
    def _get_local_tensor(tensor: torch.Tensor) -> torch.Tensor:
        return local_tensor(tensor)

    @staticmethod
    def _wrap_state_as_dtensor(state: dict[str, Any], param: torch.Tensor) -> None:
        """Give every >=1-D state tensor the mesh / placements of ``param`` so that
        ``torch.distributed.checkpoint`` treats it as the shard it is
        (``flashoptim/optimizers.py:618-654``)."""
        if not hasattr(param, "device_mesh"):
            return
        from torch.distributed.tensor import DTensor

        mesh, placements = param.device_mesh, param.placements
        for mesh_dim, placement in enumerate(placements):
            if hasattr(placement, "dim"):
                size = mesh.size(mesh_dim)
                if param.shape[placement.dim] % size != 0:
                    raise ValueError(
                        f"a parameter of shape {tuple(param.shape)} is split over {size} ranks along "
                        f"dimension {placement.dim}, which {size} does not divide: its optimizer state "
                        "cannot be described as an even DTensor shard for torch.distributed.checkpoint. "
                        f"Make shape[{placement.dim}] a multiple of {size} (pad or reshape)."
                    )
        for key, val in state.items():
            if isinstance(val, torch.Tensor) and not isinstance(val, DTensor) and val.dim() > 0:
                state[key] = DTensor.from_local(val, mesh, placements)

    # ------------------------------------------------------------------ numerics check
    def _recompute_stats_for_param(self, p: torch.Tensor) -> None:
        local = local_tensor(p.detach())
        value = maxabs(local) if local.numel() else 0.0
        if hasattr(p, "device_mesh"):
            import torch.distributed as dist

            t = torch.tensor([value], dtype=torch.float32, device=local.device)
            mesh = p.device_mesh
            for dim in range(mesh.ndim):
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=mesh.get_group(dim))
            value = float(t.item())
        self._transient_state.setdefault(id(p), {})["maxabs"] = value

    def recompute_param_stats(self) -> None:
        """Refresh the cached ``max|w|`` of every parameter (one sync each)."""
        for group in self.param_groups:
            for p in group["params"]:
                self._recompute_stats_for_param(p)

    def _check_param_numerics(self, p: torch.Tensor, lr: float, master_bytewidth: int) -> None:
        if lr == 0.0:
            return
        mx = self._transient_state.get(id(p), {}).get("maxabs", 0)
        if mx <= 0 or not math.isfinite(mx):
            return
        need = oracle.log2_min_expressible_step(p.dtype, mx, master_bytewidth)
        have = math.log2(lr * self._min_step_size_relative_to_lr())
        if need > have:
            bits = max(oracle.DTYPE_WIDTHS[p.dtype], master_bytewidth) * 8
            raise NumericsError(
                f"lr={lr:.3g} is too small for this tensor: its largest weight is {mx:.5g} in "
                f"{p.dtype} with {bits}-bit master weights, where the smallest representable change "
                f"is about {2**need:.5g}, but a step moves a weight by about {2**have:.5g}. Raise the "
                "learning rate, use master_weight_bits=32, or scale the weights down; "
                "check_numerics=False switches this test off. The weight statistics are cached: "
                "after loading a checkpoint (or from time to time) recompute_param_stats() refreshes them."
            )

    # ------------------------------------------------------------------ state creation
    def _ensure_state_initialized(self, p: torch.Tensor, hparams: dict[str, Any]) -> None:
        if self._check_numerics and self._transient_state.get(id(p), {}).get("maxabs") is None:
            self._recompute_stats_for_param(p)
        state = self.state[p]
        ready = self.__dict__.setdefault("_state_ready", set())
        if state and id(p) in ready:
            return  # created (or loaded) earlier; an emptied state is rebuilt below
        ready.add(id(p))
        p_local = local_tensor(p)
        quantize = hparams.get("quantize", self._quantize)
        # states start at zero unless a subclass says otherwise; zero states are two memsets,
        # not a pass of the quantiser over a tensor of zeros
        zero_init = type(self)._initial_value_for_state_var is FlashOptimizer._initial_value_for_state_var
        for key, spec in self._quantized_state_spec().items():
            if key not in state:
                kw = dict(try_quantize=quantize, signed=spec.signed, sqrt=spec.sqrt, softsign=spec.softsign,
                          storage_dtype=p_local.dtype)
                if zero_init:
                    state[key] = MaybeQuantizedTensor.zeros(p_local.detach(), **kw)
                else:
                    state[key] = MaybeQuantizedTensor(self._initial_value_for_state_var(p_local.detach(), key), **kw)
        err_bytes = hparams["master_bytewidth"] - oracle.DTYPE_WIDTHS[p.dtype]
        if state.get("error_bits") is None and err_bytes > 0:
            state["error_bits"] = torch.zeros_like(
                p_local, dtype=torch.int8 if err_bytes == 1 else torch.int16,
                memory_format=torch.contiguous_format,
            )

    # ------------------------------------------------------------------ stepping
    def _find_group(self, p: torch.Tensor) -> dict[str, Any]:
        for group in self.param_groups:
            if any(q is p for q in group["params"]):
                return group
        raise ValueError(f"Parameter {p.shape} {p.dtype} not managed by this optimizer.")

    def _group_index_of_params(self) -> dict[int, int]:
        """``id(param) -> index of its param group``, rebuilt only when the groups changed
        (the collective-fused paths look parameters up once per bucket or FSDP group)."""
        sig = tuple((id(g["params"]), len(g["params"])) for g in self.param_groups)
        cache = self.__dict__.get("_index_cache")
        if cache is None or cache[0] != sig:
            cache = (sig, {id(p): gi for gi, g in enumerate(self.param_groups) for p in g["params"]})
            self.__dict__["_index_cache"] = cache
        return cache[1]

    def _group_index(self, group: dict[str, Any]) -> int:
        for i, g in enumerate(self.param_groups):
            if g is group:
                return i
        return -1

    def _step_group(self, params: list[torch.Tensor], group: dict[str, Any], group_index: int) -> None:
        """Update ``params`` (all in ``group``).  State is created for every one of
        them; those without a gradient are otherwise left alone."""
        fused_items: list[tuple[torch.Tensor, torch.Tensor, dict[str, Any]]] = []
        updated: list[torch.Tensor] = []
        for p in params:
            self._ensure_state_initialized(p, group)
            if self._peer_stepped and id(p) in self._peer_stepped:
                self._peer_stepped.discard(id(p))  # updated inside the collective already
                continue
            # zero-sized shards and frozen parameters keep their (empty) state: DCP
            # expects a state entry for every parameter of every group
            if p.numel() < 1 or not p.requires_grad or p.grad is None:
                continue
            if self._check_numerics:
                self._check_param_numerics(p, group["lr"], group["master_bytewidth"])
            state = self.state[p]
            p_local = local_tensor(p)
            g_local = local_tensor(p.grad)
            if p_local.numel() < 1:
                continue
            updated.append(p)
            if p_local.is_cuda and self._fused:
                if not p_local.is_contiguous():
                    raise RuntimeError(
                        f"the fused kernels need a contiguous parameter; got shape {tuple(p_local.shape)} "
                        f"with strides {p_local.stride()}. Make it contiguous or construct the optimizer "
                        "with fused=False."
                    )
                if not g_local.is_contiguous():
                    raise RuntimeError(
                        f"the fused kernels need a contiguous gradient; got shape {tuple(g_local.shape)} "
                        f"with strides {g_local.stride()}. Construct the optimizer with fused=False for "
                        "such gradients."
                    )
                if g_local.dtype != p_local.dtype:
                    g_local = g_local.to(p_local.dtype)
                fused_items.append((p_local, g_local, state))
            else:
                self._pre_step(state)
                self._eager_step(p_local, g_local, state.get("error_bits"), state, group)
        if fused_items:
            self._pre_step_many([it[2] for it in fused_items])
            self._fused_step(fused_items, group, group_index)
        if updated and self._local_update_listeners:
            for fn in self._local_update_listeners:
                fn(updated)

    @torch.no_grad()
    def step_param(self, p: torch.Tensor, group: Optional[dict[str, Any]] = None) -> None:
        """Update one parameter from its ``.grad`` (used by gradient-release hooks).

        Raises:
            RuntimeError: fused path and the parameter or gradient is not contiguous.
            NumericsError: ``check_numerics=True`` and ``lr`` is too small.
        """
        if group is None:
            group = self._find_group(p)
        self._step_group([p], group, self._group_index(group))

    @torch.no_grad()
    def step(self, closure: Optional[Callable] = None) -> Optional[torch.Tensor]:
        if self._gradient_release:
            warnings.warn(
                "gradient release is active: the gradient hooks already update the parameters during "
                "backward, so optimizer.step() does nothing.",
                stacklevel=2,
            )
            return None
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            self._step_group(group["params"], group, gi)
        for fn in self._post_step_callbacks:
            fn()
        if self._fused and torch.cuda.is_available():
            # a bounded wait that ran out inside a step kernel means part of an update is
            # missing; reported here without waiting for the device, one or two steps late
            # (ops.step.check_kernel_status() gives the current answer, e.g. before a checkpoint)
            poll_kernel_status()
        return loss

    def _refuse_second_fused_update(self, p: torch.Tensor) -> None:
        """A collective-fused update is the optimizer step of that backward pass.  A second
        synchronised backward before ``step()`` / ``step_param()`` has acknowledged the first
        would update twice where the plain path accumulates and steps once."""
        if id(p) in self._peer_stepped:
            raise RuntimeError(
                "a parameter was updated inside the gradient collective twice without optimizer.step() in "
                "between; accumulate gradients without synchronisation (DDP no_sync(), FSDP2 "
                "set_requires_gradient_sync(False)) and synchronise only the last backward pass"
            )

    @torch.no_grad()
    def step_from_peers(self, params: list[torch.Tensor], peer: Any) -> None:
        """Update ``params`` from gradients that still sit, unreduced, in every rank's
        symmetric buffer (``peer.offsets[id(local tensor)]`` = byte offset of each one).

        The launches run on the current stream.  Each parameter is marked so that the
        following ``step()`` / ``step_param()`` leaves it alone once.
        """
        by_group: dict[int, list[torch.Tensor]] = {}
        index_of = self._group_index_of_params()
        for p in params:
            by_group.setdefault(index_of[id(p)], []).append(p)
        for gi, plist in by_group.items():
            group = self.param_groups[gi]
            items = []
            for p in plist:
                self._ensure_state_initialized(p, group)
                p_local = local_tensor(p)
                if p_local.numel() < 1 or not p.requires_grad:
                    continue
                self._refuse_second_fused_update(p)
                if not (p_local.is_cuda and p_local.is_contiguous()):
                    raise RuntimeError("steps fused with the collective need contiguous CUDA parameters")
                if self._check_numerics:
                    self._check_param_numerics(p, group["lr"], group["master_bytewidth"])
                items.append((p_local, int(peer.offsets[id(p_local)]), self.state[p]))
                self._peer_stepped.add(id(p))
            if items:
                self._pre_step_many([it[2] for it in items])
                self._fused_step(items, group, gi, peer=peer)

    @torch.no_grad()
    def step_with_grads(self, params: list[torch.Tensor], grads: list[torch.Tensor]) -> None:
        """Update ``params`` from explicitly given (already reduced) gradient tensors
        instead of ``.grad``, with the fused kernels on the current stream, and mark them
        so that the following ``step()`` / ``step_param()`` leaves them alone once."""
        index_of = self._group_index_of_params()
        by_group: dict[int, list] = {}
        for p, g in zip(params, grads):
            by_group.setdefault(index_of[id(p)], []).append((p, g))
        for gi, pairs in by_group.items():
            group = self.param_groups[gi]
            items = []
            for p, g in pairs:
                self._ensure_state_initialized(p, group)
                p_local = local_tensor(p)
                if p_local.numel() < 1 or not p.requires_grad:
                    continue
                self._refuse_second_fused_update(p)
                if not (p_local.is_cuda and p_local.is_contiguous() and g.is_contiguous()
                        and g.dtype == p_local.dtype and g.numel() == p_local.numel()):
                    raise RuntimeError("step_with_grads needs contiguous CUDA tensors of the parameter's dtype")
                if self._check_numerics:
                    self._check_param_numerics(p, group["lr"], group["master_bytewidth"])
                items.append((p_local, g, self.state[p]))
                self._peer_stepped.add(id(p))
            if items:
                self._pre_step_many([it[2] for it in items])
                self._fused_step(items, group, gi)

    def zero_grad(self, set_to_none: bool = True) -> None:
        if self._gradient_release:
            warnings.warn(
                "gradient release is active: each gradient is freed by its hook right after the "
                "update, so optimizer.zero_grad() does nothing.",
                stacklevel=2,
            )
            return
        super().zero_grad(set_to_none=set_to_none)

    def _table(self, key: Any, device: torch.device) -> SegmentTable:
        t = self._tables.get(key)
        if t is None:
            t = self._tables[key] = SegmentTable(device)
        return t

    # ------------------------------------------------------------------ checkpointing
    def _state_dict_for_param(
        self, idx: int, packed_state: dict[int, Any], hparams: dict[str, Any], param: torch.Tensor
    ) -> dict[str, Any]:
        out = dict(packed_state[idx])  # shallow copy: self.state stays untouched
        for key in self._quantized_state_spec():
            if key in out:
                q = out.pop(key)
                assert isinstance(q, MaybeQuantizedTensor)
                out.update(q.state_dict(name=key, allow_quantized=self._compress_state_dict))
        if "error_bits" in out:
            # torch casts state tensors to the param dtype on load and FSDP wants them
            # param-shaped, so the codes are disguised as the param dtype: same width ->
            # reinterpret the bits, int8 next to a 2-byte param -> exact value conversion.
            pw = oracle.DTYPE_WIDTHS[param.dtype]
            ew = hparams["master_bytewidth"] - pw
            errs = out["error_bits"]
            if ew == pw:
                out["error_bits"] = errs.view(dtype=param.dtype)
            elif ew == 1 and pw == 2:
                out["error_bits"] = errs.to(dtype=param.dtype)
            else:
                raise NotImplementedError(
                    f"Cannot save {ew}B error correction tensor for {pw}B parameter: state "
                    "tensors must have the parameter's shape and survive a cast to its dtype."
                )
        self._wrap_state_as_dtensor(out, param)
        return out

    def state_dict(self) -> dict[str, Any]:
        d = super().state_dict()
        packed_state, packed_groups = d["state"], d["param_groups"]
        for live, saved in zip(self.param_groups, packed_groups):
            for param, idx in zip(live["params"], saved["params"]):
                if idx in packed_state:
                    packed_state[idx] = self._state_dict_for_param(idx, packed_state, saved, param)
        return d

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        """Load a checkpoint written by this library, by the reference, or by a stock
        PyTorch optimizer with the same state names (moments are re-quantised)."""
        sd = dict(state_dict)
        shielded_state = {}
        moment_keys = set(self._quantized_state_spec())

        def shield(k: str, v: Any) -> Any:
            # moments (either flavour) keep their checkpoint dtype until they are
            # re-quantised: a detour through an fp16 parameter dtype would flush
            # small second moments to zero, through bf16 it would round the scales
            if isinstance(v, torch.Tensor) and (k in moment_keys or k.split("::")[0] in moment_keys):
                return _Shielded(v)
            return v

        for idx, pstate in state_dict["state"].items():
            if isinstance(pstate, dict):
                pstate = {k: shield(k, v) for k, v in pstate.items()}
            shielded_state[idx] = pstate
        sd["state"] = shielded_state
        super().load_state_dict(sd)
        for group in self.param_groups:
            group.setdefault("initial_lr", group["lr"])
        self._tables.clear()

    def _load_state_for_param(
        self, param: torch.Tensor, pstate: dict[str, Any], hparams: dict[str, Any]
    ) -> dict[str, Any]:
        specs = self._quantized_state_spec()
        new_state: dict[str, Any] = {}
        for key, value in pstate.items():
            if not any(key == k or key.startswith(f"{k}::") for k in specs):
                new_state[key] = value
        quantize = hparams.get("quantize", self._quantize)
        for key, spec in specs.items():
            live = pstate.get(key)
            if isinstance(live, MaybeQuantizedTensor):  # un-pickling a live optimizer
                new_state[key] = live
                continue
            if any(k == key or k.startswith(f"{key}::") for k in pstate):
                new_state[key] = MaybeQuantizedTensor.from_state_dict(
                    pstate, name=key, try_quantize=quantize, signed=spec.signed, sqrt=spec.sqrt,
                    softsign=spec.softsign, storage_dtype=param.dtype,
                )
        mbw = hparams.get("master_bytewidth")
        errs = pstate.get("error_bits")
        if mbw is None or errs is None:
            # a checkpoint without master_bytewidth never carried correction codes
            new_state.pop("error_bits", None)
            return new_state
        mbw = int(mbw)
        pw = oracle.DTYPE_WIDTHS[param.dtype]
        need = mbw - pw
        src_dtype = errs.dtype
        if need == 1 and errs.dtype != torch.int8:
            errs = errs.to(dtype=torch.int8)
        elif need == 2 and errs.dtype != torch.int16:
            errs = errs.contiguous().view(dtype=torch.int16)
        if pw + oracle.DTYPE_WIDTHS[errs.dtype] != mbw:
            raise ValueError(
                f"Loading errors of dtype {src_dtype} for param of dtype {param.dtype} cannot "
                f"yield master_weight_bits={mbw * 8}."
            )
        new_state["error_bits"] = errs
        return new_state

    _PRIVATE_ATTRS = (
        "_fused", "_quantize", "_master_bytewidth", "_compress_state_dict", "_check_numerics",
        "_gradient_release", "_decoupled", "_decouple_lr", "_nesterov",
    )

    def __setstate__(self, state: dict[str, Any]) -> None:
        # Reached two ways: from Optimizer.load_state_dict with {"state", "param_groups"}
        # (values are checkpoint tensors) and from unpickling / deepcopy (values are live
        # MaybeQuantizedTensor objects, plus the private attributes of __getstate__).
        super().__setstate__(state)
        self.__dict__.setdefault("_tables", {})
        self.__dict__.setdefault("_transient_state", {})
        self.__dict__.setdefault("_peer_stepped", set())
        self.__dict__.setdefault("_post_step_callbacks", [])
        self.__dict__.setdefault("_local_update_listeners", [])
        self._tables.clear()
        self._transient_state.clear()
        self.__dict__.setdefault("_state_ready", set()).clear()
        opt_state = cast(dict[torch.Tensor, Any], state["state"])
        for group in cast(list[dict[str, Any]], state["param_groups"]):
            for param in group["params"]:
                if param not in opt_state:
                    continue
                pstate = opt_state[param]
                p_local = local_tensor(param)
                for key, val in list(pstate.items()):
                    if isinstance(val, _Shielded):
                        pstate[key] = local_tensor(val.tensor).to(device=p_local.device)
                    elif isinstance(val, torch.Tensor):
                        pstate[key] = local_tensor(val)
                opt_state[param] = self._load_state_for_param(param, pstate, group)
            # after loading, so the loader can tell "came with the checkpoint" from "our default"
            group.setdefault("master_bytewidth", self._master_bytewidth)

    def __getstate__(self) -> dict[str, Any]:
        d = dict(super().__getstate__())
        for name in self._PRIVATE_ATTRS:
            if name in self.__dict__:
                d[name] = self.__dict__[name]
        return d

    # ------------------------------------------------------------------ fp32 export / import
    def get_fp32_model_state_dict(self, model: nn.Module) -> dict[str, torch.Tensor]:
        """``model.state_dict()`` in fp32, parameters rebuilt from parameter + correction.

        Pass the DDP wrapper or the bare module.  For FSDP2 the entries of
        corrected parameters are local shards (plain tensors).
        """
        module = cast(nn.Module, model.module if hasattr(model, "module") else model)
        out = {k: v.detach().float() for k, v in module.state_dict().items()}
        for name, param in module.named_parameters():
            state = self.state.get(param, {})
            if "error_bits" in state:
                out[name] = reconstruct_fp32_param(local_tensor(param.detach()), state["error_bits"])
        return out

    def set_fp32_model_state_dict(self, model: nn.Module, fp32_state_dict: dict[str, torch.Tensor]) -> None:
        """Inverse of :meth:`get_fp32_model_state_dict`: write rounded weights into the
        model and the matching correction codes into the optimizer state."""
        module = cast(nn.Module, model.module if hasattr(model, "module") else model)
        for name, param in module.named_parameters():
            if name not in fp32_state_dict:
                continue
            value = fp32_state_dict[name]
            if value.dtype != torch.float32:
                raise ValueError(f"Expected fp32 value for '{name}', got {value.dtype}.")
            local_param = local_tensor(param.data)
            local_value = local_tensor(value)
            if local_value.device != local_param.device:
                local_value = local_value.to(local_param.device)
            local_param.copy_(local_value.to(param.dtype))
            state = self.state.get(param, {})
            if "error_bits" in state:
                width = local_param.element_size() + state["error_bits"].element_size()
                state["error_bits"] = compute_ecc_bits(local_value, local_param, master_bytewidth=width)
        self._tables.clear()
