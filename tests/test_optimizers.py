"""Optimizer behaviour on CPU (PyTorch formulation) and on CUDA (fused kernels):
modelled on the reference's ``test/test_optimizers.py``."""

import copy
import warnings

import pytest
import torch
import torch.nn as nn

import flashoptim_b200 as fo
from flashoptim_b200 import (
    FlashAdam, FlashAdamW, FlashLion, FlashSGD, FlashSGDW, NumericsError, cast_model,
    enable_gradient_release,
)
from flashoptim_b200.optim.state import MaybeQuantizedTensor

from helpers import cossim, nmse
from reference_optimizers import ReferenceAdamW, ReferenceLion, ReferenceSGD

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]

OPTS = {
    "adam": (FlashAdam, dict(lr=1e-2, weight_decay=1e-3)),
    "adamw": (FlashAdamW, dict(lr=1e-2, weight_decay=1e-2)),
    "lion": (FlashLion, dict(lr=1e-3, weight_decay=1e-2)),
    "sgd": (FlashSGD, dict(lr=1e-1, momentum=0.9, weight_decay=1e-4)),
    "sgd_nesterov": (FlashSGD, dict(lr=1e-1, momentum=0.9, nesterov=True)),
    "sgdw": (FlashSGDW, dict(lr=1e-1, momentum=0.9, weight_decay=1e-3)),
    "sgdw_nomom": (FlashSGDW, dict(lr=1e-1, weight_decay=1e-3)),
}
# (dtype, master_weight_bits, quantize)
CONFIGS = [
    (torch.bfloat16, 24, True), (torch.bfloat16, 32, True), (torch.bfloat16, None, True),
    (torch.bfloat16, 24, False), (torch.float16, 24, True), (torch.float32, None, True),
    (torch.float32, None, False),
]


def _model(device, dtype, seed=0, d_in=32, d_h=64, d_out=8):
    torch.manual_seed(seed)
    m = nn.Sequential(nn.Linear(d_in, d_h), nn.ReLU(), nn.Linear(d_h, d_out)).to(device)
    if dtype != torch.float32:
        cast_model(m, dtype)
    return m


def _data(device, dtype, n=64, d_in=32, d_out=8, seed=1):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, d_in, generator=g).to(device=device, dtype=dtype)
    y = torch.randint(0, d_out, (n,), generator=g).to(device)
    return x, y


def _make(name, params, mwb, quantize, **over):
    cls, kw = OPTS[name]
    kw = dict(kw)
    kw.update(over)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return cls(params, master_weight_bits=mwb, quantize=quantize, **kw)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", list(OPTS))
@pytest.mark.parametrize("dtype,mwb,quantize", CONFIGS)
def test_descends_and_updates_state(device, name, dtype, mwb, quantize):
    model = _model(device, dtype)
    opt = _make(name, model.parameters(), mwb, quantize)
    x, y = _data(device, dtype)
    w0 = [p.detach().clone() for p in model.parameters()]
    losses = []
    for _ in range(12):
        loss = nn.functional.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    assert losses[-1] < losses[0] * 0.98, losses
    assert all(not torch.equal(a, p.detach()) for a, p in zip(w0, model.parameters()))
    for p in model.parameters():
        st = opt.state[p]
        for key in opt._quantized_state_spec():
            s = st[key]
            assert isinstance(s, MaybeQuantizedTensor)
            assert s.is_quantized() == quantize
            assert s.materialize().float().abs().sum() > 0
        if mwb is not None and dtype != torch.float32:
            assert st["error_bits"].dtype == (torch.int8 if mwb == 24 else torch.int16)
            assert st["error_bits"].shape == p.shape
        else:
            assert "error_bits" not in st


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", ["adamw", "lion", "sgdw"])
def test_zero_grads_still_decay_and_decay_moments(device, name):
    model = _model(device, torch.bfloat16)
    opt = _make(name, model.parameters(), 24, True)
    x, y = _data(device, torch.bfloat16)
    nn.functional.cross_entropy(model(x).float(), y).backward()
    opt.step()
    key = "exp_avg" if name != "sgdw" else "momentum_buffer"
    p = next(model.parameters())
    m_before = opt.state[p][key].materialize().clone()
    w_before = opt.get_fp32_model_state_dict(model)["0.weight"].clone()
    for q in model.parameters():
        q.grad.zero_()
    opt.step()
    m_after = opt.state[p][key].materialize()
    assert m_after.abs().sum() < m_before.abs().sum()
    assert not torch.equal(w_before, opt.get_fp32_model_state_dict(model)["0.weight"])


def _run_trajectory(device, name, dtype, mwb, quantize, fused, steps=20, **over):
    model = _model(device, dtype, seed=3)
    opt = _make(name, model.parameters(), mwb, quantize, fused=fused, **over)
    x, y = _data(device, dtype, seed=4)
    for _ in range(steps):
        nn.functional.cross_entropy(model(x).float(), y).backward()
        opt.step()
        opt.zero_grad()
    return torch.cat([v.flatten().float().cpu() for v in opt.get_fp32_model_state_dict(model).values()])


def _truth_trajectory(name, steps=20, **over):
    """fp32 parameters, fp32 states, plain PyTorch."""
    model = _model("cpu", torch.float32, seed=3)
    cls, kw = OPTS[name]
    kw = dict(kw)
    kw.update(over)
    if name in ("adam", "adamw"):
        ref = ReferenceAdamW(model.parameters(), decoupled=(name == "adamw"), **kw)
    elif name == "lion":
        ref = ReferenceLion(model.parameters(), **kw)
    else:
        nest = kw.pop("nesterov", False)
        ref = ReferenceSGD(model.parameters(), nesterov=nest, decoupled=name.startswith("sgdw"), **kw)
    x, y = _data("cpu", torch.float32, seed=4)
    for _ in range(steps):
        nn.functional.cross_entropy(model(x), y).backward()
        ref.step()
        ref.zero_grad()
    return torch.cat([p.detach().flatten() for p in model.state_dict().values()])


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", ["adam", "adamw", "sgd", "sgd_nesterov", "sgdw", "sgdw_nomom"])
def test_matches_fp32_truth(device, name):
    """Unquantised fp32 run equals the plain PyTorch optimizer; quantised / ECC / fused
    variants stay within the reference's similarity thresholds of it."""
    truth = _truth_trajectory(name)
    exact = _run_trajectory(device, name, torch.float32, None, False, fused=True)
    assert torch.allclose(exact, truth, rtol=2e-4, atol=2e-5), (exact - truth).abs().max()
    for dtype, mwb, quantize, fused in [
        (torch.float32, None, True, True), (torch.float32, None, True, False),
        (torch.bfloat16, 24, True, True), (torch.bfloat16, 32, True, True),
        (torch.bfloat16, 24, True, False), (torch.bfloat16, 24, False, True),
    ]:
        got = _run_trajectory(device, name, dtype, mwb, quantize, fused)
        # a bf16 model also computes its gradients in bf16, so it drifts further from the fp32 run
        min_cs, max_nmse = (0.999, 2e-3) if dtype == torch.float32 else (0.995, 1e-2)
        assert cossim(got, truth) > min_cs, (name, dtype, mwb, quantize, fused, cossim(got, truth))
        assert nmse(truth, got) < max_nmse, (name, dtype, mwb, quantize, fused, nmse(truth, got))
    other = _truth_trajectory("lion")
    assert nmse(truth, other) > nmse(truth, exact) * 10  # a different optimizer is clearly different


@pytest.mark.parametrize("device", DEVICES)
def test_lion_matches_truth(device):
    truth = _truth_trajectory("lion")
    for dtype, mwb, quantize, fused in [(torch.float32, None, False, True), (torch.bfloat16, 32, True, True),
                                        (torch.bfloat16, 24, True, False)]:
        got = _run_trajectory(device, "lion", dtype, mwb, quantize, fused)
        assert cossim(got, truth) > 0.995 and nmse(truth, got) < 1e-2


@pytest.mark.parametrize("device", [pytest.param("cuda", marks=pytest.mark.gpu)])
@pytest.mark.parametrize("name", ["adamw", "lion", "sgdw"])
@pytest.mark.parametrize("dtype,mwb,quantize", CONFIGS)
def test_fused_matches_unfused(device, name, dtype, mwb, quantize):
    fused = _run_trajectory(device, name, dtype, mwb, quantize, fused=True, steps=10)
    unfused = _run_trajectory(device, name, dtype, mwb, quantize, fused=False, steps=10)
    assert cossim(fused, unfused) > 0.999
    assert nmse(unfused, fused) < 5e-4


@pytest.mark.parametrize("device", DEVICES)
def test_ecc_increases_precision(device):
    """Tiny steps on a large matrix: bf16 alone loses them, 24-bit keeps most, 32-bit nearly all."""
    torch.manual_seed(0)
    n = 512
    w0 = torch.randn(n, n)
    grad = torch.randn(n, n)
    truth = w0.clone()
    lr, steps = 1e-3, 30
    for _ in range(steps):
        truth -= lr * grad
    errs = {}
    for mwb in (None, 24, 32):
        p = nn.Parameter(w0.to(device=device, dtype=torch.bfloat16))
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            opt = FlashSGD([p], lr=lr, master_weight_bits=mwb)
        for _ in range(steps):
            p.grad = grad.to(device=device, dtype=torch.bfloat16)
            opt.step()
        st = opt.state[p]
        rec = fo.reconstruct_fp32_param(p.detach(), st["error_bits"]) if "error_bits" in st else p.detach().float()
        errs[mwb] = (rec.cpu() - truth).abs().mean().item()
    assert errs[None] > 5 * errs[24] > 0
    assert errs[24] >= errs[32]


@pytest.mark.parametrize("device", DEVICES)
def test_check_numerics(device):
    p = nn.Parameter(torch.full((64,), 100.0, device=device, dtype=torch.bfloat16))
    p.grad = torch.ones_like(p)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = FlashAdamW([p], lr=1e-3, master_weight_bits=None, check_numerics=True)
    with pytest.raises(NumericsError):
        opt.step()
    opt2 = FlashAdamW([p], lr=1e-3, master_weight_bits=32, check_numerics=True)
    opt2.step()  # 32-bit masters resolve the step
    # cached statistics: shrinking the weights only helps after a refresh
    with torch.no_grad():
        p.fill_(1e-4)
    with pytest.raises(NumericsError):
        opt.step()
    opt.recompute_param_stats()
    opt.step()
    # lr == 0 is always allowed
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt3 = FlashLion([nn.Parameter(torch.full((8,), 1e4, device=device, dtype=torch.bfloat16))], lr=0.0,
                         master_weight_bits=None, check_numerics=True)
    opt3.param_groups[0]["params"][0].grad = torch.ones(8, device=device, dtype=torch.bfloat16)
    opt3.step()


def test_constructor_validation():
    p = [nn.Parameter(torch.zeros(4, dtype=torch.bfloat16))]
    with pytest.raises(ValueError):
        FlashAdamW(p, lr=-1.0)
    with pytest.raises(ValueError):
        FlashAdamW(p, master_weight_bits=16)
    with pytest.raises(ValueError):
        FlashAdamW(p, quantize=False, compress_state_dict=True)
    with pytest.raises(ValueError):
        FlashAdamW(p, betas=(1.5, 0.9))
    with pytest.raises(ValueError):
        FlashAdamW(p, eps=-1)
    with pytest.raises(ValueError):
        FlashLion(p, weight_decay=-1)
    with pytest.raises(ValueError):
        FlashSGD(p, nesterov=True, momentum=0.0)
    with pytest.raises(ValueError):
        FlashSGD(p, nesterov=True, momentum=0.9, dampening=0.1)
    with pytest.warns(UserWarning):
        FlashAdamW(p, master_weight_bits=None)


def test_ineffective_master_weight_bits(monkeypatch):
    p = [nn.Parameter(torch.zeros(4))]
    monkeypatch.delenv("FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS", raising=False)
    with pytest.raises(ValueError):
        FlashAdamW(p, master_weight_bits=24)
    monkeypatch.setenv("FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS", "1")
    FlashAdamW(p, master_weight_bits=24)


def test_repr_lists_configuration():
    opt = FlashAdamW([nn.Parameter(torch.zeros(4, dtype=torch.bfloat16))], lr=3e-4)
    r = repr(opt)
    for token in ("FlashAdamW", "fused: True", "quantize: True", "master_bytewidth: 3",
                  "gradient_release: False", "Parameter Group 0", "lr: 0.0003"):
        assert token in r


@pytest.mark.parametrize("device", DEVICES)
def test_multiple_param_groups(device):
    model = _model(device, torch.bfloat16)
    params = list(model.parameters())
    opt = FlashAdamW([{"params": params[:2], "lr": 1e-2}, {"params": params[2:], "lr": 0.0, "weight_decay": 0.0}])
    frozen = [p.detach().clone() for p in params[2:]]
    moved = [p.detach().clone() for p in params[:2]]
    x, y = _data(device, torch.bfloat16)
    for _ in range(3):
        nn.functional.cross_entropy(model(x).float(), y).backward()
        opt.step()
        opt.zero_grad()
    assert all(torch.equal(a, p.detach()) for a, p in zip(frozen, params[2:]))
    assert all(not torch.equal(a, p.detach()) for a, p in zip(moved, params[:2]))
    for g in opt.param_groups:
        assert g["initial_lr"] == g["lr"] and g["master_bytewidth"] == 3 and g["quantize"] is True


@pytest.mark.parametrize("device", DEVICES)
def test_decouple_lr_matches_reference(device):
    for decouple_lr in (False, True):
        wd = 1e-3 if decouple_lr else 1e-1
        model = _model(device, torch.float32, seed=5)
        ref_model = copy.deepcopy(model).cpu()
        opt = FlashAdamW(model.parameters(), lr=1e-2, weight_decay=wd, decouple_lr=decouple_lr,
                         quantize=False, master_weight_bits=None)
        ref = ReferenceAdamW(ref_model.parameters(), lr=1e-2, weight_decay=wd, decouple_lr=decouple_lr)
        x, y = _data(device, torch.float32)
        for step in range(6):
            for g in list(opt.param_groups) + list(ref.param_groups):
                g["lr"] = 1e-2 * (0.8 ** step)  # a schedule: lr / initial_lr matters
            nn.functional.cross_entropy(model(x), y).backward()
            nn.functional.cross_entropy(ref_model(x.cpu()), y.cpu()).backward()
            opt.step(); ref.step(); opt.zero_grad(); ref.zero_grad()
        for a, b in zip(model.parameters(), ref_model.parameters()):
            assert torch.allclose(a.detach().cpu(), b.detach(), rtol=2e-4, atol=2e-6)
    # decoupled AdamW with default decouple_lr equals torch.optim.AdamW
    model = _model(device, torch.float32, seed=6)
    tmodel = copy.deepcopy(model)
    opt = FlashAdamW(model.parameters(), lr=1e-2, weight_decay=1e-2, quantize=False, master_weight_bits=None)
    topt = torch.optim.AdamW(tmodel.parameters(), lr=1e-2, weight_decay=1e-2)
    x, y = _data(device, torch.float32)
    for _ in range(5):
        nn.functional.cross_entropy(model(x), y).backward()
        nn.functional.cross_entropy(tmodel(x), y).backward()
        opt.step(); topt.step(); opt.zero_grad(); topt.zero_grad()
    for a, b in zip(model.parameters(), tmodel.parameters()):
        assert torch.allclose(a, b, rtol=2e-4, atol=2e-6)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("name", ["adamw", "lion", "sgdw"])
def test_gradient_release_matches_manual_step(device, name):
    m1 = _model(device, torch.bfloat16, seed=7)
    m2 = copy.deepcopy(m1)
    o1 = _make(name, m1.parameters(), 24, True)
    o2 = _make(name, m2.parameters(), 24, True)
    handle = enable_gradient_release(m2, o2)
    assert handle.active and "gradient_release: True" in repr(o2)
    x, y = _data(device, torch.bfloat16)
    for _ in range(4):
        nn.functional.cross_entropy(m1(x).float(), y).backward()
        o1.step(); o1.zero_grad()
        nn.functional.cross_entropy(m2(x).float(), y).backward()
        assert all(p.grad is None for p in m2.parameters())  # freed inside backward
        with pytest.warns(UserWarning):
            o2.step()
        with pytest.warns(UserWarning):
            o2.zero_grad()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)
    handle.remove()
    assert not handle.active
    nn.functional.cross_entropy(m2(x).float(), y).backward()
    assert all(p.grad is not None for p in m2.parameters())
    o2.step()  # no warning, steps normally again
    # pre_step veto keeps gradients
    m3 = _model(device, torch.bfloat16, seed=7)
    o3 = _make(name, m3.parameters(), 24, True)
    w3 = [p.detach().clone() for p in m3.parameters()]
    enable_gradient_release(m3, o3, pre_step=lambda p, g: False)
    nn.functional.cross_entropy(m3(x).float(), y).backward()
    assert all(p.grad is not None for p in m3.parameters())
    assert all(torch.equal(a, p.detach()) for a, p in zip(w3, m3.parameters()))
    with pytest.raises(NotImplementedError):
        enable_gradient_release(m1, o1, grad_scaler=object())


@pytest.mark.parametrize("device", DEVICES)
def test_gradient_release_tied_parameters_step_once(device):
    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(16, 8)
            self.head = nn.Linear(8, 16, bias=False)
            self.head.weight = self.emb.weight

        def forward(self, t):
            return self.head(self.emb(t))

    torch.manual_seed(0)
    m1 = Tied().to(device); cast_model(m1)
    m2 = copy.deepcopy(m1)
    assert m2.head.weight is m2.emb.weight
    o1 = FlashAdamW(m1.parameters(), lr=1e-2)
    o2 = FlashAdamW(m2.parameters(), lr=1e-2)
    enable_gradient_release(m2, o2)
    t = torch.randint(0, 16, (4, 5), device=device)
    for _ in range(3):
        m1(t).float().square().mean().backward(); o1.step(); o1.zero_grad()
        m2(t).float().square().mean().backward()
    assert torch.equal(m1.emb.weight, m2.emb.weight)
    assert int(o2.state[m2.emb.weight]["step"].item()) == 3


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("mwb", [24, 32])
def test_fp32_state_dict_round_trip(device, mwb):
    model = _model(device, torch.bfloat16)
    opt = FlashAdamW(model.parameters(), lr=1e-2, master_weight_bits=mwb)
    x, y = _data(device, torch.bfloat16)
    for _ in range(3):
        nn.functional.cross_entropy(model(x).float(), y).backward()
        opt.step(); opt.zero_grad()
    sd = opt.get_fp32_model_state_dict(model)
    assert all(v.dtype == torch.float32 for v in sd.values())
    narrow = {k: v.detach().clone() for k, v in model.state_dict().items()}
    ecc = {k: opt.state[p]["error_bits"].clone() for k, p in model.named_parameters()}
    assert any((sd[k] != narrow[k].float()).any() for k in narrow)  # the correction carries information
    with torch.no_grad():
        for p in model.parameters():
            p.zero_()
            opt.state[p]["error_bits"].zero_()
    opt.set_fp32_model_state_dict(model, sd)
    back = opt.get_fp32_model_state_dict(model)
    for k, p in model.named_parameters():
        # The master value survives.  Its split may not: a correction of exactly +-half an
        # ULP puts the fp32 value on a bf16 rounding tie, which may round to the other
        # neighbour (with the opposite correction).
        same = p.detach() == narrow[k]
        assert same.float().mean() > 0.98
        step = torch.exp2(fo.ops.oracle.ecc_log_scale(p.detach()).float()) / (127 if mwb == 24 else 32767)
        assert ((back[k] - sd[k]).abs() <= 1.01 * step).all()
        d = (opt.state[p]["error_bits"].int() - ecc[k].int()).abs()[same]
        assert d.max() <= (0 if mwb == 24 else 1)
    with pytest.raises(ValueError):
        opt.set_fp32_model_state_dict(model, {k: v.half() for k, v in sd.items()})


@pytest.mark.parametrize("device", DEVICES)
def test_sgd_without_momentum_keeps_no_state(device):
    model = _model(device, torch.bfloat16)
    opt = FlashSGD(model.parameters(), lr=1e-1)
    x, y = _data(device, torch.bfloat16)
    nn.functional.cross_entropy(model(x).float(), y).backward()
    opt.step()
    for p in model.parameters():
        assert set(opt.state[p]) == {"error_bits"}


@pytest.mark.parametrize("device", [pytest.param("cuda", marks=pytest.mark.gpu)])
def test_fused_rejects_non_contiguous(device):
    w = torch.randn(8, 16, device=device, dtype=torch.bfloat16).t()
    p = nn.Parameter(w)
    assert not p.is_contiguous()
    p.grad = torch.ones_like(p)
    opt = FlashAdamW([p], lr=1e-3)
    with pytest.raises(RuntimeError):
        opt.step()
    opt2 = FlashAdamW([p], lr=1e-3, fused=False)
    opt2.step()


@pytest.mark.parametrize("device", DEVICES)
def test_params_without_grad_and_empty_params(device):
    a = nn.Parameter(torch.randn(10, device=device).bfloat16())
    b = nn.Parameter(torch.randn(10, device=device).bfloat16())
    c = nn.Parameter(torch.zeros(0, device=device).bfloat16())
    frozen = nn.Parameter(torch.randn(4, device=device).bfloat16(), requires_grad=False)
    opt = FlashAdamW([a, b, c, frozen], lr=1e-2)
    a.grad = torch.ones_like(a)
    c.grad = torch.zeros_like(c)
    b0 = b.detach().clone()
    opt.step()
    assert torch.equal(b, b0)
    # state exists for every parameter (checkpointing tools expect that)
    for p in (a, b, c, frozen):
        assert "exp_avg" in opt.state[p] and "step" in opt.state[p]
    assert int(opt.state[a]["step"]) == 1 and int(opt.state[b]["step"]) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["adamw", "lion", "sgdw"])
def test_step_with_explicit_gradients_equals_step(name):
    """``step_with_grads`` (used by the two-shot DDP route) updates like ``step()`` and makes
    the following ``step()`` skip those parameters once."""
    m1 = _model("cuda", torch.bfloat16, seed=11)
    m2 = copy.deepcopy(m1)
    o1 = _make(name, m1.parameters(), 24, True)
    o2 = _make(name, m2.parameters(), 24, True)
    x, y = _data("cuda", torch.bfloat16)
    for _ in range(3):
        nn.functional.cross_entropy(m1(x).float(), y).backward()
        o1.step(); o1.zero_grad()
        nn.functional.cross_entropy(m2(x).float(), y).backward()
        params = list(m2.parameters())
        o2.step_with_grads(params, [p.grad.clone() for p in params])
        o2.step()  # must not apply the gradients a second time
        o2.zero_grad()
    for a, b in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(a, b)


# ---------------------------------------------------------------- memory accounting


def _state_bytes(opt):
    total = 0
    for st in opt.state.values():
        for v in st.values():
            if isinstance(v, MaybeQuantizedTensor):
                parts = [v.quantized, v.scales] if v.is_quantized() else [v.data]
            elif isinstance(v, torch.Tensor) and v.dim() > 0:
                parts = [v]
            else:
                parts = []
            total += sum(t.numel() * t.element_size() for t in parts)
    return total


@pytest.mark.parametrize("cls,kw,mwb,quantize,want", [
    # int8 correction + two moments of (1 byte + one fp16 scale per 32 elements)
    (FlashAdamW, {}, 24, True, 1 + 2 * (1 + 2 / 32)),
    (FlashAdamW, {}, 32, True, 2 + 2 * (1 + 2 / 32)),
    (FlashAdamW, {}, None, True, 2 * (1 + 2 / 32)),
    (FlashAdamW, {}, 24, False, 1 + 2 * 2),        # bf16 moments
    (FlashLion, {}, 24, True, 1 + (1 + 2 / 32)),
    (FlashSGDW, {"momentum": 0.9}, 24, True, 1 + (1 + 2 / 32)),
    (FlashSGDW, {}, 24, True, 1.0),                # momentum-free SGD keeps no moment
])
def test_optimizer_state_bytes_per_parameter(cls, kw, mwb, quantize, want):
    """The memory the states take is what the format promises: 3.125 bytes per bf16 parameter
    for AdamW with 24-bit masters (a conventional mixed-precision AdamW keeps 12: fp32 master
    weights and two fp32 moments), 2.06 for Lion."""
    n = 1 << 14
    p = nn.Parameter(torch.randn(n).to(torch.bfloat16))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        opt = cls([p], lr=1e-3, master_weight_bits=mwb, quantize=quantize, **kw)
    p.grad = torch.randn(n).to(torch.bfloat16) * 1e-2
    opt.step()
    assert _state_bytes(opt) / n == pytest.approx(want)


def test_second_collective_fused_update_without_step_is_refused():
    p = nn.Parameter(torch.randn(64).to(torch.bfloat16))
    opt = FlashAdamW([p], lr=1e-3)
    opt._peer_stepped.add(id(p))  # what a fused reduce-scatter / all-reduce update leaves behind
    peer = type("Peer", (), {"offsets": {id(p.data): 0}})()
    with pytest.raises(RuntimeError, match="twice without optimizer.step"):
        opt.step_from_peers([p], peer)
    with pytest.raises(RuntimeError, match="twice without optimizer.step"):
        opt.step_with_grads([p], [torch.zeros_like(p)])
    p.grad = torch.zeros_like(p)
    opt.step()  # acknowledges the fused update (and skips the parameter once)
    assert id(p) not in opt._peer_stepped
