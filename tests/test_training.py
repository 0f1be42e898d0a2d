"""End-to-end training slices (modelled on the reference's ``test/test_training.py``):
the 784->256->10 classifier against fp32 AdamW, autocast modes, resume."""

import copy

import pytest
import torch
import torch.nn as nn

from flashoptim_b200 import FlashAdamW, cast_model
from flashoptim_b200.models import make_mlp

from helpers import nmse
from test_optimizers import DEVICES


def _mnist_like(device, seed=0, n=64):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, 784, generator=g).to(device), torch.randint(0, 10, (n,), generator=g).to(device)


def _train(model, opt, x, y, steps, cast=None):
    losses = []
    for _ in range(steps):
        xx = x if cast is None else x.to(cast)
        loss = nn.functional.cross_entropy(model(xx).float(), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    return losses


@pytest.mark.parametrize("device", DEVICES)
def test_mlp_200_steps_tracks_fp32_adamw(device):
    """bf16 model + FlashAdamW (24-bit masters, 8-bit states) vs fp32 torch.optim.AdamW."""
    torch.manual_seed(0)
    ref = make_mlp().to(device)
    model = copy.deepcopy(ref)
    cast_model(model, torch.bfloat16)
    x, y = _mnist_like(device)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01)
    fopt = FlashAdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01, master_weight_bits=24)
    lr_ = _train(ref, ropt, x, y, 200)
    lf = _train(model, fopt, x, y, 200, cast=torch.bfloat16)
    assert lf[-1] < 0.05 * lf[0]
    # same trajectory: early losses agree closely, the whole curve correlates
    assert all(abs(a - b) < 0.05 * a + 2e-2 for a, b in zip(lr_[:50], lf[:50]))
    a, b = torch.tensor(lr_), torch.tensor(lf)
    assert torch.corrcoef(torch.stack([a, b]))[0, 1] > 0.995
    assert nmse(a, b) < 5e-3
    # state dict round trip then identical continuation
    sd = copy.deepcopy(fopt.state_dict())
    model2 = copy.deepcopy(model)
    fopt2 = FlashAdamW(model2.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01, master_weight_bits=24,
                       compress_state_dict=True)
    fopt2.load_state_dict(sd)
    l1 = _train(model, fopt, x, y, 5, cast=torch.bfloat16)
    l2 = _train(model2, fopt2, x, y, 5, cast=torch.bfloat16)
    assert all(abs(p - q) <= 5e-2 * abs(p) + 1e-4 for p, q in zip(l1, l2))


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("mode", ["bf16_autocast", "bf16_native", "fp16_autocast_scaler"])
def test_mixed_precision_modes(device, mode):
    if mode == "fp16_autocast_scaler" and device == "cpu":
        pytest.skip("fp16 GradScaler path is exercised on CUDA")
    torch.manual_seed(1)
    base = make_mlp(64, 32, 10).to(device)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(128, 64, generator=g).to(device)
    y = torch.randint(0, 10, (128,), generator=g).to(device)
    ref = copy.deepcopy(base)
    ropt = torch.optim.AdamW(ref.parameters(), lr=3e-3)
    truth = _train(ref, ropt, x, y, 40)
    model = copy.deepcopy(base)
    losses = []
    if mode == "bf16_native":
        cast_model(model, torch.bfloat16)
        opt = FlashAdamW(model.parameters(), lr=3e-3, master_weight_bits=24)
        losses = _train(model, opt, x, y, 40, cast=torch.bfloat16)
    else:
        opt = FlashAdamW(model.parameters(), lr=3e-3, master_weight_bits=None)
        amp_dtype = torch.bfloat16 if mode == "bf16_autocast" else torch.float16
        scaler = torch.amp.GradScaler(device) if mode == "fp16_autocast_scaler" else None
        for _ in range(40):
            with torch.autocast(device_type=device, dtype=amp_dtype):
                loss = nn.functional.cross_entropy(model(x).float(), y)
            if scaler is not None:
                scaler.scale(loss).backward()
                scaler.step(opt)
                scaler.update()
            else:
                loss.backward()
                opt.step()
            opt.zero_grad()
            losses.append(loss.item())
    a, b = torch.tensor(truth), torch.tensor(losses)
    assert b[-1] < 0.7 * b[0]
    assert nmse(a, b) < 2e-2
    assert torch.corrcoef(torch.stack([a, b]))[0, 1] > 0.99


@pytest.mark.parametrize("device", DEVICES)
def test_joint_checkpoint_resume_gives_same_losses(device, tmp_path):
    torch.manual_seed(3)
    model = make_mlp(64, 32, 10).to(device)
    cast_model(model)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(64, 64, generator=g).to(device)
    y = torch.randint(0, 10, (64,), generator=g).to(device)
    opt = FlashAdamW(model.parameters(), lr=1e-3, compress_state_dict=True)
    _train(model, opt, x, y, 10, cast=torch.bfloat16)
    torch.save({"m": model.state_dict(), "o": opt.state_dict()}, tmp_path / "c.pt")
    cont = _train(model, opt, x, y, 10, cast=torch.bfloat16)
    ck = torch.load(tmp_path / "c.pt", weights_only=True)
    model2 = make_mlp(64, 32, 10).to(device)
    cast_model(model2)
    model2.load_state_dict(ck["m"])
    opt2 = FlashAdamW(model2.parameters(), lr=1e-3, compress_state_dict=True)
    opt2.load_state_dict(ck["o"])
    res = _train(model2, opt2, x, y, 10, cast=torch.bfloat16)
    assert all(abs(a - b) <= 2e-4 * abs(a) for a, b in zip(cont, res)), (cont, res)
