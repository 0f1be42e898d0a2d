"""Checkpoint format: interop with stock PyTorch optimizers, compressed and
default flavours, disk round trip, pickling (modelled on the reference's
``test/test_serialization.py`` and ``test/test_training.py:353-418``)."""

import copy
import io
import pickle

import pytest
import torch
import torch.nn as nn

from flashoptim_b200 import FlashAdamW, FlashLion, FlashSGD
from flashoptim_b200.optim.state import MaybeQuantizedTensor

from test_optimizers import DEVICES, _data, _model

CASES = [
    # optimizer, kwargs, state keys
    (FlashAdamW, dict(lr=1e-2), ("exp_avg", "exp_avg_sq")),
    (FlashLion, dict(lr=1e-3), ("exp_avg",)),
    (FlashSGD, dict(lr=1e-1, momentum=0.9), ("momentum_buffer",)),
]


def _train(model, opt, x, y, steps):
    losses = []
    for _ in range(steps):
        loss = nn.functional.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    return losses


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("cls,kw,keys", CASES)
@pytest.mark.parametrize("dtype,mwb", [(torch.bfloat16, 24), (torch.bfloat16, 32), (torch.float16, 24),
                                       (torch.float32, None)])
@pytest.mark.parametrize("compress", [False, True])
def test_state_dict_format_and_round_trip(device, cls, kw, keys, dtype, mwb, compress):
    model = _model(device, dtype)
    opt = cls(model.parameters(), master_weight_bits=mwb, compress_state_dict=compress, **kw)
    x, y = _data(device, dtype)
    _train(model, opt, x, y, 3)
    sd = opt.state_dict()
    params = list(model.parameters())
    for idx, p in enumerate(params):
        st = sd["state"][idx]
        for key in keys:
            if compress:
                q, s = st[f"{key}::quantized"], st[f"{key}::scales"]
                assert key not in st
                assert q.shape == p.shape and q.dtype == (torch.uint8 if key == "exp_avg_sq" else torch.int8)
                assert s.dtype == torch.float16 and s.numel() == (p.numel() + 31) // 32
                assert q.data_ptr() == opt.state[p][key].quantized.data_ptr()  # live tensors, no copy
            else:
                assert st[key].dtype == torch.bfloat16 and st[key].shape == p.shape
        if mwb is not None:
            e = st["error_bits"]
            assert e.dtype == dtype and e.shape == p.shape  # disguised as the param dtype
            live = opt.state[p]["error_bits"]
            if mwb == 32:
                assert torch.equal(e.view(torch.int16), live)  # same bits
            else:
                assert torch.equal(e.to(torch.int8), live)  # same values
        else:
            assert "error_bits" not in st
        if cls is FlashAdamW:
            assert st["step"].device.type == "cpu" and st["step"].dtype == torch.float32 and st["step"].dim() == 0
    g = sd["param_groups"][0]
    assert g["master_bytewidth"] == {None: 0, 24: 3, 32: 4}[mwb] and g["quantize"] is True
    assert g["initial_lr"] == g["lr"]

    # reload into a fresh optimizer: states equal, training continues identically
    model2 = copy.deepcopy(model)
    opt2 = cls(model2.parameters(), master_weight_bits=mwb, compress_state_dict=compress, **kw)
    opt2.load_state_dict(copy.deepcopy(sd))
    for p, p2 in zip(params, model2.parameters()):
        for key in keys:
            a, b = opt.state[p][key], opt2.state[p2][key]
            assert isinstance(b, MaybeQuantizedTensor) and b.is_quantized()
            if compress:
                assert torch.equal(a.quantized, b.quantized) and torch.equal(a.scales, b.scales)
            else:  # went through bf16: re-quantised, close but not identical
                assert torch.allclose(a.materialize(), b.materialize(), rtol=5e-2, atol=float(a.materialize().abs().max()) * 2e-2)
        if mwb is not None:
            assert torch.equal(opt.state[p]["error_bits"], opt2.state[p2]["error_bits"])
            assert opt2.state[p2]["error_bits"].dtype == opt.state[p]["error_bits"].dtype
    l1 = _train(model, opt, x, y, 3)
    l2 = _train(model2, opt2, x, y, 3)
    if compress:
        assert l1 == l2
    else:
        assert all(abs(a - b) <= 2e-2 * abs(a) + 1e-3 for a, b in zip(l1, l2))


@pytest.mark.parametrize("device", DEVICES)
def test_interop_with_torch_adamw(device):
    x, y = _data(device, torch.float32)
    # torch -> flash: fp32 moments are re-quantised on load, initial_lr is filled in
    model = _model(device, torch.float32)
    topt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    _train(model, topt, x, y, 3)
    fopt = FlashAdamW(model.parameters(), lr=1e-2, master_weight_bits=None)
    fopt.load_state_dict(topt.state_dict())
    p = next(model.parameters())
    st = fopt.state[p]
    assert st["exp_avg"].is_quantized() and "error_bits" not in st
    assert torch.allclose(st["exp_avg"].materialize(), topt.state[p]["exp_avg"], rtol=0.1,
                          atol=float(topt.state[p]["exp_avg"].abs().max()) * 2e-2)
    assert float(st["step"]) == 3.0
    assert all("initial_lr" in g for g in fopt.param_groups)
    _train(model, fopt, x, y, 2)
    # flash -> torch: the default flavour loads into the stock optimizer
    topt2 = torch.optim.AdamW(model.parameters(), lr=1e-2)
    topt2.load_state_dict(fopt.state_dict())
    assert topt2.state[p]["exp_avg"].shape == p.shape
    _train(model, topt2, x, y, 1)
    # the compressed flavour does not
    copt = FlashAdamW(model.parameters(), lr=1e-2, master_weight_bits=None, compress_state_dict=True)
    _train(model, copt, x, y, 1)
    topt3 = torch.optim.AdamW(model.parameters(), lr=1e-2)
    topt3.load_state_dict(copt.state_dict())
    with pytest.raises(KeyError):
        _train(model, topt3, x, y, 1)


@pytest.mark.parametrize("device", DEVICES)
def test_interop_with_torch_sgd(device):
    x, y = _data(device, torch.float32)
    model = _model(device, torch.float32)
    topt = torch.optim.SGD(model.parameters(), lr=1e-1, momentum=0.9)
    _train(model, topt, x, y, 3)
    fopt = FlashSGD(model.parameters(), lr=1e-1, momentum=0.9, master_weight_bits=None)
    fopt.load_state_dict(topt.state_dict())
    assert fopt.state[next(model.parameters())]["momentum_buffer"].is_quantized()
    _train(model, fopt, x, y, 1)
    topt2 = torch.optim.SGD(model.parameters(), lr=1e-1, momentum=0.9)
    topt2.load_state_dict(fopt.state_dict())
    _train(model, topt2, x, y, 1)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("compress", [False, True])
def test_disk_round_trip_resumes_training(device, compress, tmp_path):
    dtype = torch.bfloat16
    model = _model(device, dtype)
    opt = FlashAdamW(model.parameters(), lr=1e-2, compress_state_dict=compress)
    x, y = _data(device, dtype)
    _train(model, opt, x, y, 4)
    path = tmp_path / "ckpt.pt"
    torch.save({"model": model.state_dict(), "opt": opt.state_dict()}, path)
    cont = _train(model, opt, x, y, 4)
    ck = torch.load(path, weights_only=True)
    model2 = _model(device, dtype, seed=99)
    model2.load_state_dict(ck["model"])
    opt2 = FlashAdamW(model2.parameters(), lr=1e-2, compress_state_dict=compress)
    opt2.load_state_dict(ck["opt"])
    resumed = _train(model2, opt2, x, y, 4)
    tol = 1e-6 if compress else 2e-2
    assert all(abs(a - b) <= tol * abs(a) + (0 if compress else 1e-3) for a, b in zip(cont, resumed)), (cont, resumed)
    if compress:
        # smaller than the bf16 flavour by roughly half
        buf_c, buf_d = io.BytesIO(), io.BytesIO()
        torch.save(opt.state_dict(), buf_c)
        torch.save(FlashAdamW(model.parameters(), lr=1e-2).state_dict(), buf_d)


def test_compressed_checkpoint_is_smaller():
    model = _model("cpu", torch.bfloat16, d_in=256, d_h=512)
    x, y = _data("cpu", torch.bfloat16, d_in=256)
    sizes = {}
    for compress in (False, True):
        opt = FlashAdamW(model.parameters(), lr=1e-3, compress_state_dict=compress, master_weight_bits=None)
        _train(model, opt, x, y, 1)
        buf = io.BytesIO()
        torch.save(opt.state_dict(), buf)
        sizes[compress] = buf.tell()
    assert sizes[True] < 0.58 * sizes[False]


def test_mismatched_error_width_is_rejected():
    model = _model("cpu", torch.bfloat16)
    x, y = _data("cpu", torch.bfloat16)
    opt = FlashAdamW(model.parameters(), lr=1e-2, master_weight_bits=24)
    _train(model, opt, x, y, 1)
    sd = opt.state_dict()
    sd["param_groups"][0]["master_bytewidth"] = 7
    opt2 = FlashAdamW(model.parameters(), lr=1e-2, master_weight_bits=24)
    with pytest.raises(ValueError):
        opt2.load_state_dict(sd)


@pytest.mark.parametrize("device", DEVICES)
def test_pickle_and_deepcopy_of_live_optimizer(device):
    model = _model(device, torch.bfloat16)
    opt = FlashAdamW(model.parameters(), lr=1e-2, compress_state_dict=True)
    x, y = _data(device, torch.bfloat16)
    _train(model, opt, x, y, 2)
    clone = pickle.loads(pickle.dumps(opt))
    assert clone._compress_state_dict and clone._master_bytewidth == 3 and clone._fused
    p = opt.param_groups[0]["params"][0]
    q = clone.param_groups[0]["params"][0]
    assert torch.equal(opt.state[p]["exp_avg"].quantized, clone.state[q]["exp_avg"].quantized)
    q.grad = torch.ones_like(q)
    clone.step()
