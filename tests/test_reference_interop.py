"""Checkpoints written by the reference load here and vice versa, in both flavours
(needs the reference installed under ``baseline/_ref`` and a GPU, since the reference
itself only runs on CUDA)."""

import copy
import os
import sys
import warnings

import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


def _reference():
    if not os.path.isdir(os.path.join(REF_DIR, "flashoptim")):
        pytest.skip("reference is not installed under baseline/_ref")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import flashoptim

    return flashoptim


def _model(seed=0):
    torch.manual_seed(seed)
    m = nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 32)).cuda()
    return m


def _train(model, opt, steps, seed=1):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(32, 64, generator=g).cuda().bfloat16()
    y = torch.randint(0, 32, (32,), generator=g).cuda()
    losses = []
    for _ in range(steps):
        loss = nn.functional.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(loss.item())
    return losses


CASES = [("FlashAdamW", dict(lr=1e-3)), ("FlashLion", dict(lr=1e-4)), ("FlashSGD", dict(lr=1e-2, momentum=0.9))]


@pytest.mark.parametrize("name,kw", CASES)
@pytest.mark.parametrize("mwb", [24, 32])
@pytest.mark.parametrize("compress", [False, True])
@pytest.mark.parametrize("direction", ["ref_to_ours", "ours_to_ref"])
def test_cross_load(name, kw, mwb, compress, direction):
    ref = _reference()
    import flashoptim_b200 as ours

    src_lib, dst_lib = (ref, ours) if direction == "ref_to_ours" else (ours, ref)
    warnings.simplefilter("ignore")
    m_src = _model()
    src_lib.cast_model(m_src, dtype=torch.bfloat16)
    o_src = getattr(src_lib, name)(m_src.parameters(), master_weight_bits=mwb, compress_state_dict=compress, **kw)
    _train(m_src, o_src, 4)
    sd = copy.deepcopy(o_src.state_dict())
    m_dst = copy.deepcopy(m_src)
    o_dst = getattr(dst_lib, name)(m_dst.parameters(), master_weight_bits=mwb, compress_state_dict=compress, **kw)
    o_dst.load_state_dict(sd)
    # the loaded optimizer writes the same checkpoint back
    sd2 = o_dst.state_dict()
    for idx, st in sd["state"].items():
        for key, val in st.items():
            got = sd2["state"][idx][key]
            assert got.dtype == val.dtype and got.shape == val.shape, (idx, key)
            if key == "error_bits":
                a = val.view(torch.int16) if mwb == 32 else val.to(torch.int8)
                b = got.view(torch.int16) if mwb == 32 else got.to(torch.int8)
                assert torch.equal(a.cpu(), b.cpu()), (idx, key)
            elif "::quantized" in key:
                assert torch.equal(val.cpu(), got.cpu()), (idx, key)
            elif "::scales" in key:
                # the reference's load rounds fp16 scales through the bf16 param dtype
                assert torch.allclose(val.float().cpu(), got.float().cpu(), rtol=1e-2, atol=1e-3), (idx, key)
            elif key == "step":
                assert float(val) == float(got)
            else:  # bf16 moments: re-quantised from bf16 on load, written back through bf16
                assert torch.allclose(val.float().cpu(), got.float().cpu(), rtol=6e-2,
                                      atol=float(val.float().abs().max()) * 2e-2), (idx, key)
    for g1, g2 in zip(sd["param_groups"], sd2["param_groups"]):
        for k in ("lr", "master_bytewidth", "quantize", "weight_decay"):
            assert g1[k] == g2[k]
    # and training continues on the same trajectory as the source optimizer
    l_src = _train(m_src, o_src, 3, seed=2)
    l_dst = _train(m_dst, o_dst, 3, seed=2)
    assert all(abs(a - b) <= 2e-2 * abs(a) + 2e-3 for a, b in zip(l_src, l_dst)), (l_src, l_dst)


def test_kernels_agree_with_reference_kernels():
    """Same inputs through the reference's Triton quantiser / ECC helpers and ours."""
    ref = _reference()
    from flashoptim.optimizers import dequantize as ref_dequantize
    from flashoptim.optimizers import quantize as ref_quantize

    import flashoptim_b200 as ours

    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(100003, device="cuda", generator=g) * 1e-2
    for signed, sqrt, softsign in [(True, False, True), (False, True, False)]:
        xi = x if signed else x.abs()
        q1, s1 = ref_quantize(xi, signed=signed, sqrt=sqrt, softsign=softsign)
        q2, s2 = ours.quantize(xi, signed=signed, sqrt=sqrt, softsign=softsign)
        d = (q1.to(torch.int16) - q2.to(torch.int16)).abs()
        assert d.max() <= 1 and (d != 0).float().mean() < 5e-3  # Triton's approximate division flips rare ties
        # Triton's approximate sqrt can move a scale by one fp16 ULP
        assert torch.allclose(s1.float(), s2.float(), rtol=2e-3, atol=0)
        a = ref_dequantize(q2, s2, signed=signed, sqrt=sqrt, softsign=softsign)
        b = ours.dequantize(q2, s2, signed=signed, sqrt=sqrt, softsign=softsign)
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-12)
    w = x.bfloat16()
    for mbw in (3, 4):
        e1 = ref.compute_ecc_bits(x, w, master_bytewidth=mbw)
        e2 = ours.compute_ecc_bits(x, w, master_bytewidth=mbw)
        assert (e1.int() - e2.int()).abs().max() <= 1
        r1 = ref.reconstruct_fp32_param(w, e2)
        r2 = ours.reconstruct_fp32_param(w, e2)
        assert torch.allclose(r1, r2, rtol=1e-6, atol=1e-30)
