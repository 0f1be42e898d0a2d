"""CPU tests of the numeric formats: group quantiser, master-weight split,
state container, numerics-check arithmetic (modelled on the reference's
``test/test_compression.py`` and ``test/test_ecc_invariants.py``)."""

import math

import pytest
import torch

from flashoptim_b200 import compute_ecc_bits, dequantize, quantize, reconstruct_fp32_param
from flashoptim_b200.ops import oracle
from flashoptim_b200.optim.state import MaybeQuantizedTensor, QuantizedTensorSpec

from helpers import cossim, ecc_invariant_violations, fp32_with_exponent

SHAPES = [(1, 1), (17, 23), (1, 1000), (64, 64), (3, 5, 7), (4096,), (33,)]
MODES = [(True, False, True), (True, False, False), (False, True, False), (False, True, True)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("signed,sqrt,softsign", MODES)
def test_quantize_round_trip(shape, dtype, signed, sqrt, softsign):
    for seed in range(4):
        torch.manual_seed(seed)
        x = (torch.randn(shape) * 10 ** (seed - 3)).to(dtype)
        if not signed:
            x = x.abs()
        q, s = quantize(x, signed=signed, sqrt=sqrt, softsign=softsign)
        assert q.shape == x.shape and q.dtype == (torch.int8 if signed else torch.uint8)
        assert s.dtype == torch.float16 and s.numel() == math.ceil(x.numel() / 32)
        y = dequantize(q, s, signed=signed, sqrt=sqrt, softsign=softsign)
        assert y.dtype == torch.float32 and y.shape == x.shape
        x32 = x.float()
        if x.numel() >= 16:
            assert cossim(x32, y) > 0.999
        # error bound: half a code step of the (companded) grid, in the quantised domain
        xd, yd = (x32.sqrt(), y.sqrt()) if sqrt else (x32, y)
        groups = oracle.num_groups(x.numel())
        pad = groups * 32 - x.numel()
        xa = torch.nn.functional.pad(xd.flatten(), (0, pad)).view(groups, 32)
        ya = torch.nn.functional.pad(yd.flatten(), (0, pad)).view(groups, 32)
        absmax = xa.abs().amax(1, keepdim=True).clamp_min(1e-12)
        qmax = 127.0 if signed else 255.0
        # derivative of the inverse compander is at most 2 (at |n| = 1); fp16 scale adds 2^-11 relative
        step = (2.0 if softsign else 1.0) * 0.5 / qmax
        bound = absmax * (1.6 * step + 2 ** -10)
        assert ((xa - ya).abs() <= bound + 1e-30).all()


@pytest.mark.parametrize("n", [33, 63, 65, 1000, 1023, 1025, 4097])
def test_quantize_tail_group(n):
    """A partial last group is scaled by its own absmax and is no less accurate."""
    torch.manual_seed(n)
    x = torch.randn(n) * 1e-2
    q, s = quantize(x)
    y = dequantize(q, s)
    tail = n - (n // 32) * 32
    tail_absmax = x[-tail:].abs().max()
    assert abs(float(s[-1]) - float(tail_absmax)) <= 3e-3 * float(tail_absmax)
    err = (x - y).abs()
    assert err[-tail:].max() <= 2 * err[:-tail].max() + 1e-12


def test_quantize_zero_and_empty():
    q, s = quantize(torch.zeros(70))
    assert (q == 0).all() and (dequantize(q, s) == 0).all()
    q, s = quantize(torch.zeros(0))
    assert q.numel() == 0 and s.numel() == 0 and dequantize(q, s).numel() == 0


def test_spec_validation():
    QuantizedTensorSpec(signed=True, sqrt=False, softsign=True)
    with pytest.raises(ValueError):
        QuantizedTensorSpec(signed=1)  # type: ignore[arg-type]


def test_maybe_quantized_tensor_states():
    x = torch.randn(100) * 1e-3
    t = MaybeQuantizedTensor(x, try_quantize=True)
    assert t.is_quantized() and t.quantized.dtype == torch.int8 and t.scales.numel() == 4
    assert t.shape == (100,) and t.numel() == 100 and not t.is_cuda
    assert cossim(t.materialize(), x) > 0.999
    sd = t.state_dict("exp_avg", allow_quantized=True)
    assert set(sd) == {"exp_avg::quantized", "exp_avg::scales"}
    sd_plain = t.state_dict("exp_avg", allow_quantized=False)
    assert set(sd_plain) == {"exp_avg"} and sd_plain["exp_avg"].dtype == torch.bfloat16
    u = MaybeQuantizedTensor(x, try_quantize=False, storage_dtype=torch.bfloat16)
    assert not u.is_quantized() and u.data.dtype == torch.bfloat16
    assert u.kernel_scales_or_self is u.data
    # both checkpoint flavours load, mixing them is rejected
    r = MaybeQuantizedTensor.from_state_dict(sd, "exp_avg")
    assert torch.equal(r.quantized, t.quantized) and torch.equal(r.scales, t.scales)
    r2 = MaybeQuantizedTensor.from_state_dict(sd_plain, "exp_avg")
    assert r2.is_quantized()
    with pytest.raises(ValueError):
        MaybeQuantizedTensor.from_state_dict({**sd, **sd_plain}, "exp_avg")


# ---------------------------------------------------------------- error correction


def _oracle_violations(x, dtype):
    return ecc_invariant_violations(
        x, dtype, lambda x, w, mbw: compute_ecc_bits(x, w, master_bytewidth=mbw), reconstruct_fp32_param,
        lambda w: torch.exp2(oracle.ecc_log_scale(w).float()))


@pytest.mark.parametrize("dtype,exponents", [
    (torch.bfloat16, [-127, -126, -100, -20, -1, 0, 1, 17, 100, 126, 127]),
    (torch.float16, [-30, -24, -15, -14, -8, -1, 0, 3, 14, 15]),
])
@pytest.mark.parametrize("sign", [0, 1])
def test_ecc_invariants(dtype, exponents, sign):
    """Every 128th mantissa of a few exponents (field 0 = fp32 subnormals included); the
    GPU suite sweeps all 2^23 mantissas of every exponent."""
    mant = torch.arange(0, 1 << 23, 128, dtype=torch.int32)
    for e in exponents:
        x = fp32_with_exponent(e + 127, sign, mant)
        e8 = compute_ecc_bits(x, x.to(dtype), master_bytewidth=3)
        assert e8.dtype == torch.int8
        assert compute_ecc_bits(x, x.to(dtype), master_bytewidth=4).dtype == torch.int16
        assert _oracle_violations(x, dtype) == {}, (dtype, e, sign)


def test_ecc_zero_and_subnormal_inputs():
    x = torch.tensor([0.0, -0.0, 1e-40, -1e-39, 6e-8, 1e-45])
    for dtype in (torch.bfloat16, torch.float16):
        w = x.to(dtype)
        for mbw in (3, 4):
            e = compute_ecc_bits(x, w, master_bytewidth=mbw)
            r = reconstruct_fp32_param(w, e)
            assert torch.isfinite(r).all()
            assert ((r - x).abs() <= (w.float() - x).abs() + 1e-45).all()


def test_ecc_api_validation():
    w = torch.zeros(4, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        reconstruct_fp32_param(torch.zeros(4), torch.zeros(4, dtype=torch.int8))
    with pytest.raises(ValueError):
        reconstruct_fp32_param(w, torch.zeros(4, dtype=torch.int32))
    with pytest.raises(ValueError):
        compute_ecc_bits(torch.zeros(4, dtype=torch.bfloat16), w)
    with pytest.raises(ValueError):
        compute_ecc_bits(torch.zeros(4), torch.zeros(4))
    with pytest.raises(ValueError):
        compute_ecc_bits(torch.zeros(4), w, master_bytewidth=6)


def test_min_expressible_step():
    # bf16, no ECC: 7 mantissa bits; a weight of 1.0 needs steps > 0.49 * 2^-7
    v = oracle.log2_min_expressible_step(torch.bfloat16, 1.0, 0)
    assert abs(v - (-(16 - 1 - 8) - math.log2(0.49))) < 1e-9
    # 24-bit masters add 8 mantissa bits, 32-bit masters 16
    assert oracle.log2_min_expressible_step(torch.bfloat16, 1.0, 3) == pytest.approx(v - 8)
    assert oracle.log2_min_expressible_step(torch.bfloat16, 1.0, 4) == pytest.approx(v - 16)
    assert oracle.log2_min_expressible_step(torch.bfloat16, 4.5, 0) == pytest.approx(v + 2)


# ---------------------------------------------------------------- property-based (hypothesis)

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

_finite = st.floats(min_value=-6.0e4, max_value=6.0e4, allow_nan=False, allow_infinity=False, width=32)


@settings(max_examples=300, deadline=None, derandomize=True)
@given(st.lists(_finite, min_size=1, max_size=200), st.sampled_from(MODES))
def test_quantiser_error_is_bounded_for_any_input(values, mode):
    """Whatever the values (mixed magnitudes, zeros, a single huge outlier per group, ragged
    tail): every element comes back within half a code step of its group's absmax (times the
    compander's slope), plus the fp16 rounding of the scale."""
    signed, sqrt, softsign = mode
    x = torch.tensor(values, dtype=torch.float32)
    if not signed:
        x = x.abs()
    q, s = quantize(x, signed=signed, sqrt=sqrt, softsign=softsign)
    assert q.shape == x.shape and s.numel() == (x.numel() + 31) // 32
    assert q.dtype == (torch.int8 if signed else torch.uint8)
    y = dequantize(q, s, signed=signed, sqrt=sqrt, softsign=softsign)
    assert torch.isfinite(y).all()
    pad = (-x.numel()) % 32
    xa = torch.nn.functional.pad(x.abs(), (0, pad)).view(-1, 32)
    absmax = xa.max(dim=1).values.repeat_interleave(32)[: x.numel()]
    levels = 127.0 if signed else 255.0
    # scales are stored in fp16: below 6.1e-5 they are subnormal (spacing 6e-8, zero below 3e-8),
    # which bounds the error absolutely instead of relatively for tiny groups
    tiny = 3.0e-8
    if sqrt:
        # codes live in the sqrt domain: sqrt(y) is within half a step of sqrt(x)
        step = absmax.sqrt() * ((2.0 if softsign else 1.0) * 0.5 / levels) * (1 + 1e-3) + 1e-30
        assert ((y.sqrt() - x.sqrt()).abs() <= step + absmax.sqrt() * 2.0 ** -10 + tiny).all()
    else:
        slope = 2.0 if softsign else 1.0   # d(inverse compander)/dy is at most 2 (at |y| = 1)
        step = absmax * (slope * 0.5 / levels)
        assert ((y - x).abs() <= step * (1 + 1e-3) + absmax * 2.0 ** -10 + tiny).all()
    if signed:
        assert (torch.sign(y) * torch.sign(x) >= 0).all()   # a value never changes sign


@settings(max_examples=300, deadline=None, derandomize=True)
@given(st.lists(st.floats(min_value=-(2.0 ** 127), max_value=2.0 ** 127, allow_nan=False, width=32), min_size=1,
                max_size=64),
       st.sampled_from([torch.bfloat16, torch.float16]), st.sampled_from([3, 4]))
def test_master_weight_split_never_hurts_for_any_input(values, dtype, mbw):
    x = torch.tensor(values, dtype=torch.float32)
    w = x.to(dtype)
    keep = torch.isfinite(w.float())
    x, w = x[keep], w[keep]
    if x.numel() == 0:
        return
    e = compute_ecc_bits(x, w, master_bytewidth=mbw)
    r = reconstruct_fp32_param(w, e)
    assert torch.isfinite(r).all()
    ulp32 = torch.exp2(torch.floor(torch.log2(x.abs().clamp_min(2.0 ** -126))) - 23)
    assert ((r - x).abs() <= (w.float() - x).abs() + ulp32).all()
    assert e.to(torch.int32).abs().max() <= (127 if mbw == 3 else 32767)


@pytest.mark.parametrize("signed,sqrt,softsign", [(True, False, True), (False, True, False)])
def test_zero_state_by_memset_equals_quantised_zeros(signed, sqrt, softsign):
    from flashoptim_b200.optim.state import MaybeQuantizedTensor

    x = torch.zeros(5, 7)
    a = MaybeQuantizedTensor(x, signed=signed, sqrt=sqrt, softsign=softsign)
    b = MaybeQuantizedTensor.zeros(x, signed=signed, sqrt=sqrt, softsign=softsign)
    assert a.quantized.dtype == b.quantized.dtype and a.quantized.shape == b.quantized.shape
    assert torch.equal(a.quantized, b.quantized) and torch.equal(a.scales, b.scales)
    assert torch.equal(a.materialize(), b.materialize())
    plain = MaybeQuantizedTensor.zeros(x, try_quantize=False, storage_dtype=torch.bfloat16)
    assert not plain.is_quantized() and plain.data.dtype == torch.bfloat16 and plain.data.shape == x.shape
