"""The FAST forms of the master-weight split, i.e. what the step kernels really execute
(``fo_common.cuh``: exponent taken by one AND, ``2^-E`` by an integer subtraction, rounding
through the mantissa trick), swept over all 2^23 fp32 mantissas of every exponent and both signs.

Part one feeds arbitrary fp32 values to the same device functions through the library's test
entry points (``fo_probe_fast_ecc_split`` / ``fo_probe_fast_ecc_merge``) and evaluates the seven
invariants of the reference's ``test/test_ecc_invariants.py:24-156``.  Part two goes through the
real ``fo_adam_step`` / ``fo_momentum_step`` kernels with a zero learning rate, zero weight decay
and a zero gradient: the master value that comes out must be the one that went in, up to the
rounding of one re-encoding, whatever the bits of parameter and correction.  Part three gives
the in-kernel quantiser groups that are hard for it.

Documented limits of the fast forms (they differ from the exact kernels only here):
bf16 values below 2^-126 (zero, subnormals) carry no correction; values whose bf16 rounding has
magnitude 2^127 or more get code 0 (their ``2^-E`` is not a normal fp32 number).  The invariant
sweep stops short of both.
"""


import pytest
import torch

from flashoptim_b200 import compute_ecc_bits, reconstruct_fp32_param
from flashoptim_b200.ops import native, oracle
from flashoptim_b200.ops.quant import quantize
from flashoptim_b200.ops.step import (
    AdamHyper, MomentumHyper, SegmentTable, launch_adam, launch_momentum, make_rows,
)
from helpers import ecc_invariant_violations, fp32_with_exponent

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def fast_split(x, dtype, err_bytes):
    lib = native.load()
    narrow = torch.empty(x.numel(), dtype=dtype, device=x.device)
    ecc = torch.empty(x.numel(), dtype=torch.int8 if err_bytes == 1 else torch.int16, device=x.device)
    native.check(lib.fo_probe_fast_ecc_split(x.data_ptr(), native.DTYPE_CODE[dtype], err_bytes, narrow.data_ptr(),
                                             ecc.data_ptr(), x.numel(), _stream()), "fo_probe_fast_ecc_split")
    return narrow, ecc


def fast_merge(narrow, ecc):
    lib = native.load()
    out = torch.empty(narrow.numel(), dtype=torch.float32, device=narrow.device)
    native.check(lib.fo_probe_fast_ecc_merge(narrow.data_ptr(), native.DTYPE_CODE[narrow.dtype], ecc.data_ptr(),
                                             ecc.element_size(), out.data_ptr(), narrow.numel(), _stream()),
                 "fo_probe_fast_ecc_merge")
    return out


def _half_ulp(w):
    return torch.exp2(oracle.ecc_log_scale(w).float())


@pytest.mark.parametrize("dtype,fields", [
    (torch.bfloat16, range(1, 253)),          # [2^-126, 2^126): nothing here rounds to 2^127 or beyond
    (torch.float16, range(127 - 30, 127 + 16)),  # 2^-30 .. 2^15: fp16 subnormals included
])
@pytest.mark.parametrize("sign", [0, 1])
def test_fast_split_invariants_all_mantissas(dtype, fields, sign):
    mant = torch.arange(0, 1 << 23, dtype=torch.int32, device="cuda")
    bad = {}
    for field in fields:
        x = fp32_with_exponent(field, sign, mant)
        finite = torch.isfinite(x.to(dtype).float())
        narrow_of = {}

        def encode(xs, w, mbw):
            # the helper hands over the finite subset; the probe wants whole units of 8
            pad = (-xs.numel()) % 8
            xp = torch.cat([xs, xs.new_zeros(pad)]) if pad else xs
            n, e = fast_split(xp.contiguous(), dtype, mbw - 2)
            narrow_of[mbw] = n[:xs.numel()]
            return e[:xs.numel()]

        def decode(w, codes):
            n0 = w.numel()
            pad = (-n0) % 8
            if pad:
                w = torch.cat([w, w.new_zeros(pad)])
                codes = torch.cat([codes, codes.new_zeros(pad)])
            return fast_merge(w.contiguous(), codes.contiguous())[:n0]

        v = ecc_invariant_violations(x, dtype, encode, decode, _half_ulp)
        # the kernel's own narrowing is the round-to-nearest-even cast
        want = x[finite].to(dtype)
        for mbw, n in narrow_of.items():
            if not torch.equal(n.view(torch.int16), want.view(torch.int16)):
                v[f"narrowing differs from the cast (mbw {mbw})"] = int(
                    (n.view(torch.int16) != want.view(torch.int16)).sum())
        if v:
            bad[field - 127] = v
    assert not bad, bad


def _noop_step(kind, p, ecc, err_bytes):
    """One real kernel launch that must not move the master value: lr = 0, no decay, zero gradient."""
    n = p.numel()
    dev = p.device
    grad = torch.zeros(n, dtype=p.dtype, device=dev)
    m, ms = quantize(torch.zeros(n, device=dev))
    table = SegmentTable(torch.device("cuda", torch.cuda.current_device()))
    if kind == "adam":
        v, vs = quantize(torch.zeros(n, device=dev), signed=False, sqrt=True, softsign=False)
        rows = make_rows([p], [grad], [ecc], [m], [ms], [v], [vs])
        launch_adam(table, rows, p.dtype, err_bytes, True,
                    AdamHyper(lr=0.0, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True))
    else:
        rows = make_rows([p], [grad], [ecc], [m], [ms], [None], [None])
        launch_momentum(table, rows, p.dtype, err_bytes, native.FO_STATE_Q8,
                        MomentumHyper(lr=0.0, mom_coef=0.9, update_coef=1.0, weight_decay=0.0, decoupled=True))


@pytest.mark.parametrize("kind", ["adam", "momentum"])
@pytest.mark.parametrize("dtype,fields", [
    (torch.bfloat16, [1, 2, 24, 64, 100, 120, 126, 127, 128, 140, 200, 251, 252]),  # 253 rounds up to 2^127
    # fp16: subnormals, the smallest normals, around one, and 2^14; in the top binade the master
    # value 65504 + half a spacing narrows to infinity, here as in the reference's recipe
    (torch.float16, [127 - 24, 127 - 15, 127 - 14, 127 - 1, 127, 127 + 14]),
])
@pytest.mark.parametrize("err_bytes", [1, 2])
def test_a_step_that_changes_nothing_keeps_every_master_value(kind, dtype, fields, err_bytes):
    """(parameter, correction) pairs covering all 2^23 mantissas of a binade and both signs go
    through the real step kernels.  Where the parameter bits come back unchanged the correction
    must too, up to the fp32 rounding of the reconstructed value (0 codes for int8, 1 for
    int16 on bf16, 8 on fp16, whose 27 bits exceed fp32); the master value may move by at most
    half a code step plus that rounding; and nothing may become non-finite."""
    mant = torch.arange(0, 1 << 23, dtype=torch.int32, device="cuda")
    s_max = 127.0 if err_bytes == 1 else 32767.0
    mbits = 7 if dtype == torch.bfloat16 else 10
    code_noise = 0 if err_bytes == 1 else (1 if dtype == torch.bfloat16 else 8)
    for field in fields:
        for sign in (0, 1):
            x = fp32_with_exponent(field, sign, mant)
            p0, e0 = fast_split(x, dtype, err_bytes)
            ok = torch.isfinite(p0.float())
            before = reconstruct_fp32_param(p0, e0)
            p, e = p0.clone(), e0.clone()
            _noop_step(kind, p, e, err_bytes)
            after = reconstruct_fp32_param(p, e)
            tag = (kind, dtype, field - 127, sign, err_bytes)
            assert torch.isfinite(after[ok]).all(), tag
            same = (p.view(torch.int16) == p0.view(torch.int16)) & ok
            drift = (e[same].to(torch.int32) - e0[same].to(torch.int32)).abs()
            assert int(drift.max()) <= code_noise, (tag, int(drift.max()))
            # where a correction of exactly half a spacing carried the narrow value across a power
            # of two, the new code is counted in the wider binade's steps
            half_ulp = torch.maximum(_half_ulp(p0), _half_ulp(p))
            ulp32 = torch.exp2(torch.floor(torch.log2(before.abs().clamp_min(2.0 ** -126))) - 23)
            bound = half_ulp * (0.5 / s_max) * 1.01 + 2 * ulp32
            moved = (after - before).abs()
            assert bool((moved[ok] <= bound[ok]).all()), (tag, float((moved[ok] / bound[ok]).max()))
            # the narrow value itself moves at most to a neighbour (a correction of exactly half a
            # spacing may round either way)
            step_ulps = ((p.float() - p0.float()).abs() / (2 * _half_ulp(p0)))[ok]
            assert float(step_ulps.max()) <= 1.0 + 2.0 ** -mbits, (tag, float(step_ulps.max()))


def _momentum_requantise(values):
    """Runs the momentum kernel so that its new state equals ``values`` exactly (old state zero,
    momentum 0, no dampening): what comes back is the in-kernel quantiser's output for them."""
    n = values.numel()
    dev = values.device
    p = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    m, ms = quantize(torch.zeros(n, device=dev))
    rows = make_rows([p], [values], [None], [m], [ms], [None], [None])
    launch_momentum(SegmentTable(torch.device("cuda", torch.cuda.current_device())), rows, torch.bfloat16, 0,
                    native.FO_STATE_Q8, MomentumHyper(lr=0.0, mom_coef=0.0, update_coef=1.0, weight_decay=0.0,
                                                      decoupled=True))
    torch.cuda.synchronize()
    return m, ms


@pytest.mark.parametrize("case", ["one huge, 31 tiny", "all equal", "absmax beyond fp16", "absmax below fp16",
                                  "alternating signs at full scale", "zeros"])
def test_in_kernel_quantiser_on_hard_groups(case):
    g = torch.Generator(device="cuda").manual_seed(3)
    n = 32 * 512
    if case == "one huge, 31 tiny":
        x = torch.randn(n, device="cuda", generator=g) * 1e-6
        x[::32] = 3.0
    elif case == "all equal":
        x = torch.full((n,), 0.37, device="cuda")
        x[n // 2:] = -0.37
    elif case == "absmax beyond fp16":
        x = torch.randn(n, device="cuda", generator=g) * 3e4
        x[::32] = 1.0e5  # > 65504: the fp16 scale overflows, as it does in the reference's recipe
    elif case == "absmax below fp16":
        x = torch.randn(n, device="cuda", generator=g) * 1e-9  # scales below 6e-8 are stored as fp16 zero
    elif case == "alternating signs at full scale":
        x = torch.ones(n, device="cuda")
        x[1::2] = -1.0
    else:
        x = torch.zeros(n, device="cuda")
    x = x.to(torch.bfloat16)
    codes, scales = _momentum_requantise(x)
    want_codes, want_scales = oracle.quantize_ref(x.float().cpu())
    d = (codes.cpu().to(torch.int16) - want_codes.to(torch.int16)).abs()
    assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 0.02, (case, int(d.max()))
    got_s, want_s = scales.cpu().float(), want_scales.float()
    both_inf = torch.isinf(got_s) & torch.isinf(want_s)
    finite = torch.isfinite(want_s)
    assert bool((torch.isinf(got_s) == torch.isinf(want_s)).all()), case
    assert torch.allclose(got_s[finite], want_s[finite], rtol=2 ** -10, atol=0), case
    assert int(both_inf.sum()) == (n // 32 if case == "absmax beyond fp16" else 0), case
    # what a later step would read back
    back = oracle.dequantize_ref(codes.cpu(), scales.cpu())
    ref = oracle.dequantize_ref(want_codes, want_scales)
    both = torch.isfinite(back) & torch.isfinite(ref)
    assert bool((torch.isfinite(back) == torch.isfinite(ref)).all()), case
    # one code step of the compander near full scale is at most scale * 2 / 127
    assert bool(((back[both] - ref[both]).abs() <= want_s.repeat_interleave(32)[both] * (2.2 / 127)).all()), case


def test_exact_and_fast_splits_agree_on_a_binade():
    """Same input, exact kernels vs fast forms: identical narrow values, codes within one
    (ties round to even in the fast form, away from zero in the exact one)."""
    mant = torch.arange(0, 1 << 23, dtype=torch.int32, device="cuda")
    for dtype, field in ((torch.bfloat16, 120), (torch.float16, 118)):
        x = fp32_with_exponent(field, 0, mant)
        for err_bytes in (1, 2):
            narrow, codes = fast_split(x, dtype, err_bytes)
            w = x.to(dtype)
            assert torch.equal(narrow.view(torch.int16), w.view(torch.int16))
            exact = compute_ecc_bits(x, w, master_bytewidth=2 + err_bytes)
            d = (codes.to(torch.int32) - exact.to(torch.int32)).abs()
            assert int(d.max()) <= 1, (dtype, err_bytes, int(d.max()))
