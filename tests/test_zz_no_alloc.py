"""The allocation-free Adam entry point (``fo_adam_step_noalloc``), called through
its exported C symbol, against the regular multi-tensor entry point.

Some callers cannot allocate device memory when they step: a gradient hook in
the middle of backward (an allocation would synchronise the device) or a host
program whose memory all belongs to another pool.  For them the library keeps
the segment table in a built-in device array; this test checks that the
variant computes what ``fo_adam_step`` computes, on two consecutive calls that
share that array, and that oversize requests are refused.

This file sorts last on purpose: a run that stops at the first failure has
then already exercised every other test.
"""

import ctypes

import pytest
import torch

from flashoptim_b200.ops import native
from flashoptim_b200.ops.quant import compute_ecc_bits, quantize
from flashoptim_b200.ops.step import AdamHyper, SegmentTable, launch_adam, make_rows

pytestmark = pytest.mark.gpu

SIZES = [4096, 33, 1, 50257, 4097, 65536 + 5, 7, 1000, 2048 * 3, 31] * 3  # 30 tensors: table path


def _entry():
    lib = native.load()
    fn = lib.fo_adam_step_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.POINTER(native.FoAdamHyper), ctypes.c_void_p]
    return fn


def _problem(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for n in SIZES:
        p32 = torch.randn(n, device="cuda", generator=g) * 0.02
        p = p32.to(torch.bfloat16)
        grad = (torch.randn(n, device="cuda", generator=g) * 1e-3).to(torch.bfloat16)
        ecc = compute_ecc_bits(p32, p, master_bytewidth=3)
        m, ms = quantize(torch.randn(n, device="cuda", generator=g) * 1e-3)
        v, vs = quantize((torch.randn(n, device="cuda", generator=g) * 1e-3).square(),
                         signed=False, sqrt=True, softsign=False)
        out.append([p, grad, ecc, m, ms, v, vs])
    return out


def _rows(prob):
    cols = list(zip(*prob))
    return make_rows(*cols)


def _assert_same(a, b, tag):
    names = ["param", "grad", "ecc", "exp_avg", "exp_avg.scales", "exp_avg_sq", "exp_avg_sq.scales"]
    for i, (ta, tb) in enumerate(zip(a, b)):
        for name, x, y in zip(names, ta, tb):
            if x.dtype in (torch.int8, torch.uint8):
                d = (x.to(torch.int16) - y.to(torch.int16)).abs()
                assert d.max() <= 1 and (d != 0).float().mean() < 0.02, f"{tag}: tensor {i} {name}"
            else:
                assert torch.allclose(x.float(), y.float(), rtol=2 ** -7, atol=1e-12), f"{tag}: tensor {i} {name}"


def test_noalloc_adam_matches_table_entry_point_twice():
    fn = _entry()
    ref, new = _problem(7), _problem(7)
    dev = torch.device("cuda", torch.cuda.current_device())
    table = SegmentTable(dev)
    stream = torch.cuda.current_stream().cuda_stream
    for step in (1, 2):
        h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, step=step, decoupled=True)
        launch_adam(table, _rows(ref), torch.bfloat16, 1, True, h)
        rows = _rows(new)
        hc = h.to_c()
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = fn(rows.ctypes.data, rows.shape[0], native.FO_BF16, 1, 1, ctypes.byref(hc), stream)
        # the caller's array is free again when the call returns, whatever memory it lives in
        rows[:] = -1
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert rc == 0, rc
        # the driver's own view of the device: nothing was allocated behind the caller's back.
        # Checked on the second call: during the first one the driver may still load the
        # kernels' code onto the device (lazy module loading), which is not an allocation of
        # this library's and happens once.
        if step == 2:
            assert free_after >= free_before, (free_before, free_after)
        _assert_same(ref, new, f"call {step}")
    assert table.uploads >= 1  # the regular path really went through its device table


def test_noalloc_refuses_oversize_requests():
    fn = _entry()
    import numpy as np

    n_seg = 2049
    rows = np.zeros((n_seg, 8), dtype=np.int64)
    rows[:, 7] = 8
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True).to_c()
    rc = fn(rows.ctypes.data, n_seg, native.FO_BF16, 1, 1, ctypes.byref(h),
            torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    torch.cuda.synchronize()


def test_noalloc_refusals_launch_nothing():
    """Every refusal happens before the first launch: bad arguments (-3) and more than 2^31
    chunks (-2) leave the tensors of a valid problem untouched."""
    fn = _entry()
    prob = _problem(11)
    before = [[t.clone() for t in ts] for ts in prob]
    rows = _rows(prob)
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True).to_c()
    stream = torch.cuda.current_stream().cuda_stream
    n = rows.shape[0]
    assert fn(rows.ctypes.data, -1, native.FO_BF16, 1, 1, ctypes.byref(h), stream) == -3       # negative count
    assert fn(None, n, native.FO_BF16, 1, 1, ctypes.byref(h), stream) == -3                     # no segments
    assert fn(rows.ctypes.data, n, native.FO_BF16, 1, 1, None, stream) == -3                    # no hyper-parameters
    assert fn(rows.ctypes.data, n, native.FO_BF16, 3, 1, ctypes.byref(h), stream) == -3         # err_bytes 3
    assert fn(rows.ctypes.data, n, native.FO_FP32, 1, 1, ctypes.byref(h), stream) == -3         # fp32 has no codes
    assert fn(rows.ctypes.data, n, 7, 1, 1, ctypes.byref(h), stream) == -3                      # unknown dtype
    neg = rows.copy()
    neg[3, 7] = -5
    assert fn(neg.ctypes.data, n, native.FO_BF16, 1, 1, ctypes.byref(h), stream) == -3          # negative length
    huge = rows.copy()
    huge[0, 7] = 2 ** 42  # 2^31 chunks of 2048 elements in one tensor
    assert fn(huge.ctypes.data, n, native.FO_BF16, 1, 1, ctypes.byref(h), stream) == -2
    torch.cuda.synchronize()
    for ts, bs in zip(prob, before):
        for t, b in zip(ts, bs):
            assert torch.equal(t, b)
