"""All 2^23 fp32 mantissas of every exponent and both signs through the CUDA
master-weight split kernels (bf16: every fp32 exponent field incl. subnormals; fp16: the
exponents fp16 covers, subnormals included) — the sweep of the reference's
``test/test_ecc_invariants.py:24-156``, with the invariants stated on fp32 errors and
evaluated with torch ops on the device instead of a counting kernel."""

import pytest
import torch

from flashoptim_b200 import compute_ecc_bits, reconstruct_fp32_param
from flashoptim_b200.ops import oracle
from helpers import ecc_invariant_violations, fp32_with_exponent

pytestmark = pytest.mark.gpu


def _half_ulp(w):
    return torch.exp2(oracle.ecc_log_scale(w).float())


@pytest.mark.parametrize("dtype,fields", [
    (torch.bfloat16, range(0, 255)),
    (torch.float16, range(127 - 30, 127 + 16)),
])
@pytest.mark.parametrize("sign", [0, 1])
def test_ecc_invariants_all_mantissas(dtype, fields, sign):
    mant = torch.arange(0, 1 << 23, dtype=torch.int32, device="cuda")
    bad = {}
    for field in fields:
        x = fp32_with_exponent(field, sign, mant)
        v = ecc_invariant_violations(
            x, dtype, lambda x, w, mbw: compute_ecc_bits(x, w, master_bytewidth=mbw), reconstruct_fp32_param,
            _half_ulp)
        if v:
            bad[field - 127] = v
    assert not bad, bad


@pytest.mark.parametrize("dtype,field", [
    (torch.bfloat16, 120), (torch.bfloat16, 0),
    # the kernels switch from two scale factors to one at |w| = 2^-94 (bf16): both sides of it
    (torch.bfloat16, 32), (torch.bfloat16, 33), (torch.bfloat16, 34), (torch.bfloat16, 254),
    (torch.float16, 118), (torch.float16, 127 - 20), (torch.float16, 127 + 15),
])
def test_cuda_codes_equal_the_cpu_formulation_on_a_full_binade(dtype, field):
    """Split and merge, bit for bit with the PyTorch formulation, over all 2^23 mantissas of one
    fp32 exponent (field 0 and fp16 field 107: subnormal narrow values; 254 / 142: the top)."""
    mant = torch.arange(0, 1 << 23, dtype=torch.int32)
    x = fp32_with_exponent(field, 1, mant)
    w = x.to(dtype)
    for mbw in (3, 4):
        got = compute_ecc_bits(x.cuda(), w.cuda(), master_bytewidth=mbw)
        want = oracle.ecc_encode_ref(x, w, mbw - 2)
        assert torch.equal(got.cpu(), want), (dtype, field, mbw)
        back = reconstruct_fp32_param(w.cuda(), got).cpu()
        assert torch.equal(back.view(torch.int32), oracle.ecc_decode_ref(w, want).view(torch.int32)), (dtype, field, mbw)
