"""sm_100a kernels against the PyTorch fp32 formulation of the same operations."""

import pytest
import torch

from flashoptim_b200.ops import native, oracle
from flashoptim_b200.ops.quant import (
    compute_ecc_bits, dequantize, maxabs, quantize, reconstruct_fp32_param,
)
from flashoptim_b200.ops.step import (
    AdamHyper, MomentumHyper, SegmentTable, launch_adam, launch_momentum, make_rows,
)

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["staged", "register"], autouse=True)
def step_variant(request):
    """Every test runs with the bulk-copy staged kernels (default) and with the register-path kernels."""
    from flashoptim_b200.ops.step import check_kernel_status, set_step_variant

    set_step_variant(1 if request.param == "staged" else 0)
    yield request.param
    set_step_variant(1)
    check_kernel_status()

SIZES = [1, 5, 31, 32, 33, 999, 1025, 4097, 2048 * 8 + 3, 1 << 20]
DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def _rand(n, dtype, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(n, device="cuda", generator=g) * scale).to(dtype)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("signed,sqrt,softsign", [(True, False, True), (False, True, False),
                                                  (True, False, False), (False, True, True)])
def test_quantize_matches_oracle_bitwise(n, dtype, signed, sqrt, softsign):
    x = _rand(n, dtype, 3e-3)
    if not signed:
        x = x.abs()
    q, s = quantize(x, signed=signed, sqrt=sqrt, softsign=softsign)
    q_ref, s_ref = oracle.quantize_ref(x.cpu(), signed=signed, sqrt=sqrt, softsign=softsign)
    assert q.dtype == q_ref.dtype and s.dtype == torch.float16
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref)
    d = dequantize(q, s, signed=signed, sqrt=sqrt, softsign=softsign)
    d_ref = oracle.dequantize_ref(q_ref, s_ref, signed=signed, sqrt=sqrt, softsign=softsign)
    assert torch.equal(d.cpu(), d_ref)


@pytest.mark.parametrize("n", [1, 33, 4097, 1 << 18])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mbw", [3, 4])
def test_ecc_matches_oracle_bitwise(n, dtype, mbw):
    x = _rand(n, torch.float32, 0.05)
    x[::7] *= 1e-30 if dtype == torch.bfloat16 else 1e-6  # subnormal-ish region
    x[::11] = 0
    w = x.to(dtype)
    e = compute_ecc_bits(x, w, master_bytewidth=mbw)
    e_ref = oracle.ecc_encode_ref(x.cpu(), w.cpu(), mbw - 2)
    assert torch.equal(e.cpu(), e_ref)
    r = reconstruct_fp32_param(w, e)
    r_ref = oracle.ecc_decode_ref(w.cpu(), e_ref)
    assert torch.equal(r.cpu(), r_ref)
    # the correction must not hurt and usually helps
    assert (r - x).abs().max() <= (w.float() - x).abs().max()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("code_dtype", [torch.int8, torch.int16])
def test_ecc_decode_every_code_value_bitwise(dtype, code_dtype):
    """Every code (all 255 int8 values, all 65535 int16 values) against several parameter
    values, bit for bit with the PyTorch formulation: the kernel divides the code by its range
    through a reciprocal and one FMA correction, which has to equal IEEE division everywhere."""
    lim = 127 if code_dtype == torch.int8 else 32767
    codes = torch.arange(-lim, lim + 1, dtype=torch.int32)
    params = torch.tensor([1.0, -0.0371, 3.1e-5, 250.0, 6.1e-5 if dtype == torch.float16 else 1e-30], dtype=dtype)
    w = params.repeat_interleave(codes.numel())
    e = codes.repeat(params.numel()).to(code_dtype)
    got = reconstruct_fp32_param(w.cuda(), e.cuda()).cpu()
    assert torch.equal(got, oracle.ecc_decode_ref(w, e))


@pytest.mark.parametrize("off", [1, 3, 4, 8])
@pytest.mark.parametrize("n", [7, 250, 4099])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("err_bytes", [1, 2])
def test_ecc_kernels_on_offset_views(off, n, dtype, err_bytes):
    """Inputs and outputs that start `off` elements into their buffers (no, 4-, 8- or 16-byte
    alignment depending on the element size) take the element-wise or the narrower vector
    paths: same bits as the oracle, and nothing written outside the view."""
    lib = native.load()
    st = native.stream_ptr(torch.device("cuda", 0))
    x = _rand(n + off, torch.float32, 0.05)[off:]
    w = _rand(n + off, dtype, 1.0)[off:]
    w.copy_(x.to(dtype))
    code_dtype = torch.int8 if err_bytes == 1 else torch.int16
    e_buf = torch.full((n + off + 9,), 77, dtype=code_dtype, device="cuda")
    rc = lib.fo_ecc_encode(x.data_ptr(), w.data_ptr(), native.DTYPE_CODE[dtype], e_buf[off:].data_ptr(), err_bytes, n, st)
    assert rc == 0
    e_ref = oracle.ecc_encode_ref(x.cpu(), w.cpu(), err_bytes)
    assert torch.equal(e_buf[off:off + n].cpu(), e_ref)
    assert (e_buf[:off] == 77).all() and (e_buf[off + n:] == 77).all()
    r_buf = torch.full((n + off + 9,), -5.0, dtype=torch.float32, device="cuda")
    rc = lib.fo_ecc_decode(w.data_ptr(), native.DTYPE_CODE[dtype], e_buf[off:].data_ptr(), err_bytes,
                           r_buf[off:].data_ptr(), n, st)
    assert rc == 0
    assert torch.equal(r_buf[off:off + n].cpu(), oracle.ecc_decode_ref(w.cpu(), e_ref))
    assert (r_buf[:off] == -5.0).all() and (r_buf[off + n:] == -5.0).all()


@pytest.mark.parametrize("off", [1, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
def test_quantize_on_offset_views(off, dtype):
    """fp32 input 16 bytes into its buffer uses two 16-byte loads per unit instead of one
    32-byte load; odd offsets go element by element; the fp32 output likewise."""
    n = 4099
    x = _rand(n + off, dtype, 3e-3)[off:]
    q_buf = torch.full((n + off + 40,), 99, dtype=torch.int8, device="cuda")
    q, s = quantize(x, out_int8=q_buf[off:off + n], signed=True, sqrt=False, softsign=True)
    q_ref, s_ref = oracle.quantize_ref(x.cpu(), signed=True, sqrt=False, softsign=True)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    assert (q_buf[:off] == 99).all() and (q_buf[off + n:] == 99).all()
    d_buf = torch.full((n + off + 40,), -5.0, dtype=torch.float32, device="cuda")
    d = dequantize(q, s, out_float=d_buf[off:off + n], signed=True, sqrt=False, softsign=True)
    assert torch.equal(d.cpu(), oracle.dequantize_ref(q_ref, s_ref, signed=True, sqrt=False, softsign=True))
    assert (d_buf[:off] == -5.0).all() and (d_buf[off + n:] == -5.0).all()


def test_maxabs():
    x = _rand(100003, torch.bfloat16, 2.0)
    assert maxabs(x) == float(x.abs().max())


def _make_problem(n, dtype, err, quantized, states, seed, unaligned=False):
    """Random param / grad / state on device plus fp32 copies of the true values."""
    off = 1 if unaligned else 0
    p32 = _rand(n + off, torch.float32, 0.02, seed)[off:]
    g = _rand(n + off, dtype, 1e-3, seed + 1)[off:]
    p = _rand(n + off, dtype, 1.0, seed + 5)[off:]
    p.copy_(p32.to(dtype))
    ecc = None
    if err:
        ecc = torch.zeros(n + off, dtype=torch.int8 if err == 1 else torch.int16, device="cuda")[off:]
        ecc.copy_(compute_ecc_bits(p32, p.contiguous(), master_bytewidth=2 + err))
    # unquantised states live in the param dtype: keep v = O(1e-3) so that fp16 can hold it
    sc = 3e-2 if (dtype == torch.float16 and not quantized) else 1e-3
    m32 = _rand(n, torch.float32, sc, seed + 2)
    v32 = _rand(n, torch.float32, sc, seed + 3).square()
    st = []
    for k in range(states):
        src = m32 if k == 0 else v32
        if quantized:
            q = torch.zeros(n + 8 * off, dtype=torch.int8 if k == 0 else torch.uint8, device="cuda")[8 * off:]
            qq, ss = quantize(src, signed=(k == 0), sqrt=(k == 1), softsign=(k == 0))
            q.copy_(qq)
            st.append((q, ss))
        else:
            f = torch.zeros(n + off, dtype=dtype, device="cuda")[off:]
            f.copy_(src.to(dtype))
            st.append((f, None))
    return p, g, ecc, st


def _oracle_adam(p, g, ecc, st, quantized, h: AdamHyper):
    pc, gc = p.cpu(), g.cpu()
    ec = None if ecc is None else ecc.cpu()
    if quantized:
        m = oracle.dequantize_ref(st[0][0].cpu(), st[0][1].cpu())
        v = oracle.dequantize_ref(st[1][0].cpu(), st[1][1].cpu(), signed=False, sqrt=True, softsign=False)
    else:
        m, v = st[0][0].cpu().float(), st[1][0].cpu().float()
    return oracle.adam_math(
        oracle.read_param_fp32(pc, ec), gc.float(), m, v, lr=h.lr, beta1=h.beta1, beta2=h.beta2,
        eps=h.eps, weight_decay=h.weight_decay, decoupled=h.decoupled, step=h.step,
    )


def _check_step_outputs(p, ecc, st, quantized, dtype, p_new, states_new, specs, tag, p_old32=None,
                        param_mask=None):
    """Compare device results after a fused step with the oracle's fp32 results.

    The parameter is compared in master space: (narrow value + decoded correction)
    against the oracle's fp32 value, within the resolution of the master format
    plus the fp32 error of the update itself (the kernel uses approximate
    reciprocal / square root: ~4e-6 relative on the step taken).
    """
    err = 0 if ecc is None else ecc.element_size()
    got = p.cpu()
    upd = (p_new - p_old32).abs() if p_old32 is not None else torch.zeros_like(p_new)
    tol_abs = 4e-6 * upd + 4e-7 * p_new.abs() + 1e-10
    if dtype == torch.float32:
        diff = (got - p_new).abs()
        bound = tol_abs
    elif err:
        rec = oracle.ecc_decode_ref(got, ecc.cpu())
        half_ulp = torch.exp2(oracle.ecc_log_scale(got).float())
        smax = 127.0 if err == 1 else 32767.0
        diff = (rec - p_new).abs()
        bound = half_ulp * (0.75 if err == 1 else 2.0) / smax + tol_abs
    else:
        half_ulp = torch.exp2(oracle.ecc_log_scale(got).float())
        diff = (got.float() - p_new).abs()
        bound = half_ulp * 1.01 + tol_abs
    ok = diff <= bound
    if param_mask is not None:
        ok = ok | ~param_mask
    assert ok.all(), f"{tag}: param off by up to {(diff / bound).max().item():.2f}x the bound"
    if dtype != torch.float32 and param_mask is None:
        mism = (got != p_new.to(dtype)).float().mean().item()
        assert mism < 1e-2, f"{tag}: {mism:.2e} of params differ from the rounded oracle value"
    for (tensor, scales), want32, spec in zip(st, states_new, specs):
        if quantized:
            q_ref, s_ref = oracle.quantize_ref(want32, **spec)
            dq = (tensor.cpu().to(torch.int16) - q_ref.to(torch.int16)).abs()
            assert dq.max() <= 1, f"{tag}: code off by {dq.max().item()}"
            assert (dq != 0).float().mean() < 0.02, f"{tag}: {(dq != 0).float().mean():.3f} codes differ"
            s_got, s_want = scales.cpu().float(), s_ref.float()
            assert torch.allclose(s_got, s_want, rtol=2e-3, atol=1e-12), tag
        else:
            ref = want32.to(dtype).float()
            atol = 1e-5 * float(ref.abs().max())  # cancellation near zero leaves absolute error
            assert torch.allclose(tensor.cpu().float(), ref, rtol=2 ** -6, atol=atol), tag


def _old_master(p, ecc):
    return oracle.read_param_fp32(p.cpu(), None if ecc is None else ecc.cpu())


ADAM_CASES = [
    (torch.bfloat16, 1, True), (torch.bfloat16, 2, True), (torch.bfloat16, 0, True),
    (torch.bfloat16, 1, False), (torch.bfloat16, 0, False), (torch.float16, 1, True),
    (torch.float16, 2, False), (torch.float32, 0, True), (torch.float32, 0, False),
]


@pytest.mark.parametrize("n", [1, 31, 33, 1025, 4097, 2048 * 8 * 3 + 77])
@pytest.mark.parametrize("dtype,err,quantized", ADAM_CASES)
@pytest.mark.parametrize("decoupled", [True, False])
def test_fused_adam_single_tensor(n, dtype, err, quantized, decoupled):
    p, g, ecc, st = _make_problem(n, dtype, err, quantized, 2, seed=n)
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5 if decoupled else 1e-2,
                  step=3, decoupled=decoupled)
    p_new, m_new, v_new = _oracle_adam(p, g, ecc, st, quantized, h)
    p_old = _old_master(p, ecc)
    rows = make_rows([p], [g], [ecc], [st[0][0]], [st[0][1]], [st[1][0]], [st[1][1]])
    launch_adam(SegmentTable(p.device), rows, dtype, err, quantized, h)
    torch.cuda.synchronize()
    specs = [dict(signed=True, sqrt=False, softsign=True), dict(signed=False, sqrt=True, softsign=False)]
    _check_step_outputs(p, ecc, st, quantized, dtype, p_new, [m_new, v_new], specs, f"adam n={n}", p_old)


@pytest.mark.parametrize("unaligned", [False, True])
def test_fused_adam_multi_tensor_table(unaligned):
    """40 tensors of odd sizes in one launch through the device-resident table,
    with guard bytes around every buffer."""
    sizes = [1, 7, 32, 33, 100, 4096, 4097, 50257, 65536 + 5] * 5
    sizes = sizes[:40]
    dtype, err, quantized = torch.bfloat16, 1, True
    probs = [_make_problem(n, dtype, err, quantized, 2, seed=100 + i, unaligned=unaligned)
             for i, n in enumerate(sizes)]
    h = AdamHyper(lr=2e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=2e-5, step=1, decoupled=True)
    wants = [_oracle_adam(p, g, ecc, st, quantized, h) for p, g, ecc, st in probs]
    olds = [_old_master(q[0], q[2]) for q in probs]
    rows = make_rows(
        [q[0] for q in probs], [q[1] for q in probs], [q[2] for q in probs],
        [q[3][0][0] for q in probs], [q[3][0][1] for q in probs],
        [q[3][1][0] for q in probs], [q[3][1][1] for q in probs],
    )
    table = SegmentTable(torch.device("cuda", torch.cuda.current_device()))
    launch_adam(table, rows, dtype, err, quantized, h)
    torch.cuda.synchronize()
    assert table.uploads == 1
    specs = [dict(signed=True, sqrt=False, softsign=True), dict(signed=False, sqrt=True, softsign=False)]
    for i, ((p, g, ecc, st), (pn, mn, vn)) in enumerate(zip(probs, wants)):
        _check_step_outputs(p, ecc, st, quantized, dtype, pn, [mn, vn], specs, f"seg {i} n={sizes[i]}", olds[i])
    # same addresses again: nothing is re-uploaded
    launch_adam(table, rows, dtype, err, quantized, h)
    torch.cuda.synchronize()
    assert table.uploads == 1


@pytest.mark.parametrize("kind", ["adam", "lion"])
def test_large_launch_grid_rounds_give_the_same_bits(kind):
    """A launch large enough for the staged kernels to use more CTAs than are resident (several
    rounds of CTAs, each striding over the chunks) must produce exactly what one round produces:
    every chunk updated once, none twice.  Two tensors, the second one odd-sized."""
    from flashoptim_b200.ops.step import set_staged_rounds

    sm = torch.cuda.get_device_properties(0).multi_processor_count
    chunk = native.load().fo_chunk_elems()
    sizes = [sm * 3 * 16 * 3 * chunk + 12345, 100003]   # > 2 rounds' worth of chunks at 16 per CTA
    dtype, err = torch.bfloat16, 1
    outs = []
    for rounds in (1, 8):
        old = set_staged_rounds(rounds)
        try:
            ps = [_rand(n, dtype, 0.02, 7 + i) for i, n in enumerate(sizes)]
            gs = [_rand(n, dtype, 1e-3, 17 + i) for i, n in enumerate(sizes)]
            es = [torch.zeros(n, dtype=torch.int8, device="cuda") for n in sizes]
            ms = [torch.zeros(n, dtype=torch.int8, device="cuda") for n in sizes]
            mss = [torch.zeros(oracle.num_groups(n), dtype=torch.float16, device="cuda") for n in sizes]
            vs = [torch.zeros(n, dtype=torch.uint8, device="cuda") for n in sizes]
            vss = [torch.zeros(oracle.num_groups(n), dtype=torch.float16, device="cuda") for n in sizes]
            table = SegmentTable(torch.device("cuda", torch.cuda.current_device()))
            for step in (1, 2):
                if kind == "adam":
                    rows = make_rows(ps, gs, es, ms, mss, vs, vss)
                    launch_adam(table, rows, dtype, err, True,
                                AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, step=step,
                                          decoupled=True))
                else:
                    rows = make_rows(ps, gs, es, ms, mss, [None] * len(sizes), [None] * len(sizes))
                    launch_momentum(table, rows, dtype, err, native.FO_STATE_Q8,
                                    MomentumHyper(lr=1e-4, mom_coef=0.99, update_coef=0.9, weight_decay=1e-6, lion=True))
            torch.cuda.synchronize()
            outs.append([t.clone() for group in (ps, es, ms, mss, vs, vss) for t in group])
        finally:
            set_staged_rounds(old)
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert not torch.equal(outs[0][0], _rand(sizes[0], dtype, 0.02, 7))   # the step did change the parameters


def test_fused_step_respects_buffer_bounds():
    """Elements outside [0, n) of every stream keep their canary values."""
    n, pad = 1000, 64
    dtype = torch.bfloat16
    big = {k: torch.full((n + 2 * pad,), 7, device="cuda", dtype=dt) for k, dt in
           [("p", dtype), ("g", dtype), ("e", torch.int8), ("m", torch.int8), ("v", torch.uint8)]}
    ms = torch.full((oracle.num_groups(n) + 2 * pad,), 3.0, device="cuda", dtype=torch.float16)
    vs = ms.clone()
    view = {k: t[pad:pad + n] for k, t in big.items()}
    view["p"].copy_(_rand(n, dtype, 0.02))
    view["g"].copy_(_rand(n, dtype, 1e-3, 1))
    view["e"].zero_(); view["m"].zero_(); view["v"].zero_()
    ng = oracle.num_groups(n)
    rows = make_rows([view["p"]], [view["g"]], [view["e"]], [view["m"]], [ms[pad:pad + ng]],
                     [view["v"]], [vs[pad:pad + ng]])
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True)
    launch_adam(SegmentTable(big["p"].device), rows, dtype, 1, True, h)
    torch.cuda.synchronize()
    for k, t in big.items():
        assert (t[:pad].float() == 7).all() and (t[pad + n:].float() == 7).all(), k
    for t in (ms, vs):
        assert (t[:pad] == 3).all() and (t[pad + ng:] == 3).all()
    assert view["m"].abs().sum() > 0 and view["v"].sum() > 0


MOM_CASES = [
    # lion, nesterov, decoupled, mom, damp, mode
    (True, False, True, 0.99, 0.0, native.FO_STATE_Q8),
    (True, False, True, 0.99, 0.0, native.FO_STATE_FULL),
    (False, False, False, 0.9, 0.0, native.FO_STATE_Q8),
    (False, True, False, 0.9, 0.0, native.FO_STATE_Q8),
    (False, False, True, 0.9, 0.1, native.FO_STATE_Q8),
    (False, False, True, 0.9, 0.0, native.FO_STATE_FULL),
    (False, False, False, 0.0, 0.0, native.FO_STATE_NONE),
    (False, False, True, 0.0, 0.0, native.FO_STATE_NONE),
]


@pytest.mark.parametrize("n", [5, 33, 4097, 2048 * 8 + 9])
@pytest.mark.parametrize("dtype,err", [(torch.bfloat16, 1), (torch.bfloat16, 2), (torch.float16, 1),
                                       (torch.bfloat16, 0), (torch.float32, 0)])
@pytest.mark.parametrize("lion,nesterov,decoupled,mom,damp,mode", MOM_CASES)
def test_fused_momentum_single_tensor(n, dtype, err, lion, nesterov, decoupled, mom, damp, mode):
    quantized = mode == native.FO_STATE_Q8
    states = 0 if mode == native.FO_STATE_NONE else 1
    p, g, ecc, st = _make_problem(n, dtype, err, quantized, states, seed=n + 17)
    h = MomentumHyper(lr=1e-3, mom_coef=mom, update_coef=0.9 if lion else 1.0 - damp,
                      weight_decay=1e-5 if (decoupled or lion) else 1e-2, lion=lion, nesterov=nesterov,
                      decoupled=decoupled)
    pc, gc = p.cpu(), g.cpu()
    ec = None if ecc is None else ecc.cpu()
    m_old = None
    if states:
        m_old = (oracle.dequantize_ref(st[0][0].cpu(), st[0][1].cpu()) if quantized
                 else st[0][0].cpu().float())
    p_new, m_new = oracle.momentum_math(
        oracle.read_param_fp32(pc, ec), gc.float(), m_old, lr=h.lr, mom_coef=h.mom_coef,
        update_coef=h.update_coef, weight_decay=h.weight_decay, decoupled=h.decoupled,
        nesterov=h.nesterov, lion=h.lion,
    )
    p_old = _old_master(p, ecc)
    rows = make_rows([p], [g], [ecc], [st[0][0] if states else None],
                     [st[0][1] if states else None], [None], [None])
    launch_momentum(SegmentTable(p.device), rows, dtype, err, mode, h)
    torch.cuda.synchronize()
    specs = [dict(signed=True, sqrt=False, softsign=True)]
    mask = None
    if lion:
        # sign() of an argument within rounding noise of zero may legitimately flip:
        # compare parameters only where the interpolated momentum is clearly non-zero
        c = m_old * h.update_coef + gc.float() * (1 - h.update_coef)
        mask = c.abs() > 1e-9
    _check_step_outputs(p, ecc, st, quantized, dtype, p_new, [m_new] if states else [], specs,
                        f"mom n={n}", p_old, param_mask=mask)
