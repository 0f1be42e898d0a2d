"""Kernels that average gradients from several ranks' buffers while updating, on ONE
GPU: the ranks' buffers are plain tensors of this process and the flags that other
ranks would publish are written by the host beforehand (kernels of different ranks
never have to run concurrently here).  Also: a wait that nothing satisfies must run
out, report through the status word and leave the context usable."""

import ctypes

import pytest
import torch

from flashoptim_b200.ops import native, oracle
from flashoptim_b200.ops.quant import compute_ecc_bits, quantize
from flashoptim_b200.ops.step import (
    AdamHyper, MomentumHyper, SegmentTable, launch_adam_peer, launch_momentum_peer, make_rows,
)
from flashoptim_b200.parallel.symm import CommTimeoutError, PeerGroup, SymmBuffer

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _state(n, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    p32 = torch.randn(n, device=DEV, generator=g) * 0.02
    p = p32.to(torch.bfloat16)
    ecc = compute_ecc_bits(p32, p, master_bytewidth=3)
    m, ms = quantize(torch.randn(n, device=DEV, generator=g) * 1e-3)
    v, vs = quantize((torch.randn(n, device=DEV, generator=g) * 1e-3).square(), signed=False, sqrt=True,
                     softsign=False)
    return [p, ecc, m, ms, v, vs]


def _emulated(world, nbytes, timeout_s=2.0):
    """One PeerGroup object per emulated rank, sharing `world` buffers and pads."""
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    pads = [torch.zeros(64 * 8, dtype=torch.int32, device=DEV) for _ in range(world)]
    groups = []
    for r in range(world):
        g = PeerGroup(group=None, timeout_s=timeout_s)
        g.world, g.rank = world, r
        groups.append(g)
    return groups, bufs, pads


def _publish_all(pads, channel, epoch):
    for pad in pads:
        pad[channel * 8: channel * 8 + 8] = epoch


@pytest.mark.parametrize("variant", [0, 1], ids=["register", "staged"])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("layout", ["ddp", "fsdp"])
def test_peer_adam_matches_local_step_on_mean_gradient(world, layout, variant):
    # full 2048-element blocks (the staged kernels' bulk copies), tails, a tensor smaller than
    # a unit group, and enough blocks that a CTA's ring wraps around when the grid is capped
    sizes = [4096, 33, 50257, 2048 * 3 + 5, 2048 * 40]
    row = sum((n + 7) // 8 * 8 for n in sizes) * 2  # bytes of one rank's (padded) row
    nbytes = row * (world if layout == "fsdp" else 1)
    groups, bufs, pads = _emulated(world, nbytes)
    gen = torch.Generator(device=DEV).manual_seed(5)
    for b in bufs:
        b.view(torch.bfloat16).copy_(torch.randn(nbytes // 2, device=DEV, generator=gen) * 1e-3)
    ranks = range(world) if layout == "fsdp" else [0, world - 1]
    for r in ranks:
        base = r * row if layout == "fsdp" else 0
        ref = [_state(n, 100 + i) for i, n in enumerate(sizes)]
        new = [_state(n, 100 + i) for i, n in enumerate(sizes)]
        offs, o = [], 0
        for n in sizes:
            offs.append(base + o)
            o += (n + 7) // 8 * 8 * 2
        # reference: mean gradient in fp32 (rank order), rounded to bf16 once, local step kernel
        grads = []
        for n, off in zip(sizes, offs):
            acc = torch.zeros(n, device=DEV)
            for b in bufs:
                acc += b[off:off + 2 * n].view(torch.bfloat16).float()
            grads.append(acc / world)
        h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=1e-5, step=2, decoupled=True)
        want = []
        for st, g32 in zip(ref, grads):
            p, ecc, m, ms, v, vs = st
            mm = oracle.dequantize_ref(m.cpu(), ms.cpu())
            vv = oracle.dequantize_ref(v.cpu(), vs.cpu(), signed=False, sqrt=True, softsign=False)
            want.append(oracle.adam_math(oracle.ecc_decode_ref(p.cpu(), ecc.cpu()), g32.cpu(), mm, vv, lr=h.lr,
                                         beta1=h.beta1, beta2=h.beta2, eps=h.eps, weight_decay=h.weight_decay,
                                         decoupled=True, step=h.step))
        _publish_all(pads, 0, 1)  # every other rank has "arrived"
        g = groups[r]
        g.variant = variant
        g.max_ctas = 3 if variant else 0  # three CTAs: each walks its ring several times around
        out = torch.zeros(row // 2, dtype=torch.bfloat16, device=DEV)
        buf = SymmBuffer(bufs[r], [b.data_ptr() for b in bufs], 0)
        args = g.comm_args(buf, 1, 0, 1, grad_out=out, grad_out_sub=base, pads=[p.data_ptr() for p in pads])
        rows = make_rows([s[0] for s in new], [None] * len(sizes), [s[1] for s in new], [s[2] for s in new],
                         [s[3] for s in new], [s[4] for s in new], [s[5] for s in new])
        rows[:, 1] = offs
        h.grad_scale = 1.0 / world
        # all-gather on write: the new parameters also go to every rank's parameter buffer
        # (same layout as the gradient rows), and channel 2 reports it with its own epoch
        pushed = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
        args.push = 1
        for q in range(world):
            args.param_out[q] = pushed[q].data_ptr()
        args.param_out_delta = 0
        args.push_epoch = 9
        args.pushed_channel = 2
        launch_adam_peer(SegmentTable(torch.device(DEV, torch.cuda.current_device())), rows, torch.bfloat16, 1,
                         True, h, args)
        g.check_status()
        for q in range(world):
            assert int(pads[q][2 * 8 + r]) == 9
            for st, n, off in zip(new, sizes, offs):
                got = pushed[q][off:off + 2 * n].view(torch.bfloat16)
                assert torch.equal(got.view(torch.int16), st[0].view(torch.int16)), (r, q, n)
            # nothing outside this rank's segments was written
            mask = torch.ones(nbytes, dtype=torch.bool, device=DEV)
            for n, off in zip(sizes, offs):
                mask[off:off + 2 * n] = False
            assert int(pushed[q][mask].count_nonzero()) == 0
        for i, (st, (pn, mn, vn), g32) in enumerate(zip(new, want, grads)):
            rec = oracle.ecc_decode_ref(st[0].cpu(), st[1].cpu())
            half_ulp = torch.exp2(oracle.ecc_log_scale(st[0].cpu()).float())
            assert ((rec - pn).abs() <= half_ulp * 0.75 / 127 + 4e-6 * (pn - oracle.ecc_decode_ref(
                ref[i][0].cpu(), ref[i][1].cpu())).abs() + 4e-7 * pn.abs() + 1e-10).all(), (r, i)
            q_ref, _ = oracle.quantize_ref(mn)
            assert (st[2].cpu().to(torch.int16) - q_ref.to(torch.int16)).abs().max() <= 1
            # averaged gradient handed back
            n = sizes[i]
            o = offs[i] - base
            got = out[o // 2: o // 2 + n].float().cpu()
            assert torch.allclose(got, g32.cpu(), rtol=2 ** -7, atol=1e-9)
        # this rank published ready and done to every pad
        for pad in pads:
            assert int(pad[0 * 8 + r]) == 1 and int(pad[1 * 8 + r]) == 1


@pytest.mark.parametrize("variant", [0, 1], ids=["register", "staged"])
def test_peer_momentum_lion_world4(variant):
    n, world = 10000, 4
    groups, bufs, pads = _emulated(world, n * 2)
    groups[1].variant = variant
    gen = torch.Generator(device=DEV).manual_seed(1)
    for b in bufs:
        b.view(torch.bfloat16).copy_(torch.randn(n, device=DEV, generator=gen) * 1e-3)
    p, ecc, m, ms, _, _ = _state(n, 3)
    g32 = sum(b.view(torch.bfloat16).float() for b in bufs) / world
    mm = oracle.dequantize_ref(m.cpu(), ms.cpu())
    p_old = oracle.ecc_decode_ref(p.cpu(), ecc.cpu())
    pn, mn = oracle.momentum_math(p_old, g32.cpu(), mm, lr=1e-4, mom_coef=0.99, update_coef=0.9,
                                  weight_decay=1e-6, decoupled=True, nesterov=False, lion=True)
    _publish_all(pads, 2, 7)
    buf = SymmBuffer(bufs[1], [b.data_ptr() for b in bufs], 0)
    args = groups[1].comm_args(buf, 7, 2, 3, pads=[q.data_ptr() for q in pads])
    rows = make_rows([p], [None], [ecc], [m], [ms], [None], [None])
    rows[:, 1] = 0
    h = MomentumHyper(lr=1e-4, mom_coef=0.99, update_coef=0.9, weight_decay=1e-6, lion=True, grad_scale=1 / world)
    launch_momentum_peer(SegmentTable(torch.device(DEV, torch.cuda.current_device())), rows, torch.bfloat16, 1,
                         native.FO_STATE_Q8, h, args)
    groups[1].check_status()
    rec = oracle.ecc_decode_ref(p.cpu(), ecc.cpu())
    c = mm * 0.9 + g32.cpu() * 0.1
    keep = c.abs() > 1e-9
    assert ((rec - pn).abs()[keep] <= 1e-6).all()
    q_ref, _ = oracle.quantize_ref(mn)
    assert (m.cpu().to(torch.int16) - q_ref.to(torch.int16)).abs().max() <= 1


def test_reduce_and_allgather_kernels():
    world, n = 4, 5003
    lib = native.load()
    groups, bufs, pads = _emulated(world, 4 * 4096)
    gen = torch.Generator(device=DEV).manual_seed(2)
    for b in bufs:
        b.view(torch.float32).copy_(torch.randn(4096, device=DEV, generator=gen))
    _publish_all(pads, 0, 1)
    buf = SymmBuffer(bufs[2], [b.data_ptr() for b in bufs], 0)
    a = groups[2].comm_args(buf, 1, 0, 1, pads=[q.data_ptr() for q in pads])
    out = torch.zeros(1000, device=DEV)
    native.check(lib.fo_reduce_peer(1000, 64, out.data_ptr(), native.FO_FP32, 0.25, ctypes.byref(a),
                                    torch.cuda.current_stream().cuda_stream), "reduce")
    groups[2].check_status()
    want = sum(b.view(torch.float32)[16:1016] for b in bufs) * 0.25
    assert torch.allclose(out, want, rtol=1e-6, atol=1e-7)
    # all-gather: rank 2 pulls slot s from rank s
    slot = 4096
    before = [b.clone() for b in bufs]
    _publish_all(pads, 2, 1)
    a = groups[2].comm_args(buf, 1, 2, 3, pads=[q.data_ptr() for q in pads])
    native.check(lib.fo_allgather_peer(slot, ctypes.byref(a), torch.cuda.current_stream().cuda_stream), "ag")
    groups[2].check_status()
    for s in range(world):
        assert torch.equal(bufs[2][s * slot:(s + 1) * slot], before[s][s * slot:(s + 1) * slot])


@pytest.mark.parametrize("n", [4096 * 4, 10007])
def test_two_shot_reduce_broadcast_kernel(n):
    """Each emulated rank averages its slice and stores it into every rank's second half."""
    world = 4
    lib = native.load()
    half = (n * 2 + 255) // 256 * 256
    groups, bufs, pads = _emulated(world, 2 * half)
    gen = torch.Generator(device=DEV).manual_seed(4)
    for b in bufs:
        b[:n * 2].view(torch.bfloat16).copy_(torch.randn(n, device=DEV, generator=gen) * 1e-3)
    want = sum(b[:n * 2].view(torch.bfloat16).float() for b in bufs) / world
    _publish_all(pads, 0, 1)
    for r in range(world):
        buf = SymmBuffer(bufs[r], [b.data_ptr() for b in bufs], 0)
        a = groups[r].comm_args(buf, 1, 0, 1, pads=[q.data_ptr() for q in pads])
        native.check(lib.fo_reduce_bcast_peer(n, 0, half, native.FO_BF16, 1.0 / world, ctypes.byref(a),
                                              torch.cuda.current_stream().cuda_stream), "reduce_bcast")
        groups[r].check_status()
    for b in bufs:  # every rank now holds the complete averaged vector
        got = b[half:half + n * 2].view(torch.bfloat16).float()
        assert torch.allclose(got, want, rtol=2 ** -7, atol=1e-9)
        assert torch.equal(got, bufs[0][half:half + n * 2].view(torch.bfloat16).float())


@pytest.mark.parametrize("variant", [0, 1], ids=["register", "staged"])
def test_wait_that_nothing_satisfies_times_out_and_leaves_state_untouched(variant):
    world, n = 2, 4096
    groups, bufs, pads = _emulated(world, n * 2, timeout_s=0.05)
    groups[0].variant = variant
    p, ecc, m, ms, v, vs = _state(n, 9)
    snap = [t.clone() for t in (p, ecc, m, ms, v, vs)]
    buf = SymmBuffer(bufs[0], [b.data_ptr() for b in bufs], 0)
    args = groups[0].comm_args(buf, 1, 0, 1, pads=[q.data_ptr() for q in pads])  # rank 1 never arrives
    rows = make_rows([p], [None], [ecc], [m], [ms], [v], [vs])
    rows[:, 1] = 0
    h = AdamHyper(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1, decoupled=True)
    table = SegmentTable(torch.device(DEV, torch.cuda.current_device()))
    launch_adam_peer(table, rows, torch.bfloat16, 1, True, h, args)
    torch.cuda.synchronize()
    assert int(groups[0].status[2]) == 0  # every CTA counted itself out: the counter is back at zero
    with pytest.raises(CommTimeoutError) as ei:
        groups[0].check_status()
    assert "missing rank 1" in str(ei.value)
    for a, b in zip(snap, (p, ecc, m, ms, v, vs)):
        assert torch.equal(a, b)  # nothing was committed
    # the context is alive and the same launch succeeds once the flag is there
    _publish_all(pads, 0, 2)
    args = groups[0].comm_args(buf, 2, 0, 1, pads=[q.data_ptr() for q in pads])
    launch_adam_peer(table, rows, torch.bfloat16, 1, True, h, args)
    groups[0].check_status()
    assert not torch.equal(snap[3], ms)  # zero gradients: the momentum shrank, so its scales moved
    # stand-alone wait kernel: same behaviour
    args = groups[0].comm_args(buf, 99, 0, 1, pads=[q.data_ptr() for q in pads])
    groups[0].wait(args, 0)
    with pytest.raises(CommTimeoutError):
        groups[0].check_status()
