"""FSDP2 ``fully_shard`` (modelled on the reference's ``test/test_fsdp2.py``): sharded
training against a single-process run, gradient release, fp32 export, and
``torch.distributed.checkpoint`` round trips.  CPU ranks over gloo; the same body on two
GPUs over NCCL."""

import os
import tempfile
import warnings

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from flashoptim_b200 import FlashAdamW, FlashLion, cast_model, enable_gradient_release

from dist_utils import run_distributed
from helpers import check_similar, get_tolerances

CONFIGS = [(torch.float32, None, False), (torch.bfloat16, 24, True), (torch.bfloat16, 32, True)]


def _net(dtype, device):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(10, 16), nn.ReLU(), nn.Linear(16, 6)).to(device)
    if dtype != torch.float32:
        cast_model(m, dtype)
    return m


def _full(t):
    return t.full_tensor() if hasattr(t, "full_tensor") else t


def _train_worker(rank, world, use_cuda):
    from torch.distributed.fsdp import fully_shard

    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    errors = []
    g = torch.Generator().manual_seed(7)
    data = [(torch.randn(world * 8, 10, generator=g), torch.randint(0, 6, (world * 8,), generator=g))
            for _ in range(5)]
    for cls, kw in ((FlashAdamW, dict(lr=5e-4, weight_decay=1e-2)), (FlashLion, dict(lr=5e-4))):
        for release in (False, True):
            for reshard in (True, False):
                for dtype, mwb, quantize in CONFIGS:
                    tag = f"{cls.__name__} release={release} reshard={reshard} {dtype} mwb={mwb}"
                    with warnings.catch_warnings():
                        warnings.simplefilter("ignore")
                        single = _net(dtype, device)
                        sharded = _net(dtype, device)
                        for layer in sharded:
                            if isinstance(layer, nn.Linear):
                                fully_shard(layer, reshard_after_forward=reshard)
                        fully_shard(sharded, reshard_after_forward=reshard)
                        o1 = cls(single.parameters(), master_weight_bits=mwb, quantize=quantize, **kw)
                        o2 = cls(sharded.parameters(), master_weight_bits=mwb, quantize=quantize, **kw)
                    handle = enable_gradient_release(sharded, o2) if release else None
                    tol = get_tolerances(dtype, quantize)
                    for step, (x, y) in enumerate(data):
                        x, y = x.to(device=device, dtype=dtype), y.to(device)
                        xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
                        nn.functional.cross_entropy(single(x).float(), y).backward()
                        o1.step(); o1.zero_grad()
                        nn.functional.cross_entropy(sharded(xs).float(), ys).backward()
                        if not release:
                            o2.step(); o2.zero_grad()
                        elif any(p.grad is not None for p in sharded.parameters()):
                            errors.append(f"{tag}: gradients survived backward under gradient release")
                        for (n1, p1), (n2, p2) in zip(single.named_parameters(), sharded.named_parameters()):
                            errors += check_similar(_full(p2.detach()), p1.detach(), tol, f"{tag} step {step} {n1}")
                    for p in sharded.parameters():
                        st = o2.state[p]
                        local = p.to_local()
                        if st["exp_avg"].shape != tuple(local.shape):
                            errors.append(f"{tag}: state is not shard-shaped")
                    if handle is not None:
                        handle.remove()
                    # fp32 export holds the local shard of corrected parameters
                    sd = o2.get_fp32_model_state_dict(sharded)
                    for n, p in sharded.named_parameters():
                        if "error_bits" in o2.state[p] and sd[n].shape != p.to_local().shape:
                            errors.append(f"{tag}: fp32 export of {n} has shape {tuple(sd[n].shape)}")
    return errors


def _dcp_worker(rank, world, use_cuda, ckpt_root):
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict, set_optimizer_state_dict
    from torch.distributed.fsdp import fully_shard

    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    errors = []
    x = torch.randn(8, 10, generator=torch.Generator().manual_seed(rank)).to(device)
    y = torch.randint(0, 6, (8,), generator=torch.Generator().manual_seed(rank + 10)).to(device)
    for compress, mwb in ((False, 24), (True, 24), (False, 32), (True, 32), (True, None)):
        tag = f"dcp compress={compress} mwb={mwb}"
        dtype = torch.bfloat16
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            model = _net(dtype, device)
            fully_shard(model)
            opt = FlashAdamW(model.parameters(), lr=1e-3, master_weight_bits=mwb, compress_state_dict=compress)
        for _ in range(2):
            nn.functional.cross_entropy(model(x.to(dtype)).float(), y).backward()
            opt.step(); opt.zero_grad()
        ckpt = os.path.join(ckpt_root, f"c{int(compress)}_{mwb}")
        osd = get_optimizer_state_dict(model, opt)
        dcp.save({"optimizer": osd}, checkpoint_id=ckpt)
        saved = {k: {kk: (_v.to_local().clone() if hasattr(_v, "to_local") else _v.clone())
                     for kk, _v in v.items()} for k, v in osd["state"].items()}
        # a fresh optimizer with different contents
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            model2 = _net(dtype, device)
            fully_shard(model2)
            opt2 = FlashAdamW(model2.parameters(), lr=1e-3, master_weight_bits=mwb, compress_state_dict=compress)
        nn.functional.cross_entropy(model2(x.to(dtype)).float() * 3, y).backward()
        opt2.step(); opt2.zero_grad()
        template = get_optimizer_state_dict(model2, opt2)
        dcp.load({"optimizer": template}, checkpoint_id=ckpt)
        set_optimizer_state_dict(model2, opt2, template)
        loaded = get_optimizer_state_dict(model2, opt2)
        for k, v in saved.items():
            for kk, want in v.items():
                got = loaded["state"][k][kk]
                got = got.to_local() if hasattr(got, "to_local") else got
                if kk == "step" or compress or kk == "error_bits":
                    if kk == "error_bits" and mwb == 32:
                        # int16 codes travel bit-cast to bf16; some patterns are NaNs, compare the bits
                        got, want = got.contiguous().view(torch.int16), want.contiguous().view(torch.int16)
                    if not torch.equal(got.cpu(), want.cpu()):
                        errors.append(f"{tag}: {k}.{kk} changed across dcp round trip")
                elif not torch.allclose(got.float().cpu(), want.float().cpu(), rtol=5e-2,
                                        atol=float(want.float().abs().max()) * 2e-2):
                    errors.append(f"{tag}: {k}.{kk} drifted across dcp round trip")
        nn.functional.cross_entropy(model2(x.to(dtype)).float(), y).backward()
        opt2.step()
        if not all(torch.isfinite(_full(p.detach()).float()).all() for p in model2.parameters()):
            errors.append(f"{tag}: non-finite weights after resuming")
        dist.barrier()
    # uneven shards are refused when checkpoint tensors are built
    odd = nn.Linear(10, 7).to(device)
    cast_model(odd)
    fully_shard(odd)
    oo = FlashAdamW(odd.parameters(), lr=1e-3)
    odd(x.to(torch.bfloat16)).float().sum().backward()
    oo.step()
    try:
        oo.state_dict()
        errors.append("uneven shards were not rejected")
    except ValueError:
        pass
    return errors


def _accum_worker(rank, world, use_cuda):
    """Gradient accumulation with ``set_requires_gradient_sync``: two micro-batches per step,
    only the second one reduce-scatters; compared every step with a single process that sees
    both micro-batches of every rank (the reference's "grad_accum" setting,
    test/test_fsdp2.py:95-115, 444-455)."""
    from torch.distributed.fsdp import fully_shard

    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    errors = []
    g = torch.Generator().manual_seed(11)
    data = [(torch.randn(world * 8, 10, generator=g), torch.randint(0, 6, (world * 8,), generator=g))
            for _ in range(8)]
    for cls, kw in ((FlashAdamW, dict(lr=5e-4, weight_decay=1e-2)), (FlashLion, dict(lr=5e-4))):
        for dtype, mwb, quantize in CONFIGS:
            tag = f"accumulation {cls.__name__} {dtype} mwb={mwb}"
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                single, sharded = _net(dtype, device), _net(dtype, device)
                for layer in sharded:
                    if isinstance(layer, nn.Linear):
                        fully_shard(layer)
                fully_shard(sharded)
                o1 = cls(single.parameters(), master_weight_bits=mwb, quantize=quantize, **kw)
                o2 = cls(sharded.parameters(), master_weight_bits=mwb, quantize=quantize, **kw)
            tol = get_tolerances(dtype, quantize)
            for step in range(4):
                for micro in range(2):
                    x, y = data[2 * step + micro]
                    x, y = x.to(device=device, dtype=dtype), y.to(device)
                    xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
                    (nn.functional.cross_entropy(single(x).float(), y) / 2).backward()
                    sharded.set_requires_gradient_sync(micro == 1)
                    (nn.functional.cross_entropy(sharded(xs).float(), ys) / 2).backward()
                o1.step(); o1.zero_grad()
                o2.step(); o2.zero_grad()
                for (n1, p1), (_, p2) in zip(single.named_parameters(), sharded.named_parameters()):
                    errors += check_similar(_full(p2.detach()), p1.detach(), tol, f"{tag} step {step} {n1}")
    return errors


def _fp32_roundtrip_worker(rank, world, use_cuda):
    """``get_fp32_model_state_dict`` -> ``set_fp32_model_state_dict`` under sharding restores
    weights and correction codes exactly, also after the model was disturbed in between, and a
    second export equals the first (the reference's test/test_fsdp2.py:646-705)."""
    from torch.distributed.fsdp import fully_shard

    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    errors = []
    g = torch.Generator().manual_seed(5)
    x = torch.randn(world * 8, 10, generator=g)
    y = torch.randint(0, 6, (world * 8,), generator=g)
    for mwb in (24, 32):
        tag = f"fp32 round trip mwb={mwb}"
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            model = _net(torch.bfloat16, device)
            for layer in model:
                if isinstance(layer, nn.Linear):
                    fully_shard(layer)
            fully_shard(model)
            opt = FlashAdamW(model.parameters(), lr=1e-3, master_weight_bits=mwb)
        xs = x[rank * 8:(rank + 1) * 8].to(device=device, dtype=torch.bfloat16)
        ys = y[rank * 8:(rank + 1) * 8].to(device)
        for _ in range(3):
            nn.functional.cross_entropy(model(xs).float(), ys).backward()
            opt.step(); opt.zero_grad()
        first = {k: v.clone() for k, v in opt.get_fp32_model_state_dict(model).items()}
        weights = {n: p.to_local().detach().clone() for n, p in model.named_parameters()}
        codes = {n: opt.state[p]["error_bits"].clone() for n, p in model.named_parameters()}
        for n, p in model.named_parameters():
            if first[n].dtype != torch.float32 or first[n].shape != p.to_local().shape:
                errors.append(f"{tag}: export of {n} is {first[n].dtype} {tuple(first[n].shape)}")
        with torch.no_grad():  # disturb weights and codes, then import the export
            for p in model.parameters():
                p.to_local().mul_(1.5)
                opt.state[p]["error_bits"].zero_()
        opt.set_fp32_model_state_dict(model, first)
        for n, p in model.named_parameters():
            if not torch.equal(p.to_local().detach(), weights[n]):
                errors.append(f"{tag}: weights of {n} differ after the import")
            if not torch.equal(opt.state[p]["error_bits"], codes[n]):
                errors.append(f"{tag}: correction codes of {n} differ after the import")
        second = opt.get_fp32_model_state_dict(model)
        for k, v in first.items():
            if not torch.equal(second[k], v):
                errors.append(f"{tag}: second export of {k} differs from the first")
        nn.functional.cross_entropy(model(xs).float(), ys).backward()
        opt.step(); opt.zero_grad()
        if not all(torch.isfinite(_full(p.detach()).float()).all() for p in model.parameters()):
            errors.append(f"{tag}: non-finite weights after continuing")
    return errors


def test_fsdp2_gloo_two_ranks():
    run_distributed(_train_worker, world_size=2, backend="gloo", args=(False,))


def test_fsdp2_gradient_accumulation_gloo():
    run_distributed(_accum_worker, world_size=2, backend="gloo", args=(False,))


def test_fsdp2_fp32_state_dict_round_trip_gloo():
    run_distributed(_fp32_roundtrip_worker, world_size=2, backend="gloo", args=(False,))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fsdp2_accumulation_and_fp32_round_trip_nccl_two_gpus():
    run_distributed(_accum_worker, world_size=2, backend="nccl", args=(True,))
    run_distributed(_fp32_roundtrip_worker, world_size=2, backend="nccl", args=(True,))


def test_fsdp2_dcp_gloo_two_ranks():
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_dcp_worker, world_size=2, backend="gloo", args=(False, d))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fsdp2_nccl_two_gpus():
    run_distributed(_train_worker, world_size=2, backend="nccl", args=(True,))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fsdp2_dcp_nccl_two_gpus():
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_dcp_worker, world_size=2, backend="nccl", args=(True, d))


def _hsdp_worker(rank, world):
    """Two-dimensional (replicate x shard) meshes: state is shard-shaped, training matches a
    single process, state_dict wraps over both mesh dimensions, and the fused path refuses."""
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    from flashoptim_b200.parallel import enable_fused_fsdp

    errors = []
    device = torch.device("cpu")
    g = torch.Generator().manual_seed(7)
    data = [(torch.randn(world * 8, 10, generator=g), torch.randint(0, 6, (world * 8,), generator=g))
            for _ in range(4)]
    for shape in ((1, world), (world, 1)):
        mesh = init_device_mesh("cpu", shape, mesh_dim_names=("replicate", "shard"))
        for dtype, mwb, quantize in CONFIGS[:2]:
            tag = f"hsdp {shape} {dtype} mwb={mwb}"
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                single, sharded = _net(dtype, device), _net(dtype, device)
                for layer in sharded:
                    if isinstance(layer, nn.Linear):
                        fully_shard(layer, mesh=mesh)
                fully_shard(sharded, mesh=mesh)
                o1 = FlashAdamW(single.parameters(), lr=5e-4, master_weight_bits=mwb, quantize=quantize)
                o2 = FlashAdamW(sharded.parameters(), lr=5e-4, master_weight_bits=mwb, quantize=quantize)
            tol = get_tolerances(dtype, quantize)
            for step, (x, y) in enumerate(data):
                x = x.to(dtype)
                xs, ys = x[rank * 8:(rank + 1) * 8], y[rank * 8:(rank + 1) * 8]
                nn.functional.cross_entropy(single(x).float(), y).backward()
                o1.step(); o1.zero_grad()
                nn.functional.cross_entropy(sharded(xs).float(), ys).backward()
                o2.step(); o2.zero_grad()
                for (n1, p1), (_, p2) in zip(single.named_parameters(), sharded.named_parameters()):
                    errors += check_similar(_full(p2.detach()), p1.detach(), tol, f"{tag} step {step} {n1}")
            for p in sharded.parameters():
                if o2.state[p]["exp_avg"].shape != tuple(p.to_local().shape):
                    errors.append(f"{tag}: state is not shard-shaped")
            sd = o2.state_dict()
            for st in sd["state"].values():
                for k, v in st.items():
                    if k != "step" and v.dim() >= 1 and not hasattr(v, "device_mesh"):
                        errors.append(f"{tag}: checkpoint entry {k} is not a DTensor")
                    elif k != "step" and v.dim() >= 1 and v.device_mesh.ndim != 2:
                        errors.append(f"{tag}: checkpoint entry {k} lost a mesh dimension")
            o3 = FlashAdamW(sharded.parameters(), lr=5e-4, master_weight_bits=mwb, quantize=quantize)
            o3.load_state_dict(sd)
            try:
                enable_fused_fsdp(sharded, o2)
                errors.append(f"{tag}: the fused path accepted an HSDP mesh")
            except ValueError:
                pass
    return errors


def test_hsdp_mesh_gloo_two_ranks():
    run_distributed(_hsdp_worker, world_size=2, backend="gloo")
