"""Spawn helpers for multi-process tests: ``gloo`` on CPU, ``nccl`` on GPUs,
rendezvous on 127.0.0.1 through a file store.  Workers collect errors instead
of raising mid-loop and all-reduce the verdict, so ranks leave together."""

from __future__ import annotations

import os
import tempfile
import time
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, backend, store_path, fn, args, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ.setdefault("MASTER_PORT", "29577")
    os.environ["FLASHOPTIM_ALLOW_INEFFECTIVE_MASTER_WEIGHT_BITS"] = "1"
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    err = ""
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, init_method=f"file://{store_path}", rank=rank, world_size=world)
        try:
            errors = fn(rank, world, *args) or []
            err = "\n".join(errors)
        except Exception:
            err = traceback.format_exc()
        flag = torch.tensor([1 if err else 0], device="cuda" if backend == "nccl" else "cpu")
        try:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        except Exception:
            pass
    except Exception:
        err = traceback.format_exc()
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
    with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
        f.write(err)


def run_distributed(fn, world_size=2, backend="gloo", args=()):
    """Run ``fn(rank, world, *args) -> list[str]`` on ``world_size`` processes; raise on any error.

    A failed run is never repeated: the workers use fixed seeds and fixed summation orders, so
    a failure that comes and goes is a race to be found, not noise.  Every rank's message is in
    the raised AssertionError and, when the environment variable
    ``FLASHOPTIM_B200_TEST_FAILURE_DIR`` names a directory, also in a text file there (one per
    failed call), so that it survives a log that was cut short."""
    try:
        _run_once(fn, world_size, backend, args)
    except AssertionError as e:
        out = os.environ.get("FLASHOPTIM_B200_TEST_FAILURE_DIR")
        if out:
            os.makedirs(out, exist_ok=True)
            name = f"{getattr(fn, '__name__', 'worker')}_{backend}_w{world_size}_{os.getpid()}_{int(time.time())}.txt"
            with open(os.path.join(out, name), "w") as f:
                f.write(f"args={args!r}\n{e}\n")
        raise


def _run_once(fn, world_size, backend, args):
    with tempfile.TemporaryDirectory() as d:
        store = os.path.join(d, "store")
        mp.spawn(_entry, args=(world_size, backend, store, fn, args, d), nprocs=world_size, join=True)
        msgs = []
        for r in range(world_size):
            path = os.path.join(d, f"rank{r}.txt")
            txt = open(path).read() if os.path.exists(path) else "rank produced no result"
            if txt:
                msgs.append(f"[rank {r}]\n{txt}")
        if msgs:
            raise AssertionError("\n".join(msgs))
