"""Flagship benchmark: Llama-3-8B-architecture training step under FSDP2.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 10 --warmup 3
    python bench.py --impl reference ...     # the unmodified reference optimizer, same model

Config (the headline one): d=4096, 32 layers, 32 heads / 8 KV heads, SwiGLU
14336, vocab 128256, RoPE theta 5e5, RMSNorm eps 1e-5, random init N(0, 0.02),
bf16 parameters, sequence 4096, micro-batch 1 per GPU, FSDP2 full shard,
FlashAdamW with 24-bit master weights, synthetic uniform token ids.  Forward
and backward are stock PyTorch in both arms; the arms differ in the optimizer
library (this one vs the reference installed under ``baseline/_ref``).

Rank 0 prints ONE JSON line.  ``value`` is whole-job tokens/s from a
device-timed loop (CUDA events, barrier + synchronize on both sides, max over
ranks) whose inputs are already on the device.  ``e2e.value`` is the same
metric for a loop that, every step, copies that step's tokens from pinned host
memory and reads the loss back to the host.  Model state (16 GB of bf16
weights alone) dwarfs the 126 MB L2, so no flush is needed between steps.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama3-70b", "llama-1b", "tiny"])
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--master-weight-bits", default="24")
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "lion"])
    ap.add_argument("--compress-state-dict", action="store_true")
    ap.add_argument("--dcp-dir", default=None,
                    help="after the timed loops, time a torch.distributed.checkpoint save + load of the "
                         "sharded optimizer state into this directory")
    ap.add_argument("--gradient-release", action="store_true")
    ap.add_argument("--activation-checkpointing", action="store_true")
    ap.add_argument("--fused-comm", default="auto", choices=["auto", "off"],
                    help="ours only: fuse the FSDP2 collectives with the update where supported")
    ap.add_argument("--comm-ctas", type=int, default=0, help="grid cap of the fused reduce-scatter kernel")
    ap.add_argument("--own-all-gather", action="store_true",
                    help="fused path: FSDP2's parameter all-gather through this library's pull kernel")
    ap.add_argument("--push-params", default="auto", choices=["auto", "on", "off"],
                    help="fused path: the update kernel also stores the new parameters into every rank's "
                         "all-gather buffer, so FSDP2's parameter all-gathers move no data; auto = on at "
                         "2 GPUs (the size it has been measured at), off otherwise")
    ap.add_argument("--push-budget-gb", type=float, default=0.0,
                    help="with the parameter push: GiB of persistent all-gather buffers per GPU (0: every group)")
    ap.add_argument("--multicast", default="auto", choices=["auto", "on", "off"],
                    help="fused path: NVSwitch multimem.ld_reduce (on) or peer loads summed in fp32 (off); "
                         "auto = peer loads at 2 GPUs, multimem above (the configurations this "
                         "benchmark has been measured in)")
    ap.add_argument("--no-multicast", action="store_true", help="same as --multicast off")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) every 200 ms."""

    def __init__(self, index: int):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.2)

    def start(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def load_module_from(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    args = parse_args()
    if args.impl == "reference":
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "flashoptim")):
            print(json.dumps({"impl": "reference",
                              "unavailable": "baseline/_ref/flashoptim is not installed (pip --target install was not run)"}))
            return
        sys.path.insert(0, ref_dir)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    # the model definition is stock PyTorch and shared by both arms; it is loaded by
    # path so that the reference arm never imports this library's package
    llama = load_module_from(os.path.join(ROOT, "flashoptim_b200", "models", "llama.py"), "_bench_llama")
    if args.impl == "reference":
        import flashoptim as lib
    else:
        import flashoptim_b200 as lib

    cfgs = {
        "llama3-8b": lambda: llama.LlamaConfig.llama3_8b(),
        "llama3-70b": lambda: llama.LlamaConfig.llama3_70b(),
        "llama-1b": lambda: llama.LlamaConfig(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim=8192),
        "tiny": lambda: llama.LlamaConfig.tiny(max_seq_len=args.seq_len),
    }
    cfg = cfgs[args.model]()
    cfg.max_seq_len = args.seq_len
    cfg.activation_checkpointing = args.activation_checkpointing or args.model == "llama3-70b"

    from torch.distributed.fsdp import fully_shard

    torch.manual_seed(1234 + rank)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)  # construct in bf16: no fp32 transient
    if args.model == "llama3-70b":
        # Too large to exist unsharded on one GPU: build on the meta device, shard, then
        # materialise and initialise only the local shards.  Parameters are already bf16,
        # so cast_model is not called here (on storage-less meta tensors the reference's
        # cast_model keys every tensor by address 0 and would merge them).
        with torch.device("meta"):
            model = llama.Llama(cfg)
        torch.set_default_dtype(prev)
        n_params = sum(p.numel() for p in model.parameters())
        for layer in model.layers:
            fully_shard(layer)
        fully_shard(model)
        model.to_empty(device=dev)
        with torch.no_grad():
            for p in model.parameters():
                local = p._local_tensor if hasattr(p, "_local_tensor") else p
                if p.dim() >= 2:
                    local.normal_(0.0, 0.02)
                else:
                    local.fill_(1.0)
    else:
        with torch.device(dev):
            model = llama.Llama(cfg)
        torch.set_default_dtype(prev)
        model.init_weights(0.02, seed=0)
        lib.cast_model(model, dtype=torch.bfloat16)
        n_params = sum(p.numel() for p in model.parameters())
        for layer in model.layers:
            fully_shard(layer)
        fully_shard(model)

    mwb = None if args.master_weight_bits.lower() == "none" else int(args.master_weight_bits)
    import warnings

    warnings.simplefilter("ignore")
    if args.optimizer == "lion":
        opt = lib.FlashLion(model.parameters(), lr=1e-5, betas=(0.9, 0.99), weight_decay=0.01,
                            master_weight_bits=mwb, compress_state_dict=args.compress_state_dict)
    else:
        opt = lib.FlashAdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01,
                             master_weight_bits=mwb, compress_state_dict=args.compress_state_dict)
    fused_comm = False
    fused_state = None
    use_multicast = (world > 2) if args.multicast == "auto" else args.multicast == "on"
    if args.no_multicast:
        use_multicast = False
    push_params = (world == 2) if args.push_params == "auto" else args.push_params == "on"
    if args.own_all_gather:
        push_params = False
    if args.impl == "ours" and args.fused_comm == "auto":
        try:
            from flashoptim_b200.parallel import fsdp as fo_fsdp

            fused_state = fo_fsdp.enable_fused_fsdp(model, opt, timeout_s=20.0, max_ctas=args.comm_ctas,
                                                    use_multicast=use_multicast, own_all_gather=args.own_all_gather,
                                                    push_params=push_params,
                                                    push_budget_bytes=int(args.push_budget_gb * 2**30) or None)
            fused_comm = fused_state is not None
        except Exception as e:  # the plain path is always available
            if rank == 0:
                print(f"[bench] fused FSDP path not enabled: {e}", file=sys.stderr)
    if args.gradient_release:
        lib.enable_gradient_release(model, opt)

    b, s = args.micro_batch, args.seq_len
    total_steps = args.warmup + 2 * args.steps + 2
    g = torch.Generator().manual_seed(1234 + rank)
    host_tokens = torch.randint(0, cfg.vocab_size, (total_steps, b, s + 1), generator=g).pin_memory()
    dev_tokens = host_tokens.to(dev)

    def train_step(tok):
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def launches() -> int:
        if args.impl != "ours":
            return 0
        from flashoptim_b200.ops import step as fo_step

        return fo_step.launch_count()

    i = 0
    fused_error = None
    for w in range(args.warmup):
        train_step(dev_tokens[i])
        i += 1
        if w == 0 and fused_state is not None:
            # After the first step every rank reports whether one of its device-side waits ran
            # out.  If any did, all ranks hand the model back to NCCL collectives together and
            # the measurement goes on without the fused path (the JSON line says so).
            try:
                fused_state.check()
            except Exception as e:
                fused_error = f"{type(e).__name__}: {e}"
            bad = torch.tensor([0 if fused_error is None else 1], device=dev, dtype=torch.int32)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if int(bad.item()):
                fused_error = fused_error or "a device-side wait ran out on another rank"
                fused_state.remove()
                fused_state, fused_comm, push_params = None, False, False
                if rank == 0:
                    print(f"[bench] fused FSDP path switched off after the first step: {fused_error}",
                          file=sys.stderr)
    torch.cuda.synchronize()
    if fused_state is not None:
        fused_state.check()  # raises if a device-side wait for another rank ran out
    torch.cuda.reset_peak_memory_stats()
    sampler = ClockSampler(local_rank)

    # ---- device-timed loop (inputs resident on the device)
    dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    l0 = launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        train_step(dev_tokens[i])
        i += 1
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    dev_ms = e0.elapsed_time(e1) / args.steps
    n_launch = launches() - l0

    # ---- end-to-end loop: pinned-host inputs in, loss out, every step
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    last_loss = 0.0
    for _ in range(args.steps):
        tok = host_tokens[i].to(dev, non_blocking=True)
        last_loss = float(train_step(tok).item())
        i += 1
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    sampler.stop()
    if fused_state is not None:
        fused_state.check()
    dist.barrier()

    dcp_times = None
    if args.dcp_dir:
        import shutil

        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import get_optimizer_state_dict, set_optimizer_state_dict

        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        osd = get_optimizer_state_dict(model, opt)
        dcp.save({"optimizer": osd}, checkpoint_id=args.dcp_dir)
        torch.cuda.synchronize()
        dist.barrier()
        t1 = time.perf_counter()
        template = get_optimizer_state_dict(model, opt)
        dcp.load({"optimizer": template}, checkpoint_id=args.dcp_dir)
        set_optimizer_state_dict(model, opt, template)
        torch.cuda.synchronize()
        dist.barrier()
        t2 = time.perf_counter()
        size = 0
        if rank == 0:
            for root, _, files in os.walk(args.dcp_dir):
                size += sum(os.path.getsize(os.path.join(root, f)) for f in files)
            shutil.rmtree(args.dcp_dir, ignore_errors=True)
        dcp_times = {"save_s": round(t1 - t0, 3), "load_s": round(t2 - t1, 3), "bytes_on_disk": size,
                     "compressed": bool(args.compress_state_dict)}

    t = torch.tensor([dev_ms, e2e_ms, torch.cuda.max_memory_allocated() / 2**30], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, peak_gib = (float(x) for x in t.tolist())
    tokens_per_step = world * b * s
    if rank == 0:
        rec = {
            "metric": "tokens_per_s",
            "value": round(tokens_per_step / (dev_ms * 1e-3), 1),
            "unit": "tokens/s",
            "impl": args.impl,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(dev_ms, 3),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights N(0,0.02)",
            "config": {
                "model": args.model, "n_params": n_params, "global_batch": world * b, "seq_len": s,
                "parallelism": f"fsdp2x{world}",
                "optimizer": f"{'FlashLion' if args.optimizer == 'lion' else 'FlashAdamW'} mwb={mwb}",
                "gradient_release": bool(args.gradient_release), "fused_comm": bool(fused_comm),
                "fused_comm_multicast": bool(fused_comm and use_multicast),
                "fused_param_push": bool(fused_comm and push_params),
                **({"fused_comm_error": fused_error} if fused_error else {}),
                "activation_checkpointing": bool(cfg.activation_checkpointing),
                "l2": "working set (>= 16 GB of weights) far exceeds the 126 MB L2; no flush",
            },
            "e2e": {
                "value": round(tokens_per_step / (e2e_ms * 1e-3), 1),
                "unit": "tokens/s",
                "ms_per_step": round(e2e_ms, 3),
                "h2d_bytes_per_step": b * (s + 1) * 8,
                "d2h_bytes_per_step": 4,
                "last_loss": last_loss,
            },
            "gpu_launches": n_launch,
            "peak_gib_per_gpu": round(peak_gib, 2),
            "clocks": sampler.summary(),
        }
        if dcp_times is not None:
            rec["dcp"] = dcp_times
        print(json.dumps(rec), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
