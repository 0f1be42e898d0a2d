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
import sys
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
    ap.add_argument("--comm-ctas", type=int, default=-1,
                    help="grid cap of the fused reduce-scatter kernel (0: fill the GPU; -1: the measured default, "
                         "flashoptim_b200.parallel.tuned_options)")
    ap.add_argument("--sweep", default=None,
                    help="ours, >= 2 GPUs: instead of the benchmark line, time every listed configuration in this "
                         "one process and print them as one JSON line.  Semicolon-separated entries "
                         "MODE[:CTAS[:LOADS]] with MODE nccl (FSDP2's NCCL collectives + this library's step), "
                         "fused (reduce-scatter fused with the update, NCCL all-gather), push (fused + all-gather "
                         "on write), pull / pullce (fused + this library's all-gather by pull kernel / by copy "
                         "engines) or agce (NCCL reduce-scatter, copy-engine all-gather), "
                         "CTAS the grid cap (0: none) and LOADS mc (multimem.ld_reduce), p2p (peer loads into "
                         "registers) or staged (bulk copies of the peers' chunks into shared memory); p2pmc / stagedmc "
                         "push the parameters with multimem.st instead of one store per rank; ce / cestaged move all "
                         "bytes with the copy engines and run the register / staged kernel on local memory; a fourth field "
                         "capall also caps the group that backward reduces last")
    ap.add_argument("--transport", default="auto", choices=["auto", "kernel", "copy_engine"],
                    help="fused path: the update kernel itself reads the peers' gradients over NVLink (kernel) "
                         "or copy engines bring them into local memory first (copy_engine); auto: the measured "
                         "default: kernel")
    ap.add_argument("--push-multicast", default="auto", choices=["auto", "on", "off"],
                    help="parameter push through multimem.st (auto: as the gradient loads; with staged kernels "
                         "above 2 GPUs)")
    ap.add_argument("--comm-kernel", default="auto", choices=["auto", "register", "staged"],
                    help="fused path: register-path or bulk-copy staged reduce-scatter + update kernels "
                         "(auto: the measured default, flashoptim_b200.parallel.tuned_options)")
    ap.add_argument("--timeline", default=None,
                    help="write a summary of a torch.profiler trace of two steps (kernel time per stream and "
                         "per kernel family, rank 0) to this file; never a benchmark number")
    ap.add_argument("--own-all-gather", action="store_true",
                    help="fused path: FSDP2's parameter all-gather through this library's pull kernel")
    ap.add_argument("--all-gather", default="auto", choices=["auto", "copy_engine", "nccl"],
                    help="fused path: copy_engine = FSDP2's parameter all-gather as cudaMemcpyAsync pulls between "
                         "two flag kernels (no SM, three group-sized buffers), the default; nccl = FSDP2's own")
    ap.add_argument("--oversized-groups", default="nccl", choices=["nccl", "fused"],
                    help="fused path: a parameter group more than twice the typical size (embedding + output "
                         "head) keeps FSDP2's NCCL collectives, so the pooled symmetric buffers stay layer-sized "
                         "(nccl, default), or is served too (fused)")
    ap.add_argument("--push-params", default="auto", choices=["auto", "on", "off"],
                    help="fused path: the update kernel also stores the new parameters into every rank's "
                         "all-gather buffer, so FSDP2's parameter all-gathers move no data (1-2 % faster than the "
                         "copy-engine all-gather, at the price of an unsharded copy of the parameters per GPU); "
                         "auto = off (the copy-engine all-gather keeps peak memory where FSDP2's own is)")
    ap.add_argument("--push-budget-gb", type=float, default=0.0,
                    help="with the parameter push: GiB of persistent all-gather buffers per GPU (0: every group)")
    ap.add_argument("--multicast", default="auto", choices=["auto", "on", "off"],
                    help="fused path: NVSwitch multimem.ld_reduce (on) or peer loads summed in fp32 (off); "
                         "auto = peer loads at 2 GPUs, multimem above (the configurations this "
                         "benchmark has been measured in)")
    ap.add_argument("--no-multicast", action="store_true", help="same as --multicast off")
    return ap.parse_args()


def load_module_from(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


# Defaults of the fused FSDP2 path: flashoptim_b200.parallel.tuned_options(world, bytes), i.e.
# what the sweeps of this script (`--sweep`) measured best on 2, 4 and 8 B200s.


def measured_hbm_gbs() -> float:
    """Copy bandwidth measured on this pool's B200s (the roofline denominator), or the
    earlier measurement of 6650 GB/s when the file is absent."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0


def _kernel_family(name: str) -> str:
    n = name.lower()
    if n.startswith("fo::") or "fo::" in n:
        return "flashoptim_b200"
    if "nccl" in n:
        return "nccl"
    if "flash" in n or "fmha" in n or "attention" in n or "sdpa" in n:
        return "attention"
    if "gemm" in n or "cutlass" in n or "nvjet" in n or "xmma" in n or "cublas" in n:
        return "gemm"
    if "memcpy" in n or "memset" in n:
        return "memcpy"
    return "other"


def _union_ms(intervals) -> float:
    total, end = 0.0, None
    for a, b in sorted(intervals):
        if end is None or a > end:
            total += b - a
            end = b
        elif b > end:
            total += b - end
            end = b
    return total / 1e3


def timeline_summary(step_fn, rank: int, path: str, fused_state) -> dict:
    """Two steps under torch.profiler (CUDA activities only) on rank 0, reduced to: wall time
    per step, busy time per stream, kernel time per family, and how long the stream that runs
    the GEMMs sat idle.  With a fused path the same is recorded again with FSDP2's NCCL
    collectives.  Diagnostic only: nothing measured under a profiler is a benchmark number."""
    import tempfile

    import torch
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    def capture(label):
        for _ in range(2):
            step_fn()
        torch.cuda.synchronize()
        dist.barrier()
        out = None
        if rank == 0:
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(2):
                    step_fn()
                torch.cuda.synchronize()
            with tempfile.TemporaryDirectory() as d:
                f = os.path.join(d, "trace.json")
                prof.export_chrome_trace(f)
                with open(f) as fh:
                    trace = json.load(fh)
            ks = [e for e in trace.get("traceEvents", [])
                  if e.get("ph") == "X" and e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset")]
            if ks:
                t0 = min(e["ts"] for e in ks)
                t1 = max(e["ts"] + e["dur"] for e in ks)
                streams, fam, fam_n, by_name = {}, {}, {}, {}
                for e in ks:
                    sid = e.get("args", {}).get("stream", -1)
                    name = e["name"] if e.get("cat") == "kernel" else e.get("cat")
                    k = _kernel_family(name)
                    streams.setdefault(sid, {"iv": [], "fam": {}})
                    streams[sid]["iv"].append((e["ts"], e["ts"] + e["dur"]))
                    streams[sid]["fam"][k] = streams[sid]["fam"].get(k, 0.0) + e["dur"] / 1e3
                    fam[k] = fam.get(k, 0.0) + e["dur"] / 1e3
                    fam_n[k] = fam_n.get(k, 0) + 1
                    short = name.split("(")[0][:70]
                    t_n = by_name.setdefault(short, [0.0, 0])
                    t_n[0] += e["dur"] / 1e3
                    t_n[1] += 1
                gemm_stream = max(streams, key=lambda sid: streams[sid]["fam"].get("gemm", 0.0))
                wall = (t1 - t0) / 1e3
                out = {
                    "label": label, "steps": 2, "wall_ms_per_step": round(wall / 2, 2),
                    "kernel_ms_per_step_by_family": {k: round(v / 2, 2) for k, v in sorted(fam.items())},
                    "launches_per_step_by_family": {k: v / 2 for k, v in sorted(fam_n.items())},
                    "top_kernels_ms_per_step": [
                        {"name": nm, "ms": round(v[0] / 2, 2), "launches": v[1] / 2}
                        for nm, v in sorted(by_name.items(), key=lambda kv: -kv[1][0])[:14]],
                    "compute_stream": gemm_stream,
                    "compute_stream_idle_ms_per_step": round((wall - _union_ms(streams[gemm_stream]["iv"])) / 2, 2),
                    "streams": {str(sid): {"busy_ms_per_step": round(_union_ms(v["iv"]) / 2, 2),
                                           "kernel_ms_per_step_by_family": {k: round(x / 2, 2) for k, x in v["fam"].items()}}
                                for sid, v in streams.items()},
                }
        else:
            for _ in range(2):
                step_fn()
            torch.cuda.synchronize()
        dist.barrier()
        return out

    records = [capture("default configuration")]
    if fused_state is not None:
        saved = (fused_state.enabled, fused_state.push_enabled)
        fused_state.enabled, fused_state.push_enabled = False, False
        records.append(capture("FSDP2's NCCL collectives + this library's step"))
        fused_state.enabled, fused_state.push_enabled = saved
    if rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(records, f, indent=1)
    return {"records": len(records)}


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
    if args.sweep and (args.impl != "ours" or world < 2):
        raise SystemExit("--sweep compares this library's collective paths: it needs --impl ours and >= 2 GPUs")
    tuned = {}
    if args.impl == "ours" and world > 1:
        from flashoptim_b200.parallel import tuned_options

        # bf16 parameters; --push-params on grants the memory for the all-gather on write
        tuned = tuned_options(world, n_params * 2, push_budget_bytes=(1 << 62) if args.push_params == "on" else 0)
    staged = tuned.get("staged", False) if args.comm_kernel == "auto" else args.comm_kernel == "staged"
    transport = "kernel" if args.transport == "auto" else args.transport
    use_multicast = tuned.get("use_multicast", False) if args.multicast == "auto" else args.multicast == "on"
    if args.no_multicast or ((staged or transport == "copy_engine") and args.multicast != "on"):
        use_multicast = False  # staged kernels and copy engines read the peers' buffers directly
    comm_ctas = tuned.get("max_ctas", 0) if args.comm_ctas < 0 else args.comm_ctas
    push_mc = tuned.get("push_multicast", use_multicast) if args.push_multicast == "auto" else args.push_multicast == "on"
    push_params = tuned.get("push_params", False) if args.push_params == "auto" else args.push_params == "on"
    ag_ce = (tuned.get("all_gather_copy_engine", False) and not push_params) if args.all_gather == "auto" \
        else args.all_gather == "copy_engine"
    own_ag = args.own_all_gather or ag_ce
    if own_ag and args.push_params != "on":
        push_params = False
    if push_params and args.all_gather == "auto" and args.push_budget_gb > 0:
        own_ag = ag_ce = True  # groups beyond the push budget: copy-engine all-gather instead of NCCL
    if args.sweep:  # every variant must be reachable by flipping switches at run time
        use_multicast, push_params, own_ag = True, True, True
    if args.impl == "ours" and args.fused_comm == "auto":
        try:
            from flashoptim_b200.parallel import fsdp as fo_fsdp

            fused_state = fo_fsdp.enable_fused_fsdp(model, opt, timeout_s=20.0, max_ctas=comm_ctas,
                                                    use_multicast=use_multicast, own_all_gather=own_ag,
                                                    all_gather_copy_engine=ag_ce,
                                                    push_params=push_params, staged=staged, push_multicast=push_mc,
                                                    transport=transport, oversized_groups=args.oversized_groups,
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
    # read-only NVML sampler, loaded by path like the model file (no package import in the reference arm)
    timing = load_module_from(os.path.join(ROOT, "flashoptim_b200", "utils", "timing.py"), "_bench_timing")
    sampler = timing.ClockSampler(local_rank)

    def timed_steps(n: int) -> float:
        """ms per step of ``n`` steps on resident inputs: CUDA events, barrier + synchronize on
        both sides, maximum over ranks."""
        nonlocal i
        dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n):
            train_step(dev_tokens[i % total_steps])
            i += 1
        t1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([t0.elapsed_time(t1) / n], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    if args.sweep:
        if fused_state is None:
            raise SystemExit(f"--sweep: the fused path could not be set up ({fused_error})")
        sampler.start()
        results = []
        for entry in args.sweep.split(";"):
            f = entry.strip().split(":")
            mode = f[0]
            ctas = int(f[1]) if len(f) > 1 and f[1] else 0
            loads = f[2] if len(f) > 2 and f[2] else "mc"
            cap_all = len(f) > 3 and f[3] == "capall"
            if mode not in ("nccl", "fused", "push", "pull", "pullce", "agce") or loads not in ("mc", "p2p", "p2pmc", "staged", "stagedmc",
                                                                      "ce", "cestaged"):
                raise SystemExit(f"--sweep: bad entry {entry!r}")
            fused_state.enabled = mode not in ("nccl", "agce")
            fused_state.ag_copy_engine = mode in ("pullce", "agce")
            fused_state.set_all_gather_mode({"push": "push", "pull": "pull", "pullce": "pull", "agce": "pull"}
                                            .get(mode, "nccl"))
            fused_state.peers.max_ctas = ctas
            fused_state.peers.use_multicast = loads == "mc"
            fused_state.peers.variant = 1 if "staged" in loads else 0
            fused_state.transport = "copy_engine" if loads.startswith("ce") else "kernel"
            fused_state.peers.push_multicast = loads.endswith("mc")
            fused_state.comms[0][1].full_grid = not cap_all and len(fused_state.comms) > 1
            for _ in range(2):  # settle: the first step after a switch still runs the old all-gathers
                train_step(dev_tokens[i % total_steps])
                i += 1
            fused_state.check()
            c0 = (fused_state.fused_calls, fused_state.fallbacks, fused_state.ag_eliminated, fused_state.ag_fallbacks)
            torch.cuda.reset_peak_memory_stats()
            ag0 = fused_state.ag_calls
            ms = timed_steps(args.steps)
            fused_state.check()
            c1 = (fused_state.fused_calls, fused_state.fallbacks, fused_state.ag_eliminated, fused_state.ag_fallbacks)
            results.append({
                "entry": entry.strip(), "mode": mode, "comm_ctas": ctas, "loads": loads if mode != "nccl" else None,
                "last_group_full_grid": not cap_all,
                "ms_per_step": round(ms, 3), "tokens_per_s": round(world * b * s / (ms * 1e-3), 1),
                "peak_gib": round((torch.cuda.max_memory_allocated() + fused_state.peers.symmetric_bytes) / 2**30, 2),
                "per_step": {k: (y - x) / args.steps for k, x, y in
                             zip(("fused_rs", "nccl_rs", "ag_eliminated", "nccl_ag"), c0, c1)},
            })
            results[-1]["per_step"]["own_ag"] = (fused_state.ag_calls - ag0) / args.steps
            if rank == 0:
                print(f"[sweep] {results[-1]}", file=sys.stderr, flush=True)
        sampler.stop()
        if args.timeline:  # the last entry's configuration against FSDP2's NCCL collectives
            timeline_summary(lambda: train_step(dev_tokens[i % total_steps]), rank, args.timeline, fused_state)
        if rank == 0:
            print(json.dumps({"sweep": results, "n_gpus": world, "steps": args.steps, "model": args.model,
                              "seq_len": s, "optimizer": args.optimizer, "master_weight_bits": mwb,
                              "gradient_release": bool(args.gradient_release), "clocks": sampler.summary()}),
                  flush=True)
        dist.destroy_process_group()
        return

    # ---- device-timed loop (inputs resident on the device)
    sampler.start()
    l0 = launches()
    dev_ms = timed_steps(args.steps)
    n_launch = launches() - l0

    # ---- end-to-end loop: pinned-host inputs in, loss out, every step
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    last_loss = 0.0
    for _ in range(args.steps):
        tok = host_tokens[i % total_steps].to(dev, non_blocking=True)
        last_loss = float(train_step(tok).item())
        i += 1
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    sampler.stop()
    if fused_state is not None:
        fused_state.check()
    dist.barrier()
    # symmetric (NVLink-mapped) buffers are not seen by PyTorch's allocator statistics
    symmetric_bytes = fused_state.peers.symmetric_bytes if fused_state is not None else 0
    peak_bytes = torch.cuda.max_memory_allocated() + symmetric_bytes
    free_b, total_b = torch.cuda.mem_get_info()
    device_used = total_b - free_b  # the driver's view: context, NCCL, allocator reserve, symmetric memory

    # ---- the optimizer step alone (the second half of the headline metric): gradients of one
    # more backward pass are kept and optimizer.step() is timed on them, on this rank's shards
    step_stats = None
    if not args.gradient_release:
        if fused_state is not None:
            fused_state.enabled = False  # this backward leaves its gradients to optimizer.step()
        model(dev_tokens[i % total_steps][:, :-1], dev_tokens[i % total_steps][:, 1:]).backward()
        i += 1
        opt.step()  # untimed: after a switch of paths the segment tables are rebuilt once
        torch.cuda.synchronize()
        reps = 10
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        h0 = time.perf_counter()
        ev[0].record()
        for k in range(reps):
            opt.step()
            ev[k + 1].record()
        step_host_ms = (time.perf_counter() - h0) * 1e3 / reps  # time the host needs to issue one step
        torch.cuda.synchronize()
        times = sorted(ev[k].elapsed_time(ev[k + 1]) for k in range(reps))
        opt.zero_grad(set_to_none=True)
        if fused_state is not None:
            fused_state.enabled = True
        local_elems = sum((p._local_tensor if hasattr(p, "_local_tensor") else p).numel() for p in model.parameters())
        t = torch.tensor([times[reps // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms = float(t.item())
        state_bytes = {"adamw": 4.25, "lion": 2.125}[args.optimizer]  # 8-bit codes + fp16 scale per 32, r+w
        ecc_bytes = {None: 0, 24: 2, 32: 4}[mwb]
        bytes_per_elem = 2 + 2 + 2 + state_bytes + ecc_bytes  # param r+w, grad r, states, correction r+w
        step_stats = {
            "step_ms": round(step_ms, 3),
            "step_ms_per_1b": round(step_ms / (local_elems / 1e9), 3),
            "step_hbm_frac": round(bytes_per_elem * local_elems / (step_ms * 1e-3) / (measured_hbm_gbs() * 1e9), 3),
            "step_host_ms": round(step_host_ms, 3),
            "step_local_params": local_elems,
            "step_bytes_per_param": bytes_per_elem,
            "step_timing": f"median of {reps} optimizer.step() calls, CUDA events, max over ranks; HBM fraction of "
                           f"the measured copy bandwidth {measured_hbm_gbs()} GB/s; when step_host_ms is not well below "
                           "step_ms the loop is bound by the host's walk over the parameter list, not by the kernel",
        }

    timeline = None
    if args.timeline:
        timeline = timeline_summary(lambda: train_step(dev_tokens[i % total_steps]), rank, args.timeline, fused_state)

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

    t = torch.tensor([e2e_ms, peak_bytes / 2**30, device_used / 2**30], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms, peak_gib, used_gib = (float(x) for x in t.tolist())
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
                "fused_comm_ctas": comm_ctas if fused_comm else None,
                "fused_comm_kernel": ("staged" if staged else "register") if fused_comm else None,
                "fused_comm_transport": transport if fused_comm else None,
                "fused_oversized_groups": args.oversized_groups if fused_comm else None,
                "fused_all_gather": (fused_state.all_gather_mode + ("/copy_engine" if fused_state.ag_copy_engine and
                                     fused_state.all_gather_mode == "pull" else "")) if fused_comm else None,
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
            "peak_gib_note": "torch.cuda.max_memory_allocated plus this library's symmetric NVLink buffers "
                             f"({symmetric_bytes / 2**30:.2f} GiB, invisible to the allocator statistics)",
            "device_used_gib_per_gpu": round(used_gib, 2),
            "clocks": sampler.summary(),
        }
        if step_stats is not None:
            rec.update(step_stats)
        if dcp_times is not None:
            rec["dcp"] = dcp_times
        if timeline is not None:
            rec["timeline_file"] = args.timeline
        print(json.dumps(rec), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
