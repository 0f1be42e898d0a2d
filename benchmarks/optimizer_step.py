"""Optimizer-step micro-benchmark on one GPU, no model.

Tensors have the shapes of a Llama-3-8B parameter list (291 tensors, 8.03 B
elements): embedding and lm_head 128256x4096; per layer (x32) q/o 4096x4096,
k/v 1024x4096, gate/up 14336x4096, down 4096x14336 and two RMSNorm weights of
4096.  Params ~ N(0, 0.02), grads ~ N(0, 1e-3), seed 0.  Every step reads and
writes far more than the 126 MB L2, so no flush is needed between iterations.

    python benchmarks/optimizer_step.py --optimizers adamw,lion,sgdw --mwb 24,32,none
    python benchmarks/optimizer_step.py --impl reference   # the reference's Triton build

    python benchmarks/optimizer_step.py --kernels [--impl reference]   # stand-alone kernels

Prints one JSON line per (optimizer, master_weight_bits): device-timed ms per
step (CUDA events around K steps), ms per 1e9 parameters, bytes per element and
the achieved fraction of the measured copy bandwidth (MEASURED_PEAKS.json), plus
the SM clocks and throttle reasons sampled through NVML (read-only) during the run.
``--kernels`` times the stand-alone group quantiser / dequantiser and the master-weight
split / merge (the reference's Triton kernels ``flashoptim/optimizers.py:2541-2676,
2779-2832``) on one 2^28-element tensor instead (``--log2-elems 26`` for a profiler capture).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def llama8b_shapes(layers: int = 32, d: int = 4096, ffn: int = 14336, vocab: int = 128256, kv: int = 1024):
    shapes = [(vocab, d)]
    for _ in range(layers):
        shapes += [(d, d), (kv, d), (kv, d), (d, d), (ffn, d), (ffn, d), (d, ffn), (d,), (d,)]
    shapes += [(d,), (vocab, d)]
    return shapes


def bytes_per_elem(opt: str, mwb) -> float:
    """HBM bytes per element of one fused step: bf16 param + grad read, param write,
    8-bit states read + written with one fp16 scale per 32 elements, codes read + written."""
    states = 2 if opt.startswith("adam") else 1
    ecc = {None: 0, 24: 1, 32: 2}[mwb]
    return 2 + 2 + 2 + states * 2 * (1 + 2 / 32) + 2 * ecc


def hbm_peak_gbs() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def load_clock_sampler():
    """The read-only NVML sampler, loaded by file path so that the reference arm does not
    import this library's package."""
    import importlib.util

    path = os.path.join(ROOT, "flashoptim_b200", "utils", "timing.py")
    spec = importlib.util.spec_from_file_location("_bench_timing", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["_bench_timing"] = mod
    spec.loader.exec_module(mod)
    return mod.ClockSampler


def time_fn(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_kernels(args, peak: float, peak_src: str) -> list[dict]:
    """Stand-alone kernels on 2^28 elements by default (0.5 GB of bf16: far beyond the 126 MB L2)."""
    dev = torch.device("cuda", 0)
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import flashoptim as lib
        from flashoptim.optimizers import dequantize, quantize
    else:
        import flashoptim_b200 as lib
        from flashoptim_b200 import dequantize, quantize
    n = 1 << args.log2_elems
    g = torch.Generator(device=dev).manual_seed(0)
    x32 = torch.empty(n, device=dev).normal_(0, 0.02, generator=g)
    xb = x32.to(torch.bfloat16)
    sq = x32.square()
    out = []

    def record(name, fn, nbytes):
        ms = time_fn(fn, args.steps, args.warmup)
        gbs = nbytes / (ms * 1e-3) / 1e9
        rec = {"impl": args.impl, "kernel": name, "n": n, "ms": round(ms, 4), "bytes": nbytes,
               "achieved_GBps": round(gbs, 1), "hbm_peak_GBps": peak, "frac_of_" + peak_src: round(gbs / peak, 4)}
        print(json.dumps(rec), flush=True)
        out.append(rec)

    scale_bytes = n // 32 * 2
    q_s = torch.empty(n, dtype=torch.int8, device=dev)
    q_u = torch.empty(n, dtype=torch.uint8, device=dev)
    sc = torch.empty(n // 32, dtype=torch.float16, device=dev)
    f32 = torch.empty(n, dtype=torch.float32, device=dev)
    record("quantize bf16 -> int8 (signed, companded)",
           lambda: quantize(xb, q_s, sc, signed=True, sqrt=False, softsign=True), n * 3 + scale_bytes)
    record("quantize fp32 -> uint8 (sqrt domain)",
           lambda: quantize(sq, q_u, sc, signed=False, sqrt=True, softsign=False), n * 5 + scale_bytes)
    quantize(xb, q_s, sc, signed=True, sqrt=False, softsign=True)
    record("dequantize int8 -> fp32 (signed, companded)",
           lambda: dequantize(q_s, sc, f32, signed=True, sqrt=False, softsign=True), n * 5 + scale_bytes)
    for bytewidth, code_bytes in ((3, 1), (4, 2)):
        ecc = lib.compute_ecc_bits(x32, xb, master_bytewidth=bytewidth)
        record(f"compute_ecc_bits fp32, bf16 -> int{8 * code_bytes}",
               lambda: lib.compute_ecc_bits(x32, xb, master_bytewidth=bytewidth), n * (4 + 2 + code_bytes))
        record(f"reconstruct_fp32_param bf16 + int{8 * code_bytes} -> fp32",
               lambda: lib.reconstruct_fp32_param(xb, ecc), n * (2 + code_bytes + 4))
    return out


def make_optimizer(impl: str, name: str, params, mwb):
    if impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import flashoptim as lib
    else:
        import flashoptim_b200 as lib
    if name == "adamw":
        return lib.FlashAdamW(params, lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01, master_weight_bits=mwb)
    if name == "lion":
        return lib.FlashLion(params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.01, master_weight_bits=mwb)
    if name == "sgdw":
        return lib.FlashSGDW(params, lr=1e-3, momentum=0.9, weight_decay=0.01, master_weight_bits=mwb)
    raise ValueError(name)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--optimizers", default="adamw,lion,sgdw")
    ap.add_argument("--mwb", default="24,32,none")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32, help="fewer layers = smaller problem (profiling)")
    ap.add_argument("--vocab", type=int, default=128256, help="smaller vocabulary = smaller problem")
    ap.add_argument("--variant", type=int, default=None, help="ours: 0 register-path kernels, 1 staged (default)")
    ap.add_argument("--kernels", action="store_true",
                    help="time the stand-alone quantise / dequantise / master-weight split kernels instead")
    ap.add_argument("--log2-elems", type=int, default=28,
                    help="--kernels: tensor size as a power of two (26 for a profiler capture: 256 MB of fp32)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.variant is not None and args.impl == "ours":
        from flashoptim_b200.ops.step import set_step_variant

        set_step_variant(args.variant)
    peak, peak_src = hbm_peak_gbs()
    sampler = load_clock_sampler()(0)
    sampler.start()
    if args.kernels:
        results = run_kernels(args, peak, peak_src)
        sampler.stop()
        clocks = {"clocks": sampler.summary()}
        print(json.dumps(clocks), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                for r in results + [clocks]:
                    f.write(json.dumps(r) + "\n")
        return
    shapes = llama8b_shapes(layers=args.layers, vocab=args.vocab)
    g = torch.Generator(device=dev).manual_seed(0)
    params = []
    for s in shapes:
        p = torch.empty(s, device=dev, dtype=torch.bfloat16)
        p.copy_(torch.randn(s, device=dev, generator=g) * 0.02) if len(s) == 1 else p.normal_(0, 0.02, generator=g)
        params.append(torch.nn.Parameter(p))
    for p in params:
        p.grad = torch.empty_like(p).normal_(0, 1e-3, generator=g)
    n_total = sum(p.numel() for p in params)
    results = []
    import warnings

    warnings.simplefilter("ignore")
    for name in args.optimizers.split(","):
        for m in args.mwb.split(","):
            mwb = None if m == "none" else int(m)
            opt = make_optimizer(args.impl, name, params, mwb)
            for _ in range(args.warmup):
                opt.step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            for _ in range(args.steps):
                opt.step()
            e1.record()
            host_ms = (time.perf_counter() - t0) * 1e3 / args.steps
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            bpe = bytes_per_elem(name, mwb)
            gbs = n_total * bpe / (ms * 1e-3) / 1e9
            rec = {
                "impl": args.impl, "optimizer": name, "master_weight_bits": mwb, "n_tensors": len(params),
                "n_params": n_total, "ms_per_step": round(ms, 4), "host_ms_per_step": round(host_ms, 4),
                "ms_per_1B_params": round(ms / (n_total / 1e9), 4), "bytes_per_elem": bpe,
                "achieved_GBps": round(gbs, 1), "hbm_peak_GBps": peak,
                "frac_of_" + peak_src: round(gbs / peak, 4), "steps": args.steps, "warmup": args.warmup,
            }
            print(json.dumps(rec), flush=True)
            results.append(rec)
            del opt
            torch.cuda.empty_cache()
    sampler.stop()
    clocks = {"clocks": sampler.summary()}
    print(json.dumps(clocks), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            for r in results + [clocks]:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
