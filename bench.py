#!/usr/bin/env python
"""Benchmark of the mixed-precision decode GEMV on the Qwen3-4B-shaped decoder block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--impl ours|reference]

A "step" is one pass over the seven linears of one decoder block (q, k, v, o, gate, up,
down; 67/32/1 NVFP4/FP8/FP16 split rounded to 128 channels, random channel permutation,
seeded synthetic weights ~ N(0, 0.02) with 1 % outlier channels x8) at M activation rows:
seven PDL-chained GEMV launches.  The metric is packed weight + scale bytes streamed per
second (GB/s).  Weight copies rotate through more than twice the L2 capacity, so every
launch reads HBM.  With N > 1 (torchrun) every rank streams its own block-sized shard; no
collective is on this path.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference operator (oracle/rdq_oracle.c, all host threads) on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "mixed_gemv_hbm_gbps"
UNIT = "GB/s"
LAYER_ORDER = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the bench runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.samples.append((time.time(), line.strip()))

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = [s for s in self.samples if t0 - 0.05 <= s[0] <= t1 + 0.15] or self.samples
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for _, line in rows:
            parts = [p.strip() for p in line.split(",")]
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


FUSE_GROUPS = [["q_proj", "k_proj", "v_proj"], ["o_proj"], ["gate_proj", "up_proj"], ["down_proj"]]


def build_block(device, seed: int, copies: int, fuse: bool):
    """`copies` independent device copies of the packed linears of one block.  With `fuse`,
    projections that read the same input (q/k/v, gate/up) are packed as one layer each."""
    import torch

    from rdquant_b200.fused_gemv_pack import fuse_layers, layer_data_from_qweight, pack_for_fused_gemv, packed_weight_bytes
    from rdquant_b200.quantize import quantize_weight
    from rdquant_b200.synthetic import QWEN3_4B_BLOCK, fixed_splits, synthetic_weight

    per_layer = {}
    for li, name in enumerate(LAYER_ORDER):
        k, n = QWEN3_4B_BLOCK[name]
        gen = torch.Generator().manual_seed(seed * 100 + li)
        w = synthetic_weight(n, k, gen)
        perm = torch.randperm(n, generator=gen)
        splits = fixed_splits(n)
        # encode on the GPU (torch ops; offline step)
        qw = quantize_weight(w.to(device).float(), perm.to(device), splits)
        per_layer[name] = (layer_data_from_qweight(qw), splits, k, n)
        del w, qw
    groups = FUSE_GROUPS if fuse else [[n] for n in LAYER_ORDER]
    units = []
    for group in groups:
        k = per_layer[group[0]][2]
        nbytes = sum(packed_weight_bytes(per_layer[g][1], k) for g in group)
        if len(group) > 1:
            data, splits = fuse_layers([(per_layer[g][0], per_layer[g][1]) for g in group])
        else:
            data, splits = per_layer[group[0]][0], per_layer[group[0]][1]
        fds = [pack_for_fused_gemv({kk: v.clone() for kk, v in data.items()}, splits, k, device) for _ in range(copies)]
        units.append({"name": "+".join(group), "k": k, "n": sum(per_layer[g][3] for g in group), "splits": splits,
                      "fds": fds, "bytes": nbytes})
    return units


def cpu_baseline(budget_s: float = 12.0) -> dict:
    """The CPU restatement of the reference operator (re-dequantises per call, like
    rdquant/ops.py:55-60) on gate_proj (2560 -> 9728) at M = 1, all host threads."""
    import numpy as np
    import torch

    from oracle import oracle_c
    from rdquant_b200.fused_gemv_pack import packed_weight_bytes
    from rdquant_b200.quantize import quantize_weight
    from rdquant_b200.synthetic import QWEN3_4B_BLOCK, fixed_splits, synthetic_weight

    oracle_c.build()
    oracle_c.set_threads(os.cpu_count() or 1)  # launchers like torchrun export OMP_NUM_THREADS=1
    k, n = QWEN3_4B_BLOCK["gate_proj"]
    gen = torch.Generator().manual_seed(4)
    w = synthetic_weight(n, k, gen)
    perm = torch.randperm(n, generator=gen)
    splits = fixed_splits(n)
    qw = quantize_weight(w.float(), perm, splits)
    q4, q8, q16 = qw.qtensors["NVFP4"], qw.qtensors["FP8"], qw.qtensors["FP16"]
    args = (np.ascontiguousarray(q4.data.numpy()), np.ascontiguousarray(q4.scales.numpy()), splits["NVFP4"],
            np.ascontiguousarray(q8.data.numpy()), float(q8.scales.item()), splits["FP8"],
            np.ascontiguousarray(q16.data.numpy()), splits["FP16"], qw.inv_permutation.numpy())
    x = torch.randn(1, k, generator=gen).half().numpy()
    oracle_c.linear(x, *args)
    calls, t0 = 0, time.perf_counter()
    while True:
        oracle_c.linear(x, *args)
        calls += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or calls >= 400:
            break
    nbytes = packed_weight_bytes(splits, k)
    return {"value": nbytes * calls / dt / 1e9, "unit": UNIT, "cores": oracle_c.threads(), "kind": "port",
            "sample": f"gate_proj 2560->9728, M=1, {calls} calls in {dt:.1f} s ({1e3 * dt / calls:.2f} ms/call)",
            "ms_per_call": 1e3 * dt / calls, "calls": calls, "bytes_per_call": nbytes}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    steps = max(args.steps, 1)
    base = cpu_baseline(budget_s=min(60.0, 0.25 * (steps + args.warmup) + 8.0))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_call"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {"workload": "qwen3-4b decoder block, 7 mixed-precision linears, M=1 decode GEMV",
                   "sample": base["sample"], "note": "reference is a Python package; timed here as its C restatement "
                   "(oracle/rdq_oracle.c) on the host cores"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_prefill(args, device, rank: int, world: int) -> None:
    """Prefill GEMM (BASELINE configs[2]): the seven linears of the block at `--prefill` tokens."""
    import torch

    from rdquant_b200 import rdquant_cuda

    m = args.prefill
    steps, warmup = max(min(args.steps, 50), 1), max(args.warmup, 3)
    units = build_block(device, seed=rank, copies=1, fuse=not args.no_fuse)
    gen = torch.Generator().manual_seed(99 + rank)
    xs = [torch.randn(m, u["k"], generator=gen).half().to(device) for u in units]
    flops = sum(2.0 * m * u["n"] * u["k"] for u in units)
    sampler = ClockSampler(device.index or 0)
    sampler.start()

    def one_step():
        for x, u in zip(xs, units):
            rdquant_cuda.mixed_gemm(x, u["fds"][0])

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for _ in range(steps):
        one_step()
    e1.record()
    e1.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t0, t1)
    peaks, kind = measured_peaks()
    tf = flops * steps / (ms * 1e-3) / 1e12
    sustained = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    line = {
        "metric": "mixed_gemm_tflops", "value": tf * world, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {"workload": f"qwen3-4b decoder block: 7 mixed-precision linears, prefill GEMM at M={m} tokens "
                               "(BASELINE configs[2])", "launches_per_step": len(units),
                   "fusion": "q/k/v and gate/up packed as one layer each" if not args.no_fuse else "none", "l2_policy": "activations + outputs of a step exceed L2 for M >= 2048"},
        "gpu_launches": steps * len(units),
        "roofline": {"bound": "tensor", "achieved": tf, "peak": sustained, "unit": "TFLOP/s", "frac": tf / sustained,
                     "traffic": None, "peak_source": kind + " (sustained cuBLAS bf16)", "kernel": "gemm_mixed_kernel"},
        "clocks": clocks,
    }
    if rank == 0:
        print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--m", type=int, default=1, help="activation rows (1..16)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--copies", type=int, default=6, help="rotating weight copies (L2 defeat)")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel", default="tiled", choices=["tiled", "generic"])
    ap.add_argument("--no-fuse", action="store_true", help="seven launches per step instead of four")
    ap.add_argument("--prefill", type=int, default=0, metavar="TOKENS",
                    help="measure the tcgen05 prefill GEMM at this many tokens instead of the decode GEMV")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from rdquant_b200 import _lib, rdquant_cuda

    _lib.lib()  # no kernels, no benchmark
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    if args.prefill > 0:
        run_prefill(args, device, rank, world)
        return
    steps, warmup, m = max(args.steps, 1), max(args.warmup, 3), args.m
    copies = max(args.copies, 2)
    layers = build_block(device, seed=rank, copies=copies, fuse=not args.no_fuse)
    step_bytes = sum(l["bytes"] for l in layers)
    flags = {"tiled": _lib.RDQ_GEMV_AUTO, "generic": _lib.RDQ_GEMV_GENERIC}[args.kernel]
    if not args.no_pdl:
        flags |= _lib.RDQ_GEMV_PDL

    gen = torch.Generator().manual_seed(1234 + rank)
    xs = [torch.randn(m, l["k"], generator=gen).half().to(device) for l in layers]
    ys = [torch.empty(m, l["n"], dtype=torch.float16, device=device) for l in layers]

    def one_step(i: int) -> None:
        c = i % copies
        for li, l in enumerate(layers):
            rdquant_cuda.mixed_gemv(xs[li], l["fds"][c], None, flags, out=ys[li])

    sampler = ClockSampler(local_rank)
    sampler.start()

    # warm-up (also brings the clocks up): W plain steps, then ~0.3 s of the same work
    for i in range(warmup):
        one_step(i)
    torch.cuda.synchronize()
    # a kernel whose bounded waits ran out leaves a status word behind: stop here rather than
    # time steps that each sit through their wait limits
    bad = sum(int(fd["tile_counters"].abs().sum().item()) for l in layers for fd in l["fds"] if "tile_counters" in fd)
    if bad:
        raise RuntimeError(f"GEMV kernels reported {bad} non-zero status words during warm-up")
    stream = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        one_step(0)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                one_step(i)
        t_spin = time.time()
        while time.time() - t_spin < 0.3:
            graph.replay()
            stream.synchronize()

        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record(stream)
        graph.replay()
        e1.record(stream)
        e1.synchronize()
        torch.cuda.synchronize()
        t1 = time.time()
        if world > 1:
            dist.barrier()
    ms = e0.elapsed_time(e1)
    status_bad = sum(int(fd["tile_counters"].abs().sum().item()) for l in layers for fd in l["fds"])

    # ---- end to end through the public API, host buffers in, host buffers out
    from rdquant_b200.inference import FusedMixedLinear, GraphedDecodeStep

    def modules_of(copy: int):
        out = []
        for l in layers:
            fd = l["fds"][copy]
            out.append(FusedMixedLinear(n_nvfp4=fd["n_fp4"], n_fp8=fd["n_fp8"], n_fp16=fd["n_fp16"], k=l["k"],
                                        inv_perm=fd["inv_perm"], bias=None, marlin_data=None, fused_data=fd))
        return out

    # one graphed step per weight copy, rotated like the device-only measurement
    runners = [GraphedDecodeStep(modules_of(c), m=m, use_pdl=not args.no_pdl) for c in range(copies)]
    for runner in runners:
        for xh, x in zip(runner.x_host, xs):
            xh.copy_(x.cpu())
    e2e_steps = min(steps, 200)
    for i in range(copies):
        runners[i].run()
    if world > 1:
        dist.barrier()
    te0 = time.perf_counter()
    for i in range(e2e_steps):
        # host activations in, host results out: one graph replay (H2D copies, GEMVs, D2H copies)
        runners[i % copies].run()
    te = time.perf_counter() - te0
    clocks = sampler.stop(t0, t1)

    # ---- max over ranks
    if world > 1:
        t = torch.tensor([ms, te], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, te = float(t[0]), float(t[1])

    value = world * step_bytes * steps / (ms * 1e-3) / 1e9
    e2e_value = world * step_bytes * e2e_steps / te / 1e9
    peaks, peak_kind = measured_peaks()
    launches = steps * len(layers)
    per_launch_bytes = step_bytes / len(layers)
    achieved = per_launch_bytes / (ms * 1e-3 / launches) / 1e9
    # dram__bytes_read + dram__bytes_write per launch from the ncu capture summarised in
    # profiles/gemv_tiled_block_m1.md (average over the four fused launches of a step)
    traffic = 19.46e6 if (m == 1 and not args.no_fuse and args.kernel == "tiled") else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {
            "workload": f"qwen3-4b decoder block: q,k,v,o,gate,up,down mixed-precision linears, M={m} decode GEMV "
                        "(BASELINE configs[1])",
            "launches_per_step": len(layers),
            "fusion": "none" if args.no_fuse else "q/k/v and gate/up packed as one layer each (they read the same input)",
            "split": "67/32/1 NVFP4/FP8/FP16, 128-aligned, random channel permutation",
            "bytes_per_step": step_bytes, "l2_policy": f"{copies} rotating weight copies = "
            f"{copies * step_bytes / 1e6:.0f} MB > 2 x L2; inputs larger than L2, no flush",
            "launch": "one CUDA graph of all timed steps, PDL-chained launches" if not args.no_pdl else "CUDA graph",
            "parallelism": "1 block-sized column shard per GPU, no collective" if world > 1 else "single GPU",
            "kernel": args.kernel,
        },
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "peak_source": peak_kind,
                     "frac_of_nominal_8tbs": achieved / 8000.0, "kernel": "gemv_%s_kernel" % args.kernel,
                     "bytes_per_launch": per_launch_bytes},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": sum(2 * m * l["k"] for l in layers),
                "d2h_bytes_per_step": sum(2 * m * l["n"] for l in layers), "steps": e2e_steps,
                "ms_per_step": 1e3 * te / e2e_steps,
                "api": "inference.GraphedDecodeStep.run(): pinned host x -> device (staging kernel reading the pinned buffer), fused GEMVs, y -> pinned host (staging kernel) as one CUDA-graph replay, synchronised every step; weight copies rotate as in the device-only measurement"},
        "clocks": clocks,
        "status_words_nonzero": status_bad,
    }
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            base = cpu_baseline()
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
