#!/usr/bin/env python
"""Benchmark of the mixed-precision linear operator on the Qwen3-4B-shaped decoder block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--impl ours|reference]

A "step" is one pass over the seven linears of one decoder block (q, k, v, o, gate, up, down;
67/32/1 NVFP4/FP8/FP16 split rounded to 128 channels, random channel permutation, seeded
synthetic weights ~ N(0, 0.02) with 1 % outlier channels x8) at M activation rows through the
decode GEMV: four PDL-chained launches (q/k/v and gate/up read the same input and are packed as
one layer each).  The metric is packed weight + scale bytes streamed per second (GB/s).  Weight
copies rotate through more than twice the L2 capacity, so every launch reads HBM.

N = 1 also reports, in the same JSON line, the tcgen05 prefill GEMM on the same block
(`prefill`: TFLOP/s at 512 / 2048 / 8192 tokens beside cuBLAS dense f16 on the same shapes, which
is what the reference's prefill runs) and whole-model greedy decoding of the 36-layer
Qwen3-4B-shaped stack (`decode`: tokens/s).

N > 1 (torchrun): ONE block is cut column-parallel at 128-channel boundaries of every format
group (rdquant_b200.parallel); every rank streams its rows, and the per-layer NCCL all-gather and
un-permute are inside the timed CUDA graph ("strong" scaling: value = the block's bytes / step).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the reference
operator (oracle/rdq_oracle.c, all host threads) on a bounded sample of the same block.
"""
import argparse
import json
import os
import statistics
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
FUSE_GROUPS = [["q_proj", "k_proj", "v_proj"], ["o_proj"], ["gate_proj", "up_proj"], ["down_proj"]]
L2_BYTES = 126e6
TOL = 2e-3


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def profiled_traffic(kernel: str, workload: str):
    """dram bytes per launch of the dominant kernel from the tracked ncu summary data
    (profiles/traffic.json), or None when no capture of this kernel / workload is on file."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as fh:
            return json.load(fh).get(kernel, {}).get(workload)
    except (OSError, ValueError):
        return None


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


def block_layers(device, seed: int):
    """Packed checkpoint tensors (on `device`) of the seven linears of one block:
    {name: (layer_data, splits, k, n)}."""
    import torch

    from rdquant_b200.fused_gemv_pack import layer_data_from_qweight
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
    return per_layer


def fused_units(per_layer, fuse: bool):
    """[(name, layer_data, splits, k, n, bytes, members)] of the launches of a step."""
    from rdquant_b200.fused_gemv_pack import fuse_layers, packed_weight_bytes

    groups = FUSE_GROUPS if fuse else [[n] for n in LAYER_ORDER]
    units = []
    for group in groups:
        k = per_layer[group[0]][2]
        nbytes = sum(packed_weight_bytes(per_layer[g][1], k) for g in group)
        if len(group) > 1:
            data, splits = fuse_layers([(per_layer[g][0], per_layer[g][1]) for g in group])
        else:
            data, splits = per_layer[group[0]][0], per_layer[group[0]][1]
        units.append({"name": "+".join(group), "data": data, "splits": splits, "k": k,
                      "n": sum(per_layer[g][3] for g in group), "bytes": nbytes, "members": group})
    return units


def build_block(device, seed: int, copies: int, fuse: bool):
    """`copies` independent device copies of the packed linears of one block.  With `fuse`,
    projections that read the same input (q/k/v, gate/up) are packed as one layer each."""
    from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv

    per_layer = block_layers(device, seed)
    units = fused_units(per_layer, fuse)
    for u in units:
        u["fds"] = [pack_for_fused_gemv({kk: v.clone() for kk, v in u["data"].items()}, u["splits"], u["k"], device)
                    for _ in range(copies)]
    return units, per_layer


def oracle_outputs(per_layer, unit, x_f16):
    """CPU oracle output [M, n] of one (possibly fused) launch: the member layers side by side."""
    import numpy as np

    from oracle import oracle_np as onp

    parts = []
    for name in unit["members"]:
        data, splits, k, _ = per_layer[name]
        layer = onp.torch_layer_to_np({kk: v.cpu() for kk, v in data.items()})
        parts.append(onp.mixed_precision_linear(x_f16, layer, splits, k))
    return np.concatenate(parts, axis=1)


def cpu_baseline(budget_s: float = 12.0) -> dict:
    """The CPU restatement of the reference operator (re-dequantises per call, like
    rdquant/ops.py:55-60) on the seven linears of the block at M = 1, all host threads."""
    import numpy as np
    import torch

    from oracle import oracle_c
    from rdquant_b200.fused_gemv_pack import packed_weight_bytes
    from rdquant_b200.quantize import quantize_weight
    from rdquant_b200.synthetic import QWEN3_4B_BLOCK, fixed_splits, synthetic_weight

    oracle_c.build()
    oracle_c.set_threads(os.cpu_count() or 1)  # launchers like torchrun export OMP_NUM_THREADS=1
    calls_args, nbytes = [], 0
    for li, name in enumerate(LAYER_ORDER):
        k, n = QWEN3_4B_BLOCK[name]
        gen = torch.Generator().manual_seed(400 + li)
        w = synthetic_weight(n, k, gen)
        perm = torch.randperm(n, generator=gen)
        splits = fixed_splits(n)
        qw = quantize_weight(w.float(), perm, splits)
        q4, q8, q16 = qw.qtensors["NVFP4"], qw.qtensors["FP8"], qw.qtensors["FP16"]
        x = torch.randn(1, k, generator=gen).half().numpy()
        calls_args.append((x, np.ascontiguousarray(q4.data.numpy()), np.ascontiguousarray(q4.scales.numpy()),
                           splits["NVFP4"], np.ascontiguousarray(q8.data.numpy()), float(q8.scales.item()),
                           splits["FP8"], np.ascontiguousarray(q16.data.numpy()), splits["FP16"],
                           qw.inv_permutation.numpy()))
        nbytes += packed_weight_bytes(splits, k)
    for a in calls_args:
        oracle_c.linear(*a)
    steps, t0 = 0, time.perf_counter()
    while True:
        for a in calls_args:
            oracle_c.linear(*a)
        steps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or steps >= 200:
            break
    return {"value": nbytes * steps / dt / 1e9, "unit": UNIT, "cores": oracle_c.threads(), "kind": "port",
            "sample": f"all 7 linears of the block, M=1, {steps} block passes in {dt:.1f} s "
                      f"({1e3 * dt / steps:.1f} ms/pass)",
            "ms_per_step": 1e3 * dt / steps, "steps": steps, "bytes_per_step": nbytes}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    base = cpu_baseline(budget_s=min(60.0, 0.25 * (max(args.steps, 1) + args.warmup) + 8.0))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {"workload": "qwen3-4b decoder block: q,k,v,o,gate,up,down mixed-precision linears, M=1 decode GEMV",
                   "sample": base["sample"], "note": "the reference operator is a Python package that cannot travel to "
                   "the GPU box; timed here as its C restatement (oracle/rdq_oracle.c) on the host cores, "
                   "re-dequantising per call like rdquant/ops.py:55-60"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def time_replays(graph, stream, replays: int):
    """Device times (ms) of `replays` replays of a CUDA graph, each bracketed by events."""
    import torch

    times = []
    for _ in range(replays):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graph.replay()
        e1.record(stream)
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    return times


def prefill_section(device, units, tokens=(512, 2048, 8192), steps: int = 10) -> dict:
    """tcgen05 prefill GEMM on the block's four launches at each token count, beside cuBLAS dense
    f16 (torch F.linear over a materialised weight: the reference's prefill path,
    rdquant/inference.py:679-687) on the same shapes in the same run."""
    import torch

    from rdquant_b200 import rdquant_cuda

    peaks, _ = measured_peaks()
    sustained = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    out = {}
    dense = [torch.randn(u["n"], u["k"], device=device, dtype=torch.float16) * 0.02 for u in units]
    for m in tokens:
        gen = torch.Generator().manual_seed(99 + m)
        xs = [torch.randn(m, u["k"], generator=gen).half().to(device) for u in units]
        flops = sum(2.0 * m * u["n"] * u["k"] for u in units)

        def ours():
            for x, u in zip(xs, units):
                rdquant_cuda.mixed_gemm(x, u["fds"][0])

        def cublas():
            for x, w in zip(xs, dense):
                torch.nn.functional.linear(x, w)

        res = {}
        for name, fn in (("tflops", ours), ("cublas_dense_tflops", cublas)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            e1.synchronize()
            res[name] = flops * steps / (e0.elapsed_time(e1) * 1e-3) / 1e12
        rdquant_cuda.check_gemm_status(device)
        res["frac_sustained"] = res["tflops"] / sustained
        res["vs_cublas_dense"] = res["tflops"] / res["cublas_dense_tflops"]
        out[str(m)] = res
        del xs
    return out


def decode_section(device, batches=(1, 8), prompt: int = 512, new_tokens: int = 256, cfg=None, rank=0, world=1,
                   gemv_block_ms=None, peer=True, fuse_prologue=True, random_perm=False) -> dict:
    """Whole-model greedy decoding (BASELINE configs[3]): random-init Qwen3-4B-shaped stack, all
    linears mixed-precision, `prompt`-token prefill through the GEMM, then `new_tokens` tokens, one
    CUDA-graph replay per token.  tokens/s = batch * new_tokens / device time of the decode loop."""
    import torch
    import torch.distributed as dist

    from rdquant_b200.decoder import QWEN3_4B, MixedDecoder

    if isinstance(cfg, str):
        from rdquant_b200.decoder import LLAMA3_70B

        cfg = {"qwen3-4b": QWEN3_4B, "llama3-70b": LLAMA3_70B}[cfg]
    cfg = cfg or QWEN3_4B
    out = {"model": cfg.name, "layers": cfg.layers, "prompt_tokens": prompt, "new_tokens": new_tokens, "batch": {},
           "channel_order": "all channels shuffled" if random_perm else
           "random assignment of channels to formats, grouped by format, original order inside a group (as the "
           "reference's allocator produces, rdquant/core/allocator.py:210-224)"}
    if world > 1:
        out["parallelism"] = f"column-parallel x{world}, " + ("all-gather fused into the GEMV epilogue (peer stores)"
                                                               if peer else "NCCL all-gather per linear")
    t_build = time.time()
    model = MixedDecoder(cfg, device, max_seq=prompt + new_tokens + 8, batch=batches[0], seed=7, rank=rank, world=world,
                         peer_gather=peer, fuse_prologue=fuse_prologue, random_perm=random_perm)
    torch.cuda.synchronize()
    t_build = time.time() - t_build
    for b in batches:
        model.reset(b)
        gen = torch.Generator().manual_seed(11)
        ids = torch.randint(0, cfg.vocab, (b, prompt), generator=gen).to(device)
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        model.prefill(ids)  # untimed pass of the same shape: library set-up, kernel selection, allocator growth
        model.reset(b)
        if world > 1:
            dist.barrier()
        e0.record()
        model.prefill(ids)
        e1.record()
        e1.synchronize()
        model.capture_decode()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e1.record()
        for _ in range(new_tokens):
            model.decode_step()
        e2.record()
        e2.synchronize()
        ms_prefill, ms_decode = e0.elapsed_time(e1), e1.elapsed_time(e2)
        if world > 1:
            t = torch.tensor([ms_decode], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_decode = float(t[0])
        res = {"tokens_per_s": b * new_tokens / (ms_decode * 1e-3), "ms_per_token": ms_decode / new_tokens,
               "prefill_ms": ms_prefill, "linear_bytes": model.linear_bytes, "build_s": round(t_build, 1),
               "linear_gbps": model.linear_bytes * new_tokens / (ms_decode * 1e-3) / 1e9}
        if gemv_block_ms is not None and b == 1 and world == 1:
            # share of a token's time the linears alone would take at the block benchmark's rate
            res["linear_only_fraction"] = gemv_block_ms * cfg.layers / res["ms_per_token"]
        out["batch"][str(b)] = res
        model.release_graph()
    del model
    torch.cuda.empty_cache()
    return out


def _note(rank: int, msg: str) -> None:
    print(f"[bench rank {rank} {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


def run_sharded(args, device, rank: int, world: int) -> None:
    """N > 1: one block, column-parallel; kernel + all-gather + un-permute per layer in the graph."""
    import torch
    import torch.distributed as dist

    from rdquant_b200 import rdquant_cuda
    from rdquant_b200.parallel import ColumnParallelMixedLinear, PeerArena, PeerGatherMixedLinear, gather_outputs

    steps, warmup, m = max(args.steps, 1), max(args.warmup, 3), args.m
    peer = args.collective == "peer"
    per_layer = block_layers(device, seed=0)  # the same block on every rank
    units = fused_units(per_layer, fuse=not args.no_fuse)
    step_bytes = sum(u["bytes"] for u in units)
    # every rank streams 1/world of the block per step: rotate enough copies to exceed 2 x L2
    copies = max(args.copies, int(2 * L2_BYTES * world / step_bytes) + 1)
    if peer:
        widest = max(u["n"] for u in units)
        arena = PeerArena(copies * len(units) * ((widest // world + 256) * world * 16 * 2 + 1024), device)
        mods = [[PeerGatherMixedLinear({kk: v.clone() for kk, v in u["data"].items()}, u["splits"], u["k"], arena)
                 for u in units] for _ in range(copies)]
    else:
        mods = [[ColumnParallelMixedLinear({kk: v.clone() for kk, v in u["data"].items()}, u["splits"], u["k"], device,
                                           rank, world) for u in units] for _ in range(copies)]
    for row in mods:
        for mod in row:
            mod.use_pdl = not args.no_pdl
    gen = torch.Generator().manual_seed(1234)
    xs_cpu = [torch.randn(m, u["k"], generator=gen).half() for u in units]
    xs = [x.to(device) for x in xs_cpu]
    ys = [None] * len(units)

    def one_step(i: int) -> None:
        for li, mod in enumerate(mods[i % copies]):
            ys[li] = mod(xs[li])

    def gathers_only(i: int) -> None:
        if peer:
            return
        for mod in mods[i % copies]:
            send, buf, idx = mod._io_buffers(m)
            gather_outputs(send, mod.plan, mod.group, buffer=buf, index=idx)

    sampler = ClockSampler(device.index or 0)
    sampler.start()
    _note(rank, "modules built")
    # every weight copy runs once before anything is captured: the first call of a module
    # allocates its buffers and copies its index table to the device
    for i in range(max(warmup, copies)):
        one_step(i)
    torch.cuda.synchronize()
    _note(rank, "warm-up done")
    # parity: the gathered outputs of one step against the CPU oracle on the whole layers
    from oracle import oracle_np as onp

    one_step(0)
    torch.cuda.synchronize()
    parity = 0.0
    if rank == 0:
        for li, u in enumerate(units):
            ref = oracle_outputs(per_layer, u, xs_cpu[li].numpy())
            parity = max(parity, float(onp.rel_err(ys[li].cpu().float().numpy(), ref)))
    # every rank must hold the same gathered outputs as rank 0
    for li in range(len(units)):
        mine = ys[li].float().sum(dtype=torch.float64).reshape(1)
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if float(hi - lo) != 0.0:
            raise RuntimeError("ranks disagree on the gathered output of layer %d" % li)
    def check_all() -> None:
        for row in mods:
            for mod in row:
                if peer:
                    mod.check_status()
                else:
                    rdquant_cuda.check_status(mod.fd)

    check_all()
    _note(rank, "parity checked")
    stream = torch.cuda.Stream(device)
    graph, ggraph = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    replays = 10
    with torch.cuda.stream(stream):
        one_step(0)
        gathers_only(0)
        stream.synchronize()
        _note(rank, "capturing")
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for i in range(steps):
                one_step(i)
        if not peer:
            with torch.cuda.graph(ggraph, stream=stream, capture_error_mode="thread_local"):
                for i in range(steps):
                    gathers_only(i)
        _note(rank, "captured")
        for _ in range(20):  # a fixed count: every rank must issue the same collectives
            graph.replay()
        stream.synchronize()
        _note(rank, "graph warm")
        dist.barrier()
        torch.cuda.synchronize()
        t0 = time.time()
        times = time_replays(graph, stream, replays)
        t1 = time.time()
        dist.barrier()
        gtimes = time_replays(ggraph, stream, 5) if not peer else [0.0]
    clocks = sampler.stop(t0, t1)
    check_all()
    _note(rank, "timed")

    # ---- end to end: host activations in, host results out, synchronised every step
    x_host = [x.clone().pin_memory() for x in xs_cpu]
    y_host = [torch.zeros(m, u["n"], dtype=torch.float16).pin_memory() for u in units]
    e2e_steps = min(steps, 200)

    def e2e_step(i: int) -> None:
        for li, mod in enumerate(mods[i % copies]):
            xs[li].copy_(x_host[li], non_blocking=True)
            y_host[li].copy_(mod(xs[li]), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    dist.barrier()
    te0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    te = time.perf_counter() - te0

    _note(rank, "e2e done")
    t = torch.tensor([statistics.median(times), min(times), max(times), statistics.median(gtimes), te],
                     dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_min, ms_max, gms, te = (float(v) for v in t)
    pt = torch.tensor([parity], dtype=torch.float64, device=device)
    dist.all_reduce(pt, op=dist.ReduceOp.MAX)
    parity = float(pt[0])
    if parity > TOL:
        raise RuntimeError(f"sharded outputs differ from the oracle: max rel err {parity:.3e} > {TOL}")

    peaks, peak_kind = measured_peaks()
    launches = steps * len(units)
    value = step_bytes * steps / (ms * 1e-3) / 1e9
    per_rank_launch_bytes = step_bytes / world / len(units)
    achieved = per_rank_launch_bytes / (ms * 1e-3 / launches) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {
            "workload": f"qwen3-4b decoder block: q,k,v,o,gate,up,down mixed-precision linears, M={m} decode GEMV",
            "launches_per_step": len(units),
            "fusion": "none" if args.no_fuse else "q/k/v and gate/up packed as one layer each (they read the same input)",
            "split": "67/32/1 NVFP4/FP8/FP16, 128-aligned, random channel permutation",
            "bytes_per_step": step_bytes,
            "parallelism": f"column-parallel x{world}: every format group of every layer cut at 128-channel "
                           "boundaries, x replicated, outputs all-gathered and un-permuted on every rank",
            "collective": (f"fused into the GEMV epilogue: each rank stores its slice into every GPU's gather buffer "
                           f"over NVLink (peer memory), flag + bounded wait + un-permute kernel; x{len(units)} per step, "
                           "inside the timed CUDA graph, no NCCL call") if peer else
                          f"all_gather_into_tensor x{len(units)} per step (NCCL, inside the timed CUDA graph)",
            "l2_policy": f"{copies} rotating weight copies = {copies * step_bytes / world / 1e6:.0f} MB per rank "
                         "> 2 x L2; no flush",
            "launch": "one CUDA graph of all timed steps; median of %d replays" % replays,
            "kernel": "tiled",
        },
        "gpu_launches": launches,
        "timing": {"replays": replays, "ms_per_step_median": ms / steps, "ms_per_step_min": ms_min / steps,
                   "ms_per_step_max": ms_max / steps},
        "collective_ms_per_step": None if peer else gms / steps,
        "parity_max_rel_err": parity,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_source": peak_kind,
                     "kernel": "gemv_tiled_kernel", "bytes_per_launch": per_rank_launch_bytes,
                     "note": "per rank: its share of a launch's bytes over the step time divided by launches; "
                             "the step time includes the all-gathers"},
        "e2e": {"value": step_bytes * e2e_steps / te / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": sum(2 * m * u["k"] for u in units),
                "d2h_bytes_per_step": sum(2 * m * u["n"] for u in units), "steps": e2e_steps,
                "ms_per_step": 1e3 * te / e2e_steps,
                "api": "parallel.%s.forward per layer: pinned host x -> device, fused GEMV + "
                       "all-gather + un-permute, y -> pinned host, synchronised every step"
                       % ("PeerGatherMixedLinear" if peer else "ColumnParallelMixedLinear")},
        "clocks": clocks,
        "cpu_baseline": None,
    }
    del graph, ggraph  # graphs that captured collectives must go before the process group does
    if args.decode:
        line["decode"] = decode_section(device, batches=(1,), prompt=args.decode_prompt, new_tokens=args.decode_tokens,
                                        cfg=args.decode_model, rank=rank, world=world, peer=peer)
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
    ap.add_argument("--prologue", choices=["all", "norm", "act", "none"], default="all",
                    help="whole-model decode: which of add+RMSNorm / SiLU x mul run inside the consuming GEMV")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM section")
    ap.add_argument("--prefill-tokens", default="512,2048,8192", help="token counts of the prefill GEMM section")
    ap.add_argument("--no-decode", dest="decode", action="store_false", help="skip whole-model decoding")
    ap.add_argument("--decode-batches", default="1,8", help="batch sizes of the whole-model decode section")
    ap.add_argument("--decode-perm", choices=["grouped", "random"], default="grouped",
                    help="channel order of the decode section's layers: grouped by format like the reference's "
                         "allocator output, or fully shuffled (worst case for the output stores)")
    ap.add_argument("--decode-model", choices=["qwen3-4b", "llama3-70b"], default="qwen3-4b",
                    help="shape of the whole-model decode section (BASELINE configs 4 / 5)")
    ap.add_argument("--decode-prompt", type=int, default=512, help="prompt tokens of the decode section")
    ap.add_argument("--decode-tokens", type=int, default=256, help="generated tokens of the decode section")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: all-gather fused into the GEMV epilogue over peer memory, or NCCL")
    ap.set_defaults(decode=True)
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
        import datetime
        import faulthandler

        # a rank that stops answering must end the run with a message, not hang it
        faulthandler.dump_traceback_later(240, exit=True)
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
        run_sharded(args, device, rank, world)
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        # Tearing the NCCL communicator down after its collectives were captured in CUDA graphs was
        # seen to block (torch 2.11, NCCL 2.28): every rank has printed and synchronised, leave.
        os._exit(0)

    steps, warmup, m = max(args.steps, 1), max(args.warmup, 3), args.m
    copies = max(args.copies, 2)
    layers, per_layer = build_block(device, seed=rank, copies=copies, fuse=not args.no_fuse)
    step_bytes = sum(l["bytes"] for l in layers)
    flags = {"tiled": _lib.RDQ_GEMV_AUTO, "generic": _lib.RDQ_GEMV_GENERIC}[args.kernel]
    if not args.no_pdl:
        flags |= _lib.RDQ_GEMV_PDL

    gen = torch.Generator().manual_seed(1234 + rank)
    xs_cpu = [torch.randn(m, l["k"], generator=gen).half() for l in layers]
    xs = [x.to(device) for x in xs_cpu]
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
    for l in layers:
        for fd in l["fds"]:
            rdquant_cuda.check_status(fd)
    stream = torch.cuda.Stream(device)
    graph = torch.cuda.CUDAGraph()
    replays = 10
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
        torch.cuda.synchronize()
        t0 = time.time()
        times = time_replays(graph, stream, replays)
        torch.cuda.synchronize()
        t1 = time.time()
    ms = statistics.median(times)
    clocks = sampler.stop(t0, t1)
    for l in layers:
        for fd in l["fds"]:
            rdquant_cuda.check_status(fd)

    # ---- parity of what was timed: the outputs of the last timed step against the CPU oracle
    from oracle import oracle_np as onp

    refs = [oracle_outputs(per_layer, l, xs_cpu[li].numpy()) for li, l in enumerate(layers)]
    parity = max(float(onp.rel_err(ys[li].cpu().float().numpy(), refs[li])) for li in range(len(layers)))
    if parity > TOL:
        raise RuntimeError(f"timed outputs differ from the oracle: max rel err {parity:.3e} > {TOL}")

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
        for xh, x in zip(runner.x_host, xs_cpu):
            xh.copy_(x)
    e2e_steps = min(steps, 200)
    for i in range(copies):
        runners[i].run()
    te0 = time.perf_counter()
    for i in range(e2e_steps):
        # host activations in, host results out: one graph replay (H2D copies, GEMVs, D2H copies)
        y_host = runners[i % copies].run()
    te = time.perf_counter() - te0
    e2e_parity = max(float(onp.rel_err(y_host[li].float().numpy(), refs[li])) for li in range(len(layers)))
    if e2e_parity > TOL:
        raise RuntimeError(f"end-to-end outputs differ from the oracle: max rel err {e2e_parity:.3e} > {TOL}")
    del runners

    value = step_bytes * steps / (ms * 1e-3) / 1e9
    e2e_value = step_bytes * e2e_steps / te / 1e9
    peaks, peak_kind = measured_peaks()
    launches = steps * len(layers)
    per_launch_bytes = step_bytes / len(layers)
    achieved = per_launch_bytes / (ms * 1e-3 / launches) / 1e9
    workload = f"block_m{m}" + ("" if not args.no_fuse else "_nofuse")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16xf16->f32", "data": "synthetic",
        "config": {
            "workload": f"qwen3-4b decoder block: q,k,v,o,gate,up,down mixed-precision linears, M={m} decode GEMV",
            "launches_per_step": len(layers),
            "fusion": "none" if args.no_fuse else "q/k/v and gate/up packed as one layer each (they read the same input)",
            "split": "67/32/1 NVFP4/FP8/FP16, 128-aligned, random channel permutation",
            "bytes_per_step": step_bytes, "l2_policy": f"{copies} rotating weight copies = "
            f"{copies * step_bytes / 1e6:.0f} MB > 2 x L2; inputs larger than L2, no flush",
            "launch": ("one CUDA graph of all timed steps, PDL-chained launches" if not args.no_pdl else "CUDA graph")
                      + "; median of %d replays" % replays,
            "parallelism": "single GPU",
            "kernel": args.kernel,
        },
        "gpu_launches": launches,
        "timing": {"replays": replays, "ms_per_step_median": ms / steps, "ms_per_step_min": min(times) / steps,
                   "ms_per_step_max": max(times) / steps},
        "parity_max_rel_err": max(parity, e2e_parity),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"],
                     "traffic": profiled_traffic("gemv_%s_kernel" % args.kernel, workload), "peak_source": peak_kind,
                     "frac_of_nominal_8tbs": achieved / 8000.0, "kernel": "gemv_%s_kernel" % args.kernel,
                     "bytes_per_launch": per_launch_bytes},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": sum(2 * m * l["k"] for l in layers),
                "d2h_bytes_per_step": sum(2 * m * l["n"] for l in layers), "steps": e2e_steps,
                "ms_per_step": 1e3 * te / e2e_steps,
                "api": "inference.GraphedDecodeStep.run(): pinned host x -> device (staging kernel reading the pinned "
                       "buffer), fused GEMVs, y -> pinned host (staging kernel) as one CUDA-graph replay; every step the "
                       "host waits for the completion word the last kernel writes to pinned memory behind its data; "
                       "weight copies rotate as in the device-only measurement"},
        "clocks": clocks,
    }
    if not args.no_prefill and m == 1:
        line["prefill"] = prefill_section(device, layers, tokens=tuple(int(t) for t in args.prefill_tokens.split(",") if t))
    for l in layers:
        l["fds"] = l["fds"][:1]
    torch.cuda.empty_cache()
    if args.decode and m == 1:
        batches = tuple(int(b) for b in args.decode_batches.split(",") if b)
        line["decode"] = decode_section(device, batches=batches, prompt=args.decode_prompt, new_tokens=args.decode_tokens,
                                        cfg=args.decode_model,
                                        gemv_block_ms=ms / steps if args.decode_model == "qwen3-4b" else None,
                                        random_perm=args.decode_perm == "random",
                                        fuse_prologue={"all": True, "none": False}.get(args.prologue, args.prologue))
        line["config"]["decode_tokens_per_s"] = line["decode"]["batch"][str(batches[0])]["tokens_per_s"]
    if not args.no_cpu_baseline:
        base = cpu_baseline()
        line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
    else:
        line["cpu_baseline"] = None
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
