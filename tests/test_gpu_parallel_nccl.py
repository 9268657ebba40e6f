"""Column-parallel mixed-precision linear on two GPUs over NCCL: each rank runs the CUDA kernels
on its row ranges, one all-gather restores the full output in original channel order.
Skipped on boxes with fewer than two GPUs (the host logic is covered on gloo ranks)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    from conftest import ORDER
    from oracle import oracle_np as onp
    from rdquant_b200.parallel import ColumnParallelMixedLinear
    from rdquant_b200.synthetic import fixed_splits, random_packed_layer

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        k, n = 2560, 4096
        splits = fixed_splits(n)
        layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=21)
        gen = torch.Generator().manual_seed(3)
        layer["bias"] = (torch.randn(n, generator=gen) * 0.5).half()
        mod = ColumnParallelMixedLinear(layer, splits, k, torch.device("cuda", rank), rank, world)
        errs = []
        for m in (1, 7, 300):
            x = torch.randn(m, k, generator=gen).half()
            with torch.no_grad():
                y = mod(x.cuda())
            torch.cuda.synchronize()
            ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), dict(zip(ORDER, (splits[o] for o in ORDER))),
                                             k, layer["bias"].float().numpy())
            errs.append(float(onp.rel_err(y.cpu().float().numpy(), ref)))
        q.put((rank, errs, list(mod.plan.n_local)))
    finally:
        dist.destroy_process_group()


def _peer_worker(rank, world, port, q):
    """All-gather fused into the GEMV epilogue (stores into the peers' gather buffers): parity, and
    the bounded wait when a rank does not deliver -- provoked on the host: rank 1 simply skips one
    step (between steps, nothing of it in flight), rank 0's wait runs out and reports it."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    from conftest import ORDER
    from oracle import oracle_np as onp
    from rdquant_b200.parallel import PeerArena, PeerGatherMixedLinear
    from rdquant_b200.synthetic import fixed_splits, random_packed_layer

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    k, n = 2560, 4096
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=22)
    gen = torch.Generator().manual_seed(4)
    layer["bias"] = (torch.randn(n, generator=gen) * 0.5).half()
    arena = PeerArena(8 << 20, torch.device("cuda", rank))
    mod = PeerGatherMixedLinear(layer, splits, k, arena, wait_ms=300)
    full = dict(zip(ORDER, (splits[o] for o in ORDER)))
    errs = []
    for m in (1, 7, 16, 1, 40):  # 40 rows: GEMM + NCCL all-gather
        x = torch.randn(m, k, generator=gen).half()
        with torch.no_grad():
            y = mod(x.cuda())
        mod.check_status()
        ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), full, k, layer["bias"].float().numpy())
        errs.append(float(onp.rel_err(y.cpu().float().numpy(), ref)))
    # ---- a rank that does not deliver: rank 1 skips this step
    timed_out = None
    x = torch.randn(1, k, generator=gen).half().cuda()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        with torch.no_grad():
            mod(x)
        try:
            mod.check_status()
            timed_out = False
        except RuntimeError as exc:
            timed_out = "rank 1 did not deliver" in str(exc)
    mod.reset_peer_state()
    with torch.no_grad():
        y = mod(x)
    mod.check_status()
    ref = onp.mixed_precision_linear(x.cpu().numpy(), onp.torch_layer_to_np(layer), full, k, layer["bias"].float().numpy())
    errs.append(float(onp.rel_err(y.cpu().float().numpy(), ref)))
    q.put((rank, errs, timed_out))
    q.close()
    q.join_thread()  # the result is on its way before the process leaves
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)  # no communicator teardown: see bench.py


def _run_two(worker):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    import queue
    import time
    deadline = time.time() + 240
    while len(results) < len(procs) and time.time() < deadline:
        try:
            results.append(q.get(timeout=2))
        except queue.Empty:
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    for p in procs:
        p.join(timeout=5 if len(results) < len(procs) else 60)
        if p.is_alive():
            p.terminate()
    assert len(results) == len(procs), "a rank ended without a result"
    assert all(p.exitcode == 0 for p in procs)
    return results


def test_two_gpus_peer_gather_and_bounded_wait():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for rank, errs, timed_out in _run_two(_peer_worker):
        assert max(errs) < TOL, (rank, errs)
        assert timed_out is (True if rank == 0 else None), (rank, timed_out)


def test_two_gpus_match_full_layer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = []
    import queue
    import time
    deadline = time.time() + 240
    while len(results) < len(procs) and time.time() < deadline:
        try:
            results.append(q.get(timeout=2))
        except queue.Empty:
            # a rank that died will never report: stop waiting (and end its peer) at once
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    for p in procs:
        p.join(timeout=5 if len(results) < len(procs) else 60)
        if p.is_alive():
            p.terminate()
    assert len(results) == len(procs), "a rank ended without a result"
    assert all(p.exitcode == 0 for p in procs)
    for rank, errs, n_local in results:
        assert max(errs) < TOL, (rank, errs)
        assert sum(n_local) == 4096
