"""Prefill GEMM (tcgen05) through the C ABI against the oracle: golden layers, random byte
patterns, the benchmark block shapes, ragged M, bias."""
import numpy as np
import pytest
import torch

from conftest import ORDER, golden_layer_torch
from oracle import oracle_np as onp
from rdquant_b200 import rdquant_cuda
from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv
from rdquant_b200.synthetic import QWEN3_4B_BLOCK, fixed_splits, random_packed_layer

pytestmark = pytest.mark.gpu
TOL = 2e-3  # max |y - y_ref| / max |y_ref|, FP32-accumulation reference


def _run(layer, splits, k, m, bias=False, seed=0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=gen).half()
    n = sum(splits.values())
    b = (torch.randn(n, generator=gen) * 0.5).half() if bias else None
    fd = pack_for_fused_gemv(layer, splits, k, "cuda", tiled=False)
    y = rdquant_cuda.mixed_gemm(x.cuda(), fd, b.cuda() if bias else None)
    torch.cuda.synchronize()
    y_ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), splits, k,
                                       b.float().numpy() if bias else None)
    return y.cpu().float().numpy(), y_ref


def test_golden_layers(layers):
    for name, case in layers.items():
        layer, splits, k = golden_layer_torch(case)
        if k % 64:
            with pytest.raises(RuntimeError):
                _run(layer, splits, k, 32)
            continue
        for m in (1, 17, 130):
            y, y_ref = _run(layer, splits, k, m, bias="bias" in layer, seed=m)
            assert onp.rel_err(y, y_ref) < TOL, (name, m)


@pytest.mark.parametrize("m", [16, 100, 128, 300])
@pytest.mark.parametrize("shape", [(128, 128, 128, 256), (64, 32, 16, 512), (256, 0, 0, 1024), (0, 48, 0, 256),
                                   (0, 0, 32, 768), (49, 46, 1, 64), (1664, 768, 128, 4096)])
def test_random_bytes(shape, m):
    n4, n8, n16, k = shape
    layer = random_packed_layer(n4, n8, n16, k, seed=k + m)
    splits = dict(zip(ORDER, (n4, n8, n16)))
    y, y_ref = _run(layer, splits, k, m, bias=(m % 2 == 0), seed=m)
    assert onp.rel_err(y, y_ref) < TOL


@pytest.mark.parametrize("name", list(QWEN3_4B_BLOCK))
def test_block_shapes_m512(name):
    k, n = QWEN3_4B_BLOCK[name]
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=len(name))
    y, y_ref = _run(layer, splits, k, 512, bias=True, seed=3)
    assert onp.rel_err(y, y_ref) < TOL, name


def test_matches_dequantised_weight_matmul():
    # size-independent property: GEMM == x @ dequant(W)^T with the bit-exact dequantisation kernel
    k, n = 2560, 4096
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=9)
    fd = pack_for_fused_gemv(layer, splits, k, "cuda", tiled=False)
    dev = {kk: v.cuda() for kk, v in layer.items()}
    w = rdquant_cuda.dequantize_packed(dev, splits, k, inv_perm=dev["inv_permutation"])
    x = torch.randn(2048, k, device="cuda").half()
    y = rdquant_cuda.mixed_gemm(x, fd)
    ref = x.float() @ w.float().T
    err = (y.float() - ref).abs().max() / ref.abs().max()
    assert float(err) < TOL


@pytest.mark.parametrize("m,n,k", [(1024, 9728, 256), (1000, 9800, 192), (4096, 2560, 320)])
def test_large_tiles(m, n, k):
    """Enough tiles to select the 256-token x 256-channel configuration (all tensor-memory
    columns, three 64 KB stages), with ragged M and N, against the oracle and against
    x @ dequant(W)^T."""
    n16 = 128
    n8 = (n // 3) // 128 * 128
    n4 = n - n8 - n16
    layer = random_packed_layer(n4, n8, n16, k, seed=m + k)
    splits = dict(zip(ORDER, (n4, n8, n16)))
    y, y_ref = _run(layer, splits, k, m, bias=True, seed=5)
    assert onp.rel_err(y, y_ref) < TOL


@pytest.mark.parametrize("m", [512, 2048, 8192])
@pytest.mark.parametrize("group", [["q_proj", "k_proj", "v_proj"], ["o_proj"], ["gate_proj", "up_proj"], ["down_proj"]])
def test_benchmark_launches(group, m):
    """The four launches the prefill benchmark times -- q+k+v (2560 -> 6144) and gate+up
    (2560 -> 19456) packed as one layer each by fuse_layers, o and down as they are -- at its three
    token counts.  Every member layer is compared with the oracle on a seeded sample of 64 rows
    (the CPU side stays in seconds at M = 8192), and the whole output with x @ dequant(W)^T, the
    weight coming from the bit-exact dequantisation kernel."""
    from rdquant_b200.fused_gemv_pack import fuse_layers

    members = []
    for i, name in enumerate(group):
        k, n = QWEN3_4B_BLOCK[name]
        splits = fixed_splits(n)
        members.append((random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=51 + i), splits))
    k = QWEN3_4B_BLOCK[group[0]][0]
    data, splits = fuse_layers(members) if len(members) > 1 else members[0]
    fd = pack_for_fused_gemv(data, splits, k, "cuda", tiled=False)
    gen = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=gen).half().cuda()
    y = rdquant_cuda.mixed_gemm(x, fd)
    rdquant_cuda.check_gemm_status(x.device)
    rows = torch.randperm(m, generator=gen)[:64].sort().values
    xs, ys = x[rows.cuda()].cpu().numpy(), y[rows.cuda()].cpu().float().numpy()
    off = 0
    for layer, sp in members:
        n = sum(sp.values())
        y_ref = onp.mixed_precision_linear(xs, onp.torch_layer_to_np(layer), sp, k)
        assert onp.rel_err(ys[:, off:off + n], y_ref) < TOL, (group, m, off)
        off += n
    assert off == y.shape[1]
    dev = {kk: v.cuda() for kk, v in data.items()}
    w = rdquant_cuda.dequantize_packed(dev, splits, k, inv_perm=dev["inv_permutation"])
    worst = 0.0
    for r0 in range(0, m, 2048):  # in panels: the FP32 product of the full problem would take gigabytes
        ref = x[r0:r0 + 2048].float() @ w.float().T
        worst = max(worst, float((y[r0:r0 + 2048].float() - ref).abs().max() / ref.abs().max()))
    assert worst < TOL
