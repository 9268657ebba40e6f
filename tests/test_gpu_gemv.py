"""Decode GEMV (M <= 16) through the C ABI against the oracle: golden layers, random byte
patterns, the benchmark shapes, both kernels, bias, determinism."""
import numpy as np
import pytest
import torch

from conftest import ORDER, golden_layer_torch
from oracle import oracle_np as onp
from rdquant_b200 import _lib, rdquant_cuda
from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv
from rdquant_b200.synthetic import QWEN3_4B_BLOCK, fixed_splits, random_packed_layer

pytestmark = pytest.mark.gpu
TOL = 2e-3  # max |y - y_ref| / max |y_ref|, FP32-accumulation reference


def _run(layer, splits, k, m, flags, bias=False, seed=0):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=gen).half()
    n = sum(splits.values())
    b = (torch.randn(n, generator=gen) * 0.5).half() if bias else None
    fd = pack_for_fused_gemv(layer, splits, k, "cuda")
    y = rdquant_cuda.mixed_gemv(x.cuda(), fd, b.cuda() if bias else None, flags)
    torch.cuda.synchronize()
    y_ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), splits, k,
                                       b.float().numpy() if bias else None)
    cnt = fd["tile_counters"].cpu()
    assert int(cnt.abs().sum()) == 0, "tile counters / status word not back to zero"
    return y.cpu().float().numpy(), y_ref, fd


@pytest.mark.parametrize("flags", [_lib.RDQ_GEMV_GENERIC, _lib.RDQ_GEMV_AUTO])
def test_golden_layers(layers, flags):
    for name, case in layers.items():
        layer, splits, k = golden_layer_torch(case)
        for m in (1, 3):
            y, y_ref, _ = _run(layer, splits, k, m, flags, bias="bias" in layer)
            assert onp.rel_err(y, y_ref) < TOL, (name, m)


@pytest.mark.parametrize("m", [1, 2, 4, 8, 9, 16])
@pytest.mark.parametrize("shape", [(128, 128, 128, 256), (64, 32, 16, 512), (256, 0, 0, 1024), (0, 48, 0, 256),
                                   (0, 0, 32, 768), (1664, 768, 128, 4096), (48, 32, 16, 1216), (16, 16, 16, 4160),
                                   (64, 0, 0, 256), (0, 64, 0, 512), (0, 0, 64, 256), (192, 64, 64, 768),
                                   (64, 64, 64, 9728)])
@pytest.mark.parametrize("flags", [_lib.RDQ_GEMV_GENERIC, _lib.RDQ_GEMV_AUTO])
def test_random_bytes(shape, m, flags):
    n4, n8, n16, k = shape
    layer = random_packed_layer(n4, n8, n16, k, seed=k + m)
    splits = dict(zip(ORDER, (n4, n8, n16)))
    y, y_ref, _ = _run(layer, splits, k, m, flags, bias=(m % 2 == 0), seed=m)
    assert onp.rel_err(y, y_ref) < TOL


@pytest.mark.parametrize("m", [1, 5, 16])
def test_many_tiles_per_cta(m):
    """Short rows, many channels: every warp group finishes several whole tiles and its ring
    wraps."""
    n4, n8, n16, k = 60800, 20480, 5120, 256
    layer = random_packed_layer(n4, n8, n16, k, seed=11)
    splits = dict(zip(ORDER, (n4, n8, n16)))
    y, y_ref, _ = _run(layer, splits, k, m, _lib.RDQ_GEMV_AUTO, bias=True, seed=m)
    assert onp.rel_err(y, y_ref) < TOL


def test_ragged_shapes_take_generic_kernel():
    for n4, n8, n16, k in [(49, 46, 1, 64), (0, 33, 7, 40), (5, 0, 0, 16)]:
        layer = random_packed_layer(n4, n8, n16, k, seed=7)
        splits = dict(zip(ORDER, (n4, n8, n16)))
        y, y_ref, _ = _run(layer, splits, k, 3, _lib.RDQ_GEMV_AUTO)
        assert onp.rel_err(y, y_ref) < TOL


def test_tiled_layout_predicate():
    """Which shapes get the tiled layout (groups in multiples of 16 rows, K divisible into chunks
    that are multiples of 64, at most 256 chunks per tile); everything else -- here K = 4288 =
    64 x 67, whose FP16 tiles would have 268 chunks -- runs the any-shape kernel and must still
    match the oracle."""
    lib = _lib.lib()
    assert lib.rdq_gemv_tiled_bytes(128, 64, 64, 512) > 0
    assert lib.rdq_gemv_tiled_bytes(16, 16, 0, 4288) > 0      # 67 / 134 chunks per tile: fine
    for shape in [(16, 16, 16, 4288), (0, 0, 16, 4288), (10, 0, 0, 256), (16, 0, 0, 100)]:
        assert lib.rdq_gemv_tiled_bytes(*shape) == 0
    n4, n8, n16, k = 16, 16, 16, 4288
    layer = random_packed_layer(n4, n8, n16, k, seed=9)
    splits = dict(zip(ORDER, (n4, n8, n16)))
    y, y_ref, fd = _run(layer, splits, k, 2, _lib.RDQ_GEMV_AUTO)
    assert fd["w_tiled"] is None
    assert onp.rel_err(y, y_ref) < TOL


@pytest.mark.parametrize("name", list(QWEN3_4B_BLOCK))
@pytest.mark.parametrize("m", [1, 4, 16])
def test_block_shapes_random_perm(name, m):
    k, n = QWEN3_4B_BLOCK[name]
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=len(name) + m)
    y, y_ref, fd = _run(layer, splits, k, m, _lib.RDQ_GEMV_AUTO | _lib.RDQ_GEMV_PDL, bias=True, seed=m)
    assert fd["w_tiled"] is not None
    assert onp.rel_err(y, y_ref) < TOL, (name, m)
    # determinism: same bits on a second launch
    gen = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=gen).half().cuda()
    y1 = rdquant_cuda.mixed_gemv(x, fd)
    y2 = rdquant_cuda.mixed_gemv(x, fd)
    assert torch.equal(y1, y2)
    # linearity in x (size-independent property): f(2x) == 2 f(x) exactly in float16 unless overflow
    y3 = rdquant_cuda.mixed_gemv((x * 2).contiguous(), fd)
    assert torch.allclose(y3.float(), 2 * y1.float(), rtol=2e-3, atol=1e-3)


def test_reference_signature_entry_point():
    n4, n8, k = 128, 64, 256
    layer = random_packed_layer(n4, n8, 0, k, seed=3)
    dev = {kk: v.cuda() for kk, v in layer.items()}
    x = torch.randn(1, k).half()
    y = rdquant_cuda.fused_mixed_gemv(x.cuda(), dev["weight_nvfp4"], dev["weight_nvfp4_scale"], 1.0, dev["weight_fp8"],
                                      dev["weight_fp8_scale"], dev["inv_permutation"], n4, n8, k)
    y_ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), {"NVFP4": n4, "FP8": n8, "FP16": 0}, k)
    assert y.shape == (1, n4 + n8) and onp.rel_err(y.cpu().float().numpy(), y_ref) < TOL
    with pytest.raises(RuntimeError):
        rdquant_cuda.fused_mixed_gemv(x.cuda().float(), dev["weight_nvfp4"], dev["weight_nvfp4_scale"], 1.0,
                                      dev["weight_fp8"], dev["weight_fp8_scale"], dev["inv_permutation"], n4, n8, k)


@pytest.mark.parametrize("m", [1, 4, 8, 16])
@pytest.mark.parametrize("group", [["q_proj", "k_proj", "v_proj"], ["gate_proj", "up_proj"]])
def test_fused_sibling_projections(group, m):
    """The layers the benchmark times: q+k+v (2560 -> 6144) and gate+up (2560 -> 19456) packed as
    one layer each by fuse_layers, PDL launch flag on, against the oracle on every member layer."""
    from rdquant_b200.fused_gemv_pack import fuse_layers

    members = []
    for i, name in enumerate(group):
        k, n = QWEN3_4B_BLOCK[name]
        splits = fixed_splits(n)
        members.append((random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=31 + i + m), splits))
    k = QWEN3_4B_BLOCK[group[0]][0]
    data, splits = fuse_layers(members)
    fd = pack_for_fused_gemv(data, splits, k, "cuda")
    assert fd["w_tiled"] is not None
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(m)).half()
    y = rdquant_cuda.mixed_gemv(x.cuda(), fd, None, _lib.RDQ_GEMV_PDL)
    rdquant_cuda.check_status(fd)
    y = y.cpu().float().numpy()
    off = 0
    for layer, sp in members:
        n = sum(sp.values())
        y_ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), sp, k)
        assert onp.rel_err(y[:, off:off + n], y_ref) < TOL, (group, m, off)
        off += n
    assert off == y.shape[1]


@pytest.mark.parametrize("k,n,m", [(2560, 6144, 1), (2560, 6144, 8), (2560, 19456, 3), (256, 768, 2), (4096, 2560, 4)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_prologue_add_rmsnorm(k, n, m, with_delta):
    """rmsnorm(x + delta) computed inside the GEMV: same result as the separate glue kernel
    followed by the plain GEMV, and the updated residual stream is written out of place."""
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=k + n + m)
    fd = pack_for_fused_gemv(layer, splits, k, "cuda")
    assert fd["w_tiled"] is not None and rdquant_cuda.gemv_stages_x(m, k)
    g = torch.Generator().manual_seed(m + k)
    x = torch.randn(m, k, generator=g).half().cuda()
    d = torch.randn(m, k, generator=g).half().cuda() if with_delta else None
    w = (1 + 0.1 * torch.randn(k, generator=g)).half().cuda()
    x0 = x.clone()
    res = torch.full_like(x, float("nan"))
    y = rdquant_cuda.mixed_gemv_norm(x, d, w, 1e-6, fd, residual_out=res, flags=_lib.RDQ_GEMV_PDL)
    assert torch.equal(x, x0)
    # separate kernels
    h = torch.empty_like(x)
    x_sep = x.clone()
    rdquant_cuda.add_rmsnorm(x_sep, d, w, h, 1e-6, 0)
    y_sep = rdquant_cuda.mixed_gemv(h, fd)
    assert torch.equal(res, x_sep)
    # the two differ only by the summation order of the mean square (a last-bit change of some
    # normalised activations)
    scale = float(y_sep.float().abs().max())
    assert float((y.float() - y_sep.float()).abs().max()) <= 4e-3 * scale
    # FP32 reference of the whole formula on the dequantised weights
    xf = x_sep.float()
    hn = ((xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).half() * w).cpu()
    y_ref = onp.mixed_precision_linear(hn.numpy(), onp.torch_layer_to_np(layer), splits, k, None)
    assert onp.rel_err(y.cpu().float().numpy(), y_ref) < TOL
    assert int(fd["tile_counters"].abs().sum()) == 0
    # residual_out is optional
    y2 = rdquant_cuda.mixed_gemv_norm(x, d, w, 1e-6, fd)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("k,n,m", [(9728, 2560, 1), (9728, 2560, 2), (512, 256, 5), (2560, 2560, 8)])
def test_prologue_silu_mul(k, n, m):
    """silu(gate) * up computed inside the GEMV: bit-identical to the separate kernels."""
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=k + n + m)
    fd = pack_for_fused_gemv(layer, splits, k, "cuda")
    assert fd["w_tiled"] is not None and rdquant_cuda.gemv_stages_x(m, k)
    gu = torch.randn(m, 2 * k, generator=torch.Generator().manual_seed(m)).half().cuda()
    y = rdquant_cuda.mixed_gemv_silu(gu, fd, flags=_lib.RDQ_GEMV_PDL)
    act = torch.empty(m, k, dtype=torch.float16, device="cuda")
    rdquant_cuda.silu_mul(gu, act, 0)
    y_sep = rdquant_cuda.mixed_gemv(act, fd)
    assert torch.equal(y, y_sep)
    assert int(fd["tile_counters"].abs().sum()) == 0


def test_prologue_refused_when_rows_do_not_fit():
    k, n, m = 9728, 2560, 8
    assert not rdquant_cuda.gemv_stages_x(m, k)
    splits = fixed_splits(n)
    layer = random_packed_layer(splits["NVFP4"], splits["FP8"], splits["FP16"], k, seed=1)
    fd = pack_for_fused_gemv(layer, splits, k, "cuda")
    gu = torch.zeros(m, 2 * k, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="shared memory"):
        rdquant_cuda.mixed_gemv_silu(gu, fd)
    x = torch.zeros(1, 2560, dtype=torch.float16, device="cuda")
    fd2 = pack_for_fused_gemv(random_packed_layer(128, 64, 64, 2560, seed=2), {"NVFP4": 128, "FP8": 64, "FP16": 64}, 2560,
                              "cuda")
    with pytest.raises(RuntimeError, match="alias"):
        rdquant_cuda.mixed_gemv_norm(x, None, x[0], 1e-6, fd2, residual_out=x)
