"""GPU encoders against the host encoders (which the golden fixtures pin to the reference):
packed NVFP4 / FP8 tensors must be byte-identical; per-row squared errors within rounding."""
import numpy as np
import pytest
import torch

from rdquant_b200 import rdquant_cuda
from rdquant_b200.core import formats

pytestmark = pytest.mark.gpu


def _weights(n, k, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    idx = torch.randperm(n, generator=g)[: max(1, n // 100)]
    w[idx] *= 8
    return w.to(dtype)


def _special(dtype):
    rows = []
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    # block scale exactly 1: every midpoint (ties go down), both signs, signed zeros, the maximum
    rows.append([6.0, -6.0, 0.0, -0.0] + mids + [-m for m in mids[:5]])
    # scale 0.5, values just above / below midpoints
    rows.append([3.0] + [m * 0.5 * (1 + 2 ** -10) for m in mids] + [-m * 0.5 * (1 - 2 ** -10) for m in mids] + [0.1])
    rows.append([0.0] * 16)                                    # all-zero block: scale 0 -> divisor 1
    rows.append([1e-6 * (i - 8) for i in range(16)])           # subnormal block scales
    rows.append([3000.0, -2999.0] + [100.0 * i for i in range(14)])  # absmax / 6 above 448: clamped scale
    rows.append([2.0 ** -12] * 8 + [-(2.0 ** -13)] * 8)
    w = torch.tensor(rows, dtype=torch.float32)
    w = torch.cat([w, w.flip(1)], dim=1)                       # two blocks per row
    return w.to(dtype)


def _host_nvfp4(w):
    qt = formats.quantize(w.cpu(), "NVFP4")
    packed = formats.qtensor_to_packed(qt)
    rec = formats.E2M1_GRID
    lut = torch.tensor(list(rec) + [-v for v in rec], dtype=torch.float32)
    deq = lut[qt.data.reshape(w.shape)] * qt.scales.reshape(w.shape[0], -1).repeat_interleave(16, dim=1)
    sq = ((w.cpu().double() - deq.double()) ** 2).sum(dim=1)
    return packed, qt.global_scale, sq


def _host_fp8(w):
    qt = formats.quantize(w.cpu(), "FP8")
    packed = formats.qtensor_to_packed(qt)
    deq = qt.data.reshape(w.shape).double() * float(qt.scales[0])
    sq = ((w.cpu().double() - deq) ** 2).sum(dim=1)
    return packed, sq


CASES = [("rand", 128, 256, 1), ("rand", 300, 2560, 2), ("rand", 64, 16, 3), ("rand", 1, 4096, 4), ("special", 0, 0, 0)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_nvfp4_bytes_match_host_encoder(case, dtype):
    kind, n, k, seed = case
    w = _special(dtype) if kind == "special" else _weights(n, k, seed, dtype)
    host, gscale, sq = _host_nvfp4(w)
    dev = rdquant_cuda.quantize_nvfp4_packed(w.cuda(), want_sqerr=True)
    assert torch.equal(dev["weight_nvfp4_scale"].cpu(), host["weight_nvfp4_scale"])
    assert torch.equal(dev["weight_nvfp4"].cpu(), host["weight_nvfp4"])
    top = float(dev["global_scale"].item())
    assert (top if top != 0 else 1.0) == pytest.approx(gscale, rel=0, abs=0)
    np.testing.assert_allclose(dev["row_sqerr"].cpu().double().numpy(), sq.numpy(), rtol=1e-4, atol=1e-30)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", CASES + [("zero", 4, 32, 0)])
def test_fp8_bytes_match_host_encoder(case, dtype):
    kind, n, k, seed = case
    if kind == "zero":
        w = torch.zeros(n, k, dtype=dtype)
    else:
        w = _special(dtype) if kind == "special" else _weights(n, k, seed, dtype)
    host, sq = _host_fp8(w)
    dev = rdquant_cuda.quantize_fp8_packed(w.cuda(), want_sqerr=True)
    assert torch.equal(dev["weight_fp8_scale"].cpu(), host["weight_fp8_scale"])
    assert torch.equal(dev["weight_fp8"].cpu(), host["weight_fp8"])
    np.testing.assert_allclose(dev["row_sqerr"].cpu().double().numpy(), sq.numpy(), rtol=1e-4, atol=1e-30)


def test_full_size_group_matches_host_and_decodes_back():
    """A benchmark-sized group (gate_proj's NVFP4 rows): bytes equal the host encoder's, and the
    bit-exact GPU decoder applied to them reproduces the host reconstruction."""
    n, k = 6528, 2560
    w = _weights(n, k, 5, torch.float16)
    host, _, _ = _host_nvfp4(w)
    enc = rdquant_cuda.quantize_nvfp4_packed(w.cuda())
    assert torch.equal(enc["weight_nvfp4"].cpu(), host["weight_nvfp4"])
    assert torch.equal(enc["weight_nvfp4_scale"].cpu(), host["weight_nvfp4_scale"])
    layer = {"weight_nvfp4": enc["weight_nvfp4"], "weight_nvfp4_scale": enc["weight_nvfp4_scale"]}
    deq = rdquant_cuda.dequantize_packed(layer, {"NVFP4": n, "FP8": 0, "FP16": 0}, k, inv_perm=None)
    err = (deq.float().cpu() - w.float()).abs().max()
    assert float(err) <= float(w.float().abs().max()) / 6 * 1.5  # at most about one grid step of the largest block


def test_layer_fast_path_equals_host_route():
    """quantize_weight_packed (GPU) == pack_layer(quantize_weight(...)) (host) tensor by tensor."""
    from rdquant_b200.integrations.hf_export import pack_layer
    from rdquant_b200.quantize import quantize_weight, quantize_weight_packed

    n, k = 512, 320
    g = torch.Generator().manual_seed(8)
    w = _weights(n, k, 8, torch.float16)
    perm = torch.randperm(n, generator=g)
    splits = {"NVFP4": 256, "FP8": 128, "FP16": 128}
    bias = torch.randn(n, generator=g).half()
    host = pack_layer(quantize_weight(w, perm, splits), bias)
    dev = quantize_weight_packed(w.cuda(), perm, splits, bias.cuda())
    assert set(host) == set(dev)
    for key in host:
        a, b = host[key], dev[key].cpu()
        assert a.dtype == b.dtype and torch.equal(a, b), key
