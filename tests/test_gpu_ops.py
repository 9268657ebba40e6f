"""The Python operator surface on the GPU: mixed_precision_linear, QuantizedLayer,
FusedMixedLinear, against the oracle on the reference's golden layers."""
import numpy as np
import pytest
import torch

from conftest import ORDER, golden_layer_torch
from oracle import oracle_np as onp
from rdquant_b200.inference import FusedMixedLinear
from rdquant_b200.ops import mixed_precision_linear
from rdquant_b200.quantize import QuantizedLayer, quantize_weight

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _qw(case):
    w = torch.from_numpy(case["weight_f16_bits"].copy()).view(torch.int16).view(torch.float16)
    perm = torch.from_numpy(case["perm"].astype(np.int64))
    return quantize_weight(w.float(), perm, dict(zip(ORDER, (int(v) for v in case["splits"]))))


def test_mixed_precision_linear_matches_reference_output(layers):
    for name, case in layers.items():
        qw = _qw(case).to("cuda")
        layer, splits, k = golden_layer_torch(case)
        bias = layer.get("bias")
        for m in (1, 3):
            x = torch.from_numpy(case[f"x{m}_f16_bits"].copy()).view(torch.int16).view(torch.float16)
            y = mixed_precision_linear(x.cuda(), qw.qtensors, qw.splits, qw.inv_permutation,
                                       bias.cuda() if bias is not None else None)
            y_ref = torch.from_numpy(case[f"y{m}_ref_f16_bits"].copy()).view(torch.int16).view(torch.float16)
            assert y.dtype == torch.float16 and y.shape == y_ref.shape
            assert onp.rel_err(y.cpu().float().numpy(), y_ref.float().numpy()) < TOL, name


def test_batch_dims_dtypes_and_layer(layers):
    case = layers["mixed_256x128"]
    qw = _qw(case).to("cuda")
    layer = QuantizedLayer(qw, None, 128, 256).cuda()
    x = torch.randn(2, 5, 128, device="cuda")
    y = layer(x)
    assert y.shape == (2, 5, 256) and y.dtype == torch.float32
    xb = x.to(torch.bfloat16)
    assert layer(xb).dtype == torch.bfloat16
    w = qw.dequantize()
    ref = x.half().float() @ w.half().float().T
    assert onp.rel_err(y.cpu().numpy().reshape(10, 256), ref.cpu().numpy().reshape(10, 256)) < TOL


def test_fused_mixed_linear_module(layers):
    case = layers["mixed_384x256"]
    layer, splits, k = golden_layer_torch(case)
    mod = FusedMixedLinear.from_layer_data(layer, splits, k, "cuda")
    assert mod.N == 384 and mod.K == 256 and mod.inv_perm.dtype == torch.int64
    for m in (1, 16, 40):
        x = torch.randn(m, k).half()
        y = mod(x.cuda())
        y_ref = onp.mixed_precision_linear(x.numpy(), onp.torch_layer_to_np(layer), splits, k)
        assert onp.rel_err(y.cpu().float().numpy(), y_ref) < TOL, m
    with pytest.raises(RuntimeError):
        mod(torch.randn(1, k).half())  # CPU input: no host path


def test_graphed_decode_step(layers):
    from rdquant_b200.inference import GraphedDecodeStep

    mods = []
    for name in ("mixed_384x256", "alloc_512x256"):
        layer, splits, k = golden_layer_torch(layers[name])
        mods.append(FusedMixedLinear.from_layer_data(layer, splits, k, "cuda"))
    step = GraphedDecodeStep(mods, m=2)
    for call in range(2):
        xs = [torch.randn(2, mod.K).half() for mod in mods]
        for xh, x in zip(step.x_host, xs):
            xh.copy_(x)
        ys = step.run()
        for mod, x, y in zip(mods, xs, ys):
            assert torch.equal(y, mod(x.cuda()).cpu()), call
