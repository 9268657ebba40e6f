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


@pytest.mark.parametrize("poll", [True, False])
def test_graphed_decode_step(layers, poll):
    """Host buffers in, host buffers out, one graph replay; completion seen by polling the word
    the last copy kernel writes behind its data, or by a stream synchronisation."""
    from rdquant_b200.inference import GraphedDecodeStep

    mods = []
    for name in ("mixed_384x256", "alloc_512x256"):
        layer, splits, k = golden_layer_torch(layers[name])
        mods.append(FusedMixedLinear.from_layer_data(layer, splits, k, "cuda"))
    step = GraphedDecodeStep(mods, m=2, poll=poll)
    for call in range(5):
        xs = [torch.randn(2, mod.K).half() for mod in mods]
        for xh, x in zip(step.x_host, xs):
            xh.copy_(x)
        ys = step.run()
        for mod, x, y in zip(mods, xs, ys):
            assert torch.equal(y, mod(x.cuda()).cpu()), call
    if poll:
        assert int(step._done_flag[0]) == 6  # the warm-up call and five replays


def test_stage_copy_signal():
    """The signalled copy: odd sizes, device -> pinned host, the flag counts the launches."""
    from rdquant_b200 import rdquant_cuda

    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    for launch, nbytes in enumerate((16, 61440, 4096 * 37 + 5, 3), start=1):
        src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
        dst = torch.zeros(nbytes, dtype=torch.uint8).pin_memory()
        rdquant_cuda.stage_copy(dst, src, state, flag)
        torch.cuda.synchronize()
        assert int(flag[0]) == launch and torch.equal(dst, src.cpu())
        back = torch.zeros_like(src)
        rdquant_cuda.stage_copy(back, dst)  # pinned host -> device, no signal
        torch.cuda.synchronize()
        assert torch.equal(back, src)
    assert state.tolist() == [0, 4]
