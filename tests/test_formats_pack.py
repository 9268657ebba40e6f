"""Encoders, byte packing and the checkpoint writer against the reference's own output
(golden fixtures).  CPU only: these are the offline / host parts of the package."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import ORDER, golden_layer_torch
from rdquant_b200.core import formats
from rdquant_b200.integrations import hf_export
from rdquant_b200.quantize import QuantizedLayer, QuantizedModel, quantize_weight


def _case_weight(case):
    w = torch.from_numpy(case["weight_f16_bits"].copy()).view(torch.int16).view(torch.float16)
    perm = torch.from_numpy(case["perm"].astype(np.int64))
    splits = dict(zip(ORDER, (int(v) for v in case["splits"])))
    return w, perm, splits


def test_quantize_and_pack_match_reference_bytes(layers):
    for name, case in layers.items():
        w, perm, splits = _case_weight(case)
        qw = quantize_weight(w.float(), perm, splits)
        ref, _, _ = golden_layer_torch(case)
        bias = ref.get("bias")
        mine = hf_export.pack_layer(qw, bias)
        assert set(mine) == set(ref), name
        for key in ref:
            a, b = mine[key], ref[key]
            assert a.dtype == b.dtype and a.shape == b.shape, (name, key)
            if a.dtype in (torch.bfloat16, torch.float16):
                a, b = a.view(torch.int16), b.view(torch.int16)
            assert torch.equal(a, b), (name, key)


def test_nvfp4_tie_breaks_and_edges():
    # exact midpoints go to the smaller magnitude; zeros, negative zero, all-zero blocks
    blk = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -5.0, 0.0, -0.0, 6.0, 0.5, 1.0, 3.0])
    q = formats.quantize(blk, "NVFP4")
    assert float(q.scales[0]) == 1.0
    assert q.data.tolist() == [0, 1, 2, 3, 4, 5, 6, 7, 8, 14, 0, 0, 7, 1, 2, 5]
    z = formats.quantize(torch.zeros(32), "NVFP4")
    assert z.global_scale == 1.0 and int(z.data.sum()) == 0
    odd = formats.quantize(torch.randn(37), "NVFP4")
    assert odd.data.numel() == 37 and odd.scales.numel() == 3


def test_fp8_scale_and_clamp():
    t = torch.tensor([448.0 * 2, -3.0, 0.1])
    q = formats.quantize(t, "FP8")
    assert q.scales.shape == (1,) and abs(float(q.scales) - 2.0) < 1e-6
    assert float(q.data.abs().max()) <= 448.0
    assert formats.quantize(torch.zeros(4), "FP8").scales.item() == 1.0


def test_nibble_pack_roundtrip():
    codes = torch.randint(0, 16, (5, 64))
    packed = formats.pack_nvfp4_codes(codes)
    assert packed.dtype == torch.uint8 and packed.shape == (5, 32)
    assert torch.equal(hf_export.unpack_nvfp4_codes(packed), codes)


def test_save_packed_roundtrip(tmp_path, layers):
    case = layers["mixed_256x128"]
    w, perm, splits = _case_weight(case)
    qw = quantize_weight(w.float(), perm, splits)
    holder = torch.nn.Module()
    holder.add_module("fc", QuantizedLayer(qw, torch.zeros(256), 128, 256))
    holder.add_module("norm", torch.nn.LayerNorm(8))
    qm = QuantizedModel(holder, formats=list(ORDER), budget_avg_bits=5.3)
    hf_export.save_packed(qm, str(tmp_path))
    cfg = json.load(open(os.path.join(tmp_path, "quantization_config.json")))
    assert cfg["quant_method"] == "rdquant" and cfg["format_order"] == list(ORDER)
    assert cfg["layers"]["fc"] == {"in_features": 128, "out_features": 256,
                                   "splits": {"NVFP4": 128, "FP8": 64, "FP16": 64}, "avg_bits": qw.avg_bits}
    _, tensors = hf_export.read_layers(str(tmp_path))
    assert tensors["fc.weight_nvfp4"].shape == (128, 64) and tensors["fc.weight_fp16"].dtype == torch.bfloat16
    assert tensors["norm.weight"].dtype == torch.float16
    back = hf_export.load_packed(str(tmp_path))
    layer = back.model.get_layer("fc")
    q2 = layer.quantized_weight
    assert torch.equal(q2.qtensors["NVFP4"].data, qw.qtensors["NVFP4"].data)
    assert torch.equal(q2.qtensors["NVFP4"].scales, qw.qtensors["NVFP4"].scales)
    assert torch.equal(q2.qtensors["FP8"].data, qw.qtensors["FP8"].data)
    assert torch.equal(q2.permutation, qw.permutation)


def test_operator_has_no_host_path(layers):
    from rdquant_b200.ops import mixed_precision_linear

    w, perm, splits = _case_weight(layers["mixed_256x128"])
    qw = quantize_weight(w.float(), perm, splits)
    with pytest.raises(RuntimeError):
        mixed_precision_linear(torch.zeros(1, 128, dtype=torch.float16), qw.qtensors, qw.splits, qw.inv_permutation)
    with pytest.raises(RuntimeError):
        formats.dequantize(qw.qtensors["FP8"])
