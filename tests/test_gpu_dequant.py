"""Bit-exact dequantisation on the GPU (through the C ABI) against the oracle and the
reference's golden weights."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, ORDER, golden_layer_np, golden_layer_torch
from oracle import oracle_np as onp
from rdquant_b200 import rdquant_cuda
from rdquant_b200.synthetic import random_packed_layer

pytestmark = pytest.mark.gpu


def _bits16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def test_exhaustive_decode_tables():
    # every E2M1 code x every E4M3 scale byte, and every E4M3 weight byte
    z = np.load(os.path.join(GOLDEN, "tables.npz"))
    codes = torch.arange(16, dtype=torch.uint8)
    row = (codes.repeat_interleave(2)[1::2] << 4 | codes.repeat_interleave(2)[0::2])  # 16 bytes: (c,c) pairs
    row = torch.stack([(c << 4) | c for c in codes]).to(torch.uint8)  # byte j = code j twice -> k = 2j, 2j+1
    n = 256
    w4 = row.repeat(n, 1)  # [256, 16] -> K = 32, two scale blocks per row
    s4 = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(n, 1).repeat(1, 2)
    layer = {"weight_nvfp4": w4.cuda(), "weight_nvfp4_scale": s4.cuda()}
    w = rdquant_cuda.dequantize_packed(layer, {"NVFP4": n}, 32)
    got = _bits16(w).reshape(n, 16, 2)[:, :, 0].T.view(np.float16)  # [code, scale]
    ref = z["products_f16_bits"].view(np.float16)
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok].view(np.uint16), ref[ok].view(np.uint16))
    assert np.isnan(got[~ok]).all()
    # E4M3 weights, scale 1 and a scale that forces float16 rounding
    w8 = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(1, 256).repeat(2, 1).contiguous()
    sc = torch.tensor([1.0, 0.0123], dtype=torch.float32)
    out = rdquant_cuda.dequantize_packed({"weight_fp8": w8.cuda(), "weight_fp8_scale": sc.cuda()}, {"FP8": 2}, 256)
    tab = torch.from_numpy(z["e4m3_f32"])
    exp = (tab.unsqueeze(0) * sc.unsqueeze(1)).half()
    good = ~torch.isnan(exp)
    assert torch.equal(out.cpu()[good].view(torch.int16), exp[good].view(torch.int16))
    assert torch.isnan(out.cpu()[~good]).all()


def test_golden_layers_bit_exact(layers):
    for name, case in layers.items():
        layer, splits, k = golden_layer_torch(case, "cuda")
        w = rdquant_cuda.dequantize_packed(layer, splits, k, inv_perm=layer["inv_permutation"])
        assert np.array_equal(_bits16(w), case["w_packed_f16_bits"]), name
        # in-memory payload (FP16 group as float16): the reference's QuantizedWeight.dequantize()
        mem = dict(layer)
        if splits["FP16"]:
            src = torch.from_numpy(case["weight_f16_bits"].copy()).view(torch.int16).view(torch.float16)
            src = src[torch.from_numpy(case["perm"].astype(np.int64))]
            mem["weight_fp16"] = src[splits["NVFP4"] + splits["FP8"]:].contiguous().cuda()
        w16 = rdquant_cuda.dequantize_packed(mem, splits, k, inv_perm=layer["inv_permutation"])
        assert np.array_equal(_bits16(w16), case["w_ref_f16_bits"]), name
        w32 = rdquant_cuda.dequantize_packed(mem, splits, k, inv_perm=layer["inv_permutation"], out_dtype=torch.float32)
        assert np.array_equal(w32.cpu().numpy().view(np.uint32), case["w_ref_f32"].view(np.uint32)), name


# K = 20 and 36 (no NVFP4 group) give rows whose 16-element runs are not 16-byte aligned in the
# f16 (K % 8 != 0) and f32 (K % 4 == 0 but full runs start at odd multiples of 16 B) outputs
@pytest.mark.parametrize("n4,n8,n16,k", [(128, 128, 128, 2560), (48, 16, 0, 64), (0, 33, 7, 40), (640, 256, 128, 256),
                                         (0, 19, 5, 20), (0, 9, 12, 36), (0, 0, 3, 17)])
def test_random_bytes_vs_oracle(n4, n8, n16, k):
    layer = random_packed_layer(n4, n8, n16, k, seed=n4 + k)
    splits = dict(zip(ORDER, (n4, n8, n16)))
    ref = onp.dequantize_layer(onp.torch_layer_to_np(layer), splits, k)
    dev = {kk: v.cuda() for kk, v in layer.items()}
    w = rdquant_cuda.dequantize_packed(dev, splits, k, inv_perm=dev["inv_permutation"])
    assert np.array_equal(_bits16(w), ref.view(np.uint16))
    w32 = rdquant_cuda.dequantize_packed(dev, splits, k, inv_perm=dev["inv_permutation"], out_dtype=torch.float32)
    ref32 = onp.dequantize_layer_f32(onp.torch_layer_to_np(layer), splits, k)
    assert np.array_equal(w32.cpu().numpy().view(np.uint32), ref32.view(np.uint32))


def test_formats_dequantize_and_qweight(layers):
    from rdquant_b200.core import formats
    from rdquant_b200.quantize import quantize_weight

    case = layers["mixed_384x256"]
    w = torch.from_numpy(case["weight_f16_bits"].copy()).view(torch.int16).view(torch.float16)
    perm = torch.from_numpy(case["perm"].astype(np.int64))
    qw = quantize_weight(w.float(), perm, dict(zip(ORDER, (int(v) for v in case["splits"])))).to("cuda")
    full = qw.dequantize()
    assert full.dtype == torch.float32
    assert np.array_equal(full.cpu().numpy().view(np.uint32), case["w_ref_f32"].view(np.uint32))
    d8 = formats.dequantize(qw.qtensors["FP8"])
    assert d8.shape == (128, 256) and d8.dtype == torch.float32


def test_bad_arguments_raise():
    with pytest.raises(RuntimeError):
        rdquant_cuda.dequantize_packed({"weight_fp8": torch.zeros(4, 8, dtype=torch.uint8),
                                        "weight_fp8_scale": torch.ones(4)}, {"FP8": 4}, 8)  # CPU tensors
    with pytest.raises(RuntimeError):
        rdquant_cuda.dequantize_packed({"weight_nvfp4": torch.zeros(4, 12, dtype=torch.uint8).cuda(),
                                        "weight_nvfp4_scale": torch.zeros(4, 1, dtype=torch.uint8).cuda()},
                                       {"NVFP4": 4}, 24)
