"""The oracle (oracle/oracle_np.py, oracle/rdq_oracle.c) against golden vectors produced by
running the reference package (tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np
import pytest

from conftest import GOLDEN, golden_layer_np
from oracle import oracle_np as onp


def test_e4m3_table_matches_torch():
    z = np.load(os.path.join(GOLDEN, "tables.npz"))
    ref = z["e4m3_f32"]
    mine = onp.e4m3_table()
    nan = np.isnan(ref)
    assert nan.sum() == 2 and nan[0x7F] and nan[0xFF]
    assert np.array_equal(np.isnan(mine), nan)
    assert np.array_equal(mine[~nan].view(np.uint32), ref[~nan].view(np.uint32))
    assert mine[1] == 2.0 ** -9 and mine[0x7E] == 448.0


def test_nvfp4_lut_and_products():
    z = np.load(os.path.join(GOLDEN, "tables.npz"))
    assert np.array_equal(onp.E2M1_LUT.view(np.uint32), z["nvfp4_lut"].view(np.uint32))
    prod = (onp.E2M1_LUT[:, None] * onp.e4m3_table()[None, :]).astype(np.float16)
    ref = z["products_f16_bits"].view(np.float16)
    ok = ~np.isnan(ref)
    assert np.array_equal(prod[ok].view(np.uint16), ref[ok].view(np.uint16))
    # every product is exactly representable in float16 (what lets the kernels scale in f16)
    exact = (onp.E2M1_LUT[:, None].astype(np.float64) * onp.e4m3_table()[None, :].astype(np.float64))
    assert np.array_equal(prod[ok].astype(np.float64), exact[ok])


def test_dequant_bit_exact(layers):
    for name, case in layers.items():
        layer, splits, k = golden_layer_np(case)
        # from the checkpoint bytes: the reference's _materialize_packed_groups
        w16 = onp.dequantize_layer(layer, splits, k)
        assert np.array_equal(w16.view(np.uint16), case["w_packed_f16_bits"]), name
        # from the in-memory payload (FP16 group not rounded through bfloat16):
        # QuantizedWeight.dequantize(), float32 and its float16 cast
        mem = dict(layer)
        if splits["FP16"]:
            src = case["weight_f16_bits"].view(np.float16)[case["perm"].astype(np.int64)]
            mem["weight_fp16"] = np.ascontiguousarray(src[splits["NVFP4"] + splits["FP8"]:])
        w16m = onp.dequantize_layer(mem, splits, k)
        assert np.array_equal(w16m.view(np.uint16), case["w_ref_f16_bits"]), name
        w32 = onp.dequantize_layer_f32(mem, splits, k)
        assert np.array_equal(w32.view(np.uint32), case["w_ref_f32"].view(np.uint32)), name


def test_operator_output(layers):
    for name, case in layers.items():
        layer, splits, k = golden_layer_np(case)
        bias = layer["bias"].view(np.float16).astype(np.float32) if "bias" in layer else None
        if splits["FP16"]:  # the reference operator ran on the in-memory payload
            src = case["weight_f16_bits"].view(np.float16)[case["perm"].astype(np.int64)]
            layer = dict(layer)
            layer["weight_fp16"] = np.ascontiguousarray(src[splits["NVFP4"] + splits["FP8"]:])
        for m in (1, 3):
            x = case[f"x{m}_f16_bits"].view(np.float16)
            y_ref = case[f"y{m}_ref_f16_bits"].view(np.float16).astype(np.float32)
            y = onp.mixed_precision_linear(x, layer, splits, k, bias)
            # the reference ran float16 F.linear (+ float16 bias add): agree to float16 rounding
            assert onp.rel_err(y, y_ref) < 1.5e-3, name


def test_c_oracle_matches_numpy(layers):
    from oracle import oracle_c

    oracle_c.build()
    tab = onp.e4m3_table()
    for name, case in layers.items():
        layer, splits, k = golden_layer_np(case)
        n4, n8, n16 = splits["NVFP4"], splits["FP8"], splits["FP16"]
        codes = onp.unpack_nibbles(layer["weight_nvfp4"]).astype(np.int64).reshape(-1) if n4 else None
        sc4 = tab[layer["weight_nvfp4_scale"]].reshape(-1).astype(np.float32) if n4 else None
        d8 = tab[layer["weight_fp8"]].reshape(-1).astype(np.float32) if n8 else None
        s8 = float(layer["weight_fp8_scale"][0]) if n8 else 1.0
        d16 = None
        if n16:
            d16 = onp.bf16_bits_to_f32(layer["weight_fp16"].view(np.uint16)).astype(np.float16).reshape(-1)
        x = case["x3_f16_bits"].view(np.float16)
        bias = layer["bias"].view(np.float16).astype(np.float32) if "bias" in layer else None
        y_c = oracle_c.linear(x, codes, sc4, n4, d8, s8, n8, d16, n16, layer["inv_permutation"], bias)
        y_np = onp.mixed_precision_linear(x, layer, splits, k, bias)
        assert onp.rel_err(y_c, y_np) < 1e-5, name


def test_inv_perm_is_a_gather():
    # y[j] = y_perm[inv_perm[j]] equals scattering y_perm[p] to perm[p] (rdquant/ops.py:62-63)
    rng = np.random.default_rng(0)
    perm = rng.permutation(50)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(50)
    yp = rng.standard_normal(50)
    scat = np.empty(50)
    scat[perm] = yp
    assert np.array_equal(yp[inv], scat)
