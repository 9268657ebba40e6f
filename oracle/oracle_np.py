"""TEST INFRASTRUCTURE ONLY -- numpy restatement of the reference's mixed-precision linear.

Parity pin: every function here is checked against golden vectors produced by running the
reference package itself (tests/golden/make_golden.py, fixtures in tests/golden/*.npz):
the 256-entry E4M3 table from torch.float8_e4m3fn, the 16 x 256 table of NVFP4 products,
packed layers written by the reference's save_packed with the reference's dequantised
weights and operator outputs.  tests/test_oracle_golden.py runs those checks on CPU.

Each function cites the reference lines it restates.
"""
from __future__ import annotations

import numpy as np

# rdquant/core/formats.py:75-81 -- E2M1 value grid, code = magnitude index + 8 * sign
E2M1_LUT = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32,
)


def e4m3_table() -> np.ndarray:
    """float32 value of every E4M3 byte under torch.float8_e4m3fn semantics
    (used by rdquant/core/formats.py:52-66 and rdquant/integrations/hf_export.py:264-267):
    bias 7, subnormals mant * 2^-9, 0x7f / 0xff NaN, no infinities, max 448."""
    out = np.empty(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = sign * m * 2.0 ** -9
        else:
            v = sign * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        out[b] = v
    return out


_E4M3 = e4m3_table()


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    """[n, K/2] uint8 -> [n, K] codes; low nibble = even k, high nibble = odd k
    (rdquant/integrations/hf_export.py:81-86, :249-262)."""
    n, half = packed.shape
    codes = np.empty((n, half * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = packed >> 4
    return codes


def nvfp4_dequantize(codes: np.ndarray, block_scales: np.ndarray, shape) -> np.ndarray:
    """rdquant/core/formats.py:145-159: LUT[code] * block_scale[i // 16]; the stored global
    scale is not applied."""
    flat = codes.reshape(-1)
    n = flat.size
    pad = (-n) % 16
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=flat.dtype)])
    vals = E2M1_LUT[flat].reshape(-1, 16) * block_scales.astype(np.float32).reshape(-1, 1)
    return vals.reshape(-1)[:n].reshape(shape)


def fp8_dequantize(values_f32: np.ndarray, scale: float, shape) -> np.ndarray:
    """rdquant/core/formats.py:196-199."""
    return (values_f32.astype(np.float32) * np.float32(scale)).reshape(shape)


def bf16_bits_to_f32(bits_u16: np.ndarray) -> np.ndarray:
    return (bits_u16.astype(np.uint32) << 16).view(np.float32)


def materialize_packed_groups(layer: dict, splits: dict, k: int) -> np.ndarray:
    """Dequantised float16 weight [N, K] in PERMUTED row order from checkpoint tensors
    (rdquant/inference.py:67-121): NVFP4 f16(LUT*e4m3(scale)), FP8 f16(f32(e4m3)*scale[n]),
    FP16 group bf16 -> f16.  ``weight_fp16`` is given as uint16 bf16 bit patterns
    (``weight_fp16_is_f16`` True: float16 array)."""
    parts = []
    n4, n8, n16 = (int(splits.get(f, 0)) for f in ("NVFP4", "FP8", "FP16"))
    if n4:
        codes = unpack_nibbles(np.asarray(layer["weight_nvfp4"]))
        sc = _E4M3[np.asarray(layer["weight_nvfp4_scale"])]
        w = E2M1_LUT[codes].reshape(n4, k // 16, 16) * sc.reshape(n4, k // 16, 1)
        parts.append(w.reshape(n4, k).astype(np.float16))
    if n8:
        w = _E4M3[np.asarray(layer["weight_fp8"])] * np.asarray(layer["weight_fp8_scale"], dtype=np.float32).reshape(n8, 1)
        parts.append(w.astype(np.float32).astype(np.float16))
    if n16:
        w16 = np.asarray(layer["weight_fp16"])
        if w16.dtype == np.float16:
            parts.append(w16.reshape(n16, k))
        else:
            parts.append(bf16_bits_to_f32(w16.view(np.uint16)).reshape(n16, k).astype(np.float16))
    return np.concatenate(parts, axis=0)


def dequantize_layer(layer: dict, splits: dict, k: int) -> np.ndarray:
    """float16 [N, K] in ORIGINAL channel order: cat(groups)[inv_perm]
    (rdquant/quantize.py:56-69, rdquant/inference.py:828-841)."""
    w = materialize_packed_groups(layer, splits, k)
    inv = np.asarray(layer["inv_permutation"]).astype(np.int64)
    return w[inv]


def dequantize_layer_f32(layer: dict, splits: dict, k: int) -> np.ndarray:
    """float32 [N, K], original order, unrounded products: QuantizedWeight.dequantize()
    (rdquant/quantize.py:50-69 over rdquant/core/formats.py:145-159, :196-199, :226-228)."""
    parts = []
    n4, n8, n16 = (int(splits.get(f, 0)) for f in ("NVFP4", "FP8", "FP16"))
    if n4:
        codes = unpack_nibbles(np.asarray(layer["weight_nvfp4"]))
        sc = _E4M3[np.asarray(layer["weight_nvfp4_scale"])]
        parts.append((E2M1_LUT[codes].reshape(n4, k // 16, 16) * sc.reshape(n4, k // 16, 1)).reshape(n4, k))
    if n8:
        parts.append((_E4M3[np.asarray(layer["weight_fp8"])]
                      * np.asarray(layer["weight_fp8_scale"], dtype=np.float32).reshape(n8, 1)).astype(np.float32))
    if n16:
        w16 = np.asarray(layer["weight_fp16"])
        if w16.dtype != np.float16:
            w16 = bf16_bits_to_f32(w16.view(np.uint16)).reshape(n16, k).astype(np.float16)
        parts.append(w16.reshape(n16, k).astype(np.float32))
    inv = np.asarray(layer["inv_permutation"]).astype(np.int64)
    return np.concatenate(parts, axis=0)[inv]


def mixed_precision_linear(x_f16: np.ndarray, layer: dict, splits: dict, k: int, bias=None) -> np.ndarray:
    """rdquant/ops.py:32-68 with FP32 accumulation: per group F.linear(x, dequant.to(f16)),
    cat, index_select(-1, inv_perm), + bias.  Returns float32 [M, N]."""
    w = materialize_packed_groups(layer, splits, k).astype(np.float32)
    y_perm = x_f16.astype(np.float32) @ w.T
    inv = np.asarray(layer["inv_permutation"]).astype(np.int64)
    y = y_perm[:, inv]
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)
    return y


def rel_err(y: np.ndarray, y_ref: np.ndarray) -> float:
    """max |y - y_ref| / max |y_ref| -- the output criterion (2e-3) of the operator."""
    den = float(np.max(np.abs(y_ref)))
    return float(np.max(np.abs(y.astype(np.float64) - y_ref.astype(np.float64)))) / (den if den > 0 else 1.0)


def torch_layer_to_np(layer_data: dict) -> dict:
    """Checkpoint-named torch tensors -> numpy (bfloat16 as uint16 bit patterns)."""
    import torch

    out = {}
    for key, t in layer_data.items():
        t = t.detach().cpu()
        if t.dtype == torch.bfloat16:
            out[key] = t.view(torch.int16).numpy().view(np.uint16)
        else:
            out[key] = t.numpy()
    return out
