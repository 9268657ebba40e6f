"""NVFP4 / FP8 / FP16 weight formats of the mixed-precision linear operator.

Public surface follows the reference (rdquant/core/formats.py:28-36, :371-395):
``QuantizedTensor``, ``quantize``, ``dequantize``, ``get_bits_per_element``.

* ``quantize`` (encode) is offline input generation and runs as torch ops on whatever
  device the tensor lives on; it reproduces the reference encoders bit for bit
  (rdquant/core/formats.py:84-142, :166-193, :206-223).
* ``dequantize`` (decode) is part of the operator and runs on the GPU through the
  bit-exact dequantisation kernel of ``librdq_b200.so``; there is no CPU decode path.

Value grids: NVFP4 code = magnitude index (0, .5, 1, 1.5, 2, 3, 4, 6) + 8 * sign, one
E4M3 scale per 16 consecutive elements, dequantised value = grid[code] * scale (the
stored ``global_scale`` is metadata, rdquant/core/formats.py:145-159).  FP8 = E4M3
(torch.float8_e4m3fn) with one FP32 scale per quantised group.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

NVFP4_BLOCK = 16
E4M3_MAX = 448.0
E2M1_MAX = 6.0
# magnitudes of the eight E2M1 codes and the decision thresholds halfway between them
E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)

_BITS = {"NVFP4": 4, "FP8": 8, "FP16": 16}


@dataclass
class QuantizedTensor:
    """Quantised payload of one format group (field-compatible with the reference)."""

    data: torch.Tensor
    scales: torch.Tensor
    format_name: str
    original_shape: torch.Size
    bits_per_element: int
    global_scale: Optional[float] = None


def _round_to_e4m3(v: torch.Tensor) -> torch.Tensor:
    """Nearest E4M3 value (saturating at +-448) as float32."""
    return v.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).to(torch.float32)


def _encode_nvfp4(t: torch.Tensor) -> QuantizedTensor:
    shape = t.shape
    v = t.reshape(-1).float()
    n = v.numel()
    tail = (-n) % NVFP4_BLOCK
    if tail:
        v = torch.cat([v, v.new_zeros(tail)])
    blocks = v.view(-1, NVFP4_BLOCK)
    scale = _round_to_e4m3(blocks.abs().amax(dim=1) / E2M1_MAX)
    top = scale.max().item() if scale.numel() else 0.0
    divisor = torch.where(scale == 0, torch.ones_like(scale), scale)
    ratio = (blocks / divisor.unsqueeze(1)).reshape(-1)
    mag = ratio.abs()
    # nearest grid point, ties to the smaller magnitude: count thresholds strictly below
    mids = torch.tensor(_E2M1_MIDPOINTS, dtype=torch.float32, device=v.device)
    code = (mag.unsqueeze(1) > mids).sum(dim=1)
    code = code + (ratio < 0).long() * 8
    return QuantizedTensor(
        data=code[:n],
        scales=scale,
        format_name="NVFP4",
        original_shape=shape,
        bits_per_element=4,
        global_scale=top if top != 0 else 1.0,
    )


def _encode_fp8(t: torch.Tensor) -> QuantizedTensor:
    shape = t.shape
    v = t.float()
    scale = v.abs().max().item() / E4M3_MAX if v.numel() else 0.0
    if scale == 0:
        scale = 1.0
    return QuantizedTensor(
        data=_round_to_e4m3(v / scale),
        scales=torch.tensor([scale], dtype=torch.float32, device=t.device),
        format_name="FP8",
        original_shape=shape,
        bits_per_element=8,
    )


def _encode_fp16(t: torch.Tensor) -> QuantizedTensor:
    return QuantizedTensor(
        data=t.float().to(torch.float16),
        scales=torch.empty(0, dtype=torch.float32, device=t.device),
        format_name="FP16",
        original_shape=t.shape,
        bits_per_element=16,
    )


_ENCODERS = {"NVFP4": _encode_nvfp4, "FP8": _encode_fp8, "FP16": _encode_fp16}


def get_bits_per_element(format_name: str) -> int:
    return _BITS[format_name]


def quantize(tensor: torch.Tensor, format_name: str) -> QuantizedTensor:
    """Encode ``tensor`` (flattened; NVFP4 blocks run over the flattened order)."""
    if format_name not in _ENCODERS:
        raise KeyError(f"unsupported format {format_name!r}; this build covers NVFP4, FP8, FP16")
    with torch.no_grad():
        return _ENCODERS[format_name](tensor)


# ---------------------------------------------------------------------------
# byte-level packing shared by the checkpoint writer and the kernel packer
# ---------------------------------------------------------------------------

def pack_nvfp4_codes(codes_2d: torch.Tensor) -> torch.Tensor:
    """[n, K] codes 0..15 -> [n, K/2] uint8, byte = code[2j+1] << 4 | code[2j]
    (rdquant/integrations/hf_export.py:81-86)."""
    lo = codes_2d[:, 0::2].to(torch.uint8)
    hi = codes_2d[:, 1::2].to(torch.uint8)
    return (hi << 4) | lo


def e4m3_bytes(values: torch.Tensor) -> torch.Tensor:
    """E4M3-representable float32 values -> their bit patterns as uint8."""
    return values.to(torch.float8_e4m3fn).view(torch.uint8)


def qtensor_to_packed(qt: QuantizedTensor) -> dict[str, torch.Tensor]:
    """Packed device/checkpoint tensors of one group, named as in the checkpoint."""
    n, k = qt.original_shape
    if qt.format_name == "NVFP4":
        if k % NVFP4_BLOCK:
            raise ValueError(f"NVFP4 packing needs in_features % 16 == 0, got {k}")
        return {
            "weight_nvfp4": pack_nvfp4_codes(qt.data.reshape(n, k)),
            "weight_nvfp4_scale": e4m3_bytes(qt.scales.reshape(n, k // NVFP4_BLOCK)),
        }
    if qt.format_name == "FP8":
        sc = qt.scales.reshape(-1).float()
        if sc.numel() == 1:
            sc = sc.expand(n)
        return {
            "weight_fp8": e4m3_bytes(qt.data.reshape(n, k)),
            "weight_fp8_scale": sc.contiguous().clone(),
        }
    if qt.format_name == "FP16":
        return {"weight_fp16": qt.data.reshape(n, k).to(torch.float16)}
    raise KeyError(qt.format_name)


def dequantize(qtensor: QuantizedTensor) -> torch.Tensor:
    """Decode to float32 of ``original_shape`` on the GPU (bit-exact kernel).

    The payload must live on a CUDA device; there is no host decode path.
    """
    from rdquant_b200 import rdquant_cuda

    if not qtensor.data.is_cuda:
        raise RuntimeError("rdquant_b200.core.formats.dequantize runs on CUDA tensors only")
    shape = tuple(qtensor.original_shape)
    if len(shape) == 2:
        n, k = shape
        flat_tail = 0
    else:
        # 1-D payloads: decode as one row (padded to a whole scale block for NVFP4)
        n, k = 1, int(torch.Size(shape).numel())
        flat_tail = (-k) % NVFP4_BLOCK if qtensor.format_name == "NVFP4" else 0
    qt = qtensor
    if flat_tail:
        pad = torch.zeros(flat_tail, dtype=qt.data.dtype, device=qt.data.device)
        qt = QuantizedTensor(torch.cat([qt.data.reshape(-1), pad]), qt.scales, qt.format_name,
                             torch.Size([1, k + flat_tail]), qt.bits_per_element, qt.global_scale)
    elif len(shape) != 2:
        qt = QuantizedTensor(qt.data, qt.scales, qt.format_name, torch.Size([1, k]),
                             qt.bits_per_element, qt.global_scale)
    packed = qtensor_to_packed(qt)
    kk = k + flat_tail
    splits = {"NVFP4": 0, "FP8": 0, "FP16": 0}
    splits[qt.format_name] = n
    w = rdquant_cuda.dequantize_packed(packed, splits, kk, inv_perm=None)
    return w[:, :k].float().reshape(shape)
