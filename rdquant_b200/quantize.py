"""Containers for a mixed-precision linear layer and the packer that fills them.

``QuantizedWeight`` / ``QuantizedLayer`` / ``QuantizedModel`` are field-compatible with
the reference (rdquant/quantize.py:31-69, :76-130, :137-226), so objects produced by the
reference's ``quantize_model`` can be handed to ``save_packed`` or the operator here
unchanged.  Format *allocation* (which channel gets which format) is an offline CPU
search that this package does not contain; ``quantize_weight`` takes the allocation
(permutation + group sizes) as input and performs the grouping and encoding of
rdquant/quantize.py:233-280.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from rdquant_b200.core.formats import QuantizedTensor, get_bits_per_element, quantize

FORMAT_ORDER = ("NVFP4", "FP8", "FP16")


@dataclass
class QuantizedWeight:
    qtensors: dict
    permutation: torch.Tensor
    inv_permutation: torch.Tensor
    splits: dict
    original_shape: torch.Size
    avg_bits: float

    def dequantize(self) -> torch.Tensor:
        """FP32 [N, K] weight in original channel order (bit-exact GPU kernel).

        Same result as the reference's ``cat(dequantize(group))[inv_perm]``
        (rdquant/quantize.py:50-69).  The payload must be on a CUDA device.
        """
        from rdquant_b200 import rdquant_cuda
        from rdquant_b200.fused_gemv_pack import layer_data_from_qweight

        n_out, n_in = self.original_shape
        layer_data = layer_data_from_qweight(self)
        dev = next(iter(layer_data.values())).device
        if dev.type != "cuda":
            raise RuntimeError("QuantizedWeight.dequantize runs on CUDA tensors only")
        return rdquant_cuda.dequantize_packed(
            layer_data, self.splits, n_in, inv_perm=self.inv_permutation.to(dev), out_dtype=torch.float32
        )

    def to(self, device) -> "QuantizedWeight":
        qts = {
            f: QuantizedTensor(q.data.to(device), q.scales.to(device), q.format_name, q.original_shape,
                               q.bits_per_element, q.global_scale)
            for f, q in self.qtensors.items()
        }
        return QuantizedWeight(qts, self.permutation.to(device), self.inv_permutation.to(device),
                               dict(self.splits), self.original_shape, self.avg_bits)


def inverse_permutation(perm: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
    return inv


def quantize_weight(weight: torch.Tensor, permutation: torch.Tensor, splits: dict) -> QuantizedWeight:
    """Group the rows of ``weight`` [N, K] by ``permutation`` and encode each format group.

    ``splits`` maps format name -> number of channels, consumed in the order NVFP4, FP8,
    FP16; each group is flattened before encoding, so NVFP4 blocks run along k and an FP8
    group shares one scale (rdquant/quantize.py:247-262).
    """
    n_out, n_in = weight.shape
    perm = permutation.to(torch.long)
    if sum(splits.get(f, 0) for f in FORMAT_ORDER) != n_out:
        raise ValueError("splits must sum to the number of output channels")
    grouped = weight[perm]
    qtensors = {}
    ordered = {}
    start = 0
    bits = 0
    for fmt in FORMAT_ORDER:
        n = int(splits.get(fmt, 0))
        if fmt in splits:
            ordered[fmt] = n
        if n == 0:
            continue
        q = quantize(grouped[start:start + n].reshape(-1).float(), fmt)
        qtensors[fmt] = QuantizedTensor(q.data, q.scales, fmt, torch.Size([n, n_in]), q.bits_per_element,
                                        q.global_scale)
        bits += get_bits_per_element(fmt) * n
        start += n
    return QuantizedWeight(
        qtensors=qtensors,
        permutation=perm.clone(),
        inv_permutation=inverse_permutation(perm),
        splits=ordered,
        original_shape=weight.shape,
        avg_bits=bits / max(n_out, 1),
    )


def quantize_weight_packed(weight: torch.Tensor, permutation: torch.Tensor, splits: dict, bias=None) -> dict:
    """GPU fast path of ``pack_layer(quantize_weight(...))``: the checkpoint tensors of one layer
    straight from a CUDA weight ``[N, K]`` (K % 16 == 0), encoded by the CUDA encoders.

    Byte-identical to the host route (rdquant/quantize.py:233-280 followed by
    rdquant/integrations/hf_export.py:58-125); tensors stay on the weight's device.
    """
    from rdquant_b200 import rdquant_cuda

    if not weight.is_cuda:
        raise RuntimeError("quantize_weight_packed runs on CUDA tensors only")
    n_out, n_in = weight.shape
    perm = permutation.to(device=weight.device, dtype=torch.long)
    if sum(splits.get(f, 0) for f in FORMAT_ORDER) != n_out:
        raise ValueError("splits must sum to the number of output channels")
    grouped = weight[perm]
    if grouped.dtype not in (torch.float16, torch.float32):
        grouped = grouped.float()
    out = {
        "splits": torch.tensor([int(splits.get(f, 0)) for f in FORMAT_ORDER], dtype=torch.int32),
        "inv_permutation": inverse_permutation(perm).to(torch.int32),
    }
    start = 0
    for fmt in FORMAT_ORDER:
        n = int(splits.get(fmt, 0))
        if n == 0:
            continue
        rows = grouped[start:start + n]
        if fmt == "NVFP4":
            enc = rdquant_cuda.quantize_nvfp4_packed(rows)
            out["weight_nvfp4"] = enc["weight_nvfp4"]
            out["weight_nvfp4_scale"] = enc["weight_nvfp4_scale"]
            top = enc["global_scale"]
            out["nvfp4_global_scale"] = torch.where(top == 0, torch.ones_like(top), top)
        elif fmt == "FP8":
            enc = rdquant_cuda.quantize_fp8_packed(rows)
            out["weight_fp8"] = enc["weight_fp8"]
            out["weight_fp8_scale"] = enc["weight_fp8_scale"]
        else:
            out["weight_fp16"] = rows.float().to(torch.float16).to(torch.bfloat16)
        start += n
    if bias is not None:
        out["bias"] = bias.detach().clone()
    return out


class QuantizedLayer(nn.Module):
    """``nn.Linear`` replacement holding a :class:`QuantizedWeight`
    (reference: rdquant/quantize.py:76-135)."""

    def __init__(self, quantized_weight: QuantizedWeight, bias: Optional[torch.Tensor],
                 in_features: int, out_features: int) -> None:
        super().__init__()
        self.quantized_weight = quantized_weight
        self.in_features = in_features
        self.out_features = out_features
        self.bias = nn.Parameter(bias.clone()) if bias is not None else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from rdquant_b200.ops import mixed_precision_linear

        qw = self.quantized_weight
        return mixed_precision_linear(x, qw.qtensors, qw.splits, qw.inv_permutation, self.bias)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"avg_bits={self.quantized_weight.avg_bits:.2f}")


class QuantizedModel(nn.Module):
    """Thin wrapper: ``.model`` holds the module tree with :class:`QuantizedLayer` leaves
    (reference: rdquant/quantize.py:137-226)."""

    def __init__(self, model: nn.Module, layer_info: Optional[dict] = None, formats=None,
                 budget_avg_bits: float = 0.0) -> None:
        super().__init__()
        self.model = model
        self.layer_info = layer_info or {}
        self.formats = list(formats) if formats is not None else list(FORMAT_ORDER)
        self.budget_avg_bits = budget_avg_bits

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def save_packed(self, path: str, source_model_dir: Optional[str] = None) -> None:
        from rdquant_b200.integrations.hf_export import save_packed

        save_packed(self, path, source_model_dir)
