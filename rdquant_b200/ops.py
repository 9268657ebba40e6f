"""Functional mixed-precision linear operator (reference: rdquant/ops.py:32-68).

``mixed_precision_linear(x, qtensors, splits, inv_perm, bias)`` computes what the reference
computes with per-group dequantise -> ``F.linear`` -> ``cat`` -> ``index_select`` -> ``+bias``,
but as one fused CUDA launch (GEMV for up to 16 rows, tcgen05 GEMM above) that writes
straight to original channel order.  CUDA only; there is no host path.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch

from rdquant_b200.core.formats import QuantizedTensor

_PACK_CACHE: "OrderedDict[int, tuple]" = OrderedDict()
_PACK_CACHE_MAX = 128  # packed layers kept alive for reuse (each entry also pins its qtensors dict)


def _packed_for(qtensors: dict, splits: dict, inv_perm: torch.Tensor, device: torch.device) -> dict:
    """Pack ``qtensors`` once per (dict object, device); later calls reuse the device buffers."""
    from rdquant_b200.core.formats import qtensor_to_packed
    from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv

    key = (id(qtensors), device.index)
    hit = _PACK_CACHE.get(key)
    if hit is not None and hit[0] is qtensors and hit[1] is inv_perm:
        _PACK_CACHE.move_to_end(key)
        return hit[2]
    layer_data = {"inv_permutation": inv_perm}
    k = None
    for fmt, qt in qtensors.items():
        if int(splits.get(fmt, 0)) == 0:
            continue
        layer_data.update(qtensor_to_packed(qt))
        k = int(qt.original_shape[-1])
    if k is None:
        raise RuntimeError("mixed_precision_linear: no non-empty format group")
    fd = pack_for_fused_gemv(layer_data, splits, k, device)
    if fd is None:
        raise RuntimeError("rdquant_b200 kernels unavailable: build librdq_b200.so and run on a CUDA device")
    _PACK_CACHE[key] = (qtensors, inv_perm, fd)
    while len(_PACK_CACHE) > _PACK_CACHE_MAX:
        _PACK_CACHE.popitem(last=False)
    return fd


def mixed_precision_linear(
    x: torch.Tensor,
    qtensors: dict,
    splits: dict,
    inv_perm: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``[..., K] -> [..., N]`` in ``x.dtype``; ``y[..., j] = y_perm[..., inv_perm[j]] + bias[j]``.

    Computation is float16 inputs with FP32 accumulation (``x`` of another dtype is cast to
    float16 and the result cast back, as ``FusedMixedLinear`` does,
    rdquant/inference.py:696, :707).
    """
    from rdquant_b200 import rdquant_cuda

    if not x.is_cuda:
        raise RuntimeError("rdquant_b200.ops.mixed_precision_linear runs on CUDA tensors only (no host path)")
    fd = _packed_for(qtensors, splits, inv_perm, x.device)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    xh = x2 if x2.dtype == torch.float16 else x2.to(torch.float16)
    xh = xh.contiguous()
    bh = None
    if bias is not None:
        bh = bias.to(device=x.device, dtype=torch.float16).contiguous()
    y = rdquant_cuda.mixed_linear(xh, fd, bh)
    n = fd["n_fp4"] + fd["n_fp8"] + fd["n_fp16"]
    return y.to(x.dtype).reshape(*lead, n)


def mixed_precision_linear_vllm(x, qtensors, splits, inv_perm, bias=None):
    """Name kept for callers of rdquant/ops.py:183-228; runs the same fused kernels."""
    return mixed_precision_linear(x, qtensors, splits, inv_perm, bias)
