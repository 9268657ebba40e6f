"""Build the device buffers of the fused mixed-precision kernels from checkpoint tensors.

Same entry points as the reference (rdquant/fused_gemv_pack.py:37-57, :275-354).  The
prefill GEMM, the dequantiser and the any-shape GEMV consume the checkpoint's row-major
tensors as they are; the decode GEMV reads a re-tiled copy of them (taken from the checkpoint
when it carries one, else produced here), so "packing" is a device copy, that copy, the
derived output permutation and the decode kernel's scratch.
"""
from __future__ import annotations

from typing import Optional

import torch

from rdquant_b200 import _lib

FORMAT_ORDER = ("NVFP4", "FP8", "FP16")


def get_rdquant_cuda():
    """The module exposing the kernels (raises if the library has not been built)."""
    _lib.lib()
    from rdquant_b200 import rdquant_cuda

    return rdquant_cuda


def fused_gemv_available() -> bool:
    """True when ``librdq_b200.so`` is built and a CUDA device is present."""
    return _lib.available() and torch.cuda.is_available()


def choose_parallel_k(num_tiles: int, k: int) -> int:
    """Kept for signature parity (rdquant/fused_gemv_pack.py:60-63); the decode kernel
    balances k inside the launch, so there is no caller-visible split factor."""
    return 1


def layer_data_from_qweight(qw) -> dict:
    """Checkpoint-named packed tensors of a ``QuantizedWeight`` (on its own device)."""
    from rdquant_b200.core.formats import qtensor_to_packed

    data = {"inv_permutation": qw.inv_permutation.to(torch.int32)}
    for fmt, qt in qw.qtensors.items():
        if int(qw.splits.get(fmt, 0)) == 0:
            continue
        data.update(qtensor_to_packed(qt))
    return data


def validate_layer_data(layer_data: dict, splits: dict, k: int) -> tuple[int, int, int]:
    n4, n8, n16 = (int(splits.get(f, 0)) for f in FORMAT_ORDER)
    if min(n4, n8, n16) < 0:
        raise ValueError("negative group size")
    if n4:
        if k % 16:
            raise ValueError(f"NVFP4 group needs K % 16 == 0, got {k}")
        if tuple(layer_data["weight_nvfp4"].shape) != (n4, k // 2):
            raise ValueError("weight_nvfp4 must be [n4, K/2]")
        if tuple(layer_data["weight_nvfp4_scale"].shape) != (n4, k // 16):
            raise ValueError("weight_nvfp4_scale must be [n4, K/16]")
    if n8:
        if tuple(layer_data["weight_fp8"].shape) != (n8, k):
            raise ValueError("weight_fp8 must be [n8, K]")
        if layer_data["weight_fp8_scale"].numel() != n8:
            raise ValueError("weight_fp8_scale must be [n8]")
    if n16 and tuple(layer_data["weight_fp16"].shape) != (n16, k):
        raise ValueError("weight_fp16 must be [n16, K]")
    if "inv_permutation" in layer_data and layer_data["inv_permutation"].numel() != n4 + n8 + n16:
        raise ValueError("inv_permutation must have N elements")
    return n4, n8, n16


def pack_for_fused_gemv(layer_data: dict, splits: dict, k: int, device,
                        honor_global_scale: bool = False, tiled: bool = True, row_major: bool = True) -> Optional[dict]:
    """Device buffers for ``rdquant_cuda.mixed_gemv`` / ``mixed_gemm``.

    Accepts any split (single-format layers, an FP16 group, groups below 128 channels);
    shapes without a tiled layout run on the any-shape kernel.  Returns ``None``
    only when the kernels are unavailable, like the reference
    (rdquant/fused_gemv_pack.py:289-290).

    ``row_major=False`` keeps only the re-tiled copy on the device when the shape has one
    (half the weight memory): the decode GEMV is unaffected, more than 16 rows then run as
    16-row panels of it instead of the tensor-core GEMM, and the dequantiser has no input.

    The NVFP4 block scales of a checkpoint are absolute, so the kernel's global-scale
    argument is 1.0 unless ``honor_global_scale`` asks for the stored value
    (rdquant/core/formats.py:145-159 never applies it).
    """
    if not fused_gemv_available():
        return None
    device = torch.device(device)
    n4, n8, n16 = validate_layer_data(layer_data, splits, k)
    n = n4 + n8 + n16
    from rdquant_b200 import rdquant_cuda

    def dev(t, dtype):
        return t.to(device=device, dtype=dtype).contiguous()

    if "inv_permutation" in layer_data:
        inv = dev(layer_data["inv_permutation"], torch.int32)
    else:
        inv = torch.arange(n, dtype=torch.int32, device=device)
    gs = 1.0
    if honor_global_scale and "nvfp4_global_scale" in layer_data:
        gs = float(layer_data["nvfp4_global_scale"].item())
    workspace, counters = rdquant_cuda.gemv_scratch(n, device)
    fd = {
        "w_fp4_q": dev(layer_data["weight_nvfp4"], torch.uint8) if n4 else None,
        "w_fp4_scales": dev(layer_data["weight_nvfp4_scale"], torch.uint8) if n4 else None,
        "w_fp4_global_scale": gs,
        "w_fp8_q": dev(layer_data["weight_fp8"], torch.uint8) if n8 else None,
        "w_fp8_scales": dev(layer_data["weight_fp8_scale"].reshape(-1), torch.float32) if n8 else None,
        # stored as bfloat16 on disk; the operator's weight is its float16 conversion
        "w_fp16": layer_data["weight_fp16"].to(device).to(torch.float16).contiguous() if n16 else None,
        "inv_perm": inv,
        "perm": rdquant_cuda.perm_from_inv_perm(inv),
        "workspace": workspace,
        "tile_counters": counters,
        "parallel_k": 1,
        "n_fp4": n4, "n_fp8": n8, "n_fp16": n16, "k": int(k),
    }
    # re-tiled copy for the fast decode kernel (None when the shape has no tiled layout): taken
    # from the checkpoint when it carries one of the right size
    # (integrations.hf_export.save_tiled_layout), else produced here
    fd["w_tiled"] = None
    if tiled:
        stored = layer_data.get("weight_tiled")
        need = rdquant_cuda.tiled_bytes(n4, n8, n16, int(k))
        if stored is not None and need and stored.dtype == torch.uint8 and stored.numel() == need:
            fd["w_tiled"] = stored.reshape(-1).to(device).contiguous()
            fd["tiled_from_checkpoint"] = True
        else:
            fd["w_tiled"] = rdquant_cuda.repack_tiled(fd)
    fd["row_major"] = True
    if not row_major and fd["w_tiled"] is not None:
        for key in ("w_fp4_q", "w_fp4_scales", "w_fp8_q", "w_fp16"):
            fd[key] = None
        fd["row_major"] = False
    return fd


def fuse_layers(layers: list) -> tuple:
    """Fuse linears that read the same input (q/k/v, gate/up) into one packed layer.

    ``layers`` is a list of ``(layer_data, splits)`` with equal ``in_features``.  The fused
    layer's output is the concatenation of the individual outputs in original channel
    order; its rows are the individual rows regrouped NVFP4 | FP8 | FP16.  One launch then
    streams all of them.  Returns ``(layer_data, splits)`` in checkpoint naming.
    """
    sizes = [[int(sp.get(f, 0)) for f in FORMAT_ORDER] for _, sp in layers]
    tot = [sum(sz[g] for sz in sizes) for g in range(3)]
    keys = (("weight_nvfp4", "weight_nvfp4_scale"), ("weight_fp8", "weight_fp8_scale"), ("weight_fp16",))
    fused = {}
    for g in range(3):
        for key in keys[g]:
            parts = [ld[key] for (ld, _), sz in zip(layers, sizes) if sz[g] > 0]
            if parts:
                fused[key] = torch.cat([p.reshape(p.shape[0], -1) if p.dim() > 1 else p for p in parts], dim=0)
    inv_parts = []
    base = [0, 0, 0]
    for (ld, _), sz in zip(layers, sizes):
        inv = ld["inv_permutation"].to(torch.int64)
        n4, n8, _n16 = sz
        pos = torch.where(inv < n4, inv + base[0],
                          torch.where(inv < n4 + n8, inv - n4 + tot[0] + base[1], inv - n4 - n8 + tot[0] + tot[1] + base[2]))
        inv_parts.append(pos)
        base = [base[g] + sz[g] for g in range(3)]
    fused["inv_permutation"] = torch.cat(inv_parts).to(torch.int32)
    if any("bias" in ld for ld, _ in layers):
        fused["bias"] = torch.cat([ld["bias"] if "bias" in ld else torch.zeros(sum(sz), dtype=torch.float16)
                                   for (ld, _), sz in zip(layers, sizes)])
    if "weight_nvfp4" in fused:
        fused["nvfp4_global_scale"] = torch.ones(1)
    return fused, dict(zip(FORMAT_ORDER, tot))


def packed_weight_bytes(splits: dict, k: int) -> int:
    """Weight + scale bytes one GEMV launch must read: the roofline numerator."""
    n4, n8, n16 = (int(splits.get(f, 0)) for f in FORMAT_ORDER)
    return n4 * (k // 2 + k // 16) + n8 * (k + 4) + n16 * 2 * k


def build_marlin_data(layer_data, splits, k, device):
    """The Marlin fallback buffers of the reference (rdquant/fused_gemv_pack.py:228-272)
    have no counterpart here: every shape runs on the fused kernels."""
    return None
