"""Packed safetensors checkpoint of a mixed-precision model (the on-disk contract).

Layout, byte for byte that of the reference (rdquant/integrations/hf_export.py:58-125,
:149-169).  For every quantised layer with prefix ``P``:

    P.splits              int32 [3]        channels per format (NVFP4, FP8, FP16)
    P.inv_permutation     int32 [N]
    P.weight_nvfp4        uint8 [n4, K/2]  byte = code[2j+1] << 4 | code[2j]
    P.weight_nvfp4_scale  uint8 [n4, K/16] E4M3 bits
    P.nvfp4_global_scale  float32 [1]
    P.weight_fp8          uint8 [n8, K]    E4M3 bits
    P.weight_fp8_scale    float32 [n8]     (group scale broadcast to every channel)
    P.weight_fp16         bfloat16 [n16, K]
    P.bias                optional, original channel order

rows in permuted (format-grouped) order; a group with no channels has no keys.  All
other parameters are stored as float16, buffers unchanged.  ``quantization_config.json``
carries ``quant_method``, ``formats``, ``budget_avg_bits``, ``format_order`` and per
layer ``in_features / out_features / splits / avg_bits``.
"""
from __future__ import annotations

import json
import os
import shutil

import torch

from rdquant_b200.core.formats import NVFP4_BLOCK, QuantizedTensor, e4m3_bytes, pack_nvfp4_codes
from rdquant_b200.quantize import FORMAT_ORDER, QuantizedLayer, QuantizedModel, QuantizedWeight

_SIDE_FILES = (
    "config.json", "tokenizer.json", "tokenizer_config.json", "special_tokens_map.json",
    "tokenizer.model", "vocab.json", "merges.txt", "added_tokens.json", "generation_config.json",
)


def _is_quantized_layer(module) -> bool:
    # duck-typed so that the reference's own QuantizedLayer objects are accepted too
    return hasattr(module, "quantized_weight") and hasattr(module.quantized_weight, "qtensors")


def pack_layer(qw, bias=None) -> dict:
    """Checkpoint tensors (without prefix) of one quantised layer."""
    n_out, n_in = qw.original_shape
    out = {
        "splits": torch.tensor([int(qw.splits.get(f, 0)) for f in FORMAT_ORDER], dtype=torch.int32),
        "inv_permutation": qw.inv_permutation.to(torch.int32).cpu(),
    }
    for fmt, qt in qw.qtensors.items():
        n = int(qw.splits.get(fmt, 0))
        if n == 0:
            continue
        if fmt == "NVFP4":
            if n_in % NVFP4_BLOCK:
                raise ValueError("packed NVFP4 needs in_features % 16 == 0")
            out["weight_nvfp4"] = pack_nvfp4_codes(qt.data.reshape(n, n_in)).cpu()
            out["weight_nvfp4_scale"] = e4m3_bytes(qt.scales.reshape(n, n_in // NVFP4_BLOCK)).cpu()
            gs = qt.global_scale if qt.global_scale is not None else 1.0
            out["nvfp4_global_scale"] = torch.tensor([gs], dtype=torch.float32)
        elif fmt == "FP8":
            out["weight_fp8"] = e4m3_bytes(qt.data.reshape(n, n_in)).cpu()
            out["weight_fp8_scale"] = torch.full((n,), float(qt.scales.reshape(-1)[0].item()), dtype=torch.float32)
        elif fmt == "FP16":
            out["weight_fp16"] = qt.data.reshape(n, n_in).to(torch.bfloat16).cpu()
        else:
            raise KeyError(f"format {fmt!r} has no packed layout")
    if bias is not None:
        out["bias"] = bias.detach().clone().cpu()
    return out


def save_packed(model, path: str, source_model_dir: str | None = None) -> None:
    """Write ``model.safetensors`` + ``quantization_config.json`` into ``path``."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    tensors: dict[str, torch.Tensor] = {}
    layers: dict[str, dict] = {}
    for name, module in model.model.named_modules():
        if not _is_quantized_layer(module):
            continue
        qw = module.quantized_weight
        bias = module.bias.data if getattr(module, "bias", None) is not None else None
        for key, value in pack_layer(qw, bias).items():
            tensors[f"{name}.{key}"] = value.contiguous()
        n_out, n_in = qw.original_shape
        layers[name] = {
            "in_features": int(n_in),
            "out_features": int(n_out),
            "splits": {f: int(qw.splits.get(f, 0)) for f in FORMAT_ORDER},
            "avg_bits": qw.avg_bits,
        }

    def _inside_quantized(pname: str) -> bool:
        return any(pname.startswith(layer + ".") for layer in layers)

    for pname, param in model.model.named_parameters():
        if not _inside_quantized(pname) and pname not in tensors:
            tensors[pname] = param.data.to(torch.float16).contiguous().cpu()
    for bname, buf in model.model.named_buffers():
        if not _inside_quantized(bname) and bname not in tensors:
            tensors[bname] = buf.contiguous().cpu()

    save_file(tensors, os.path.join(path, "model.safetensors"))

    config = {
        "quant_method": "rdquant",
        "formats": list(getattr(model, "formats", FORMAT_ORDER)),
        "budget_avg_bits": getattr(model, "budget_avg_bits", 0.0),
        "format_order": list(FORMAT_ORDER),
        "layers": layers,
    }
    info = getattr(model, "layer_info", None)
    if info:
        config["layer_info"] = {
            lname: {
                "splits": dict(res.splits),
                "avg_bits": res.avg_bits,
                "total_distortion": getattr(res, "total_distortion", 0.0),
                "lambda_star": getattr(res, "lambda_star", 0.0),
            }
            for lname, res in info.items()
        }
    with open(os.path.join(path, "quantization_config.json"), "w") as fh:
        json.dump(config, fh, indent=2)

    if source_model_dir and os.path.isdir(source_model_dir):
        for fname in _SIDE_FILES:
            src = os.path.join(source_model_dir, fname)
            if os.path.isfile(src):
                shutil.copy2(src, os.path.join(path, fname))


TILED_FILE = "model.tiled.safetensors"
TILED_LAYOUT = "rdq_b200_tiled_v1"


def save_tiled_layout(path: str, device: str = "cuda") -> dict:
    """Add the decode kernel's in-memory tiling to a packed checkpoint, so that loading it is a
    plain upload with no re-tiling pass.

    For every quantised layer whose shape has a tiled layout, the image stream
    ``rdq_gemv_repack`` produces (include/rdq_b200.h) is written as ``<layer>.weight_tiled``
    (uint8) into ``model.tiled.safetensors`` next to ``model.safetensors``; the latter is not
    touched, so the checkpoint still round-trips through the reference's ``load_packed``
    (rdquant/integrations/hf_export.py:199-375).  The file's metadata names the layout version;
    :func:`rdquant_b200.inference.load_for_inference` ignores a file of another version or a
    tensor whose size does not match ``rdq_gemv_tiled_bytes``.  Needs a CUDA device (the tiling
    is produced by the device kernel).  Returns ``{"layers": count, "bytes": total}``.
    """
    from safetensors.torch import save_file

    from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv

    config, tensors = read_layers(path)
    out: dict[str, torch.Tensor] = {}
    for name, lconf in config["layers"].items():
        pre = name + "."
        layer_data = {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}
        fd = pack_for_fused_gemv(layer_data, lconf["splits"], lconf["in_features"], device)
        if fd is None:
            raise RuntimeError("save_tiled_layout needs the built rdquant_b200 kernels and a CUDA device")
        if fd.get("w_tiled") is not None:
            out[pre + "weight_tiled"] = fd["w_tiled"].cpu().contiguous()
        del fd
    save_file(out, os.path.join(path, TILED_FILE), metadata={"layout": TILED_LAYOUT})
    return {"layers": len(out), "bytes": int(sum(t.numel() for t in out.values()))}


def read_tiled_layout(path: str) -> dict:
    """``{tensor name: uint8 tensor}`` of ``model.tiled.safetensors`` (empty when the file is
    absent or of another layout version)."""
    from safetensors import safe_open

    fname = os.path.join(path, TILED_FILE)
    if not os.path.isfile(fname):
        return {}
    out = {}
    with safe_open(fname, framework="pt", device="cpu") as fh:
        if (fh.metadata() or {}).get("layout") != TILED_LAYOUT:
            return {}
        for key in fh.keys():
            out[key] = fh.get_tensor(key)
    return out


def unpack_nvfp4_codes(packed: torch.Tensor) -> torch.Tensor:
    """[n, K/2] uint8 -> [n, K] int64 codes (low nibble = even k)."""
    n, half = packed.shape
    codes = torch.empty(n, half * 2, dtype=torch.int64, device=packed.device)
    codes[:, 0::2] = (packed & 0x0F).to(torch.int64)
    codes[:, 1::2] = (packed >> 4).to(torch.int64)
    return codes


def read_layers(path: str, device: str = "cpu"):
    """(quantization config, {tensor name: tensor}) of a packed checkpoint."""
    from safetensors import safe_open

    with open(os.path.join(path, "quantization_config.json")) as fh:
        config = json.load(fh)
    tensors = {}
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device=device) as fh:
        for key in fh.keys():
            tensors[key] = fh.get_tensor(key)
    return config, tensors


def qweight_from_layer_data(layer_data: dict, splits: dict, n_in: int, avg_bits: float = 0.0) -> QuantizedWeight:
    """Rebuild the in-memory representation of one layer from its checkpoint tensors
    (rdquant/integrations/hf_export.py:233-325)."""
    inv = layer_data["inv_permutation"].to(torch.int64)
    n_out = inv.numel()
    perm = torch.empty_like(inv)
    perm[inv] = torch.arange(n_out, dtype=torch.int64, device=inv.device)
    qts = {}
    n4, n8, n16 = (int(splits.get(f, 0)) for f in FORMAT_ORDER)
    if n4:
        codes = unpack_nvfp4_codes(layer_data["weight_nvfp4"]).reshape(-1)
        sc = layer_data["weight_nvfp4_scale"].view(torch.float8_e4m3fn).to(torch.float32).reshape(-1)
        gs = float(layer_data["nvfp4_global_scale"].item()) if "nvfp4_global_scale" in layer_data else 1.0
        qts["NVFP4"] = QuantizedTensor(codes, sc, "NVFP4", torch.Size([n4, n_in]), 4, gs)
    if n8:
        vals = layer_data["weight_fp8"].view(torch.float8_e4m3fn).to(torch.float32).reshape(-1)
        # the in-memory FP8 format has a single group scale: element 0 of the stored vector
        qts["FP8"] = QuantizedTensor(vals, layer_data["weight_fp8_scale"][0:1].clone(), "FP8",
                                     torch.Size([n8, n_in]), 8)
    if n16:
        qts["FP16"] = QuantizedTensor(layer_data["weight_fp16"].to(torch.float16).reshape(-1),
                                      torch.empty(0, dtype=torch.float32), "FP16", torch.Size([n16, n_in]), 16)
    return QuantizedWeight(qts, perm, inv, {f: int(splits.get(f, 0)) for f in FORMAT_ORDER},
                           torch.Size([n_out, n_in]), avg_bits)


class _LayerContainer(torch.nn.Module):
    """Holds loaded layers under their dotted checkpoint names."""

    def __init__(self, layers: dict) -> None:
        super().__init__()
        self._names = {}
        for name, layer in layers.items():
            safe = name.replace(".", "__")
            self._names[safe] = name
            self.add_module(safe, layer)

    def named_modules(self, memo=None, prefix: str = "", remove_duplicate: bool = True):
        yield prefix, self
        for safe, mod in self._modules.items():
            yield self._names.get(safe, safe), mod

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for safe, mod in self._modules.items():
            for pname, p in mod.named_parameters():
                yield f"{self._names.get(safe, safe)}.{pname}", p

    def get_layer(self, name: str):
        return self._modules[name.replace(".", "__")]


def load_packed(path: str, device: str = "cpu") -> QuantizedModel:
    """Load a packed checkpoint into :class:`QuantizedModel` of :class:`QuantizedLayer`."""
    config, tensors = read_layers(path, device)
    layers = {}
    for name, lconf in config["layers"].items():
        pre = name + "."
        layer_data = {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}
        qw = qweight_from_layer_data(layer_data, lconf["splits"], lconf["in_features"], lconf.get("avg_bits", 0.0))
        layers[name] = QuantizedLayer(qw, layer_data.get("bias"), lconf["in_features"], lconf["out_features"])
    return QuantizedModel(_LayerContainer(layers), layer_info={},
                          formats=config.get("formats", list(FORMAT_ORDER)),
                          budget_avg_bits=config.get("budget_avg_bits", 0.0))
