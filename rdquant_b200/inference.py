"""Inference modules over the fused kernels (reference: rdquant/inference.py).

``FusedMixedLinear`` keeps the constructor and attributes of the reference module
(rdquant/inference.py:408-512) and ``load_for_inference`` its signature (:715-722).  Both
decode (M <= 16, one GEMV launch) and prefill (tcgen05 GEMM) run from the packed tensors;
no dequantised FP16 copy of the weights is kept, so ``use_dense_prefill`` costs no memory.
"""
from __future__ import annotations

import json
import time
import os
from typing import Optional

import torch
import torch.nn as nn

from rdquant_b200 import _lib
from rdquant_b200.fused_gemv_pack import (
    build_marlin_data,
    fused_gemv_available,
    get_rdquant_cuda,
    pack_for_fused_gemv,
)

_FD_TENSORS = ("w_fp4_q", "w_fp4_scales", "w_fp8_q", "w_fp8_scales", "w_fp16", "w_tiled", "perm", "inv_perm",
               "workspace", "tile_counters")


def _normalize_torch_dtype(dtype_like) -> torch.dtype:
    if isinstance(dtype_like, torch.dtype):
        return dtype_like
    table = {"float16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16,
             "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if isinstance(dtype_like, str):
        return table.get(dtype_like.lower(), torch.bfloat16)
    return torch.bfloat16


def _materialize_packed_groups(layer_data: dict, splits: dict, n_in: int) -> dict:
    """Dequantised FP16 groups in permuted order (rdquant/inference.py:67-121), computed by
    the dequantisation kernel; tensors must already be on a CUDA device."""
    cuda = get_rdquant_cuda()
    out = {"w_nvfp4": None, "w_fp8": None, "w_fp16": None}
    for fmt, key in (("NVFP4", "w_nvfp4"), ("FP8", "w_fp8"), ("FP16", "w_fp16")):
        if int(splits.get(fmt, 0)) > 0:
            only = {f: (int(splits[f]) if f == fmt else 0) for f in ("NVFP4", "FP8", "FP16")}
            out[key] = cuda.dequantize_packed(layer_data, only, n_in, inv_perm=None)
    return out


class FusedMixedLinear(nn.Module):
    """Packed mixed-precision linear: fused GEMV for decode, tcgen05 GEMM for prefill."""

    def __init__(
        self,
        *,
        n_nvfp4: int,
        n_fp8: int,
        n_fp16: int,
        k: int,
        inv_perm: torch.Tensor,
        bias: Optional[torch.Tensor],
        marlin_data: Optional[dict] = None,
        fused_data: Optional[dict] = None,
        w_fp16_fp16: Optional[torch.Tensor] = None,
        w_prefill_fp16: Optional[torch.Tensor] = None,
    ) -> None:
        super().__init__()
        self.n_nvfp4, self.n_fp8, self.n_fp16 = int(n_nvfp4), int(n_fp8), int(n_fp16)
        self.N = self.n_nvfp4 + self.n_fp8 + self.n_fp16
        self.K = int(k)
        self.register_buffer("inv_perm", inv_perm.to(torch.int64))
        self.register_buffer("_inv_perm_i32", inv_perm.to(torch.int32))
        self.bias = nn.Parameter(bias.clone()) if bias is not None else None
        # marlin_data / w_fp16_fp16 / w_prefill_fp16 belong to the reference's fallback paths
        # and are accepted but unused: every shape runs from the packed buffers.
        self._has_marlin = False
        self._has_fused = fused_data is not None
        self.use_pdl = False
        self._fd_scalars = {}
        if fused_data is not None:
            if (fused_data["n_fp4"], fused_data["n_fp8"], fused_data["n_fp16"], fused_data["k"]) != (
                    self.n_nvfp4, self.n_fp8, self.n_fp16, self.K):
                raise ValueError("fused_data does not match the layer's group sizes / K")
            for name in _FD_TENSORS:
                t = fused_data.get(name)
                if t is not None:
                    self.register_buffer(f"_fused_{name}", t, persistent=False)
            self._fd_scalars = {kk: v for kk, v in fused_data.items() if kk not in _FD_TENSORS}
        self._fd_cache = None
        self._bias_h = None

    def _apply(self, fn, recurse=True):
        self._fd_cache = None
        self._bias_h = None
        return super()._apply(fn, recurse)

    def _fd(self) -> dict:
        if self._fd_cache is None:
            fd = dict(self._fd_scalars)
            for name in _FD_TENSORS:
                fd[name] = getattr(self, f"_fused_{name}", None)
            self._fd_cache = fd
        return self._fd_cache

    def _can_use_fused(self, x_2d: torch.Tensor) -> bool:
        return self._has_fused and x_2d.is_cuda

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        orig_shape = x.shape
        x_2d = x.reshape(-1, self.K)
        if not self._can_use_fused(x_2d):
            raise RuntimeError("No compatible fused backend available (needs CUDA tensors and packed buffers)")
        cuda = get_rdquant_cuda()
        x_half = x_2d if x_2d.dtype == torch.float16 else x_2d.half()
        x_half = x_half.contiguous()
        bias_h = None
        if self.bias is not None:
            if self._bias_h is None or self._bias_h.device != x.device:
                self._bias_h = self.bias.detach().to(device=x.device, dtype=torch.float16).contiguous()
            bias_h = self._bias_h
        flags = _lib.RDQ_GEMV_PDL if self.use_pdl else 0
        y = cuda.mixed_linear(x_half, self._fd(), bias_h, flags)
        return y.to(x.dtype).reshape(*orig_shape[:-1], self.N)

    def extra_repr(self) -> str:
        return f"K={self.K}, N={self.N}, nvfp4/fp8/fp16={self.n_nvfp4}/{self.n_fp8}/{self.n_fp16}"

    @classmethod
    def from_layer_data(cls, layer_data: dict, splits: dict, k: int, device, row_major: bool = True) -> "FusedMixedLinear":
        fd = pack_for_fused_gemv(layer_data, dict(splits), k, device, row_major=row_major)
        if fd is None:
            raise RuntimeError("rdquant_b200 kernels unavailable: build librdq_b200.so and run on a CUDA device")
        bias = layer_data.get("bias")
        return cls(n_nvfp4=fd["n_fp4"], n_fp8=fd["n_fp8"], n_fp16=fd["n_fp16"], k=k,
                   inv_perm=fd["inv_perm"], bias=bias.to(device) if bias is not None else None,
                   marlin_data=None, fused_data=fd)


class GraphedDecodeStep:
    """One decode step over several packed linears as a single CUDA-graph replay.

    The graph holds, for every layer, the copy of its activation rows from a pinned host
    buffer to the device, the fused GEMV (programmatic dependent launch between layers) and
    the copy of the result to a pinned host buffer.  ``run()`` replays it and waits for the
    results, so a caller holding host-side activations pays one launch per step instead of
    three calls per layer.  The wait is a poll of a word in pinned host memory that the last
    copy kernel writes behind its data (``poll=False``: a stream synchronisation).  (The reference's end-to-end timings rely on CUDA-graph capture
    of the decode step the same way, benchmarks/bench_e2e.py:103-155.)
    """

    def __init__(self, modules, m: int = 1, use_pdl: bool = True, poll: bool = True) -> None:
        self.modules = list(modules)
        self.poll = poll
        dev = self.modules[0].inv_perm.device
        # one pinned staging buffer each way: a single copy node per direction in the graph
        ks = [m * mod.K for mod in self.modules]
        ns = [m * mod.N for mod in self.modules]
        self._x_all_host = torch.zeros(sum(ks), dtype=torch.float16).pin_memory()
        self._y_all_host = torch.zeros(sum(ns), dtype=torch.float16).pin_memory()
        self._x_all_dev = torch.zeros(sum(ks), dtype=torch.float16, device=dev)
        self._y_all_dev = torch.zeros(sum(ns), dtype=torch.float16, device=dev)

        def views(flat, sizes, cols):
            out, off = [], 0
            for sz, c in zip(sizes, cols):
                out.append(flat[off:off + sz].view(m, c))
                off += sz
            return out

        self.x_host = views(self._x_all_host, ks, [mod.K for mod in self.modules])
        self.y_host = views(self._y_all_host, ns, [mod.N for mod in self.modules])
        self._x_dev = views(self._x_all_dev, ks, [mod.K for mod in self.modules])
        self._y_dev = views(self._y_all_dev, ns, [mod.N for mod in self.modules])
        self._stream = torch.cuda.Stream(dev)
        self._graph = torch.cuda.CUDAGraph()
        cuda = get_rdquant_cuda()
        flags = _lib.RDQ_GEMV_PDL if use_pdl else 0
        biases = [mod.bias.detach().to(device=dev, dtype=torch.float16).contiguous() if mod.bias is not None else None
                  for mod in self.modules]

        def body():
            # staging by kernel: the GPU reads / writes the pinned buffers over PCIe itself
            # (a memcpy node would add ~10 us of fixed latency each way)
            cuda.stage_copy(self._x_all_dev, self._x_all_host)
            for i, mod in enumerate(self.modules):
                cuda.mixed_gemv(self._x_dev[i], mod._fd(), biases[i], flags, out=self._y_dev[i])
            if self.poll:
                cuda.stage_copy(self._y_all_host, self._y_all_dev, self._done_state, self._done_flag)
            else:
                cuda.stage_copy(self._y_all_host, self._y_all_dev)

        self._done_state = torch.zeros(2, dtype=torch.int32, device=dev)
        self._done_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._done_view = self._done_flag.numpy()
        self._launches = 0
        with torch.cuda.stream(self._stream):
            body()  # first calls outside capture (library set-up, lazy module loading)
            self._launches += 1
            self._stream.synchronize()
            with torch.cuda.graph(self._graph, stream=self._stream):
                body()

    def run(self):
        """Replay: ``x_host`` -> device -> linears -> ``y_host``; returns ``y_host`` when complete."""
        self._graph.replay()  # on the caller's current stream
        self._launches += 1
        if self.poll:
            # the copy kernel writes the launch count behind its data (system-scope release)
            view, want = self._done_view, self._launches
            deadline = None
            while int(view[0]) != want:
                if deadline is None:
                    deadline = time.monotonic() + 10.0
                elif time.monotonic() > deadline:
                    torch.cuda.current_stream(self._x_all_dev.device).synchronize()
                    raise RuntimeError(f"decode step did not signal completion (flag {int(view[0])}, expected {want})")
        else:
            torch.cuda.current_stream(self._x_all_dev.device).synchronize()
        return self.y_host


# The grouped two-launch module of the reference (rdquant/inference.py:144-391) has the same
# contract; one class serves both names.
MarlinMixedLinear = FusedMixedLinear


def _set_module(model: nn.Module, name: str, new_module: nn.Module) -> None:
    parts = name.split(".")
    parent = model
    for part in parts[:-1]:
        parent = getattr(parent, part)
    setattr(parent, parts[-1], new_module)


def replace_quantized_layers(model: nn.Module, layer_configs: dict, tensors: dict, device, row_major: bool = True) -> None:
    """Install a :class:`FusedMixedLinear` for every layer of ``layer_configs``."""
    for layer_name, lconf in layer_configs.items():
        pre = layer_name + "."
        layer_data = {k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)}
        mod = FusedMixedLinear.from_layer_data(layer_data, lconf["splits"], lconf["in_features"], device, row_major=row_major)
        _set_module(model, layer_name, mod)


def load_for_inference(
    checkpoint_dir: str,
    model_class=None,
    device: str = "cuda",
    use_marlin: bool = True,
    use_fused_gemv: bool = True,
    use_dense_prefill: bool = True,
    decode_only: bool = False,
) -> nn.Module:
    """Load a packed checkpoint into a HuggingFace model whose quantised linears are
    :class:`FusedMixedLinear`.

    ``use_marlin`` / ``use_fused_gemv`` / ``use_dense_prefill`` are accepted for signature
    parity (rdquant/inference.py:715-722); the fused kernels serve decode and prefill alike.
    ``decode_only=True`` keeps only the decode kernel's tiled copy of every layer on the device
    (half the weight memory; the reference's dense prefill instead adds an FP16 copy,
    rdquant/inference.py:742-744): prompts then run as 16-row panels of the decode kernel.
    """
    from safetensors import safe_open
    from transformers import AutoConfig, AutoModelForCausalLM

    target = torch.device(device)
    if target.type != "cuda" or not fused_gemv_available():
        raise RuntimeError("load_for_inference needs a CUDA device and the built rdquant_b200 kernels")
    if model_class is None:
        model_class = AutoModelForCausalLM

    with open(os.path.join(checkpoint_dir, "quantization_config.json")) as fh:
        qconfig = json.load(fh)
    layer_configs = qconfig["layers"]

    config = AutoConfig.from_pretrained(checkpoint_dir)
    model_dtype = _normalize_torch_dtype(getattr(config, "torch_dtype", None) or getattr(config, "dtype", torch.bfloat16))
    with torch.device("meta"):
        model = model_class.from_config(config)
    model = model.to_empty(device="cpu")
    model.eval()

    tensors: dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(checkpoint_dir, "model.safetensors"), framework="pt", device="cpu") as fh:
        for key in fh.keys():
            tensors[key] = fh.get_tensor(key)

    # the decode kernel's tiling, when the checkpoint carries it (hf_export.save_tiled_layout)
    from rdquant_b200.integrations.hf_export import read_tiled_layout

    tensors.update(read_tiled_layout(checkpoint_dir))
    replace_quantized_layers(model, layer_configs, tensors, target, row_major=not decode_only)

    quant_layers = tuple(name + "." for name in layer_configs)
    for pname, param in model.named_parameters():
        if not pname.startswith(quant_layers) and pname in tensors:
            param.data.copy_(tensors[pname].to(param.dtype))
    for bname, buf in model.named_buffers():
        if not bname.startswith(quant_layers) and bname in tensors:
            buf.copy_(tensors[bname].to(buf.dtype))

    if getattr(config, "tie_word_embeddings", False):
        if hasattr(model, "lm_head") and hasattr(model, "model") and hasattr(model.model, "embed_tokens"):
            model.lm_head.weight = model.model.embed_tokens.weight

    model = model.to(device)
    model.eval()
    del model_dtype
    return model
