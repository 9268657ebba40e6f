"""Generate the golden fixtures of tests/golden/ by RUNNING THE REFERENCE PACKAGE.

Needs a checkout of the reference package, named by the environment variable
RDQUANT_REFERENCE; it is not needed to run the tests, only to regenerate the fixtures:

    RDQUANT_REFERENCE=<path to the RDQuant checkout> python tests/golden/make_golden.py

Writes
  tables.npz        E4M3 decode table from torch.float8_e4m3fn, the reference's NVFP4 LUT,
                    and float16 bits of every LUT[code] * e4m3(scale) product
  layers.npz        small layers: source weight, permutation, splits, the tensors the
                    reference's save_packed wrote, the reference's dequantised weight from
                    the in-memory payload (float32 and its float16 cast) and from the
                    checkpoint bytes (float16; the FP16 group passes through bfloat16
                    there), and the reference operator's output
  config1_alloc.npz permutation / splits chosen by the reference's Lagrangian allocator for
                    the K=2560, N=9728 layer at 5.3 average bits (seed 0), SHA-256 of the source
                    weight, of every tensor the reference's save_packed wrote for it and of its
                    dequantised weight, 24 rows of that weight, and the reference operator's
                    output for a seeded activation row
"""
import os
import sys
import tempfile

import numpy as np
import torch

REF = os.environ.get("RDQUANT_REFERENCE")
if not REF:
    raise SystemExit("set RDQUANT_REFERENCE to the RDQuant checkout the fixtures are generated from")
sys.path.insert(0, REF)

from rdquant.core import formats as rf  # noqa: E402
from rdquant.core.allocator import AllocationResult, allocate_layer  # noqa: E402
from rdquant.integrations.hf_export import save_packed  # noqa: E402
from rdquant.ops import mixed_precision_linear  # noqa: E402
from rdquant.quantize import QuantizedLayer, QuantizedModel, _quantize_weight  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ORDER = ["NVFP4", "FP8", "FP16"]


def tables():
    e4m3 = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn).to(torch.float32)
    lut = rf._NVFP4_LUT.clone()
    prod = (lut[:, None] * e4m3[None, :]).half()
    np.savez_compressed(os.path.join(HERE, "tables.npz"), e4m3_f32=e4m3.numpy(), nvfp4_lut=lut.numpy(),
                        products_f16_bits=prod.view(torch.int16).numpy().view(np.uint16))


def manual_alloc(n_out, splits, gen):
    perm = torch.randperm(n_out, generator=gen)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(n_out)
    return AllocationResult(assignments={}, permutation=perm, inv_permutation=inv,
                            splits={f: splits[f] for f in ORDER if f in splits}, avg_bits=0.0,
                            total_distortion=0.0, lambda_star=0.0, format_stats={})


def one_layer(name, n_out, n_in, splits, seed, with_bias, budget=None):
    gen = torch.Generator().manual_seed(seed)
    w = (torch.randn(n_out, n_in, generator=gen) * 0.02).half()
    idx = torch.randperm(n_out, generator=gen)[: max(n_out // 50, 1)]
    w[idx] *= 8
    if budget is not None:
        alloc = allocate_layer(w.float(), budget, ORDER)
    else:
        alloc = manual_alloc(n_out, splits, gen)
    qw = _quantize_weight(w.float(), alloc)
    bias = (torch.randn(n_out, generator=gen) * 0.1).half() if with_bias else None
    layer = QuantizedLayer(qw, bias, n_in, n_out)
    holder = torch.nn.Module()
    holder.add_module("fc", layer)
    qm = QuantizedModel(model=holder, layer_info={}, formats=ORDER, budget_avg_bits=0.0)
    from safetensors import safe_open
    with tempfile.TemporaryDirectory() as d:
        save_packed(qm, d)
        saved = {}
        with safe_open(os.path.join(d, "model.safetensors"), framework="pt", device="cpu") as fh:
            for key in fh.keys():
                saved[key] = fh.get_tensor(key)
    out = {f"{name}/weight_f16_bits": w.view(torch.int16).numpy().view(np.uint16),
           f"{name}/perm": alloc.permutation.numpy().astype(np.int32),
           f"{name}/splits": np.array([qw.splits.get(f, 0) for f in ORDER], dtype=np.int32)}
    for key, t in saved.items():
        short = key[len("fc."):]
        if t.dtype == torch.bfloat16:
            out[f"{name}/saved/{short}"] = t.view(torch.int16).numpy().view(np.uint16)
        elif t.dtype == torch.float16:
            out[f"{name}/saved/{short}"] = t.view(torch.int16).numpy().view(np.uint16)
        else:
            out[f"{name}/saved/{short}"] = t.numpy()
    from rdquant.inference import _materialize_packed_groups
    layer_data = {key[len("fc."):]: t for key, t in saved.items()}
    mat = _materialize_packed_groups(layer_data, {f: qw.splits.get(f, 0) for f in ORDER}, n_in)
    pieces = [mat[key] for key in ("w_nvfp4", "w_fp8", "w_fp16") if mat[key] is not None]
    w_packed = torch.cat(pieces, dim=0)[qw.inv_permutation]  # float16 [N, K] from the checkpoint bytes
    out[f"{name}/w_packed_f16_bits"] = w_packed.view(torch.int16).numpy().view(np.uint16)
    w_ref = qw.dequantize()  # float32 [N, K], original order, from the in-memory payload
    out[f"{name}/w_ref_f32"] = w_ref.numpy()
    out[f"{name}/w_ref_f16_bits"] = w_ref.half().view(torch.int16).numpy().view(np.uint16)
    for m in (1, 3):
        x = torch.randn(m, n_in, generator=gen).half()
        y = mixed_precision_linear(x, qw.qtensors, qw.splits, qw.inv_permutation, bias)
        out[f"{name}/x{m}_f16_bits"] = x.view(torch.int16).numpy().view(np.uint16)
        out[f"{name}/y{m}_ref_f16_bits"] = y.view(torch.int16).numpy().view(np.uint16)
    return out


def layers():
    cases = [
        ("mixed_256x128", 256, 128, {"NVFP4": 128, "FP8": 64, "FP16": 64}, 1, True, None),
        ("mixed_384x256", 384, 256, {"NVFP4": 128, "FP8": 128, "FP16": 128}, 2, False, None),
        ("fp4only_128x256", 128, 256, {"NVFP4": 128, "FP8": 0, "FP16": 0}, 3, False, None),
        ("fp8only_48x80", 48, 80, {"NVFP4": 0, "FP8": 48, "FP16": 0}, 4, True, None),
        ("fp16only_32x40", 32, 40, {"NVFP4": 0, "FP8": 0, "FP16": 32}, 5, False, None),
        ("alloc_96x64", 96, 64, None, 6, True, 6.0),
        ("alloc_512x256", 512, 256, None, 7, False, 5.3),
    ]
    out = {}
    for c in cases:
        out.update(one_layer(*c))
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **out)
    print({k: v.tolist() for k, v in out.items() if k.endswith("/splits")})


def _sha(t: torch.Tensor) -> np.ndarray:
    import hashlib

    raw = t.contiguous().view(torch.uint8).numpy().tobytes()
    return np.frombuffer(hashlib.sha256(raw).digest(), dtype=np.uint8).copy()


def config1():
    """BASELINE configs[0] at full size: K = 2560, N = 9728, seed 0, allocator at 5.3 bits.  The
    weight itself is regenerated from the seed by the tests; pinned here are its hash, the
    allocator's result, hashes of the reference's packed checkpoint tensors and of its
    dequantised weight, a few rows of that weight, and the reference operator's output."""
    g = torch.Generator().manual_seed(0)
    n, k = 9728, 2560
    w = (torch.randn(n, k, generator=g) * 0.02).half()
    idx = torch.randperm(n, generator=g)[: n // 100]
    w[idx] *= 8
    alloc = allocate_layer(w.float(), 5.3, ORDER)
    print("config1 splits", alloc.splits, "avg bits", alloc.avg_bits)
    qw = _quantize_weight(w.float(), alloc)
    x = torch.randn(1, k, generator=g).half()
    y = mixed_precision_linear(x, qw.qtensors, qw.splits, qw.inv_permutation, None)
    w_ref = qw.dequantize().half()  # [N, K] original order
    layer = QuantizedLayer(qw, None, k, n)
    holder = torch.nn.Module()
    holder.add_module("fc", layer)
    qm = QuantizedModel(model=holder, layer_info={}, formats=ORDER, budget_avg_bits=5.3)
    from safetensors import safe_open
    hashes = {}
    with tempfile.TemporaryDirectory() as d:
        save_packed(qm, d)
        with safe_open(os.path.join(d, "model.safetensors"), framework="pt", device="cpu") as fh:
            for key in fh.keys():
                t = fh.get_tensor(key)
                hashes["sha_" + key[len("fc."):]] = _sha(t)
    rows = np.linspace(0, n - 1, 24).astype(np.int64)
    np.savez_compressed(os.path.join(HERE, "config1_alloc.npz"), perm=alloc.permutation.numpy().astype(np.int32),
                        splits=np.array([alloc.splits.get(f, 0) for f in ORDER], dtype=np.int32),
                        avg_bits=np.float64(alloc.avg_bits), sha_weight_f16=_sha(w), sha_w_ref_f16=_sha(w_ref),
                        sample_rows=rows, w_ref_rows_f16_bits=w_ref[rows].view(torch.int16).numpy().view(np.uint16),
                        x_f16_bits=x.view(torch.int16).numpy().view(np.uint16),
                        y_ref_f16_bits=y.view(torch.int16).numpy().view(np.uint16), **hashes)


if __name__ == "__main__":
    tables()
    layers()
    config1()
