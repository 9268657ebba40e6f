"""The reference's import names resolve to this package, and objects produced by OTHER code with
the reference's field layout (its own ``_quantize_weight`` when a checkout is named by
RDQUANT_REFERENCE, or any look-alike) are accepted by the operator."""
import importlib
import os
import sys
import types

import numpy as np
import pytest
import torch

from conftest import ORDER, golden_layer_torch


def test_alias_modules():
    import rdquant
    import rdquant_cuda
    from rdquant.fused_gemv_pack import fused_gemv_available, get_rdquant_cuda, pack_for_fused_gemv  # noqa: F401
    from rdquant.inference import FusedMixedLinear, MarlinMixedLinear, load_for_inference  # noqa: F401
    from rdquant.integrations.hf_export import load_packed, save_packed  # noqa: F401
    from rdquant.ops import mixed_precision_linear, mixed_precision_linear_vllm  # noqa: F401

    import rdquant_b200.ops

    assert rdquant.ops is rdquant_b200.ops and rdquant.load_for_inference is load_for_inference
    assert importlib.import_module("rdquant.core.formats").QuantizedTensor is rdquant_b200.ops.QuantizedTensor
    assert hasattr(rdquant_cuda, "fused_mixed_gemv") and hasattr(rdquant_cuda, "mixed_gemv")


def _foreign(qt):
    """A payload object that is NOT this package's dataclass but has the reference's fields
    (rdquant/core/formats.py:28-36)."""
    return types.SimpleNamespace(data=qt.data, scales=qt.scales, format_name=qt.format_name,
                                 original_shape=qt.original_shape, bits_per_element=qt.bits_per_element,
                                 global_scale=qt.global_scale)


def test_reference_objects_pack_to_the_golden_bytes(layers):
    """With a reference checkout: feed what ITS _quantize_weight returns into this package's packer."""
    ref = os.environ.get("RDQUANT_REFERENCE")
    if not ref:
        pytest.skip("RDQUANT_REFERENCE not set")
    saved = {k: v for k, v in sys.modules.items() if k == "rdquant" or k.startswith("rdquant.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, ref)
    try:
        from rdquant.core.allocator import AllocationResult
        from rdquant.quantize import _quantize_weight

        from rdquant_b200.core.formats import qtensor_to_packed

        case = layers["mixed_384x256"]
        w = torch.from_numpy(case["weight_f16_bits"].copy()).view(torch.int16).view(torch.float16)
        perm = torch.from_numpy(case["perm"].astype(np.int64))
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel())
        splits = dict(zip(ORDER, (int(v) for v in case["splits"])))
        alloc = AllocationResult(assignments={}, permutation=perm, inv_permutation=inv, splits=splits, avg_bits=0.0,
                                 total_distortion=0.0, lambda_star=0.0, format_stats={})
        qw = _quantize_weight(w.float(), alloc)
        golden, _, _ = golden_layer_torch(case)
        for fmt, qt in qw.qtensors.items():
            for key, t in qtensor_to_packed(qt).items():
                if key == "weight_fp16":
                    continue  # the checkpoint stores this group as bfloat16
                assert torch.equal(t.reshape(golden[key].shape), golden[key]), key
    finally:
        sys.path.remove(ref)
        for k in [k for k in sys.modules if k == "rdquant" or k.startswith("rdquant.")]:
            del sys.modules[k]
        sys.modules.update(saved)


@pytest.mark.gpu
def test_operator_accepts_foreign_payload_objects(layers):
    from oracle import oracle_np as onp
    from rdquant.ops import mixed_precision_linear
    from rdquant_b200.quantize import quantize_weight

    case = layers["mixed_384x256"]
    w = torch.from_numpy(case["weight_f16_bits"].copy()).view(torch.int16).view(torch.float16)
    perm = torch.from_numpy(case["perm"].astype(np.int64))
    splits = dict(zip(ORDER, (int(v) for v in case["splits"])))
    qw = quantize_weight(w.float(), perm, splits)
    foreign = {fmt: _foreign(qt) for fmt, qt in qw.qtensors.items()}
    for m in (1, 3):
        x = torch.from_numpy(case[f"x{m}_f16_bits"].copy()).view(torch.int16).view(torch.float16)
        y = mixed_precision_linear(x.cuda(), foreign, qw.splits, qw.inv_permutation)
        y_ref = case[f"y{m}_ref_f16_bits"].view(np.float16).astype(np.float32)
        assert onp.rel_err(y.cpu().float().numpy(), y_ref) < 2e-3
