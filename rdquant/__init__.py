"""``rdquant`` import names for the mixed-precision linear path, served by ``rdquant_b200``.

Code written against the reference package (rdquant/__init__.py:3-13) keeps its imports:
``rdquant.ops.mixed_precision_linear``, ``rdquant.inference.FusedMixedLinear`` /
``load_for_inference``, ``rdquant.fused_gemv_pack.pack_for_fused_gemv``,
``rdquant.integrations.hf_export.save_packed`` / ``load_packed``, ``rdquant.quantize`` and
``rdquant.core.formats``.  Only the operator path is provided: the allocator, calibration,
evaluation and INT4 modules of the reference are not part of this package, and
``quantize_model`` / ``quantize_and_export`` (which drive them) are therefore absent.
"""
import importlib
import sys

from rdquant_b200.quantize import QuantizedLayer, QuantizedModel, QuantizedWeight

__all__ = ["QuantizedModel", "QuantizedLayer", "QuantizedWeight", "load_for_inference"]

for _name in ("core", "core.formats", "integrations", "integrations.hf_export", "quantize", "ops",
              "fused_gemv_pack", "inference"):
    _mod = importlib.import_module("rdquant_b200." + _name)
    sys.modules[__name__ + "." + _name] = _mod
    if "." not in _name:
        globals()[_name] = _mod

from rdquant_b200.inference import load_for_inference  # noqa: E402
