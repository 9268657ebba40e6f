"""rdquant_b200 -- B200 (sm_100a) implementation of RDQuant's mixed-precision linear operator.

Same Python surface as the reference package for this path:
``ops.mixed_precision_linear``, ``inference.FusedMixedLinear`` / ``load_for_inference``,
``fused_gemv_pack.pack_for_fused_gemv`` and ``integrations.hf_export.save_packed`` /
``load_packed`` (reference: rdquant/__init__.py:3-13).
"""
from rdquant_b200.quantize import QuantizedLayer, QuantizedModel, QuantizedWeight

__all__ = ["QuantizedLayer", "QuantizedModel", "QuantizedWeight", "load_for_inference"]


def __getattr__(name):
    if name == "load_for_inference":
        from rdquant_b200.inference import load_for_inference

        return load_for_inference
    raise AttributeError(name)
