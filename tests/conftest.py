import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
ORDER = ("NVFP4", "FP8", "FP16")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built kernels")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_layers():
    """{case name: {key: array}} from tests/golden/layers.npz."""
    z = np.load(os.path.join(GOLDEN, "layers.npz"))
    out = {}
    for key in z.files:
        case, rest = key.split("/", 1)
        out.setdefault(case, {})[rest] = z[key]
    return out


def golden_layer_np(case: dict):
    """(layer dict in checkpoint naming with numpy arrays, splits dict, K)."""
    layer = {k[len("saved/"):]: v for k, v in case.items() if k.startswith("saved/")}
    splits = dict(zip(ORDER, (int(v) for v in case["splits"])))
    k = case["weight_f16_bits"].shape[1]
    return layer, splits, k


def golden_layer_torch(case: dict, device="cpu"):
    """Checkpoint-named torch tensors of a golden case (bf16 / f16 restored from bits)."""
    import torch

    layer, splits, k = golden_layer_np(case)
    out = {}
    for key, arr in layer.items():
        t = torch.from_numpy(np.ascontiguousarray(arr))
        if key == "weight_fp16":
            t = t.view(torch.int16).view(torch.bfloat16)
        elif key == "bias":
            t = t.view(torch.int16).view(torch.float16)
        out[key] = t.to(device)
    return out, splits, k


@pytest.fixture(scope="session")
def layers():
    return golden_layers()
