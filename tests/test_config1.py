"""BASELINE configs[0] at full size: the K = 2560 -> N = 9728 layer whose formats the reference's
Lagrangian allocator chose (seed 0: 6656 NVFP4 / 2944 FP8 / 128 FP16 channels).  The fixture
tests/golden/config1_alloc.npz holds what the REFERENCE produced for it (hashes of its packed
checkpoint tensors and of its dequantised weight, 24 rows of that weight, its operator output).

CPU: this package's encoders + checkpoint writer reproduce the reference's bytes, and the oracle
reproduces the reference's dequantised weight and output -- pins both at full size.
GPU: the dequantisation kernel is bit-exact against the reference's weight and the decode GEMV
matches the reference operator's output."""
import hashlib
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, ORDER
from oracle import oracle_np as onp
from rdquant_b200.integrations import hf_export
from rdquant_b200.quantize import quantize_weight

TOL = 2e-3


def _sha(t: torch.Tensor) -> bytes:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).digest()


@pytest.fixture(scope="module")
def config1():
    z = np.load(os.path.join(GOLDEN, "config1_alloc.npz"))
    g = torch.Generator().manual_seed(0)
    n, k = 9728, 2560
    w = (torch.randn(n, k, generator=g) * 0.02).half()
    idx = torch.randperm(n, generator=g)[: n // 100]
    w[idx] *= 8
    if _sha(w) != z["sha_weight_f16"].tobytes():
        pytest.skip("this torch build draws different random numbers than the one that made the fixture")
    perm = torch.from_numpy(z["perm"].astype(np.int64))
    splits = dict(zip(ORDER, (int(v) for v in z["splits"])))
    qw = quantize_weight(w.float(), perm, splits)
    packed = hf_export.pack_layer(qw, None)
    return z, qw, packed, splits, k, n


def test_packed_bytes_equal_the_reference_checkpoint(config1):
    z, qw, packed, splits, k, n = config1
    assert splits == {"NVFP4": 6656, "FP8": 2944, "FP16": 128}
    for key, t in packed.items():
        assert _sha(t) == z["sha_" + key].tobytes(), key


def test_oracle_reproduces_the_reference_at_full_size(config1):
    z, qw, packed, splits, k, n = config1
    layer = onp.torch_layer_to_np(packed)
    # the reference's dequantised weight comes from the in-memory payload, whose FP16 group is the
    # original float16 rows (the checkpoint stores that group as bfloat16)
    layer["weight_fp16"] = qw.qtensors["FP16"].data.reshape(splits["FP16"], k).numpy()
    w = onp.dequantize_layer(layer, splits, k)
    assert hashlib.sha256(np.ascontiguousarray(w).view(np.uint16).tobytes()).digest() == z["sha_w_ref_f16"].tobytes()
    assert np.array_equal(w[z["sample_rows"]].view(np.uint16), z["w_ref_rows_f16_bits"])
    x = z["x_f16_bits"].view(np.float16)
    y = onp.mixed_precision_linear(x, layer, splits, k)
    y_ref = z["y_ref_f16_bits"].view(np.float16).astype(np.float32)
    assert onp.rel_err(y, y_ref) < 1e-3  # the reference output is rounded to float16


@pytest.mark.gpu
def test_gpu_dequant_bit_exact_and_gemv(config1):
    from rdquant_b200 import _lib, rdquant_cuda
    from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv

    z, qw, packed, splits, k, n = config1
    dev = {kk: v.cuda() for kk, v in packed.items()}
    dev["weight_fp16"] = qw.qtensors["FP16"].data.reshape(splits["FP16"], k).cuda()  # float16 payload, see above
    w = rdquant_cuda.dequantize_packed(dev, splits, k, inv_perm=dev["inv_permutation"])
    assert _sha(w.cpu()) == z["sha_w_ref_f16"].tobytes(), "dequantised weight differs from the reference's"
    x = torch.from_numpy(z["x_f16_bits"].copy()).view(torch.int16).view(torch.float16)
    y_ref = z["y_ref_f16_bits"].view(np.float16).astype(np.float32)
    fd = pack_for_fused_gemv(packed, splits, k, "cuda")
    assert fd["w_tiled"] is not None
    for flags in (_lib.RDQ_GEMV_PDL, _lib.RDQ_GEMV_GENERIC):
        y = rdquant_cuda.mixed_gemv(x.cuda(), fd, None, flags)
        rdquant_cuda.check_status(fd)
        # the checkpoint's FP16 group went through bfloat16; those 128 channels differ from the
        # in-memory operator by that rounding, the others only by summation order
        assert onp.rel_err(y.cpu().float().numpy(), y_ref) < 4e-3
        keep = (qw.inv_permutation < splits["NVFP4"] + splits["FP8"]).numpy()
        assert onp.rel_err(y.cpu().float().numpy()[:, keep], y_ref[:, keep]) < TOL
    # the same layer from the in-memory float16 payload: every channel within the tolerance
    exact = dict(packed)
    exact["weight_fp16"] = qw.qtensors["FP16"].data.reshape(splits["FP16"], k)
    fd2 = pack_for_fused_gemv(exact, splits, k, "cuda")
    y = rdquant_cuda.mixed_gemv(x.cuda(), fd2, None, _lib.RDQ_GEMV_PDL)
    rdquant_cuda.check_status(fd2)
    assert onp.rel_err(y.cpu().float().numpy(), y_ref) < TOL
