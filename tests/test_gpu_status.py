"""Device-side error reporting: a kernel whose bounded wait runs out must be visible to the
caller.  The time-out is provoked on the host side of the contract -- a self-test flag makes one
warp wait, after all its work, on a barrier that nothing completes -- never by a fault."""
import ctypes

import pytest
import torch

from conftest import ORDER
from oracle import oracle_np as onp
from rdquant_b200 import _lib, rdquant_cuda
from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv
from rdquant_b200.synthetic import random_packed_layer

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _layer(shape=(256, 128, 64, 1024), seed=3):
    n4, n8, n16, k = shape
    splits = dict(zip(ORDER, shape[:3]))
    layer = random_packed_layer(n4, n8, n16, k, seed=seed)
    return layer, splits, k, pack_for_fused_gemv(layer, splits, k, "cuda")


def test_gemv_tiled_timeout_is_reported_and_cleared():
    layer, splits, k, fd = _layer()
    lib = _lib.lib()
    x = torch.randn(2, k, generator=torch.Generator().manual_seed(1)).half().cuda()
    y_ok = rdquant_cuda.mixed_gemv(x, fd)
    rdquant_cuda.check_status(fd)  # clean
    rdquant_cuda.mixed_gemv(x, fd, None, _lib.RDQ_GEMV_TEST_TIMEOUT)
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        rdquant_cuda.check_status(fd)
    assert int(fd["tile_counters"].abs().sum()) == 0, "reset must clear the status word"
    rdquant_cuda.check_status(fd)
    y_again = rdquant_cuda.mixed_gemv(x, fd)
    rdquant_cuda.check_status(fd)
    assert torch.equal(y_ok, y_again)
    # the raw entry point returns RDQ_E_DEVICE
    rdquant_cuda.mixed_gemv(x, fd, None, _lib.RDQ_GEMV_TEST_TIMEOUT)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.rdq_gemv_tiled_status(_p(fd["workspace"]), _p(fd["tile_counters"]), 0, stream)
    assert rc == _lib.RDQ_E_DEVICE and b"status 9" in lib.rdq_last_error()
    assert lib.rdq_gemv_tiled_status(_p(fd["workspace"]), _p(fd["tile_counters"]), 1, stream) == _lib.RDQ_E_DEVICE
    assert lib.rdq_gemv_tiled_status(_p(fd["workspace"]), _p(fd["tile_counters"]), 0, stream) == 0


def test_validate_mode_checks_every_call(monkeypatch):
    layer, splits, k, fd = _layer(seed=4)
    x = torch.randn(1, k, generator=torch.Generator().manual_seed(2)).half().cuda()
    monkeypatch.setattr(rdquant_cuda, "VALIDATE", True)
    rdquant_cuda.mixed_gemv(x, fd)
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        rdquant_cuda.mixed_gemv(x, fd, None, _lib.RDQ_GEMV_TEST_TIMEOUT)
    rdquant_cuda.mixed_gemv(x, fd)  # state was reset by the failed check


def test_gemm_timeout_is_reported_and_cleared():
    layer, splits, k, fd = _layer(seed=5)
    lib = _lib.lib()
    x = torch.randn(64, k, generator=torch.Generator().manual_seed(3)).half().cuda()
    y_ok = rdquant_cuda.mixed_gemm(x, fd)
    rdquant_cuda.check_gemm_status(x.device)
    lib.rdq_gemm_test_timeout(1)
    try:
        rdquant_cuda.mixed_gemm(x, fd)
    finally:
        lib.rdq_gemm_test_timeout(0)
    with pytest.raises(RuntimeError, match="prefill GEMM: a bounded device-side wait"):
        rdquant_cuda.check_gemm_status(x.device)
    rdquant_cuda.check_gemm_status(x.device)  # cleared by the failed check
    y_again = rdquant_cuda.mixed_gemm(x, fd)
    rdquant_cuda.check_gemm_status(x.device)
    assert torch.equal(y_ok, y_again)
    ref = onp.mixed_precision_linear(x.cpu().numpy(), onp.torch_layer_to_np(layer), splits, k)
    assert onp.rel_err(y_again.cpu().float().numpy(), ref) < 2e-3
