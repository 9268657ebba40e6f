"""rdq_gemv_tiled_noalloc: the tiled decode GEMV for hosts that may not allocate device
memory (its scratch is a device array inside the library).  Called through the C ABI twice
in a row -- the array keeps the previous call's state, so the second call checks that the
first one left it clean -- and compared with rdq_gemv_tiled, which uses caller scratch.
Collected last on purpose: a failure here cannot hide the results of the other tests."""
import ctypes

import pytest
import torch

from conftest import ORDER
from rdquant_b200 import _lib, rdquant_cuda
from rdquant_b200.fused_gemv_pack import pack_for_fused_gemv
from rdquant_b200.synthetic import random_packed_layer

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("shape,m", [((1664, 768, 128, 4096), 1), ((640, 256, 128, 2560), 4)])
def test_no_alloc_entry_matches_scratch_entry(shape, m):
    n4, n8, n16, k = shape
    splits = dict(zip(ORDER, shape[:3]))
    fd = pack_for_fused_gemv(random_packed_layer(n4, n8, n16, k, seed=21), splits, k, "cuda")
    assert fd["w_tiled"] is not None
    x = torch.randn(m, k, generator=torch.Generator().manual_seed(5)).half().cuda()
    bias = (torch.randn(n4 + n8 + n16, generator=torch.Generator().manual_seed(6)) * 0.3).half().cuda()
    y_ref = rdquant_cuda.mixed_gemv(x, fd, bias)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib = _lib.lib()
    for call in range(2):
        y = torch.zeros_like(y_ref)
        rc = lib.rdq_gemv_tiled_noalloc(_p(x), m, _p(fd["w_tiled"]), _p(fd["w_fp8_scales"]), 1.0, _p(fd["perm"]),
                                        _p(bias), _p(y), n4, n8, n16, k, 0, stream)
        assert rc == 0, lib.rdq_last_error()
        torch.cuda.synchronize()
        err = (y.float() - y_ref.float()).abs().max() / y_ref.float().abs().max()
        assert float(err) < TOL, (call, float(err))
        assert torch.equal(y, y_ref), f"call {call}: not the same bits as the scratch entry point"
        assert lib.rdq_gemv_tiled_noalloc_status(0, stream) == 0, lib.rdq_last_error()


def test_no_alloc_entry_rejects_bad_shapes():
    lib = _lib.lib()
    rc = lib.rdq_gemv_tiled_noalloc(None, 17, None, None, 1.0, None, None, None, 16, 0, 0, 256, 0, None)
    assert rc == -2 and b"activation rows" in lib.rdq_last_error()
    rc = lib.rdq_gemv_tiled_noalloc(None, 1, None, None, 1.0, None, None, None, 10, 0, 0, 256, 0, None)
    assert rc == -2 and b"tiled layout" in lib.rdq_last_error()


def test_no_alloc_entry_reports_and_clears_a_timeout():
    """The status word of the built-in array is readable and the array can be put back to idle:
    a launch that gave up a wait (here the self-test wait on a barrier nothing completes) must
    not poison the calls that follow."""
    n4, n8, n16, k = 256, 128, 64, 1024
    splits = dict(zip(ORDER, (n4, n8, n16)))
    fd = pack_for_fused_gemv(random_packed_layer(n4, n8, n16, k, seed=22), splits, k, "cuda")
    x = torch.randn(1, k, generator=torch.Generator().manual_seed(7)).half().cuda()
    y_ref = rdquant_cuda.mixed_gemv(x, fd)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib = _lib.lib()

    def call(flags):
        y = torch.zeros_like(y_ref)
        rc = lib.rdq_gemv_tiled_noalloc(_p(x), 1, _p(fd["w_tiled"]), _p(fd["w_fp8_scales"]), 1.0, _p(fd["perm"]),
                                        None, _p(y), n4, n8, n16, k, flags, stream)
        assert rc == 0, lib.rdq_last_error()
        return y

    call(_lib.RDQ_GEMV_TEST_TIMEOUT)
    assert lib.rdq_gemv_tiled_noalloc_status(1, stream) == _lib.RDQ_E_DEVICE
    assert b"status 9" in lib.rdq_last_error()
    assert lib.rdq_gemv_tiled_noalloc_status(0, stream) == 0
    y = call(0)
    assert lib.rdq_gemv_tiled_noalloc_status(0, stream) == 0
    assert torch.equal(y, y_ref)
