"""The C-ABI library builds for sm_100a without a GPU, loads, and exports every entry point
that include/rdq_b200.h declares.  No compute calls here."""
import ctypes
import os
import re

from conftest import ROOT
from rdquant_b200 import _lib


def _declared():
    text = open(os.path.join(ROOT, "include", "rdq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rdq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_header():
    _lib.build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert "rdq_gemv_mixed" in names and "rdq_gemm_mixed" in names and "rdq_dequant_packed" in names
    for name in names:
        assert hasattr(handle, name), f"{name} declared in rdq_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == [n for n in names if n in _lib.EXPORTS]
    assert set(names) == set(_lib.EXPORTS)


def test_argument_validation_needs_no_gpu():
    lib = _lib.lib()
    assert lib.rdq_version() >= 100
    # n_fp4 > 0 with K not a multiple of 16 is rejected before anything touches the device
    rc = lib.rdq_dequant_packed(None, None, 1.0, None, None, None, 0, None, None, 0, 16, 0, 0, 24, None)
    assert rc == -1 and b"multiple of 16" in lib.rdq_last_error()
    rc = lib.rdq_gemv_mixed(None, 17, None, None, 1.0, None, None, None, None, None, None, 0, 16, 0, 32, None, None, 0, None)
    assert rc != 0
