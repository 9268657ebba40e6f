"""TEST INFRASTRUCTURE ONLY -- ctypes binding of oracle/rdq_oracle.c (the timed CPU baseline)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "librdq_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "rdq_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        # -march=native is avoided: the library travels to another host
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-o", LIB, src], check=True, cwd=_HERE)
    return LIB


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = ctypes.CDLL(LIB)
        _lib.rdq_oracle_threads.restype = ctypes.c_int
        _lib.rdq_oracle_linear.restype = None
    return _lib


def set_threads(n: int) -> None:
    """Use n OpenMP threads (torchrun exports OMP_NUM_THREADS=1; the timed baseline wants all cores)."""
    l = lib()
    l.rdq_oracle_set_threads.argtypes = [ctypes.c_int]
    l.rdq_oracle_set_threads.restype = None
    l.rdq_oracle_set_threads(int(n))


def threads() -> int:
    return int(lib().rdq_oracle_threads())


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def linear(x_f16: np.ndarray, codes4, scales4, n4, data8, scale8, n8, data16, n16, inv_perm, bias=None) -> np.ndarray:
    """float32 [M, N]; arguments are the reference's QuantizedTensor payloads as numpy arrays
    (int64 codes, float32 block scales, float32 FP8 values, float16 data)."""
    m, k = x_f16.shape
    n = n4 + n8 + n16
    x = np.ascontiguousarray(x_f16.view(np.uint16))
    scratch = np.empty((m, n), dtype=np.float32)
    y = np.empty((m, n), dtype=np.float32)
    d16 = None if data16 is None else np.ascontiguousarray(data16.view(np.uint16))
    inv = np.ascontiguousarray(inv_perm.astype(np.int64))
    b = None if bias is None else np.ascontiguousarray(bias.astype(np.float32))
    lib().rdq_oracle_linear(_p(x), ctypes.c_int(m), ctypes.c_int(k), _p(codes4), _p(scales4), ctypes.c_int(n4),
                            _p(data8), ctypes.c_float(scale8), ctypes.c_int(n8), _p(d16), ctypes.c_int(n16),
                            _p(inv), _p(b), _p(scratch), _p(y))
    return y
