"""Module name under which the reference looks for its kernel extension
(rdquant/fused_gemv_pack.py:37-42 imports ``rdquant_cuda``); here it is the ctypes binding of
``librdq_b200.so``."""
from rdquant_b200.rdquant_cuda import *  # noqa: F401,F403
from rdquant_b200.rdquant_cuda import (  # noqa: F401
    check_gemm_status,
    check_status,
    dequantize_packed,
    fused_mixed_gemv,
    mixed_gemm,
    mixed_gemv,
    mixed_linear,
)
