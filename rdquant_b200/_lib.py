"""Build and load ``librdq_b200.so`` -- the C-ABI library holding the sm_100a kernels.

The library is built in-tree with ``nvcc`` (``build()``) and bound with ``ctypes``;
signatures follow ``include/rdq_b200.h``.  There is no fallback: if the library is
missing or a call fails, a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(CSRC, "librdq_b200.so")
SOURCES = [
    "rdq_api.cu",
    "rdq_dequant.cu",
    "rdq_gemv_generic.cu",
    "rdq_gemv_tiled.cu",
    "rdq_gemm.cu",
    "rdq_quantize.cu",
    "rdq_stage.cu",
    "rdq_glue.cu",
]
HEADERS = ["rdq_common.cuh", "rdq_kernels.cuh", "rdq_gemv_tiled_kernel.inl", "rdq_gemm_kernel.inl",
           os.path.join("..", "..", "include", "rdq_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]

RDQ_GEMV_AUTO = 0
RDQ_GEMV_GENERIC = 1
RDQ_GEMV_PDL = 16
RDQ_GEMV_TEST_TIMEOUT = 64

RDQ_E_DEVICE = -4

_lock = threading.Lock()
_lib = None


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    for f in SOURCES + HEADERS:
        p = os.path.join(CSRC, f)
        if os.path.exists(p) and os.path.getmtime(p) > t:
            return True
    return False


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the kernels for sm_100a into ``csrc/librdq_b200.so`` (needs nvcc, no GPU)."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, *SOURCES, "-lcuda"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


def _bind(lib: ctypes.CDLL) -> None:
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.rdq_version.restype = i32
    lib.rdq_version.argtypes = []
    lib.rdq_last_error.restype = ctypes.c_char_p
    lib.rdq_last_error.argtypes = []
    lib.rdq_dequant_packed.restype = i32
    lib.rdq_dequant_packed.argtypes = [vp, vp, f32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.rdq_gemv_scratch_size.restype = i32
    lib.rdq_gemv_scratch_size.argtypes = [i32, ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
    lib.rdq_gemv_mixed.restype = i32
    lib.rdq_gemv_mixed.argtypes = [vp, i32, vp, vp, f32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, vp, i32, vp]
    lib.rdq_gemv_tiled_bytes.restype = ctypes.c_size_t
    lib.rdq_gemv_tiled_bytes.argtypes = [i32, i32, i32, i32]
    lib.rdq_gemv_repack.restype = i32
    lib.rdq_gemv_repack.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.rdq_gemv_tiled.restype = i32
    lib.rdq_gemv_tiled.argtypes = [vp, i32, vp, vp, f32, vp, vp, vp, i32, i32, i32, i32, vp, vp, i32, vp]
    lib.rdq_gemv_tiled_stages_x.restype = i32
    lib.rdq_gemv_tiled_stages_x.argtypes = [i32, i32]
    lib.rdq_gemv_tiled_xop.restype = i32
    lib.rdq_gemv_tiled_xop.argtypes = [i32, vp, vp, vp, vp, f32, i32, vp, vp, f32, vp, vp, vp, i32, i32, i32, i32, vp, vp,
                                       i32, vp]
    lib.rdq_gemv_tiled_peer.restype = i32
    lib.rdq_gemv_tiled_peer.argtypes = [vp, i32, vp, vp, f32, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, vp, vp, i32, vp]
    lib.rdq_peer_gather.restype = i32
    lib.rdq_peer_gather.argtypes = [vp, vp, vp, ctypes.c_longlong, vp, i32, vp, vp, i32, i32, vp]
    lib.rdq_gemv_tiled_noalloc.restype = i32
    lib.rdq_gemv_tiled_noalloc.argtypes = [vp, i32, vp, vp, f32, vp, vp, vp, i32, i32, i32, i32, i32, vp]
    lib.rdq_gemv_tiled_status.restype = i32
    lib.rdq_gemv_tiled_status.argtypes = [vp, vp, i32, vp]
    lib.rdq_gemv_tiled_noalloc_status.restype = i32
    lib.rdq_gemv_tiled_noalloc_status.argtypes = [i32, vp]
    lib.rdq_gemm_status.restype = i32
    lib.rdq_gemm_status.argtypes = [i32, vp]
    lib.rdq_gemm_test_timeout.restype = None
    lib.rdq_gemm_test_timeout.argtypes = [i32]
    lib.rdq_gemm_mixed.restype = i32
    lib.rdq_gemm_mixed.argtypes = [vp, i32, vp, vp, f32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.rdq_gemm_mixed_ws.restype = i32
    lib.rdq_gemm_mixed_ws.argtypes = [vp, i32, vp, vp, f32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp, ctypes.c_size_t, vp]
    lib.rdq_gemm_workspace_size.restype = i32
    lib.rdq_gemm_workspace_size.argtypes = [i32, i32, i32, ctypes.POINTER(ctypes.c_size_t)]
    lib.rdq_quantize_nvfp4.restype = i32
    lib.rdq_quantize_nvfp4.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp]
    lib.rdq_quantize_fp8.restype = i32
    lib.rdq_quantize_fp8.argtypes = [vp, i32, i32, i32, vp, vp, vp, vp, vp]
    lib.rdq_add_rmsnorm.restype = i32
    lib.rdq_add_rmsnorm.argtypes = [vp, vp, vp, vp, i32, i32, f32, i32, vp]
    lib.rdq_qk_rope_cache.restype = i32
    lib.rdq_qk_rope_cache.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp]
    lib.rdq_attn_decode_scratch_size.restype = i32
    lib.rdq_attn_decode_scratch_size.argtypes = [i32, i32, i32, i32, ctypes.POINTER(ctypes.c_size_t)]
    lib.rdq_attn_decode.restype = i32
    lib.rdq_attn_decode.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp]
    lib.rdq_rope_attn_decode_scratch_size.restype = i32
    lib.rdq_rope_attn_decode_scratch_size.argtypes = [i32, i32, i32, i32, i32, ctypes.POINTER(ctypes.c_size_t)]
    lib.rdq_rope_attn_decode.restype = i32
    lib.rdq_rope_attn_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, f32, i32, vp]
    lib.rdq_silu_mul.restype = i32
    lib.rdq_silu_mul.argtypes = [vp, vp, i32, i32, i32, vp]
    lib.rdq_stage_copy.restype = i32
    lib.rdq_stage_copy.argtypes = [vp, vp, ctypes.c_size_t, vp]
    lib.rdq_stage_copy_signal.restype = i32
    lib.rdq_stage_copy_signal.argtypes = [vp, vp, ctypes.c_size_t, vp, vp, vp]


EXPORTS = [
    "rdq_version",
    "rdq_last_error",
    "rdq_dequant_packed",
    "rdq_gemv_scratch_size",
    "rdq_gemv_mixed",
    "rdq_gemv_tiled_bytes",
    "rdq_gemv_repack",
    "rdq_gemv_tiled",
    "rdq_gemv_tiled_noalloc",
    "rdq_gemv_tiled_peer",
    "rdq_gemv_tiled_xop",
    "rdq_gemv_tiled_stages_x",
    "rdq_peer_gather",
    "rdq_gemv_tiled_status",
    "rdq_gemv_tiled_noalloc_status",
    "rdq_gemm_status",
    "rdq_gemm_test_timeout",
    "rdq_gemm_mixed",
    "rdq_gemm_mixed_ws",
    "rdq_gemm_workspace_size",
    "rdq_quantize_nvfp4",
    "rdq_quantize_fp8",
    "rdq_stage_copy",
    "rdq_stage_copy_signal",
    "rdq_add_rmsnorm",
    "rdq_qk_rope_cache",
    "rdq_attn_decode_scratch_size",
    "rdq_attn_decode",
    "rdq_rope_attn_decode_scratch_size",
    "rdq_rope_attn_decode",
    "rdq_silu_mul",
]


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    """Return the loaded library; raise ``RuntimeError`` if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: the CUDA kernels are not built. "
                    "Run `python -c 'import __graft_entry__ as g; g.build()'` or rdquant_b200._lib.build()."
                )
            handle = ctypes.CDLL(LIB_PATH)
            _bind(handle)
            _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().rdq_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")
