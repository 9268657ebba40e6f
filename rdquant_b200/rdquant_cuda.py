"""Torch-facing wrappers over the C ABI of ``librdq_b200.so``.

Plays the role of the reference's pybind extension module ``rdquant_cuda``
(rdquant/csrc/bindings.cpp:979-990): validate tensors, allocate the output with torch,
hand raw device pointers and the current CUDA stream to the C entry points.  Failures
surface as ``RuntimeError`` like the reference's ``TORCH_CHECK``s.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from rdquant_b200 import _lib

MAX_GEMV_M = 16
# RDQ_B200_VALIDATE=1: synchronise after every GEMV / GEMM call and raise if the kernel gave up a
# bounded device-side wait (debugging aid; costs a device round trip per call)
VALIDATE = os.environ.get("RDQ_B200_VALIDATE", "0") not in ("", "0")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _need_cuda(name: str, t: Optional[torch.Tensor], dtype=None) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")


class _on_device:
    """Make ``device`` current for the duration of a call (the C ABI uses the current device)."""

    def __init__(self, device: torch.device) -> None:
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


def perm_from_inv_perm(inv_perm: torch.Tensor) -> torch.Tensor:
    """int32 ``perm`` with ``perm[inv_perm[j]] = j``: permuted row p is original channel perm[p]
    (rdquant/core/allocator.py:222-224, rdquant/integrations/hf_export.py:243-245)."""
    inv = inv_perm.to(torch.int64)
    perm = torch.empty_like(inv)
    perm[inv] = torch.arange(inv.numel(), dtype=torch.int64, device=inv.device)
    return perm.to(torch.int32)


def gemv_scratch(n_out: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """(workspace, tile_counters) for the stream GEMV of a layer with ``n_out`` channels."""
    device = torch.device(device)
    ws, cnt = ctypes.c_size_t(0), ctypes.c_size_t(0)
    with _on_device(device):
        _lib.check(_lib.lib().rdq_gemv_scratch_size(int(n_out), ctypes.byref(ws), ctypes.byref(cnt)),
                   "rdq_gemv_scratch_size")
    # idle workspace words read 0xffffffff (the tiled kernel's "no partial sum yet" mark)
    workspace = torch.full((max(ws.value // 4, 1),), -1, dtype=torch.int32, device=device).view(torch.float32)
    counters = torch.zeros(max(cnt.value // 4, 1), dtype=torch.int32, device=device)
    return workspace, counters


def check_status(fd: dict) -> None:
    """Wait for the work queued on the current stream and raise ``RuntimeError`` if a tiled-GEMV
    launch on this layer's scratch gave up a bounded wait (its output is then invalid).  The
    scratch is put back to its idle state in that case, so the layer stays usable."""
    ws, cnt = fd.get("workspace"), fd.get("tile_counters")
    if ws is None or cnt is None:
        return
    with _on_device(ws.device):
        rc = _lib.lib().rdq_gemv_tiled_status(_ptr(ws), _ptr(cnt), 1, _stream(ws.device))
    _lib.check(rc, "rdq_gemv_tiled_status")


def check_gemm_status(device) -> None:
    """The same for the prefill GEMM (one status word per device, cleared when it is reported)."""
    device = torch.device(device)
    with _on_device(device):
        rc = _lib.lib().rdq_gemm_status(1, _stream(device))
    _lib.check(rc, "rdq_gemm_status")


_scratch_by_device: dict = {}


def _shared_scratch(device) -> tuple[torch.Tensor, torch.Tensor]:
    """One scratch pair per device for callers that bring none (the reference-signature entry
    point): the kernel leaves it idle after every launch, and launches on one device are ordered
    by the current stream."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    pair = _scratch_by_device.get(key)
    if pair is None:
        pair = gemv_scratch(0, device)
        _scratch_by_device[key] = pair
    return pair


def dequantize_packed(layer_data: dict, splits: dict, k: int, inv_perm: Optional[torch.Tensor] = None,
                      out_dtype: torch.dtype = torch.float16, global_scale: float = 1.0) -> torch.Tensor:
    """Dequantise packed checkpoint tensors to ``[N, K]`` in original channel order.

    ``layer_data`` uses the checkpoint key names (``weight_nvfp4`` ...); ``weight_fp16`` may be
    bfloat16 (as stored on disk) or float16.  ``out_dtype`` float16 gives the operator's weight,
    float32 the unrounded products of ``formats.dequantize``.
    """
    n4, n8, n16 = (int(splits.get(f, 0)) for f in ("NVFP4", "FP8", "FP16"))
    w4 = layer_data.get("weight_nvfp4") if n4 else None
    s4 = layer_data.get("weight_nvfp4_scale") if n4 else None
    w8 = layer_data.get("weight_fp8") if n8 else None
    s8 = layer_data.get("weight_fp8_scale") if n8 else None
    w16 = layer_data.get("weight_fp16") if n16 else None
    some = next(t for t in (w4, w8, w16) if t is not None)
    device = some.device
    _need_cuda("weight_nvfp4", w4, torch.uint8)
    _need_cuda("weight_nvfp4_scale", s4, torch.uint8)
    _need_cuda("weight_fp8", w8, torch.uint8)
    _need_cuda("weight_fp8_scale", s8, torch.float32)
    _need_cuda("weight_fp16", w16)
    if w4 is not None and (tuple(w4.shape) != (n4, k // 2) or tuple(s4.shape) != (n4, k // 16)):
        raise RuntimeError("weight_nvfp4 must be [n4, K/2] and weight_nvfp4_scale [n4, K/16]")
    if w8 is not None and (tuple(w8.shape) != (n8, k) or s8.numel() != n8):
        raise RuntimeError("weight_fp8 must be [n8, K] and weight_fp8_scale [n8]")
    is_bf16 = 0
    if w16 is not None:
        if tuple(w16.shape) != (n16, k):
            raise RuntimeError("weight_fp16 must be [n16, K]")
        if w16.dtype == torch.bfloat16:
            is_bf16 = 1
        elif w16.dtype != torch.float16:
            raise RuntimeError("weight_fp16 must be float16 or bfloat16")
    if out_dtype not in (torch.float16, torch.float32):
        raise RuntimeError("out_dtype must be float16 or float32")
    inv32 = None
    if inv_perm is not None:
        inv32 = inv_perm.to(device=device, dtype=torch.int32).contiguous()
        if inv32.numel() != n4 + n8 + n16:
            raise RuntimeError("inv_perm must have N elements")
    out = torch.empty(n4 + n8 + n16, k, dtype=out_dtype, device=device)
    with _on_device(device):
        rc = _lib.lib().rdq_dequant_packed(_ptr(w4), _ptr(s4), float(global_scale), _ptr(w8), _ptr(s8), _ptr(w16),
                                           is_bf16, _ptr(inv32), _ptr(out), int(out_dtype == torch.float32),
                                           n4, n8, n16, int(k), _stream(device))
    _lib.check(rc, "rdq_dequant_packed")
    return out


def tiled_bytes(n4: int, n8: int, n16: int, k: int) -> int:
    """Size of the tiled copy of a layer (0: the shape has no tiled layout)."""
    return int(_lib.lib().rdq_gemv_tiled_bytes(n4, n8, n16, k))


def repack_tiled(fd: dict) -> Optional[torch.Tensor]:
    """Re-tile the row-major buffers of a ``pack_for_fused_gemv`` dict for the fast GEMV;
    ``None`` when the shape has no tiled layout."""
    n4, n8, n16, k = fd["n_fp4"], fd["n_fp8"], fd["n_fp16"], fd["k"]
    nbytes = int(_lib.lib().rdq_gemv_tiled_bytes(n4, n8, n16, k))
    if nbytes == 0:
        return None
    some = next(t for t in (fd.get("w_fp4_q"), fd.get("w_fp8_q"), fd.get("w_fp16")) if t is not None)
    out = torch.empty(nbytes, dtype=torch.uint8, device=some.device)
    with _on_device(some.device):
        rc = _lib.lib().rdq_gemv_repack(_ptr(fd.get("w_fp4_q")), _ptr(fd.get("w_fp4_scales")), _ptr(fd.get("w_fp8_q")),
                                        _ptr(fd.get("w_fp16")), _ptr(out), n4, n8, n16, k, _stream(some.device))
    _lib.check(rc, "rdq_gemv_repack")
    return out


def mixed_gemv(x: torch.Tensor, fd: dict, bias: Optional[torch.Tensor] = None, flags: int = 0,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y[M, N] = x[M, K] @ W.T (+ bias)`` for M <= 16 from a ``pack_for_fused_gemv`` dict.

    Runs on the tiled layout when the dict carries one (``w_tiled``) and ``flags`` does not
    force one of the row-major kernels."""
    _need_cuda("x", x, torch.float16)
    if x.dim() != 2:
        raise RuntimeError("x must be 2-D [M, K]")
    m, k = x.shape
    if k != fd["k"]:
        raise RuntimeError(f"x.size(1)={k} must match K={fd['k']}")
    if m > MAX_GEMV_M:
        raise RuntimeError(f"decode GEMV takes at most {MAX_GEMV_M} rows, got {m}")
    n4, n8, n16 = fd["n_fp4"], fd["n_fp8"], fd["n_fp16"]
    n = n4 + n8 + n16
    if bias is not None:
        _need_cuda("bias", bias, torch.float16)
        if bias.numel() != n:
            raise RuntimeError("bias must have N elements")
    y = out if out is not None else torch.empty(m, n, dtype=torch.float16, device=x.device)
    if fd.get("w_tiled") is not None and (flags & 15) == _lib.RDQ_GEMV_AUTO:
        with _on_device(x.device):
            rc = _lib.lib().rdq_gemv_tiled(
                _ptr(x), m, _ptr(fd["w_tiled"]), _ptr(fd.get("w_fp8_scales")), float(fd.get("w_fp4_global_scale", 1.0)),
                _ptr(fd.get("perm")), _ptr(bias), _ptr(y), n4, n8, n16, k, _ptr(fd.get("workspace")),
                _ptr(fd.get("tile_counters")), int(flags), _stream(x.device))
        _lib.check(rc, "rdq_gemv_tiled")
        if VALIDATE:
            check_status(fd)
        return y
    if not fd.get("row_major", True):
        raise RuntimeError("this layer was packed without its row-major tensors: only the tiled decode kernel can run it")
    with _on_device(x.device):
        rc = _lib.lib().rdq_gemv_mixed(
            _ptr(x), m, _ptr(fd.get("w_fp4_q")), _ptr(fd.get("w_fp4_scales")), float(fd.get("w_fp4_global_scale", 1.0)),
            _ptr(fd.get("w_fp8_q")), _ptr(fd.get("w_fp8_scales")), _ptr(fd.get("w_fp16")), _ptr(fd.get("perm")),
            _ptr(bias), _ptr(y), n4, n8, n16, k, _ptr(fd.get("workspace")), _ptr(fd.get("tile_counters")),
            int(flags), _stream(x.device))
    _lib.check(rc, "rdq_gemv_mixed")
    return y


XOP_ADD_RMSNORM = 1
XOP_SILU_MUL = 2


def gemv_stages_x(m: int, k: int) -> bool:
    """True when the tiled GEMV keeps ``m`` activation rows of length ``k`` in shared memory,
    which the activation prologues of :func:`mixed_gemv_norm` / :func:`mixed_gemv_silu` need."""
    return bool(_lib.lib().rdq_gemv_tiled_stages_x(int(m), int(k)))


def _gemv_xop(op: int, x, aux, weight, x_out, eps: float, m: int, k: int, fd: dict, bias, flags: int, out):
    if fd.get("w_tiled") is None:
        raise RuntimeError("the activation prologue needs the tiled layout (w_tiled)")
    n4, n8, n16 = fd["n_fp4"], fd["n_fp8"], fd["n_fp16"]
    if k != fd["k"]:
        raise RuntimeError(f"activation length {k} must match K={fd['k']}")
    y = out if out is not None else torch.empty(m, n4 + n8 + n16, dtype=torch.float16, device=x.device)
    with _on_device(x.device):
        rc = _lib.lib().rdq_gemv_tiled_xop(
            op, _ptr(x), _ptr(aux), _ptr(weight), _ptr(x_out), float(eps), m, _ptr(fd["w_tiled"]),
            _ptr(fd.get("w_fp8_scales")), float(fd.get("w_fp4_global_scale", 1.0)), _ptr(fd.get("perm")), _ptr(bias),
            _ptr(y), n4, n8, n16, k, _ptr(fd.get("workspace")), _ptr(fd.get("tile_counters")), int(flags),
            _stream(x.device))
    _lib.check(rc, "rdq_gemv_tiled_xop")
    if VALIDATE:
        check_status(fd)
    return y


def mixed_gemv_norm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, fd: dict,
                    residual_out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, flags: int = 0,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = rmsnorm(x + delta) @ W.T`` in one launch; ``x + delta`` goes to ``residual_out``
    (a buffer other than ``x`` and ``delta``)."""
    _need_cuda("x", x, torch.float16)
    m, k = x.shape
    return _gemv_xop(XOP_ADD_RMSNORM, x, delta, weight, residual_out, eps, m, k, fd, bias, flags, out)


def mixed_gemv_silu(gate_up: torch.Tensor, fd: dict, bias: Optional[torch.Tensor] = None, flags: int = 0,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y = (silu(gate_up[:, :K]) * gate_up[:, K:]) @ W.T`` in one launch."""
    _need_cuda("gate_up", gate_up, torch.float16)
    m, k2 = gate_up.shape
    return _gemv_xop(XOP_SILU_MUL, gate_up, None, None, None, 0.0, m, k2 // 2, fd, bias, flags, out)


_gemm_ws: dict = {}  # device -> scratch tensor of the split-k GEMM


def mixed_gemm(x: torch.Tensor, fd: dict, bias: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Prefill GEMM ``y[M, N] = x[M, K] @ W.T (+ bias)`` on the tcgen05 path."""
    _need_cuda("x", x, torch.float16)
    if x.dim() != 2:
        raise RuntimeError("x must be 2-D [M, K]")
    m, k = x.shape
    if k != fd["k"]:
        raise RuntimeError(f"x.size(1)={k} must match K={fd['k']}")
    n4, n8, n16 = fd["n_fp4"], fd["n_fp8"], fd["n_fp16"]
    n = n4 + n8 + n16
    if bias is not None:
        _need_cuda("bias", bias, torch.float16)
    y = out if out is not None else torch.empty(m, n, dtype=torch.float16, device=x.device)
    if out is not None and (tuple(out.shape) != (m, n) or out.dtype != torch.float16 or not out.is_contiguous()):
        raise RuntimeError("out must be a contiguous float16 [M, N] tensor")
    if m == 0 or n == 0:
        return y
    if not fd.get("row_major", True):
        raise RuntimeError("this layer was packed without its row-major tensors: the prefill GEMM cannot run it")
    with _on_device(x.device):
        # scratch for problems with few tiles (the library then splits the k range); the
        # per-device buffer only grows and is reused by later calls on the same stream order
        need = ctypes.c_size_t(0)
        _lib.check(_lib.lib().rdq_gemm_workspace_size(m, n, k, ctypes.byref(need)), "rdq_gemm_workspace_size")
        ws = None
        if need.value:
            ws = _gemm_ws.get(x.device)
            if ws is None or ws.numel() < need.value:
                ws = torch.empty(need.value, dtype=torch.uint8, device=x.device)
                _gemm_ws[x.device] = ws
        rc = _lib.lib().rdq_gemm_mixed_ws(
            _ptr(x), m, _ptr(fd.get("w_fp4_q")), _ptr(fd.get("w_fp4_scales")), float(fd.get("w_fp4_global_scale", 1.0)),
            _ptr(fd.get("w_fp8_q")), _ptr(fd.get("w_fp8_scales")), _ptr(fd.get("w_fp16")), _ptr(fd.get("inv_perm")),
            _ptr(bias), _ptr(y), n4, n8, n16, k, _ptr(ws), need.value, _stream(x.device))
    _lib.check(rc, "rdq_gemm_mixed")
    if VALIDATE:
        check_gemm_status(x.device)
    return y


def mixed_linear(x: torch.Tensor, fd: dict, bias: Optional[torch.Tensor] = None, flags: int = 0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GEMV for M <= 16, GEMM above."""
    if x.shape[0] <= MAX_GEMV_M:
        return mixed_gemv(x, fd, bias, flags, out=out)
    if fd["k"] % 64 == 0 and fd.get("row_major", True):
        return mixed_gemm(x, fd, bias, out=out)
    # the tensor-core GEMM tiles K in blocks of 64 and reads the row-major tensors; other K, and
    # layers packed without them, run the decode kernel over 16-row panels (the reference's
    # dense prefill takes any K, rdquant/inference.py:679-687)
    n = fd["n_fp4"] + fd["n_fp8"] + fd["n_fp16"]
    y = out if out is not None else torch.empty(x.shape[0], n, dtype=torch.float16, device=x.device)
    for r0 in range(0, x.shape[0], MAX_GEMV_M):
        mixed_gemv(x[r0:r0 + MAX_GEMV_M], fd, bias, flags, out=y[r0:r0 + MAX_GEMV_M])
    return y


def fused_mixed_gemv(x: torch.Tensor, w_fp4: torch.Tensor, w_fp4_scales: torch.Tensor, w_fp4_global_scale: float,
                     w_fp8: torch.Tensor, w_fp8_scales: torch.Tensor, inv_perm: torch.Tensor,
                     N_fp4: int, N_fp8: int, K: int) -> torch.Tensor:
    """Signature of the reference's ``rdquant_cuda.fused_mixed_gemv``
    (rdquant/csrc/bindings.cpp:156-201) on row-major checkpoint tensors, for M <= 16.

    Output placement follows the operator's definition ``y[j] = y_perm[inv_perm[j]]``
    (rdquant/ops.py:62-63).
    """
    for name, t in (("w_fp4", w_fp4), ("w_fp4_scales", w_fp4_scales), ("w_fp8", w_fp8)):
        _need_cuda(name, t, torch.uint8)
    _need_cuda("w_fp8_scales", w_fp8_scales, torch.float32)
    _need_cuda("inv_perm", inv_perm)
    if x.dim() != 2 or x.size(1) != K:
        raise RuntimeError("x must be [M, K]")
    if w_fp4.size(0) != N_fp4 or w_fp8.size(0) != N_fp8:
        raise RuntimeError("weight rows must match N_fp4/N_fp8")
    if N_fp4 and (w_fp4.size(1) * 2 != K or tuple(w_fp4_scales.shape) != (N_fp4, K // 16)):
        raise RuntimeError("w_fp4 must be [N_fp4, K/2] and w_fp4_scales [N_fp4, K/16]")
    if N_fp8 and (w_fp8.size(1) != K or w_fp8_scales.numel() != N_fp8):
        raise RuntimeError("w_fp8 must be [N_fp8, K] and w_fp8_scales [N_fp8]")
    if inv_perm.numel() != N_fp4 + N_fp8:
        raise RuntimeError("inv_perm must have N_fp4 + N_fp8 elements")
    ws, cnt = _shared_scratch(x.device)
    fd = {
        "w_fp4_q": w_fp4 if N_fp4 else None, "w_fp4_scales": w_fp4_scales if N_fp4 else None,
        "w_fp4_global_scale": float(w_fp4_global_scale),
        "w_fp8_q": w_fp8 if N_fp8 else None, "w_fp8_scales": w_fp8_scales if N_fp8 else None,
        "w_fp16": None, "perm": perm_from_inv_perm(inv_perm), "workspace": ws, "tile_counters": cnt,
        "n_fp4": int(N_fp4), "n_fp8": int(N_fp8), "n_fp16": 0, "k": int(K),
    }
    return mixed_gemv(x, fd)


def quantize_nvfp4_packed(w: torch.Tensor, want_sqerr: bool = False) -> dict:
    """Encode a CUDA weight group ``[n, K]`` (f16 or f32, K % 16 == 0) as NVFP4 on the GPU.

    Returns the checkpoint tensors ``weight_nvfp4`` u8 [n, K/2] and ``weight_nvfp4_scale`` u8
    [n, K/16], bit-identical to the reference encoder + writer (rdquant/core/formats.py:84-142,
    rdquant/integrations/hf_export.py:81-92), ``global_scale`` (largest block scale; 0.0 for an
    all-zero group, which ``quantize.quantize_weight_packed`` stores as 1.0 like the reference) and, on request, ``row_sqerr`` f32 [n] = per-row sum of squared reconstruction errors.
    """
    _need_cuda("w", w)
    if w.dim() != 2 or w.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("quantize_nvfp4_packed expects a 2-D float16 or float32 CUDA tensor")
    w = w.contiguous()
    n, k = w.shape
    codes = torch.empty(n, k // 2, dtype=torch.uint8, device=w.device)
    scales = torch.empty(n, max(k // 16, 0), dtype=torch.uint8, device=w.device)
    sq = torch.empty(n, dtype=torch.float32, device=w.device) if want_sqerr else None
    top = torch.zeros(1, dtype=torch.float32, device=w.device)
    with _on_device(w.device):
        _lib.check(_lib.lib().rdq_quantize_nvfp4(_ptr(w), int(w.dtype == torch.float32), n, k, _ptr(codes), _ptr(scales),
                                                 _ptr(sq), _ptr(top), _stream(w.device)), "rdq_quantize_nvfp4")
    out = {"weight_nvfp4": codes, "weight_nvfp4_scale": scales, "global_scale": top}
    if want_sqerr:
        out["row_sqerr"] = sq
    return out


def quantize_fp8_packed(w: torch.Tensor, want_sqerr: bool = False) -> dict:
    """Encode a CUDA weight group ``[n, K]`` as FP8 (E4M3, one scale for the group) on the GPU.

    Returns ``weight_fp8`` u8 [n, K] and ``weight_fp8_scale`` f32 [n] (the group scale repeated),
    bit-identical to the reference (rdquant/core/formats.py:166-193,
    rdquant/integrations/hf_export.py:99-110), and optionally ``row_sqerr``.
    """
    _need_cuda("w", w)
    if w.dim() != 2 or w.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("quantize_fp8_packed expects a 2-D float16 or float32 CUDA tensor")
    w = w.contiguous()
    n, k = w.shape
    out8 = torch.empty(n, k, dtype=torch.uint8, device=w.device)
    sc = torch.empty(n, dtype=torch.float32, device=w.device)
    sq = torch.empty(n, dtype=torch.float32, device=w.device) if want_sqerr else None
    scratch = torch.zeros(1, dtype=torch.float32, device=w.device)
    with _on_device(w.device):
        _lib.check(_lib.lib().rdq_quantize_fp8(_ptr(w), int(w.dtype == torch.float32), n, k, _ptr(out8), _ptr(sc), _ptr(sq),
                                               _ptr(scratch), _stream(w.device)), "rdq_quantize_fp8")
    out = {"weight_fp8": out8, "weight_fp8_scale": sc}
    if want_sqerr:
        out["row_sqerr"] = sq
    return out


def stage_copy(dst: torch.Tensor, src: torch.Tensor, state: Optional[torch.Tensor] = None,
               flag: Optional[torch.Tensor] = None) -> None:
    """Copy ``src`` into ``dst`` (same byte size, contiguous) with a small kernel on the current
    stream.  One side lives on the GPU, the other may be pinned host memory: inside a CUDA
    graph this replaces a memcpy node and its fixed latency.

    With ``state`` (two zeroed CUDA int32) and ``flag`` (one pinned host int32) the kernel then
    writes the number of such copies completed so far to ``flag``: the host may poll it
    instead of synchronising the stream."""
    dev_t = dst if dst.is_cuda else src
    if not dev_t.is_cuda:
        raise RuntimeError("stage_copy needs one CUDA tensor")
    for t in (dst, src):
        if not t.is_contiguous() or not (t.is_cuda or t.is_pinned()):
            raise RuntimeError("stage_copy expects contiguous CUDA or pinned host tensors")
    nbytes = dst.numel() * dst.element_size()
    if nbytes != src.numel() * src.element_size():
        raise RuntimeError("stage_copy: size mismatch")
    if (state is None) != (flag is None):
        raise RuntimeError("stage_copy: state and flag go together")
    with _on_device(dev_t.device):
        if flag is None:
            _lib.check(_lib.lib().rdq_stage_copy(_ptr(dst), _ptr(src), nbytes, _stream(dev_t.device)), "rdq_stage_copy")
        else:
            if not (state.is_cuda and state.dtype == torch.int32 and state.numel() >= 2 and flag.is_pinned()
                    and flag.dtype == torch.int32):
                raise RuntimeError("stage_copy: state must be 2 CUDA int32, flag a pinned host int32")
            _lib.check(_lib.lib().rdq_stage_copy_signal(_ptr(dst), _ptr(src), nbytes, _ptr(state), _ptr(flag),
                                                        _stream(dev_t.device)), "rdq_stage_copy_signal")


# ---- decode-step glue (rdq_glue.cu): thin wrappers, all tensors preallocated by the caller

def _need_f16(name: str, t: torch.Tensor) -> None:
    _need_cuda(name, t, torch.float16)


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float, flags: int = 0) -> torch.Tensor:
    """``x += delta`` (in place; ``delta`` may be None) and ``out = rmsnorm(x) * weight``; x, out ``[B, H]``."""
    for name, t in (("x", x), ("weight", weight), ("out", out)):
        _need_f16(name, t)
    if delta is not None:
        _need_f16("delta", delta)
        if delta.shape != x.shape:
            raise RuntimeError("delta must have the shape of x")
    b, h = x.shape
    if out.shape != x.shape or weight.numel() != h:
        raise RuntimeError("add_rmsnorm: shape mismatch")
    with _on_device(x.device):
        rc = _lib.lib().rdq_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(weight), _ptr(out), b, h, float(eps), int(flags),
                                        _stream(x.device))
    _lib.check(rc, "rdq_add_rmsnorm")
    return out


def qk_rope_cache(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], cos: torch.Tensor,
                  sin: torch.Tensor, pos: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  eps: float, flags: int = 0) -> None:
    """Per-head q/k RMSNorm (optional) + rotary embedding at position ``pos`` (int64 device scalar);
    q -> ``q_out [B, nq, dh]``, k / v -> ``k_cache`` / ``v_cache [B, nkv, S, dh]`` row ``pos``."""
    for name, t in (("qkv", qkv), ("cos", cos), ("sin", sin), ("q_out", q_out), ("k_cache", k_cache), ("v_cache", v_cache)):
        _need_f16(name, t)
    _need_cuda("pos", pos, torch.int64)
    b, nq, dh = q_out.shape
    _, nkv, s, _ = k_cache.shape
    if qkv.shape != (b, (nq + 2 * nkv) * dh) or v_cache.shape != k_cache.shape or cos.shape != (s, dh) or sin.shape != (s, dh):
        raise RuntimeError("qk_rope_cache: shape mismatch")
    with _on_device(qkv.device):
        rc = _lib.lib().rdq_qk_rope_cache(_ptr(qkv), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin), _ptr(pos), _ptr(q_out),
                                          _ptr(k_cache), _ptr(v_cache), b, nq, nkv, dh, s, float(eps), int(flags),
                                          _stream(qkv.device))
    _lib.check(rc, "rdq_qk_rope_cache")


def attn_decode_scratch(b: int, nq: int, dh: int, s: int, device) -> torch.Tensor:
    need = ctypes.c_size_t(0)
    _lib.check(_lib.lib().rdq_attn_decode_scratch_size(b, nq, dh, s, ctypes.byref(need)), "rdq_attn_decode_scratch_size")
    return torch.empty(max(need.value // 4, 1), dtype=torch.float32, device=device)


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: torch.Tensor, scratch: torch.Tensor,
                out: torch.Tensor, scale: float, flags: int = 0) -> torch.Tensor:
    """``out [B, nq * dh] = softmax(q K^T * scale) V`` over cache rows ``0 .. pos`` (grouped-query)."""
    for name, t in (("q", q), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _need_f16(name, t)
    _need_cuda("pos", pos, torch.int64)
    _need_cuda("scratch", scratch, torch.float32)
    b, nq, dh = q.shape
    _, nkv, s, _ = k_cache.shape
    if out.shape != (b, nq * dh):
        raise RuntimeError("attn_decode: out must be [B, nq * dh]")
    with _on_device(q.device):
        rc = _lib.lib().rdq_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(pos), _ptr(scratch), _ptr(out), b, nq, nkv,
                                        dh, s, float(scale), int(flags), _stream(q.device))
    _lib.check(rc, "rdq_attn_decode")
    return out


def rope_attn_scratch(b: int, nq: int, nkv: int, dh: int, s: int, device) -> torch.Tensor:
    """Zeroed scratch of :func:`rope_attn_decode` (arrival counters + per-split partials)."""
    need = ctypes.c_size_t(0)
    _lib.check(_lib.lib().rdq_rope_attn_decode_scratch_size(b, nq, nkv, dh, s, ctypes.byref(need)),
               "rdq_rope_attn_decode_scratch_size")
    return torch.zeros((need.value + 3) // 4, dtype=torch.float32, device=device)


def rope_attn_decode(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor], cos: torch.Tensor,
                     sin: torch.Tensor, pos: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, scratch: torch.Tensor,
                     out: torch.Tensor, nq: int, scale: float, eps: float, flags: int = 0) -> torch.Tensor:
    """:func:`qk_rope_cache` and :func:`attn_decode` as one launch: the new token's q / k are
    normalised and rotated, k / v written to cache row ``pos``, and ``out [B, nq * dh]`` is the
    attention of the new token over rows ``0 .. pos``."""
    for name, t in (("qkv", qkv), ("cos", cos), ("sin", sin), ("k_cache", k_cache), ("v_cache", v_cache), ("out", out)):
        _need_f16(name, t)
    _need_cuda("pos", pos, torch.int64)
    _need_cuda("scratch", scratch, torch.float32)
    b, nkv, s, dh = k_cache.shape
    if qkv.shape != (b, (nq + 2 * nkv) * dh) or out.shape != (b, nq * dh):
        raise RuntimeError("rope_attn_decode: qkv must be [B, (nq + 2 nkv) * dh] and out [B, nq * dh]")
    with _on_device(qkv.device):
        rc = _lib.lib().rdq_rope_attn_decode(_ptr(qkv), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin), _ptr(pos),
                                             _ptr(k_cache), _ptr(v_cache), _ptr(scratch), _ptr(out), b, nq, nkv, dh, s,
                                             float(scale), float(eps), int(flags), _stream(qkv.device))
    _lib.check(rc, "rdq_rope_attn_decode")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, flags: int = 0) -> torch.Tensor:
    """``out [B, F] = silu(gate_up[:, :F]) * gate_up[:, F:]``."""
    _need_f16("gate_up", gate_up)
    _need_f16("out", out)
    b, f = out.shape
    if gate_up.shape != (b, 2 * f):
        raise RuntimeError("silu_mul: gate_up must be [B, 2 F]")
    with _on_device(out.device):
        rc = _lib.lib().rdq_silu_mul(_ptr(gate_up), _ptr(out), b, f, int(flags), _stream(out.device))
    _lib.check(rc, "rdq_silu_mul")
    return out
