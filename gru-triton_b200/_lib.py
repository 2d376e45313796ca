"""ctypes binding of ``libb200gru.so`` (the C ABI declared in ``include/b200gru.h``).

The library is built in-tree by ``build.py``.  There is no fallback: if it is
missing, or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional, Tuple

import torch

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("B200GRU_LIB", os.path.join(PKG_DIR, "lib", "libb200gru.so"))

KIND = {"dense": 0, "diagonal": 1, "monarch": 2, "butterfly": 3}
Quant = Optional[Tuple[float, int, int]]


class CQuant(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_float), ("qmin", ctypes.c_int), ("qmax", ctypes.c_int),
                ("enabled", ctypes.c_int)]


class CShape(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("T", ctypes.c_int), ("B", ctypes.c_int), ("H", ctypes.c_int),
                ("nblocks", ctypes.c_int), ("log2_hpad", ctypes.c_int)]


class CGemmArgs(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int), ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("A", ctypes.c_void_p), ("B", ctypes.c_void_p),
                ("a_planes", ctypes.c_int), ("b_planes", ctypes.c_int),
                ("a_mn_major", ctypes.c_int), ("b_mn_major", ctypes.c_int),
                ("lda", ctypes.c_longlong), ("ldb", ctypes.c_longlong),
                ("a_plane_stride", ctypes.c_longlong), ("b_plane_stride", ctypes.c_longlong),
                ("npairs", ctypes.c_int), ("pair_a", ctypes.c_int * 9), ("pair_b", ctypes.c_int * 9),
                ("split_k", ctypes.c_int), ("tile_n", ctypes.c_int), ("chunk_kblocks", ctypes.c_int), ("accumulate", ctypes.c_int),
                ("alpha", ctypes.c_float),
                ("row_scale", ctypes.c_void_p), ("col_scale", ctypes.c_void_p), ("bias", ctypes.c_void_p),
                ("C", ctypes.c_void_p), ("ldc", ctypes.c_longlong), ("split_stride", ctypes.c_longlong)]


_P = ctypes.c_void_p
_GP = ctypes.POINTER(CGemmArgs)
_QP = ctypes.POINTER(CQuant)
_SP = ctypes.POINTER(CShape)
_I = ctypes.c_int
_Z = ctypes.c_size_t

# name -> (restype, argtypes); every symbol include/b200gru.h declares
SIGNATURES = {
    "b200gru_workspace_bytes": (_Z, [_SP, _I]),
    "b200gru_save_bytes": (_Z, [_SP]),
    "b200gru_scan_forward": (_I, [_SP, _P, _P, _P, _P, _QP, _QP, _P, _P, _P, _Z, _P]),
    "b200gru_scan_backward": (_I, [_SP, _P, _P, _P, _P, _P, _P, _P, _QP, _QP, _P, _P, _P, _P, _P, _Z, _P]),
    "b200gru_dense_forward": (_I, [_P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P, _P, _Z, _P]),
    "b200gru_dense_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P, _P, _P, _P, _Z, _P]),
    "b200gru_diagonal_forward": (_I, [_P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P]),
    "b200gru_diagonal_backward": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P, _P, _P, _P, _Z, _P]),
    "b200gru_monarch_forward": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _QP, _QP, _P, _P, _P, _Z, _P]),
    "b200gru_monarch_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _QP, _QP, _P, _P, _P, _P, _P, _Z, _P]),
    "b200gru_butterfly_forward": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _QP, _QP, _P, _P, _P, _Z, _P]),
    "b200gru_butterfly_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _QP, _QP, _P, _P, _P, _P, _P, _Z, _P]),
    "b200gru_diagonal_backward_noalloc": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P, _P, _P, _P]),
    "b200gru_quantize_rows": (_I, [_P, _I, _I, _I, _P, _P, _P, _P]),
    "b200gru_quantize_rows_backward": (_I, [_P, _P, _I, _I, _I, _P, _P]),
    "b200gru_dense_q8_forward": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P, _P, _Z, _P]),
    "b200gru_dense_q8_backward": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _QP, _QP, _P, _P, _P, _P,
                                       _P, _Z, _P]),
    "b200gru_tc_gemm": (_I, [_GP, _P]),
    "b200gru_tc_gemm_splits": (_I, [_GP, _I]),
    "b200gru_split_bf16": (_I, [_P, _P, _Z, _Z, _I, _P, _I, _P]),
    "b200gru_split_f16": (_I, [_P, _P, _I, _I, _Z, _P, _P]),
    "b200gru_column_sums_workspace_bytes": (_Z, [_Z, _I]),
    "b200gru_column_sums": (_I, [_P, _Z, _I, _P, _P, _Z, _P]),
    "b200gru_calibration_workspace_bytes": (_Z, [_SP]),
    "b200gru_calibration_scan": (_I, [_SP, _P, _P, _P, _P, _I, ctypes.c_double, _P, _P, _I, _P, _P, _I, _P, _P, _Z, _P]),
    "b200gru_device_status": (_I, [_I]),
    "b200gru_test_select_kernels": (None, [_I, _I]),
    "b200gru_test_wait_timeout": (_I, [_P]),
    "b200gru_launch_count": (ctypes.c_ulonglong, []),
    "b200gru_strerror": (ctypes.c_char_p, [_I]),
    "b200gru_last_cuda_error": (ctypes.c_char_p, []),
    "b200gru_version": (_I, []),
}

_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library once and type its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"CUDA library not found at {LIB_PATH}. Build it first: "
                    "python gru-triton_b200/build.py  (there is no CPU or Triton fallback)")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
    return _lib


class DeviceWaitTimeout(RuntimeError):
    """A bounded in-kernel wait gave up: the results of the launches since the last check are invalid."""


def check_device_status(reset: bool = True) -> None:
    """Synchronise the current device and raise :class:`DeviceWaitTimeout` if any kernel of the
    library reported that one of its bounded waits ran out (``b200gru_device_status``)."""
    st = load().b200gru_device_status(1 if reset else 0)
    if st > 0:
        raise DeviceWaitTimeout("a bounded wait inside a b200gru kernel gave up (peer CTA, bulk copy or tensor-core "
                                "pipeline never delivered); results since the last check are invalid")
    if st < 0:
        raise RuntimeError("b200gru_device_status: CUDA error " + load().b200gru_last_cuda_error().decode())


# B200GRU_CHECK_STATUS=1: check the health word after every scan call (synchronises: a debugging aid).
# Without it the word is checked where the wrappers synchronise anyway (GRULayer.calibrate) and on demand.
_EAGER_STATUS = os.environ.get("B200GRU_CHECK_STATUS", "0") not in ("", "0")


def _after_call() -> None:
    if _EAGER_STATUS:
        check_device_status()


def _cquant(q: Quant) -> CQuant:
    if q is None:
        return CQuant(1.0, 0, 0, 0)
    scale, qmin, qmax = q
    return CQuant(float(scale), int(qmin), int(qmax), 1)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _raise(rc: int, what: str):
    lib = load()
    msg = lib.b200gru_strerror(rc).decode()
    detail = lib.b200gru_last_cuda_error().decode()
    text = f"{what}: {msg}" + (f" ({detail})" if detail and rc == 3 else "")
    raise (ValueError if rc == 1 else RuntimeError)(text)


def make_shape(kind: str, T: int, B: int, H: int, nblocks: int = 1, log2_hpad: int = 0) -> CShape:
    return CShape(KIND[kind], T, B, H, nblocks, log2_hpad)


def _workspace(lib, shape: CShape, backward: int, device) -> Optional[torch.Tensor]:
    n = lib.b200gru_workspace_bytes(ctypes.byref(shape), backward)
    if n == ctypes.c_size_t(-1).value:
        raise RuntimeError("shape not supported by the CUDA scan library")
    return torch.empty(n, dtype=torch.uint8, device=device) if n else None


def launch_count() -> int:
    return int(load().b200gru_launch_count())


def quantize_rows(W: torch.Tensor, bits: int = 8):
    """Per-output-row symmetric fake-quant of ``W[rows, cols]``: ``(codes int8, scales, Wq)``."""
    lib = load()
    W = W.contiguous()
    rows, cols = W.shape
    codes = torch.empty((rows, cols), device=W.device, dtype=torch.int8)
    scales = torch.empty((rows,), device=W.device, dtype=torch.float32)
    Wq = torch.empty_like(W)
    with torch.cuda.device(W.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200gru_quantize_rows(_ptr(W), rows, cols, bits, _ptr(codes), _ptr(scales), _ptr(Wq),
                                       ctypes.c_void_p(stream))
    if rc:
        _raise(rc, "quantize_rows")
    return codes, scales, Wq


def quantize_rows_backward(W: torch.Tensor, dWq: torch.Tensor, bits: int = 8) -> torch.Tensor:
    """Gradient of :func:`quantize_rows` with respect to ``W`` (straight-through, dynamic scale)."""
    lib = load()
    W, dWq = W.contiguous(), dWq.contiguous()
    rows, cols = W.shape
    dW = torch.empty_like(W)
    with torch.cuda.device(W.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200gru_quantize_rows_backward(_ptr(W), _ptr(dWq), rows, cols, bits, _ptr(dW), ctypes.c_void_p(stream))
    if rc:
        _raise(rc, "quantize_rows_backward")
    return dW


def column_sums(x: torch.Tensor) -> torch.Tensor:
    """``x.reshape(-1, x.shape[-1]).sum(0)`` in a fixed summation order (CUDA float32, contiguous)."""
    lib = load()
    x = x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    out = torch.empty((cols,), device=x.device, dtype=torch.float32)
    if rows == 0 or cols == 0:
        return out.zero_()
    n = lib.b200gru_column_sums_workspace_bytes(rows, cols)
    ws = torch.empty((max(n, 1),), device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200gru_column_sums(_ptr(x), rows, cols, _ptr(out), _ptr(ws), n, ctypes.c_void_p(stream))
    if rc:
        _raise(rc, "column_sums")
    return out


def scan_forward(kind: str, gi, h0, W, bh, h_in_quant: Quant, h_out_quant: Quant, *, nblocks: int = 1,
                 log2_hpad: int = 0, want_save: bool = False, codes=None, scales=None):
    """Run the forward scan on the current stream of ``gi``'s device.
    Returns ``(out, save)``; ``save`` is None unless asked for (and the kind has one).
    ``codes`` / ``scales`` (dense only): the int8 form of ``W`` from :func:`quantize_rows`."""
    lib = load()
    T, B, _ = gi.shape
    H = h0.shape[1]
    shape = make_shape(kind, T, B, H, nblocks, log2_hpad)
    out = torch.empty((T, B, H), device=gi.device, dtype=torch.float32)
    save = None
    if want_save and kind != "diagonal":
        save = torch.empty((4, T, B, H), device=gi.device, dtype=torch.float32)
    ws = _workspace(lib, shape, 0, gi.device)
    qi, qo = _cquant(h_in_quant), _cquant(h_out_quant)
    with torch.cuda.device(gi.device):
        stream = torch.cuda.current_stream().cuda_stream
        if codes is not None:
            rc = lib.b200gru_dense_q8_forward(_ptr(gi), _ptr(h0), _ptr(W), _ptr(codes), _ptr(scales), _ptr(bh), T, B, H,
                                              ctypes.byref(qi), ctypes.byref(qo), _ptr(out), _ptr(save), _ptr(ws),
                                              0 if ws is None else ws.numel(), ctypes.c_void_p(stream))
        else:
            rc = lib.b200gru_scan_forward(ctypes.byref(shape), _ptr(gi), _ptr(h0), _ptr(W), _ptr(bh),
                                          ctypes.byref(qi), ctypes.byref(qo), _ptr(out), _ptr(save), _ptr(ws),
                                          0 if ws is None else ws.numel(), ctypes.c_void_p(stream))
    if rc:
        _raise(rc, f"{kind} scan forward")
    _after_call()
    return out, save


def calibration_scan(kind: str, gi, h0, W, bh, qmax: int, momentum: float, in_stats, out_stats, *,
                     nblocks: int = 1, log2_hpad: int = 0):
    """Observing-mode forward scan.  ``in_stats`` / ``out_stats``: ``(min, max, initialized)`` with
    one-element float32 CUDA tensors that are updated in place.  Returns ``out[T,B,H]``."""
    lib = load()
    T, B, _ = gi.shape
    H = h0.shape[1]
    shape = make_shape(kind, T, B, H, nblocks, log2_hpad)
    out = torch.empty((T, B, H), device=gi.device, dtype=torch.float32)
    n = lib.b200gru_calibration_workspace_bytes(ctypes.byref(shape))
    if n == ctypes.c_size_t(-1).value:
        raise RuntimeError("shape not supported by the CUDA scan library")
    ws = torch.empty(n, dtype=torch.uint8, device=gi.device)
    with torch.cuda.device(gi.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200gru_calibration_scan(ctypes.byref(shape), _ptr(gi), _ptr(h0), _ptr(W), _ptr(bh), int(qmax),
                                          float(momentum), _ptr(in_stats[0]), _ptr(in_stats[1]), int(in_stats[2]),
                                          _ptr(out_stats[0]), _ptr(out_stats[1]), int(out_stats[2]), _ptr(out),
                                          _ptr(ws), ws.numel(), ctypes.c_void_p(stream))
    if rc:
        _raise(rc, f"{kind} calibration scan")
    _after_call()
    return out


def scan_backward(kind: str, gi, h0, W, bh, out, dout, save, h_in_quant: Quant, h_out_quant: Quant, *,
                  nblocks: int = 1, log2_hpad: int = 0, codes=None, scales=None):
    """Run the backward scan.  Returns ``(dgi, dh0, dW, dbh)``."""
    lib = load()
    T, B, _ = gi.shape
    H = h0.shape[1]
    shape = make_shape(kind, T, B, H, nblocks, log2_hpad)
    dgi = torch.empty_like(gi)
    dh0 = torch.empty_like(h0)
    dW = torch.empty_like(W)
    dbh = torch.empty_like(bh)
    ws = _workspace(lib, shape, 2 if save is not None else 1, gi.device)
    qi, qo = _cquant(h_in_quant), _cquant(h_out_quant)
    with torch.cuda.device(gi.device):
        stream = torch.cuda.current_stream().cuda_stream
        if codes is not None:
            rc = lib.b200gru_dense_q8_backward(_ptr(gi), _ptr(h0), _ptr(W), _ptr(codes), _ptr(scales), _ptr(bh),
                                               _ptr(out), _ptr(dout), _ptr(save), T, B, H, ctypes.byref(qi),
                                               ctypes.byref(qo), _ptr(dgi), _ptr(dh0), _ptr(dW), _ptr(dbh), _ptr(ws),
                                               0 if ws is None else ws.numel(), ctypes.c_void_p(stream))
        else:
            rc = lib.b200gru_scan_backward(ctypes.byref(shape), _ptr(gi), _ptr(h0), _ptr(W), _ptr(bh), _ptr(out),
                                           _ptr(dout), _ptr(save), ctypes.byref(qi), ctypes.byref(qo), _ptr(dgi),
                                           _ptr(dh0), _ptr(dW), _ptr(dbh), _ptr(ws),
                                           0 if ws is None else ws.numel(), ctypes.c_void_p(stream))
    if rc:
        _raise(rc, f"{kind} scan backward")
    _after_call()
    return dgi, dh0, dW, dbh
