"""Dense hidden weights: ``gh = fq_in(h) @ Wh_cat^T + bh_cat``.

Python surface of ``gru_qat.triton_kernels.scan`` (src/gru_qat/triton_kernels/scan.py):
``gru_scan_persistent`` / ``gru_scan`` and the non-autograd forward / backward
entry points, all routed to the sm_100a cluster kernels of ``libb200gru.so``.
There is one CUDA implementation; the "persistent" and "autotuned" names of the
reference both land on it, and the tile keyword arguments are accepted and ignored.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import torch_ref
from ._scan_common import (check_quant, common_shapes, make_scan_function, prep, require_cuda,
                           require_f32, run_backward, run_forward)

Quant = Optional[Tuple[float, int, int]]


def _validate(gi, h0, Wh_cat, bh_cat, h_in_quant, h_out_quant, out=None, dout=None):
    extra = {k: v for k, v in (("out", out), ("dout", dout)) if v is not None}
    require_cuda(gi=gi, h0=h0, Wh_cat=Wh_cat, bh_cat=bh_cat, **extra)
    require_f32(gi=gi, h0=h0, Wh_cat=Wh_cat, bh_cat=bh_cat, **extra)
    T, B, H = common_shapes(gi, h0, bh_cat)
    if tuple(Wh_cat.shape) != (3 * H, H):
        raise ValueError(f"Wh_cat shape must be (3H, H)=({3 * H}, {H}); got {tuple(Wh_cat.shape)}")
    for name, t in extra.items():
        if tuple(t.shape) != (T, B, H):
            raise ValueError(f"{name} shape must be (T, B, H)=({T}, {B}, {H}); got {tuple(t.shape)}")
    check_quant("h_in_quant", h_in_quant)
    check_quant("h_out_quant", h_out_quant)


def _forward_impl(gi, h0, Wh_cat, bh_cat, *, h_in_quant=None, h_out_quant=None, _want_save=False):
    _validate(gi, h0, Wh_cat, bh_cat, h_in_quant, h_out_quant)
    gi, h0, Wh_cat, bh_cat = prep(gi, h0, Wh_cat, bh_cat)
    return run_forward("dense", gi, h0, Wh_cat, bh_cat, h_in_quant, h_out_quant, want_save=_want_save)


def _backward_impl(gi, h0, Wh_cat, bh_cat, out, dout, *, h_in_quant=None, h_out_quant=None, _save=None):
    _validate(gi, h0, Wh_cat, bh_cat, h_in_quant, h_out_quant, out, dout)
    gi, h0, Wh_cat, bh_cat, out, dout = prep(gi, h0, Wh_cat, bh_cat, out, dout)
    return run_backward("dense", gi, h0, Wh_cat, bh_cat, out, dout, _save, h_in_quant, h_out_quant)


def gru_scan_forward_persistent(gi, h0, Wh_cat, bh_cat, *, block_b=8, block_oh=128, block_k=32,
                                num_warps=4, num_stages=2, h_in_quant: Quant = None,
                                h_out_quant: Quant = None) -> torch.Tensor:
    """out[T,B,H] of the whole scan in one launch (scan.py:213-293)."""
    return _forward_impl(gi, h0, Wh_cat, bh_cat, h_in_quant=h_in_quant, h_out_quant=h_out_quant)[0]


def gru_scan_backward_persistent(gi, h0, Wh_cat, bh_cat, out, dout, *, block_b=16, block_oh=64,
                                 block_k=32, num_warps=4, num_stages=2, h_in_quant: Quant = None,
                                 h_out_quant: Quant = None):
    """(dgi, dh0, dWh, dbh) (scan.py:646-752)."""
    return _backward_impl(gi, h0, Wh_cat, bh_cat, out, dout, h_in_quant=h_in_quant,
                          h_out_quant=h_out_quant)


def gru_scan_forward(gi, h0, Wh_cat, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Same contract as the persistent forward (scan.py:1688-1765)."""
    return _forward_impl(gi, h0, Wh_cat, bh_cat, h_in_quant=h_in_quant, h_out_quant=h_out_quant)[0]


def gru_scan_backward_cuda(gi, h0, Wh_cat, bh_cat, out, dout, *, h_in_quant: Quant = None,
                           h_out_quant: Quant = None):
    """Same contract as the persistent backward (scan.py:1355-1447)."""
    return _backward_impl(gi, h0, Wh_cat, bh_cat, out, dout, h_in_quant=h_in_quant,
                          h_out_quant=h_out_quant)


gru_scan_backward_triton = gru_scan_backward_cuda      # the reference's name for this entry point


def _gru_scan_backward_pytorch(gi, h0, Wh_cat, bh_cat, out, dout, *, h_in_quant: Quant = None,
                               h_out_quant: Quant = None):
    """Plain-PyTorch reverse scan (scan.py:1460-1550); any device, slow."""
    return torch_ref.scan_backward("dense", gi, h0, Wh_cat, bh_cat, out, dout,
                                   h_in_quant=h_in_quant, h_out_quant=h_out_quant)


def gru_scan_forward_pytorch(gi, h0, Wh_cat, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Plain-PyTorch forward scan; any device, slow."""
    return torch_ref.scan_forward("dense", gi, h0, Wh_cat, bh_cat, h_in_quant=h_in_quant,
                                  h_out_quant=h_out_quant)


_USE_NATIVE_BACKWARD = True     # False: autograd uses the plain-PyTorch backward instead


def _dispatch_backward(gi, h0, Wh_cat, bh_cat, out, dout, *, h_in_quant=None, h_out_quant=None, _save=None):
    if _USE_NATIVE_BACKWARD:
        return _backward_impl(gi, h0, Wh_cat, bh_cat, out, dout, h_in_quant=h_in_quant,
                              h_out_quant=h_out_quant, _save=_save)
    return _gru_scan_backward_pytorch(gi, h0, Wh_cat, bh_cat, out, dout, h_in_quant=h_in_quant,
                                      h_out_quant=h_out_quant)


GRUScanPersistentFunction = make_scan_function("persistent", _forward_impl, _dispatch_backward)
GRUScanFunction = GRUScanPersistentFunction


def gru_scan_persistent(gi, h0, Wh_cat, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Differentiable dense scan: ``out[T,B,H]`` (scan.py:1667-1685).

    ``gi[T,B,3H]`` is the input projection with bias, gates stacked r,z,n; ``Wh_cat[3H,H]``
    and ``bh_cat[3H]`` likewise.  ``h_in_quant`` / ``h_out_quant`` = ``(scale, qmin, qmax)``
    enable the frozen per-tensor symmetric fake-quant of h inside the kernel."""
    return GRUScanPersistentFunction.apply(gi, h0, Wh_cat, bh_cat, h_in_quant, h_out_quant)


def gru_scan(gi, h0, Wh_cat, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Same as :func:`gru_scan_persistent` (scan.py:1607-1627)."""
    return GRUScanFunction.apply(gi, h0, Wh_cat, bh_cat, h_in_quant, h_out_quant)
