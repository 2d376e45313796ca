"""Diagonal hidden weights: ``gh_g = w_g * fq_in(h) + b_g``.

Python surface of ``gru_qat.triton_kernels.scan_diagonal``
(src/gru_qat/triton_kernels/scan_diagonal.py), routed to the register-resident
streaming kernels of ``libb200gru.so``.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import torch_ref
from ._scan_common import (check_quant, common_shapes, make_scan_function, prep, require_cuda,
                           require_f32, run_backward, run_forward)

Quant = Optional[Tuple[float, int, int]]


def extract_diagonal_factors(cell: nn.Module):
    """``(Wh_diag[3,H], bh_cat[3H])`` of a cell built with a diagonal hidden side
    (scan_diagonal.py:33-63); zeros for a bias-free cell."""
    if cell._hidden_dense:
        raise ValueError("cell hidden side is dense; nothing to extract")
    Wh_diag = torch.stack([cell.struct_Wh_r.weight, cell.struct_Wh_z.weight, cell.struct_Wh_n.weight], dim=0)
    if cell.b_hr is None:
        bh_cat = torch.zeros(3 * cell.hidden_size, device=Wh_diag.device, dtype=Wh_diag.dtype)
    else:
        bh_cat = torch.cat([cell.b_hr, cell.b_hz, cell.b_hn])
    return Wh_diag, bh_cat


def _validate(gi, h0, Wh_diag, bh_cat, h_in_quant, h_out_quant, out=None, dout=None):
    extra = {k: v for k, v in (("out", out), ("dout", dout)) if v is not None}
    require_cuda(gi=gi, h0=h0, Wh_diag=Wh_diag, bh_cat=bh_cat, **extra)
    require_f32(gi=gi, h0=h0, Wh_diag=Wh_diag, bh_cat=bh_cat, **extra)
    T, B, H = common_shapes(gi, h0, bh_cat)
    if tuple(Wh_diag.shape) != (3, H):
        raise ValueError(f"Wh_diag shape must be (3, H)=(3, {H}); got {tuple(Wh_diag.shape)}")
    for name, t in extra.items():
        if tuple(t.shape) != (T, B, H):
            raise ValueError(f"{name} shape must be (T, B, H)=({T}, {B}, {H}); got {tuple(t.shape)}")
    check_quant("h_in_quant", h_in_quant)
    check_quant("h_out_quant", h_out_quant)


def _forward_impl(gi, h0, Wh_diag, bh_cat, *, h_in_quant=None, h_out_quant=None, _want_save=False):
    _validate(gi, h0, Wh_diag, bh_cat, h_in_quant, h_out_quant)
    gi, h0, Wh_diag, bh_cat = prep(gi, h0, Wh_diag, bh_cat)
    return run_forward("diagonal", gi, h0, Wh_diag, bh_cat, h_in_quant, h_out_quant)


def _backward_impl(gi, h0, Wh_diag, bh_cat, out, dout, *, h_in_quant=None, h_out_quant=None, _save=None):
    _validate(gi, h0, Wh_diag, bh_cat, h_in_quant, h_out_quant, out, dout)
    gi, h0, Wh_diag, bh_cat, out, dout = prep(gi, h0, Wh_diag, bh_cat, out, dout)
    return run_backward("diagonal", gi, h0, Wh_diag, bh_cat, out, dout, None, h_in_quant, h_out_quant)


def gru_scan_diagonal_forward_cuda(gi, h0, Wh_diag, bh_cat, *, block_b=32, block_h=64, num_warps=4,
                                   num_stages=2, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """out[T,B,H] (scan_diagonal.py:226-282); tile arguments are ignored."""
    return _forward_impl(gi, h0, Wh_diag, bh_cat, h_in_quant=h_in_quant, h_out_quant=h_out_quant)[0]


def gru_scan_diagonal_backward_cuda(gi, h0, Wh_diag, bh_cat, out, dout, *, block_b=32, block_h=64,
                                    num_warps=4, num_stages=2, h_in_quant: Quant = None,
                                    h_out_quant: Quant = None):
    """(dgi, dh0, dWh_diag[3,H], dbh[3H]) (scan_diagonal.py:490-561)."""
    return _backward_impl(gi, h0, Wh_diag, bh_cat, out, dout, h_in_quant=h_in_quant,
                          h_out_quant=h_out_quant)


gru_scan_diagonal_forward_triton = gru_scan_diagonal_forward_cuda
gru_scan_diagonal_backward_triton = gru_scan_diagonal_backward_cuda


def gru_scan_diagonal_forward_pytorch(gi, h0, Wh_diag, bh_cat, *, h_in_quant: Quant = None,
                                      h_out_quant: Quant = None):
    """Plain-PyTorch forward (scan_diagonal.py:79-124)."""
    return torch_ref.scan_forward("diagonal", gi, h0, Wh_diag, bh_cat, h_in_quant=h_in_quant,
                                  h_out_quant=h_out_quant)


def gru_scan_diagonal_backward_pytorch(gi, h0, Wh_diag, bh_cat, out, dout, *, h_in_quant: Quant = None,
                                       h_out_quant: Quant = None):
    """Plain-PyTorch backward (scan_diagonal.py:564-647)."""
    return torch_ref.scan_backward("diagonal", gi, h0, Wh_diag, bh_cat, out, dout,
                                   h_in_quant=h_in_quant, h_out_quant=h_out_quant)


GRUScanDiagonalFunction = make_scan_function("diagonal", _forward_impl, _backward_impl)


def gru_scan_diagonal(gi, h0, Wh_diag, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Differentiable diagonal scan (scan_diagonal.py:684-715)."""
    return GRUScanDiagonalFunction.apply(gi, h0, Wh_diag, bh_cat, h_in_quant, h_out_quant)
