"""Block-diagonal ("monarch") hidden weights: one ``[nblocks, blksz, blksz]`` factor per gate.

Python surface of ``gru_qat.triton_kernels.scan_monarch``
(src/gru_qat/triton_kernels/scan_monarch.py).  Block n of h_t depends only on
block n of h_{t-1}, so the scan is nblocks independent small GRUs; the CUDA
kernels give each (block, batch tile) its own cluster and need no grid barrier.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import torch_ref
from ._scan_common import (check_quant, common_shapes, make_scan_function, prep, require_cuda,
                           require_f32, run_backward, run_forward)

Quant = Optional[Tuple[float, int, int]]


def extract_monarch_factors(cell: nn.Module):
    """``(Wh_struct[3,nblocks,blksz,blksz], bh_cat[3H])`` (scan_monarch.py:22-58)."""
    if cell._hidden_dense:
        raise ValueError("cell hidden side is dense; nothing to extract")
    Wh_struct = torch.stack([cell.struct_Wh_r.weight, cell.struct_Wh_z.weight, cell.struct_Wh_n.weight], dim=0)
    if cell.b_hr is None:
        bh_cat = torch.zeros(3 * cell.hidden_size, device=Wh_struct.device, dtype=Wh_struct.dtype)
    else:
        bh_cat = torch.cat([cell.b_hr, cell.b_hz, cell.b_hn])
    return Wh_struct, bh_cat


def _validate(gi, h0, Wh_struct, bh_cat, h_in_quant, h_out_quant, out=None, dout=None):
    extra = {k: v for k, v in (("out", out), ("dout", dout)) if v is not None}
    require_cuda(gi=gi, h0=h0, Wh_struct=Wh_struct, bh_cat=bh_cat, **extra)
    require_f32(gi=gi, h0=h0, Wh_struct=Wh_struct, bh_cat=bh_cat, **extra)
    T, B, H = common_shapes(gi, h0, bh_cat)
    if Wh_struct.dim() != 4 or Wh_struct.shape[0] != 3:
        raise ValueError("Wh_struct must be [3, nblocks, blksz, blksz]; got shape "
                         f"{tuple(Wh_struct.shape)}")
    _, nblocks, ob, ib = Wh_struct.shape
    if nblocks == 0 or not (ob == ib == H // nblocks) or nblocks * ob != H:
        raise ValueError("Wh_struct block dims must be square and tile H: expected out_blksz == "
                         f"in_blksz == H // nblocks; got out_blksz={ob}, in_blksz={ib}, H={H}, "
                         f"nblocks={nblocks}")
    for name, t in extra.items():
        if tuple(t.shape) != (T, B, H):
            raise ValueError(f"{name} shape must be (T, B, H)=({T}, {B}, {H}); got {tuple(t.shape)}")
    check_quant("h_in_quant", h_in_quant)
    check_quant("h_out_quant", h_out_quant)
    return nblocks


def _forward_impl(gi, h0, Wh_struct, bh_cat, *, h_in_quant=None, h_out_quant=None, _want_save=False):
    nb = _validate(gi, h0, Wh_struct, bh_cat, h_in_quant, h_out_quant)
    gi, h0, Wh_struct, bh_cat = prep(gi, h0, Wh_struct, bh_cat)
    return run_forward("monarch", gi, h0, Wh_struct, bh_cat, h_in_quant, h_out_quant, nblocks=nb,
                       want_save=_want_save)


def _backward_impl(gi, h0, Wh_struct, bh_cat, out, dout, *, h_in_quant=None, h_out_quant=None, _save=None):
    nb = _validate(gi, h0, Wh_struct, bh_cat, h_in_quant, h_out_quant, out, dout)
    gi, h0, Wh_struct, bh_cat, out, dout = prep(gi, h0, Wh_struct, bh_cat, out, dout)
    return run_backward("monarch", gi, h0, Wh_struct, bh_cat, out, dout, _save, h_in_quant, h_out_quant,
                        nblocks=nb)


def gru_scan_monarch_forward_cuda(gi, h0, Wh_struct, bh_cat, *, block_b=None, block_k=None, num_warps=4,
                                  num_stages=None, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """out[T,B,H] (scan_monarch.py:320-406); tile arguments are ignored."""
    return _forward_impl(gi, h0, Wh_struct, bh_cat, h_in_quant=h_in_quant, h_out_quant=h_out_quant)[0]


def gru_scan_monarch_backward_cuda(gi, h0, Wh_struct, bh_cat, out, dout, *, block_b=None, block_k=None,
                                   num_warps=4, num_stages=None, h_in_quant: Quant = None,
                                   h_out_quant: Quant = None):
    """(dgi, dh0, dWh_struct, dbh) (scan_monarch.py:776-884)."""
    return _backward_impl(gi, h0, Wh_struct, bh_cat, out, dout, h_in_quant=h_in_quant,
                          h_out_quant=h_out_quant)


gru_scan_monarch_forward_triton = gru_scan_monarch_forward_cuda
gru_scan_monarch_backward_triton = gru_scan_monarch_backward_cuda


def gru_scan_monarch_forward_pytorch(gi, h0, Wh_struct, bh_cat, *, h_in_quant: Quant = None,
                                     h_out_quant: Quant = None):
    """Plain-PyTorch forward (scan_monarch.py:74-127)."""
    return torch_ref.scan_forward("monarch", gi, h0, Wh_struct, bh_cat, h_in_quant=h_in_quant,
                                  h_out_quant=h_out_quant)


def gru_scan_monarch_backward_pytorch(gi, h0, Wh_struct, bh_cat, out, dout, *, h_in_quant: Quant = None,
                                      h_out_quant: Quant = None):
    """Plain-PyTorch backward (scan_monarch.py:955-1053)."""
    return torch_ref.scan_backward("monarch", gi, h0, Wh_struct, bh_cat, out, dout,
                                   h_in_quant=h_in_quant, h_out_quant=h_out_quant)


GRUScanMonarchFunction = make_scan_function("monarch", _forward_impl, _backward_impl)


def gru_scan_monarch(gi, h0, Wh_struct, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Differentiable block-diagonal scan (scan_monarch.py:927-952)."""
    return GRUScanMonarchFunction.apply(gi, h0, Wh_struct, bh_cat, h_in_quant, h_out_quant)
