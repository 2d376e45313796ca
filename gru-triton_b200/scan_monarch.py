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


# ---------------------------------------------------------------------------
# two-factor Monarch (extension; the reference's API has one factor per gate)
# ---------------------------------------------------------------------------

def monarch_permutation(nblocks: int, blksz: int, device=None) -> torch.Tensor:
    """Index vector of the Monarch (stride) permutation P of a length ``nblocks * blksz`` vector read
    as an ``[nblocks, blksz]`` grid: ``(P v)[j * nblocks + i] = v[i * blksz + j]``."""
    return torch.arange(nblocks * blksz, device=device).reshape(nblocks, blksz).t().reshape(-1)


def monarch2_dense(W1: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
    """``Wh_cat[3H, H]`` of the two-factor operator ``M_g = P^T . blockdiag(W2[g]) . P . blockdiag(W1[g])``
    (``W1``, ``W2``: ``[3, nblocks, blksz, blksz]``); differentiable in both factors."""
    _, nb, bs, _ = W1.shape
    perm = monarch_permutation(nb, bs, W1.device)
    inv = torch.argsort(perm)
    mats = []
    for g in range(3):
        B1 = torch.block_diag(*W1[g])
        B2 = torch.block_diag(*W2[g])
        mats.append((B2 @ B1[perm])[inv])
    return torch.cat(mats, dim=0)


def gru_scan_monarch2(gi, h0, W1, W2, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Differentiable scan with TWO block-diagonal factors per gate separated by the Monarch
    permutation, ``gh_g = P^T B2_g P B1_g fq_in(h) + bh_g`` -- the operator BASELINE config 3 words
    literally.  The reference cannot express it (one factor per gate, scan_monarch.py:110-112), so
    there is no reference parity for this entry point; its checker is a dense materialisation.

    The product couples all hidden units (it is no longer ``nblocks`` independent GRUs), so the scan
    itself runs on the dense kernels with the materialised ``[3H, H]`` matrix; gradients reach the
    two factors through the materialisation."""
    require_cuda(gi=gi, h0=h0, W1=W1, W2=W2, bh_cat=bh_cat)
    require_f32(gi=gi, h0=h0, W1=W1, W2=W2, bh_cat=bh_cat)
    T, B, H = common_shapes(gi, h0, bh_cat)
    if W1.dim() != 4 or W1.shape != W2.shape or W1.shape[0] != 3 or W1.shape[2] != W1.shape[3] \
            or W1.shape[1] * W1.shape[2] != H:
        raise ValueError("W1 and W2 must both be [3, nblocks, blksz, blksz] with nblocks * blksz == H; got "
                         f"{tuple(W1.shape)} and {tuple(W2.shape)} for H={H}")
    from .scan import gru_scan_persistent
    return gru_scan_persistent(gi, h0, monarch2_dense(W1, W2), bh_cat, h_in_quant=h_in_quant,
                               h_out_quant=h_out_quant)
