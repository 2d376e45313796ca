"""Butterfly hidden weights: ``nblocks * log2(H_pad)`` stages of 2x2 mixing per gate.

Python surface of ``gru_qat.triton_kernels.scan_butterfly``
(src/gru_qat/triton_kernels/scan_butterfly.py).  ``twiddles`` is
``[3, nblocks, log2(H_pad), H_pad/2, 2, 2]``; H itself may be smaller than the
power of two H_pad (zero padding).
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from . import torch_ref
from ._scan_common import (check_quant, common_shapes, make_scan_function, prep, require_cuda,
                           require_f32, run_backward, run_forward)
from .ste import fake_quant_ste

Quant = Optional[Tuple[float, int, int]]


def _bias_cat(cell, like):
    if cell.b_hr is None:
        return torch.zeros(3 * cell.hidden_size, device=like.device, dtype=like.dtype)
    return torch.cat([cell.b_hr, cell.b_hz, cell.b_hn])


def extract_butterfly_factors(cell: nn.Module):
    """The three per-gate butterfly modules and ``bh_cat`` (scan_butterfly.py:52-94)."""
    if cell._hidden_dense:
        raise ValueError("cell hidden side is dense; nothing to extract")
    modules: List[nn.Module] = [cell.struct_Wh_r.b, cell.struct_Wh_z.b, cell.struct_Wh_n.b]
    return modules, _bias_cat(cell, next(modules[0].parameters()))


def extract_butterfly_twiddles(cell: nn.Module):
    """``(twiddles[3,nblocks,log_n,n/2,2,2], bh_cat[3H])`` (scan_butterfly.py:1142-1182)."""
    if cell._hidden_dense:
        raise ValueError("cell hidden side is dense; nothing to extract")
    tw = torch.stack([getattr(cell, f"struct_Wh_{g}").b.twiddle.squeeze(0) for g in "rzn"], dim=0)
    return tw, _bias_cat(cell, tw)


def gru_scan_butterfly(gi, h0, butterfly_modules, bh_cat, *, h_in_quant: Quant = None,
                       h_out_quant: Quant = None):
    """Per-step Python loop over the butterfly modules with autograd
    (scan_butterfly.py:109-160); any device.  The fused CUDA scan is
    :func:`gru_scan_butterfly_cuda`."""
    T, _, three_h = gi.shape
    H = three_h // 3

    def fq(x, params):
        if params is None:
            return x
        s, lo, hi = params
        return fake_quant_ste(x, torch.tensor(s, device=x.device, dtype=x.dtype),
                              torch.tensor(0.0, device=x.device, dtype=x.dtype), lo, hi)

    Wr, Wz, Wn = butterfly_modules
    bh = bh_cat.view(3, H)
    h, outs = h0, []
    for t in range(T):
        hq = fq(h, h_in_quant)
        r = torch.sigmoid(gi[t, :, :H] + Wr(hq) + bh[0])
        z = torch.sigmoid(gi[t, :, H:2 * H] + Wz(hq) + bh[1])
        n = torch.tanh(gi[t, :, 2 * H:] + r * (Wn(hq) + bh[2]))
        h = fq((1.0 - z) * n + z * h, h_out_quant)
        outs.append(h)
    return torch.stack(outs, dim=0)


def _validate(gi, h0, twiddles, bh_cat, h_in_quant, h_out_quant, out=None, dout=None):
    extra = {k: v for k, v in (("out", out), ("dout", dout)) if v is not None}
    require_cuda(gi=gi, h0=h0, twiddles=twiddles, bh_cat=bh_cat, **extra)
    require_f32(gi=gi, h0=h0, twiddles=twiddles, bh_cat=bh_cat, **extra)
    T, B, H = common_shapes(gi, h0, bh_cat)
    if twiddles.dim() != 6 or twiddles.shape[0] != 3 or tuple(twiddles.shape[4:]) != (2, 2):
        raise ValueError("twiddles shape must be (3, nblocks, log_H, H//2, 2, 2); got "
                         f"{tuple(twiddles.shape)}")
    _, nblocks, log_n, half, _, _ = twiddles.shape
    h_pad = 2 * half
    if nblocks == 0 or not (h_pad >= H and h_pad & (h_pad - 1) == 0):
        raise ValueError(f"twiddles imply H_PAD={h_pad}, which must be >= H={H} and a power of two "
                         f"(shape {tuple(twiddles.shape)})")
    if 1 << log_n != h_pad:
        raise ValueError(f"twiddles log_H={log_n} inconsistent with H_PAD={h_pad}: expected "
                         f"1 << log_H == H_PAD (shape {tuple(twiddles.shape)})")
    for name, t in extra.items():
        if tuple(t.shape) != (T, B, H):
            raise ValueError(f"{name} shape must be (T, B, H)=({T}, {B}, {H}); got {tuple(t.shape)}")
    check_quant("h_in_quant", h_in_quant)
    check_quant("h_out_quant", h_out_quant)
    return nblocks, log_n


def _forward_impl(gi, h0, twiddles, bh_cat, *, h_in_quant=None, h_out_quant=None, _want_save=False):
    nb, log_n = _validate(gi, h0, twiddles, bh_cat, h_in_quant, h_out_quant)
    gi, h0, twiddles, bh_cat = prep(gi, h0, twiddles, bh_cat)
    return run_forward("butterfly", gi, h0, twiddles, bh_cat, h_in_quant, h_out_quant, nblocks=nb,
                       log2_hpad=log_n, want_save=_want_save)


def _backward_impl(gi, h0, twiddles, bh_cat, out, dout, *, h_in_quant=None, h_out_quant=None, _save=None):
    nb, log_n = _validate(gi, h0, twiddles, bh_cat, h_in_quant, h_out_quant, out, dout)
    gi, h0, twiddles, bh_cat, out, dout = prep(gi, h0, twiddles, bh_cat, out, dout)
    return run_backward("butterfly", gi, h0, twiddles, bh_cat, out, dout, _save, h_in_quant, h_out_quant,
                        nblocks=nb, log2_hpad=log_n)


def gru_scan_butterfly_forward_cuda(gi, h0, twiddles, bh_cat, *, block_b=8, num_warps=4, num_stages=1,
                                    h_in_quant: Quant = None, h_out_quant: Quant = None):
    """out[T,B,H] (scan_butterfly.py:369-459); tile arguments are ignored."""
    return _forward_impl(gi, h0, twiddles, bh_cat, h_in_quant=h_in_quant, h_out_quant=h_out_quant)[0]


def gru_scan_butterfly_backward_cuda(gi, h0, twiddles, bh_cat, out, dout, *, block_b=8, num_warps=4,
                                     num_stages=1, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """(dgi, dh0, dtwiddles, dbh) (scan_butterfly.py:971-1075)."""
    return _backward_impl(gi, h0, twiddles, bh_cat, out, dout, h_in_quant=h_in_quant,
                          h_out_quant=h_out_quant)


gru_scan_butterfly_forward_triton = gru_scan_butterfly_forward_cuda
gru_scan_butterfly_backward_triton = gru_scan_butterfly_backward_cuda


def gru_scan_butterfly_forward_pytorch(gi, h0, twiddles, bh_cat, *, h_in_quant: Quant = None,
                                       h_out_quant: Quant = None):
    """Plain-PyTorch forward of the same stage arithmetic; any device, slow."""
    return torch_ref.scan_forward("butterfly", gi, h0, twiddles, bh_cat, h_in_quant=h_in_quant,
                                  h_out_quant=h_out_quant)


def gru_scan_butterfly_backward_pytorch(gi, h0, twiddles, bh_cat, out, dout, *, h_in_quant: Quant = None,
                                        h_out_quant: Quant = None):
    """Plain-PyTorch backward; any device, slow."""
    return torch_ref.scan_backward("butterfly", gi, h0, twiddles, bh_cat, out, dout,
                                   h_in_quant=h_in_quant, h_out_quant=h_out_quant)


GRUScanButterflyFunction = make_scan_function("butterfly", _forward_impl, _backward_impl)
GRUScanButterflyTritonFunction = GRUScanButterflyFunction


def gru_scan_butterfly_cuda(gi, h0, twiddles, bh_cat, *, h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Differentiable butterfly scan (scan_butterfly.py:1115-1139)."""
    return GRUScanButterflyFunction.apply(gi, h0, twiddles, bh_cat, h_in_quant, h_out_quant)


gru_scan_butterfly_triton = gru_scan_butterfly_cuda
