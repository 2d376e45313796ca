"""Validation and autograd plumbing shared by the four scan modules."""

from __future__ import annotations

from typing import Any

import torch

from . import _lib


def require_cuda(**tensors) -> None:
    bad = {k: v.device for k, v in tensors.items() if not v.is_cuda}
    if bad:
        raise ValueError("the CUDA scan needs CUDA tensors; got " +
                         ", ".join(f"{k}={d}" for k, d in bad.items()))


def require_f32(**tensors) -> None:
    for k, v in tensors.items():
        if v.dtype != torch.float32:
            raise ValueError(f"{k} dtype must be float32; got {v.dtype}")


def common_shapes(gi, h0, bh_cat):
    """Check gi[T,B,3H], h0[B,H], bh_cat[3H]; T and B must be positive."""
    if gi.dim() != 3 or gi.shape[2] % 3 != 0:
        raise ValueError(f"gi must be [T, B, 3H]; got {tuple(gi.shape)}")
    T, B, three_h = gi.shape
    H = three_h // 3
    if T == 0 or B == 0 or H == 0:
        raise ValueError(f"T, B and H must be > 0; got T={T}, B={B}, H={H}")
    if tuple(h0.shape) != (B, H):
        raise ValueError(f"h0 shape must be (B, H)=({B}, {H}); got {tuple(h0.shape)}")
    if tuple(bh_cat.shape) != (3 * H,):
        raise ValueError(f"bh_cat shape must be (3H,)=({3 * H},); got {tuple(bh_cat.shape)}")
    return T, B, H


def check_quant(name, q) -> None:
    if q is None:
        return
    if len(q) != 3 or not (float(q[0]) > 0.0):
        raise ValueError(f"{name} must be (scale > 0, qmin, qmax); got {q!r}")


def make_scan_function(kind: str, fwd, bwd):
    """autograd.Function over ``fwd(gi,h0,W,bh,h_in_quant=,h_out_quant=,_want_save=)`` and
    ``bwd(gi,h0,W,bh,out,dout,h_in_quant=,h_out_quant=,_save=)``: saves the forward's inputs,
    its output and (when a gradient is wanted) the gate activations."""

    class _ScanFunction(torch.autograd.Function):
        @staticmethod
        def forward(ctx: Any, gi, h0, W, bh, h_in_quant, h_out_quant):
            want = any(ctx.needs_input_grad[:4])
            out, save = fwd(gi, h0, W, bh, h_in_quant=h_in_quant, h_out_quant=h_out_quant,
                            _want_save=want)
            ctx.has_save = save is not None
            if save is not None:
                ctx.save_for_backward(gi, h0, W, bh, out, save)
            else:
                ctx.save_for_backward(gi, h0, W, bh, out)
            ctx.h_in_quant, ctx.h_out_quant = h_in_quant, h_out_quant
            return out

        @staticmethod
        def backward(ctx: Any, dout):
            saved = ctx.saved_tensors
            gi, h0, W, bh, out = saved[:5]
            save = saved[5] if ctx.has_save else None
            grads = bwd(gi, h0, W, bh, out, dout, h_in_quant=ctx.h_in_quant,
                        h_out_quant=ctx.h_out_quant, _save=save)
            return (*grads, None, None)

    _ScanFunction.__name__ = f"GRUScan{kind.capitalize()}Function"
    return _ScanFunction


def prep(*tensors):
    return tuple(t.contiguous() for t in tensors)


run_forward = _lib.scan_forward
run_backward = _lib.scan_backward
