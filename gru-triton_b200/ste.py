"""Straight-through estimators used by the fake-quantizers.

Same contract as ``gru_qat.ste`` (src/gru_qat/ste.py:17-95): rounding is
half-to-even with an identity gradient; clamping passes the gradient only where
the (already rounded) input lies inside ``[qmin, qmax]``.
"""

from __future__ import annotations

import torch


class STERound(torch.autograd.Function):
    """``round`` forward, identity backward."""

    @staticmethod
    def forward(ctx, x):
        return x.round()

    @staticmethod
    def backward(ctx, grad):
        return grad


class STEClamp(torch.autograd.Function):
    """``clamp(x, qmin, qmax)`` forward; gradient gated by ``qmin <= x <= qmax``."""

    @staticmethod
    def forward(ctx, x, qmin, qmax):
        ctx.save_for_backward(x)
        ctx.bounds = (qmin, qmax)
        return x.clamp(qmin, qmax)

    @staticmethod
    def backward(ctx, grad):
        (x,) = ctx.saved_tensors
        lo, hi = ctx.bounds
        inside = (x >= lo) & (x <= hi)
        return grad * inside, None, None


def fake_quant_ste(x, scale, zero_point, qmin, qmax):
    """Quantise-dequantise ``x`` with straight-through gradients.

    ``q = clamp(round(x / scale + zero_point), qmin, qmax)``; result
    ``(q - zero_point) * scale``.  ``scale`` / ``zero_point`` broadcast against ``x``.
    """
    q = STERound.apply(x / scale + zero_point)
    q = STEClamp.apply(q, qmin, qmax)
    return (q - zero_point) * scale
