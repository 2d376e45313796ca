"""Plain-PyTorch scan-form forward/backward of the four hidden kinds.

These back the ``*_forward_pytorch`` / ``*_backward_pytorch`` names that the
reference package exposes next to its kernels (scan.py:1460-1550,
scan_diagonal.py:79-124 and 564-647, scan_monarch.py:74-127 and 955-1053) and
that its tests use as ground truth.  They run on whatever device their inputs
live on and are never called by the CUDA scan path.
"""

from __future__ import annotations

import torch

from .structure import butterfly_apply


def fake_quant(x, params):
    """(fq(x), straight-through mask) for ``params = (scale, qmin, qmax)``; identity for None."""
    if params is None:
        return x, None
    scale, qmin, qmax = params
    code = torch.round(x / scale)
    return code.clamp(qmin, qmax) * scale, (code >= qmin) & (code <= qmax)


def _product(kind, hq, W):
    """Hidden-side product of the three gates, no bias: [B, 3, H]."""
    B, H = hq.shape
    if kind == "dense":
        return (hq @ W.T).view(B, 3, H)
    if kind == "diagonal":
        return W[None] * hq[:, None]
    if kind == "monarch":
        nb, bs = W.shape[1], W.shape[2]
        return torch.einsum("bni,gnoi->bgno", hq.view(B, nb, bs), W).reshape(B, 3, H)
    if kind == "butterfly":
        n = 2 * W.shape[3]
        hp = torch.nn.functional.pad(hq, (0, n - H)) if n > H else hq
        return torch.stack([butterfly_apply(W[g], hp)[:, :H] for g in range(3)], dim=1)
    raise ValueError(f"unknown kind {kind!r}")


def _step(kind, gi_t, h_prev, W, bh, h_in_quant):
    H = h_prev.shape[1]
    hq, mask_in = fake_quant(h_prev, h_in_quant)
    gh = _product(kind, hq, W) + bh.view(1, 3, H)
    r = torch.sigmoid(gi_t[:, :H] + gh[:, 0])
    z = torch.sigmoid(gi_t[:, H:2 * H] + gh[:, 1])
    n = torch.tanh(gi_t[:, 2 * H:] + r * gh[:, 2])
    return hq, mask_in, r, z, n, gh[:, 2], (1.0 - z) * n + z * h_prev


def scan_forward(kind, gi, h0, W, bh, *, h_in_quant=None, h_out_quant=None):
    h, outs = h0, []
    for t in range(gi.shape[0]):
        h_raw = _step(kind, gi[t], h, W, bh, h_in_quant)[-1]
        h, _ = fake_quant(h_raw, h_out_quant)
        outs.append(h)
    return torch.stack(outs, dim=0)


def scan_backward(kind, gi, h0, W, bh, out, dout, *, h_in_quant=None, h_out_quant=None):
    """(dgi, dh0, dW, dbh) by the reverse recurrence; the hidden product's own
    gradients come from autograd on a single step (exact for these linear maps)."""
    T = gi.shape[0]
    dgi = torch.zeros_like(gi)
    dW = torch.zeros_like(W)
    dbh = torch.zeros_like(bh)
    dh_acc = torch.zeros_like(h0)
    for t in reversed(range(T)):
        h_prev = h0 if t == 0 else out[t - 1]
        hq, mask_in, r, z, n, gh_n, h_raw = _step(kind, gi[t], h_prev, W, bh, h_in_quant)
        dh = dout[t] + dh_acc
        if h_out_quant is not None:
            dh = dh * fake_quant(h_raw, h_out_quant)[1]
        dgn = dh * (1.0 - z) * (1.0 - n * n)
        dgz = dh * (h_prev - n) * z * (1.0 - z)
        dgr = dgn * gh_n * r * (1.0 - r)
        dgi[t] = torch.cat([dgr, dgz, dgn], dim=-1)
        dgh = torch.stack([dgr, dgz, dgn * r], dim=1)
        with torch.enable_grad():
            hq_l = hq.detach().requires_grad_(True)
            W_l = W.detach().requires_grad_(True)
            g_h, g_W = torch.autograd.grad(_product(kind, hq_l, W_l), (hq_l, W_l), dgh)
        if mask_in is not None:
            g_h = g_h * mask_in
        dW += g_W
        dbh += dgh.sum(0).reshape(-1)
        dh_acc = dh * z + g_h
    return dgi, dh_acc, dW, dbh
