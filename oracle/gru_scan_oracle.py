"""CPU oracle for the persistent GRU scan -- TEST INFRASTRUCTURE, NOT PRODUCT.

A restatement, in plain torch CPU tensor ops, of the reference's multi-step GRU
scan for the four hidden-weight kinds (dense, diagonal, block-diagonal "monarch",
butterfly), forward and backward, with optional frozen per-tensor symmetric
fake-quant of the hidden state.  Only tests, the smoke check and the CPU-baseline
leg of the benchmark may import this module; the CUDA product never does.

Every function cites the reference source (path inside LarocheC/gru-triton) that
it follows.  Pinning status:

* dense, diagonal -- pinned: golden vectors produced by the reference's own
  ``GRUCellQuant`` per-step path and scan-form PyTorch functions
  (``tests/golden/make_golden.py``) are replayed by ``tests/test_oracle_golden.py``.
* monarch -- pinned to the reference's own pure-torch restatement
  (``src/gru_qat/triton_kernels/scan_monarch.py:74-127, 955-1053``); parity with
  the third-party ``torch-structured 1.2.1`` ``BlockdiagLinear`` itself is unpinned
  (that package is not available offline).
* butterfly -- PARITY UNPINNED against ``torch-structured 1.2.1``
  ``butterfly_multiply``: the reference holds no pure-torch butterfly and the
  third-party op is absent.  The stage arithmetic is restated from
  ``src/gru_qat/triton_kernels/scan_butterfly.py:276-317`` and is cross-checked
  against the reference's *dense* scan run on the materialised butterfly matrix.

All functions are dtype-agnostic (float32 for parity, float64 for error audits).
"""

from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

Quant = Optional[Tuple[float, int, int]]

KINDS = ("dense", "diagonal", "monarch", "butterfly")


# ---------------------------------------------------------------------------
# fake-quant
# ---------------------------------------------------------------------------

def fake_quant(x: torch.Tensor, params: Quant):
    """Per-tensor symmetric fake-quant and its straight-through clip mask.

    Follows ``src/gru_qat/triton_kernels/scan.py:1450-1457``: true division,
    round-half-to-even, the mask tests the rounded *unclamped* code.
    ``params=None`` is the identity with no mask.
    """
    if params is None:
        return x, None
    scale, qmin, qmax = params
    q = torch.round(x / scale)
    mask = (q >= qmin) & (q <= qmax)
    return q.clamp(qmin, qmax) * scale, mask


def quant_codes(x: torch.Tensor, params: Quant) -> torch.Tensor:
    """Integer codes ``clamp(rint(x / s), qmin, qmax)`` (as the input's dtype)."""
    scale, qmin, qmax = params
    return torch.round(x / scale).clamp(qmin, qmax)


def tie_distance(x: torch.Tensor, params: Quant) -> torch.Tensor:
    """Distance of ``x / s`` from the nearest half-way rounding point, in code units."""
    scale, _, _ = params
    v = x.double() / scale
    return (v - torch.floor(v) - 0.5).abs()


# ---------------------------------------------------------------------------
# butterfly arithmetic (restated from scan_butterfly.py:276-317)
# ---------------------------------------------------------------------------

def _log_stride(blk: int, s: int, log_n: int) -> int:
    # even block index: strides 1,2,4,...; odd: reversed (scan_butterfly.py:280-284)
    return s if blk % 2 == 0 else log_n - 1 - s


def butterfly_multiply(twiddle: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Apply one gate's butterfly to rows of ``x``.

    ``twiddle``: [nblocks, log_n, n/2, 2(m_new), 2(m_old)]; ``x``: [B, n] with n a
    power of two.  Position ``i`` at a stage with stride ``S = 1 << ls``:
    ``member = (i >> ls) & 1``, ``pair = (i >> (ls+1)) * S + (i & (S-1))`` and
    ``new[i] = t[pair, member, member] * a[i] + t[pair, member, 1-member] * a[i ^ S]``
    (scan_butterfly.py:286-317).  The twiddle's stage axis is indexed by the
    iteration number, not by the stride (scan_butterfly.py:299-312).
    """
    nblocks, log_n, half, _, _ = twiddle.shape
    n = half * 2
    B = x.shape[0]
    a = x
    for blk in range(nblocks):
        for s in range(log_n):
            ls = _log_stride(blk, s, log_n)
            S = 1 << ls
            hi = n // (2 * S)
            av = a.reshape(B, hi, 2, S)                       # [b, hi, m_old, lo]
            tv = twiddle[blk, s].reshape(hi, S, 2, 2)          # [hi, lo, m_new, m_old]
            a = torch.einsum("hlnm,bhml->bhnl", tv, av).reshape(B, n)
    return a


def butterfly_multiply_t(twiddle: torch.Tensor, d: torch.Tensor) -> torch.Tensor:
    """Transpose of :func:`butterfly_multiply` (gradient w.r.t. its input).

    Follows the reverse-stage walk of scan_butterfly.py:762-812:
    ``d_old[m_old] = sum_{m_new} t[m_new, m_old] * d_new[m_new]``.
    """
    nblocks, log_n, half, _, _ = twiddle.shape
    n = half * 2
    B = d.shape[0]
    a = d
    for blk in reversed(range(nblocks)):
        for s in reversed(range(log_n)):
            ls = _log_stride(blk, s, log_n)
            S = 1 << ls
            hi = n // (2 * S)
            dv = a.reshape(B, hi, 2, S)                       # [b, hi, m_new, lo]
            tv = twiddle[blk, s].reshape(hi, S, 2, 2)
            a = torch.einsum("hlnm,bhnl->bhml", tv, dv).reshape(B, n)
    return a


def butterfly_multiply_states(twiddle: torch.Tensor, x: torch.Tensor):
    """Forward butterfly keeping the input of every stage (for twiddle grads)."""
    nblocks, log_n, half, _, _ = twiddle.shape
    n = half * 2
    B = x.shape[0]
    a = x
    states = []
    for blk in range(nblocks):
        for s in range(log_n):
            states.append(a)
            ls = _log_stride(blk, s, log_n)
            S = 1 << ls
            hi = n // (2 * S)
            av = a.reshape(B, hi, 2, S)
            tv = twiddle[blk, s].reshape(hi, S, 2, 2)
            a = torch.einsum("hlnm,bhml->bhnl", tv, av).reshape(B, n)
    return a, states


def butterfly_backward(twiddle: torch.Tensor, states, d_out: torch.Tensor):
    """Gradients of one butterfly multiply: (d_input, d_twiddle).

    ``d_t[pair, m_new, m_old] += d_new[m_new] * old[m_old]`` summed over the batch
    (scan_butterfly.py:814-919).
    """
    nblocks, log_n, half, _, _ = twiddle.shape
    n = half * 2
    B = d_out.shape[0]
    dtw = torch.zeros_like(twiddle)
    a = d_out
    for blk in reversed(range(nblocks)):
        for s in reversed(range(log_n)):
            ls = _log_stride(blk, s, log_n)
            S = 1 << ls
            hi = n // (2 * S)
            old = states[blk * log_n + s].reshape(B, hi, 2, S)
            dv = a.reshape(B, hi, 2, S)
            tv = twiddle[blk, s].reshape(hi, S, 2, 2)
            dtw[blk, s] = torch.einsum("bhnl,bhml->hlnm", dv, old).reshape(half, 2, 2)
            a = torch.einsum("hlnm,bhnl->bhml", tv, dv).reshape(B, n)
    return a, dtw


def butterfly_dense_matrix_loops(twiddle: torch.Tensor) -> torch.Tensor:
    """Materialise one gate's butterfly as a dense [n, n] matrix with scalar loops.

    Written index-by-index from the formulas of scan_butterfly.py:286-317,
    independently of the vectorised :func:`butterfly_multiply`, so that the two
    check one another.  ``y = x @ M.T``.  Differentiable w.r.t. ``twiddle``.
    """
    nblocks, log_n, half, _, _ = twiddle.shape
    n = half * 2
    M = torch.eye(n, dtype=twiddle.dtype)
    for blk in range(nblocks):
        for s in range(log_n):
            ls = _log_stride(blk, s, log_n)
            S = 1 << ls
            rows = []
            for i in range(n):
                member = (i >> ls) & 1
                pair = (i >> (ls + 1)) * S + (i & (S - 1))
                partner = i ^ S
                row = (twiddle[blk, s, pair, member, member] * M[i]
                       + twiddle[blk, s, pair, member, 1 - member] * M[partner])
                rows.append(row)
            M = torch.stack(rows, dim=0)
    return M


# ---------------------------------------------------------------------------
# hidden operators: gh = HiddenOp(hq)  ->  [B, 3, H]
# ---------------------------------------------------------------------------

def _pad_cols(x: torch.Tensor, n: int) -> torch.Tensor:
    if x.shape[-1] == n:
        return x
    return torch.nn.functional.pad(x, (0, n - x.shape[-1]))


def hidden_op(kind: str, hq: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """Hidden-side product of all three gates, without bias: [B, 3, H]."""
    B, H = hq.shape
    if kind == "dense":
        # scan.py:1498 -- gh = hq @ Wh_cat.T, rows of Wh_cat ordered r,z,n
        return (hq @ W.T).reshape(B, 3, H)
    if kind == "diagonal":
        # scan_diagonal.py:108-110
        return W.unsqueeze(0) * hq.unsqueeze(1)
    if kind == "monarch":
        # scan_monarch.py:110-112
        _, nb, bs, _ = W.shape
        return torch.einsum("bni,gnoi->bgno", hq.reshape(B, nb, bs), W).reshape(B, 3, H)
    if kind == "butterfly":
        n = W.shape[3] * 2
        xp = _pad_cols(hq, n)
        return torch.stack([butterfly_multiply(W[g], xp)[:, :H] for g in range(3)], dim=1)
    raise ValueError(f"unknown kind {kind!r}")


def hidden_op_backward(kind: str, hq: torch.Tensor, W: torch.Tensor, dgh: torch.Tensor):
    """(d_hq [B,H], dW like W) for ``gh = hidden_op(kind, hq, W)`` given dgh [B,3,H]."""
    B, H = hq.shape
    if kind == "dense":
        d2 = dgh.reshape(B, 3 * H)
        return d2 @ W, d2.T @ hq                                   # scan.py:1541-1545
    if kind == "diagonal":
        return (dgh * W.unsqueeze(0)).sum(1), (dgh * hq.unsqueeze(1)).sum(0)   # scan_diagonal.py:630-643
    if kind == "monarch":
        _, nb, bs, _ = W.shape
        dc = dgh.reshape(B, 3, nb, bs)
        hc = hq.reshape(B, nb, bs)
        dW = torch.einsum("bgno,bni->gnoi", dc, hc)                  # scan_monarch.py:1041
        dh = torch.einsum("bgno,gnoi->bni", dc, W).reshape(B, H)     # scan_monarch.py:1042-1045
        return dh, dW
    if kind == "butterfly":
        n = W.shape[3] * 2
        xp = _pad_cols(hq, n)
        dh = torch.zeros_like(xp)
        dW = torch.zeros_like(W)
        for g in range(3):
            _, states = butterfly_multiply_states(W[g], xp)
            d_in, dtw = butterfly_backward(W[g], states, _pad_cols(dgh[:, g], n))
            dh = dh + d_in
            dW[g] = dtw
        return dh[:, :H], dW
    raise ValueError(f"unknown kind {kind!r}")


# ---------------------------------------------------------------------------
# scan forward / backward (scan form)
# ---------------------------------------------------------------------------

def gate_math(gi_t: torch.Tensor, gh: torch.Tensor, bh: torch.Tensor, h_prev: torch.Tensor):
    """r, z, n, gh_n, h_raw of one step (gru_cell.py:452-462, scan.py:1491-1505)."""
    H = h_prev.shape[-1]
    gh = gh + bh.reshape(1, 3, H)
    r = torch.sigmoid(gi_t[:, 0:H] + gh[:, 0])
    z = torch.sigmoid(gi_t[:, H:2 * H] + gh[:, 1])
    n = torch.tanh(gi_t[:, 2 * H:3 * H] + r * gh[:, 2])
    h_raw = (1.0 - z) * n + z * h_prev
    return r, z, n, gh[:, 2], h_raw


def scan_forward(kind: str, gi: torch.Tensor, h0: torch.Tensor, W: torch.Tensor,
                 bh: torch.Tensor, h_in_quant: Quant = None, h_out_quant: Quant = None,
                 return_raw: bool = False):
    """Forward scan, all T steps: out[T,B,H] (and the pre-quant h_raw if asked).

    Only the product side sees ``fq_in(h)``; the blend uses the stored h
    (gru_cell.py:452-464; scan_monarch.py:105-124).
    """
    T, B, _ = gi.shape
    H = h0.shape[-1]
    out = torch.empty(T, B, H, dtype=gi.dtype)
    raw = torch.empty(T, B, H, dtype=gi.dtype) if return_raw else None
    h = h0
    for t in range(T):
        hq, _ = fake_quant(h, h_in_quant)
        _, _, _, _, h_raw = gate_math(gi[t], hidden_op(kind, hq, W), bh, h)
        if return_raw:
            raw[t] = h_raw
        h, _ = fake_quant(h_raw, h_out_quant)
        out[t] = h
    return (out, raw) if return_raw else out


def scan_forward_teacher_forced(kind: str, gi, h_prev_all, W, bh,
                                h_in_quant: Quant = None, wide: bool = False):
    """One step from every given predecessor state: h_raw[t] from h_prev_all[t].

    Used by the int8 tie protocol: feeding the device's own ``h_{t-1}`` makes every
    step an independent comparison, so a single rounding tie cannot cascade.

    ``wide``: the input fake-quant runs in the inputs' own precision (its codes are part of the
    reference semantics), everything after it -- hidden product, gates, blend -- in float64, so the
    returned h_raw carries no summation-order noise of its own (an fp32 CPU product of H terms
    differs between BLAS builds and thread counts by more than a tie window of 1e-4 code units).
    """
    T, B, _ = gi.shape
    raw = torch.empty_like(h_prev_all, dtype=torch.float64 if wide else h_prev_all.dtype)
    Ww, bw = (W.double(), bh.double()) if wide else (W, bh)
    for t in range(T):
        hq, _ = fake_quant(h_prev_all[t], h_in_quant)
        if wide:
            raw[t] = gate_math(gi[t].double(), hidden_op(kind, hq.double(), Ww), bw, h_prev_all[t].double())[4]
        else:
            raw[t] = gate_math(gi[t], hidden_op(kind, hq, W), bh, h_prev_all[t])[4]
    return raw


def scan_backward(kind: str, gi, h0, W, bh, out, dout,
                  h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Reverse scan: (dgi, dh0, dW, dbh).  Follows scan.py:1460-1550 (dense),
    scan_diagonal.py:564-647, scan_monarch.py:955-1053, scan_butterfly.py:642-968."""
    T, B, _ = gi.shape
    H = h0.shape[-1]
    dgi = torch.zeros_like(gi)
    dW = torch.zeros_like(W)
    dbh = torch.zeros_like(bh)
    dh_acc = torch.zeros_like(h0)
    for t in reversed(range(T)):
        h_prev = h0 if t == 0 else out[t - 1]
        hq, mask_in = fake_quant(h_prev, h_in_quant)
        r, z, n, gh_n, h_raw = gate_math(gi[t], hidden_op(kind, hq, W), bh, h_prev)
        dh = dout[t] + dh_acc
        if h_out_quant is not None:
            dh = dh * fake_quant(h_raw, h_out_quant)[1]
        dn = dh * (1.0 - z)
        dz = dh * (h_prev - n)
        dh_direct = dh * z
        dgn = dn * (1.0 - n * n)
        dr = dgn * gh_n
        dgh_n = dgn * r
        dgz = dz * z * (1.0 - z)
        dgr = dr * r * (1.0 - r)
        dgi[t] = torch.cat([dgr, dgz, dgn], dim=-1)
        dgh = torch.stack([dgr, dgz, dgh_n], dim=1)
        dh_via, dW_t = hidden_op_backward(kind, hq, W, dgh)
        if mask_in is not None:
            dh_via = dh_via * mask_in
        dW = dW + dW_t
        dbh = dbh + dgh.sum(0).reshape(-1)
        dh_acc = dh_direct + dh_via
    return dgi, dh_acc, dW, dbh


# ---------------------------------------------------------------------------
# autograd form (the literal GRUCellQuant route: STE round / clipped clamp)
# ---------------------------------------------------------------------------

class _STERound(torch.autograd.Function):          # ste.py:17-35
    @staticmethod
    def forward(ctx, x):
        return torch.round(x)

    @staticmethod
    def backward(ctx, g):
        return g


class _STEClamp(torch.autograd.Function):          # ste.py:38-62
    @staticmethod
    def forward(ctx, x, lo, hi):
        ctx.save_for_backward(x)
        ctx.lo, ctx.hi = lo, hi
        return torch.clamp(x, lo, hi)

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        return g * ((x >= ctx.lo) & (x <= ctx.hi)), None, None


def fake_quant_ste(x: torch.Tensor, params: Quant) -> torch.Tensor:
    """``ste.py:65-95`` with zero_point = 0: gradient crosses ``/ s`` and ``* s``."""
    if params is None:
        return x
    scale, qmin, qmax = params
    s = torch.tensor(scale, dtype=x.dtype)
    q = _STERound.apply(x / s + 0.0)
    q = _STEClamp.apply(q, qmin, qmax)
    return (q - 0.0) * s


def scan_forward_autograd(kind: str, gi, h0, W, bh,
                          h_in_quant: Quant = None, h_out_quant: Quant = None):
    """Differentiable per-step loop in the op order of ``GRUCellQuant.step_with_gi``
    (gru_cell.py:437-464) / ``step_structured`` (gru_cell.py:301-349)."""
    T = gi.shape[0]
    H = h0.shape[-1]
    h = h0
    outs = []
    for t in range(T):
        hq = fake_quant_ste(h, h_in_quant)
        gh = hidden_op(kind, hq, W) + bh.reshape(1, 3, H)
        r = torch.sigmoid(gi[t, :, 0:H] + gh[:, 0])
        z = torch.sigmoid(gi[t, :, H:2 * H] + gh[:, 1])
        n = torch.tanh(gi[t, :, 2 * H:3 * H] + r * gh[:, 2])
        h = fake_quant_ste((1.0 - z) * n + z * h, h_out_quant)
        outs.append(h)
    return torch.stack(outs, dim=0)


# ---------------------------------------------------------------------------
# whole-layer CPU path (the timed CPU baseline: input projection + scan + grads)
# ---------------------------------------------------------------------------

def per_row_weight_fake_quant(Wm: torch.Tensor, bits: int = 8) -> torch.Tensor:
    """Dynamic per-output-row symmetric weight fake-quant (quantizers.py:118-134,
    177-189): ``s_row = max(|row|).clamp(1e-8) / qmax``."""
    qmax = 2 ** (bits - 1) - 1
    s = Wm.abs().amax(dim=1, keepdim=True).clamp(min=1e-8) / qmax
    q = _STEClamp.apply(_STERound.apply(Wm / s + 0.0), -qmax, qmax)
    return (q - 0.0) * s


def layer_train_step(kind: str, x, h0, Wi_cat, bi_cat, W, bh,
                     h_in_quant: Quant = None, h_out_quant: Quant = None,
                     weight_bits: int = 32, backward: bool = True):
    """One training step of a fused-gate layer on CPU, per-step like
    ``GRULayer.forward`` with ``use_triton=False`` (gru_layer.py:202-232):
    ``gi = x @ Wi_cat.T + bi_cat``, the per-step autograd loop, loss ``out.sum()``.
    Returns (out, grads-dict)."""
    leaves = [t.detach().clone().requires_grad_(backward) for t in (Wi_cat, bi_cat, W, bh)]
    Wi_l, bi_l, W_l, bh_l = leaves
    Wi_q, W_q = Wi_l, W_l
    if weight_bits < 32:
        Wi_q = per_row_weight_fake_quant(Wi_l, weight_bits)
        if kind == "dense":
            W_q = per_row_weight_fake_quant(W_l, weight_bits)
    gi = torch.nn.functional.linear(x, Wi_q, bi_l)
    out = scan_forward_autograd(kind, gi, h0, W_q, bh_l, h_in_quant, h_out_quant)
    grads = {}
    if backward:
        out.sum().backward()
        grads = {"dWi": Wi_l.grad, "dbi": bi_l.grad, "dW": W_l.grad, "dbh": bh_l.grad}
    return out.detach(), grads


# ---------------------------------------------------------------------------
# two-factor Monarch (extension of this build; PARITY UNPINNED: the reference has no such operator)
# ---------------------------------------------------------------------------

def monarch2_dense_loops(W1: torch.Tensor, W2: torch.Tensor) -> torch.Tensor:
    """Dense ``[3H, H]`` matrix of ``gh_g = P^T B2_g P B1_g h`` by scalar index loops, where B1 / B2
    are block-diagonal with blocks ``W1[g, i]`` / ``W2[g, i]`` and P is the Monarch stride
    permutation ``(P v)[j * nblocks + i] = v[i * blksz + j]`` (BASELINE config 3's wording; the
    reference itself has one factor per gate, scan_monarch.py:110-112)."""
    _, nb, bs, _ = W1.shape
    H = nb * bs
    out = torch.zeros(3 * H, H, dtype=W1.dtype)
    for g in range(3):
        for col in range(H):
            v = [0.0] * H
            v[col] = 1.0
            # B1
            a = [0.0] * H
            for i in range(nb):
                for o in range(bs):
                    a[i * bs + o] = sum(float(W1[g, i, o, k]) * v[i * bs + k] for k in range(bs) if v[i * bs + k] != 0.0)
            # P
            p = [0.0] * H
            for i in range(nb):
                for j in range(bs):
                    p[j * nb + i] = a[i * bs + j]
            # B2
            c = [0.0] * H
            for i in range(nb):
                for o in range(bs):
                    c[i * bs + o] = sum(float(W2[g, i, o, k]) * p[i * bs + k] for k in range(bs) if p[i * bs + k] != 0.0)
            # P^T
            for i in range(nb):
                for j in range(bs):
                    out[g * H + i * bs + j, col] = c[j * nb + i]
    return out


# ---------------------------------------------------------------------------
# seeded synthetic problems (shared by tests, smoke and bench)
# ---------------------------------------------------------------------------

def make_weights(kind: str, H: int, gen: torch.Generator, *, nblocks: int = 4,
                 butterfly_nblocks: int = 1, dtype=torch.float32):
    """Random hidden weights of the right shape for ``kind`` plus ``bh`` [3H]."""
    k = H ** -0.5

    def U(*shape, a=k):
        return (torch.rand(*shape, generator=gen, dtype=torch.float64) * 2 - 1).mul(a).to(dtype)

    if kind == "dense":
        W = U(3 * H, H)
    elif kind == "diagonal":
        W = U(3, H, a=1.0)
    elif kind == "monarch":
        bs = H // nblocks
        W = (torch.randn(3, nblocks, bs, bs, generator=gen, dtype=torch.float64)
             * bs ** -0.5).to(dtype)
    elif kind == "butterfly":
        n = 1 << max(1, math.ceil(math.log2(H)))
        W = U(3, butterfly_nblocks, int(math.log2(n)), n // 2, 2, 2, a=2 ** -0.5)
    else:
        raise ValueError(kind)
    return W, U(3 * H)


def make_problem(kind: str, T: int, B: int, H: int, seed: int = 0, *, nblocks: int = 4,
                 butterfly_nblocks: int = 1, gi_scale: float = 1.0, h0_scale: float = 0.5,
                 dtype=torch.float32):
    """Seeded (gi, h0, W, bh, dout) for a scan-level parity case."""
    gen = torch.Generator().manual_seed(seed)
    W, bh = make_weights(kind, H, gen, nblocks=nblocks,
                         butterfly_nblocks=butterfly_nblocks, dtype=dtype)
    gi = (torch.randn(T, B, 3 * H, generator=gen, dtype=torch.float64) * gi_scale).to(dtype)
    h0 = (torch.randn(B, H, generator=gen, dtype=torch.float64) * h0_scale).to(dtype)
    dout = torch.randn(T, B, H, generator=gen, dtype=torch.float64).to(dtype)
    return gi, h0, W, bh, dout
