"""The CPU oracle replayed against golden vectors produced by the reference."""

from __future__ import annotations

import os

import pytest
import torch

from conftest import BUTTERFLY_REFERENCE_GOLDEN, SCAN_GOLDEN_FLAT, load_golden, rel_err
from oracle import gru_scan_oracle as orc

FWD_TOL = 1e-5     # fp32 forward: 1e-5 absolute and relative
GRAD_TOL = 1e-4    # fp32 gradients: 1e-4 relative


@pytest.mark.parametrize("kind,name", SCAN_GOLDEN_FLAT)
def test_scan_forward_matches_reference(kind, name):
    g = load_golden(name)
    out = orc.scan_forward(kind, g["gi"], g["h0"], g["W"], g["bh"], g["q_in"], g["q_out"])
    if g["q_out"] is not None and kind != "butterfly":
        assert torch.equal(out, g["out"])           # same ops, same machine arithmetic
    assert (out - g["out"]).abs().max().item() < FWD_TOL
    assert rel_err(out, g["out"]) < FWD_TOL


@pytest.mark.parametrize("kind,name", SCAN_GOLDEN_FLAT)
def test_scan_backward_matches_reference(kind, name):
    g = load_golden(name)
    got = orc.scan_backward(kind, g["gi"], g["h0"], g["W"], g["bh"], g["out"], g["dout"],
                            g["q_in"], g["q_out"])
    for nm, a in zip(("dgi", "dh0", "dW", "dbh"), got):
        assert rel_err(a, g[nm]) < GRAD_TOL, nm


@pytest.mark.parametrize("kind,name", SCAN_GOLDEN_FLAT)
def test_autograd_form_matches_scan_form(kind, name):
    g = load_golden(name)
    leaves = [g[k].clone().requires_grad_(True) for k in ("gi", "h0", "W", "bh")]
    out = orc.scan_forward_autograd(kind, *leaves, g["q_in"], g["q_out"])
    out.backward(g["dout"])
    assert rel_err(out.detach(), g["out"]) < FWD_TOL
    for nm, leaf in zip(("dgi", "dh0", "dW", "dbh"), leaves):
        assert rel_err(leaf.grad, g[nm]) < GRAD_TOL, nm


@pytest.mark.parametrize("name", BUTTERFLY_REFERENCE_GOLDEN)
def test_butterfly_oracle_matches_the_references_own_kernels(name):
    """The fixtures are outputs of the reference's Triton butterfly scan (forward and backward,
    scan_butterfly.py:369-459, 971-1075) run on a B200: they pin the oracle's reading of the stage
    order (reversed on odd factors), the twiddle axis and the 2x2 orientation.  That kernel has no
    tensor-core product, so it agrees with fp32 CPU arithmetic far inside the usual bars."""
    g = load_golden(name)
    out = orc.scan_forward("butterfly", g["gi"], g["h0"], g["W"], g["bh"], g["q_in"], g["q_out"])
    assert (out - g["out"]).abs().max().item() < FWD_TOL
    got = orc.scan_backward("butterfly", g["gi"], g["h0"], g["W"], g["bh"], g["out"], g["dout"],
                            g["q_in"], g["q_out"])
    for nm, a in zip(("dgi", "dh0", "dW", "dbh"), got):
        assert rel_err(a, g[nm]) < GRAD_TOL, nm


@pytest.mark.parametrize("n,nblocks", [(2, 1), (8, 1), (16, 2), (32, 3)])
def test_butterfly_vectorised_equals_index_loops(n, nblocks):
    gen = torch.Generator().manual_seed(n + nblocks)
    import math
    tw = torch.randn(nblocks, int(math.log2(n)), n // 2, 2, 2, generator=gen, dtype=torch.float64)
    x = torch.randn(5, n, generator=gen, dtype=torch.float64)
    M = orc.butterfly_dense_matrix_loops(tw)
    y = orc.butterfly_multiply(tw, x)
    assert (y - x @ M.T).abs().max() < 1e-12
    d = torch.randn(5, n, generator=gen, dtype=torch.float64)
    assert (orc.butterfly_multiply_t(tw, d) - d @ M).abs().max() < 1e-12
    # twiddle gradient against autograd through the loop materialisation
    tw_l = tw.clone().requires_grad_(True)
    (x @ orc.butterfly_dense_matrix_loops(tw_l).T * d).sum().backward()
    _, states = orc.butterfly_multiply_states(tw, x)
    d_in, dtw = orc.butterfly_backward(tw, states, d)
    assert (dtw - tw_l.grad).abs().max() < 1e-10
    assert (d_in - d @ M).abs().max() < 1e-12


@pytest.mark.parametrize("name,kind", [("layer_dense_fp32", "dense"), ("layer_dense_w8h8", "dense"),
                                       ("layer_diagonal_fp32", "diagonal"),
                                       ("layer_diagonal_q8", "diagonal")])
def test_layer_train_step_matches_reference(name, kind):
    g = load_golden(name)
    P = {k[2:]: v for k, v in g.items() if k.startswith("p:")}
    G = {k[2:]: v for k, v in g.items() if k.startswith("g:")}
    Wi = torch.cat([P["cell.W_ir"], P["cell.W_iz"], P["cell.W_in"]], 0)
    bi = torch.cat([P["cell.b_ir"], P["cell.b_iz"], P["cell.b_in"]])
    bh = torch.cat([P["cell.b_hr"], P["cell.b_hz"], P["cell.b_hn"]])
    if kind == "dense":
        W = torch.cat([P["cell.W_hr"], P["cell.W_hz"], P["cell.W_hn"]], 0)
        gW = torch.cat([G["cell.W_hr"], G["cell.W_hz"], G["cell.W_hn"]], 0)
    else:
        W = torch.stack([P[f"cell.struct_Wh_{c}.weight"] for c in "rzn"], 0)
        gW = torch.stack([G[f"cell.struct_Wh_{c}.weight"] for c in "rzn"], 0)
    wbits = 8 if name.endswith("w8h8") else 32
    out, grads = orc.layer_train_step(kind, g["x"], g["h0"], Wi, bi, W, bh,
                                      g["q_in"], g["q_out"], weight_bits=wbits)
    assert (out - g["out"]).abs().max().item() < FWD_TOL
    assert rel_err(grads["dW"], gW) < GRAD_TOL
    assert rel_err(grads["dWi"], torch.cat([G["cell.W_ir"], G["cell.W_iz"], G["cell.W_in"]], 0)) < GRAD_TOL
    assert rel_err(grads["dbh"], torch.cat([G["cell.b_hr"], G["cell.b_hz"], G["cell.b_hn"]])) < GRAD_TOL
    assert rel_err(grads["dbi"], torch.cat([G["cell.b_ir"], G["cell.b_iz"], G["cell.b_in"]])) < GRAD_TOL


# The unmodified reference package: $GRU_QAT_REFERENCE_SRC, else the copy oracle/make_ref.py installs.
REF_SRC = os.environ.get("GRU_QAT_REFERENCE_SRC",
                         os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref"))


@pytest.mark.skipif(not os.path.isfile(os.path.join(REF_SRC, "gru_qat", "__init__.py")),
                    reason="reference package not installed (python oracle/make_ref.py)")
@pytest.mark.parametrize("kind", ["dense", "diagonal", "monarch"])
@pytest.mark.parametrize("quant", [None, ((0.02, -127, 127), (0.015, -127, 127))])
def test_oracle_against_live_reference(kind, quant):
    """Where the reference checkout exists, compare fresh seeds directly."""
    import sys
    sys.path.insert(0, REF_SRC)
    try:
        from gru_qat.triton_kernels import scan as rs, scan_diagonal as rd, scan_monarch as rm
    finally:
        sys.path.remove(REF_SRC)
    gi, h0, W, bh, dout = orc.make_problem(kind, 9, 4, 32, seed=123, nblocks=4)
    qi, qo = quant if quant else (None, None)
    out = orc.scan_forward(kind, gi, h0, W, bh, qi, qo)
    mine = orc.scan_backward(kind, gi, h0, W, bh, out, dout, qi, qo)
    if kind == "dense":
        ref = rs._gru_scan_backward_pytorch(gi, h0, W, bh, out, dout, h_in_quant=qi, h_out_quant=qo)
    elif kind == "diagonal":
        assert torch.equal(out, rd.gru_scan_diagonal_forward_pytorch(gi, h0, W, bh, h_in_quant=qi, h_out_quant=qo))
        ref = rd.gru_scan_diagonal_backward_pytorch(gi, h0, W, bh, out, dout, h_in_quant=qi, h_out_quant=qo)
    else:
        assert rel_err(out, rm.gru_scan_monarch_forward_pytorch(gi, h0, W, bh, h_in_quant=qi, h_out_quant=qo)) < FWD_TOL
        ref = rm.gru_scan_monarch_backward_pytorch(gi, h0, W, bh, out, dout, h_in_quant=qi, h_out_quant=qo)
    for a, b in zip(mine, ref):
        assert rel_err(a, b) < GRAD_TOL
