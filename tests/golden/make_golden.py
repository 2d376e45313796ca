"""Generate the golden fixtures under tests/golden/ from the reference itself.

Run where the reference package is importable: from ``$GRU_QAT_REFERENCE_SRC`` (the
checkout's ``src`` directory) or, by default, from the copy that ``python oracle/make_ref.py``
installs into ``oracle/_ref``:

    python tests/golden/make_golden.py

The reference (LarocheC/gru-triton, package ``gru_qat``) is pure Python; its
CPU per-step ``GRUCellQuant`` path and its scan-form PyTorch functions run
without a GPU.  This script feeds them small seeded inputs and stores inputs and
outputs as ``.npz`` files, which then travel with the repository to machines
that do not have the reference.

What produces what:

* ``scan_dense_*``     -- ``GRUCellQuant.step_with_gi`` loop + autograd
                          (gru_cell.py:437-464) cross-checked against
                          ``_gru_scan_backward_pytorch`` (scan.py:1460-1550).
* ``scan_diagonal_*``  -- ``gru_scan_diagonal_forward_pytorch`` /
                          ``..._backward_pytorch`` (scan_diagonal.py:79-124, 564-647).
* ``scan_monarch_*``   -- ``gru_scan_monarch_forward_pytorch`` /
                          ``..._backward_pytorch`` (scan_monarch.py:74-127, 955-1053).
* ``scan_butterfly_*`` -- the reference's DENSE scan run on the butterfly matrix
                          materialised index-by-index from scan_butterfly.py:286-317;
                          twiddle gradients by autograd through that materialisation.
                          (The third-party ``torch_structured`` op is unavailable:
                          the stage convention itself is restated, not executed.)
* ``layer_*``          -- ``GRULayer(use_triton=False)`` forward + ``out.sum().backward()``
                          (gru_layer.py:202-232) for dense and diagonal layers.
* ``calib_diagonal``   -- ``GRULayer.calibrate`` + ``freeze`` (gru_layer.py:308-342).
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF_SRC = os.environ.get("GRU_QAT_REFERENCE_SRC", os.path.join(REPO, "oracle", "_ref"))
sys.path.insert(0, REF_SRC)
sys.path.insert(0, REPO)

from gru_qat import GRULayer, QuantizerConfig, QuantRecipe, StructureConfig  # noqa: E402
from gru_qat.triton_kernels import scan as ref_scan  # noqa: E402
from gru_qat.triton_kernels import scan_diagonal as ref_diag  # noqa: E402
from gru_qat.triton_kernels import scan_monarch as ref_mon  # noqa: E402

from oracle import gru_scan_oracle as orc  # noqa: E402  (problem generator + loop materialiser only)

H_SCALE = 0.02
QP = (H_SCALE, -127, 127)


def _np(t):
    return t.detach().cpu().numpy()


def _save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **{k: (_np(v) if torch.is_tensor(v) else np.asarray(v))
                                 for k, v in arrays.items()})
    print(f"wrote {name}.npz  ({os.path.getsize(path)} bytes)")


def _recipe(hidden_bits=32, weight_bits=32, hidden_mode="frozen"):
    return QuantRecipe(
        weight=QuantizerConfig(bits=weight_bits, axis=0, name="W"),
        input_act=QuantizerConfig(bits=32, name="x_id"),
        hidden=QuantizerConfig(bits=hidden_bits, mode=hidden_mode, name="h"),
    )


def _set_h_scale(layer, s_in, s_out):
    for q, s in ((layer.cell.quant_h_in, s_in), (layer.cell.quant_h_out, s_out)):
        q.scale = torch.tensor(s)
        q.zero_point = torch.tensor(0.0)
        q.config.mode = "frozen"


def _quant_args(quant):
    if quant is None:
        return {"q_in": np.zeros(0), "q_out": np.zeros(0)}
    return {"q_in": np.array(quant[0], dtype=np.float64),
            "q_out": np.array(quant[1], dtype=np.float64)}


# ---------------------------------------------------------------------------
# scan level
# ---------------------------------------------------------------------------

def scan_dense(name, T, B, H, seed, quant):
    gi, h0, W, bh, dout = orc.make_problem("dense", T, B, H, seed)
    layer = GRULayer(H, H, _recipe(8 if quant else 32), gate_layout="fused",
                     pre_batch_input=True)
    if quant:
        _set_h_scale(layer, quant[0][0], quant[1][0])
    cell = layer.cell
    with torch.no_grad():
        cell.W_hr.copy_(W[0:H]); cell.W_hz.copy_(W[H:2 * H]); cell.W_hn.copy_(W[2 * H:])
        cell.b_hr.copy_(bh[0:H]); cell.b_hz.copy_(bh[H:2 * H]); cell.b_hn.copy_(bh[2 * H:])
    gi_l = gi.clone().requires_grad_(True)
    h0_l = h0.clone().requires_grad_(True)
    w = cell.quantize_weights()
    h = h0_l
    outs = []
    for t in range(T):
        h = cell.step_with_gi(gi_l[t], h, w)
        outs.append(h)
    out = torch.stack(outs)
    out.backward(dout)
    dW = torch.cat([cell.W_hr.grad, cell.W_hz.grad, cell.W_hn.grad], 0)
    dbh = torch.cat([cell.b_hr.grad, cell.b_hz.grad, cell.b_hn.grad])
    # the reference's own scan-form backward must agree with its cell path
    qi, qo = (quant if quant else (None, None))
    sg = ref_scan._gru_scan_backward_pytorch(gi, h0, W, bh, out.detach(), dout,
                                             h_in_quant=qi, h_out_quant=qo)
    for a, b_, nm in zip(sg, (gi_l.grad, h0_l.grad, dW, dbh), ("dgi", "dh0", "dW", "dbh")):
        err = (a - b_).abs().max().item()
        assert err < 1e-4 * max(1.0, b_.abs().max().item()), (name, nm, err)
    _save(name, gi=gi, h0=h0, W=W, bh=bh, dout=dout, out=out, dgi=gi_l.grad,
          dh0=h0_l.grad, dW=dW, dbh=dbh, **_quant_args(quant))


def scan_formfn(name, kind, T, B, H, seed, quant, nblocks=4):
    gi, h0, W, bh, dout = orc.make_problem(kind, T, B, H, seed, nblocks=nblocks)
    mod = ref_diag if kind == "diagonal" else ref_mon
    fwd = getattr(mod, f"gru_scan_{kind}_forward_pytorch")
    bwd = getattr(mod, f"gru_scan_{kind}_backward_pytorch")
    qi, qo = (quant if quant else (None, None))
    out = fwd(gi, h0, W, bh, h_in_quant=qi, h_out_quant=qo)
    dgi, dh0, dW, dbh = bwd(gi, h0, W, bh, out, dout, h_in_quant=qi, h_out_quant=qo)
    _save(name, gi=gi, h0=h0, W=W, bh=bh, dout=dout, out=out, dgi=dgi, dh0=dh0,
          dW=dW, dbh=dbh, **_quant_args(quant))


def scan_butterfly(name, T, B, H, seed, quant, butterfly_nblocks=1):
    gi, h0, tw, bh, dout = orc.make_problem("butterfly", T, B, H, seed,
                                            butterfly_nblocks=butterfly_nblocks)
    tw_l = tw.clone().requires_grad_(True)
    # dense matrix of each gate's butterfly, by scalar loops over the index formulas
    M = torch.cat([orc.butterfly_dense_matrix_loops(tw_l[g])[:H, :H] for g in range(3)], 0)
    Wd = M.detach()
    qi, qo = (quant if quant else (None, None))
    out = ref_scan_forward_dense(gi, h0, Wd, bh, qi, qo)
    dgi, dh0, dWd, dbh = ref_scan._gru_scan_backward_pytorch(
        gi, h0, Wd, bh, out, dout, h_in_quant=qi, h_out_quant=qo)
    M.backward(dWd)          # chain rule: d twiddle = d(dense W) . dM/dtwiddle
    _save(name, gi=gi, h0=h0, W=tw, bh=bh, dout=dout, out=out, dgi=dgi, dh0=dh0,
          dW=tw_l.grad, dbh=dbh, **_quant_args(quant))


def ref_scan_forward_dense(gi, h0, Wd, bh, qi, qo):
    """Dense forward through the reference cell (step_with_gi)."""
    T, B, _ = gi.shape
    H = h0.shape[1]
    layer = GRULayer(H, H, _recipe(8 if qi else 32), gate_layout="fused",
                     pre_batch_input=True)
    if qi:
        _set_h_scale(layer, qi[0], qo[0])
    cell = layer.cell
    with torch.no_grad():
        cell.W_hr.copy_(Wd[0:H]); cell.W_hz.copy_(Wd[H:2 * H]); cell.W_hn.copy_(Wd[2 * H:])
        cell.b_hr.copy_(bh[0:H]); cell.b_hz.copy_(bh[H:2 * H]); cell.b_hn.copy_(bh[2 * H:])
        w = cell.quantize_weights()
        h = h0
        outs = []
        for t in range(T):
            h = cell.step_with_gi(gi[t], h, w)
            outs.append(h)
    return torch.stack(outs)


# ---------------------------------------------------------------------------
# layer level
# ---------------------------------------------------------------------------

def layer_case(name, kind, T, B, I, H, seed, quant, weight_bits=32):
    torch.manual_seed(seed)
    structure = None if kind == "dense" else StructureConfig(kind=kind)
    layer = GRULayer(I, H, _recipe(8 if quant else 32, weight_bits), gate_layout="fused",
                     structure_hidden=structure, use_triton=False)
    if kind == "diagonal":
        with torch.no_grad():
            for m in (layer.cell.struct_Wh_r, layer.cell.struct_Wh_z, layer.cell.struct_Wh_n):
                m.weight.uniform_(-1.0, 1.0)
    if quant:
        _set_h_scale(layer, quant[0][0], quant[1][0])
    x = torch.randn(T, B, I)
    h0 = torch.randn(B, H) * 0.3
    out, hT = layer(x, h0)
    out.sum().backward()
    arrays = {"x": x, "h0": h0, "out": out, "hT": hT}
    for k, p in layer.named_parameters():
        arrays["p:" + k] = p
        arrays["g:" + k] = p.grad
    _save(name, **arrays, **_quant_args(quant))


def calib_case(name, T, B, H, seed):
    torch.manual_seed(seed)
    layer = GRULayer(H, H, _recipe(8, 32, hidden_mode="dynamic"), gate_layout="fused",
                     structure_hidden=StructureConfig(kind="diagonal"))
    batches = [torch.randn(T, B, H) for _ in range(3)]
    summary = layer.calibrate(batches, n_batches=3)
    layer.freeze()
    arrays = {f"x{i}": b for i, b in enumerate(batches)}
    for k, p in layer.named_parameters():
        arrays["p:" + k] = p
    arrays["s_in"] = layer.cell.quant_h_in.scale
    arrays["s_out"] = layer.cell.quant_h_out.scale
    arrays["rmin_in"] = np.float64(summary["cell.quant_h_in"]["running_min"])
    arrays["rmax_in"] = np.float64(summary["cell.quant_h_in"]["running_max"])
    arrays["rmin_out"] = np.float64(summary["cell.quant_h_out"]["running_min"])
    arrays["rmax_out"] = np.float64(summary["cell.quant_h_out"]["running_max"])
    xe = torch.randn(T, B, H)
    out, _ = layer(xe)          # frozen per-step path after calibration
    arrays["x_eval"] = xe
    arrays["out_eval"] = out
    _save(name, **arrays)


def main():
    torch.set_num_threads(1)
    Q = (QP, QP)
    Q2 = ((0.02, -127, 127), (0.013, -127, 127))     # distinct in/out scales
    scan_dense("scan_dense_fp32", 6, 3, 16, 1, None)
    scan_dense("scan_dense_q8", 6, 3, 16, 2, Q)
    scan_dense("scan_dense_q8_asym", 5, 2, 24, 3, Q2)
    scan_formfn("scan_diagonal_fp32", "diagonal", 7, 3, 20, 4, None)
    scan_formfn("scan_diagonal_q8", "diagonal", 7, 3, 20, 5, Q)
    scan_formfn("scan_monarch_fp32", "monarch", 6, 3, 32, 6, None, nblocks=4)
    scan_formfn("scan_monarch_q8", "monarch", 6, 3, 24, 7, Q2, nblocks=2)
    scan_butterfly("scan_butterfly_fp32", 5, 3, 16, 8, None)
    scan_butterfly("scan_butterfly_q8", 5, 2, 16, 9, Q)
    scan_butterfly("scan_butterfly_nb2", 4, 2, 8, 10, None, butterfly_nblocks=2)
    scan_butterfly("scan_butterfly_pad", 4, 2, 12, 11, None)   # H=12 -> H_pad=16
    layer_case("layer_dense_fp32", "dense", 6, 3, 12, 16, 12, None)
    layer_case("layer_dense_w8h8", "dense", 6, 3, 12, 16, 13, Q, weight_bits=8)
    layer_case("layer_diagonal_fp32", "diagonal", 6, 3, 12, 16, 14, None)
    layer_case("layer_diagonal_q8", "diagonal", 6, 3, 12, 16, 15, Q2)
    calib_case("calib_diagonal", 8, 4, 16, 16)


if __name__ == "__main__":
    main()
