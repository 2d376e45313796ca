"""One GRU time step with fake-quant insertion points.

Interface and arithmetic follow ``gru_qat.gru_cell.GRUCellQuant``
(src/gru_qat/gru_cell.py:64-553); parameter and quantizer attribute names are
kept so that a ``state_dict`` moves between the two packages.  This per-step
path is what ``calibrate()`` runs and what CPU tensors take; CUDA layers with a
structured hidden side are routed to the persistent scan kernels by ``GRULayer``.

    r = sigmoid(W_ir x + b_ir + W_hr hq + b_hr)      hq = quant_h_in(h)
    z = sigmoid(W_iz x + b_iz + W_hz hq + b_hz)
    n = tanh   (W_in x + b_in + r * (W_hn hq + b_hn))
    h' = quant_h_out((1 - z) * n + z * h)             (blend uses the unquantised h)
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .quantizers import FakeQuantize, QuantizerConfig, QuantRecipe, make_quantizer
from .structure import StructureConfig, make_structured_linear

GateLayout = Literal["split", "fused"]
_GATES = ("r", "z", "n")
_BIASES = tuple(f"b_{side}{g}" for side in "ih" for g in _GATES)


@dataclass
class CellWeights:
    """Fake-quantised dense weights of one forward pass (quantised once, reused
    at every step).  The ``*_cat`` fields exist for ``gate_layout='fused'``: rows
    stacked r, z, n."""

    Wir: torch.Tensor
    Wiz: torch.Tensor
    Win: torch.Tensor
    Whr: torch.Tensor
    Whz: torch.Tensor
    Whn: torch.Tensor
    Wi_cat: Optional[torch.Tensor] = None
    Wh_cat: Optional[torch.Tensor] = None
    bi_cat: Optional[torch.Tensor] = None
    bh_cat: Optional[torch.Tensor] = None


def _is_dense(cfg: Optional[StructureConfig]) -> bool:
    return cfg is None or cfg.kind == "dense"


class GRUCellQuant(nn.Module):
    def __init__(self, input_size: int, hidden_size: int, recipe: QuantRecipe, *,
                 gate_layout: GateLayout = "split", bias: bool = True,
                 structure_input: Optional[StructureConfig] = None,
                 structure_hidden: Optional[StructureConfig] = None) -> None:
        super().__init__()
        if gate_layout == "fused" and recipe.weight.axis != 0:
            raise ValueError("fused gate layout requires recipe.weight.axis=0; "
                             f"got axis={recipe.weight.axis}. Per-tensor weight quant "
                             "is not supported with fused gates.")
        self.input_size, self.hidden_size, self.gate_layout = input_size, hidden_size, gate_layout
        self._input_dense, self._hidden_dense = _is_dense(structure_input), _is_dense(structure_hidden)
        self._structure_input, self._structure_hidden = structure_input, structure_hidden

        for side, dense, n_in, cfg in (("i", self._input_dense, input_size, structure_input),
                                       ("h", self._hidden_dense, hidden_size, structure_hidden)):
            for g in _GATES:
                if dense:
                    setattr(self, f"W_{side}{g}", nn.Parameter(torch.empty(hidden_size, n_in)))
                else:
                    setattr(self, f"struct_W{side}_{g}",
                            make_structured_linear(cfg, n_in, hidden_size, bias=False))
            if not dense:          # structured products are fake-quantised on their OUTPUT
                for g in _GATES:
                    setattr(self, f"quant_struct_W{side}_{g}", make_quantizer(recipe.weight))

        for name in _BIASES:
            if bias:
                setattr(self, name, nn.Parameter(torch.zeros(hidden_size)))
            else:
                self.register_parameter(name, None)
        self.reset_parameters()

        self.quant_x = make_quantizer(recipe.input_act)
        self.quant_h_in = make_quantizer(recipe.hidden)
        self.quant_h_out = make_quantizer(recipe.hidden)
        for side in "ih":
            for g in _GATES:
                setattr(self, f"quant_W_{side}{g}", make_quantizer(recipe.weight))
        gate_cfg = recipe.gate_act or QuantizerConfig(bits=32, name="gate_id")
        for g in _GATES:
            setattr(self, f"quant_gate_{g}", make_quantizer(gate_cfg))

    # ------------------------------------------------------------------
    @property
    def is_structured(self) -> bool:
        return not (self._input_dense and self._hidden_dense)

    def reset_parameters(self) -> None:
        k = self.hidden_size ** -0.5
        names = []
        if self._input_dense:
            names += [f"W_i{g}" for g in _GATES]
        if self._hidden_dense:
            names += [f"W_h{g}" for g in _GATES]
        for name in names + list(_BIASES):
            p = getattr(self, name)
            if p is not None:
                nn.init.uniform_(p, -k, k)

    def _cat_bias(self, side: str):
        if self.b_ir is None:
            return None
        return torch.cat([getattr(self, f"b_{side}{g}") for g in _GATES])

    # ------------------------------------------------------------------
    def quantize_weights(self) -> CellWeights:
        """All six dense weights through their quantizers, once per forward."""
        if self.is_structured:
            raise RuntimeError("quantize_weights() is dense-only; use the structured "
                               "forward path (cell.forward(x, h)) for structured cells.")
        q = {f"{s}{g}": getattr(self, f"quant_W_{s}{g}")(getattr(self, f"W_{s}{g}"))
             for s in "ih" for g in _GATES}
        w = CellWeights(q["ir"], q["iz"], q["in"], q["hr"], q["hz"], q["hn"])
        if self.gate_layout == "fused":
            w.Wi_cat = torch.cat([w.Wir, w.Wiz, w.Win], dim=0)
            w.Wh_cat = torch.cat([w.Whr, w.Whz, w.Whn], dim=0)
            w.bi_cat, w.bh_cat = self._cat_bias("i"), self._cat_bias("h")
        return w

    def quantize_input_weights(self):
        """``(Wi_cat, bi_cat)`` for one GEMM over the whole sequence (dense input side)."""
        if not self._input_dense:
            raise RuntimeError("quantize_input_weights() requires dense input side; "
                               "cell has structured input.")
        Wi = torch.cat([getattr(self, f"quant_W_i{g}")(getattr(self, f"W_i{g}")) for g in _GATES], dim=0)
        return Wi, self._cat_bias("i")

    # ------------------------------------------------------------------
    def _finish(self, pre_r, pre_z, gi_n, gh_n, h):
        r = torch.sigmoid(self.quant_gate_r(pre_r))
        z = torch.sigmoid(self.quant_gate_z(pre_z))
        n = torch.tanh(self.quant_gate_n(gi_n + r * gh_n))
        return self.quant_h_out((1.0 - z) * n + z * h)

    def _side(self, side: str, act):
        """Per-gate projections of one side (dense with weight quant, or structured
        with output quant), bias included."""
        outs = []
        dense = self._input_dense if side == "i" else self._hidden_dense
        for g in _GATES:
            b = getattr(self, f"b_{side}{g}")
            if dense:
                Wq = getattr(self, f"quant_W_{side}{g}")(getattr(self, f"W_{side}{g}"))
                outs.append(F.linear(act, Wq, b))
            else:
                y = getattr(self, f"quant_struct_W{side}_{g}")(getattr(self, f"struct_W{side}_{g}")(act))
                outs.append(y if b is None else y + b)
        return outs

    def step_structured(self, x, h):
        gi_r, gi_z, gi_n = self._side("i", self.quant_x(x))
        gh_r, gh_z, gh_n = self._side("h", self.quant_h_in(h))
        return self._finish(gi_r + gh_r, gi_z + gh_z, gi_n, gh_n, h)

    def step(self, x, h, w: CellWeights):
        xq, hq = self.quant_x(x), self.quant_h_in(h)
        if self.gate_layout == "fused":
            gi_r, gi_z, gi_n = F.linear(xq, w.Wi_cat, w.bi_cat).chunk(3, dim=-1)
            gh_r, gh_z, gh_n = F.linear(hq, w.Wh_cat, w.bh_cat).chunk(3, dim=-1)
            return self._finish(gi_r + gh_r, gi_z + gh_z, gi_n, gh_n, h)
        pre_r = F.linear(xq, w.Wir, self.b_ir) + F.linear(hq, w.Whr, self.b_hr)
        pre_z = F.linear(xq, w.Wiz, self.b_iz) + F.linear(hq, w.Whz, self.b_hz)
        return self._finish(pre_r, pre_z, F.linear(xq, w.Win, self.b_in), F.linear(hq, w.Whn, self.b_hn), h)

    def input_projection(self, x_seq, w: CellWeights):
        """``quant_x(x_seq) @ Wi_cat^T + bi_cat`` for all steps at once: [T, B, 3H]."""
        if self.gate_layout != "fused":
            raise RuntimeError("input_projection requires gate_layout='fused'")
        return F.linear(self.quant_x(x_seq), w.Wi_cat, w.bi_cat)

    def step_with_gi(self, gi_t, h, w: CellWeights):
        gh_r, gh_z, gh_n = F.linear(self.quant_h_in(h), w.Wh_cat, w.bh_cat).chunk(3, dim=-1)
        gi_r, gi_z, gi_n = gi_t.chunk(3, dim=-1)
        return self._finish(gi_r + gh_r, gi_z + gh_z, gi_n, gh_n, h)

    def structured_input_projection(self, x_seq):
        """Structured input side applied to the whole sequence: [T, B, 3H]."""
        if self._input_dense:
            raise RuntimeError("structured_input_projection() requires a structured input side; use "
                               "input_projection() / quantize_input_weights() for the dense path.")
        T, B, _ = x_seq.shape
        flat = self.quant_x(x_seq).reshape(T * B, self.input_size)
        return torch.cat(self._side("i", flat), dim=-1).reshape(T, B, 3 * self.hidden_size)

    def forward(self, x, h):
        if self.is_structured:
            return self.step_structured(x, h)
        return self.step(x, h, self.quantize_weights())

    @classmethod
    def from_recipe(cls, input_size, hidden_size, recipe, **kwargs):
        return cls(input_size, hidden_size, recipe, **kwargs)

    def freeze_quantizers(self) -> None:
        for m in self.modules():
            if isinstance(m, FakeQuantize):
                m.freeze()
