"""Sequence driver over ``GRUCellQuant``.

Interface of ``gru_qat.gru_layer.GRULayer`` (src/gru_qat/gru_layer.py:52-342):
same constructor keywords, ``forward(x, h0=None) -> (out, h_T)``,
``calibrate()`` / ``freeze()``.  With ``use_triton`` in effect (the keyword keeps
the reference's name; there is no Triton here) a CUDA input takes the fast path:
one GEMM for the input projection of the whole sequence, then ONE persistent
CUDA scan over all T steps.  Eligible: diagonal / monarch / butterfly hidden
side with fused gates, as in the reference, and -- an extension the reference
does not have (its dense layers always step in Python, gru_layer.py:109-124) --
fully dense layers with fused gates and no gate-activation quantizer.  CPU
tensors, ineligible layers and ``calibrate()`` run the per-step loop.
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn as nn

from .gru_cell import GateLayout, GRUCellQuant
from .quantizers import FakeQuantize, FakeQuantizePerChannel, FakeQuantizePerTensor, Identity, QuantRecipe
from .structure import StructureConfig

_FAST_KINDS = ("diagonal", "monarch", "butterfly")


def _extract_h_quant_params(quantizer: FakeQuantize):
    """``(scale, qmin, qmax)`` if the quantizer is frozen, per-tensor and symmetric --
    the only form the scan kernels apply -- else None (gru_layer.py:30-48).

    The reference reads the scale with ``.item()`` at every forward (a device-to-host sync);
    here the host copy is kept beside the quantizer and re-read only when the scale tensor was
    replaced or written, so a frozen layer's forward neither synchronises nor breaks a CUDA-graph
    capture."""
    cfg = quantizer.config
    if cfg.mode != "frozen" or not isinstance(quantizer, FakeQuantizePerTensor) or not cfg.symmetric:
        return None
    scale = quantizer.scale
    key = (id(scale), scale._version, scale.device)
    cached = getattr(quantizer, "_host_scale", None)
    if cached is None or cached[0] != key:
        cached = (key, float(scale.item()))
        quantizer._host_scale = cached
    return cached[1], int(quantizer.qmin), int(quantizer.qmax)


class GRULayer(nn.Module):
    def __init__(self, input_size: int, hidden_size: int, recipe: QuantRecipe, *,
                 batch_first: bool = False, gate_layout: GateLayout = "split",
                 compile_step: bool = False, pre_batch_input: bool = False,
                 structure_input: Optional[StructureConfig] = None,
                 structure_hidden: Optional[StructureConfig] = None,
                 use_triton="auto") -> None:
        super().__init__()
        if pre_batch_input and gate_layout != "fused":
            raise ValueError("pre_batch_input=True requires gate_layout='fused'")
        self.cell = GRUCellQuant(input_size, hidden_size, recipe, gate_layout=gate_layout,
                                 structure_input=structure_input, structure_hidden=structure_hidden)
        if self.cell.is_structured and pre_batch_input:
            raise ValueError("pre_batch_input is not supported in structured mode "
                             "(no dense Wi_cat to pre-project).")
        self.hidden_size, self.batch_first, self.pre_batch_input = hidden_size, batch_first, pre_batch_input
        self._calibrating = False

        kind = structure_hidden.kind if structure_hidden is not None else None
        if kind in (None, "dense"):
            kind = "dense"
            eligible = (not self.cell.is_structured and gate_layout == "fused" and
                        all(isinstance(getattr(self.cell, f"quant_gate_{g}"), Identity) for g in "rzn"))
        else:
            eligible = kind in _FAST_KINDS and gate_layout == "fused"
        self._fast_dispatch_eligible = eligible
        self._dispatch_kind = kind if eligible else None
        if use_triton == "auto":
            self.use_triton = eligible
        else:
            self.use_triton = bool(use_triton)
            if self.use_triton and not eligible:
                raise ValueError("use_triton=True requires gate_layout='fused' and either structure_hidden.kind in "
                                 "{'diagonal', 'monarch', 'butterfly'} or a fully dense layer without gate-"
                                 "activation quantizers.")

        if self.cell.is_structured:
            body = self.cell.step_structured
        elif pre_batch_input:
            body = self.cell.step_with_gi
        else:
            body = self.cell.step
        self._compiled_step = torch.compile(body, mode="default", dynamic=False) if compile_step else body

    # ------------------------------------------------------------------
    def forward(self, x: torch.Tensor, h0: Optional[torch.Tensor] = None):
        if self.batch_first:
            x = x.transpose(0, 1)
        T, B, _ = x.shape
        if T == 0:
            raise ValueError(f"seq length T must be > 0; got T={T}")
        if B == 0:
            raise ValueError(f"batch size B must be > 0; got B={B}")
        if h0 is None:
            h0 = x.new_zeros(B, self.hidden_size)

        if self.use_triton and x.is_cuda:
            return self._forward_fast_dispatch(x, h0)
        if self._calibrating and x.is_cuda and self._device_calibration_ok():
            return self._forward_calibration_scan(x, h0)

        step, h, outs = self._compiled_step, h0, []
        if self.cell.is_structured:
            for t in range(T):
                h = step(x[t], h)
                outs.append(h)
        else:
            w = self.cell.quantize_weights()
            seq = self.cell.input_projection(x, w) if self.pre_batch_input else x
            for t in range(T):
                h = step(seq[t], h, w)
                outs.append(h)
        out = torch.stack(outs, dim=0)
        return (out.transpose(0, 1) if self.batch_first else out), h

    # ------------------------------------------------------------------
    def _device_calibration_ok(self) -> bool:
        """calibrate() can observe on the device when the layer is dispatchable, the two hidden
        quantizers are the per-tensor symmetric observers and nothing else on the path quantises
        activations (input, gate and structured-output quantizers are identities)."""
        cell = self.cell
        if not self._fast_dispatch_eligible:
            return False
        qi, qo = cell.quant_h_in, cell.quant_h_out
        for q in (qi, qo):
            if not isinstance(q, FakeQuantizePerTensor) or not q.config.symmetric or q.config.mode != "min_max":
                return False
            if q.running_min.numel() != 1 or not q.running_min.is_cuda or q.running_min.dtype != torch.float32:
                return False
        if int(qi.qmax) != int(qo.qmax):
            return False
        others = [cell.quant_x] + [getattr(cell, f"quant_gate_{g}") for g in "rzn"]
        others += [m for n, m in cell.named_children() if n.startswith("quant_struct_W")]
        return all(isinstance(q, Identity) for q in others)

    def _forward_calibration_scan(self, x, h0):
        """One calibration forward on the device: the scan with both hidden quantizers observing
        (dynamic scale per call, running range blended with the observers' momentum), the same
        arithmetic the per-step cell performs in ``min_max`` mode (quantizers.py:95-156)."""
        from . import _lib
        from .quantizers import _EMA_MOMENTUM
        cell = self.cell
        gi = self._input_projection_fast(x) if cell._input_dense else cell.structured_input_projection(x)
        kind, kw = self._dispatch_kind, {}
        if kind == "dense":
            W = torch.cat([getattr(cell, f"quant_W_h{g}")(getattr(cell, f"W_h{g}")) for g in "rzn"], dim=0)
            bh = cell._cat_bias("h")
            bh = gi.new_zeros(3 * self.hidden_size) if bh is None else bh
        elif kind == "diagonal":
            from .scan_diagonal import extract_diagonal_factors
            W, bh = extract_diagonal_factors(cell)
        elif kind == "monarch":
            from .scan_monarch import extract_monarch_factors
            W, bh = extract_monarch_factors(cell)
            kw["nblocks"] = W.shape[1]
        else:
            from .scan_butterfly import extract_butterfly_twiddles
            W, bh = extract_butterfly_twiddles(cell)
            kw["nblocks"], kw["log2_hpad"] = W.shape[1], W.shape[2]
        qi, qo = cell.quant_h_in, cell.quant_h_out
        out = _lib.calibration_scan(kind, gi.contiguous(), h0.contiguous(), W.detach().contiguous(),
                                    bh.detach().contiguous(), int(qi.qmax), _EMA_MOMENTUM,
                                    (qi.running_min, qi.running_max, qi._initialized),
                                    (qo.running_min, qo.running_max, qo._initialized), **kw)
        qi._initialized = qo._initialized = True
        return (out.transpose(0, 1) if self.batch_first else out), out[-1]

    def _weight_bits_on_device(self, side: str):
        """Bit width if the three weight quantizers of a side are the per-output-row symmetric
        dynamic int<=8 kind the weight-prep kernel implements, 32 if they are identities, else None
        (then the quantizer modules themselves run, as in the per-step path)."""
        qs = [getattr(self.cell, f"quant_W_{side}{g}") for g in "rzn"]
        if all(isinstance(q, Identity) for q in qs):
            return 32
        c = qs[0].config
        if (all(isinstance(q, FakeQuantizePerChannel) for q in qs) and c.axis == 0 and c.symmetric and
                c.mode == "dynamic" and c.bits <= 8 and
                all(q.config.bits == c.bits and q.config.mode == "dynamic" and q.config.symmetric for q in qs)):
            return int(c.bits)
        return None

    def _input_projection_fast(self, x):
        """``gi[T,B,3H]`` on the tensor cores (fp32-accurate split products)."""
        from . import tc
        cell = self.cell
        bits = self._weight_bits_on_device("i")
        xq = cell.quant_x(x)
        I = cell.input_size
        if bits is None or I % 8 or self.hidden_size % 8 or xq.dtype != torch.float32:
            Wi_cat, bi_cat = cell.quantize_input_weights()
            return nn.functional.linear(xq, Wi_cat, bi_cat)
        Wi_raw = torch.cat([getattr(cell, f"W_i{g}") for g in "rzn"], dim=0)
        return tc.linear(xq, Wi_raw, cell._cat_bias("i"), weight_bits=bits)

    def _forward_fast_dispatch(self, x, h0):
        """Input projection hoisted to one GEMM, then the persistent CUDA scan
        (gru_layer.py:234-302)."""
        cell = self.cell
        if cell._input_dense:
            gi = self._input_projection_fast(x)
        else:
            gi = cell.structured_input_projection(x)
        quant = dict(h_in_quant=_extract_h_quant_params(cell.quant_h_in),
                     h_out_quant=_extract_h_quant_params(cell.quant_h_out))

        if self._dispatch_kind == "dense":
            from . import tc
            from .scan import gru_scan_persistent
            bits = self._weight_bits_on_device("h")
            bh_cat = cell._cat_bias("h")
            if bh_cat is None:
                bh_cat = gi.new_zeros(3 * self.hidden_size)
            if bits is not None and bits <= 8 and self.hidden_size % 4 == 0:
                Wh_raw = torch.cat([getattr(cell, f"W_h{g}") for g in "rzn"], dim=0)
                out = tc.gru_scan_dense_q8(gi, h0, Wh_raw, bh_cat, weight_bits=bits, **quant)
            else:
                Wh_cat = torch.cat([getattr(cell, f"quant_W_h{g}")(getattr(cell, f"W_h{g}")) for g in "rzn"], dim=0)
                out = gru_scan_persistent(gi, h0, Wh_cat, bh_cat, **quant)
        elif self._dispatch_kind == "diagonal":
            from .scan_diagonal import extract_diagonal_factors, gru_scan_diagonal
            out = gru_scan_diagonal(gi, h0, *extract_diagonal_factors(cell), **quant)
        elif self._dispatch_kind == "monarch":
            from .scan_monarch import extract_monarch_factors, gru_scan_monarch
            out = gru_scan_monarch(gi, h0, *extract_monarch_factors(cell), **quant)
        elif self._dispatch_kind == "butterfly":
            from .scan_butterfly import extract_butterfly_twiddles, gru_scan_butterfly_cuda
            out = gru_scan_butterfly_cuda(gi, h0, *extract_butterfly_twiddles(cell), **quant)
        else:
            raise RuntimeError(f"unexpected dispatch kind {self._dispatch_kind!r}")
        h_T = out[-1]
        return (out.transpose(0, 1) if self.batch_first else out), h_T

    # ------------------------------------------------------------------
    @torch.no_grad()
    def calibrate(self, loader: Iterable[object], n_batches: int = 64, *, only_activations: bool = True,
                  device_scan: bool = True):
        """Observe activation ranges over ``n_batches`` forwards.  The fast path reads frozen scales
        but never runs the hidden quantizers, so it is switched off for the duration, as in the
        reference (gru_layer.py:323-339).  CUDA batches of a dispatchable layer whose only
        activation quantizers are the two hidden-state observers are observed on the device by
        the calibration scan; everything else steps the cell in Python.  Call :meth:`freeze`
        afterwards."""
        from .calibration import calibrate as _calibrate
        saved, self.use_triton = self.use_triton, False
        self._calibrating = bool(saved) and device_scan
        try:
            return _calibrate(self, loader, n_batches=n_batches, only_activations=only_activations)
        finally:
            self.use_triton = saved
            self._calibrating = False

    def freeze(self) -> None:
        self.cell.freeze_quantizers()
