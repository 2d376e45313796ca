"""Activation-range calibration (interface of ``gru_qat.calibration``,
src/gru_qat/calibration.py:30-135)."""

from __future__ import annotations

from typing import Iterable

import torch
import torch.nn as nn

from .quantizers import FakeQuantize

_ACTIVATION_LEAVES = frozenset(
    ["quant_x", "quant_h_in", "quant_h_out"]
    + [f"quant_gate_{g}" for g in "rzn"]
    + [f"quant_struct_W{s}_{g}" for s in "ih" for g in "rzn"]
)


@torch.no_grad()
def calibrate(module: nn.Module, loader: Iterable[object], n_batches: int = 64, *,
              only_activations: bool = True, verbose: bool = False):
    """Put the chosen quantizers in ``min_max`` mode with fresh statistics, run up to
    ``n_batches`` eval-mode forwards, and report the observed ranges per quantizer.
    Does not freeze."""
    chosen = [(name, m) for name, m in module.named_modules()
              if isinstance(m, FakeQuantize)
              and (not only_activations or name.rsplit(".", 1)[-1] in _ACTIVATION_LEAVES)]
    for _, m in chosen:
        dev = m.scale.device
        m.config.mode = "min_max"
        m.running_min = torch.tensor(float("inf"), device=dev)
        m.running_max = torch.tensor(float("-inf"), device=dev)
        m._initialized = False

    was_training = module.training
    module.eval()
    try:
        for i, batch in enumerate(loader):
            if i >= n_batches:
                break
            if isinstance(batch, torch.Tensor):
                module(batch)
            elif isinstance(batch, (tuple, list)):
                module(*batch)
            elif isinstance(batch, dict):
                module(**batch)
            else:
                raise TypeError(f"calibrate: loader yielded unsupported type {type(batch)}; "
                                "expected Tensor / tuple / list / dict")
            if verbose:
                print(f"[calibrate] batch {i + 1}/{n_batches}")
    finally:
        if was_training:
            module.train()

    def _val(t):
        return t.item() if t.numel() == 1 else t.flatten().tolist()

    return {name: {"running_min": _val(m.running_min), "running_max": _val(m.running_max),
                   "bits": m.config.bits, "axis": m.config.axis, "initialized": bool(m._initialized)}
            for name, m in chosen}


def freeze_all(module: nn.Module) -> None:
    for m in module.modules():
        if isinstance(m, FakeQuantize):
            m.freeze()
