"""Fake-quantize modules and recipes (host-side configuration of the GRU layer).

Interface and numerics follow ``gru_qat.quantizers`` (src/gru_qat/quantizers.py):
``QuantizerConfig`` / ``QuantRecipe`` / ``PRESETS`` / ``make_quantizer`` and the
``FakeQuantize`` family with the three observer modes ``dynamic``, ``min_max``
(EMA, momentum 0.99, first call initialises) and ``frozen``.  Only a frozen,
per-tensor, symmetric hidden quantizer crosses into the CUDA scan, as the tuple
``(scale, qmin, qmax)``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Callable, Literal, Optional

import torch
import torch.nn as nn

from .ste import fake_quant_ste

ObserverMode = Literal["dynamic", "min_max", "frozen"]
_EMA_MOMENTUM = 0.99


@dataclass
class QuantizerConfig:
    """Knobs of one quantizer.  ``axis=None`` is per-tensor; an integer axis is
    per-channel, or per-group when ``group_size`` is also given.  ``bits >= 32``
    selects the identity."""

    bits: int = 8
    symmetric: bool = True
    axis: Optional[int] = None
    group_size: Optional[int] = None
    mode: ObserverMode = "dynamic"
    learnable_scale: bool = False
    name: str = "default"


def _code_range(bits: int, symmetric: bool):
    if symmetric:
        top = 2 ** (bits - 1) - 1
        return -top, top
    return 0.0, 2 ** bits - 1.0


class FakeQuantize(nn.Module):
    """Base class: subclasses say how ``(scale, zero_point)`` derive from a tensor."""

    def __init__(self, config: QuantizerConfig) -> None:
        super().__init__()
        self.config = config
        self.qmin, self.qmax = _code_range(config.bits, config.symmetric)
        self.register_buffer("scale", torch.tensor(1.0))
        self.register_buffer("zero_point", torch.tensor(0.0))
        self.register_buffer("running_min", torch.tensor(float("inf")))
        self.register_buffer("running_max", torch.tensor(float("-inf")))
        self._initialized = False

    # -- subclass hook -----------------------------------------------------
    def _compute_scale_zp(self, x):
        raise NotImplementedError

    # -- shared machinery --------------------------------------------------
    def _scale_zp_from_min_max(self, lo, hi):
        if self.config.symmetric:
            scale = torch.maximum(hi.abs(), lo.abs()).clamp(min=1e-8) / self.qmax
            return scale, torch.zeros_like(scale)
        scale = (hi - lo).clamp(min=1e-8) / (self.qmax - self.qmin)
        return scale, torch.round(self.qmin - lo / scale)

    def _update_observer(self, x) -> None:
        xd = x.detach()
        if self.config.axis is None:
            lo, hi = xd.min(), xd.max()
        else:
            other = [d for d in range(xd.ndim) if d != self.config.axis]
            lo, hi = xd.amin(dim=other), xd.amax(dim=other)
        if self._initialized:
            m = _EMA_MOMENTUM
            lo = m * self.running_min + (1 - m) * lo
            hi = m * self.running_max + (1 - m) * hi
        self.running_min, self.running_max = lo, hi
        self._initialized = True

    def forward(self, x):
        mode = self.config.mode
        if mode == "frozen":
            scale, zp = self.scale, self.zero_point
        else:
            scale, zp = self._compute_scale_zp(x)
            if mode == "min_max":
                self._update_observer(x)
        return fake_quant_ste(x, scale, zp, self.qmin, self.qmax)

    def freeze(self) -> None:
        """Fix ``(scale, zero_point)``; a ``min_max`` observer contributes its running range."""
        if self.config.mode == "min_max":
            scale, zp = self._scale_zp_from_min_max(self.running_min, self.running_max)
            self.scale, self.zero_point = scale.detach(), zp.detach()
        self.config.mode = "frozen"


class Identity(FakeQuantize):
    """Pass-through (``bits >= 32``)."""

    def __init__(self, config: Optional[QuantizerConfig] = None) -> None:
        super().__init__(config or QuantizerConfig(name="identity"))

    def forward(self, x):
        return x

    def _compute_scale_zp(self, x):
        return self.scale, self.zero_point


class FakeQuantizePerTensor(FakeQuantize):
    def _compute_scale_zp(self, x):
        return self._scale_zp_from_min_max(x.min(), x.max())


class FakeQuantizePerChannel(FakeQuantize):
    def _compute_scale_zp(self, x):
        other = [d for d in range(x.ndim) if d != self.config.axis]
        return self._scale_zp_from_min_max(x.amin(dim=other, keepdim=True), x.amax(dim=other, keepdim=True))


class FakeQuantizePerGroup(FakeQuantize):
    """Groups of ``group_size`` consecutive indices along ``axis`` share a scale."""

    def _compute_scale_zp(self, x):
        axis, g = self.config.axis, self.config.group_size
        n = x.shape[axis]
        if n % g:
            raise ValueError(f"per-group quant: axis {axis} dim {n} not divisible by group_size {g}")
        moved = x.movedim(axis, 0)
        grouped = moved.reshape(n // g, g, *moved.shape[1:])
        dims = list(range(1, grouped.ndim))
        scale, zp = self._scale_zp_from_min_max(grouped.amin(dim=dims, keepdim=True),
                                                grouped.amax(dim=dims, keepdim=True))
        back = lambda t: t.expand_as(grouped).reshape(moved.shape).movedim(0, axis)  # noqa: E731
        return back(scale), back(zp)


def make_quantizer(config: QuantizerConfig) -> FakeQuantize:
    """Build the quantizer a config describes.  The config is deep-copied so that
    ``freeze()`` on one quantizer never flips the mode of a sibling built from the
    same recipe field."""
    config = copy.deepcopy(config)
    if config.bits >= 32:
        return Identity(config)
    if config.axis is None:
        return FakeQuantizePerTensor(config)
    if config.group_size is None:
        return FakeQuantizePerChannel(config)
    return FakeQuantizePerGroup(config)


QuantizerFactory = Callable[[], FakeQuantize]


def factory(config: QuantizerConfig) -> QuantizerFactory:
    return lambda: make_quantizer(config)


@dataclass
class QuantRecipe:
    """The quantizer configs of one GRU cell: weights, input activation, hidden
    state, and (optionally) gate pre-activations."""

    weight: QuantizerConfig = field(default_factory=lambda: QuantizerConfig(bits=8, axis=0, name="W"))
    input_act: QuantizerConfig = field(default_factory=lambda: QuantizerConfig(bits=8, name="x"))
    hidden: QuantizerConfig = field(default_factory=lambda: QuantizerConfig(bits=8, name="h"))
    gate_act: Optional[QuantizerConfig] = None


PRESETS = {
    "fp32": QuantRecipe(
        weight=QuantizerConfig(bits=32, name="W_id"),
        input_act=QuantizerConfig(bits=32, name="x_id"),
        hidden=QuantizerConfig(bits=32, name="h_id"),
    ),
    "int8_per_channel": QuantRecipe(),
    "int4_per_group_64": QuantRecipe(weight=QuantizerConfig(bits=4, axis=0, group_size=64, name="W")),
}
