"""Structured hidden/input weight parameterisations.

Interface follows ``gru_qat.structure`` (src/gru_qat/structure.py:34-187):
``StructureConfig`` + ``make_structured_linear``.  The reference builds its
block-diagonal ("monarch") and butterfly layers from the third-party
``torch_structured`` package; this module carries self-contained equivalents
with the same parameter names and shapes, so that the scan's factor extractors
read them the same way:

* ``BlockdiagLinear.weight``  -- ``[nblocks, out_blk, in_blk]``; ``y[.., n*ob+o] =
  sum_i W[n,o,i] x[.., n*ib+i]`` (the product of scan_monarch.py:110-112).
* ``Butterfly.twiddle``       -- ``[1, nblocks, log2(n), n/2, 2, 2]``; stage
  arithmetic of scan_butterfly.py:276-317 (even blocks: strides 1,2,4,..; odd
  blocks: reversed; input zero-padded to the next power of two).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Literal

import torch
import torch.nn as nn

StructuredKind = Literal["dense", "diagonal", "monarch", "circulant", "butterfly", "ldr"]


@dataclass
class StructureConfig:
    kind: StructuredKind = "dense"
    nblocks: int = 4               # monarch: number of diagonal blocks
    butterfly_nblocks: int = 1     # butterfly: stacked factors (depth = nblocks * log2 n)
    ldr_rank: int = 2
    init: str = "randn"


def _is_pow2(n: int) -> bool:
    return n > 0 and n & (n - 1) == 0


def _validate_shapes(kind, in_features, out_features, cfg) -> None:
    square = in_features == out_features
    if kind in ("diagonal", "circulant", "ldr") and not square:
        raise ValueError(f"{kind} requires square (in == out); got in={in_features}, out={out_features}")
    if kind == "monarch" and (in_features % cfg.nblocks or out_features % cfg.nblocks):
        raise ValueError(f"monarch requires in/out divisible by nblocks={cfg.nblocks}; "
                         f"got in={in_features}, out={out_features}")
    if kind == "circulant" and not _is_pow2(in_features):
        raise ValueError(f"circulant requires power-of-2 size; got {in_features}")
    if kind == "butterfly":
        if in_features < 2 or out_features < 2:
            raise ValueError("butterfly requires in/out >= 2 (a size-1 butterfly factorization has 0 "
                             f"stages and is undefined); got in={in_features}, out={out_features}")
        big = max(in_features, out_features)
        padded = 1 << math.ceil(math.log2(big))
        if padded > 2 * big:
            raise ValueError(f"butterfly: zero-padding to {padded} more than doubles the requested "
                             "size; pick a closer-to-pow-of-2 dim")


class _DiagonalLinear(nn.Module):
    """``y = x * w`` with one weight per feature."""

    def __init__(self, n: int, *, bias: bool = False) -> None:
        super().__init__()
        self.n = n
        self.weight = nn.Parameter(torch.empty(n))
        self.bias = nn.Parameter(torch.zeros(n)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.uniform_(self.weight, -self.n ** -0.5, self.n ** -0.5)

    def forward(self, x):
        y = x * self.weight
        return y if self.bias is None else y + self.bias


class BlockdiagLinear(nn.Module):
    """One block-diagonal factor: ``nblocks`` independent ``[out_blk, in_blk]`` blocks."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, nblocks: int = 4) -> None:
        super().__init__()
        self.in_features, self.out_features, self.nblocks = in_features, out_features, nblocks
        self.in_blksz, self.out_blksz = in_features // nblocks, out_features // nblocks
        self.weight = nn.Parameter(torch.empty(nblocks, self.out_blksz, self.in_blksz))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.uniform_(self.weight, -self.in_blksz ** -0.5, self.in_blksz ** -0.5)

    def forward(self, x):
        lead = x.shape[:-1]
        xb = x.reshape(-1, self.nblocks, self.in_blksz)
        y = torch.einsum("bni,noi->bno", xb, self.weight).reshape(*lead, self.out_features)
        return y if self.bias is None else y + self.bias


def butterfly_apply(twiddle: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Rows of ``x`` [N, n] through ``twiddle`` [nblocks, log2 n, n/2, 2(new), 2(old)]."""
    nblocks, log_n, half = twiddle.shape[:3]
    n = 2 * half
    N = x.shape[0]
    for blk in range(nblocks):
        for s in range(log_n):
            ls = s if blk % 2 == 0 else log_n - 1 - s
            stride = 1 << ls
            groups = n // (2 * stride)
            xv = x.reshape(N, groups, 2, stride)
            tv = twiddle[blk, s].reshape(groups, stride, 2, 2)
            x = torch.einsum("glnm,bgml->bgnl", tv, xv).reshape(N, n)
    return x


class Butterfly(nn.Module):
    """Product of ``nblocks * log2(n)`` sparse 2x2-mixing stages, n = next power of two."""

    def __init__(self, in_size: int, out_size: int, bias: bool = False, init: str = "randn",
                 nblocks: int = 1) -> None:
        super().__init__()
        self.in_size, self.out_size, self.nblocks = in_size, out_size, nblocks
        self.log_n = max(1, math.ceil(math.log2(max(in_size, out_size))))
        self.n = 1 << self.log_n
        if init == "randn":
            tw = torch.randn(1, nblocks, self.log_n, self.n // 2, 2, 2) * 2 ** -0.5
        elif init == "identity":
            tw = torch.eye(2).expand(1, nblocks, self.log_n, self.n // 2, 2, 2).clone()
        else:
            raise ValueError(f"unknown butterfly init {init!r}")
        self.twiddle = nn.Parameter(tw)
        self.bias = nn.Parameter(torch.zeros(out_size)) if bias else None

    def forward(self, x):
        lead = x.shape[:-1]
        flat = x.reshape(-1, self.in_size)
        if self.in_size < self.n:
            flat = nn.functional.pad(flat, (0, self.n - self.in_size))
        y = butterfly_apply(self.twiddle[0], flat)[:, : self.out_size].reshape(*lead, self.out_size)
        return y if self.bias is None else y + self.bias


class _ButterflyLinear(nn.Module):
    """Holds the butterfly as ``.b`` (the attribute the twiddle extractor reads)."""

    def __init__(self, butterfly: nn.Module) -> None:
        super().__init__()
        self.b = butterfly

    def forward(self, x):
        return self.b(x)


class _CirculantLinear(nn.Module):
    """``y = irfft(rfft(col) * rfft(x))``: multiplication by a circulant matrix."""

    def __init__(self, n: int, *, bias: bool = False) -> None:
        super().__init__()
        self.n = n
        self.col = nn.Parameter(torch.randn(n) / n ** 0.5)
        self.bias = nn.Parameter(torch.zeros(n)) if bias else None

    def forward(self, x):
        y = torch.fft.irfft(torch.fft.rfft(self.col) * torch.fft.rfft(x, dim=-1), n=self.n, dim=-1)
        return y if self.bias is None else y + self.bias


class _LDRLinear(nn.Module):
    def __init__(self, ldr: nn.Module) -> None:
        super().__init__()
        self.ldr = ldr

    def forward(self, x):
        return self.ldr(x)


def make_structured_linear(cfg: StructureConfig, in_features: int, out_features: int, *,
                           bias: bool = False) -> nn.Module:
    """An ``nn.Linear``-like module parameterised as ``cfg.kind`` asks."""
    if cfg.kind == "dense":
        return nn.Linear(in_features, out_features, bias=bias)
    _validate_shapes(cfg.kind, in_features, out_features, cfg)
    if cfg.kind == "diagonal":
        return _DiagonalLinear(in_features, bias=bias)
    if cfg.kind == "monarch":
        return BlockdiagLinear(in_features, out_features, bias=bias, nblocks=cfg.nblocks)
    if cfg.kind == "circulant":
        return _CirculantLinear(in_features, bias=bias)
    if cfg.kind == "butterfly":
        return _ButterflyLinear(Butterfly(in_features, out_features, bias=bias, init=cfg.init,
                                          nblocks=cfg.butterfly_nblocks))
    if cfg.kind == "ldr":
        try:
            from torch_structured.structured.layers import LDRSubdiagonal
        except ImportError as e:
            raise ImportError("kind='ldr' needs the optional torch-structured package") from e
        return _LDRLinear(LDRSubdiagonal(layer_size=in_features, r=cfg.ldr_rank, bias=bias))
    raise ValueError(f"unknown structured kind: {cfg.kind!r}")
