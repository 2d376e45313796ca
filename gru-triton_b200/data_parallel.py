"""Batch sharding across GPUs.

Sequences are independent, so the scan itself needs no communication: each rank
runs the same weights on its own slice of the batch.  The only collective of a
training step is one all-reduce (sum) of the weight gradients, moved as a single
flat fp32 bucket so that one NCCL launch covers {dWh, dWi, dbh, dbi}.
"""

from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch
import torch.distributed as dist


def shard_bounds(batch: int, rank: int, world: int):
    """[lo, hi) of rank's contiguous batch slice; sizes differ by at most one."""
    base, rem = divmod(batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_batch(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """This rank's slice of ``x`` along the batch dimension (``dim=1`` for [T,B,..], 0 for h0)."""
    lo, hi = shard_bounds(x.shape[dim], rank, world)
    return x.narrow(dim, lo, hi - lo)


class GradBucket:
    """Flat buffer over a fixed list of parameters' gradients; one all-reduce per step.

    ``pack`` and ``unpack`` move all gradients with one multi-tensor copy each, so the bucket adds
    two small kernels and one NCCL launch to a step; all three are stream operations without host
    synchronisation and can sit inside a CUDA-graph capture of the step."""

    def __init__(self, params: Sequence[torch.Tensor]):
        self.params: List[torch.Tensor] = list(params)
        self.sizes = [p.numel() for p in self.params]
        self.flat: Optional[torch.Tensor] = None
        self._views: List[torch.Tensor] = []

    def _ensure(self) -> None:
        if self.flat is None:
            p0 = self.params[0]
            self.flat = torch.zeros(sum(self.sizes), dtype=p0.dtype, device=p0.device)
            self._views = [v.view_as(p) for v, p in zip(self.flat.split(self.sizes), self.params)]

    def pack(self) -> None:
        """Gradients -> flat buffer (parameters without a gradient contribute zeros)."""
        self._ensure()
        have = [(v, p.grad) for v, p in zip(self._views, self.params) if p.grad is not None]
        for v, p in zip(self._views, self.params):
            if p.grad is None:
                v.zero_()
        if have:
            torch._foreach_copy_([v for v, _ in have], [g for _, g in have])

    def unpack(self) -> None:
        """Reduced flat buffer -> ``.grad`` of every parameter."""
        dst, src = [], []
        for v, p in zip(self._views, self.params):
            if p.grad is None:
                p.grad = v.clone()
            else:
                dst.append(p.grad)
                src.append(v)
        if dst:
            torch._foreach_copy_(dst, src)

    def all_reduce(self, group=None, async_op: bool = False):
        """Sum the gradients of all ranks in place.  Returns the work handle when async
        (then call :meth:`scatter` once it has completed)."""
        self.pack()
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        if async_op:
            return work
        self.unpack()
        return None

    def scatter(self) -> None:
        """Write the reduced bucket back into ``.grad`` (after an async reduce completes)."""
        self.unpack()


def all_reduce_gradients(params: Iterable[torch.Tensor], group=None) -> None:
    """Convenience: build a bucket over ``params`` and sum-reduce it once."""
    GradBucket(list(params)).all_reduce(group=group)
