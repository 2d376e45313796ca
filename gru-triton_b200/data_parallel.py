"""Batch sharding across GPUs.

Sequences are independent, so the scan itself needs no communication: each rank
runs the same weights on its own slice of the batch.  The only collective of a
training step is the all-reduce (sum) of the weight gradients, moved as flat fp32
buckets: one bucket over {dWh, dWi, dbh, dbi} (``GradBucket``), or one bucket per group of
parameters reduced on a side stream as soon as the backward pass has produced the group's
gradients (``OverlappedReducer``: the hidden-path gradients travel while the input projection's
backward still runs).
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

    def all_reduce_in_place(self, group=None) -> None:
        """Sum the gradients of all ranks where they lie: one coalesced collective over the ``.grad``
        tensors themselves (the backend groups them into one launch), no flat copy in or out.
        Every rank must hold a gradient for the same parameters."""
        grads = [p.grad for p in self.params if p.grad is not None]
        if not grads:
            return
        with dist._coalescing_manager(group=group):
            for g in grads:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)


class OverlappedReducer:
    """All-reduce of several gradient buckets, each started the moment its last gradient exists.

    ``buckets``: lists of parameters, in the order the backward pass completes them.  A
    post-accumulate hook on every parameter counts a bucket's finished gradients; the last one
    launches pack -> all-reduce -> unpack of that bucket on a side CUDA stream that first waits for
    the producing stream, so the collective overlaps whatever the backward pass still has to do.
    By default a bucket is reduced in place (one coalesced collective over its ``.grad`` tensors);
    with ``in_place=False``, or when a parameter of the bucket has no gradient, through the flat
    copy of ``GradBucket``.
    ``finish()`` reduces the buckets whose hooks never fired (parameters without a gradient), makes
    the current stream wait for the side stream and re-arms the counters.  Everything is a stream
    operation: a step using it can be captured in a CUDA graph (the side stream becomes a parallel
    branch of the graph).  On CPU tensors (gloo) the reductions run in place, in the same order."""

    def __init__(self, buckets: Sequence[Sequence[torch.Tensor]], group=None, in_place: bool = True):
        self.group = group
        self.in_place = in_place          # coalesced all-reduce of the .grad tensors; else flat buckets
        self.buckets = [GradBucket(list(ps)) for ps in buckets if len(ps)]
        self._done = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self._stream: Optional[torch.cuda.Stream] = None
        self._handles = []
        for bi, b in enumerate(self.buckets):
            for p in b.params:
                self._handles.append(p.register_post_accumulate_grad_hook(self._make_hook(bi)))

    def _make_hook(self, bi: int):
        def hook(_param):
            self._done[bi] += 1
            if self._done[bi] == len(self.buckets[bi].params) and not self._launched[bi]:
                self._launch(bi)
        return hook

    def _launch(self, bi: int) -> None:
        self._launched[bi] = True
        b = self.buckets[bi]
        if b.params[0].is_cuda:
            if self._stream is None:
                self._stream = torch.cuda.Stream(device=b.params[0].device)
            self._stream.wait_stream(torch.cuda.current_stream(b.params[0].device))
            with torch.cuda.stream(self._stream):
                self._reduce(b)
        else:
            self._reduce(b)

    def _reduce(self, b: GradBucket) -> None:
        if self.in_place and all(p.grad is not None for p in b.params):
            b.all_reduce_in_place(group=self.group)
        else:
            b.all_reduce(group=self.group)

    def finish(self) -> None:
        """Call after ``backward()``: every bucket reduced, gradients visible to the current stream."""
        for bi in range(len(self.buckets)):
            if not self._launched[bi]:
                self._launch(bi)
        if self._stream is not None:
            torch.cuda.current_stream(self.buckets[0].params[0].device).wait_stream(self._stream)
        self._done = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []


def hidden_then_input_buckets(module: torch.nn.Module):
    """Two parameter groups of a ``GRULayer`` in the order its backward pass finishes them: the
    hidden path (scan backward: W_h*, b_h*, structured hidden factors), then everything else (the
    input projection's weights and biases)."""
    hidden, rest = [], []
    for name, p in module.named_parameters():
        leaf = name.rsplit(".", 1)[-1]
        (hidden if ("W_h" in name or "b_h" in leaf or "struct_Wh" in name) else rest).append(p)
    return [hidden, rest]


def all_reduce_gradients(params: Iterable[torch.Tensor], group=None) -> None:
    """Convenience: build a bucket over ``params`` and sum-reduce it once."""
    GradBucket(list(params)).all_reduce(group=group)
