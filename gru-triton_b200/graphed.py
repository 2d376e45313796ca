"""CUDA-graph capture of a whole step (forward, loss, backward) of a layer.

A train step at the small shapes of this path (T=64, B=32) is a few dozen kernels of a few
microseconds each, so the Python and launch overhead of issuing them one by one is as long as the
GPU work.  ``GraphedStep`` runs the step a few times to warm every lazy initialisation, captures
it once into a CUDA graph on static input buffers, and afterwards replays it with one launch.
Everything the library enqueues goes to the current stream and nothing in it allocates or
synchronises, so its kernels are capturable as they are; the frozen quantiser scales are read on
the host (``.item()``) when the layer is built, outside the capture.

The reference has no counterpart (its ``compile_step`` option wraps the per-step cell in
``torch.compile``, src/gru_qat/gru_layer.py:126-151).
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    """``step = GraphedStep(fn, example_inputs)``; ``result = step(*inputs)``.

    ``fn(*inputs)`` must be a pure function of its tensor arguments and of module state that does
    not change shape (parameters may change value: they are read at replay time), must not
    synchronise with the host, and returns a tensor or a tuple of tensors.  Gradients produced
    inside ``fn`` (``backward()``) land in ``.grad`` tensors that keep their addresses across
    replays when ``fn`` resets them with ``set_to_none=True`` inside the step.
    """

    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3):
        self.static_inputs = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                fn(*self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_outputs = fn(*self.static_inputs)

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_outputs
