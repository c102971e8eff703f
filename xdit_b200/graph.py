"""CUDA-graph capture of a launch-bound step.

One ``USP`` call on a small shard is a handful of short kernels and NCCL collectives: on a B200
the host (Python dispatch, buffer allocation, tensor-map encoding, collective launch) is slower
than the GPU work of a Flux-sized layer.  ``GraphedStep`` captures a whole step (for example the
attention calls of all layers of one denoising step) once and replays it, so that the host cost
is one graph launch.  Buffers allocated while capturing live in the graph's private pool and keep
their addresses, which is what lets the kernels' baked-in pointers and tensor maps stay valid.

The reference reaches for ``torch.compile`` at this point (``xfuser/model_executor/models/
runner_models/base_model.py:413-427``); streams and graphs do the same job here without a
tracing compiler.
"""
from __future__ import annotations

from typing import Callable

import torch


class GraphedStep:
    """Capture ``fn()`` (no arguments; it closes over static input tensors) and replay it."""

    def __init__(self, fn: Callable[[], object], warmup: int = 3):
        self._fn = fn
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):  # collectives and allocators must be warm before capture
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(self.graph):
            self.result = fn()

    def replay(self):
        self.graph.replay()
        return self.result

    __call__ = replay
