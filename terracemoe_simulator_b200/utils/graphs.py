"""CUDA-graph capture of launch-bound forward passes.

A MoE layer at serving batch sizes (a few hundred tokens) is a chain of ~15 short kernels whose
launch latency exceeds their run time.  ``GraphedForward`` warms the callable up on a side stream
(first-call set-up such as kernel attributes and the context binding for tensor-map encoding
happens there), captures one call under ``torch.no_grad()`` into a ``torch.cuda.CUDAGraph`` with
static input and output buffers, and replays it for every later call: one launch per forward.

Every kernel of this package launches on the current stream, allocates through the caching
allocator only and never synchronises with the host, which is what makes the capture legal; the
tile schedules of the grouped GEMMs are derived on the device from the routing result, so one
captured graph serves any routing.  Shapes are fixed at capture; a different token count needs
its own ``GraphedForward``.  The reference has no counterpart (it has no launch-bound path).
"""
from __future__ import annotations

import torch


class GraphedForward:
    def __init__(self, fn, example: torch.Tensor, warmup: int = 3):
        if not example.is_cuda:
            raise ValueError("CUDA graphs need a CUDA tensor")
        self.fn = fn
        self.x = example.detach().clone()
        side = torch.cuda.Stream(example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):
                fn(self.x)
        torch.cuda.current_stream(example.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.y = fn(self.x)
        self.replays = 0

    def __call__(self, x: torch.Tensor):
        if x.shape != self.x.shape or x.dtype != self.x.dtype:
            raise ValueError(f"captured for {tuple(self.x.shape)} {self.x.dtype}, "
                             f"got {tuple(x.shape)} {x.dtype}")
        self.x.copy_(x)
        self.graph.replay()
        self.replays += 1
        return self.y
