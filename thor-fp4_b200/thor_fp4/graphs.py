"""CUDA-graph capture of FP4 modules (API of src/thor_fp4/graphs.py:19-50 in the
reference project).  The engine resolves its per-shape plans (tensor maps, tile
width, buffers) on the first eager call and allocates nothing afterwards, so a
warmed function captures and replays as one launch.
"""
from __future__ import annotations

import torch

__all__ = ["Graphed", "capture_module"]


class Graphed:
    """Capture fn(*inputs) with static input / output buffers.

    Calls copy the new inputs into the static buffers, replay the graph and return
    the static output (valid until the next call)."""

    def __init__(self, fn, *example_inputs, warmup: int = 3, pool=None):
        self.fn = fn
        self.static_in = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                out = fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.static_out = out
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool):
            self.static_out = fn(*self.static_in)

    def __call__(self, *inputs):
        for s, t in zip(self.static_in, inputs):
            s.copy_(t)
        self.graph.replay()
        return self.static_out


def capture_module(model: torch.nn.Module, *example_inputs, warmup: int = 3) -> Graphed:
    return Graphed(lambda *xs: model(*xs), *example_inputs, warmup=warmup)
