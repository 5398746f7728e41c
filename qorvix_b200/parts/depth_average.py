"""The stream after each run as a weighted sum of the embedding's output and all runs' results so far.  The results
are kept for the step in one float32 stack [runs + 1, tokens, width]; one kernel stores the run's result (stream +
pending delta, summed in float32) and forms the weighted sum in place of the stream."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import PreNormed
from .registry import register_part


class DepthAverage:
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.weights = [source.get(name, dtype=torch.float32) for name in spec.weights]

    def begin(self, residual):
        """The stack of a step, with the embedding's output in its first place."""
        stack = torch.empty((len(self.weights) + 1, *residual.shape), device=residual.device, dtype=torch.float32)
        ops.cast_rows(stack[0], residual)
        return stack

    def after(self, run: int, residual, pending, stack):
        """The stream that run + 1 reads (in place of `residual`; nothing is pending after it)."""
        if isinstance(pending, PreNormed):
            pending = None                  # the product is in the stream already
        if pending is not None and pending.dtype != torch.float32:
            delta = torch.empty(residual.shape, device=residual.device, dtype=torch.float32)
            ops.cast_rows(delta, pending)
            pending = delta
        ops.depth_mix(residual, pending, stack, self.weights[run], run + 2)
        return residual


register_part("stream", "depth_average", DepthAverage)
