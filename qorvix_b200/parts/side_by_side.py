"""Two mixers that read the same input, their results added with a factor each.  Each keeps a cache or state of its
own (the pair's cache_spec() is the tuple of the two, its cache a view with one entry per part).  Parts that can share
their projections (parts/shared_io.py) share them: the rows both want of the input become one product, each part writes
its activations, times its factor, into its columns of one buffer, and the two output matrices side by side are one
product over that buffer.  Other parts run whole and their outputs are summed in float32."""
from __future__ import annotations

import torch

from ..csrc import ops
from .registry import build_part, register_part
from .shared_io import SharedIOMixer, stack_rows


class SideBySide(SharedIOMixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.left = build_part("mixer", spec.left, source, rt)
        self.right = build_part("mixer", spec.right, source, rt)
        self.scales = (float(spec.left_scale), float(spec.right_scale))
        self.shared = isinstance(self.left, SharedIOMixer) and isinstance(self.right, SharedIOMixer)
        if self.shared:
            self.in_rows = self.left.in_rows + self.right.in_rows
            self.out_cols = self.left.out_cols + self.right.out_cols

    def cache_spec(self):
        return (self.left.cache_spec(), self.right.cache_spec())

    def reads_cache_of(self):
        if self.left.reads_cache_of() is not None or self.right.reads_cache_of() is not None:
            raise ValueError("a mixer that stands beside another keeps its own cache")
        return None

    # ------------------------------------------------------------------ shared projections
    def in_weights(self):
        return stack_rows([self.left.in_weights(), self.right.in_weights()])

    def out_weight(self):
        wl, wr = self.left.out_weight(), self.right.out_weight()
        dt = torch.float32 if torch.float32 in (wl.dtype, wr.dtype) else wl.dtype
        return torch.cat([wl.to(dt), wr.to(dt)], dim=1)

    def out_bias(self):
        total = None
        for part, s in zip((self.left, self.right), self.scales):
            b = part.out_bias()
            if b is not None:
                total = b.float() * s if total is None else total + b.float() * s
        return total

    def release_weights(self):
        self.left.release_weights()
        self.right.release_weights()

    def heads_out(self, proj, ctx, cache, out, factor=1.0):
        a, c = self.left.in_rows, self.left.out_cols
        self.left.heads_out(proj[:, :a], ctx, cache.views[0], out[:, :c], factor * self.scales[0])
        self.right.heads_out(proj[:, a:], ctx, cache.views[1], out[:, c:], factor * self.scales[1])

    def forward(self, x, ctx, cache):
        if self.shared:
            return super().forward(x, ctx, cache)
        yl = self.left.forward(x, ctx, cache.views[0])
        yr = self.right.forward(x, ctx, cache.views[1])
        out = torch.empty(yl.shape, device=yl.device, dtype=torch.float32)
        d = yl.shape[1]
        sl, sr = (torch.full((d,), s, device=yl.device, dtype=torch.float32) for s in self.scales)
        ops.scale_sum2(out, yl.contiguous(), sl, yr.contiguous(), sr)
        return out


register_part("mixer", "side_by_side", SideBySide)
