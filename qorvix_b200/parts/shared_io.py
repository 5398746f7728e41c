"""Mixers whose input and output projections can be shared with their neighbours.

Such a mixer states the rows it wants of ONE product with its input (`in_weights()`), turns its slice of that product's
float32 result into the activations ahead of its output projection (`heads_out(proj, ctx, cache, out, factor)`, written in
the compute type into `out`, which may be a column slice of a wider buffer, times `factor`), and names its output matrix
(`out_weight()`, and `out_bias()` or None).  Alone, the mixer runs exactly these pieces with products of its own
(`SharedIOMixer.forward`).  Beside another mixer (parts/side_by_side.py) the two inputs' rows become one product and the two
output matrices one product over the concatenated activations.  A block may also hand it further rows that read the same
input (`take_extra_rows`), whose float32 result it leaves in `extra_out` after every forward: the gate of the block's
residual, for instance.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer
from .linear import Linear


def stack_rows(mats):
    """Matrices that read the same input, one below the other (float32 if any of them is stored in float32)."""
    dt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
    return torch.cat([m.to(dt) for m in mats], dim=0)


class SharedIOMixer(Mixer):
    in_rows: int = 0              # rows of in_weights()
    out_cols: int = 0             # columns of out_weight()

    def in_weights(self) -> torch.Tensor:
        raise NotImplementedError

    def heads_out(self, proj, ctx, cache, out, factor: float = 1.0) -> None:
        raise NotImplementedError

    def out_weight(self) -> torch.Tensor:
        raise NotImplementedError

    def out_bias(self):
        return None

    # ------------------------------------------------------------------ running alone
    _in = _out = _bias = _extra = None
    extra_out = None

    def take_extra_rows(self, weight: torch.Tensor) -> None:
        """Further rows [n, hidden] for the input product; their float32 result is `extra_out` after forward()."""
        if self._in is not None:
            raise RuntimeError("extra rows must be handed over before the first step")
        self._extra = weight

    def _build(self):
        mats = [self.in_weights()] + ([self._extra] if self._extra is not None else [])
        self._in = Linear(stack_rows(mats))
        self._out = Linear(self.out_weight())
        b = self.out_bias()
        self._bias = b.float().contiguous() if b is not None else None
        self.release_weights()

    def release_weights(self) -> None:
        """Called once the products hold copies of the matrices: drop what in_weights() / out_weight() kept."""

    def forward(self, x, ctx, cache):
        if self._in is None:
            self._build()
        proj = self._in(x, out_dtype=torch.float32)
        self.extra_out = proj[:, self.in_rows:] if self._extra is not None else None
        heads = torch.empty((x.shape[0], self.out_cols), device=x.device, dtype=x.dtype)
        self.heads_out(proj[:, : self.in_rows], ctx, cache, heads, 1.0)
        y = self._out(heads, out_dtype=torch.float32)
        if self._bias is not None:
            ops.add_vector(y, self._bias)
        return y
