"""Norm without statistics: out = tanh(alpha x) * w + b with one scalar alpha per norm; no mean, no variance, so a row's
result needs no pass over the row first.  The residual sum that precedes it is fused in, in float32, as for the RMS norm."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, PreNormed
from .registry import register_part


class TanhNorm(Norm):
    folds_into_products = False        # not a scaling of the row: nothing for the products around it to take over

    def __init__(self, spec, source, rt):
        self.size = int(spec.size)
        self.weight = source.get(spec.weight, dtype=torch.float32)
        self.bias = source.get(spec.bias, dtype=torch.float32)
        self.alpha = float(source.get(spec.alpha, dtype=torch.float32).reshape(-1)[0].item())
        self.rt = rt

    def add_norm(self, residual, delta, rows=None):
        if isinstance(delta, PreNormed):
            delta = None                    # the product is in the stream already
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), device=residual.device, dtype=self.rt.dtype)
        ops.add_tanhnorm(out, residual, delta, self.weight, self.bias, self.alpha, row_idx=rows)
        return out


register_part("norm", "tanh_norm", TanhNorm)
