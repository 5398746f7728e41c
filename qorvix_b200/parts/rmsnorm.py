"""RMSNorm: out = (x * 1/sqrt(mean(x^2) + eps)) * w, no bias (reference: runtime/src/ops.cpp:8-13); a spec
with `one_plus` stores its weight around zero and the rows are scaled by 1 + w (formed once, in float32); a spec with
`scalar` stores one number for all coordinates.  The residual sum that precedes it is fused in: the
residual stream is float32 and the delta is added in float32 in the same pass."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, PreNormed
from .registry import register_part


class RMSNorm(Norm):
    def __init__(self, spec, source, rt):
        self.eps = float(spec.eps)
        self.size = int(spec.size)
        self.weight = source.get(spec.weight, dtype=torch.float32)   # tiny; always read as float32
        if getattr(spec, "scalar", False):                           # one number for all coordinates
            self.weight = self.weight.reshape(1).expand(self.size).contiguous()
        if getattr(spec, "one_plus", False):
            self.weight = (self.weight.double() + 1.0).float()       # exact: a bfloat16 value plus one fits float32's 24 bits or rounds once
        self.rt = rt

    folds_into_products = True         # x * rsqrt(mean(x^2) + eps) * weight

    def scale_weight(self):
        return self.weight

    def add_norm(self, residual, delta, rows=None):
        """residual[T,d] float32 (+= delta in place when rows is None).  rows: int32 row
        indices; then only those rows are normed and the residual is left as it is."""
        if isinstance(delta, PreNormed):
            delta = None                    # the product is in the stream already
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), device=residual.device, dtype=self.rt.dtype)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, row_idx=rows)
        return out


    def add_normed(self, residual, y, cast=None):
        """residual (float32) += rmsnorm(y) * weight: the norm on a sublayer's output (post-norm blocks).  `cast`, if
        given, receives the new stream in the compute type."""
        ops.post_rmsnorm_add(residual, y, self.weight, self.eps, cast=cast)


register_part("norm", "rmsnorm", RMSNorm)
