"""Embeddings that are more than one table.  A plain table needs no part (the model gathers its rows);
an embedding part has `forward(out, ctx, cache)` filling the float32 residual stream and may keep a
small state per request (`cache_spec()`), which the cache manager zeroes at admission."""
from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec
from ..csrc import ops
from .registry import register_part


class BigramEmbedding:
    """Token row plus the row of a hashed (previous token, token) pair.  The previous token of a
    segment's first token is the request's state: one int32 per request slot."""

    def __init__(self, spec, source, rt):
        self.spec = spec
        self.table = source.get(spec.table)
        self.pair = source.get(spec.pair_table)
        if self.pair.dtype != self.table.dtype:
            self.pair = self.pair.to(self.table.dtype)

    @property
    def weight(self) -> torch.Tensor:
        return self.table

    def cache_spec(self):
        return FixedStateSpec((1,), "int32")

    def forward(self, out, ctx, cache) -> None:
        s = self.spec
        ops.embed_pair(out, self.table, self.pair, ctx.token_ids, ctx, cache.tensor.reshape(-1), s.buckets, s.mul_prev, s.mul_cur)


class PositionedEmbedding:
    """Token row plus the row of a learned position table, the sum (float32) optionally through a tanh norm; one kernel.
    It keeps no state: the position of a token is the step's."""

    def __init__(self, spec, source, rt):
        self.spec = spec
        self.table = source.get(spec.table)
        self.pos = source.get(spec.pos_table)
        if self.pos.dtype != self.table.dtype:
            self.pos = self.pos.to(self.table.dtype)
        self.norm_w = self.norm_b = None
        self.alpha = 1.0
        if spec.norm is not None:
            self.norm_w = source.get(spec.norm.weight, dtype=torch.float32)
            self.norm_b = source.get(spec.norm.bias, dtype=torch.float32)
            self.alpha = float(source.get(spec.norm.alpha, dtype=torch.float32).reshape(-1)[0].item())

    @property
    def weight(self) -> torch.Tensor:
        return self.table

    def cache_spec(self):
        return None

    def forward(self, out, ctx, cache) -> None:
        ops.embed_pos(out, self.table, self.pos, ctx.token_ids, ctx.tok_pos, self.spec.pos_scale, self.norm_w, self.norm_b, self.alpha)


register_part("embedding", "bigram_embedding", BigramEmbedding)
register_part("embedding", "positioned_embedding", PositionedEmbedding)
