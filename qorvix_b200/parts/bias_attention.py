"""Softmax attention over the paged cache whose positions enter through a learned bias per (distance bucket, head) on
the scores and a temperature on the queries; no rotation.  q, k, v and the output gate come from one product with float32
sums; one kernel adds the biases, scales q by its position's temperature and writes k and v into the token's cache row
(all keys, then all values, so the value size need not be the key size); attention reads keys and values from the pages
only, so a prompt portion and a single decoded token take the same path."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..cache.spec import PagedRowsSpec
from ..csrc import ops
from .registry import register_part
from .shared_io import SharedIOMixer, stack_rows


def distance_buckets(rows: int, far: float, positions: int) -> np.ndarray:
    """bucket[n] for distances n = 0 .. min(positions - 1, ceil(far)): one row per distance below half the rows, the other
    rows spaced evenly in the logarithm of the distance up to `far`; from `far` on every distance has the last row, so
    the table ends there.  Computed in float32, as positions are."""
    half = rows // 2
    last = max(0, min(int(positions) - 1, int(math.ceil(far))))
    n = np.arange(last + 1, dtype=np.int64)
    out = n.copy()
    big = n >= half
    if big.any():
        if half <= 0 or not far > half:
            raise ValueError(f"a distance bias of {rows} rows needs bias_max above {half}")
        ratio = np.log(n[big].astype(np.float32) / np.float32(half)) / np.float32(math.log(far / half)) * np.float32(rows - half)
        out[big] = np.minimum(rows - 1, half + np.floor(ratio.astype(np.float32)).astype(np.int64))
    return out.astype(np.int32)


class BiasedAttention(SharedIOMixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.G, self.n, self.dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        if self.H % self.G:
            raise ValueError(f"num_heads {self.H} is not a multiple of num_kv_heads {self.G}")
        self._w_in = stack_rows([source.get(n) for n in (spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj)])
        self._w_out = source.get(spec.o_proj)
        self._b_out = source.get(spec.o_proj + ".b", dtype=torch.float32)
        self.bq, self.bk, self.bv = (source.get(n + ".b", dtype=torch.float32) for n in (spec.q_proj, spec.k_proj, spec.v_proj))
        self.in_rows = self.H * self.n + self.G * (self.n + self.dv) + self.H * self.dv
        self.out_cols = self.H * self.dv
        self.rel = source.get(spec.rel_bias, dtype=torch.float32)                                  # [rows, heads]
        self.bucket = torch.from_numpy(distance_buckets(spec.bias_rows, spec.bias_max, rt.max_positions)).to(rt.device)
        # the tensor-core kernel reads the bias per (head, distance)
        self.table = ops.bias_attention_table(self.bucket, self.rel) if rt.dtype == torch.bfloat16 else None

    def cache_spec(self):
        return PagedRowsSpec(self.G * (self.n + self.dv), 0)

    def in_weights(self):
        return self._w_in

    def out_weight(self):
        return self._w_out

    def out_bias(self):
        return self._b_out

    def release_weights(self):
        self._w_in = self._w_out = None

    def heads_out(self, proj, ctx, cache, out, factor=1.0):
        s, H, G, n, dv = self.spec, self.H, self.G, self.n, self.dv
        T = proj.shape[0]
        bt = ctx.block_tables[cache.group]
        q = torch.empty((T, H * n), device=proj.device, dtype=self.rt.dtype)
        k_off, v_off, g_off = H * n, H * n + G * n, H * n + G * (n + dv)
        ops.bias_attn_prepare(q, proj, 0, k_off, v_off, self.bq, self.bk, self.bv, cache.tensor, ctx, bt, H, G, n, dv, cache.page_size,
                              s.temp_coef, s.temp_every)
        ops.bias_attention(out, q, cache.tensor, ctx, bt, H, G, n, dv, cache.page_size, s.scale, self.bucket, self.rel,
                           proj[:, g_off: g_off + H * dv], factor, table_of_distances=self.table)


register_part("mixer", "biased_attention", BiasedAttention)
