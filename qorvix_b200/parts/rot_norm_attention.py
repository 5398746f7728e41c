"""Causal grouped-query attention whose queries and keys are rotated and then unit-normed, with a temperature per head
and values that layers may share.  q, k and v are one fused product with float32 sums; `rot_norm_prepare` rotates, norms
and scales in float32, blends the values with the sharing layer's where asked, writes q in the compute type and k and v
into the token's cache row [keys of all key/value heads | their values]; attention itself is the kernel family that reads
such rows (csrc/bias_attention.cu), run without a bias table.  Key and value sizes are unrelated."""
from __future__ import annotations

import torch

from ..cache.spec import PagedRowsSpec
from ..csrc import ops
from .base import Mixer
from .linear import Linear
from .registry import build_part, register_part
from .shared_io import stack_rows


class RotNormAttention(Mixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.G, self.n, self.dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim
        if self.H % self.G:
            raise ValueError(f"num_heads {self.H} is not a multiple of num_kv_heads {self.G}")
        self.qkv = Linear(stack_rows([source.get(spec.q_proj), source.get(spec.k_proj), source.get(spec.v_proj)]))
        self.o_proj = Linear(source.get(spec.o_proj))
        self.position = build_part("position", spec.position, source, rt)
        self.table = self.position.table() if self.position is not None else None
        if self.position is not None and (self.table is None or getattr(spec.position, "pairing", "split_half") != "split_half"):
            raise ValueError("this attention rotates split halves from a cos/sin table: its position must be a rotary encoding "
                             "with pairing='split_half'")
        self.rot = self.table.shape[1] * 2 if self.table is not None else 0
        self.temp = source.get(spec.head_temp, dtype=torch.float32).contiguous() if spec.head_temp is not None else None
        self.role = spec.v_share_role
        if self.role not in (None, "source", "blend"):
            raise ValueError(f"unknown role '{self.role}' in value sharing (known: source, blend)")
        if self.role is not None and not spec.v_share:
            raise ValueError("a layer that shares values names what it shares (v_share)")
        self.lam = float(source.get(spec.v_blend, dtype=torch.float32).item()) if self.role == "blend" else 0.0
        # the tensor-core kernel reads a bias per head and distance: one column of zeros serves every distance
        self.no_bias = torch.zeros((self.H, 1), device=rt.device, dtype=torch.float32) if rt.dtype == torch.bfloat16 else None
        self.scale, self.eps = float(spec.scale), float(spec.eps)

    def cache_spec(self):
        return PagedRowsSpec(self.G * (self.n + self.dv), 0)

    def forward(self, x, ctx, cache):
        H, G, n, dv = self.H, self.G, self.n, self.dv
        bt = ctx.block_tables[cache.group]
        proj = self.qkv(x, out_dtype=torch.float32)
        k_off, v_off = H * n, (H + G) * n
        v_other = None
        if self.role == "source":
            ctx.shared[self.spec.v_share] = proj[:, v_off: v_off + G * dv]
        elif self.role == "blend":
            v_other = ctx.shared.get(self.spec.v_share)
            if v_other is None or tuple(v_other.shape) != (proj.shape[0], G * dv):
                raise ValueError(f"no layer ahead of this one has left values of {G} x {dv} under '{self.spec.v_share}'")
        q = torch.empty((proj.shape[0], H * n), device=proj.device, dtype=self.rt.dtype)
        ops.rot_norm_prepare(q, proj, 0, k_off, v_off, cache.tensor, self.table, self.rot, True, self.eps, self.temp, v_other, self.lam,
                             ctx, bt, H, G, n, dv, cache.page_size)
        out = torch.empty((proj.shape[0], H * dv), device=proj.device, dtype=self.rt.dtype)
        ops.bias_attention(out, q, cache.tensor, ctx, bt, H, G, n, dv, cache.page_size, self.scale, None, None, None, 1.0,
                           table_of_distances=self.no_bias)
        return self.o_proj(out, out_dtype=self.rt.dtype)


register_part("mixer", "rot_norm_attention", RotNormAttention)
