"""Attention over a cached low-rank latent.  Per token only the normed latent c (kv_rank entries) and one
rotated key part shared by all heads are kept, in pages; a head's unrotated keys and its values are
W_uk c and W_uv c.  The kernels never expand them: the query is carried into the latent space
(W_uk^T q), attention runs over the cache rows as they are, and W_uv is applied to the weighted latent
(csrc/latent_attention.cu).  Query, down projection and gate come from one fused product; a model whose queries pass a
normed latent of their own has that latent's down matrix in the fused product and one more product behind the norm, and
the gate may be absent."""
from __future__ import annotations

import torch

from ..cache.spec import PagedRowsSpec
from ..csrc import ops
from .base import Mixer
from .linear import Linear
from .registry import build_part, register_part


class LatentAttention(Mixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dn, self.dr, self.dv, self.rank = spec.num_heads, spec.head_dim, spec.rot_dim, spec.value_dim, spec.kv_rank
        # with a query latent (q_down, q_norm) q_proj is [H * (dn + dr), q_rank] and reads the normed latent; its down matrix
        # rides in the fused product instead of q_proj
        self.q_rank = int(getattr(spec, "q_rank", 0) or 0)
        gate_name = getattr(spec, "gate_proj", None)
        first = source.get(spec.q_down) if self.q_rank else source.get(spec.q_proj)
        mats = [first, source.get(spec.kv_down)] + ([source.get(gate_name)] if gate_name is not None else [])
        dt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.q_off, self.kv_off = 0, mats[0].shape[0]
        self.gate_off = self.kv_off + mats[1].shape[0] if gate_name is not None else None
        rows = sum(m.shape[0] for m in mats)
        if dt == torch.bfloat16 and rows % 8:
            # rows of zeros behind the last matrix: every token's row of the fused product then starts on 16 bytes,
            # which the tensor-core kernels that read q and the gate out of it ask for
            mats.append(torch.zeros((-rows) % 8, mats[0].shape[1], device=mats[0].device, dtype=dt))
        self.proj = Linear(torch.cat([m.to(dt) for m in mats], dim=0))
        del mats, first
        if self.q_rank:
            self.q_norm = source.get(spec.q_norm, dtype=torch.float32)
            self.q_up = Linear(source.get(spec.q_proj))
        self.kv_norm = source.get(spec.kv_norm, dtype=torch.float32)
        self.k_up = source.get(spec.k_up)
        self.v_up = source.get(spec.v_up).to(self.k_up.dtype)
        # the tensor-core kernels read each head's key matrix with the latent index outermost
        self.k_up_t = (self.k_up.view(self.H, self.dn, self.rank).transpose(1, 2).contiguous()
                       if self.k_up.dtype == torch.bfloat16 else None)
        self.o_proj = Linear(source.get(spec.o_proj))
        self.position = build_part("position", spec.position, source, rt)
        pairing = getattr(spec.position, "pairing", "")
        if pairing not in ("interleaved", "split_half") or self.position.table() is None:
            raise ValueError("latent attention rotates pairs of entries from a cos/sin table: its position must be a rotary "
                             "encoding with pairing 'interleaved' or 'split_half'")
        self.split_half = pairing == "split_half"
        self.rot = self.position.table().shape[1] * 2
        self.window, self.scale, self.eps = int(spec.window), float(spec.scale), float(spec.eps)

    def cache_spec(self):
        return PagedRowsSpec(self.rank + self.dr, self.window)

    def forward(self, x, ctx, cache):
        H, dn, dr, dv, rank = self.H, self.dn, self.dr, self.dv, self.rank
        bt = ctx.block_tables[cache.group]
        proj = self.proj(x, out_dtype=self.rt.dtype)
        if self.q_rank:
            cq = torch.empty((proj.shape[0], self.q_rank), device=proj.device, dtype=self.rt.dtype)
            ops.rmsnorm_rows(cq, proj[:, : self.q_rank], self.q_norm, self.eps)
            q = self.q_up(cq, out_dtype=self.rt.dtype)
        else:
            q = proj[:, : self.kv_off]
        ops.latent_prepare(proj, q, self.kv_off, cache.tensor, self.kv_norm, self.eps, self.position.table(), ctx, bt,
                           H, dn, dr, rank, self.rot, cache.page_size, split_half=self.split_half)
        gate = proj[:, self.gate_off: self.gate_off + H * dv] if self.gate_off is not None else None
        out = torch.empty((proj.shape[0], H * dv), device=proj.device, dtype=self.rt.dtype)
        ops.latent_attention(out, q, gate, cache.tensor, self.k_up, self.v_up, ctx, bt,
                             H, dn, dr, dv, rank, cache.page_size, self.window, self.scale, wuk_t=self.k_up_t)
        return self.o_proj(out, out_dtype=self.rt.dtype)


register_part("mixer", "latent_attention", LatentAttention)
