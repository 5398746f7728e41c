"""Block arrangements.  'pre_norm' is the reference's (runtime/src/text_model.cpp:146-168):
    x += mixer(norm(x));  x += feed_forward(norm(x))
The residual stream is float32.  A block hands the feed-forward's output on as a pending
delta, which the next norm adds in its own pass.  'post_norm' puts the norms on the parts' outputs instead."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Block, PreNormed
from .linear import Linear
from .registry import build_part, register_part


class PreNormBlock(Block):
    def __init__(self, spec, source, rt):
        self.mixer_norm = build_part("norm", spec.mixer_norm, source, rt)
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.ffn_norm = build_part("norm", spec.ffn_norm, source, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)

    def forward(self, residual, pending, ctx, cache):
        # Few tokens: a part that folds norms (folds_norms) is told which norm (one that folds into products) reads the stream
        # after it; it may then add its output to the stream in its last product's epilogue and hand
        # on that norm's half-done input (a PreNormed) instead of a delta, and the part after the norm
        # finishes the norm in its first product.  Anything else takes the norm kernel.
        fold = ops.folded_norm_enabled(residual.shape[0])
        after = getattr(ctx, "next_norm", None)            # the norm the block after this one starts with
        if self.mixer is not None:
            x = self._normed(self.mixer_norm, self.mixer, residual, pending)
            if fold and getattr(self.mixer, "folds_norms", False):
                nxt = self.ffn_norm if self.feed_forward is not None else after
                pending = self.mixer.forward(x, ctx, cache, residual=residual, next_norm=nxt if _folds(nxt) else None)
            else:
                pending = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is not None:
            x = self._normed(self.ffn_norm, self.feed_forward, residual, pending)
            if fold and getattr(self.feed_forward, "folds_norms", False):
                pending = self.feed_forward.forward(x, ctx, residual=residual, next_norm=after if _folds(after) else None)
            else:
                pending = self.feed_forward.forward(x, ctx)
        return residual, pending

    @staticmethod
    def _normed(norm, part, residual, pending):
        """The input of `part`: the PreNormed as it is when it was made for this norm and the part takes
        one, else the normed rows."""
        if isinstance(pending, PreNormed) and pending.norm is norm and getattr(part, "folds_norms", False):
            return pending
        return norm.add_norm(residual, pending)

    def first_norm(self):
        """The norm this block reads the stream with first (what the block ahead may prepare for)."""
        if self.mixer is not None:
            return self.mixer_norm
        return self.ffn_norm if self.feed_forward is not None else None


def _folds(norm) -> bool:
    """Whether a norm lets the products around it take over its passes (see parts/base.py)."""
    return norm is not None and getattr(norm, "folds_into_products", False)


class ParallelBlock(Block):
    """x += mixer(norm_a(x)) + feed_forward(norm_b(x)): both parts read the stream as it enters the block.
    When both norms are RMS norms of one eps their rows share the root mean square and come from one pass; a
    block without a second norm gives both parts the one normed input.  With per-feature factors s1, s2 of the
    parts' outputs and a multiplier m the block adds m * (s1 * mixer + s2 * feed_forward); m is folded into the
    factors when the block is built, and the sum is formed in float32."""

    def __init__(self, spec, source, rt):
        self.rt = rt
        self.mixer_norm = build_part("norm", spec.mixer_norm, source, rt)
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)
        self.ffn_norm = build_part("norm", getattr(spec, "ffn_norm", None), source, rt) if self.feed_forward is not None else None
        mult = float(getattr(spec, "residual_mult", 1.0))
        names = (getattr(spec, "mixer_scale", None), getattr(spec, "ffn_scale", None))
        self.scaled = mult != 1.0 or any(n is not None for n in names)
        self.mixer_scale = self.ffn_scale = None
        if self.scaled:
            width = self.mixer_norm.size
            s1, s2 = (source.get(n, dtype=torch.float32) if n is not None else torch.ones(width, device=rt.device, dtype=torch.float32)
                      for n in names)
            self.mixer_scale, self.ffn_scale = (s1 * mult).contiguous(), (s2 * mult).contiguous()

    def forward(self, residual, pending, ctx, cache):
        if isinstance(pending, PreNormed):
            pending = None                       # the product is in the stream already
        a, b = self.mixer_norm, self.ffn_norm
        if self.feed_forward is None:
            mixed = self.mixer.forward(a.add_norm(residual, pending), ctx, cache)
            if not self.scaled:
                return residual, mixed
            delta = torch.empty(residual.shape, device=residual.device, dtype=torch.float32)
            ops.scale_sum2(delta, mixed, self.mixer_scale)
            return residual, delta
        if b is None:
            h1 = h2 = a.add_norm(residual, pending)
        elif _folds(a) and _folds(b) and a.eps == b.eps and a.size == b.size:
            h1 = torch.empty((residual.shape[0], a.size), device=residual.device, dtype=self.rt.dtype)
            h2 = torch.empty_like(h1)
            ops.add_rmsnorm2(h1, h2, residual, pending, a.scale_weight(), b.scale_weight(), a.eps)
        else:
            h1 = a.add_norm(residual, pending)
            h2 = b.add_norm(residual, None)
        mixed = self.mixer.forward(h1, ctx, cache)
        if getattr(self.feed_forward, "takes_addend", False):
            if self.scaled:
                return residual, self.feed_forward.forward(h2, ctx, add=mixed, add_scale=self.mixer_scale, scale=self.ffn_scale)
            return residual, self.feed_forward.forward(h2, ctx, add=mixed)
        fed = self.feed_forward.forward(h2, ctx)
        delta = torch.empty(residual.shape, device=residual.device, dtype=torch.float32)
        if self.scaled:
            ops.scale_sum2(delta, mixed, self.mixer_scale, fed, self.ffn_scale)
        else:
            ops.sum2(delta, mixed, fed)
        return residual, delta

    def first_norm(self):
        return None                              # two norms read the stream: nothing for the block ahead to prepare


class GatedPreNormBlock(Block):
    """x += mixer(h) * sigmoid(W1 h + b1), h = norm_a(x);  x += feed_forward(h) * sigmoid(W2 h + b2), h = norm_b(x): the
    pre-norm block with a gate on each part's result, computed from the part's own input.  The gates' pre-activations leave
    their products in float32; sigmoid, the multiplication and the residual sum are float32.  A mixer that shares its input
    product (parts/shared_io.py) takes the gate's rows into it."""

    def __init__(self, spec, source, rt):
        self.rt = rt
        self.mixer_norm = build_part("norm", spec.mixer_norm, source, rt)
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)
        self.ffn_norm = build_part("norm", spec.ffn_norm, source, rt) if self.feed_forward is not None else None
        self.mixer_gate = self.ffn_gate = None
        self.mixer_gate_bias = self.ffn_gate_bias = None
        self.gate_in_mixer = False
        name = getattr(spec, "mixer_gate", None)
        if self.mixer is not None and name is not None:
            self.mixer_gate_bias = source.get(name + ".b", dtype=torch.float32)
            if hasattr(self.mixer, "take_extra_rows") and getattr(self.mixer, "shared", True):
                self.mixer.take_extra_rows(source.get(name))
                self.gate_in_mixer = True
            else:
                self.mixer_gate = Linear(source.get(name))
        name = getattr(spec, "ffn_gate", None)
        if self.feed_forward is not None and name is not None:
            self.ffn_gate = Linear(source.get(name))
            self.ffn_gate_bias = source.get(name + ".b", dtype=torch.float32)

    def forward(self, residual, pending, ctx, cache):
        if isinstance(pending, PreNormed):
            pending = None                       # the product is in the stream already
        if self.mixer is not None:
            h = self.mixer_norm.add_norm(residual, pending)
            y = self.mixer.forward(h, ctx, cache)
            if self.gate_in_mixer:
                pending = self._gated(y, self.mixer.extra_out, self.mixer_gate_bias)
            elif self.mixer_gate is not None:
                pending = self._gated(y, self.mixer_gate(h, out_dtype=torch.float32), self.mixer_gate_bias)
            else:
                pending = y
        if self.feed_forward is not None:
            h = self.ffn_norm.add_norm(residual, pending)
            y = self.feed_forward.forward(h, ctx)
            pending = self._gated(y, self.ffn_gate(h, out_dtype=torch.float32), self.ffn_gate_bias) if self.ffn_gate is not None else y
        return residual, pending

    @staticmethod
    def _gated(y, pre, bias):
        out = torch.empty(y.shape, device=y.device, dtype=torch.float32)
        ops.sigmoid_gate(out, y, pre, bias)
        return out

    def first_norm(self):
        return None                              # its norms do not fold into products


class PostNormBlock(Block):
    """x += norm_a(mixer(x));  x += norm_b(feed_forward(x)): the parts read the stream itself and the norms sit on their
    outputs, so the stream is always whole (nothing is pending behind this block).  A norm here offers
    add_normed(residual, y, cast): the float32 stream takes the normed output and, where a product reads the stream next,
    leaves in the compute type in the same pass.  A mixer that declares takes_stream reads the float32 stream (its own
    first pass turns it into the compute type); any other part reads the stream's copy in the compute type."""

    def __init__(self, spec, source, rt):
        self.rt = rt
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.mixer_norm = build_part("norm", spec.mixer_norm, source, rt) if self.mixer is not None else None
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)
        self.ffn_norm = build_part("norm", spec.ffn_norm, source, rt) if self.feed_forward is not None else None
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "add_normed"):
                raise ValueError("a post-norm block needs norms that can be added to the stream (add_normed)")

    def _compute_copy(self, residual):
        if self.rt.dtype == torch.float32:
            return residual
        x = torch.empty(residual.shape, device=residual.device, dtype=self.rt.dtype)
        ops.cast_rows(x, residual)
        return x

    def forward(self, residual, pending, ctx, cache):
        if pending is not None and not isinstance(pending, PreNormed):       # left by a block of another kind
            ops.sum2(residual, residual, pending.contiguous())
        x = None                                    # the stream in the compute type, where a pass already left it
        if self.mixer is not None:
            h = residual if getattr(self.mixer, "takes_stream", False) else self._compute_copy(residual)
            y = self.mixer.forward(h, ctx, cache)
            if self.feed_forward is not None and self.rt.dtype != torch.float32:
                x = torch.empty(residual.shape, device=residual.device, dtype=self.rt.dtype)
            self.mixer_norm.add_normed(residual, y, cast=x)
        if self.feed_forward is not None:
            y = self.feed_forward.forward(x if x is not None else self._compute_copy(residual), ctx)
            self.ffn_norm.add_normed(residual, y)
        return residual, None

    def first_norm(self):
        return None                              # no norm reads the stream


register_part("block", "pre_norm", PreNormBlock)
register_part("block", "post_norm", PostNormBlock)
register_part("block", "gated_pre_norm", GatedPreNormBlock)
register_part("block", "parallel", ParallelBlock)
