"""A decoder assembled from a ModelSpec: embedding, blocks in the spec's order, final norm,
output head.  It knows nothing of any one architecture; the counterpart of the
reference's TextModel::forwardFromState (runtime/src/text_model.cpp:133-176) for a batch of
tokens from several requests.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from ..parts.base import Runtime
from ..parts.linear import Linear
from ..parts.registry import build_part


class TextModel:
    def __init__(self, spec, source, rt: Runtime):
        self.spec = spec
        self.rt = rt
        source.check(spec.expected_shapes(), optional=spec.optional_tensors, ignored=getattr(spec, "ignored_tensors", ()))
        if isinstance(spec.embedding, str):
            self.embedder = None
            self.embedding = source.get(spec.embedding)
        else:                                      # an embedding part (more than one table, state of its own)
            self.embedder = build_part("embedding", spec.embedding, source, rt)
            self.embedding = self.embedder.weight
        self.blocks = [build_part("block", _BlockView(layer), source, rt) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, source, rt)
        self.lm_head = Linear(source.get(spec.lm_head)) if spec.lm_head is not None else Linear(self.embedding)
        self.order: List[int] = list(spec.order)
        # a stretch of layers that runs again: where the stream re-enters it (None: no such stretch)
        self.loop = build_part("stream", getattr(spec, "loop", None), source, rt)
        # the stream after each run as a weighted sum of all runs' results (None: the run's result as it is)
        self.depth = build_part("stream", getattr(spec, "depth_average", None), source, rt)
        self._more_views = {}          # run -> the indices of the further caches of a mixer that keeps several
        self.stream_tap = None         # callable(run, residual, pending) after every run: for tests and debugging
        self._native = None            # the native executor of this model over a cache, made on first use (False: not applicable)

    def cache_needs(self):
        """What each RUN of the execution order wants of the cache manager: (cache spec or None, index
        of the run whose cache it reads or None).  A layer that the order names twice keeps a cache per
        run: in a later step its first run must find the keys its first run wrote, not its second's.
        A mixer that reads another layer's cache reads that layer's latest run before its own."""
        needs = []
        more = []                                  # (run, further specs) of mixers that keep several caches
        last_run_of = {}
        for run, li in enumerate(self.order):
            m = getattr(self.blocks[li], "mixer", None)
            spec = m.cache_spec() if m is not None else None
            if isinstance(spec, (tuple, list)):    # a mixer of several parts: the first is the run's own entry
                more.append((run, list(spec[1:])))
                spec = spec[0]
            src = m.reads_cache_of() if m is not None else None
            src_run = None
            if src is not None:
                if src not in last_run_of:
                    raise ValueError(f"layer {li} reads the cache of layer {src}, which has not run before it")
                src_run = last_run_of[src]
            needs.append((spec, src_run))
            last_run_of[li] = run
        if self.embedder is not None or more:      # the embedding's own state comes after the runs
            needs.append((self.embedder.cache_spec() if self.embedder is not None else None, None))
        self._more_views = {}
        for run, specs in more:                    # then the further caches, which the run's view lists
            self._more_views[run] = list(range(len(needs), len(needs) + len(specs)))
            needs.extend((sp, None) for sp in specs)
        return needs

    def _view(self, cache, run: int):
        """What run `run` sees of the cache: its layer's view, or one view per part of a mixer that keeps several."""
        view = cache.layer_view(run)
        extra = self._more_views.get(run)
        if not extra:
            return view
        from ..cache.manager import CompositeCacheView
        return CompositeCacheView(views=[view] + [cache.layer_view(i) for i in extra])

    def forward(self, ctx, cache) -> Optional[torch.Tensor]:
        """Runs the tokens of `ctx`; returns float32 logits [wanted rows, vocab] (None if none wanted)."""
        T = ctx.num_tokens
        if self._native is None:
            from ..engine.native_executor import NativeExecutor
            self._native = NativeExecutor.try_build(self, cache) or False
        if self._native:
            # every block is one the native executor knows: the whole step in one call
            return self._native.forward(ctx)
        residual = torch.empty((T, self.spec.hidden_size), device=self.rt.device, dtype=torch.float32)
        if self.embedder is not None:
            self.embedder.forward(residual, ctx, cache.layer_view(len(self.order)))
        else:
            ops.embed(residual, self.embedding, ctx.token_ids)
        pending = None
        x0 = None
        if self.loop is not None:                  # the embedding's output, kept for the passes' re-entries
            x0 = torch.empty_like(residual)
            ops.cast_rows(x0, residual)
        stack = self.depth.begin(residual) if self.depth is not None else None
        for run, li in enumerate(self.order):
            if self.loop is not None and run in self.loop.pass_of:
                residual, pending = self.loop.forward(run, residual, pending, x0), None
            # which norm reads the stream after this block (a block that can prepares that norm's input);
            # none after the last block: the final norm gathers the wanted rows
            nxt = self.blocks[self.order[run + 1]] if run + 1 < len(self.order) else None
            ctx.next_norm = nxt.first_norm() if hasattr(nxt, "first_norm") else None
            residual, pending = self.blocks[li].forward(residual, pending, ctx, self._view(cache, run))
            if self.depth is not None:
                residual, pending = self.depth.after(run, residual, pending, stack), None
            if self.stream_tap is not None:
                self.stream_tap(run, residual, pending)
        if ctx.num_wanted == 0:
            return None
        h = self.final_norm.add_norm(residual, pending, rows=ctx.want_rows)
        logits = self.lm_head(h, out_dtype=torch.float32)
        if self.spec.logit_softcap:
            ops.softcap(logits, self.spec.logit_softcap)
        if getattr(self.spec, "logit_scale", 1.0) != 1.0:
            ops.scale(logits, self.spec.logit_scale)
        return logits


class _BlockView:
    """Lets a LayerSpec be built through the block registry: its `kind` is the arrangement."""

    def __init__(self, layer):
        self.kind = layer.block
        self.mixer, self.feed_forward = layer.mixer, layer.feed_forward
        self.mixer_norm, self.ffn_norm = layer.mixer_norm, layer.ffn_norm
        self.mixer_scale, self.ffn_scale = getattr(layer, "mixer_scale", None), getattr(layer, "ffn_scale", None)
        self.residual_mult = getattr(layer, "residual_mult", 1.0)
        self.mixer_gate, self.ffn_gate = getattr(layer, "mixer_gate", None), getattr(layer, "ffn_gate", None)
