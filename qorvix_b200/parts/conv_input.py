"""A mixer behind a short causal convolution of its input: h <- h + conv(h), per channel over time, no bias, no
activation; the last taps - 1 inputs of a request are state (a slot of the cache manager, zeroed at admission), so a
prompt may be cut anywhere.  The wrapped mixer keeps its own cache or state; this part's cache_spec() lists them ahead of
the convolution's.  The input may be the float32 stream itself (blocks whose parts read the stream): the sum is formed
in float32 and leaves in the compute type."""
from __future__ import annotations

import torch

from ..cache.manager import CompositeCacheView
from ..cache.spec import FixedStateSpec
from ..csrc import ops
from .base import Mixer
from .registry import build_part, register_part


class ConvInput(Mixer):
    takes_stream = True            # forward() accepts the float32 stream as x

    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.inner = build_part("mixer", spec.inner, source, rt)
        self.weight = source.get(spec.weight, dtype=torch.float32).contiguous()       # [hidden, taps]; small: float32 on every path
        self.taps = int(spec.taps)
        if tuple(self.weight.shape) != (spec.hidden_size, self.taps):
            raise ValueError(f"{spec.weight} has shape {tuple(self.weight.shape)}, not {(spec.hidden_size, self.taps)}")
        inner = self.inner.cache_spec()
        self._inner_specs = list(inner) if isinstance(inner, (tuple, list)) else [inner]

    def cache_spec(self):
        return tuple(self._inner_specs + [FixedStateSpec((max(1, (self.taps - 1) * self.spec.hidden_size),), "float32")])

    def reads_cache_of(self):
        return self.inner.reads_cache_of()

    def forward(self, x, ctx, cache):
        views = cache.views
        h = torch.empty(x.shape, device=x.device, dtype=self.rt.dtype)
        ops.conv_state(h, x, self.weight, None, views[-1].tensor, ctx, act=False, add_input=True)
        inner_view = views[0] if len(self._inner_specs) == 1 else CompositeCacheView(views=list(views[:-1]))
        return self.inner.forward(h, ctx, inner_view)


register_part("mixer", "conv_input", ConvInput)
