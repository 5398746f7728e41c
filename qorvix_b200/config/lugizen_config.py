"""Configuration of the Lugizen decoder, read from its own config.json keys.

A Lugizen model is a list of layers whose norms sit on the sublayers' outputs: x += norm1(mixer(x + conv(x))),
x += norm2(ff(x)), the norms having one number as weight and the mixer's input first passing a short causal
convolution per channel.  The mixer is rotary grouped-query attention with unit-normed queries and keys and a
temperature per head ('attention', optionally blending its values with those of the first such layer), attention
over a low-rank latent with a sliding window ('latent_attention'), or a delta rule with a decay per key channel
('channel_delta'); the feed-forward is dense (tanh form of GELU), routed experts, or absent.  config.json gives every
size and constant layer by layer, so nothing about a layer is assumed from another.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .deganex_config import _need, _positive_int
from .model_config import ConfigError, ModelConfig

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "rot"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot", "mask"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}
MIXER_SIZES = {
    "attention": ("heads", "kv_heads", "dim", "vdim"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class LugizenConfig(ModelConfig):
    """Field names follow config.json; `layers` keeps each layer's entry as it is written there."""
    vocab_size: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    canon_taps: int = 1
    layers: Tuple[dict, ...] = field(default_factory=tuple)

    @staticmethod
    def from_dict(d: dict) -> "LugizenConfig":
        layers = _need(d, "layers", "config")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = LugizenConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Lugizen"])[0]),
            vocab_size=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
            norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
            canon_taps=_positive_int(_need(d, "canon", "config"), "taps", "canon"),
            layers=tuple(copy.deepcopy(l) for l in layers), eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if self.canon_taps > 16:
            raise ConfigError(f"config.json: canon.taps {self.canon_taps} is more than the 16 the convolution kernel takes")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a known mixer (known: {', '.join(MIXER_KEYS)})")
            m = _need(layer, "mixer", where)
            for key in MIXER_KEYS[kind]:
                _need(m, key, where + ".mixer")
            for key in MIXER_SIZES[kind]:
                _positive_int(m, key, where + ".mixer")
            if "kv_heads" in m and m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {where}.mixer.heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
            if "rot" in MIXER_KEYS[kind]:
                dims = _need(m["rot"], "dims", where + ".mixer.rot")
                _need(m["rot"], "base", where + ".mixer.rot")
                limit = m["rot_dim"] if kind == "latent_attention" else m["dim"]
                if not isinstance(dims, int) or dims < 0 or dims % 2 or dims > limit:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims {dims!r} must be even and at most {limit}")
            if kind == "latent_attention":
                _positive_int(m["mask"], "size", where + ".mixer.mask")
            if kind == "channel_delta" and m["conv"] > 16:
                raise ConfigError(f"config.json: {where}.mixer.conv {m['conv']} is more than the 16 taps the convolution kernel takes")
            f = layer.get("mlp")
            if f is None:
                continue
            fk = _need(f, "kind", where + ".mlp")
            if fk not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}.mlp.kind '{fk}' is not known (known: {', '.join(MLP_KINDS)})")
            if fk == "dense":
                _positive_int(f, "ff", where + ".mlp")
            else:
                _positive_int(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert")
                r = _need(f, "router", where + ".mlp")
                experts, top = _positive_int(r, "experts", where + ".mlp.router"), _positive_int(r, "top", where + ".mlp.router")
                if top > experts:
                    raise ConfigError(f"config.json: {where}.mlp.router.top {top} is more than its {experts} experts")

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "canon": {"taps": self.canon_taps},
                             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
