"""Configuration of the Tubazen decoder, read from its own config.json keys.

A Tubazen model is a list of pre-norm layers whose mixer is gated linear attention ('gla') or two mixers
side by side ('parallel': softmax attention with a learned distance bias beside a generalized delta rule),
each followed by an optional dense gated feed-forward; every sublayer's result passes a sigmoid gate, and
the stream after a layer is a weighted sum of all layers' results so far.  config.json gives every size and
constant layer by layer, so nothing about a layer is assumed from another.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .deganex_config import _need, _positive_int
from .model_config import ConfigError, ModelConfig

GLA_KEYS = ("heads", "dim", "vdim", "tau")
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max", "q_temp")
RIGHT_KEYS = ("heads", "dim")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class TubazenConfig(ModelConfig):
    """Field names follow config.json; `layers` keeps each layer's entry as it is written there."""
    vocab_size: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    logit_scale: float = 1.0
    max_positions: int = 0
    layers: Tuple[dict, ...] = field(default_factory=tuple)

    @staticmethod
    def from_dict(d: dict) -> "TubazenConfig":
        layers = _need(d, "layers", "config")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = TubazenConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Tubazen"])[0]),
            vocab_size=_positive_int(d, "vocab", "config"), width=_positive_int(d, "width", "config"),
            norm_eps=float(_need(_need(d, "norm", "config"), "eps", "norm")),
            logit_scale=float(d.get("logit_scale", 1.0)), max_positions=_positive_int(d, "max_positions", "config"),
            layers=tuple(copy.deepcopy(l) for l in layers), eos_token_id=d.get("eos_token_id"))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            m = _need(layer, "mixer", where)
            if kind == "gla":
                for key in GLA_KEYS:
                    _need(m, key, where + ".mixer")
                for key in ("heads", "dim", "vdim"):
                    _positive_int(m, key, where + ".mixer")
                if not float(m["tau"]) > 0:
                    raise ConfigError(f"config.json: {where}.mixer.tau must be positive")
            elif kind == "parallel":
                left, right = _need(m, "left", where + ".mixer"), _need(m, "right", where + ".mixer")
                for key in LEFT_KEYS:
                    _need(left, key, where + ".mixer.left")
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(left, key, where + ".mixer.left")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.mixer.left.heads {left['heads']} is not a multiple of kv_heads {left['kv_heads']}")
                _need(left["q_temp"], "coef", where + ".mixer.left.q_temp")
                _positive_int(left["q_temp"], "every", where + ".mixer.left.q_temp")
                if not float(left["bias_max"]) > 0:
                    raise ConfigError(f"config.json: {where}.mixer.left.bias_max must be positive")
                for key in RIGHT_KEYS:
                    _positive_int(right, key, where + ".mixer.right")
            else:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a known mixer (known: gla, parallel)")
            f = layer.get("mlp")
            if f is None:
                continue
            fk = _need(f, "kind", where + ".mlp")
            if fk not in MLP_KINDS:
                raise ConfigError(f"config.json: {where}.mlp.kind '{fk}' is not known (known: {', '.join(MLP_KINDS)})")
            _positive_int(f, "ff", where + ".mlp")

    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale, "max_positions": self.max_positions,
                             "layers": [copy.deepcopy(l) for l in self.layers]}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
