"""The Tubazen decoder as data: TubazenConfig -> ModelSpec.

The embedding adds a learned position row to the token row and norms the sum; all norms are the tanh norm
(no statistics).  Every layer is a pre-norm block whose two results each pass a sigmoid gate computed from the
sublayer's input; its mixer is gated linear attention, or softmax attention with a learned distance bias
beside a generalized delta rule; its feed-forward is dense and gated with the tanh form of GELU.  After each
layer the stream becomes a weighted sum of the embedding's output and all layers' results so far.  The logits
carry a fixed factor.
Tensor names: embed, pos, embed.norm(.b/.alpha), l<i>.norm1/.norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.rg1/.rg2(.b),
l<i>.dwa, final.norm, head.
"""
from __future__ import annotations

import math

from ..config import register_architecture
from ..config.tubazen_config import TubazenConfig
from ..parts.spec import (BiasedAttentionSpec, ChannelDecaySpec, DeltaRuleSpec, DepthAverageSpec, GLASpec, LayerSpec, ModelSpec,
                          PositionedEmbeddingSpec, SideBySideSpec, SwiGLUSpec, TanhNormSpec)

DELTA_DECAY_RATE = math.exp(-0.5)         # the delta rule's decay is exp(-rate * sigmoid(.)): never below exp(-rate)


def _gla(m: dict, p: str, width: int, eps: float, rank: int) -> GLASpec:
    decay = ChannelDecaySpec(rank=rank, down=p + "a1", up=p + "a2", bias=p + "a2.b", form="pow_sigmoid", param=float(m["tau"]))
    return GLASpec(hidden_size=width, num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"], eps=eps, q_proj=p + "q",
                   k_proj=p + "k", v_proj=p + "v", gate_proj=p + "g", decay=decay, norm=p + "norm", o_proj=p + "o")


def _left(m: dict, p: str, width: int, rows: int) -> BiasedAttentionSpec:
    return BiasedAttentionSpec(hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                               scale=float(m["scale"]), bias_rows=rows, bias_max=float(m["bias_max"]), temp_coef=float(m["q_temp"]["coef"]),
                               temp_every=int(m["q_temp"]["every"]), q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", gate_proj=p + "g",
                               rel_bias=p + "rel", o_proj=p + "o")


def _right(m: dict, p: str, width: int, eps: float, rank: int) -> DeltaRuleSpec:
    decay = ChannelDecaySpec(rank=rank, down=p + "w1", up=p + "w2", bias=p + "w0", form="exp_neg_sigmoid", param=DELTA_DECAY_RATE,
                             inner_tanh=True)
    return DeltaRuleSpec(hidden_size=width, num_heads=m["heads"], head_dim=m["dim"], eps=eps, r_proj=p + "r", k_proj=p + "k",
                         v_proj=p + "v", gate_proj=p + "g", a_proj=p + "a", decay=decay, norm=p + "norm", o_proj=p + "o")


def tubazen_spec(cfg: TubazenConfig, shapes=None) -> ModelSpec:
    """shapes: name -> shape of the stored tensors.  Two sizes are given by tensors only (the rank of the decays' low-rank
    products and the rows of the distance-bias table); without shapes (random-weights mode) they take `rank` / `bias_rows`
    of the layer's mixer entry if present, else 16 and 32."""
    width, eps = cfg.width, cfg.norm_eps
    shapes = shapes or {}

    def size_of(name, entry, key, default):
        if name in shapes:
            return int(shapes[name][0])
        return int(entry.get(key, default))

    layers, mixes = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "gla":
            mixer = _gla(m, p + "mix.", width, eps, size_of(p + "mix.a1", m, "rank", 16))
        else:
            lp, rp = p + "mix.left.", p + "mix.right."
            mixer = SideBySideSpec(left=_left(m["left"], lp, width, size_of(lp + "rel", m["left"], "bias_rows", 32)),
                                   right=_right(m["right"], rp, width, eps, size_of(rp + "w1", m["right"], "rank", 16)),
                                   left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)))
        f = layer.get("mlp")
        ff = SwiGLUSpec(width, f["ff"], p + "mlp.gate", p + "mlp.up", p + "mlp.down", activation="gelu_tanh") if f is not None else None
        layers.append(LayerSpec(mixer_norm=TanhNormSpec(width, p + "norm1"), mixer=mixer,
                                ffn_norm=TanhNormSpec(width, p + "norm2") if ff is not None else None, feed_forward=ff,
                                block="gated_pre_norm", mixer_gate=p + "rg1", ffn_gate=p + "rg2" if ff is not None else None))
        mixes.append(p + "dwa")
    embedding = PositionedEmbeddingSpec(cfg.vocab_size, width, cfg.max_positions, "embed", "pos", norm=TanhNormSpec(width, "embed.norm"))
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=width, embedding=embedding, layers=layers,
                     final_norm=TanhNormSpec(width, "final.norm"), lm_head="head", max_position=cfg.max_positions,
                     logit_scale=cfg.logit_scale, depth_average=DepthAverageSpec(tuple(mixes), width))


register_architecture("Tubazen", TubazenConfig.from_dict, tubazen_spec, shapes_from_tensors=True)
