"""The Lugizen decoder as data: LugizenConfig -> ModelSpec.

Every layer is a post-norm block, x += norm1(mixer(x + conv(x))), x += norm2(ff(x)), whose norms are RMS norms with one
number as weight and whose mixer reads its input through a short causal convolution per channel.  The mixer is rotary
grouped-query attention with unit-normed queries and keys and a temperature per head (layers that say so blend their
values with those of the first such layer), attention over a low-rank latent with a latent for the queries too and a
sliding window, or a delta rule with a decay per key channel; the feed-forward is dense with the tanh form of GELU,
routed experts, or absent.
Tensor names: embed, l<i>.norm1/.norm2, l<i>.canon1, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.lugizen_config import LugizenConfig
from ..parts.spec import (ActMLPSpec, ChannelDeltaSpec, ConvInputSpec, LatentAttentionSpec, LayerSpec, ModelSpec, MoESpec,
                          RMSNormSpec, RotarySpec, RotNormAttentionSpec)

V_SHARE = "first_values"           # the name under which the first value-mixing layer leaves its values for the others


def _rotary(rot: dict, size: int):
    if not rot["dims"]:
        return None
    return RotarySpec(head_dim=size, rotary_dim=int(rot["dims"]), theta=float(rot["base"]), pairing="split_half")


def _attention(m: dict, p: str, width: int, eps: float, role):
    return RotNormAttentionSpec(hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], value_dim=m["vdim"],
                                scale=float(m["scale"]), eps=eps, q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", o_proj=p + "o",
                                position=_rotary(m["rot"], m["dim"]), head_temp=p + "temp", v_share=V_SHARE if role else None,
                                v_share_role=role, v_blend=p + "vmix" if role else None)


def _latent(m: dict, p: str, width: int, eps: float):
    position = _rotary(m["rot"], m["rot_dim"]) or RotarySpec(head_dim=m["rot_dim"], rotary_dim=0, theta=1.0, pairing="split_half")
    return LatentAttentionSpec(hidden_size=width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
                               kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=eps, position=position, q_proj=p + "uq",
                               kv_down=p + "dkv", kv_norm=p + "dkv.norm", k_up=p + "uk", v_up=p + "uv", gate_proj=None, o_proj=p + "o",
                               window=int(m["mask"]["size"]), q_rank=m["q_rank"], q_down=p + "dq", q_norm=p + "dq.norm")


def _delta(m: dict, p: str, width: int, eps: float, decay_rank: int, gate_rank: int):
    return ChannelDeltaSpec(hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                            conv_taps=m["conv"], decay_rank=decay_rank, gate_rank=gate_rank, eps=eps, q_proj=p + "q", k_proj=p + "k",
                            v_proj=p + "v", beta_proj=p + "b", a_down=p + "a1", a_up=p + "a2", dt_bias=p + "dt_bias", a_log=p + "A_log",
                            gate_down=p + "g1", gate_up=p + "g2", norm=p + "norm", o_proj=p + "o")


def lugizen_spec(cfg: LugizenConfig, shapes=None) -> ModelSpec:
    """shapes: name -> shape of the stored tensors.  The ranks of the delta rule's two low-rank products are given by tensors
    only; without shapes (random-weights mode) they take `decay_rank` / `gate_rank` of the layer's mixer entry if present,
    else 16."""
    width, eps = cfg.width, cfg.norm_eps
    shapes = shapes or {}

    def rows_of(name, entry, key):
        if name in shapes:
            return int(shapes[name][0])
        return int(entry.get(key, 16))

    layers = []
    shared_values = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            role = None
            if m.get("v_mix"):
                role = "blend" if shared_values else "source"
                shared_values = True
            mixer = _attention(m, p + "mix.", width, eps, role)
        elif kind == "latent_attention":
            mixer = _latent(m, p + "mix.", width, eps)
        else:
            mixer = _delta(m, p + "mix.", width, eps, rows_of(p + "mix.a1", m, "decay_rank"), rows_of(p + "mix.g1", m, "gate_rank"))
        mixer = ConvInputSpec(inner=mixer, hidden_size=width, taps=cfg.canon_taps, weight=p + "canon1")
        f = layer.get("mlp")
        if f is None:
            ff = None
        elif f["kind"] == "dense":
            ff = ActMLPSpec(width, f["ff"], p + "mlp.up", p + "mlp.down", activation="gelu_tanh")
        else:
            ff = MoESpec(hidden_size=width, experts=f["router"]["experts"], top=f["router"]["top"], expert_ff=f["expert"]["ff"],
                         router=p + "mlp.router", expert_prefix=p + "mlp.e")
        layers.append(LayerSpec(mixer=mixer, feed_forward=ff, mixer_norm=RMSNormSpec(width, eps, p + "norm1", scalar=True),
                                ffn_norm=RMSNormSpec(width, eps, p + "norm2", scalar=True) if ff is not None else None, block="post_norm"))
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden_size=width, embedding="embed", layers=layers,
                     final_norm=RMSNormSpec(width, eps, "final.norm", scalar=True), lm_head="head")


register_architecture("Lugizen", LugizenConfig.from_dict, lugizen_spec, shapes_from_tensors=True)
