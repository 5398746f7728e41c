"""Small Lugizen configurations with weights drawn for the tests: matrices scaled so that activations are of order one,
attention is peaked (a key one place off, a window one token off or another request's page then shows in the logits),
decays close to one so that old tokens still weigh in the recurrent state, values blended between layers with a
weight far from 0 and 1.  Sizes differ from layer to layer on purpose: grouped and ungrouped heads, value sizes that are
not the key size, rotation over a part of a head, over all of it or none, ranks that are no powers of two, layers without
a feed-forward, every order of the kinds of layers, windows shorter and longer than the prompts."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from qorvix_b200.weights import write_safetensors


def attn(heads=4, kv_heads=2, dim=24, vdim=40, sharp=2.0, rot_dims=16, base=10000.0, v_mix=False):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": sharp / dim ** 0.5, "rot": {"base": base, "dims": rot_dims}}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, q_rank=28, window=37, sharp=2.0, base=50000.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": sharp / (dim + rot_dim) ** 0.5, "rot": {"base": base, "dims": rot_dim}, "mask": {"size": window}}}


def delta(heads=4, kv_heads=2, dim=20, vdim=12, conv=3, decay_rank=5, gate_rank=7):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": decay_rank, "gate_rank": gate_rank}}


def dense(ff=88):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(layers, vocab=211, width=72, eps=2e-5, taps=3):
    return {"architecture": "Lugizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}


def stored(cfg):
    """The configuration as config.json holds it: the sizes that only tensors give (the delta rule's ranks) are taken out."""
    out = json.loads(json.dumps(cfg))
    for l in out["layers"]:
        l["mixer"].pop("decay_rank", None)
        l["mixer"].pop("gate_rank", None)
    return out


# A: every kind of layer and feed-forward, grouped heads, three layers that blend values and one that does not
CONFIG_A = config([layer(latent(), dense()), layer(delta(), moe()), layer(attn(v_mix=True), moe(experts=5, top=3, ff=16)),
                   layer(attn(v_mix=True, sharp=2.5), None), layer(attn(heads=2, kv_heads=1, dim=16, vdim=8, rot_dims=16), dense(40)),
                   layer(attn(v_mix=True, rot_dims=8, base=300.0), dense(24)), layer(latent(heads=2, dim=10, rot_dim=6, vdim=30, kv_rank=17, q_rank=9, window=5), moe())])
# B: ones everywhere: one head, one expert of which one is used, one tap (no convolution at all), a window of one token
CONFIG_B = config([layer(attn(heads=1, kv_heads=1, dim=36, vdim=20, rot_dims=2, v_mix=True), moe(experts=1, top=1, ff=30)),
                   layer(delta(heads=1, kv_heads=1, dim=64, vdim=64, conv=1, decay_rank=1, gate_rank=1), dense(24)),
                   layer(latent(heads=1, dim=12, rot_dim=4, vdim=12, kv_rank=12, q_rank=12, window=1), None)],
                  vocab=150, width=48, eps=1e-6, taps=1)
# C: sizes in multiples of 64 and windows that end on page borders; the recurrent layer first
CONFIG_C = config([layer(delta(heads=4, kv_heads=4, dim=64, vdim=64, conv=4, decay_rank=16, gate_rank=8), moe(experts=8, top=4, ff=64)),
                   layer(latent(heads=4, dim=48, rot_dim=16, vdim=64, kv_rank=64, q_rank=64, window=64), dense(128)),
                   layer(attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64, v_mix=True), moe(experts=16, top=2, ff=128)),
                   layer(latent(heads=2, dim=64, rot_dim=32, vdim=32, kv_rank=128, q_rank=32, window=48), None),
                   layer(attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, v_mix=True), dense(64))],
                  vocab=190, width=128, eps=4e-6, taps=4)
# D: attention only, seventeen query heads on a key/value head, no rotation in one layer, sizes that are multiples of nothing
CONFIG_D = config([layer(attn(heads=17, kv_heads=1, dim=6, vdim=10, rot_dims=6), dense(30)),
                   layer(attn(heads=3, kv_heads=3, dim=14, vdim=6, rot_dims=0, v_mix=True), moe(experts=3, top=3, ff=10)),
                   layer(delta(heads=6, kv_heads=2, dim=10, vdim=22, conv=5, decay_rank=3, gate_rank=2), None),
                   layer(attn(heads=6, kv_heads=3, dim=10, vdim=6, rot_dims=4, v_mix=True), moe(experts=7, top=1, ff=13)),
                   layer(latent(heads=5, dim=6, rot_dim=2, vdim=22, kv_rank=9, q_rank=5, window=200), dense(13))],
                  vocab=97, width=44, eps=3e-5, taps=6)


def _rnd(g, *shape):
    return torch.randn(shape, generator=g)


def _round(w):
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def attn_weights(m, width, g):
    H, G, n, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    fan = width ** -0.5
    w = {"q": _rnd(g, H * n, width) * fan, "k": _rnd(g, G * n, width) * fan, "v": _rnd(g, G * dv, width) * fan,
         "o": _rnd(g, width, H * dv) * (H * dv) ** -0.5, "temp": 1.0 + 0.3 * _rnd(g, H)}
    if m.get("v_mix"):
        w["vmix"] = torch.tensor(0.35) + 0.1 * _rnd(g)
    return _round(w)


def latent_weights(m, width, g):
    H, n, r, dv, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    fan = width ** -0.5
    return _round({"dq": _rnd(g, qr, width) * fan, "dq.norm": 1 + 0.2 * _rnd(g, qr), "uq": _rnd(g, H * (n + r), qr) * qr ** -0.5,
                   "dkv": _rnd(g, rank + r, width) * fan, "dkv.norm": 1 + 0.2 * _rnd(g, rank), "uk": _rnd(g, H * n, rank) * rank ** -0.5,
                   "uv": _rnd(g, H * dv, rank) * rank ** -0.5, "o": _rnd(g, width, H * dv) * (H * dv) ** -0.5})


def delta_weights(m, width, g):
    H, G, n, dv, taps, ra, rg = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], m["decay_rank"], m["gate_rank"]
    fan = width ** -0.5
    w = {"q": _rnd(g, G * n, width) * fan * 2, "k": _rnd(g, G * n, width) * fan * 2, "v": _rnd(g, H * dv, width) * fan * 2,
         "b": _rnd(g, H, width) * fan * 2, "A_log": -1.0 + 0.5 * _rnd(g, H), "norm": 1 + 0.2 * _rnd(g, dv),
         "a1": _rnd(g, ra, width) * fan, "a2": _rnd(g, H * n, ra) * ra ** -0.5, "dt_bias": -2.0 + _rnd(g, H * n),
         "g1": _rnd(g, rg, width) * fan, "g2": _rnd(g, H * dv, rg) * rg ** -0.5 * 2, "o": _rnd(g, width, H * dv) * (H * dv) ** -0.5}
    for name, ch in (("q", G * n), ("k", G * n), ("v", H * dv)):
        w[name + ".conv"] = _rnd(g, ch, taps) * 0.5 + torch.cat([torch.zeros(ch, taps - 1), torch.ones(ch, 1)], dim=1)
    return _round(w)


def mixer_weights(l, width, g):
    return {"attention": attn_weights, "latent_attention": latent_weights, "channel_delta": delta_weights}[l["type"]](l["mixer"], width, g)


def mlp_weights(f, width, g):
    fan = width ** -0.5
    if f["kind"] == "dense":
        ff = f["ff"]
        return _round({"up": _rnd(g, ff, width) * fan * 1.5, "down": _rnd(g, width, ff) * ff ** -0.5})
    ff, E = f["expert"]["ff"], f["router"]["experts"]
    w = {"router": _rnd(g, E, width) * fan * 8}            # logits well apart: few tokens sit on a close call between two experts
    for e in range(E):
        w[f"e{e}.gate"] = _rnd(g, ff, width) * fan * 1.5
        w[f"e{e}.up"] = _rnd(g, ff, width) * fan * 1.5
        w[f"e{e}.down"] = _rnd(g, width, ff) * ff ** -0.5
    return _round(w)


def layer_weights(l, i, width, taps, g):
    p = f"l{i}."
    w = {p + "norm1": 1.0 + 0.2 * _rnd(g), p + "canon1": _rnd(g, width, taps) * 0.3}
    for k, v in mixer_weights(l, width, g).items():
        w[p + "mix." + k] = v
    if l.get("mlp") is not None:
        w[p + "norm2"] = 0.8 + 0.2 * _rnd(g)
        for k, v in mlp_weights(l["mlp"], width, g).items():
            w[p + "mlp." + k] = v
    return w


def model_weights(cfg, seed):
    """name -> tensor as a checkpoint stores it (bfloat16)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w = {"embed": _rnd(g, vocab, width), "head": _rnd(g, vocab, width) * width ** -0.5 * 3, "final.norm": 1.0 + 0.1 * _rnd(g)}
    for i, l in enumerate(cfg["layers"]):
        w.update(layer_weights(l, i, width, cfg["canon"]["taps"], g))
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def as_float64(weights):
    return {k: v.double() for k, v in weights.items()}


def make_model_dir(cfg, seed) -> Path:
    d = Path(tempfile.mkdtemp(prefix="qv_lugizen_"))
    (d / "config.json").write_text(json.dumps(stored(cfg)))
    write_safetensors(d / "model.safetensors", model_weights(cfg, seed).items())
    return d
