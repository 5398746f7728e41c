"""Small Tubazen configurations with weights drawn for the tests: matrices scaled so that activations are of order one,
attention is peaked and the distance bias is large (a key one place off, a wrong bucket or another request's page then
shows in the logits), decays spread over (0, 1) so that old tokens still weigh.  Sizes differ from layer to layer on
purpose: grouped and ungrouped heads, value sizes that are not the key size, ranks and table sizes that are no powers of
two, layers without a feed-forward, any order of the two kinds of layers."""
from __future__ import annotations

import json
import math
import tempfile
from pathlib import Path

import torch

from qorvix_b200.weights import write_safetensors


def gla(heads=3, dim=20, vdim=28, tau=7.0, rank=5):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def left(heads=4, kv_heads=2, dim=24, vdim=40, sharp=3.0, bias_max=50, rows=14, coef=0.4, every=7):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": sharp / dim ** 0.5, "bias_max": bias_max,
            "q_temp": {"coef": coef, "every": every}, "bias_rows": rows}


def right(heads=2, dim=18, rank=6):
    return {"heads": heads, "dim": dim, "rank": rank}


def pair(l=None, r=None, left_scale=1.3, right_scale=0.8):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right(), "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff=88):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(layers, vocab=211, width=72, eps=2e-5, logit_scale=0.7, positions=256):
    return {"architecture": "Tubazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "max_positions": positions, "layers": layers}


def stored(cfg):
    """The configuration as config.json holds it: the sizes that only tensors give (ranks, table rows) are taken out."""
    out = json.loads(json.dumps(cfg))
    for l in out["layers"]:
        l["mixer"].pop("rank", None)
        if l["type"] == "parallel":
            l["mixer"]["left"].pop("bias_rows", None)
            l["mixer"]["right"].pop("rank", None)
    return out


# A: both kinds of layers, grouped heads, a layer without feed-forward
CONFIG_A = config([layer(gla(), dense()), layer(pair(), dense(ff=40)), layer(gla(heads=2, dim=33, vdim=12, tau=2.5, rank=3), None),
                   layer(pair(left(heads=6, kv_heads=1, dim=8, vdim=8, bias_max=23, rows=9, coef=1.1, every=3), right(heads=3, dim=40, rank=2),
                              left_scale=0.6, right_scale=1.7), dense(ff=50))])
# B: side-by-side layers first, one head everywhere, factor one on the logits, temperature steps longer than the prompts
CONFIG_B = config([layer(pair(left(heads=1, kv_heads=1, dim=36, vdim=20, bias_max=200, rows=32, coef=0.35, every=1000), right(heads=1, dim=64, rank=16),
                              left_scale=1.0, right_scale=1.0), dense(ff=24)),
                   layer(gla(heads=1, dim=64, vdim=64, tau=12.0, rank=16), dense(ff=96))],
                  vocab=150, width=48, eps=1e-6, logit_scale=1.0)
# C: sizes in multiples of 16 and 32; only side-by-side layers; the bias table ends before the longest distance
CONFIG_C = config([layer(pair(left(heads=4, kv_heads=4, dim=32, vdim=64, bias_max=40, rows=16, every=16), right(heads=2, dim=32, rank=8)), dense(ff=96)),
                   layer(pair(left(heads=8, kv_heads=2, dim=16, vdim=32, bias_max=90, rows=20, every=5), right(heads=4, dim=16, rank=4)), None)],
                  vocab=190, width=64, eps=4e-6, logit_scale=0.25)
# D: only gated linear attention; sizes that are multiples of neither 8 nor 16 anywhere
CONFIG_D = config([layer(gla(heads=3, dim=10, vdim=14, tau=3.0, rank=7), dense(ff=30)), layer(gla(heads=2, dim=70, vdim=6, tau=30.0, rank=1), dense(ff=13)),
                   layer(gla(heads=5, dim=6, vdim=22, tau=1.0, rank=9), None)], vocab=97, width=44, eps=3e-5, logit_scale=2.0)


def _rnd(g, *shape):
    return torch.randn(*shape, generator=g)


def _round(w):
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()}


def gla_weights(l, width, g):
    m = l["mixer"]
    H, n, dv, R = m["heads"], m["dim"], m["vdim"], m["rank"]
    fan = width ** -0.5
    return _round({"q": _rnd(g, H * n, width) * fan * 2, "k": _rnd(g, H * n, width) * fan, "v": _rnd(g, H * dv, width) * fan,
                   "g": _rnd(g, H * dv, width) * fan, "o": _rnd(g, width, H * dv) * (H * dv) ** -0.5, "norm": 1 + 0.2 * _rnd(g, dv),
                   "a1": _rnd(g, R, width) * fan, "a2": _rnd(g, H * n, R) * R ** -0.5 * 2, "a2.b": 1.5 + _rnd(g, H * n)})


def left_weights(m, width, g):
    H, G, n, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    fan = width ** -0.5
    return _round({"q": _rnd(g, H * n, width) * fan, "q.b": 0.3 * _rnd(g, H * n), "k": _rnd(g, G * n, width) * fan, "k.b": 0.3 * _rnd(g, G * n),
                   "v": _rnd(g, G * dv, width) * fan, "v.b": 0.3 * _rnd(g, G * dv), "g": _rnd(g, H * dv, width) * fan,
                   "rel": 1.5 * _rnd(g, m["bias_rows"], H), "o": _rnd(g, width, H * dv) * (H * dv) ** -0.5, "o.b": 0.2 * _rnd(g, width)})


def right_weights(m, width, g):
    H, n, R = m["heads"], m["dim"], m["rank"]
    fan = width ** -0.5
    w = {name: _rnd(g, H * n, width) * fan for name in ("r", "k", "v", "g", "a")}
    w.update({"a.b": 0.5 * _rnd(g, H * n), "w1": _rnd(g, R, width) * fan, "w2": _rnd(g, H * n, R) * R ** -0.5 * 2, "w0": _rnd(g, H * n),
              "norm": 1 + 0.2 * _rnd(g, H * n), "o": _rnd(g, width, H * n) * (H * n) ** -0.5})
    return _round(w)


def mixer_weights(l, width, g):
    if l["type"] == "gla":
        return gla_weights(l, width, g)
    w = {"left." + k: v for k, v in left_weights(l["mixer"]["left"], width, g).items()}
    w.update({"right." + k: v for k, v in right_weights(l["mixer"]["right"], width, g).items()})
    return w


def mlp_weights(f, width, g):
    ff, fan = f["ff"], width ** -0.5
    return _round({"gate": _rnd(g, ff, width) * fan * 1.5, "up": _rnd(g, ff, width) * fan * 1.5, "down": _rnd(g, width, ff) * ff ** -0.5})


def norm_weights(name, width, g):
    return {name: 1 + 0.2 * _rnd(g, width), name + ".b": 0.1 * _rnd(g, width), name + ".alpha": (0.6 + 0.2 * torch.rand((), generator=g))}


def model_weights(cfg, seed):
    """name -> tensor as a checkpoint stores it (bfloat16)."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = cfg["width"], cfg["vocab"]
    w = {"embed": _rnd(g, vocab, width), "pos": 0.5 * _rnd(g, cfg["max_positions"], width), "head": _rnd(g, vocab, width) * width ** -0.5 * 3}
    w.update(norm_weights("embed.norm", width, g))
    w.update(norm_weights("final.norm", width, g))
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        w.update(norm_weights(p + "norm1", width, g))
        for k, v in mixer_weights(l, width, g).items():
            w[p + "mix." + k] = v
        w[p + "rg1"] = _rnd(g, width, width) * width ** -0.5
        w[p + "rg1.b"] = 0.5 * _rnd(g, width)
        if l.get("mlp") is not None:
            w.update(norm_weights(p + "norm2", width, g))
            for k, v in mlp_weights(l["mlp"], width, g).items():
                w[p + "mlp." + k] = v
            w[p + "rg2"] = _rnd(g, width, width) * width ** -0.5
            w[p + "rg2.b"] = 0.5 * _rnd(g, width)
        w[p + "dwa"] = (1.0 / (i + 2)) + 0.3 * _rnd(g, i + 2)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def as_float64(weights):
    return {k: v.double() for k, v in weights.items()}


def make_model_dir(cfg, seed) -> Path:
    d = Path(tempfile.mkdtemp(prefix="qv_tubazen_"))
    (d / "config.json").write_text(json.dumps(stored(cfg)))
    write_safetensors(d / "model.safetensors", model_weights(cfg, seed).items())
    return d
