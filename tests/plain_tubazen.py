"""Plain, slow Tubazen decoder: whole sequences, no cache, one function per mechanism, all float64.

The oracle of the Tubazen tests.  It shares no code with the product package: its own reading of the
configuration (a dict as config.json holds it) and its own arithmetic.  A sequence is run whole.

Notation: h is a part's input [T, width]; W[name] a weight [out, in] applied as h @ W^T; positions count
from 0; `unit(x)` is x over its root mean square (eps under the root).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def tanh_norm(x, W, name):
    """The norm without statistics: tanh(alpha x) w + b."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def distance_bucket(n, rows, far):
    """Row of the distance table for distance n >= 0: one row per distance below half the rows, then rows
    spaced evenly in the logarithm of the distance up to `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log((p + 1) // every + 1)


def biased_attention(h, W, p, m):
    """Grouped-query softmax attention without rotation: queries scaled by a temperature that grows with the
    position, a learned bias per (distance bucket, head) added to the scaled scores, sigmoid output gate."""
    T = h.shape[0]
    H, G, n, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, n)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, n)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, dv)
    rel = W[p + "rel"]
    rows = rel.shape[0]
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        qi = q[i] * query_temperature(i, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))
        for hd in range(H):
            g = hd // (H // G)
            s = (k[: i + 1, g] @ qi[hd]) * float(m["scale"])
            s = s + torch.stack([rel[distance_bucket(i - j, rows, float(m["bias_max"])), hd] for j in range(i + 1)])
            out[i, hd] = torch.softmax(s, dim=0) @ v[: i + 1, g]
    gate = torch.sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ W[p + "o"].T + W[p + "o.b"]


def delta_rule(h, W, p, m, eps, state=None):
    """Per head a dim x dim state: S = diag(w) S - (a u)(u^T S) + k v^T, both first terms reading the old
    state, u the key over its length; o = S^T r, divided by its root mean square, weighted and gated."""
    T = h.shape[0]
    H, n = m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).reshape(T, H, n)
    k = (h @ W[p + "k"].T).reshape(T, H, n)
    v = (h @ W[p + "v"].T).reshape(T, H, n)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(T, H, n)
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).reshape(T, H, n)
    S = torch.zeros(H, n, n, dtype=F64) if state is None else state
    o = torch.zeros(T, H, n, dtype=F64)
    for t in range(T):
        for hd in range(H):
            u = k[t, hd] / torch.sqrt((k[t, hd] ** 2).sum() + 1e-6)
            old = S[hd]
            S[hd] = w[t, hd][:, None] * old - torch.outer(a[t, hd] * u, u @ old) + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ r[t, hd]
    o = unit(o, eps).reshape(T, H * n) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def gated_linear_attention(h, W, p, m, eps, state=None):
    """Per head a dim x vdim state with a decay per key channel: S = diag(alpha) S + k v^T, o = S^T q."""
    T = h.shape[0]
    H, n, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, n) * n ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, n)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / float(m["tau"]))).reshape(T, H, n)
    S = torch.zeros(H, n, dv, dtype=F64) if state is None else state
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hd in range(H):
            S[hd] = alpha[t, hd][:, None] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = (unit(o, eps) * W[p + "norm"]).reshape(T, H * dv) * silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def side_by_side(h, W, p, m, eps):
    left = biased_attention(h, W, p + "left.", m["left"])
    right = delta_rule(h, W, p + "right.", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def mixer(kind, h, W, p, m, eps):
    if kind == "gla":
        return gated_linear_attention(h, W, p, m, eps)
    if kind == "parallel":
        return side_by_side(h, W, p, m, eps)
    raise ValueError(kind)


def dense_feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def gated(h, W, name):
    """The gate of a sublayer's result: sigmoid of a product with the sublayer's input."""
    return torch.sigmoid(h @ W[name].T + W[name + ".b"])


def layer(x, W, i, entry, eps):
    p = f"l{i}."
    h = tanh_norm(x, W, p + "norm1")
    x = x + mixer(entry["type"], h, W, p + "mix.", entry["mixer"], eps) * gated(h, W, p + "rg1")
    if entry.get("mlp") is not None:
        h = tanh_norm(x, W, p + "norm2")
        x = x + dense_feed_forward(h, W, p + "mlp.") * gated(h, W, p + "rg2")
    return x


def embedding(tokens, W):
    T = len(tokens)
    x = W["embed"][torch.tensor(tokens)] + W["pos"][:T]
    return tanh_norm(x, W, "embed.norm")


def forward(cfg, W, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence.  W: name -> float64 tensor.  streams (a list) receives the
    stream after every layer."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = embedding(tokens, W)
    kept = [x]                                   # the embedding's output and every layer's own result
    for i, entry in enumerate(cfg["layers"]):
        kept.append(layer(x, W, i, entry, eps))
        mix = W[f"l{i}.dwa"]
        x = sum(mix[j] * kept[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x)
    return (tanh_norm(x, W, "final.norm") @ W["head"].T) * float(cfg["logit_scale"])
