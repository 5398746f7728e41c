"""Plain, slow Lugizen decoder: whole sequences, no cache, one function per mechanism, all float64.

The oracle of the Lugizen tests.  It shares no code with the product package: its own reading of the
configuration (a dict as config.json holds it) and its own arithmetic.  A sequence is run whole; the recurrent
mixer and the convolutions may be handed a state to continue from, for the tests of single mechanisms.

Notation: h is a part's input [T, width]; W[name] a weight [out, in] applied as h @ W^T; positions count from 0;
`unit(x)` is x over its root mean square (eps under the root).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64
KEY_EPS = 1e-6                     # under the root of the recurrence's unit vectors


def unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def scalar_norm(x, g, eps):
    """RMS norm whose weight is one number for all coordinates."""
    return unit(x, eps) * g


def causal_conv(x, w, before=None):
    """y_t = sum_j w[:, j] x_(t - taps + 1 + j): the last column weighs the current token; `before` holds the
    taps - 1 inputs ahead of x (zeros at a sequence's start).  Returns y and the last taps - 1 inputs."""
    T, C = x.shape
    taps = w.shape[1]
    if before is None:
        before = torch.zeros(taps - 1, C, dtype=x.dtype)
    xx = torch.cat([before, x], dim=0)
    y = torch.zeros(T, C, dtype=x.dtype)
    for j in range(taps):
        y = y + xx[j: j + T] * w[:, j]
    return y, xx[xx.shape[0] - (taps - 1):]


def rotate_half(x, pos, dims, base):
    """Rotates the first `dims` entries of the last axis: entry i pairs with entry i + dims/2, by the angle
    pos * base^(-2i/dims).  x [T, heads, n], pos [T]."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = pos.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def softmax_attention(q, k, v, scale, window=0):
    """q [T, H, n], k [T, G, n], v [T, G, dv]; scale a number or one per head; causal; window > 0: key j is seen
    from position i when 0 <= i - j < window."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window > 0 else 0
        for h in range(H):
            g = h // (H // G)
            sc = scale[h] if torch.is_tensor(scale) else scale
            s = (k[lo: i + 1, g] @ q[i, h]) * sc
            out[i, h] = torch.softmax(s, dim=0) @ v[lo: i + 1, g]
    return out


def attention(h, W, p, m, eps, v_first=None, pos0=0):
    """Grouped-query attention: rotation of part of every head, then q and k over their root mean square, a
    temperature per head on the scores, optionally the values blended with those of an earlier layer.
    Returns (output, the values before blending)."""
    T = h.shape[0]
    H, G, n, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = rotate_half((h @ W[p + "q"].T).reshape(T, H, n), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((h @ W[p + "k"].T).reshape(T, G, n), pos, m["rot"]["dims"], m["rot"]["base"])
    q, k = unit(q, eps), unit(k, eps)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    own = v
    if v_first is not None:
        lam = W[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    out = softmax_attention(q, k, v, float(m["scale"]) * W[p + "temp"])
    return out.reshape(T, H * dv) @ W[p + "o"].T, own


def latent_attention(h, W, p, m, eps, pos0=0):
    """Attention over a low-rank latent: queries through a normed latent of their own; keys and values expanded
    from the normed latent c; one rotated key part shared by all heads; sliding window."""
    T = h.shape[0]
    H, n, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(pos0, pos0 + T)
    cq = unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, n + r)
    down = h @ W[p + "dkv"].T
    c = unit(down[:, :rank], eps) * W[p + "dkv.norm"]
    kr = rotate_half(down[:, None, rank:], pos, r, m["rot"]["base"])                       # [T, 1, r]
    qr = rotate_half(q[..., n:], pos, r, m["rot"]["base"])
    kn = (c @ W[p + "uk"].T).reshape(T, H, n)
    v = (c @ W[p + "uv"].T).reshape(T, H, dv)
    qq = torch.cat([q[..., :n], qr], dim=-1)
    kk = torch.cat([kn, kr.expand(T, H, r)], dim=-1)
    out = softmax_attention(qq, kk, v, float(m["scale"]), window=int(m["mask"]["size"]))
    return out.reshape(T, H * dv) @ W[p + "o"].T


def channel_delta(h, W, p, m, eps, state=None):
    """Delta rule with a decay per head and key channel.  Per head: S <- g * S (rows), u = beta (v - S^T k),
    S <- S + k u^T, o = S^T q.  state: None or (S [H, n, dv], the convolutions' earlier inputs for q, k, v);
    returns (output, state)."""
    T = h.shape[0]
    H, G, n, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    S, tails = (torch.zeros(H, n, dv, dtype=F64), [None, None, None]) if state is None else state
    outs, new_tails = [], []
    for name, tail in zip(("q", "k", "v"), tails):
        y, t = causal_conv(h @ W[p + name].T, W[p + name + ".conv"], tail)
        outs.append(silu(y))
        new_tails.append(t)
    q = outs[0].reshape(T, G, n)
    k = outs[1].reshape(T, G, n)
    v = outs[2].reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + KEY_EPS) * n ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + KEY_EPS)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                                  # [T, H]
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    rate = torch.exp(W[p + "A_log"]).repeat_interleave(n)
    decay = torch.exp(-rate * torch.nn.functional.softplus(z)).reshape(T, H, n)
    o = torch.zeros(T, H, dv, dtype=F64)
    S = S.clone()
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            o[t, hd] = S[hd].T @ q[t, g]
    o = unit(o, eps) * W[p + "norm"]
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ W[p + "o"].T, (S, new_tails)


def dense_ff(h, W, p):
    return gelu_tanh(h @ W[p + "up"].T) @ W[p + "down"].T


def routed_ff(h, W, p, f):
    """Every token uses the `top` experts with the largest router logits, weighted by the softmax over those logits."""
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ W[p + "router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = torch.topk(z[t], top).indices
        wts = torch.softmax(z[t, chosen], dim=0)
        for e, wt in zip(chosen.tolist(), wts):
            q = f"{p}e{e}."
            out[t] = out[t] + wt * ((silu(h[t] @ W[q + "gate"].T) * (h[t] @ W[q + "up"].T)) @ W[q + "down"].T)
    return out


def forward(cfg, W, tokens, taps=None):
    """Logits [T, vocab] of one whole sequence; taps, if a list, receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = x + causal_conv(x, W[p + "canon1"])[0]
        if layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, own = attention(h, W, p + "mix.", m, eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = own
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, W, p + "mix.", m, eps)
        elif layer["type"] == "channel_delta":
            y, _ = channel_delta(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + scalar_norm(y, W[p + "norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            y = dense_ff(x, W, p + "mlp.") if f["kind"] == "dense" else routed_ff(x, W, p + "mlp.", f)
            x = x + scalar_norm(y, W[p + "norm2"], eps)
        if taps is not None:
            taps.append(x.clone())
    return scalar_norm(x, W["final.norm"], eps) @ W["head"].T
