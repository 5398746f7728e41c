"""Mixers whose state per request is a matrix per head that decays channel by channel: gated linear attention, the
generalized delta rule and the delta rule that removes from the decayed state.  Both are the recurrence S = diag(w) S - (a u)(u^T S) + k v^T, y = S^T q (csrc/channel_scan.cu; the
removal term only for the delta rule).  The state is float32, lives in the cache manager's request slots (zeroed at
admission) and is carried from step to step, so a prompt may be cut anywhere.  Decays, removal rates, unit keys, the
recurrence and the norms behind it are float32 on every path; the projections leave float32 sums."""
from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec
from ..csrc import ops
from .registry import register_part
from .shared_io import SharedIOMixer, stack_rows

_FORMS = {"pow_sigmoid": ops.GATE_POW_SIGMOID, "exp_neg_sigmoid": ops.GATE_EXP_NEG_SIGMOID}


class _ChannelDecay:
    """w = g(W2 f(W1 h) + bias) per head and key channel; W1's rows ride in the mixer's input product."""

    def __init__(self, spec, source):
        if spec.form not in _FORMS:
            raise ValueError(f"unknown decay form '{spec.form}' (known: {', '.join(_FORMS)})")
        self.kind = _FORMS[spec.form]
        # sigmoid(z)^(1/tau) = exp(log sigmoid(z) / tau);  exp(-rate sigmoid(z))
        self.param = 1.0 / float(spec.param) if spec.form == "pow_sigmoid" else float(spec.param)
        self.inner_tanh = bool(spec.inner_tanh)
        self.rank = int(spec.rank)
        self.down = source.get(spec.down)
        self.up = source.get(spec.up, dtype=torch.float32).t().contiguous()     # [rank, channels]; small: float32 on every path
        self.bias = source.get(spec.bias, dtype=torch.float32)

    def apply(self, low_rank):
        out = torch.empty((low_rank.shape[0], self.up.shape[1]), device=low_rank.device, dtype=torch.float32)
        ops.channel_gates(out, low_rank, self.up, self.bias, self.inner_tanh, self.kind, self.param)
        return out


class GLA(SharedIOMixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.dk, self.dv = spec.num_heads, spec.key_dim, spec.value_dim
        self.decay = _ChannelDecay(spec.decay, source)
        self._w_in = stack_rows([source.get(n) for n in (spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj)] + [self.decay.down])
        self._w_out = source.get(spec.o_proj)
        self.decay.down = None
        self.in_rows = 2 * self.H * self.dk + 2 * self.H * self.dv + self.decay.rank
        self.out_cols = self.H * self.dv
        self.norm = source.get(spec.norm, dtype=torch.float32).repeat(self.H).contiguous()     # one weight for all heads

    def cache_spec(self):
        return FixedStateSpec((ops.channel_scan_state_floats(self.H, self.dk, self.dv),), "float32")

    def in_weights(self):
        return self._w_in

    def out_weight(self):
        return self._w_out

    def release_weights(self):
        self._w_in = self._w_out = None

    def heads_out(self, proj, ctx, cache, out, factor=1.0):
        H, dk, dv = self.H, self.dk, self.dv
        a, b, c, d = H * dk, 2 * H * dk, 2 * H * dk + H * dv, 2 * H * dk + 2 * H * dv
        w = self.decay.apply(proj[:, d: d + self.decay.rank])
        y = torch.empty((proj.shape[0], H * dv), device=proj.device, dtype=torch.float32)
        ops.channel_scan(y, proj[:, :a], proj[:, a:b], proj[:, b:c], w, None, None, dk ** -0.5, cache.tensor, ctx, H, dk, dv)
        ops.head_norm_gate(out, y, proj[:, c:d], self.norm, H, self.spec.eps, ops.HEAD_GATE_SILU, factor)


class DeltaRule(SharedIOMixer):
    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.n = spec.num_heads, spec.head_dim
        self.decay = _ChannelDecay(spec.decay, source)
        names = (spec.r_proj, spec.k_proj, spec.v_proj, spec.gate_proj, spec.a_proj)
        self._w_in = stack_rows([source.get(n) for n in names] + [self.decay.down])
        self._w_out = source.get(spec.o_proj)
        self.decay.down = None
        self.in_rows = 5 * self.H * self.n + self.decay.rank
        self.out_cols = self.H * self.n
        self.a_bias = source.get(spec.a_proj + ".b", dtype=torch.float32)
        self.norm = source.get(spec.norm, dtype=torch.float32)

    def cache_spec(self):
        return FixedStateSpec((ops.channel_scan_state_floats(self.H, self.n, self.n),), "float32")

    def in_weights(self):
        return self._w_in

    def out_weight(self):
        return self._w_out

    def release_weights(self):
        self._w_in = self._w_out = None

    def heads_out(self, proj, ctx, cache, out, factor=1.0):
        H, n = self.H, self.n
        W = H * n
        T = proj.shape[0]
        w = self.decay.apply(proj[:, 5 * W: 5 * W + self.decay.rank])
        u = torch.empty((T, W), device=proj.device, dtype=torch.float32)
        au = torch.empty_like(u)
        ops.unit_keys(u, au, proj[:, W: 2 * W], proj[:, 4 * W: 5 * W], self.a_bias, H, n, self.spec.key_eps)
        y = torch.empty((T, W), device=proj.device, dtype=torch.float32)
        ops.channel_scan(y, proj[:, :W], proj[:, W: 2 * W], proj[:, 2 * W: 3 * W], w, au, u, 1.0, cache.tensor, ctx, H, n, n)
        ops.head_norm_gate(out, y, proj[:, 3 * W: 4 * W], self.norm, H, self.spec.eps, ops.HEAD_GATE_SIGMOID, factor)


class ChannelDelta(SharedIOMixer):
    """Delta rule with a decay per head and key channel whose removal reads the decayed state: S' = diag(g) S,
    S = S' + k (beta (v - S'^T k))^T, o = S^T q.  In the scan's terms (both first terms from the old state) the decay is g, the
    removal's reading vector g * k and its writing vector, like the written key, beta k (`delta_operands`).  q, k and v pass a
    short convolution with SiLU first (float32, from the product's float32 sums; its last inputs are a second state slot);
    query/key heads may serve several value heads."""

    def __init__(self, spec, source, rt):
        self.spec, self.rt = spec, rt
        self.H, self.G, self.dk, self.dv = spec.num_heads, spec.num_kv_heads, spec.key_dim, spec.value_dim
        if self.H % self.G:
            raise ValueError(f"num_heads {self.H} is not a multiple of num_kv_heads {self.G}")
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        names = (spec.q_proj, spec.k_proj, spec.v_proj, spec.beta_proj, spec.a_down, spec.gate_down)
        self._w_in = stack_rows([source.get(n) for n in names])
        self._w_out = source.get(spec.o_proj)
        self.conv_ch = 2 * G * dk + H * dv
        self.in_rows = self.conv_ch + H + spec.decay_rank + spec.gate_rank
        self.out_cols = H * dv
        self.taps = int(spec.conv_taps)
        self.conv_w = torch.cat([source.get(n + ".conv", dtype=torch.float32) for n in (spec.q_proj, spec.k_proj, spec.v_proj)], dim=0).contiguous()
        if tuple(self.conv_w.shape) != (self.conv_ch, self.taps):
            raise ValueError(f"the convolutions' weights have shape {tuple(self.conv_w.shape)}, not {(self.conv_ch, self.taps)}")
        # the low-rank up matrices are small: float32 and transposed on every path
        self.a_up = source.get(spec.a_up, dtype=torch.float32).t().contiguous()                 # [decay_rank, H * dk]
        self.dt_bias = source.get(spec.dt_bias, dtype=torch.float32).contiguous()
        self.rate = torch.exp(source.get(spec.a_log, dtype=torch.float32).double()).float().repeat_interleave(dk).contiguous()
        self.g_up = source.get(spec.gate_up, dtype=torch.float32).t().contiguous()              # [gate_rank, H * dv]
        self.norm = source.get(spec.norm, dtype=torch.float32).repeat(H).contiguous()           # one weight for all heads

    def cache_spec(self):
        return (FixedStateSpec((ops.channel_scan_state_floats(self.H, self.dk, self.dv),), "float32"),
                FixedStateSpec((max(1, (self.taps - 1) * self.conv_ch),), "float32"))

    def in_weights(self):
        return self._w_in

    def out_weight(self):
        return self._w_out

    def release_weights(self):
        self._w_in = self._w_out = None

    def heads_out(self, proj, ctx, cache, out, factor=1.0):
        H, G, dk, dv, C = self.H, self.G, self.dk, self.dv, self.conv_ch
        T, dev = proj.shape[0], proj.device
        b0 = C
        a0 = b0 + H
        g0 = a0 + self.spec.decay_rank
        scan_state, conv_state = cache.views[0].tensor, cache.views[1].tensor
        conv = torch.empty((T, C), device=dev, dtype=torch.float32)
        ops.conv_state(conv, proj[:, :C], self.conv_w, None, conv_state, ctx, act=True)
        decay = torch.empty((T, H * dk), device=dev, dtype=torch.float32)
        ops.channel_gates(decay, proj[:, a0:g0], self.a_up, self.dt_bias, False, ops.GATE_EXP_NEG_SOFTPLUS, 0.0, rate=self.rate)
        gate = torch.empty((T, H * dv), device=dev, dtype=torch.float32)
        ops.channel_gates(gate, proj[:, g0: g0 + self.spec.gate_rank], self.g_up, None, False, ops.GATE_LINEAR, 0.0)
        qh = torch.empty((T, H * dk), device=dev, dtype=torch.float32)
        kb, ug = torch.empty_like(qh), torch.empty_like(qh)
        ops.delta_operands(qh, kb, ug, conv[:, : G * dk], conv[:, G * dk: 2 * G * dk], proj[:, b0:a0], decay, H, G, dk, self.spec.key_eps,
                           dk ** -0.5)
        y = torch.empty((T, H * dv), device=dev, dtype=torch.float32)
        ops.channel_scan(y, qh, kb, conv[:, 2 * G * dk:], decay, kb, ug, 1.0, scan_state, ctx, H, dk, dv)
        ops.head_norm_gate(out, y, gate, self.norm, H, self.spec.eps, ops.HEAD_GATE_SIGMOID, factor)


register_part("mixer", "channel_delta", ChannelDelta)
register_part("mixer", "gla", GLA)
register_part("mixer", "delta_rule", DeltaRule)
