"""Mixers whose state per request is a matrix per head that decays channel by channel: gated linear attention and the
generalized delta rule.  Both are the recurrence S = diag(w) S - (a u)(u^T S) + k v^T, y = S^T q (csrc/channel_scan.cu; the
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


register_part("mixer", "gla", GLA)
register_part("mixer", "delta_rule", DeltaRule)
