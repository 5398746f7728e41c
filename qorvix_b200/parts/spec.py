"""Layer descriptions as data.  An architecture turns its configuration into a ModelSpec: a
list of LayerSpecs (each naming its mixer, feed-forward, norms and arrangement, with all
sizes and constants as fields) and the order in which layers run.  Parts are built from
these specs through the registry in parts/registry.py; no part knows which model it is in.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

# tensor table entries: name -> (shape, kind) with kind in {"matrix", "norm", "normal:<mean>:<std>"}
# (how random weights are drawn)
TensorTable = Dict[str, Tuple[Tuple[int, ...], str]]


@dataclass(frozen=True)
class YarnScaling:
    """Stretching of rotary frequencies for contexts beyond the trained length: pairs whose waves turn more
    than `fast` times over `original` positions keep their frequency, those that turn fewer than `slow`
    times are slowed by `factor`, those between blend linearly over the pair index; cosine and sine are
    both multiplied by 0.1 ln(factor) + 1."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding.  `rotary_dim` leading dims of each head are rotated in
    split-half pairs (i, i + rotary_dim/2); the reference's NeoX mode (runtime/src/ops.cpp:141-146)."""
    head_dim: int
    rotary_dim: int
    theta: float
    scaling: Optional[object] = None          # config.RopeScaling (llama3 rule), YarnScaling, or None
    kind: str = "rotary"
    pairing: str = "split_half"               # "interleaved": entry 2i is paired with 2i+1 (mixers that rotate themselves)

    def tensors(self) -> TensorTable:
        return {}


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float
    weight: str
    kind: str = "rmsnorm"
    one_plus: bool = False                    # the stored weight lies around zero: the rows are scaled by 1 + w
    scalar: bool = False                      # the stored weight is one number for all coordinates

    def tensors(self) -> TensorTable:
        return {self.weight: (() if self.scalar else (self.size,), "normal:0:0.1" if self.one_plus else "norm")}


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention with its four projections."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    position: Optional[object] = None         # a position-encoding spec, or None
    window: int = 0                           # 0: all keys; n: the last n keys
    kv_from: Optional[int] = None             # read this layer's cache instead of keeping one
    kind: str = "attention"

    def tensors(self) -> TensorTable:
        t = {self.q_proj: ((self.num_heads * self.head_dim, self.hidden_size), "matrix"),
             self.o_proj: ((self.hidden_size, self.num_heads * self.head_dim), "matrix")}
        if self.kv_from is None:
            t[self.k_proj] = ((self.num_kv_heads * self.head_dim, self.hidden_size), "matrix")
            t[self.v_proj] = ((self.num_kv_heads * self.head_dim, self.hidden_size), "matrix")
        if self.position is not None:
            t.update(self.position.tensors())       # a position encoding may have weights of its own
        return t


@dataclass(frozen=True)
class SwiGLUSpec:
    """Dense gated feed-forward: down(act(gate x) * up x); act 'silu' or 'gelu_tanh' (the tanh form of GELU)."""
    hidden_size: int
    intermediate_size: int
    gate_proj: str
    up_proj: str
    down_proj: str
    kind: str = "swiglu"
    activation: str = "silu"

    def tensors(self) -> TensorTable:
        return {self.gate_proj: ((self.intermediate_size, self.hidden_size), "matrix"),
                self.up_proj: ((self.intermediate_size, self.hidden_size), "matrix"),
                self.down_proj: ((self.hidden_size, self.intermediate_size), "matrix")}


@dataclass(frozen=True)
class BigramEmbeddingSpec:
    """Token embedding plus a row of a second table chosen by a hash of (previous token, token):
    (prev * mul_prev + token * mul_cur) mod buckets; a request's first token takes row `buckets`."""
    vocab_size: int
    hidden_size: int
    table: str
    pair_table: str
    buckets: int
    mul_prev: int
    mul_cur: int
    kind: str = "bigram_embedding"

    def tensors(self) -> TensorTable:
        return {self.table: ((self.vocab_size, self.hidden_size), "matrix"),
                self.pair_table: ((self.buckets + 1, self.hidden_size), "matrix")}


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are expanded from a cached low-rank latent; each head's
    query and key have `head_dim` unrotated entries followed by `rot_dim` rotated ones, the rotated key
    part being one vector shared by all heads; optionally a sigmoid gate multiplies the heads' outputs
    (gate_proj), and optionally the queries pass a latent of their own: c = rmsnorm(q_down x) * q_norm,
    q = q_proj c with q_proj [heads * (head_dim + rot_dim), q_rank]."""
    hidden_size: int
    num_heads: int
    head_dim: int                 # unrotated query/key entries per head
    rot_dim: int                  # rotated query/key entries per head
    value_dim: int
    kv_rank: int
    scale: float
    eps: float                    # of the latents' RMS norms
    position: object              # RotarySpec over rot_dim; pairing 'interleaved' or 'split_half'
    q_proj: str
    kv_down: str                  # [kv_rank + rot_dim, hidden]
    kv_norm: str
    k_up: str                     # [heads * head_dim, kv_rank]
    v_up: str                     # [heads * value_dim, kv_rank]
    gate_proj: Optional[str]
    o_proj: str
    window: int = 0
    kind: str = "latent_attention"
    q_rank: int = 0               # > 0: the queries' latent size
    q_down: Optional[str] = None  # [q_rank, hidden]
    q_norm: Optional[str] = None  # [q_rank]

    def tensors(self) -> TensorTable:
        H, d = self.num_heads, self.hidden_size
        t = {self.kv_down: ((self.kv_rank + self.rot_dim, d), "matrix"),
             self.kv_norm: ((self.kv_rank,), "norm"),
             self.k_up: ((H * self.head_dim, self.kv_rank), "matrix"),
             self.v_up: ((H * self.value_dim, self.kv_rank), "matrix"),
             self.o_proj: ((d, H * self.value_dim), "matrix")}
        if self.q_rank:
            t[self.q_down] = ((self.q_rank, d), "matrix")
            t[self.q_norm] = ((self.q_rank,), "norm")
            t[self.q_proj] = ((H * (self.head_dim + self.rot_dim), self.q_rank), "matrix")
        else:
            t[self.q_proj] = ((H * (self.head_dim + self.rot_dim), d), "matrix")
        if self.gate_proj is not None:
            t[self.gate_proj] = ((H * self.value_dim, d), "matrix")
        return t


@dataclass(frozen=True)
class MLSTMSpec:
    """Matrix-memory LSTM: per head a key_dim x value_dim state with exponential input and forget gates
    (pre-activations soft-limited to +-gate_cap) and a running maximum for stability; heads are
    unit-normed, weighted and gated with a sigmoid before the output projection."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    i_proj: str
    i_bias: str
    f_proj: str
    f_bias: str
    norm: str
    o_proj: str
    kind: str = "mlstm"

    def tensors(self) -> TensorTable:
        H, d, dk, dv = self.num_heads, self.hidden_size, self.key_dim, self.value_dim
        return {self.q_proj: ((H * dk, d), "matrix"), self.k_proj: ((H * dk, d), "matrix"),
                self.v_proj: ((H * dv, d), "matrix"), self.gate_proj: ((H * dv, d), "matrix"),
                self.o_proj: ((d, H * dv), "matrix"), self.norm: ((H * dv,), "norm"),
                self.i_proj: ((H, d), "matrix"), self.i_bias: ((H,), "normal:0:0.5"),
                self.f_proj: ((H, d), "matrix"), self.f_bias: ((H,), "normal:3:0.5")}


@dataclass(frozen=True)
class Mamba2Spec:
    """Selective state space with a scalar decay per head (state_dim x value_dim state), a short causal
    convolution over x, B and C ahead of it and a SiLU gate followed by an RMS norm in equal parts behind."""
    hidden_size: int
    num_heads: int
    value_dim: int
    state_dim: int
    groups: int
    conv_taps: int
    norm_groups: int
    eps: float
    in_proj: str                  # rows [z | x | B | C | dt]
    conv_weight: str
    conv_bias: str
    dt_bias: str
    a_log: str
    skip: str
    norm: str
    o_proj: str
    kind: str = "mamba2"

    @property
    def inner(self) -> int:
        return self.num_heads * self.value_dim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state_dim

    def tensors(self) -> TensorTable:
        H, d = self.num_heads, self.hidden_size
        return {self.in_proj: ((self.inner + self.conv_channels + H, d), "matrix"),
                self.conv_weight: ((self.conv_channels, self.conv_taps), "normal:0:0.3"),
                self.conv_bias: ((self.conv_channels,), "normal:0:0.1"),
                self.dt_bias: ((H,), "normal:-1:0.5"), self.a_log: ((H,), "normal:0:0.5"),
                self.skip: ((H,), "norm"), self.norm: ((self.inner,), "norm"),
                self.o_proj: ((d, self.inner), "matrix")}


@dataclass(frozen=True)
class MoESpec:
    """Routed feed-forward: `experts` gated feed-forwards of which each token uses `top`, weighted by the
    softmax over the chosen router logits; optionally a shared gated feed-forward for every token, scaled
    by the sigmoid of one number per token."""
    hidden_size: int
    experts: int
    top: int
    expert_ff: int
    router: str
    expert_prefix: str            # expert e's matrices are <prefix><e>.gate / .up / .down
    shared: Optional[SwiGLUSpec] = None
    shared_gate: Optional[str] = None
    kind: str = "moe"

    def expert_names(self, e: int):
        p = f"{self.expert_prefix}{e}."
        return p + "gate", p + "up", p + "down"

    def tensors(self) -> TensorTable:
        t: TensorTable = {self.router: ((self.experts, self.hidden_size), "matrix")}
        for e in range(self.experts):
            g, u, dn = self.expert_names(e)
            t[g] = ((self.expert_ff, self.hidden_size), "matrix")
            t[u] = ((self.expert_ff, self.hidden_size), "matrix")
            t[dn] = ((self.hidden_size, self.expert_ff), "matrix")
        if self.shared is not None:
            t.update(self.shared.tensors())
            t[self.shared_gate] = ((1, self.hidden_size), "matrix")
        return t


@dataclass(frozen=True)
class DiffAttentionSpec:
    """Causal grouped-query differential attention: every head has two query/key maps of `head_dim` entries
    each over the head's one set of values; the head's output is map 1 minus `lam` times map 2 (lam =
    exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number a layer), divided by its root mean square over
    `value_dim` and scaled by 1 - diff.  q, k and v have biases; each map of q and k is RMS-normed over
    head_dim with a weight shared by heads and maps, then rotated."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int                 # entries of one map of a head's query or key
    value_dim: int
    scale: float
    diff: float
    eps: float
    q_proj: str                   # [heads * 2 * head_dim, hidden], head by head [map 1 | map 2]; bias: name + ".b"
    k_proj: str
    v_proj: str
    q_norm: str
    k_norm: str
    lam_q1: str
    lam_k1: str
    lam_q2: str
    lam_k2: str
    o_proj: str
    position: Optional[object] = None
    window: int = 0
    kind: str = "diff_attention"

    def tensors(self) -> TensorTable:
        H, G, n, dv, d = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.hidden_size
        t: TensorTable = {self.q_proj: ((H * 2 * n, d), "matrix"), self.q_proj + ".b": ((H * 2 * n,), "normal:0:0.02"),
                          self.k_proj: ((G * 2 * n, d), "matrix"), self.k_proj + ".b": ((G * 2 * n,), "normal:0:0.02"),
                          self.v_proj: ((G * dv, d), "matrix"), self.v_proj + ".b": ((G * dv,), "normal:0:0.02"),
                          self.q_norm: ((n,), "norm"), self.k_norm: ((n,), "norm"),
                          self.o_proj: ((d, H * dv), "matrix")}
        for name in (self.lam_q1, self.lam_k1, self.lam_q2, self.lam_k2):
            t[name] = ((n,), "normal:0:0.1")
        if self.position is not None:
            t.update(self.position.tensors())
        return t


@dataclass(frozen=True)
class ActMLPSpec:
    """Ungated feed-forward: down(act(up x)), no biases; act 'relu2' is the square of relu, 'gelu_tanh' the tanh form of GELU."""
    hidden_size: int
    intermediate_size: int
    up_proj: str
    down_proj: str
    activation: str = "relu2"
    kind: str = "act_mlp"

    def tensors(self) -> TensorTable:
        return {self.up_proj: ((self.intermediate_size, self.hidden_size), "matrix"),
                self.down_proj: ((self.hidden_size, self.intermediate_size), "matrix")}


@dataclass(frozen=True)
class TableMoESpec:
    """Small ungated experts (down(act(up x))) chosen without a router: row `token id` of an integer table
    [vocab, top] lists the token's experts (the entries of a row differ), each weighted 1/top; optionally a
    shared expert of the same form for every token, added as it is."""
    hidden_size: int
    vocab_size: int
    experts: int
    top: int
    expert_ff: int
    table: str
    expert_prefix: str            # expert e's matrices are <prefix><e>.up / .down
    shared: Optional[ActMLPSpec] = None
    activation: str = "relu2"
    kind: str = "table_moe"

    def expert_names(self, e: int):
        p = f"{self.expert_prefix}{e}."
        return p + "up", p + "down"

    def tensors(self) -> TensorTable:
        t: TensorTable = {self.table: ((self.vocab_size, self.top), f"choices:{self.experts}")}
        for e in range(self.experts):
            u, dn = self.expert_names(e)
            t[u] = ((self.expert_ff, self.hidden_size), "matrix")
            t[dn] = ((self.hidden_size, self.expert_ff), "matrix")
        if self.shared is not None:
            t.update(self.shared.tensors())
        return t


@dataclass(frozen=True)
class LoopSpec:
    """Re-entry of the residual stream at the start of each pass over a stretch of layers that runs several
    times: before run `first_runs[t]` of the execution order, x = W [x ; x0] + step[t], with x0 the embedding's
    output, W [width, 2 width] and step [passes, width]."""
    first_runs: Tuple[int, ...]
    in_proj: str
    step: str
    hidden_size: int
    kind: str = "loop_entry"

    def tensors(self) -> TensorTable:
        return {self.in_proj: ((self.hidden_size, 2 * self.hidden_size), "matrix"),
                self.step: ((len(self.first_runs), self.hidden_size), "normal:0:0.02")}


@dataclass(frozen=True)
class TanhNormSpec:
    """Norm without statistics: tanh(alpha x) w + b with a scalar alpha, stored beside the weight as <weight>.alpha and <weight>.b."""
    size: int
    weight: str
    kind: str = "tanh_norm"

    @property
    def bias(self) -> str:
        return self.weight + ".b"

    @property
    def alpha(self) -> str:
        return self.weight + ".alpha"

    def tensors(self) -> TensorTable:
        return {self.weight: ((self.size,), "norm"), self.bias: ((self.size,), "normal:0:0.1"), self.alpha: ((), "normal:0.7:0.1")}


@dataclass(frozen=True)
class PositionedEmbeddingSpec:
    """Token row plus the row of a learned position table (times pos_scale), then an optional norm of the sum."""
    vocab_size: int
    hidden_size: int
    positions: int
    table: str
    pos_table: str
    norm: Optional[object] = None             # a TanhNormSpec, or None
    pos_scale: float = 1.0
    kind: str = "positioned_embedding"

    def tensors(self) -> TensorTable:
        t: TensorTable = {self.table: ((self.vocab_size, self.hidden_size), "matrix"),
                          self.pos_table: ((self.positions, self.hidden_size), "matrix")}
        if self.norm is not None:
            t.update(self.norm.tensors())
        return t


@dataclass(frozen=True)
class ChannelDecaySpec:
    """A decay per head and key channel from a low-rank product: z = W2 f(W1 h) + bias, f the identity or tanh, then
    'pow_sigmoid': sigmoid(z)^(1/tau), or 'exp_neg_sigmoid': exp(-rate * sigmoid(z))."""
    rank: int
    down: str                     # W1 [rank, hidden]
    up: str                       # W2 [heads * key_dim, rank]
    bias: str                     # [heads * key_dim]
    form: str                     # "pow_sigmoid" | "exp_neg_sigmoid"
    param: float                  # tau | rate
    inner_tanh: bool = False


@dataclass(frozen=True)
class GLASpec:
    """Gated linear attention: per head a key_dim x value_dim state, S = diag(decay) S + k v^T, o = S^T q with q scaled by
    key_dim^(-1/2); each head's o is RMS-normed over value_dim with a weight shared by the heads, gated by SiLU of a
    projection and projected."""
    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    decay: ChannelDecaySpec
    norm: str                     # [value_dim]
    o_proj: str
    kind: str = "gla"

    def tensors(self) -> TensorTable:
        H, d, dk, dv, dc = self.num_heads, self.hidden_size, self.key_dim, self.value_dim, self.decay
        return {self.q_proj: ((H * dk, d), "matrix"), self.k_proj: ((H * dk, d), "matrix"), self.v_proj: ((H * dv, d), "matrix"),
                self.gate_proj: ((H * dv, d), "matrix"), self.o_proj: ((d, H * dv), "matrix"), self.norm: ((dv,), "norm"),
                dc.down: ((dc.rank, d), "matrix"), dc.up: ((H * dk, dc.rank), "normal:0:0.3"), dc.bias: ((H * dk,), "normal:2:1")}


@dataclass(frozen=True)
class DeltaRuleSpec:
    """Generalized delta rule: per head a dim x dim state, S = diag(w) S - (a u)(u^T S) + k v^T with u the key over its
    length (key_eps under the root) and a = sigmoid(W_a h + b) the removal rate per key channel, both first terms reading
    the old state; o = S^T r is divided by its root mean square per head, weighted over all heads' entries, gated by
    the sigmoid of a projection and projected."""
    hidden_size: int
    num_heads: int
    head_dim: int
    eps: float
    r_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    a_proj: str                   # bias: name + ".b"
    decay: ChannelDecaySpec
    norm: str                     # [heads * head_dim]
    o_proj: str
    key_eps: float = 1e-6
    kind: str = "delta_rule"

    def tensors(self) -> TensorTable:
        H, d, n, dc = self.num_heads, self.hidden_size, self.head_dim, self.decay
        t: TensorTable = {name: ((H * n, d), "matrix") for name in (self.r_proj, self.k_proj, self.v_proj, self.gate_proj, self.a_proj)}
        t.update({self.a_proj + ".b": ((H * n,), "normal:0:0.5"), self.norm: ((H * n,), "norm"), self.o_proj: ((d, H * n), "matrix"),
                  dc.down: ((dc.rank, d), "matrix"), dc.up: ((H * n, dc.rank), "normal:0:0.3"), dc.bias: ((H * n,), "normal:0:1")})
        return t


@dataclass(frozen=True)
class BiasedAttentionSpec:
    """Causal grouped-query softmax attention without rotation.  Positions enter through a learned bias on the scores,
    bias[bucket(i - j), head] with `bias_rows` rows (one per distance below half the rows, the rest spaced evenly in the
    logarithm of the distance up to bias_max), and through a temperature on the query, 1 + temp_coef ln(floor((p + 1) /
    temp_every) + 1).  q, k, v and the output projection have biases (name + ".b"); the heads' outputs are multiplied by
    the sigmoid of a projection of the mixer's input."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    bias_rows: int
    bias_max: float
    temp_coef: float
    temp_every: int
    q_proj: str
    k_proj: str
    v_proj: str
    gate_proj: str
    rel_bias: str
    o_proj: str
    kind: str = "biased_attention"

    def tensors(self) -> TensorTable:
        H, G, n, dv, d = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.hidden_size
        return {self.q_proj: ((H * n, d), "matrix"), self.q_proj + ".b": ((H * n,), "normal:0:0.02"),
                self.k_proj: ((G * n, d), "matrix"), self.k_proj + ".b": ((G * n,), "normal:0:0.02"),
                self.v_proj: ((G * dv, d), "matrix"), self.v_proj + ".b": ((G * dv,), "normal:0:0.02"),
                self.gate_proj: ((H * dv, d), "matrix"), self.rel_bias: ((self.bias_rows, H), "normal:0:0.5"),
                self.o_proj: ((d, H * dv), "matrix"), self.o_proj + ".b": ((d,), "normal:0:0.02")}


@dataclass(frozen=True)
class RotNormAttentionSpec:
    """Causal grouped-query softmax attention whose queries and keys are rotated over their first rotary_dim entries
    (`position`, a RotarySpec in split halves, or None) and then divided by their root mean square over the head (no
    weight; eps under the root); the score is (q . k) * scale * head_temp[h] (head_temp: a number per head, or None).
    Key and value sizes are unrelated.  Values may be shared between layers: the layer with v_share_role 'source'
    publishes its values of the step's tokens under the name v_share, a layer with role 'blend' replaces its values
    by (1 - lam) v + lam v_source before they are cached, lam being the number stored as v_blend."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    value_dim: int
    scale: float
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    position: Optional[object] = None
    head_temp: Optional[str] = None
    v_share: Optional[str] = None
    v_share_role: Optional[str] = None        # 'source' | 'blend' | None
    v_blend: Optional[str] = None             # a number; stored in every sharing layer, used by 'blend' layers
    kind: str = "rot_norm_attention"

    def tensors(self) -> TensorTable:
        H, G, n, dv, d = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.hidden_size
        t: TensorTable = {self.q_proj: ((H * n, d), "matrix"), self.k_proj: ((G * n, d), "matrix"), self.v_proj: ((G * dv, d), "matrix"),
                          self.o_proj: ((d, H * dv), "matrix")}
        if self.head_temp is not None:
            t[self.head_temp] = ((H,), "normal:1:0.2")
        if self.v_blend is not None:
            t[self.v_blend] = ((), "normal:0.4:0.1")
        if self.position is not None:
            t.update(self.position.tensors())
        return t


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """Delta rule with a decay per head and key channel whose removal reads the decayed state.  Per head (head h reads
    query/key group h // (heads / kv_heads)): S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    q, k, v pass a short causal convolution per channel (<name>.conv, [channels, taps], the current token's tap last) and SiLU;
    q and k are then unit vectors per head (key_eps under the root), q times key_dim^(-1/2); beta = sigmoid(W_b x);
    g = exp(-exp(a_log[h]) softplus(W_a2 W_a1 x + dt_bias)); o is divided by its root mean square per head, weighted
    (norm, [value_dim], shared by the heads) and multiplied by sigmoid(W_g2 W_g1 x)."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    decay_rank: int               # rows of a_down
    gate_rank: int                # rows of gate_down
    eps: float
    q_proj: str
    k_proj: str
    v_proj: str
    beta_proj: str
    a_down: str
    a_up: str
    dt_bias: str
    a_log: str
    gate_down: str
    gate_up: str
    norm: str
    o_proj: str
    key_eps: float = 1e-6
    kind: str = "channel_delta"

    def tensors(self) -> TensorTable:
        H, G, dk, dv, d = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim, self.hidden_size
        t: TensorTable = {self.q_proj: ((G * dk, d), "matrix"), self.k_proj: ((G * dk, d), "matrix"), self.v_proj: ((H * dv, d), "matrix"),
                          self.beta_proj: ((H, d), "matrix"), self.a_down: ((self.decay_rank, d), "matrix"),
                          self.a_up: ((H * dk, self.decay_rank), "normal:0:0.3"), self.dt_bias: ((H * dk,), "normal:-1:1"),
                          self.a_log: ((H,), "normal:-1:0.5"), self.gate_down: ((self.gate_rank, d), "matrix"),
                          self.gate_up: ((H * dv, self.gate_rank), "normal:0:0.3"), self.norm: ((dv,), "norm"),
                          self.o_proj: ((d, H * dv), "matrix")}
        for name, ch in ((self.q_proj, G * dk), (self.k_proj, G * dk), (self.v_proj, H * dv)):
            t[name + ".conv"] = ((ch, self.conv_taps), "normal:0:0.4")
        return t


@dataclass(frozen=True)
class ConvInputSpec:
    """A mixer whose input h first becomes h + conv(h), a causal convolution over time per channel without bias or activation
    (weight [hidden, taps], the current token's tap last, zeros before a sequence's start); the last taps - 1 inputs are
    part of the request's state."""
    inner: object
    hidden_size: int
    taps: int
    weight: str
    kind: str = "conv_input"

    def tensors(self) -> TensorTable:
        t = dict(self.inner.tensors())
        t[self.weight] = ((self.hidden_size, self.taps), "normal:0:0.3")
        return t


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; the result is left_scale * left + right_scale * right."""
    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "side_by_side"

    def tensors(self) -> TensorTable:
        t = dict(self.left.tensors())
        t.update(self.right.tensors())
        return t


@dataclass(frozen=True)
class DepthAverageSpec:
    """After run i of the execution order the stream becomes a weighted sum of the embedding's output and the results of
    runs 0..i (each taken before this averaging): weights[i] names a vector of i + 2 factors."""
    weights: Tuple[str, ...]
    hidden_size: int
    kind: str = "depth_average"

    def tensors(self) -> TensorTable:
        return {name: ((i + 2,), "normal:0.3:0.2") for i, name in enumerate(self.weights)}


@dataclass(frozen=True)
class LayerSpec:
    """One block: which parts and how they are arranged ('pre_norm': x += mixer(norm(x));
    x += ffn(norm(x)), the reference's order, runtime/src/text_model.cpp:146-168; 'parallel':
    x += mixer(norm_a(x)) + ffn(norm_b(x)), both reading the stream as it enters; a parallel block whose
    ffn_norm is None while it has a feed-forward gives both parts the one normed input).
    mixer_scale / ffn_scale name per-feature factors of the two parts' outputs ("layer scale") and
    residual_mult multiplies what the block adds to the stream; the parallel block applies them.
    'gated_pre_norm' is 'pre_norm' with each part's output multiplied by sigmoid(W h + b), h being the part's input:
    mixer_gate / ffn_gate name W [width, width], the bias is name + ".b".
    'post_norm': x += mixer_norm(mixer(x)); x += ffn_norm(feed_forward(x)): the parts read the stream itself and the norms
    sit on their outputs."""
    mixer: object
    feed_forward: object
    mixer_norm: object
    ffn_norm: object
    block: str = "pre_norm"
    mixer_scale: Optional[str] = None
    ffn_scale: Optional[str] = None
    residual_mult: float = 1.0
    mixer_gate: Optional[str] = None
    ffn_gate: Optional[str] = None

    def tensors(self) -> TensorTable:
        t: TensorTable = {}
        for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward):
            if part is not None:
                t.update(part.tensors())
        width = getattr(self.mixer_norm, "size", None)
        for name in (self.mixer_gate, self.ffn_gate):
            if name is not None:
                t[name] = ((width, width), "matrix")
                t[name + ".b"] = ((width,), "normal:0:0.5")
        for name in (self.mixer_scale, self.ffn_scale):
            if name is not None:
                t[name] = ((width,), "norm")
        return t


@dataclass
class ModelSpec:
    """A whole decoder: embedding, layers, the order they run in, final norm, output head."""
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: object                         # the table's tensor name, or an embedding spec (built as a part)
    layers: List[LayerSpec]
    final_norm: object
    lm_head: Optional[str]                    # None: the head is the embedding table (tied)
    order: List[int] = None                   # layer indices in execution order; may repeat
    optional_tensors: Tuple[str, ...] = ()    # may be stored but are not used (e.g. a tied head's copy)
    ignored_tensors: Tuple[str, ...] = ()     # name patterns (fnmatch) of stored buffers that are no weights
    max_position: int = 0
    logit_softcap: float = 0.0                # > 0: logits = cap * tanh(logits / cap)
    loop: Optional[LoopSpec] = None           # where and how the stream re-enters a stretch of layers that runs again
    logit_scale: float = 1.0                  # a fixed factor on the logits
    depth_average: Optional[DepthAverageSpec] = None    # the stream after each run as a weighted sum of the runs' results

    def __post_init__(self):
        if self.order is None:
            self.order = list(range(len(self.layers)))
        for i in self.order:
            if not 0 <= i < len(self.layers):
                raise ValueError(f"layer order names layer {i}, the model has {len(self.layers)}")

    def tensor_table(self) -> TensorTable:
        if isinstance(self.embedding, str):
            t: TensorTable = {self.embedding: ((self.vocab_size, self.hidden_size), "matrix")}
        else:
            t = dict(self.embedding.tensors())
        for layer in self.layers:
            t.update(layer.tensors())
        t.update(self.final_norm.tensors())
        if self.loop is not None:
            t.update(self.loop.tensors())
        if self.depth_average is not None:
            t.update(self.depth_average.tensors())
        if self.lm_head is not None:
            t[self.lm_head] = ((self.vocab_size, self.hidden_size), "matrix")
        return t

    def expected_shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: s for n, (s, _) in self.tensor_table().items()}
