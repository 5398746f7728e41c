"""Tubazen on the CPU: configuration, the model as data, tensor tables, sizes that only tensors give, the table of
distance buckets against the plain rule, and random-weights mode."""
import json
import math

import pytest
import torch

import plain_tubazen as plain
import tubazen_helpers as th
from qorvix_b200.config import ConfigError, TubazenConfig, lookup_architecture
from qorvix_b200.parts.bias_attention import distance_buckets
from qorvix_b200.parts.spec import BiasedAttentionSpec, DeltaRuleSpec, GLASpec, SideBySideSpec, SwiGLUSpec, TanhNormSpec
from qorvix_b200.weights import SafetensorsFile, write_random_model

CONFIGS = (th.CONFIG_A, th.CONFIG_B, th.CONFIG_C, th.CONFIG_D)


def spec_of(raw, shapes=None):
    arch = lookup_architecture("Tubazen")
    cfg = arch.config_from_dict(raw)
    return cfg, arch.spec_for(cfg, shapes)


def test_config_round_trip_and_registry():
    for raw in CONFIGS:
        cfg, spec = spec_of(raw)
        assert isinstance(cfg, TubazenConfig) and cfg.to_dict() == json.loads(json.dumps(raw))
        assert cfg.vocab_size == raw["vocab"] and cfg.logit_scale == raw["logit_scale"] == spec.logit_scale
        assert spec.max_position == raw["max_positions"] and spec.order == list(range(len(raw["layers"])))


def test_sizes_that_only_tensors_give_come_from_their_shapes():
    """config.json as stored says neither the rank of the decays' products nor the rows of the bias table."""
    for raw in CONFIGS:
        drawn = {k: tuple(v.shape) for k, v in th.model_weights(raw, 1).items()}
        _, spec = spec_of(th.stored(raw), drawn)
        assert spec.expected_shapes() == drawn
        _, from_keys = spec_of(raw)                      # random-weights mode reads them from keys of its own
        assert from_keys.expected_shapes() == drawn
    _, spec = spec_of(th.stored(th.CONFIG_A), {k: tuple(v.shape) for k, v in th.model_weights(th.CONFIG_A, 1).items()})
    kinds = [type(l.mixer) for l in spec.layers]
    assert kinds == [GLASpec, SideBySideSpec, GLASpec, SideBySideSpec]
    assert spec.layers[2].feed_forward is None and spec.layers[2].ffn_gate is None and spec.layers[2].ffn_norm is None
    assert isinstance(spec.layers[0].feed_forward, SwiGLUSpec) and spec.layers[0].feed_forward.activation == "gelu_tanh"
    assert all(isinstance(l.mixer_norm, TanhNormSpec) and l.block == "gated_pre_norm" for l in spec.layers)
    m = spec.layers[0].mixer
    assert (m.num_heads, m.key_dim, m.value_dim, m.decay.rank, m.decay.param, m.decay.form) == (3, 20, 28, 5, 7.0, "pow_sigmoid")
    pair = spec.layers[3].mixer
    l, r = pair.left, pair.right
    assert isinstance(l, BiasedAttentionSpec) and isinstance(r, DeltaRuleSpec) and (pair.left_scale, pair.right_scale) == (0.6, 1.7)
    assert (l.num_heads, l.num_kv_heads, l.head_dim, l.value_dim, l.bias_rows, l.bias_max, l.temp_coef, l.temp_every) == (6, 1, 8, 8, 9, 23.0, 1.1, 3)
    assert (r.num_heads, r.head_dim, r.decay.rank, r.decay.inner_tanh, r.decay.form) == (3, 40, 2, True, "exp_neg_sigmoid")
    assert r.decay.param == pytest.approx(math.exp(-0.5)) and r.key_eps == 1e-6
    assert spec.depth_average.weights == tuple(f"l{i}.dwa" for i in range(4))


@pytest.mark.parametrize("change,key", [
    (lambda c: c.pop("vocab"), "config.vocab"), (lambda c: c["norm"].pop("eps"), "norm.eps"), (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "layers[0].mixer.tau"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("kv_heads"), "layers[1].mixer.left.kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(heads=3), "layers[1].mixer.left.heads"),
    (lambda c: c["layers"][1]["mixer"]["left"]["q_temp"].pop("every"), "q_temp.every"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "layers[1].mixer.right"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][0].update(type="convolution"), "layers[0].type")])
def test_errors_name_the_key(change, key):
    raw = json.loads(json.dumps(th.CONFIG_A))
    change(raw)
    with pytest.raises(ConfigError) as e:
        spec_of(raw)
    assert key in str(e.value)


@pytest.mark.parametrize("rows,far", [(14, 50), (9, 23), (32, 200), (16, 40), (20, 90), (7, 11.5), (33, 700), (2, 5)])
def test_distance_buckets_against_the_plain_rule(rows, far):
    got = distance_buckets(rows, far, 4096)
    assert len(got) == math.ceil(far) + 1 and got[-1] == rows - 1        # from `far` on every distance has the last row
    assert list(got[: rows // 2]) == list(range(rows // 2)) and all(a <= b for a, b in zip(got, got[1:]))
    want = [plain.distance_bucket(n, rows, far) for n in range(len(got))]
    # float32 against float64: they may differ only where the logarithm's multiple falls on a whole number
    half = rows // 2
    for n, (a, b) in enumerate(zip(got, want)):
        if a != b:
            x = math.log(n / half) / math.log(far / half) * (rows - half)
            assert abs(x - round(x)) < 1e-4 and abs(int(a) - b) == 1
    assert plain.distance_bucket(10 ** 6, rows, far) == rows - 1
    assert len(distance_buckets(rows, far, 5)) == 5                      # no longer than the positions there are


def test_random_model_has_every_tensor(tmp_path):
    cfg, spec = spec_of(th.CONFIG_A)
    write_random_model(tmp_path, cfg, seed=3)
    f = SafetensorsFile(tmp_path / "model.safetensors")
    assert {n: tuple(f.shape(n)) for n in f.names()} == spec.expected_shapes()
    assert f.shape("l0.norm1.alpha") == () and f.shape("l3.dwa") == (5,)
    assert json.loads((tmp_path / "config.json").read_text()) == cfg.to_dict()
