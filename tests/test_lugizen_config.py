"""Lugizen on the CPU: configuration, the model as data, tensor tables, sizes that only tensors give, random-weights mode,
and the plain implementation's pieces against each other."""
import json

import pytest
import torch

import lugizen_helpers as lh
import plain_lugizen as plain
from qorvix_b200.config import ConfigError, LugizenConfig, lookup_architecture
from qorvix_b200.parts.spec import (ActMLPSpec, ChannelDeltaSpec, ConvInputSpec, LatentAttentionSpec, MoESpec, RMSNormSpec,
                                    RotNormAttentionSpec)
from qorvix_b200.weights import SafetensorsFile, write_random_model

CONFIGS = (lh.CONFIG_A, lh.CONFIG_B, lh.CONFIG_C, lh.CONFIG_D)


def spec_of(raw, shapes=None):
    arch = lookup_architecture("Lugizen")
    cfg = arch.config_from_dict(raw)
    return cfg, arch.spec_for(cfg, shapes)


def test_config_round_trip_and_registry():
    for raw in CONFIGS:
        cfg, spec = spec_of(raw)
        assert isinstance(cfg, LugizenConfig) and cfg.to_dict() == json.loads(json.dumps(raw))
        assert cfg.vocab_size == raw["vocab"] and cfg.canon_taps == raw["canon"]["taps"] and cfg.norm_eps == raw["norm"]["eps"]
        assert spec.order == list(range(len(raw["layers"]))) and spec.lm_head == "head" and spec.embedding == "embed"


def test_the_model_as_data():
    """config.json as stored does not say the ranks of the delta rule's low-rank products."""
    for raw in CONFIGS:
        drawn = {k: tuple(v.shape) for k, v in lh.model_weights(raw, 1).items()}
        _, spec = spec_of(lh.stored(raw), drawn)
        assert spec.expected_shapes() == drawn
        _, from_keys = spec_of(raw)                      # random-weights mode reads them from keys of its own
        assert from_keys.expected_shapes() == drawn
    _, spec = spec_of(lh.stored(lh.CONFIG_A), {k: tuple(v.shape) for k, v in lh.model_weights(lh.CONFIG_A, 1).items()})
    assert all(isinstance(l.mixer, ConvInputSpec) and l.mixer.taps == 3 and l.block == "post_norm" for l in spec.layers)
    assert all(isinstance(l.mixer_norm, RMSNormSpec) and l.mixer_norm.scalar for l in spec.layers) and spec.final_norm.scalar
    kinds = [type(l.mixer.inner) for l in spec.layers]
    assert kinds == [LatentAttentionSpec, ChannelDeltaSpec, RotNormAttentionSpec, RotNormAttentionSpec, RotNormAttentionSpec,
                     RotNormAttentionSpec, LatentAttentionSpec]
    # the first layer that blends values is their source, later ones blend, a layer that does not say so stays out
    assert [l.mixer.inner.v_share_role for l in spec.layers[2:6]] == ["source", "blend", None, "blend"]
    assert spec.layers[4].mixer.inner.v_blend is None and spec.layers[3].mixer.inner.v_blend == "l3.mix.vmix"
    assert spec.layers[3].feed_forward is None and spec.layers[3].ffn_norm is None
    assert isinstance(spec.layers[0].feed_forward, ActMLPSpec) and spec.layers[0].feed_forward.activation == "gelu_tanh"
    ff = spec.layers[2].feed_forward
    assert isinstance(ff, MoESpec) and (ff.experts, ff.top, ff.expert_ff, ff.shared) == (5, 3, 16, None)
    la = spec.layers[6].mixer.inner
    assert (la.num_heads, la.head_dim, la.rot_dim, la.value_dim, la.kv_rank, la.q_rank, la.window, la.gate_proj) == (2, 10, 6, 30, 17, 9, 5, None)
    assert la.position.pairing == "split_half" and la.position.rotary_dim == 6 and la.position.theta == 50000.0
    d = spec.layers[1].mixer.inner
    assert (d.num_heads, d.num_kv_heads, d.key_dim, d.value_dim, d.conv_taps, d.decay_rank, d.gate_rank, d.key_eps) == (4, 2, 20, 12, 3, 5, 7, 1e-6)
    a = spec.layers[5].mixer.inner
    assert (a.position.rotary_dim, a.position.theta, a.head_temp, a.scale) == (8, 300.0, "l5.mix.temp", 2.0 / 24 ** 0.5)
    _, no_rot = spec_of(lh.CONFIG_D)
    assert no_rot.layers[1].mixer.inner.position is None


@pytest.mark.parametrize("change,key", [
    (lambda c: c.pop("vocab"), "config.vocab"), (lambda c: c["norm"].pop("eps"), "norm.eps"), (lambda c: c.pop("canon"), "config.canon"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "layers[0].mixer.q_rank"),
    (lambda c: c["layers"][0]["mixer"]["mask"].pop("size"), "mask.size"),
    (lambda c: c["layers"][2]["mixer"].update(heads=3), "layers[2].mixer.heads"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=26), "layers[2].mixer.rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "layers[1].mixer.conv"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "layers[1].mlp.router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "layers[0].mlp.kind"),
    (lambda c: c["layers"][0].update(type="convolution"), "layers[0].type")])
def test_errors_name_the_key(change, key):
    raw = json.loads(json.dumps(lh.CONFIG_A))
    change(raw)
    with pytest.raises(ConfigError) as e:
        spec_of(raw)
    assert key in str(e.value)


def test_random_model_has_every_tensor(tmp_path):
    cfg, spec = spec_of(lh.CONFIG_A)
    write_random_model(tmp_path, cfg, seed=3)
    f = SafetensorsFile(tmp_path / "model.safetensors")
    assert {n: tuple(f.shape(n)) for n in f.names()} == spec.expected_shapes()
    assert f.shape("l0.norm1") == () and f.shape("l1.mix.q.conv") == (40, 3) and f.shape("l2.mix.vmix") == ()
    assert json.loads((tmp_path / "config.json").read_text()) == cfg.to_dict()


def test_plain_pieces_agree_with_one_another():
    """The oracle's own consistency: a convolution and the recurrent mixer continued from a state equal the whole run, and the
    window of latent attention drops exactly the keys that are `size` or more back."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(20, 6, generator=g, dtype=torch.float64)
    w = torch.randn(6, 4, generator=g, dtype=torch.float64)
    whole, _ = plain.causal_conv(x, w)
    a, tail = plain.causal_conv(x[:7], w)
    b, _ = plain.causal_conv(x[7:], w, tail)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)
    assert torch.allclose(whole[0], x[0] * w[:, 3]) and torch.allclose(whole[1], x[1] * w[:, 3] + x[0] * w[:, 2])
    m = lh.delta()["mixer"]
    W = {"p." + k: v.double() for k, v in lh.delta_weights(m, 32, g).items()}
    h = torch.randn(15, 32, generator=g, dtype=torch.float64)
    whole, _ = plain.channel_delta(h, W, "p.", m, 1e-5)
    first, st = plain.channel_delta(h[:6], W, "p.", m, 1e-5)
    rest, _ = plain.channel_delta(h[6:], W, "p.", m, 1e-5, st)
    assert torch.allclose(torch.cat([first, rest]), whole, atol=1e-10)
    q, k, v = (torch.randn(9, 1, 4, generator=g, dtype=torch.float64) for _ in range(3))
    k[2] *= 50.0
    q[5] = k[2]                                              # position 5 looks straight at key 2: three back
    seen = plain.softmax_attention(q, k, v, 1.0, window=4)[5, 0]
    unseen = plain.softmax_attention(q, k, v, 1.0, window=3)[5, 0]
    assert torch.allclose(seen, v[2, 0], atol=1e-6) and not torch.allclose(unseen, v[2, 0], atol=1e-2)
