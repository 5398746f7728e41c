"""The Tubazen parts and the whole decoder against the plain implementation (tests/plain_tubazen.py): each mechanism
alone in portions and token by token, the edges of the distance buckets and of the temperature's steps, one far token
among hundreds, then whole models under every way of cutting, batching and reusing pages and slots, in float32 and
bfloat16, and greedy generation through the scheduler."""
import math

import pytest
import torch

import plain_tubazen as plain
import tubazen_helpers as th
from qorvix_b200 import LLM, ModelRunner, SamplingParams, StepEntry
from qorvix_b200.cache import CacheManager
from qorvix_b200.cache.manager import CompositeCacheView
from qorvix_b200.config import lookup_architecture
from qorvix_b200.csrc import ops
from qorvix_b200.engine.batch import BatchBuilder
from qorvix_b200.parts import Runtime, build_part
from qorvix_b200.weights import TensorSource

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]
CUTS = (33, 2, 1, 40, 1, 13, 2, 3)          # 95 tokens: page edges (16, 32, ...) fall inside portions and between them
EPS = 2e-5
WIDTH = 72


def close(got, want, dtype, what="", loose=1.0):
    bound = (1e-4 if dtype in (torch.float32, "float32") else 3e-2 * loose) * max(1.0, float(want.abs().max()))
    err = (got.double().cpu() - want).abs().amax(dim=-1)
    bad = torch.nonzero(err > bound)
    assert not bad.numel(), f"{what}: {bad.numel()} of {err.numel()} rows off, first {int(bad[0])} (err {float(err.max()):.3e}, allowed {bound:.3e})"


def close_model(got, want, dtype, what=""):
    """Whole models.  float32: every row within 1e-4 of the largest logit.  bfloat16: rows are measured by their root
    mean square error against the logits' root mean square: the typical row within 2 %, few beyond 8 %, none beyond
    40 %; a wrong key or another request's page or state moves rows by far more in these sharpened models."""
    if dtype in (torch.float32, "float32"):
        return close(got, want, dtype, what)
    d = got.double().cpu() - want
    rel = d.pow(2).mean(dim=-1).sqrt() / want.pow(2).mean().sqrt()
    over = int((rel > 0.08).sum())
    assert float(rel.median()) < 0.02 and over <= max(1, rel.numel() // 30) and float(rel.max()) < 0.4, \
        f"{what}: median {float(rel.median()):.3e}, {over} of {rel.numel()} rows over 8 %, worst {float(rel.max()):.3e} at row {int(rel.argmax())}"


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def bf(x):
    return x.to(torch.bfloat16).float()


def layer_spec(layer, width=WIDTH):
    """The framework's own spec builder for one layer of a configuration."""
    arch = lookup_architecture("Tubazen")
    return arch.spec_for(arch.config_from_dict(th.config([layer], width=width, eps=EPS))).layers[0]


def source(tensors, dtype):
    return TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in tensors.items()}, device=DEV, compute_dtype=dtype)


def view_of(part, cache):
    """What the model hands a mixer: the layer's view, or one view per part of a mixer that keeps several."""
    if isinstance(part.cache_spec(), (tuple, list)):
        return CompositeCacheView(views=[cache.layer_view(i) for i in range(len(part.cache_spec()))])
    return cache.layer_view(0)


def run_in_portions(part, cache, x, cuts, dtype, rid="r"):
    """Feeds x [T, width] through a mixer in the given portions of one request; returns the outputs."""
    builder = BatchBuilder(DEV)
    if not cache.has(rid):
        cache.admit(rid)
    outs, i = [], 0
    for n in cuts:
        assert cache.reserve(rid, n)
        segs = [dict(tokens=[0] * n, pos0=cache.length(rid), slot=cache.slot(rid), want=[], first=i == 0)]
        tables = {g: [cache.block_table(rid, g)] for g in cache.paged_groups()}
        ctx = builder.build(segs, tables, cache.scratch_page)
        outs.append(part.forward(x[i:i + n].to(dtype).to(DEV), ctx, view_of(part, cache)))
        cache.commit(rid, n)
        i += n
    return torch.cat(outs).float()


def mixer_setup(layer, dtype, which=None, seed=1, tweak=None, max_tokens=256):
    """A mixer of the layer (which: None the layer's own, 'left' / 'right' one side of a pair alone) with weights drawn
    by the helpers, its cache, and the weights in float64 under the names the plain implementation reads."""
    spec = layer_spec(th.layer(layer, None)).mixer
    w = {"l0.mix." + k: v for k, v in th.mixer_weights(layer, WIDTH, torch.Generator().manual_seed(seed)).items()}
    if which is not None:
        spec = getattr(spec, which)
    if tweak:
        tweak(w)
    part = build_part("mixer", spec, source(w, dtype), Runtime(DEV, dtype, 512))
    specs = part.cache_spec()
    needs = [(s, None) for s in specs] if isinstance(specs, (tuple, list)) else [(specs, None)]
    cache = CacheManager(needs, max_tokens=max_tokens, page_size=16, max_requests=2, device=DEV, dtype=dtype)
    return part, cache, {k: v.to(torch.bfloat16).double() for k, v in w.items()}      # as stored


def portions_then_token_by_token(part, cache, x, want, dtype, loose=1.0):
    close(run_in_portions(part, cache, x, CUTS, dtype), want, dtype, "portions", loose)
    # the same request again after another took and left its slot, one token at a time after a short start: a state or
    # a cache row that the first run left behind would show
    cache.release("r")
    cache.admit("filler"); cache.release("filler")
    close(run_in_portions(part, cache, x[:60], (5,) + (1,) * 55, dtype, rid="again"), want[:60], dtype, "token by token", loose)
    cache.release("again")
    close(run_in_portions(part, cache, x[:31], (2,) * 15 + (1,), dtype, rid="pairs"), want[:31], dtype, "two at a time", loose)
    cache.check_invariants()


# ---------------------------------------------------------------------------------------------- small parts alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 7, 256])
def test_tanh_norm_alone(width, dtype):
    from qorvix_b200.parts.spec import TanhNormSpec
    w = {k: bf(v) for k, v in th.norm_weights("n", width, torch.Generator().manual_seed(3)).items()}
    part = build_part("norm", TanhNormSpec(width, "n"), source(w, dtype), Runtime(DEV, dtype, 64))
    x, delta = rnd(19, width, seed=1) * 2, rnd(19, width, seed=2)
    for pending in (None, delta.to(DEV), delta.to(dtype).to(DEV)):
        res = x.clone().to(DEV)
        got = part.add_norm(res, pending)
        total = x.double() + (pending.double().cpu() if pending is not None else 0)
        close(got, plain.tanh_norm(total, {k: v.double() for k, v in w.items()}, "n"), dtype, "norm")
        close(res, total, torch.float32, "the stream holds the sum")
    rows = torch.tensor([4, 0, 18], dtype=torch.int32, device=DEV)
    res = x.clone().to(DEV)
    close(part.add_norm(res, delta.to(DEV), rows=rows), plain.tanh_norm((x + delta).double()[[4, 0, 18]], {k: v.double() for k, v in w.items()}, "n"),
          dtype, "chosen rows")


@pytest.mark.parametrize("dtype", DTYPES)
def test_positioned_embedding_alone(dtype):
    from qorvix_b200.parts.spec import PositionedEmbeddingSpec, TanhNormSpec
    vocab, width, positions = 50, 40, 64
    g = torch.Generator().manual_seed(5)
    w = {"embed": bf(torch.randn(vocab, width, generator=g)), "pos": bf(0.5 * torch.randn(positions, width, generator=g))}
    w.update({k: bf(v) for k, v in th.norm_weights("embed.norm", width, g).items()})
    spec = PositionedEmbeddingSpec(vocab, width, positions, "embed", "pos", norm=TanhNormSpec(width, "embed.norm"))
    part = build_part("embedding", spec, source(w, dtype), Runtime(DEV, dtype, 64))
    toks = [int(t) for t in torch.randint(0, vocab, (30,), generator=g)]
    W = {k: v.double() for k, v in w.items()}
    want = plain.embedding(toks, W)
    # two requests in one step, each at its own positions: the second starts at 0 again, the first goes on from 12
    ctx = BatchBuilder(DEV).build([dict(tokens=toks[12:30], pos0=12, slot=0, want=[], first=False),
                                   dict(tokens=toks[:12], pos0=0, slot=1, want=[], first=True)], {}, 0)
    out = torch.empty(30, width, device=DEV, dtype=torch.float32)
    part.forward(out, ctx, None)
    close(out, torch.cat([want[12:], want[:12]]), torch.float32, "embedding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_depth_average_alone(dtype):
    from qorvix_b200.parts.spec import DepthAverageSpec
    width, runs, T = 24, 3, 11
    mix = {f"l{i}.dwa": bf(1.0 / (i + 2) + 0.3 * rnd(i + 2, seed=10 + i)) for i in range(runs)}
    part = build_part("stream", DepthAverageSpec(tuple(mix), width), source(mix, dtype), Runtime(DEV, dtype, 64))
    x0 = rnd(T, width, seed=1)
    stream = x0.clone().to(DEV)
    stack = part.begin(stream)
    kept, x = [x0.double()], x0.double()
    for i in range(runs):
        delta = rnd(T, width, seed=20 + i)
        pending = None if i == 1 else (delta.to(DEV) if i == 0 else delta.to(dtype).to(DEV))
        kept.append(x + (pending.double().cpu() if pending is not None else 0))
        x = sum(mix[f"l{i}.dwa"].double()[j] * kept[j] for j in range(i + 2))
        stream = part.after(i, stream, pending, stack)
        close(stream, x, torch.float32, f"after run {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ff", [88, 13, 96])
def test_dense_feed_forward_alone(ff, dtype):
    spec = layer_spec(th.layer(th.gla(), th.dense(ff))).feed_forward
    w = {"l0.mlp." + k: v for k, v in th.mlp_weights(th.dense(ff), WIDTH, torch.Generator().manual_seed(2)).items()}
    part = build_part("feed_forward", spec, source(w, dtype), Runtime(DEV, dtype, 64))
    x = bf(rnd(37, WIDTH, seed=6))
    ctx = BatchBuilder(DEV).build([dict(tokens=[0] * 37, pos0=0, slot=0, want=[], first=True)], {}, 0)
    close(part.forward(x.to(dtype).to(DEV), ctx).float(), plain.dense_feed_forward(x.double(), {k: v.double() for k, v in w.items()}, "l0.mlp."), dtype, "ff")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", [th.layer(th.gla(), th.dense()), th.layer(th.pair(), None), th.layer(th.pair(), th.dense(24))])
def test_gated_block_alone(layer, dtype):
    """A whole layer: both norms, the mixer, the feed-forward and the two gates that read the sublayers' inputs."""
    spec = layer_spec(layer)
    g = torch.Generator().manual_seed(7)
    cfg = th.config([layer], width=WIDTH, eps=EPS)
    w = {k: v.float() for k, v in th.model_weights(cfg, 9).items() if k.startswith("l0.") and k != "l0.dwa"}
    from qorvix_b200.models.text_model import _BlockView
    part = build_part("block", _BlockView(spec), source(w, dtype), Runtime(DEV, dtype, 512))
    specs = part.mixer.cache_spec()
    needs = [(s, None) for s in specs] if isinstance(specs, (tuple, list)) else [(specs, None)]
    cache = CacheManager(needs, max_tokens=128, page_size=16, max_requests=2, device=DEV, dtype=dtype)
    x = rnd(50, WIDTH, seed=8)
    want = plain.layer(x.double(), {k: v.double() for k, v in w.items()}, 0, layer, EPS)
    builder = BatchBuilder(DEV)
    cache.admit("r")
    outs, i = [], 0
    for n in (17, 2, 1, 30):
        assert cache.reserve("r", n)
        ctx = builder.build([dict(tokens=[0] * n, pos0=i, slot=cache.slot("r"), want=[], first=i == 0)],
                            {gr: [cache.block_table("r", gr)] for gr in cache.paged_groups()}, cache.scratch_page)
        res, pend = part.forward(x[i:i + n].clone().to(DEV), None, ctx, view_of(part.mixer, cache))
        outs.append(res + pend.float())
        cache.commit("r", n)
        i += n
    close(torch.cat(outs), want, dtype, "layer", loose=2.0)


# ---------------------------------------------------------------------------------------------- mixers alone

def inputs(T, seed=3):
    return bf(rnd(T, WIDTH, seed=seed))


GLA_CASES = [th.gla(), th.gla(heads=2, dim=33, vdim=12, tau=2.5, rank=3), th.gla(heads=1, dim=70, vdim=6, tau=30.0, rank=1),
             th.gla(heads=5, dim=6, vdim=22, tau=1.0, rank=9), th.gla(heads=1, dim=136, vdim=40, tau=4.0, rank=4)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(GLA_CASES)))
def test_gated_linear_attention_alone(case, dtype):
    layer = GLA_CASES[case]
    part, cache, w = mixer_setup(layer, dtype)
    x = inputs(95)
    want = plain.gated_linear_attention(x.double(), w, "l0.mix.", layer["mixer"], EPS)
    portions_then_token_by_token(part, cache, x, want, dtype)


DELTA_CASES = [th.right(), th.right(heads=1, dim=64, rank=16), th.right(heads=3, dim=40, rank=2), th.right(heads=1, dim=132, rank=3),
               th.right(heads=4, dim=7, rank=1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(DELTA_CASES)))
def test_delta_rule_alone(case, dtype):
    layer = th.pair(r=DELTA_CASES[case])
    part, cache, w = mixer_setup(layer, dtype, which="right")
    x = inputs(95, seed=4)
    want = plain.delta_rule(x.double(), w, "l0.mix.right.", layer["mixer"]["right"], EPS)
    portions_then_token_by_token(part, cache, x, want, dtype, loose=2.0)


def test_delta_rule_removal_reads_the_old_state():
    """With a removal rate near one and the same key twice, the second token removes what the first wrote before it
    writes; an implementation whose removal read the new state, or none, gives another result than the oracle's."""
    def tweak(w):
        w["l0.mix.right.a.b"] += 6.0
    layer = th.pair(r=th.right(heads=2, dim=18, rank=6))
    part, cache, w = mixer_setup(layer, torch.float32, which="right", tweak=tweak)
    x = inputs(12, seed=5)
    x[5] = x[4]
    want = plain.delta_rule(x.double(), w, "l0.mix.right.", layer["mixer"]["right"], EPS)
    close(run_in_portions(part, cache, x, (4, 1, 1, 6), torch.float32), want, torch.float32, "removal")
    off = {k: v.clone() for k, v in w.items()}
    off["l0.mix.right.a.b"] -= 40.0                         # no removal at all: the oracle tells the two apart
    other = plain.delta_rule(x.double(), off, "l0.mix.right.", layer["mixer"]["right"], EPS)
    assert float((other - want).abs().max()) > 0.05 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["gla", "delta"])
def test_one_far_token_in_the_state(kind, dtype):
    """Decays close to one: a token at position 3 that stands out is still in the state 200 tokens later, through
    portions and single tokens; the outputs there differ from those of a sequence without it."""
    def tweak(w):
        for k in w:
            if k.endswith("a2.b"):
                w[k] += 7.0                                # sigmoid(z)^(1/tau) close to one
            if k.endswith("w0"):
                w[k] -= 7.0                                # exp(-rate * sigmoid(z)) close to one
            if k.endswith("right.a.b"):
                w[k] -= 4.0                                # little removal
    if kind == "gla":
        layer = th.gla(heads=2, dim=24, vdim=20, tau=9.0, rank=4)
        part, cache, w = mixer_setup(layer, dtype, tweak=tweak, max_tokens=320)
        fn = lambda x: plain.gated_linear_attention(x.double(), w, "l0.mix.", layer["mixer"], EPS)
    else:
        layer = th.pair(r=th.right(heads=2, dim=24, rank=4))
        part, cache, w = mixer_setup(layer, dtype, which="right", tweak=tweak, max_tokens=320)
        fn = lambda x: plain.delta_rule(x.double(), w, "l0.mix.right.", layer["mixer"]["right"], EPS)
    x = 0.3 * rnd(230, WIDTH, seed=8)
    x[3] = 6.0 * rnd(WIDTH, seed=9)
    x = bf(x)
    want = fn(x)
    close(run_in_portions(part, cache, x, (150, 41, 2, 7, 2) + (1,) * 28, dtype), want, dtype, "far token", loose=2.0)
    blind = x.clone()
    blind[3] = 0.0
    gap = (want[200:] - fn(blind)[200:]).abs().amax(dim=-1)
    assert float(gap.min()) > 0.05 * float(want[200:].abs().max())


LEFT_CASES = [th.left(), th.left(heads=6, kv_heads=1, dim=8, vdim=8, bias_max=23, rows=9, coef=1.1, every=3),
              th.left(heads=1, kv_heads=1, dim=36, vdim=20, bias_max=200, rows=32, coef=0.35, every=1000),
              th.left(heads=4, kv_heads=4, dim=32, vdim=64, bias_max=40, rows=16, every=16),
              th.left(heads=8, kv_heads=2, dim=16, vdim=32, bias_max=90, rows=20, every=5),
              th.left(heads=4, kv_heads=2, dim=64, vdim=128, bias_max=60.5, rows=11, coef=0.0, every=1),
              th.left(heads=3, kv_heads=3, dim=128, vdim=16, bias_max=3, rows=2, coef=2.0, every=2),
              th.left(heads=2, kv_heads=1, dim=21, vdim=13, bias_max=77, rows=15, every=40),
              th.left(heads=16, kv_heads=1, dim=40, vdim=56, bias_max=30, rows=12, every=9),          # sixteen heads share the keys
              th.left(heads=34, kv_heads=2, dim=8, vdim=72, bias_max=100, rows=6, coef=0.7, every=11),  # seventeen do
              th.left(heads=2, kv_heads=2, dim=72, vdim=8, bias_max=64, rows=64, every=32)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", range(len(LEFT_CASES)))
def test_biased_attention_alone(case, dtype):
    layer = th.pair(l=LEFT_CASES[case])
    part, cache, w = mixer_setup(layer, dtype, which="left")
    x = inputs(95, seed=6)
    want = plain.biased_attention(x.double(), w, "l0.mix.left.", layer["mixer"]["left"])
    portions_then_token_by_token(part, cache, x, want, dtype, loose=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [dict(heads=2, kv_heads=1, dim=24, vdim=40), dict(heads=4, kv_heads=2, dim=32, vdim=64)])
@pytest.mark.parametrize("rows,far", [(14, 50), (8, 198), (8, 197), (20, 400)])
def test_one_bucket_of_the_distance_bias_stands_out(rows, far, sizes, dtype):
    """The table holds -9 everywhere but in one row, so every query looks at the keys whose distance falls into that
    row: the row of distance 197 (position 200 looking back at position 3).  Every edge of that bucket is an edge of the
    visible set, in portions and in decoding; one row up or down is another function, which the oracle confirms."""
    m = th.left(bias_max=far, rows=rows, sharp=0.5, coef=0.2, every=64, **sizes)
    layer = th.pair(l=m)
    row = plain.distance_bucket(197, rows, float(far))

    def table(r):
        def tweak(w):
            w["l0.mix.left.rel"][:] = -9.0
            w["l0.mix.left.rel"][r] = 9.0
        return tweak

    part, cache, w = mixer_setup(layer, dtype, which="left", seed=4, tweak=table(row), max_tokens=320)
    x = inputs(230, seed=8)
    want = plain.biased_attention(x.double(), w, "l0.mix.left.", m)
    close(run_in_portions(part, cache, x, (150, 41, 2, 7, 2) + (1,) * 28, dtype), want, dtype, f"bucket {row}", loose=2.0)
    _, _, w2 = mixer_setup(layer, dtype, which="left", seed=4, tweak=table(row - 1), max_tokens=32)
    other = plain.biased_attention(x.double(), w2, "l0.mix.left.", m)
    assert float((other[200:] - want[200:]).abs().max()) > 0.05 * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("every", [1, 2, 16, 95, 1000])
def test_query_temperature_steps(every, dtype):
    """A large coefficient: the step of the temperature (at positions every - 1, 2 every - 1, ...) moves the outputs."""
    m = th.left(coef=1.5, every=every, sharp=2.0)
    layer = th.pair(l=m)
    part, cache, w = mixer_setup(layer, dtype, which="left", seed=7)
    x = inputs(100, seed=2)
    want = plain.biased_attention(x.double(), w, "l0.mix.left.", m)
    close(run_in_portions(part, cache, x, (15, 1, 1, 14, 2, 60, 1, 1, 1, 4), dtype), want, dtype, f"every {every}", loose=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scales", [(1.3, 0.8), (1.0, 1.0), (0.0, 2.0), (-0.7, 0.0)])
def test_mixers_side_by_side(scales, dtype):
    layer = th.pair(left_scale=scales[0], right_scale=scales[1])
    part, cache, w = mixer_setup(layer, dtype)
    x = inputs(95, seed=12)
    want = plain.side_by_side(x.double(), w, "l0.mix.", layer["mixer"], EPS)
    portions_then_token_by_token(part, cache, x, want, dtype, loose=2.0)


# ---------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module")
def models():
    out = {}
    for name, cfg in (("A", th.CONFIG_A), ("B", th.CONFIG_B), ("C", th.CONFIG_C), ("D", th.CONFIG_D)):
        seed = 11 + len(out)
        out[name] = (th.make_model_dir(cfg, seed), cfg, th.as_float64(th.model_weights(cfg, seed)), {})
    return out


def plain_logits(model, toks):
    _, cfg, weights, memo = model
    key = tuple(toks)
    if key not in memo:
        memo[key] = plain.forward(cfg, weights, list(toks))
    return memo[key]


def tokens(vocab, n, seed):
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed))]


def runner(model, dtype, max_tokens=256, **kw):
    return ModelRunner(model[0], dtype=dtype, max_tokens=max_tokens, page_size=16, max_requests=kw.pop("max_requests", 4), **kw)


NAMES = ["A", "B", "C", "D"]
MODEL_DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_the_stream_after_every_layer(models, name, dtype):
    m = models[name]
    r = runner(m, dtype, use_graphs=False)          # the tap copies to the host, which a captured step cannot
    for n, seed in ((1, 1), (2, 2), (17, 3), (64, 4), (97, 5)):
        toks = tokens(m[1]["vocab"], n, seed)
        taps = []
        r.model.stream_tap = lambda run, res, pend: taps.append((res + pend.float() if pend is not None else res).double().cpu())
        out = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        r.model.stream_tap = None
        close_model(out, plain_logits(m, toks), dtype, f"whole n={n}")
        streams = []
        plain.forward(m[1], m[2], toks, streams)
        assert len(taps) == len(streams)
        for run, (got, want) in enumerate(zip(taps, streams)):
            close(got, want, dtype, f"stream after layer {run}, n={n}", loose=3.0)
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("graphs", [True, False])
def test_prefill_then_long_decode(models, name, dtype, graphs):
    m = models[name]
    toks = tokens(m[1]["vocab"], 130, 21)
    want = plain_logits(m, toks)
    r = runner(m, dtype, use_graphs=graphs)
    outs = [r.step([StepEntry("d", toks[:30], [29])])]
    for t in toks[30:]:
        outs.append(r.step([StepEntry("d", [t], [0])]))
    close_model(torch.cat(outs), want[29:], dtype, "decode")


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(models, name, dtype):
    """No prompt portion at all: the first tokens of a sequence through the single-token path."""
    m = models[name]
    toks = tokens(m[1]["vocab"], 40, 22)
    r = runner(m, dtype)
    outs = [r.step([StepEntry("t", [t], [0])]) for t in toks]
    close_model(torch.cat(outs), plain_logits(m, toks), dtype, "from the first token")


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_many_sizes(models, name, dtype):
    m = models[name]
    toks = tokens(m[1]["vocab"], 120, 31)
    want = plain_logits(m, toks)
    r = runner(m, dtype)
    for cuts in ((2,) * 10 + (100,), (31, 1, 2, 16, 3, 47, 2, 18), (1, 15, 16, 17, 63, 8), (7,) * 17 + (1,)):
        assert sum(cuts) == 120
        outs, i = [], 0
        for n in cuts:
            outs.append(r.step([StepEntry("p", toks[i:i + n], list(range(n)))]))
            i += n
        r.release("p")
        close_model(torch.cat(outs), want, dtype, f"cuts {cuts[:4]}..")


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Four requests of unequal length advance in unequal portions beside one another in a pool that holds little more
    than they need; two end early and two new ones take their slots and pages.  Every row equals the request alone."""
    m = models[name]
    V = m[1]["vocab"]
    reqs = {"a": tokens(V, 90, 41), "b": tokens(V, 33, 42), "c": tokens(V, 61, 43), "d": tokens(V, 5, 44),
            "e": tokens(V, 70, 45), "f": tokens(V, 18, 46)}
    plan = [{"a": 40, "b": 2, "c": 17, "d": 5}, {"a": 1, "b": 30, "c": 1}, {"a": 16, "b": 1, "c": 3, "e": 2}, {"a": 1, "c": 31, "e": 37, "f": 1},
            {"a": 32, "c": 1, "e": 1, "f": 16}, {"c": 1, "e": 30, "f": 1}, {"c": 7}]
    r = runner(m, dtype, max_tokens=288)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step.items():
            entries.append(StepEntry(k, reqs[k][at[k]: at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = r.step(entries, end=end)
        row = 0
        for k, n in step.items():
            got[k].append(out[row: row + n])
            row += n
        r.cache.check_invariants()
    for k, toks in reqs.items():
        assert at[k] == len(toks)
        close_model(torch.cat(got[k]), plain_logits(m, toks), dtype, f"request {k}")
    assert r.cache.free_slots() == 4 and not r.cache.live_requests()


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
def test_logits_do_not_depend_on_the_batch(models, dtype):
    """A request's logits with three others in the step equal its logits alone: bit for bit in float32 (every sum has a
    fixed order), to rounding in bfloat16."""
    m = models["A"]
    V = m[1]["vocab"]
    toks = tokens(V, 50, 51)
    r = runner(m, dtype)
    alone = torch.cat([r.step([StepEntry("x", toks[:20], list(range(20)))]), r.step([StepEntry("x", toks[20:], list(range(30)))], end=["x"])])
    others = [StepEntry(k, tokens(V, n, 60 + n), []) for k, n in (("o1", 3), ("o2", 1), ("o3", 37))]
    first = r.step(others[:2] + [StepEntry("x", toks[:20], list(range(20)))] + others[2:])
    rest = r.step([StepEntry("o1", [1], []), StepEntry("x", toks[20:], list(range(30))), StepEntry("o2", [2, 3], [])])
    both = torch.cat([first, rest])
    if dtype == "float32":
        assert torch.equal(both, alone)
    else:
        close_model(both, alone.double().cpu(), dtype, "beside others")


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_scheduler(models, name, dtype):
    m = models[name]
    V = m[1]["vocab"]
    prompts = [tokens(V, n, 70 + n) for n in (9, 40, 3)]
    llm = LLM(str(m[0]), dtype=dtype, max_tokens=512, max_concurrent=2, max_batch_tokens=32)       # portions of prompts beside decoding; a third request waits for a slot
    results = llm.generate(prompts, SamplingParams.greedy_params(max_new_tokens=10))
    slack = 1e-3 if dtype == "float32" else 0.05
    for p, res in zip(prompts, results):
        assert len(res.tokens) == 10
        seq = list(p)
        for i, tok in enumerate(res.tokens):
            # along the engine's own continuation, every token must be the plain implementation's best or within
            # rounding of it (a near tie may fall either way)
            full = plain_logits(m, seq)[-1]
            assert float(full[tok]) >= float(full.max()) - slack * float(full.abs().max()), f"token {i} of a prompt of {len(p)}: {tok}, plain {int(full.argmax())}"
            seq.append(tok)


# ---------------------------------------------------------------------------------------------- kernels alone, larger shapes

def step_ctx(seg_lens, pos0):
    """A step's context for kernels run alone: segments in the given order, every one with its own state slot."""
    from types import SimpleNamespace
    i32 = dict(dtype=torch.int32, device=DEV)
    qs = [0]
    for n in seg_lens:
        qs.append(qs[-1] + n)
    return SimpleNamespace(
        num_segments=len(seg_lens), num_tokens=qs[-1], max_q_len=max(seg_lens), seg_len=list(seg_lens), seg_start_pos=list(pos0),
        max_ctx_len=max(p + n for p, n in zip(pos0, seg_lens)), captured=False, seg_q_start=torch.tensor(qs, **i32),
        seg_pos0=torch.tensor(pos0, **i32), seg_slot=torch.arange(len(seg_lens), **i32),
        tok_seg=torch.cat([torch.full((n,), s, **i32) for s, n in enumerate(seg_lens)]),
        tok_pos=torch.cat([torch.arange(p, p + n, **i32) for p, n in zip(pos0, seg_lens)]))


@pytest.mark.parametrize("H,G,n,dv", [(16, 1, 128, 128), (8, 2, 64, 128), (4, 4, 104, 24), (6, 3, 16, 64)])
def test_tensor_core_attention_on_long_contexts_and_unequal_segments(H, G, n, dv, monkeypatch):
    """Single tokens at contexts from 1 to several hundred (many slices, some empty) ahead of portions that start in the
    middle of a context, pages scattered over the pool; every (token, head) against float64 sums over its own keys."""
    from qorvix_b200.parts.bias_attention import distance_buckets
    page, rows, far, scale = 16, 10, 150.0, 0.3
    seg_lens, pos0 = [1, 1, 1, 1, 70, 3, 129], [0, 31, 64, 700, 390, 255, 0]
    ctx = step_ctx(seg_lens, pos0)
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx.max_ctx_len // page)
    g = torch.Generator().manual_seed(5)
    order = torch.randperm(S * blocks, generator=g).to(torch.int32).view(S, blocks)          # no request's pages lie in a row
    cache = (torch.randn(S * blocks + 1, page, G * (n + dv), generator=g) * 0.7).to(torch.bfloat16)
    q = torch.randn(T, H * n, generator=g).to(torch.bfloat16)
    gate = torch.randn(T, H * dv, generator=g)
    rel = torch.randn(rows, H, generator=g) * 2
    bucket = torch.from_numpy(distance_buckets(rows, far, 1024))
    out = torch.empty(T, H * dv, dtype=torch.bfloat16, device=DEV)
    table = ops.bias_attention_table(bucket.to(DEV), rel.to(DEV))

    def no_other_kernel(*a, **k):
        raise AssertionError("these sizes belong to the tensor-core kernel")
    monkeypatch.setattr(ops, "bias_attention_generic", no_other_kernel)
    ops.bias_attention(out, q.to(DEV), cache.to(DEV), ctx, order.to(DEV), H, G, n, dv, page, scale, bucket.to(DEV), rel.to(DEV),
                       gate.to(DEV), 0.9, table_of_distances=table)
    ops.check_kernel_errors()
    want = torch.zeros(T, H * dv, dtype=torch.float64)
    t = 0
    for s, (m, p0) in enumerate(zip(seg_lens, pos0)):
        L = p0 + m
        rows_of = torch.stack([cache[int(order[s, j // page]), j % page] for j in range(L)]).double()     # [L, G * (n + dv)]
        for i in range(m):
            pos = p0 + i
            for h in range(H):
                kv = h // (H // G)
                k, v = rows_of[: pos + 1, kv * n: (kv + 1) * n], rows_of[: pos + 1, G * n + kv * dv: G * n + (kv + 1) * dv]
                dist = torch.arange(pos, -1, -1).clamp(max=len(bucket) - 1)
                sc = (k @ q[t, h * n: (h + 1) * n].double()) * scale + rel[bucket[dist].long(), h].double()
                o = torch.softmax(sc, 0) @ v
                want[t, h * dv: (h + 1) * dv] = o * torch.sigmoid(gate[t, h * dv: (h + 1) * dv].double()) * 0.9
            t += 1
    close(out.float(), want, torch.bfloat16, "attention", loose=0.5)


@pytest.mark.parametrize("removal", [False, True])
@pytest.mark.parametrize("H,dk,dv", [(2, 256, 20), (3, 64, 72), (1, 12, 130), (5, 100, 8)])
def test_channel_scan_with_unequal_segments_and_carried_states(H, dk, dv, removal):
    """Single tokens beside portions longer than a stage of the ring, every segment from a state of its own that is not
    zero; outputs and the states left behind against the recurrence written out in float64."""
    seg_lens = [1, 1, 45, 2, 16, 33]
    ctx = step_ctx(seg_lens, [0] * len(seg_lens))
    S, T = len(seg_lens), sum(seg_lens)
    g = torch.Generator().manual_seed(dk + dv)
    f = lambda *shape: torch.randn(*shape, generator=g)
    q, k, v = f(T, H * dk) * 0.3, f(T, H * dk) * 0.3, f(T, H * dv)
    w = torch.sigmoid(f(T, H * dk) + 2)
    u = torch.nn.functional.normalize(f(T, H, dk), dim=-1).reshape(T, H * dk)
    au = u * torch.sigmoid(f(T, H * dk))
    n_state = ops.channel_scan_state_floats(H, dk, dv)
    state = torch.zeros(S, n_state, device=DEV)
    y = torch.empty(T, H * dv, device=DEV)
    dev = lambda x: x.to(DEV).contiguous()
    args = (dev(q), dev(k), dev(v), dev(w), dev(au) if removal else None, dev(u) if removal else None, 0.5)
    ops.channel_scan(y, *args, state, ctx, H, dk, dv)              # a first step leaves states that are not zero
    y2 = torch.empty_like(y)
    ops.channel_scan(y2, *args, state, ctx, H, dk, dv)             # the same tokens again, from those states
    ops.check_kernel_errors()
    want = torch.zeros(2, T, H * dv, dtype=torch.float64)
    t0 = 0
    for m in seg_lens:
        for h in range(H):
            Sm = torch.zeros(dk, dv, dtype=torch.float64)
            for rep in range(2):
                for t in range(t0, t0 + m):
                    sl = slice(h * dk, (h + 1) * dk)
                    new = w[t, sl].double()[:, None] * Sm + k[t, sl].double()[:, None] * v[t, h * dv: (h + 1) * dv].double()[None, :]
                    if removal:
                        new = new - au[t, sl].double()[:, None] * (u[t, sl].double() @ Sm)[None, :]
                    Sm = new
                    want[rep, t, h * dv: (h + 1) * dv] = (Sm.T @ q[t, sl].double()) * 0.5
        t0 += m
    close(y, want[0], torch.float32, "first step")
    close(y2, want[1], torch.float32, "second step")


@pytest.mark.parametrize("T,N,R", [(1, 70, 5), (8, 64, 64), (19, 300, 7), (9, 2048, 33)])
@pytest.mark.parametrize("form", ["pow_sigmoid", "exp_neg_sigmoid"])
def test_channel_gates_alone(T, N, R, form):
    g = torch.Generator().manual_seed(T + N)
    x1, w2, b = torch.randn(T, R + 3, generator=g), torch.randn(N, R, generator=g) * 0.5, torch.randn(N, generator=g)
    out = torch.empty(T, N, device=DEV)
    inner = form == "exp_neg_sigmoid"
    kind, p = (ops.GATE_POW_SIGMOID, 1 / 7.0) if form == "pow_sigmoid" else (ops.GATE_EXP_NEG_SIGMOID, 0.6)
    ops.channel_gates(out, x1.to(DEV)[:, 1: 1 + R], w2.t().contiguous().to(DEV), b.to(DEV), inner, kind, p)
    xin = x1[:, 1: 1 + R].double()
    z = (torch.tanh(xin) if inner else xin) @ w2.double().t() + b.double()
    want = torch.sigmoid(z) ** (1 / 7.0) if form == "pow_sigmoid" else torch.exp(-0.6 * torch.sigmoid(z))
    close(out, want, torch.float32, "gates")
