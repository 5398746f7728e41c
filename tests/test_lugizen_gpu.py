"""The Lugizen parts and the whole decoder against the plain implementation (tests/plain_lugizen.py): each mechanism
alone in portions and token by token, keys just inside and just outside a window and one far key among hundreds with one
score made to stand out, values blended between layers, a far token in the recurrent state, then whole models under every
way of cutting, batching and reusing pages and slots, in float32 and bfloat16, and greedy generation through the scheduler."""
import pytest
import torch

import lugizen_helpers as lh
import plain_lugizen as plain
from qorvix_b200 import LLM, ModelRunner, SamplingParams, StepEntry
from qorvix_b200.cache import CacheManager
from qorvix_b200.cache.manager import CompositeCacheView
from qorvix_b200.config import lookup_architecture
from qorvix_b200.csrc import ops
from qorvix_b200.engine.batch import BatchBuilder
from qorvix_b200.parts import Runtime, build_part
from qorvix_b200.parts.spec import RMSNormSpec
from qorvix_b200.weights import TensorSource

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")
DTYPES = [torch.float32, torch.bfloat16]
CUTS = (33, 2, 1, 40, 1, 13, 2, 3)          # 95 tokens: page edges (16, 32, ...) fall inside portions and between them
EPS = 2e-5
WIDTH = 72


def close(got, want, dtype, what="", loose=1.0, stray=0):
    """Every row within the bound; `stray` rows may lie beyond it (whole models in bfloat16: a token whose two best experts
    lie close may take the other one)."""
    bound = (1e-4 if dtype in (torch.float32, "float32") else 3e-2 * loose) * max(1.0, float(want.abs().max()))
    err = (got.double().cpu() - want).abs().amax(dim=-1)
    bad = torch.nonzero(err > bound)
    assert bad.numel() <= stray, f"{what}: {bad.numel()} of {err.numel()} rows off, first {int(bad[0])} (err {float(err.max()):.3e}, allowed {bound:.3e})"


def close_model(got, want, dtype, what=""):
    """Whole models.  float32: every row within 1e-4 of the largest logit.  bfloat16: rows are measured by their root
    mean square error against the logits' root mean square: the typical row within 3 %, few beyond 10 % (a token whose
    two best experts lie close may take the other one after rounding), none beyond 60 %; a wrong key, a window one token
    off or another request's page or state moves most rows by far more in these sharpened models, whose every sublayer's
    output is normed to full size."""
    if dtype in (torch.float32, "float32"):
        return close(got, want, dtype, what)
    d = got.double().cpu() - want
    rel = d.pow(2).mean(dim=-1).sqrt() / want.pow(2).mean().sqrt()
    over = int((rel > 0.10).sum())
    assert float(rel.median()) < 0.03 and over <= max(1, rel.numel() // 20) and float(rel.max()) < 0.6, \
        f"{what}: median {float(rel.median()):.3e}, {over} of {rel.numel()} rows over 10 %, worst {float(rel.max()):.3e} at row {int(rel.argmax())}"


def rnd(*shape, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def bf(x):
    return x.to(torch.bfloat16).float()


def layer_spec(layer, width=WIDTH, taps=3):
    """The framework's own spec builder for one layer of a configuration."""
    arch = lookup_architecture("Lugizen")
    return arch.spec_for(arch.config_from_dict(lh.config([layer], width=width, eps=EPS, taps=taps))).layers[0]


def source(tensors, dtype):
    return TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in tensors.items()}, device=DEV, compute_dtype=dtype)


def view_of(part, cache):
    """What the model hands a mixer: the layer's view, or one view per part of a mixer that keeps several."""
    if isinstance(part.cache_spec(), (tuple, list)):
        return CompositeCacheView(views=[cache.layer_view(i) for i in range(len(part.cache_spec()))])
    return cache.layer_view(0)


def cache_for(parts, dtype, max_tokens=256, max_requests=2):
    needs = []
    for part in parts:
        specs = part.cache_spec()
        needs += [(s, None) for s in specs] if isinstance(specs, (tuple, list)) else [(specs, None)]
    return CacheManager(needs, max_tokens=max_tokens, page_size=16, max_requests=max_requests, device=DEV, dtype=dtype)


def step_of(cache, rid, n, first):
    assert cache.reserve(rid, n)
    segs = [dict(tokens=[0] * n, pos0=cache.length(rid), slot=cache.slot(rid), want=[], first=first)]
    tables = {g: [cache.block_table(rid, g)] for g in cache.paged_groups()}
    return BatchBuilder(DEV).build(segs, tables, cache.scratch_page)


def run_in_portions(part, cache, x, cuts, dtype, rid="r"):
    """Feeds x [T, width] through a mixer in the given portions of one request; returns the outputs.  A mixer that reads
    the stream itself gets float32 rows."""
    if not cache.has(rid):
        cache.admit(rid)
    outs, i = [], 0
    for n in cuts:
        ctx = step_of(cache, rid, n, i == 0)
        xin = x[i:i + n].to(torch.float32 if getattr(part, "takes_stream", False) else dtype).to(DEV)
        outs.append(part.forward(xin, ctx, view_of(part, cache)))
        cache.commit(rid, n)
        i += n
    return torch.cat(outs).float()


def mixer_setup(layer, dtype, wrapped=False, seed=1, tweak=None, max_tokens=256, taps=3):
    """The mixer of a layer alone (wrapped: behind the convolution of its input) with weights drawn by the helpers, its
    cache, and the weights in float64 under the names the plain implementation reads."""
    spec = layer_spec(lh.layer(layer, None), taps=taps).mixer
    g = torch.Generator().manual_seed(seed)
    w = {"l0.mix." + k: v for k, v in lh.mixer_weights(layer, WIDTH, g).items()}
    w["l0.canon1"] = lh._rnd(g, WIDTH, taps) * 0.3
    if tweak:
        tweak(w)
    part = build_part("mixer", spec if wrapped else spec.inner, source(w, dtype), Runtime(DEV, dtype, 512))
    return part, cache_for([part], dtype, max_tokens), {k: v.to(torch.bfloat16).double() for k, v in w.items()}      # as stored


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


def inputs(T, seed=3):
    return bf(rnd(T, WIDTH, seed=seed))


# ---------------------------------------------------------------------------------------------- small parts alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 7, 256])
def test_norm_on_a_sublayers_output(width, dtype):
    """stream += y / rms(y) * g with one number g; the stream's copy in the compute type comes from the same pass."""
    norm = build_part("norm", RMSNormSpec(width, EPS, "n", scalar=True), source({"n": torch.tensor(1.3)}, dtype), Runtime(DEV, dtype, 64))
    x, y = rnd(19, width, seed=1), bf(rnd(19, width, seed=2) * 3)
    res = x.to(DEV).clone()
    cast = torch.empty(19, width, device=DEV, dtype=dtype)
    norm.add_normed(res, y.to(dtype).to(DEV), cast=cast)
    g = float(torch.tensor(1.3).to(torch.bfloat16))
    want = x.double() + plain.scalar_norm(y.double(), g, EPS)
    close(res, want, torch.float32, "stream")
    close(cast.float(), want, dtype, "copy")
    out = norm.add_norm(x.to(DEV).clone(), None)                       # the same norm ahead of the output head
    close(out.float(), plain.scalar_norm(x.double(), g, EPS), dtype, "final")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_convolution_of_the_mixers_input(taps, dtype):
    """h + conv(h) in portions down to one token, the tail carried in the request's slot; the slot is used again."""
    from qorvix_b200.parts.spec import ConvInputSpec
    from qorvix_b200.parts.base import Mixer
    from qorvix_b200.parts.registry import register_part, unregister_part

    class Through(Mixer):
        def __init__(self, spec, source, rt):
            pass

        def forward(self, x, ctx, cache):
            return x

    class ThroughSpec:
        kind = "test_through"

        def tensors(self):
            return {}
    register_part("mixer", "test_through", Through, replace=True)
    try:
        w = rnd(WIDTH, taps, seed=taps) * 0.5
        part = build_part("mixer", ConvInputSpec(ThroughSpec(), WIDTH, taps, "c"), source({"c": w}, dtype), Runtime(DEV, dtype, 256))
        cache = cache_for([part], dtype)
        x = rnd(95, WIDTH, seed=9)                  # float32 rows: the stream itself
        want = x.double() + plain.causal_conv(x.double(), bf(w).double())[0]
        close(run_in_portions(part, cache, x, CUTS, dtype), want, dtype, "portions")
        cache.release("r")
        close(run_in_portions(part, cache, x[:40], (1,) * 40, dtype, rid="again"), want[:40], dtype, "token by token")
    finally:
        unregister_part("mixer", "test_through")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ff", [88, 13, 96])
def test_dense_feed_forward_alone(ff, dtype):
    spec = layer_spec(lh.layer(lh.attn(), lh.dense(ff))).feed_forward
    w = {"l0.mlp." + k: v for k, v in lh.mlp_weights(lh.dense(ff), WIDTH, torch.Generator().manual_seed(ff)).items()}
    part = build_part("feed_forward", spec, source(w, dtype), Runtime(DEV, dtype, 64))
    x = inputs(21)
    close(part.forward(x.to(dtype).to(DEV), None).float(), plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}, "l0.mlp."), dtype, "dense")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,ff,T", [(6, 2, 24, 37), (1, 1, 30, 5), (5, 5, 16, 1), (16, 4, 64, 300), (7, 1, 13, 70)])
def test_routed_feed_forward_alone(experts, top, ff, T, dtype):
    f = lh.moe(experts, top, ff)
    spec = layer_spec(lh.layer(lh.attn(), f)).feed_forward
    w = {"l0.mlp." + k: v for k, v in lh.mlp_weights(f, WIDTH, torch.Generator().manual_seed(experts)).items()}
    part = build_part("feed_forward", spec, source(w, dtype), Runtime(DEV, dtype, 64))
    x = inputs(T, seed=experts + T)
    want = plain.routed_ff(x.double(), {k: v.double() for k, v in w.items()}, "l0.mlp.", f)
    close(part.forward(x.to(dtype).to(DEV), None).float(), want, dtype, "experts")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,E,top", [(72, 6, 2), (2048, 64, 6), (70, 5, 5)])
def test_the_router_does_not_depend_on_the_number_of_tokens(d, E, top, dtype):
    """Long steps form the logits by groups of tokens, short ones token by token: choices and weights are the same bit for bit."""
    x = (rnd(600, d, seed=d) * 0.5).to(dtype).to(DEV)
    w = (rnd(E, d, seed=E) * d ** -0.5 * 4).to(dtype).to(DEV)

    def route(rows):
        idx = torch.empty(rows.shape[0], top, device=DEV, dtype=torch.int32)
        wts = torch.empty(rows.shape[0], top, device=DEV, dtype=torch.float32)
        ops.moe_route(idx, wts, None, rows, w, None)
        return idx, wts
    whole_idx, whole_w = route(x)
    parts = [route(x[a:b]) for a, b in ((0, 1), (1, 200), (200, 257), (257, 600))]
    assert torch.equal(whole_idx, torch.cat([p[0] for p in parts])) and torch.equal(whole_w, torch.cat([p[1] for p in parts]))
    z = x.double().cpu() @ w.double().cpu().T
    assert torch.equal(whole_idx[:, 0].cpu().long(), z.argmax(dim=1)) or dtype == torch.bfloat16


# ---------------------------------------------------------------------------------------------- attention

ATTN_CASES = [lh.attn(), lh.attn(heads=6, kv_heads=1, dim=8, vdim=8, rot_dims=8), lh.attn(heads=17, kv_heads=1, dim=6, vdim=10, rot_dims=2),
              lh.attn(heads=4, kv_heads=4, dim=64, vdim=32, rot_dims=32, base=300.0), lh.attn(heads=2, kv_heads=2, dim=14, vdim=130, rot_dims=0),
              lh.attn(heads=8, kv_heads=2, dim=128, vdim=128, rot_dims=64, sharp=4.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wrapped", [False, True])
@pytest.mark.parametrize("case", range(len(ATTN_CASES)))
def test_attention_alone(case, wrapped, dtype):
    layer = ATTN_CASES[case]
    part, cache, W = mixer_setup(layer, dtype, wrapped=wrapped, seed=case + 1)
    x = rnd(95, WIDTH, seed=case) if wrapped else inputs(95, seed=case)
    h = x.double() + plain.causal_conv(x.double(), W["l0.canon1"])[0] if wrapped else x.double()
    want, _ = plain.attention(h, W, "l0.mix.", layer["mixer"], EPS)
    portions_then_token_by_token(part, cache, x, want, dtype, loose=1.5 if wrapped else 1.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, dim=24, vdim=40), dict(heads=4, kv_heads=2, dim=64, vdim=64)])
def test_values_blended_with_the_first_layers(sizes, dtype):
    """Two layers in one step: the first leaves its values for the step's tokens, the second blends its own with them before
    they are cached, so tokens decoded later read blended values of the prompt; a third layer that does not blend stays out."""
    first, second = lh.attn(v_mix=True, **sizes), lh.attn(v_mix=True, rot_dims=8, **sizes)
    arch = lookup_architecture("Lugizen")
    spec = arch.spec_for(arch.config_from_dict(lh.config([lh.layer(first, None), lh.layer(second, None)], width=WIDTH, eps=EPS)))
    g = torch.Generator().manual_seed(7)
    w = {"l0.mix." + k: v for k, v in lh.attn_weights(first["mixer"], WIDTH, g).items()}
    w.update({"l1.mix." + k: v for k, v in lh.attn_weights(second["mixer"], WIDTH, g).items()})
    w["l1.mix.vmix"] = torch.tensor(0.75)
    rt = Runtime(DEV, dtype, 512)
    a = build_part("mixer", spec.layers[0].mixer.inner, source(w, dtype), rt)
    b = build_part("mixer", spec.layers[1].mixer.inner, source(w, dtype), rt)
    cache = cache_for([a, b], dtype)
    W = {k: v.to(torch.bfloat16).double() for k, v in w.items()}
    xa, xb = inputs(70, seed=1), inputs(70, seed=2)
    _, v_first = plain.attention(xa.double(), W, "l0.mix.", first["mixer"], EPS)
    want, _ = plain.attention(xb.double(), W, "l1.mix.", second["mixer"], EPS, v_first)
    unblended, _ = plain.attention(xb.double(), W, "l1.mix.", second["mixer"], EPS)
    assert float((want - unblended).abs().max()) > 0.05                                   # the blend shows
    cache.admit("r")
    outs, i = [], 0
    for n in (20, 1, 1, 30, 2, 1, 15):
        ctx = step_of(cache, "r", n, i == 0)
        a.forward(xa[i:i + n].to(dtype).to(DEV), ctx, cache.layer_view(0))
        outs.append(b.forward(xb[i:i + n].to(dtype).to(DEV), ctx, cache.layer_view(1)))
        cache.commit("r", n)
        i += n
    close(torch.cat(outs).float(), want, dtype, "blended values")


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


def scattered_rows(S, blocks, page, width, g, dtype):
    """A pool whose pages no request holds in a row, filled with random rows."""
    order = torch.randperm(S * blocks, generator=g).to(torch.int32).view(S, blocks)
    rows = (torch.randn(S * blocks + 1, page, width, generator=g) * 0.7).to(torch.bfloat16)
    return order, rows.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,n,dv", [(8, 2, 64, 64), (4, 4, 24, 40), (17, 1, 16, 8)])
def test_one_far_key_among_hundreds(H, G, n, dv, dtype):
    """Without a bias table, single tokens at contexts up to several hundred ahead of portions deep in their contexts, pages
    scattered: every query is made to look at one key far back (its own first key, or the key at a page's border), whose
    score stands out; the result is then that key's value, and a kernel that lost it among the slices shows."""
    page, scale = 16, 0.5
    seg_lens, pos0 = [1, 1, 1, 1, 70, 3, 40], [0, 31, 64, 700, 390, 255, 0]
    ctx = step_ctx(seg_lens, pos0)
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx.max_ctx_len // page)
    g = torch.Generator().manual_seed(5)
    order, cache = scattered_rows(S, blocks, page, G * (n + dv), g, torch.float32)
    q = torch.randn(T, H * n, generator=g) * 0.3
    target = []                                    # the key every token looks at
    t = 0
    for s, (m, p0) in enumerate(zip(seg_lens, pos0)):
        for i in range(m):
            pos = p0 + i
            j = 0 if t % 3 == 0 else (pos // page) * page if t % 3 == 1 else max(0, pos - 1 - (pos % 7))
            target.append(j)
            for h in range(H):
                kv = h // (H // G)
                q[t, h * n: (h + 1) * n] += 6.0 * cache[int(order[s, j // page]), j % page, kv * n: (kv + 1) * n]
            t += 1
    cache, q = cache.to(dtype), q.to(torch.bfloat16).to(dtype)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    table = torch.zeros(H, 1, device=DEV) if dtype == torch.bfloat16 else None
    ops.bias_attention(out, q.to(DEV), cache.to(DEV), ctx, order.to(DEV), H, G, n, dv, page, scale, None, None, None, 1.0, table_of_distances=table)
    ops.check_kernel_errors()
    want = torch.zeros(T, H * dv, dtype=torch.float64)
    t = 0
    for s, (m, p0) in enumerate(zip(seg_lens, pos0)):
        L = p0 + m
        rows_of = torch.stack([cache[int(order[s, j // page]), j % page] for j in range(L)]).double()
        for i in range(m):
            pos = p0 + i
            for h in range(H):
                kv = h // (H // G)
                k, v = rows_of[: pos + 1, kv * n: (kv + 1) * n], rows_of[: pos + 1, G * n + kv * dv: G * n + (kv + 1) * dv]
                w = torch.softmax((k @ q[t, h * n: (h + 1) * n].double()) * scale, 0)
                if n >= 24:
                    assert float(w[target[t]]) > 0.5, "the test's far key was meant to stand out"
                want[t, h * dv: (h + 1) * dv] = w @ v
            t += 1
    close(out.float(), want, dtype, "attention", loose=0.5)


# ---------------------------------------------------------------------------------------------- latent attention

LATENT_CASES = [lh.latent(), lh.latent(heads=2, dim=10, rot_dim=6, vdim=30, kv_rank=17, q_rank=9, window=5),
                lh.latent(heads=1, dim=12, rot_dim=4, vdim=12, kv_rank=12, q_rank=12, window=1),
                lh.latent(heads=4, dim=48, rot_dim=16, vdim=64, kv_rank=64, q_rank=64, window=64),
                lh.latent(heads=2, dim=64, rot_dim=32, vdim=32, kv_rank=128, q_rank=32, window=48),
                lh.latent(heads=5, dim=6, rot_dim=2, vdim=22, kv_rank=9, q_rank=5, window=200)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wrapped", [False, True])
@pytest.mark.parametrize("case", range(len(LATENT_CASES)))
def test_latent_attention_alone(case, wrapped, dtype):
    layer = LATENT_CASES[case]
    part, cache, W = mixer_setup(layer, dtype, wrapped=wrapped, seed=case + 1)
    x = rnd(95, WIDTH, seed=case) if wrapped else inputs(95, seed=case)
    h = x.double() + plain.causal_conv(x.double(), W["l0.canon1"])[0] if wrapped else x.double()
    want = plain.latent_attention(h, W, "l0.mix.", layer["mixer"], EPS)
    portions_then_token_by_token(part, cache, x, want, dtype, loose=1.5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank,dr,dn,dv,H", [(64, 16, 48, 64, 4), (40, 8, 24, 20, 3), (128, 32, 64, 32, 2)])
@pytest.mark.parametrize("window", [1, 16, 37, 64])
def test_keys_just_inside_and_just_outside_the_window(window, rank, dr, dn, dv, H, dtype):
    """The kernels alone over cache rows of the test's making: every query looks hard at the key `window` back (just outside)
    and, half as hard, at the key `window - 1` back (just inside): the result is the inside key's latent, in portions that
    start at any place of a context and for single tokens, pages scattered."""
    page, scale = 16, 1.0
    seg_lens, pos0 = [1, 1, 1, 1, 70, 3, 40], [0, window - 1, window, 300, 130, 2 * window + 5, 0]
    ctx = step_ctx(seg_lens, pos0)
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx.max_ctx_len // page)
    g = torch.Generator().manual_seed(window + rank)
    order, cache = scattered_rows(S, blocks, page, rank + dr, g, torch.float32)
    wuk = (torch.randn(H * dn, rank, generator=g) * rank ** -0.5).to(torch.bfloat16).float()
    wuv = (torch.randn(H * dv, rank, generator=g) * rank ** -0.5).to(torch.bfloat16).float()
    q = torch.randn(T, H * (dn + dr), generator=g) * 0.2
    t = 0
    for s, (m, p0) in enumerate(zip(seg_lens, pos0)):
        for i in range(m):
            pos = p0 + i
            for j, gain in ((pos - window, 6.0), (pos - window + 1, 3.0)):
                if j < 0:
                    continue
                row = cache[int(order[s, j // page]), j % page]
                for h in range(H):                   # the rotated part is shared by the heads: the query meets the key there
                    q[t, h * (dn + dr) + dn: (h + 1) * (dn + dr)] += gain * row[rank:]
            t += 1
    cache, q = cache.to(dtype), q.to(torch.bfloat16).to(dtype)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    wk, wv = wuk.to(dtype).to(DEV), wuv.to(dtype).to(DEV)
    wk_t = wk.view(H, dn, rank).transpose(1, 2).contiguous() if dtype == torch.bfloat16 else None
    ops.latent_attention(out, q.to(DEV), None, cache.to(DEV), wk, wv, ctx, order.to(DEV), H, dn, dr, dv, rank, page, window, scale, wuk_t=wk_t)
    ops.check_kernel_errors()
    want = torch.zeros(T, H * dv, dtype=torch.float64)
    t = 0
    for s, (m, p0) in enumerate(zip(seg_lens, pos0)):
        rows_of = torch.stack([cache[int(order[s, j // page]), j % page] for j in range(p0 + m)]).double()
        for i in range(m):
            pos = p0 + i
            lo = max(0, pos - window + 1)
            for h in range(H):
                qh = q[t, h * (dn + dr): (h + 1) * (dn + dr)].double()
                keys = torch.cat([rows_of[lo: pos + 1, :rank] @ wuk[h * dn: (h + 1) * dn].double().T, rows_of[lo: pos + 1, rank:]], dim=1)
                w = torch.softmax((keys @ qh) * scale, 0)
                want[t, h * dv: (h + 1) * dv] = (w @ rows_of[lo: pos + 1, :rank]) @ wuv[h * dv: (h + 1) * dv].double().T
            t += 1
    close(out.float(), want, dtype, "latent attention", loose=0.7)


# ---------------------------------------------------------------------------------------------- delta rule

DELTA_CASES = [lh.delta(), lh.delta(heads=1, kv_heads=1, dim=64, vdim=64, conv=1, decay_rank=1, gate_rank=1),
               lh.delta(heads=6, kv_heads=2, dim=10, vdim=22, conv=5, decay_rank=3, gate_rank=2),
               lh.delta(heads=2, kv_heads=1, dim=132, vdim=8, conv=2, decay_rank=9, gate_rank=4),
               lh.delta(heads=4, kv_heads=4, dim=64, vdim=64, conv=4, decay_rank=16, gate_rank=8)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wrapped", [False, True])
@pytest.mark.parametrize("case", range(len(DELTA_CASES)))
def test_delta_rule_alone(case, wrapped, dtype):
    layer = DELTA_CASES[case]
    part, cache, W = mixer_setup(layer, dtype, wrapped=wrapped, seed=case + 1)
    x = rnd(95, WIDTH, seed=case) if wrapped else inputs(95, seed=case)
    h = x.double() + plain.causal_conv(x.double(), W["l0.canon1"])[0] if wrapped else x.double()
    want, _ = plain.channel_delta(h, W, "l0.mix.", layer["mixer"], EPS)
    portions_then_token_by_token(part, cache, x, want, dtype, loose=1.5)


def test_removal_reads_the_decayed_state():
    """With strong decays the two orders (removal from the state before or after the decay) differ by far more than
    rounding; the kernels follow the plain implementation, which decays first."""
    layer = lh.delta(heads=2, kv_heads=1, dim=16, vdim=16)

    def strong(w):
        w["l0.mix.dt_bias"] = torch.full_like(w["l0.mix.dt_bias"], 1.0)
        w["l0.mix.A_log"] = torch.full_like(w["l0.mix.A_log"], 0.5)
    part, cache, W = mixer_setup(layer, torch.float32, tweak=strong)
    x = inputs(40, seed=8)
    want, _ = plain.channel_delta(x.double(), W, "l0.mix.", layer["mixer"], EPS)
    close(run_in_portions(part, cache, x, (40,), torch.float32), want, torch.float32, "decay first")


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_token_in_the_state(dtype):
    """Decays next to one: what the first token wrote is still read four hundred tokens later, in portions and token by token."""
    layer = lh.delta(heads=2, kv_heads=1, dim=32, vdim=24)

    def slow(w):
        w["l0.mix.dt_bias"] = torch.full_like(w["l0.mix.dt_bias"], -9.0)
        w["l0.mix.b"] = w["l0.mix.b"] * 0.0                  # beta one half everywhere
    part, cache, W = mixer_setup(layer, dtype, tweak=slow, max_tokens=512)
    x = inputs(420, seed=4) * 0.2
    x[0] = inputs(1, seed=5)[0] * 6.0                        # one loud token at the start
    want, _ = plain.channel_delta(x.double(), W, "l0.mix.", layer["mixer"], EPS)
    quiet = x.clone(); quiet[0] = 0.0
    other, _ = plain.channel_delta(quiet.double(), W, "l0.mix.", layer["mixer"], EPS)
    assert float((want[-1] - other[-1]).abs().max()) > 0.05 * float(want[-1].abs().max())      # the far token still shows at the end
    close(run_in_portions(part, cache, x, (300, 100, 2) + (1,) * 18, dtype), want, dtype, "far token", loose=1.5)


@pytest.mark.parametrize("T,N,R", [(1, 70, 5), (19, 300, 7), (9, 2048, 33)])
def test_decays_from_a_step_size(T, N, R):
    g = torch.Generator().manual_seed(T + N)
    x1, w2, b = torch.randn(T, R + 3, generator=g), torch.randn(N, R, generator=g) * 0.5, torch.randn(N, generator=g)
    rate = torch.exp(torch.randn(N, generator=g))
    out, lin = torch.empty(T, N, device=DEV), torch.empty(T, N, device=DEV)
    ops.channel_gates(out, x1.to(DEV)[:, 1: 1 + R], w2.t().contiguous().to(DEV), b.to(DEV), False, ops.GATE_EXP_NEG_SOFTPLUS, 0.0, rate=rate.to(DEV))
    ops.channel_gates(lin, x1.to(DEV)[:, 1: 1 + R], w2.t().contiguous().to(DEV), None, False, ops.GATE_LINEAR, 0.0)
    z = x1[:, 1: 1 + R].double() @ w2.double().t()
    close(out, torch.exp(-rate.double() * torch.nn.functional.softplus(z + b.double())), torch.float32, "decays")
    close(lin, z, torch.float32, "pre-activations")


# ---------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module")
def models():
    out = {}
    for name, cfg in (("A", lh.CONFIG_A), ("B", lh.CONFIG_B), ("C", lh.CONFIG_C), ("D", lh.CONFIG_D)):
        seed = 11 + len(out)
        out[name] = (lh.make_model_dir(cfg, seed), cfg, lh.as_float64(lh.model_weights(cfg, seed)), {})
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


def for_most(dtype, run, seeds=(0, 100, 200)):
    """float32: run(seed) holds for the first seed.  bfloat16: of three drawings of the tokens at most one may fail: every
    sublayer's output is normed to full size, so a token whose expert or mixer happens to answer quietly carries its rounding
    at full size into the stream and on to every later token that attends to it.  A fault of the cache, a window or a
    kernel fails every drawing."""
    if dtype == "float32":
        return run(seeds[0])
    failed = []
    for s in seeds:
        try:
            run(s)
        except AssertionError as e:
            failed.append(str(e)[:300])
    assert len(failed) <= 1, " | ".join(failed)


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_and_the_stream_after_every_layer(models, name, dtype):
    m = models[name]
    r = runner(m, dtype, use_graphs=False)          # the tap copies to the host, which a captured step cannot

    def whole(n, seed):
        toks = tokens(m[1]["vocab"], n, seed)
        taps = []
        r.model.stream_tap = lambda run, res, pend: taps.append((res + pend.float() if pend is not None else res).double().cpu())
        try:
            out = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        finally:
            r.model.stream_tap = None
        close_model(out, plain_logits(m, toks), dtype, f"whole n={n}")
        streams = []
        plain.forward(m[1], m[2], toks, streams)
        assert len(taps) == len(streams)
        for run, (got, want) in enumerate(zip(taps, streams)):
            close(got, want, dtype, f"stream after layer {run}, n={n}", loose=3.0, stray=0 if dtype == "float32" else max(1, n // 20))
    for n, seed in ((1, 1), (2, 2), (17, 3), (64, 4), (97, 5)):
        for_most(dtype, lambda s: whole(n, seed + s))
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("graphs", [True, False])
def test_prefill_then_long_decode(models, name, dtype, graphs):
    """Decoding runs past every window of the model's layers (pages behind a window go back to the pool on the way)."""
    m = models[name]
    r = runner(m, dtype, use_graphs=graphs)

    def decode(s):
        toks = tokens(m[1]["vocab"], 130, 21 + s)
        want = plain_logits(m, toks)
        try:
            outs = [r.step([StepEntry("d", toks[:30], [29])])]
            for t in toks[30:]:
                outs.append(r.step([StepEntry("d", [t], [0])]))
        finally:
            r.release("d")
        close_model(torch.cat(outs), want[29:], dtype, "decode")
    for_most(dtype, decode)
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(models, name, dtype):
    """No prompt portion at all: the first tokens of a sequence through the single-token path."""
    m = models[name]
    r = runner(m, dtype)

    def from_first(s):
        toks = tokens(m[1]["vocab"], 40, 22 + s)
        try:
            outs = [r.step([StepEntry("t", [t], [0])]) for t in toks]
        finally:
            r.release("t")
        close_model(torch.cat(outs), plain_logits(m, toks), dtype, "from the first token")
    for_most(dtype, from_first)


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_many_sizes(models, name, dtype):
    m = models[name]
    r = runner(m, dtype)

    def portions(s):
        toks = tokens(m[1]["vocab"], 120, 31 + s)
        want = plain_logits(m, toks)
        for cuts in ((2,) * 10 + (100,), (31, 1, 2, 16, 3, 47, 2, 18), (1, 15, 16, 17, 63, 8), (7,) * 17 + (1,)):
            assert sum(cuts) == 120
            outs, i = [], 0
            try:
                for n in cuts:
                    outs.append(r.step([StepEntry("p", toks[i:i + n], list(range(n)))]))
                    i += n
            finally:
                r.release("p")
            close_model(torch.cat(outs), want, dtype, f"cuts {cuts[:4]}..")
    for_most(dtype, portions)


@pytest.mark.parametrize("dtype", MODEL_DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype):
    """Four requests of unequal length advance in unequal portions beside one another in a pool that holds little more
    than they need; two end early and two new ones take their slots and pages.  Every row equals the request alone."""
    m = models[name]
    V = m[1]["vocab"]
    plan = [{"a": 40, "b": 2, "c": 17, "d": 5}, {"a": 1, "b": 30, "c": 1}, {"a": 16, "b": 1, "c": 3, "e": 2}, {"a": 1, "c": 31, "e": 37, "f": 1},
            {"a": 32, "c": 1, "e": 1, "f": 16}, {"c": 1, "e": 30, "f": 1}, {"c": 7}]
    r = runner(m, dtype, max_tokens=288)

    def mixed(s):
        reqs = {"a": tokens(V, 90, 41 + s), "b": tokens(V, 33, 42 + s), "c": tokens(V, 61, 43 + s), "d": tokens(V, 5, 44 + s),
                "e": tokens(V, 70, 45 + s), "f": tokens(V, 18, 46 + s)}
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
        assert r.cache.free_slots() == 4 and not r.cache.live_requests()
        for k, toks in reqs.items():
            assert at[k] == len(toks)
            close_model(torch.cat(got[k]), plain_logits(m, toks), dtype, f"request {k}")
    for_most(dtype, mixed)


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
    llm = LLM(str(m[0]), dtype=dtype, max_tokens=512, max_concurrent=2, max_batch_tokens=32)       # portions of prompts beside decoding; a third request waits for a slot
    slack = 1e-3 if dtype == "float32" else 0.15           # a token of another request's cache lies a whole logit range below

    def generate(s):
        prompts = [tokens(V, n, 70 + n + s) for n in (9, 40, 3)]
        results = llm.generate(prompts, SamplingParams.greedy_params(max_new_tokens=10))
        for p, res in zip(prompts, results):
            assert len(res.tokens) == 10
            seq = list(p)
            for i, tok in enumerate(res.tokens):
                # along the engine's own continuation, every token must be the plain implementation's best or within
                # rounding of it (a near tie may fall either way)
                full = plain_logits(m, seq)[-1]
                assert float(full[tok]) >= float(full.max()) - slack * float(full.abs().max()), f"token {i} of a prompt of {len(p)}: {tok}, plain {int(full.argmax())}"
                seq.append(tok)
    for_most(dtype, generate)
