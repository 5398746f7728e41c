"""Prefill and decode throughput of a Deganex, a Lotirax, a Tubazen or a Lugizen model at layer sizes that resemble real models, beside the
Llama decoder at equal width, depth and (active) feed-forward size, and the design's kernels alone with their roofline
fractions beside the Llama kernels they correspond to.

    python bench.py --design deganex|lotirax|tubazen|lugizen [--layers-per-kind 2] [--batch 8] [--ctx 1024] [--prefill-tokens 2048]
    python -m qorvix_b200.design_bench [--design lotirax|tubazen|lugizen]

Random bfloat16 weights; timing with CUDA events after warm-up; kernels alone are timed in captured chains over
buffers larger than L2 (kernel_bench.timed_chain).  Figures go out as one JSON line.
"""
from __future__ import annotations

import argparse
import json
import statistics
from types import SimpleNamespace

import torch

from . import kernel_bench as kb
from .csrc import ops

# Layer sizes: latent attention as in 16-head models with a 512-wide latent; the matrix-memory LSTM with four wide
# heads; the state space with 64 heads of 64 over a state of 128; 64 routed experts of which 6 serve a token, and
# a shared expert twice as wide as a routed one.
WIDTH, VOCAB = 2048, 32000
ATTN = {"heads": 16, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}
MLSTM = {"heads": 4, "dim": 256, "vdim": 512, "gate_cap": 15.0}
MAMBA = {"heads": 64, "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}
MOE = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 64, "top": 6}, "shared": {"ff": 2816}}


def deganex_config(layers_per_kind: int) -> dict:
    kinds = [("latent_attention", ATTN), ("mlstm", MLSTM), ("mamba2", MAMBA)]
    layers = [{"type": k, "mixer": m, "mlp": MOE} for _ in range(layers_per_kind) for k, m in kinds]
    return {"architecture": "Deganex", "vocab": VOCAB, "width": WIDTH, "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 17}}, "layers": layers}


def llama_config(n_layers: int) -> dict:
    active_ff = MOE["router"]["top"] * MOE["expert"]["ff"] + MOE["shared"]["ff"]
    return {"architectures": ["LlamaForCausalLM"], "vocab_size": VOCAB, "hidden_size": WIDTH, "intermediate_size": active_ff,
            "num_hidden_layers": n_layers, "num_attention_heads": 16, "num_key_value_heads": 16, "head_dim": 128,
            "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False}


def _runner(raw, pool_tokens, concurrent):
    from .config import architecture_of, lookup_architecture
    from .engine import ModelRunner
    from .weights import random_tensors
    cfg = lookup_architecture(architecture_of(raw)).config_from_dict(raw)
    tensors = dict(random_tensors(cfg, seed=0, device="cuda", dtype=torch.bfloat16))
    r = ModelRunner(config=cfg, tensors=tensors, dtype="bfloat16", max_tokens=pool_tokens, max_requests=concurrent, max_model_len=8192)
    del tensors
    return cfg, r


def _tokens(vocab, n, seed):
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed))]


def model_throughput(raw, batch, ctx, prefill_tokens, steps, warmup) -> dict:
    """Prefill of one prompt and decode of `batch` requests at `ctx` cached tokens, through the step function."""
    from .engine import StepEntry
    cfg, r = _runner(raw, max(prefill_tokens + 64, batch * (ctx + steps + warmup + 80)), max(batch, 1))
    V = cfg.vocab_size
    ms = []
    for it in range(4):
        p = _tokens(V, prefill_tokens, it)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        r.step([StepEntry("pre", p, [prefill_tokens - 1])], end=["pre"])
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            ms.append(e0.elapsed_time(e1))
    pre_ms = statistics.median(ms)
    ids = list(range(batch))
    for i in ids:
        r.step([StepEntry(i, _tokens(V, ctx - 1, 100 + i), [])])
    dec = r.decoder(ids)
    dec.start([1] * batch)
    for _ in range(warmup):
        dec.step()
    torch.cuda.synchronize()
    n0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        dec.step()
    e1.record()
    torch.cuda.synchronize()
    dec_ms = e0.elapsed_time(e1) / steps
    launches = (ops.launch_count() - n0) // steps
    dec.finish()
    ops.check_kernel_errors()
    out = {"prefill_tokens": prefill_tokens, "prefill_ms": round(pre_ms, 3), "prefill_tok_s": round(prefill_tokens / pre_ms * 1e3, 1),
           "decode_batch": batch, "decode_ctx": ctx, "decode_ms_per_step": round(dec_ms, 4), "decode_tok_s": round(batch / dec_ms * 1e3, 1),
           "launches_per_decode_step": int(launches)}
    del r, dec
    torch.cuda.empty_cache()
    return out


def _ctx(seg_lens, pos0, device="cuda"):
    """A step context of the given segments (all state slots distinct), for kernels run alone."""
    S, T = len(seg_lens), sum(seg_lens)
    qs = [0]
    for n in seg_lens:
        qs.append(qs[-1] + n)
    i32 = dict(dtype=torch.int32, device=device)
    return SimpleNamespace(
        num_segments=S, num_tokens=T, max_q_len=max(seg_lens), seg_q_start=torch.tensor(qs, **i32),
        seg_slot=torch.arange(S, **i32), tok_seg=torch.repeat_interleave(torch.arange(S, **i32), torch.tensor(seg_lens, device=device)).to(torch.int32),
        tok_pos=torch.cat([torch.arange(p, p + n, **i32) for p, n in zip(pos0, seg_lens)]))


def latent_attention_case(seg_lens, ctx_len, peaks, page=16, window=0, gated=True) -> dict:
    """Latent attention of the given segments, each ending at ctx_len cached tokens (prepare excluded); window > 0: the last
    `window` keys only; gated False: without the output gate."""
    H, dn, dr, dv, rank = ATTN["heads"], ATTN["dim"], ATTN["rot_dim"], ATTN["vdim"], ATTN["kv_rank"]
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx_len // page)
    row_bytes = (rank + dr) * 2
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * ctx_len * row_bytes)) + 1))
    caches = torch.randn(copies, S * blocks + 1, page, rank + dr, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(S * blocks, dtype=torch.int32, device="cuda").view(S, blocks)
    ctx = _ctx(seg_lens, [ctx_len - n for n in seg_lens])
    ctx.seg_len, ctx.seg_start_pos, ctx.max_ctx_len, ctx.captured = list(seg_lens), [ctx_len - n for n in seg_lens], ctx_len, False
    ctx.seg_pos0 = torch.tensor(ctx.seg_start_pos, dtype=torch.int32, device="cuda")
    q = torch.randn(T, H * (dn + dr), device="cuda", dtype=torch.bfloat16) * 0.3
    gate = torch.randn(T, H * dv, device="cuda", dtype=torch.bfloat16) if gated else None
    wuk = torch.randn(H * dn, rank, device="cuda", dtype=torch.bfloat16) * 0.05
    wuv = torch.randn(H * dv, rank, device="cuda", dtype=torch.bfloat16) * 0.05
    wuk_t = wuk.view(H, dn, rank).transpose(1, 2).contiguous()
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)
    us = kb.timed_chain(lambda i: ops.latent_attention(out, q, gate, caches[i % copies], wuk, wuv, ctx, table, H, dn, dr, dv, rank, page, window,
                                                       ATTN["scale"], wuk_t=wuk_t), launches=8)
    seen = lambda pos: min(pos + 1, window) if window else pos + 1                      # keys a query at `pos` sees
    pairs = sum(seen(ctx_len - n + i) for n in seg_lens for i in range(n))              # (query, key) pairs per head
    flops = H * pairs * (2.0 * (rank + dr) + 2.0 * rank) + T * H * 2.0 * rank * (dn + dv)
    rows = sum(min(ctx_len, window + n - 1) if window else ctx_len for n in seg_lens)   # cache rows the step must read
    return kb._figures(us, rows * row_bytes + (q.numel() + (gate.numel() if gated else 0) + out.numel()) * 2, flops, peaks)


def scan_case(kind, seg_lens, peaks) -> dict:
    """The recurrence of the matrix-memory LSTM ('mlstm') or the state space ('mamba2') over the given segments."""
    S, T = len(seg_lens), sum(seg_lens)
    ctx = _ctx(seg_lens, [0] * S)
    if kind == "mlstm":
        H, dk, dv, code, qg = MLSTM["heads"], MLSTM["dim"], MLSTM["vdim"], ops.SCAN_GATED_MAX, 1
    else:
        H, dk, dv, code, qg = MAMBA["heads"], MAMBA["state"], MAMBA["vdim"], ops.SCAN_DECAY, MAMBA["heads"] // MAMBA["groups"]
    n_state = ops.linear_scan_state_floats(code, H, dk, dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * n_state * 4)) + 1))
    states = torch.zeros(copies, S, n_state, device="cuda", dtype=torch.float32)
    q = torch.randn(T, (H // qg) * dk, device="cuda", dtype=torch.bfloat16) * 0.1
    k = torch.randn(T, (H // qg) * dk, device="cuda", dtype=torch.bfloat16) * 0.1
    v = torch.randn(T, H * dv, device="cuda", dtype=torch.bfloat16)
    g1 = torch.randn(T, H, device="cuda", dtype=torch.float32)
    g2 = torch.randn(T, H, device="cuda", dtype=torch.float32) + 3
    p = torch.zeros(H, device="cuda", dtype=torch.float32)
    y = torch.empty(T, H * dv, device="cuda", dtype=torch.float32)
    us = kb.timed_chain(lambda i: ops.linear_scan(code, y, q, k, v, g1, g2 if kind == "mlstm" else None, p, p, p, 15.0, 1.0,
                                                  states[i % copies], ctx, H, dk, dv, q_group=qg), launches=8)
    nbytes = 2 * S * n_state * 4 + (q.numel() + k.numel() + v.numel()) * 2 + y.numel() * 4
    return kb._figures(us, nbytes, 4.0 * T * H * dk * dv, peaks)


def experts_case(T, peaks) -> dict:
    """Both products of the routed experts for T tokens (router and grouping included, shared expert excluded)."""
    E, top, ff, d = MOE["router"]["experts"], MOE["router"]["top"], MOE["expert"]["ff"], WIDTH
    wbytes = E * 3 * ff * d * 2
    copies = max(2, int(2.5 * kb.L2_BYTES // wbytes) + 1)
    wg = [ops.moe_pack_experts(torch.randn(E, ff, d, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    wu = [ops.moe_pack_experts(torch.randn(E, ff, d, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    wd = [ops.moe_pack_experts(torch.randn(E, d, ff, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    router = torch.randn(E, d, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
    R = T * top
    top_idx = torch.empty(T, top, device="cuda", dtype=torch.int32)
    top_w = torch.empty(T, top, device="cuda", dtype=torch.float32)
    tile_rows = ops.moe_tile_rows(True)
    ints = torch.empty(3 * R + 3 * ops.moe_max_tiles(R, E, tile_rows), device="cuda", dtype=torch.int32)
    row_token, slot_row, scratch, tiles = ints[:R], ints[R:2 * R], ints[2 * R:3 * R], ints[3 * R:]
    act = torch.empty(R, ff, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(R, d, device="cuda", dtype=torch.float32)
    delta = torch.empty(T, d, device="cuda", dtype=torch.float32)

    def run(i):
        ops.moe_route(top_idx, top_w, None, x, router, None)
        ops.moe_group(row_token, slot_row, tiles, top_idx, scratch, E, tile_rows)
        ops.moe_experts_tc(True, act, x, wg[i % copies], wu[i % copies], row_token, tiles)
        ops.moe_experts_tc(False, y, act, wd[i % copies], None, row_token, tiles)
        ops.moe_combine(delta, None, y, slot_row, top_w, None, None)

    us = kb.timed_chain(run, launches=6)
    touched = min(E, R)                                        # experts whose weights a step must read at least
    nbytes = touched * 3 * ff * d * 2 + T * d * 2 + R * (ff * 2 * 2 + d * 4 * 2) + T * d * 4
    return kb._figures(us, nbytes, 2.0 * R * 3 * ff * d, peaks)


# ---------------------------------------------------------------------------------------------- Lotirax
# Sixteen heads of two 64-wide maps over 128 values, four key/value heads, a window of 1,024 keys, rotation over the
# whole map with stretching; dense feed-forwards of 8,192 alternate with 64 small experts of 1,024 of which 4 serve a
# token beside a shared one of 2,048; the two middle layers run twice.
LOT_ATTN = {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.125, "diff": 0.2, "mask": {"size": 1024},
            "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 16.0, "slow": 2.0}}}
LOT_DENSE = {"kind": "dense", "ff": 8192}
LOT_MOE = {"kind": "moe", "expert": {"ff": 1024}, "router": {"experts": 64, "top": 4}, "shared": {"ff": 2048}}


def lotirax_config() -> dict:
    layers = [{"type": "attention", "mixer": LOT_ATTN, "mlp": f} for f in (LOT_DENSE, LOT_MOE, LOT_DENSE, LOT_MOE)]
    return {"architecture": "Lotirax", "vocab": VOCAB, "width": WIDTH, "norm": {"eps": 1e-5}, "residual_mult": 0.25, "layers": layers,
            "loop": {"start": 1, "stop": 3, "times": 2}}


def lotirax_llama_config(n_layers: int) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "vocab_size": VOCAB, "hidden_size": WIDTH, "intermediate_size": LOT_DENSE["ff"],
            "num_hidden_layers": n_layers, "num_attention_heads": LOT_ATTN["heads"], "num_key_value_heads": LOT_ATTN["kv_heads"],
            "head_dim": 128, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": True}


def diff_attention_case(seg_lens, ctx_len, peaks, page=16) -> dict:
    """Differential attention of the given segments, each ending at ctx_len cached tokens (the preparing kernel excluded)."""
    a = LOT_ATTN
    H, G, n, dv, W = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["mask"]["size"]
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx_len // page)
    width = G * (2 * n + dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * min(ctx_len, W + max(seg_lens)) * width * 2)) + 1))
    caches = torch.randn(copies, S * blocks + 1, page, width, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(S * blocks, dtype=torch.int32, device="cuda").view(S, blocks)
    ctx = _ctx(seg_lens, [ctx_len - m for m in seg_lens])
    ctx.seg_len, ctx.seg_start_pos, ctx.max_ctx_len, ctx.captured = list(seg_lens), [ctx_len - m for m in seg_lens], ctx_len, False
    ctx.seg_pos0 = torch.tensor(ctx.seg_start_pos, dtype=torch.int32, device="cuda")
    q = torch.randn(T, H * 2 * n, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)
    us = kb.timed_chain(lambda i: ops.diff_attention(out, q, caches[i % copies], ctx, table, H, G, n, dv, page, W, a["scale"], 0.4, 1e-5, 0.7),
                        launches=8)
    pairs = sum(sum(min(p + 1, W) for p in range(ctx_len - m, ctx_len)) for m in seg_lens)      # (query, key) pairs per head
    keys_read = sum(min(ctx_len, W + m - 1) for m in seg_lens)
    flops = H * pairs * (4.0 * n + 4.0 * dv)
    return kb._figures(us, keys_read * width * 2 + (q.numel() + out.numel()) * 2, flops, peaks)


def diff_prepare_case(T, peaks, page=16) -> dict:
    """Bias, per-map norm, rotation and cache write of T tokens of one request."""
    from .parts.rotary import inverse_frequencies
    a = LOT_ATTN
    H, G, n, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    cols, width = (H + G) * 2 * n + G * dv, G * (2 * n + dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (T * (cols * 4 + width * 2 + H * 2 * n * 2))) + 1))
    projs = torch.randn(copies, T, cols, device="cuda", dtype=torch.float32)
    blocks = -(-T // page)
    caches = torch.zeros(copies, blocks + 1, page, width, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(blocks, dtype=torch.int32, device="cuda").view(1, blocks)
    ctx = _ctx([T], [0])
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inverse_frequencies(n, a["rot"]["base"])[None, :]
    cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().cuda().contiguous()
    bias = torch.randn(cols, device="cuda")
    w = torch.ones(n, device="cuda")
    q = torch.empty(copies, T, H * 2 * n, device="cuda", dtype=torch.bfloat16)
    us = kb.timed_chain(lambda i: ops.diff_prepare(q[i % copies], projs[i % copies], bias, w, w, 1e-5, cos_sin, ctx, table, caches[i % copies],
                                                   H, G, n, dv, n, page), launches=8)
    return kb._figures(us, T * (cols * 4 + width * 2 + H * 2 * n * 2), 0.0, peaks)


def table_experts_case(T, peaks) -> dict:
    """Both products of the table-routed ungated experts for T tokens (look-up and grouping included, shared expert excluded)."""
    E, top, ff, d = LOT_MOE["router"]["experts"], LOT_MOE["router"]["top"], LOT_MOE["expert"]["ff"], WIDTH
    wbytes = E * 2 * ff * d * 2
    copies = max(2, int(2.5 * kb.L2_BYTES // wbytes) + 1)
    wu = [ops.moe_pack_experts(torch.randn(E, ff, d, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    wd = [ops.moe_pack_experts(torch.randn(E, d, ff, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    table = torch.argsort(torch.rand(VOCAB, E, device="cuda"), dim=1)[:, :top].to(torch.int32).contiguous()
    ids = torch.randint(0, VOCAB, (T,), device="cuda", dtype=torch.int32)
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
    R = T * top
    top_idx = torch.empty(T, top, device="cuda", dtype=torch.int32)
    top_w = torch.empty(T, top, device="cuda", dtype=torch.float32)
    tile_rows = ops.moe_tile_rows(True)
    ints = torch.empty(3 * R + 3 * ops.moe_max_tiles(R, E, tile_rows), device="cuda", dtype=torch.int32)
    row_token, slot_row, scratch, tiles = ints[:R], ints[R:2 * R], ints[2 * R:3 * R], ints[3 * R:]
    act = torch.empty(R, ff, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(R, d, device="cuda", dtype=torch.float32)
    delta = torch.empty(T, d, device="cuda", dtype=torch.float32)
    scale = torch.ones(d, device="cuda")

    def run(i):
        ops.moe_route_table(top_idx, top_w, table, ids, E)
        ops.moe_group(row_token, slot_row, tiles, top_idx, scratch, E, tile_rows)
        ops.moe_experts_tc(2, act, x, wu[i % copies], None, row_token, tiles)
        ops.moe_experts_tc(0, y, act, wd[i % copies], None, row_token, tiles)
        ops.moe_combine(delta, None, y, slot_row, top_w, None, None, ff_scale=scale)

    us = kb.timed_chain(run, launches=6)
    touched = min(E, R)
    nbytes = touched * 2 * ff * d * 2 + T * d * 2 + R * (ff * 2 * 2 + d * 4 * 2) + T * d * 4
    return kb._figures(us, nbytes, 2.0 * R * 2 * ff * d, peaks)


def run_lotirax(args, peaks) -> dict:
    raw = lotirax_config()
    n_runs = 6
    res = {"lotirax": model_throughput(raw, args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup),
           "llama_equal_size": model_throughput(lotirax_llama_config(n_runs), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup)}
    T, B, C = args.prefill_tokens, args.batch, args.ctx
    res["kernels"] = {
        f"diff_attention_prefill_t{T}": diff_attention_case([T], T, peaks),
        f"diff_attention_decode_b{B}_ctx{C}": diff_attention_case([1] * B, C, peaks),
        f"diff_prepare_t{T}": diff_prepare_case(T, peaks), f"diff_prepare_t{B}": diff_prepare_case(B, peaks),
        f"table_experts_prefill_t{T}": table_experts_case(T, peaks), f"table_experts_decode_b{B}": table_experts_case(B, peaks),
    }
    from .config import LlamaConfig
    like = kb.headline_kernels(LlamaConfig.from_dict(lotirax_llama_config(n_runs)), B, C, T, peaks)
    ops.check_kernel_errors()
    res["llama_kernels"] = {k: v for k, v in like.items() if "attention" in k or "gate_up" in k or "down" in k}
    return res


# ------------------------------------------------------------------ Tubazen
# Gated linear attention with eight heads of 128 key channels over 256 values; attention with a distance bias, 16 heads of
# 128 on 4 key/value heads, beside a delta rule of 32 heads of 64; gated feed-forwards of 5,632.
TUB_GLA = {"heads": 8, "dim": 128, "vdim": 256, "tau": 8.0, "rank": 64}
TUB_LEFT = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "bias_max": 4096, "bias_rows": 64,
            "q_temp": {"coef": 0.2, "every": 512}}
TUB_RIGHT = {"heads": 32, "dim": 64, "rank": 64}
TUB_FF = {"kind": "dense", "ff": 5632}


def tubazen_config(layers_per_kind: int) -> dict:
    pair = {"type": "parallel", "mixer": {"left": TUB_LEFT, "right": TUB_RIGHT, "left_scale": 1.0, "right_scale": 1.0}, "mlp": TUB_FF}
    layers = [{"type": "gla", "mixer": TUB_GLA, "mlp": TUB_FF}, pair] * layers_per_kind
    return {"architecture": "Tubazen", "vocab": VOCAB, "width": WIDTH, "norm": {"eps": 1e-5}, "logit_scale": 1.0, "max_positions": 8192,
            "layers": layers}


def tubazen_llama_config(n_layers: int) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "vocab_size": VOCAB, "hidden_size": WIDTH, "intermediate_size": TUB_FF["ff"],
            "num_hidden_layers": n_layers, "num_attention_heads": TUB_LEFT["heads"], "num_key_value_heads": TUB_LEFT["kv_heads"],
            "head_dim": 128, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False}


def bias_attention_case(seg_lens, ctx_len, peaks, page=16) -> dict:
    """Attention with a distance bias over the given segments, each ending at ctx_len cached tokens (the preparing kernel excluded)."""
    from .parts.bias_attention import distance_buckets
    a = TUB_LEFT
    H, G, n, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx_len // page)
    width = G * (n + dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * ctx_len * width * 2)) + 1))
    caches = torch.randn(copies, S * blocks + 1, page, width, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(S * blocks, dtype=torch.int32, device="cuda").view(S, blocks)
    ctx = _ctx(seg_lens, [ctx_len - m for m in seg_lens])
    ctx.seg_len, ctx.seg_start_pos, ctx.max_ctx_len, ctx.captured = list(seg_lens), [ctx_len - m for m in seg_lens], ctx_len, False
    ctx.seg_pos0 = torch.tensor(ctx.seg_start_pos, dtype=torch.int32, device="cuda")
    q = torch.randn(T, H * n, device="cuda", dtype=torch.bfloat16)
    gate = torch.randn(T, H * dv, device="cuda", dtype=torch.float32)
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)
    rel = torch.randn(a["bias_rows"], H, device="cuda", dtype=torch.float32)
    bucket = torch.from_numpy(distance_buckets(a["bias_rows"], a["bias_max"], 8192)).cuda()
    bias = ops.bias_attention_table(bucket, rel)
    us = kb.timed_chain(lambda i: ops.bias_attention(out, q, caches[i % copies], ctx, table, H, G, n, dv, page, a["scale"], bucket, rel, gate,
                                                     1.0, table_of_distances=bias), launches=8)
    pairs = sum(m * (ctx_len - m) + m * (m + 1) // 2 for m in seg_lens)
    return kb._figures(us, S * ctx_len * width * 2 + (q.numel() + out.numel()) * 2 + gate.numel() * 4, H * pairs * (2.0 * n + 2.0 * dv), peaks)


def bias_prepare_case(T, peaks, page=16) -> dict:
    """Biases, the queries' temperature and the cache write of T tokens of one request."""
    a = TUB_LEFT
    H, G, n, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    cols, width = (H + G) * n + G * dv, G * (n + dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (T * (cols * 4 + width * 2 + H * n * 2))) + 1))
    projs = torch.randn(copies, T, cols, device="cuda", dtype=torch.float32)
    blocks = -(-T // page)
    caches = torch.zeros(copies, blocks + 1, page, width, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(blocks, dtype=torch.int32, device="cuda").view(1, blocks)
    ctx = _ctx([T], [0])
    bq, bk, bv = (torch.randn(m, device="cuda") for m in (H * n, G * n, G * dv))
    q = torch.empty(copies, T, H * n, device="cuda", dtype=torch.bfloat16)
    us = kb.timed_chain(lambda i: ops.bias_attn_prepare(q[i % copies], projs[i % copies], 0, H * n, (H + G) * n, bq, bk, bv, caches[i % copies], ctx,
                                                        table, H, G, n, dv, page, 0.2, 512), launches=8)
    return kb._figures(us, T * (cols * 4 + width * 2 + H * n * 2), 0.0, peaks)


def channel_scan_case(kind, seg_lens, peaks, scan_only=False) -> dict:
    """The recurrence with a decay per key channel: gated linear attention ('gla') or the delta rule ('delta'), with the kernels that
    form its decays (and unit keys) and the norm behind it, or (scan_only) the recurrence's kernel alone."""
    S, T = len(seg_lens), sum(seg_lens)
    ctx = _ctx(seg_lens, [0] * S)
    if kind == "gla":
        H, dk, dv, R = TUB_GLA["heads"], TUB_GLA["dim"], TUB_GLA["vdim"], TUB_GLA["rank"]
    else:
        H, dk, dv, R = TUB_RIGHT["heads"], TUB_RIGHT["dim"], TUB_RIGHT["dim"], TUB_RIGHT["rank"]
    n_state = ops.channel_scan_state_floats(H, dk, dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * n_state * 4)) + 1))
    states = torch.zeros(copies, S, n_state, device="cuda", dtype=torch.float32)
    f32 = dict(device="cuda", dtype=torch.float32)
    q, k, a = (torch.randn(T, H * dk, **f32) * 0.1 for _ in range(3))
    v, g = torch.randn(T, H * dv, **f32), torch.randn(T, H * dv, **f32)
    low, w2, wb = torch.randn(T, R, **f32), torch.randn(R, H * dk, **f32) * 0.1, torch.randn(H * dk, **f32) + 3
    nw = torch.ones(H * dv, **f32)
    w, u, au = (torch.empty(T, H * dk, **f32) for _ in range(3))
    y = torch.empty(T, H * dv, **f32)
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)

    ops.channel_gates(w, low, w2, wb, kind != "gla", ops.GATE_POW_SIGMOID if kind == "gla" else ops.GATE_EXP_NEG_SIGMOID, 0.125 if kind == "gla" else 0.6065)
    ops.unit_keys(u, au, k, a, wb, H, dk, 1e-6)

    def run(i):
        if scan_only:
            rem = kind != "gla"
            ops.channel_scan(y, q, k, v, w, au if rem else None, u if rem else None, 1.0, states[i % copies], ctx, H, dk, dv)
        elif kind == "gla":
            ops.channel_gates(w, low, w2, wb, False, ops.GATE_POW_SIGMOID, 1.0 / 8.0)
            ops.channel_scan(y, q, k, v, w, None, None, dk ** -0.5, states[i % copies], ctx, H, dk, dv)
            ops.head_norm_gate(out, y, g, nw, H, 1e-5, ops.HEAD_GATE_SILU)
        else:
            ops.channel_gates(w, low, w2, wb, True, ops.GATE_EXP_NEG_SIGMOID, 0.6065)
            ops.unit_keys(u, au, k, a, wb, H, dk, 1e-6)
            ops.channel_scan(y, q, k, v, w, au, u, 1.0, states[i % copies], ctx, H, dk, dv)
            ops.head_norm_gate(out, y, g, nw, H, 1e-5, ops.HEAD_GATE_SIGMOID)

    us = kb.timed_chain(run, launches=6)
    if scan_only:
        vecs = (3 if kind == "gla" else 5) * H * dk + 2 * H * dv
        return kb._figures(us, 2 * S * n_state * 4 + T * vecs * 4, (4.0 if kind == "gla" else 8.0) * T * H * dk * dv, peaks)
    vecs = (3 if kind == "gla" else 4) * H * dk + 2 * H * dv
    nbytes = 2 * S * n_state * 4 + T * vecs * 4 + T * H * dv * 2
    return kb._figures(us, nbytes, (4.0 if kind == "gla" else 8.0) * T * H * dk * dv, peaks)


def run_tubazen(args, peaks) -> dict:
    n_layers = 2 * args.layers_per_kind
    res = {"tubazen": model_throughput(tubazen_config(args.layers_per_kind), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup),
           "llama_equal_size": model_throughput(tubazen_llama_config(n_layers), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup)}
    T, B, C = args.prefill_tokens, args.batch, args.ctx
    res["kernels"] = {
        f"bias_attention_prefill_t{T}": bias_attention_case([T], T, peaks),
        f"bias_attention_decode_b{B}_ctx{C}": bias_attention_case([1] * B, C, peaks),
        f"bias_prepare_t{T}": bias_prepare_case(T, peaks), f"bias_prepare_t{B}": bias_prepare_case(B, peaks),
        f"gla_scan_prefill_t{T}": channel_scan_case("gla", [T], peaks), f"gla_scan_decode_b{B}": channel_scan_case("gla", [1] * B, peaks),
        f"delta_scan_prefill_t{T}": channel_scan_case("delta", [T], peaks), f"delta_scan_decode_b{B}": channel_scan_case("delta", [1] * B, peaks),
        # the recurrence's kernel alone, as the other designs' recurrences are timed
        f"gla_scan_alone_prefill_t{T}": channel_scan_case("gla", [T], peaks, True), f"gla_scan_alone_decode_b{B}": channel_scan_case("gla", [1] * B, peaks, True),
        f"delta_scan_alone_prefill_t{T}": channel_scan_case("delta", [T], peaks, True),
        f"delta_scan_alone_decode_b{B}": channel_scan_case("delta", [1] * B, peaks, True),
    }
    # the like kernels of the other designs: the differential attention and the recurrences with one decay a head
    res["like_kernels"] = {
        f"diff_attention_prefill_t{T}": diff_attention_case([T], T, peaks), f"diff_attention_decode_b{B}_ctx{C}": diff_attention_case([1] * B, C, peaks),
        f"mlstm_scan_prefill_t{T}": scan_case("mlstm", [T], peaks), f"mlstm_scan_decode_b{B}": scan_case("mlstm", [1] * B, peaks),
        f"mamba2_scan_prefill_t{T}": scan_case("mamba2", [T], peaks), f"mamba2_scan_decode_b{B}": scan_case("mamba2", [1] * B, peaks),
    }
    from .config import LlamaConfig
    like = kb.headline_kernels(LlamaConfig.from_dict(tubazen_llama_config(n_layers)), B, C, T, peaks)
    ops.check_kernel_errors()
    res["llama_kernels"] = {k: v for k, v in like.items() if "attention" in k or "gate_up" in k or "down" in k}
    return res


# ------------------------------------------------------------------ Lugizen
# Latent attention as above with a 768-wide latent for the queries and a window of 1,024; a delta rule of 16 value heads of 128 on
# 8 query/key heads of 128 with convolutions of four taps and low-rank decays and gates of rank 64; rotary attention with
# unit-normed queries and keys, 16 heads of 128 on 4 key/value heads, values blended between layers; 64 experts of 1,408 of which
# 6 serve a token, or a dense feed-forward of the same active size; a convolution of four taps ahead of every mixer.
LUG_LATENT = dict(ATTN, q_rank=768, mask={"size": 1024})
LUG_DELTA = {"heads": 16, "kv_heads": 8, "dim": 128, "vdim": 128, "conv": 4, "decay_rank": 64, "gate_rank": 64}
LUG_ATTN = {"heads": 16, "kv_heads": 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "rot": {"base": 10000.0, "dims": 64}, "v_mix": True}
LUG_MOE = {"kind": "moe", "expert": {"ff": 1408}, "router": {"experts": 64, "top": 6}}
LUG_DENSE = {"kind": "dense", "ff": 6 * 1408}


def lugizen_config(layers_per_kind: int) -> dict:
    kinds = [("latent_attention", LUG_LATENT, LUG_DENSE), ("channel_delta", LUG_DELTA, LUG_MOE), ("attention", LUG_ATTN, LUG_MOE)]
    layers = [{"type": k, "mixer": m, "mlp": f} for _ in range(layers_per_kind) for k, m, f in kinds]
    return {"architecture": "Lugizen", "vocab": VOCAB, "width": WIDTH, "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "layers": layers}


def lugizen_llama_config(n_layers: int) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "vocab_size": VOCAB, "hidden_size": WIDTH, "intermediate_size": LUG_DENSE["ff"],
            "num_hidden_layers": n_layers, "num_attention_heads": 16, "num_key_value_heads": 4, "head_dim": 128,
            "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "tie_word_embeddings": False}


def plain_attention_case(seg_lens, ctx_len, peaks, page=16) -> dict:
    """Softmax attention over cache rows [keys | values] without a bias table (the preparing kernel excluded)."""
    a = LUG_ATTN
    H, G, n, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    S, T = len(seg_lens), sum(seg_lens)
    blocks = -(-ctx_len // page)
    width = G * (n + dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * ctx_len * width * 2)) + 1))
    caches = torch.randn(copies, S * blocks + 1, page, width, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(S * blocks, dtype=torch.int32, device="cuda").view(S, blocks)
    ctx = _ctx(seg_lens, [ctx_len - m for m in seg_lens])
    ctx.seg_len, ctx.seg_start_pos, ctx.max_ctx_len, ctx.captured = list(seg_lens), [ctx_len - m for m in seg_lens], ctx_len, False
    ctx.seg_pos0 = torch.tensor(ctx.seg_start_pos, dtype=torch.int32, device="cuda")
    q = torch.randn(T, H * n, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)
    none = torch.zeros(H, 1, device="cuda", dtype=torch.float32)
    us = kb.timed_chain(lambda i: ops.bias_attention(out, q, caches[i % copies], ctx, table, H, G, n, dv, page, a["scale"], None, None, None,
                                                     1.0, table_of_distances=none), launches=8)
    pairs = sum(m * (ctx_len - m) + m * (m + 1) // 2 for m in seg_lens)
    return kb._figures(us, S * ctx_len * width * 2 + (q.numel() + out.numel()) * 2, H * pairs * (2.0 * n + 2.0 * dv), peaks)


def rot_norm_prepare_case(T, peaks, page=16) -> dict:
    """Rotation, unit norms, temperature, blended values and the cache write of T tokens of one request."""
    a = LUG_ATTN
    H, G, n, dv, rot = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["rot"]["dims"]
    cols, width = (H + G) * n + G * dv, G * (n + dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (T * (cols * 4 + G * dv * 4 + width * 2 + H * n * 2))) + 1))
    projs = torch.randn(copies, T, cols, device="cuda", dtype=torch.float32)
    firsts = torch.randn(copies, T, G * dv, device="cuda", dtype=torch.float32)
    blocks = -(-T // page)
    caches = torch.zeros(copies, blocks + 1, page, width, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(blocks, dtype=torch.int32, device="cuda").view(1, blocks)
    ctx = _ctx([T], [0])
    ang = torch.arange(T, device="cuda", dtype=torch.float32)[:, None] * torch.rand(rot // 2, device="cuda")[None, :]
    cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
    temp = torch.rand(H, device="cuda") + 0.5
    q = torch.empty(copies, T, H * n, device="cuda", dtype=torch.bfloat16)
    us = kb.timed_chain(lambda i: ops.rot_norm_prepare(q[i % copies], projs[i % copies], 0, H * n, (H + G) * n, caches[i % copies], cos_sin, rot, True,
                                                       1e-5, temp, firsts[i % copies], 0.4, ctx, table, H, G, n, dv, page), launches=8)
    return kb._figures(us, T * (cols * 4 + G * dv * 4 + width * 2 + H * n * 2), 0.0, peaks)


def channel_delta_case(seg_lens, peaks, scan_only=False) -> dict:
    """The delta rule on the decayed state: its chain (convolutions with SiLU, decays, gate pre-activations, operands, recurrence,
    norm and gate), or (scan_only) the recurrence's kernel alone."""
    m = LUG_DELTA
    H, G, dk, dv, taps, ra, rg = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], m["decay_rank"], m["gate_rank"]
    S, T = len(seg_lens), sum(seg_lens)
    ctx = _ctx(seg_lens, [0] * S)
    C = 2 * G * dk + H * dv
    n_state = ops.channel_scan_state_floats(H, dk, dv)
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (S * n_state * 4)) + 1))
    states = torch.zeros(copies, S, n_state, device="cuda", dtype=torch.float32)
    tails = torch.zeros(S, (taps - 1) * C, device="cuda", dtype=torch.float32)
    f32 = dict(device="cuda", dtype=torch.float32)
    proj = torch.randn(T, C + H + ra + rg, **f32) * 0.3
    conv_w = torch.randn(C, taps, **f32) * 0.3
    a_up, dt_bias, rate = torch.randn(ra, H * dk, **f32) * 0.1, torch.randn(H * dk, **f32) - 2, torch.rand(H * dk, **f32)
    g_up, nw = torch.randn(rg, H * dv, **f32) * 0.1, torch.ones(H * dv, **f32)
    conv, decay, gate = torch.empty(T, C, **f32), torch.empty(T, H * dk, **f32), torch.empty(T, H * dv, **f32)
    qh, kb_, ug = (torch.empty(T, H * dk, **f32) for _ in range(3))
    y = torch.empty(T, H * dv, **f32)
    out = torch.empty(T, H * dv, device="cuda", dtype=torch.bfloat16)

    def prepare():
        ops.conv_state(conv, proj[:, :C], conv_w, None, tails, ctx, act=True)
        ops.channel_gates(decay, proj[:, C + H: C + H + ra], a_up, dt_bias, False, ops.GATE_EXP_NEG_SOFTPLUS, 0.0, rate=rate)
        ops.channel_gates(gate, proj[:, C + H + ra:], g_up, None, False, ops.GATE_LINEAR, 0.0)
        ops.delta_operands(qh, kb_, ug, conv[:, : G * dk], conv[:, G * dk: 2 * G * dk], proj[:, C: C + H], decay, H, G, dk, 1e-6, dk ** -0.5)
    prepare()

    def run(i):
        if not scan_only:
            prepare()
        ops.channel_scan(y, qh, kb_, conv[:, 2 * G * dk:], decay, kb_, ug, 1.0, states[i % copies], ctx, H, dk, dv)
        if not scan_only:
            ops.head_norm_gate(out, y, gate, nw, H, 1e-5, ops.HEAD_GATE_SIGMOID)

    us = kb.timed_chain(run, launches=6)
    vecs = 4 * H * dk + 2 * H * dv                           # the scan reads decay, written key, reading key, query and value; writes the output
    nbytes = 2 * S * n_state * 4 + T * vecs * 4
    if not scan_only:
        nbytes += T * ((C + H + ra + rg) * 4 + H * dv * 2)
    return kb._figures(us, nbytes, 8.0 * T * H * dk * dv, peaks)


def stream_passes_case(T, peaks) -> dict:
    """The two passes a post-norm layer makes over the stream beside its products: the convolution ahead of the mixer (float32 stream
    in, compute type out) and the norm of a sublayer's output added to the stream (with the stream's copy in the compute type)."""
    d, taps = WIDTH, 4
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (T * d * 12)) + 1))
    res = torch.randn(copies, T, d, device="cuda", dtype=torch.float32)
    y = torch.randn(copies, T, d, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(copies, T, d, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(d, taps, device="cuda", dtype=torch.float32) * 0.3
    g = torch.ones(d, device="cuda", dtype=torch.float32)
    tails = torch.zeros(1, (taps - 1) * d, device="cuda", dtype=torch.float32)
    ctx = _ctx([T], [0])
    conv_us = kb.timed_chain(lambda i: ops.conv_state(h[i % copies], res[i % copies], w, None, tails, ctx, act=False, add_input=True), launches=8)
    norm_us = kb.timed_chain(lambda i: ops.post_rmsnorm_add(res[i % copies], y[i % copies], g, 1e-5, cast=h[i % copies]), launches=8)
    return {"conv_input": kb._figures(conv_us, T * d * 6, 0.0, peaks), "norm_on_output": kb._figures(norm_us, T * d * 12, 0.0, peaks)}


def add_rmsnorm_case(T, peaks) -> dict:
    """The pre-norm decoders' pass over the stream: the pending delta added and the normed rows written."""
    d = WIDTH
    copies = max(2, min(8, int(2.5 * kb.L2_BYTES // (T * d * 12)) + 1))
    res = torch.randn(copies, T, d, device="cuda", dtype=torch.float32)
    y = torch.randn(copies, T, d, device="cuda", dtype=torch.bfloat16)
    h = torch.empty(copies, T, d, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(d, device="cuda", dtype=torch.float32)
    us = kb.timed_chain(lambda i: ops.add_rmsnorm(h[i % copies], res[i % copies], y[i % copies], g, 1e-5), launches=8)
    return kb._figures(us, T * d * 12, 0.0, peaks)


def run_lugizen(args, peaks) -> dict:
    n_layers = 3 * args.layers_per_kind
    res = {"lugizen": model_throughput(lugizen_config(args.layers_per_kind), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup),
           "deganex_equal_size": model_throughput(deganex_config(args.layers_per_kind), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup),
           "llama_equal_size": model_throughput(lugizen_llama_config(n_layers), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup)}
    T, B, C = args.prefill_tokens, args.batch, args.ctx
    W = LUG_LATENT["mask"]["size"]
    res["kernels"] = {
        f"latent_attention_window{W}_prefill_t{T}": latent_attention_case([T], T, peaks, window=W, gated=False),
        f"latent_attention_window{W}_decode_b{B}_ctx{C}": latent_attention_case([1] * B, C, peaks, window=W, gated=False),
        f"attention_prefill_t{T}": plain_attention_case([T], T, peaks), f"attention_decode_b{B}_ctx{C}": plain_attention_case([1] * B, C, peaks),
        f"rot_norm_prepare_t{T}": rot_norm_prepare_case(T, peaks), f"rot_norm_prepare_t{B}": rot_norm_prepare_case(B, peaks),
        f"channel_delta_prefill_t{T}": channel_delta_case([T], peaks), f"channel_delta_decode_b{B}": channel_delta_case([1] * B, peaks),
        f"channel_delta_scan_alone_prefill_t{T}": channel_delta_case([T], peaks, True),
        f"channel_delta_scan_alone_decode_b{B}": channel_delta_case([1] * B, peaks, True),
        f"experts_prefill_t{T}": experts_case(T, peaks), f"experts_decode_b{B}": experts_case(B, peaks),
        f"stream_passes_t{T}": stream_passes_case(T, peaks), f"stream_passes_t{B}": stream_passes_case(B, peaks),
    }
    # the like kernels of the closest designs: Deganex's latent attention (no window, gated) and experts (the same kernels), Tubazen's
    # attention with a distance bias, its preparing kernel and its delta rule's chain, the pre-norm decoders' norm pass
    res["like_kernels"] = {
        f"latent_attention_prefill_t{T}": latent_attention_case([T], T, peaks), f"latent_attention_decode_b{B}_ctx{C}": latent_attention_case([1] * B, C, peaks),
        f"bias_attention_prefill_t{T}": bias_attention_case([T], T, peaks), f"bias_attention_decode_b{B}_ctx{C}": bias_attention_case([1] * B, C, peaks),
        f"bias_prepare_t{T}": bias_prepare_case(T, peaks), f"bias_prepare_t{B}": bias_prepare_case(B, peaks),
        f"delta_scan_prefill_t{T}": channel_scan_case("delta", [T], peaks), f"delta_scan_decode_b{B}": channel_scan_case("delta", [1] * B, peaks),
        f"delta_scan_alone_prefill_t{T}": channel_scan_case("delta", [T], peaks, True),
        f"delta_scan_alone_decode_b{B}": channel_scan_case("delta", [1] * B, peaks, True),
        f"add_rmsnorm_t{T}": add_rmsnorm_case(T, peaks), f"add_rmsnorm_t{B}": add_rmsnorm_case(B, peaks),
    }
    from .config import LlamaConfig
    like = kb.headline_kernels(LlamaConfig.from_dict(lugizen_llama_config(n_layers)), B, C, T, peaks)
    ops.check_kernel_errors()
    res["llama_kernels"] = {k: v for k, v in like.items() if "attention" in k or "gate_up" in k or "down" in k}
    return res


def run(args, peaks) -> dict:
    n_layers = 3 * args.layers_per_kind
    res = {"deganex": model_throughput(deganex_config(args.layers_per_kind), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup),
           "llama_equal_size": model_throughput(llama_config(n_layers), args.batch, args.ctx, args.prefill_tokens, args.steps, args.warmup)}
    T, B, C = args.prefill_tokens, args.batch, args.ctx
    kernels = {
        f"latent_attention_prefill_t{T}": latent_attention_case([T], T, peaks),
        f"latent_attention_decode_b{B}_ctx{C}": latent_attention_case([1] * B, C, peaks),
        f"mlstm_scan_prefill_t{T}": scan_case("mlstm", [T], peaks), f"mlstm_scan_decode_b{B}": scan_case("mlstm", [1] * B, peaks),
        f"mamba2_scan_prefill_t{T}": scan_case("mamba2", [T], peaks), f"mamba2_scan_decode_b{B}": scan_case("mamba2", [1] * B, peaks),
        f"experts_prefill_t{T}": experts_case(T, peaks), f"experts_decode_b{B}": experts_case(B, peaks),
    }
    from .config import LlamaConfig
    like = kb.headline_kernels(LlamaConfig.from_dict(llama_config(n_layers)), B, C, T, peaks)
    ops.check_kernel_errors()
    res["kernels"] = kernels
    res["llama_kernels"] = {k: v for k, v in like.items() if "attention" in k or "gate_up" in k or "down" in k}
    return res


def main(argv=None, peaks=None, extra=None) -> int:
    """extra: a callable whose dict (the clocks sampled during the run, for instance) joins the JSON line."""
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--design", default="deganex", choices=["deganex", "lotirax", "tubazen", "lugizen"])
    ap.add_argument("--layers-per-kind", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    args, _ = ap.parse_known_args(argv)
    peaks = peaks or {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if args.design == "lotirax":
        res, model = run_lotirax(args, peaks), f"Lotirax, width {WIDTH}, 4 layers of which 2 run twice"
    elif args.design == "tubazen":
        res, model = run_tubazen(args, peaks), f"Tubazen, width {WIDTH}, {2 * args.layers_per_kind} layers"
    elif args.design == "lugizen":
        res, model = run_lugizen(args, peaks), f"Lugizen, width {WIDTH}, {3 * args.layers_per_kind} layers"
    else:
        res, model = run(args, peaks), f"Deganex, width {WIDTH}, {3 * args.layers_per_kind} layers"
    d = res[args.design]
    if extra is not None:
        res = dict(res, **extra())
    print(json.dumps({"metric": f"{args.design}_decode_tokens_per_s", "value": d["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
                      "data": "synthetic (random weights and tokens)", "peaks": peaks,
                      "config": {"model": model, "batch": args.batch, "ctx": args.ctx,
                                 "prefill_tokens": args.prefill_tokens, "l2": "kernels alone rotate over buffers larger than L2"},
                      **res}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
