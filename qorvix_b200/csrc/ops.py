"""Python face of the CUDA kernels: each function checks its tensors and launches one kernel
of this folder on torch's current stream.  Nothing here computes on the CPU or calls a
library kernel; a missing or unbuildable library raises.
"""
from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import KernelBuildError, load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dt_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


# Every entry point's C signature.  With the types declared once, a call passes plain Python
# numbers (None for a null pointer) and ctypes builds no wrapper object per argument.
_V, _I, _F, _L = c_void_p, c_int, c_float, c_longlong
_ARGTYPES = {
    "qv_error_string": [_I],
    "qv_embed": [_V, _V, _V, _I, _I, _I, _I, _V],
    "qv_add_rmsnorm": [_V, _V, _V, _V, _V, _I, _I, _F, _I, _I, _I, _V],
    "qv_rope_kv_write": [_V, _I, _V, _V, _I, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_swiglu": [_V, _V, _I, _I, _I, _I, _V],
    "qv_cast": [_V, _V, _L, _I, _I, _V],
    "qv_cast_rows": [_V, _L, _V, _L, _I, _I, _I, _I, _V],
    "qv_gemm_simt": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_gemm_bf16_tc": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _V, _I, _I, _V],
    "qv_packed_weight_bytes": [_I, _I],
    "qv_pack_weight_tiles": [_V, _V, _I, _I, _I, _V],
    "qv_gemm_bf16_packed": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _V, _I, _I, _V],
    "qv_gemm_bf16_qkv_rope": [_V, _V, _V, _I, _I, _I, _I, _V, _V, _I, _V, _V, _V, _I, _V, _I, _I, _I, _I, _V],
    "qv_gemm_bf16_norm": [_V, _V, _V, _I, _I, _I, _I, _I, _I, _V, _I, _V, _I, _V, _V, _V, _I, _F, _F, _V],
    "qv_gemm_bf16_set_prefill_bn": [_I],
    "qv_gemm_bf16_set_split_workspace": [_V, _V, _I],
    "qv_gemm_bf16_split_slot_bytes": [],
    "qv_attention_generic": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V],
    "qv_attn_prefill_bf16": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V],
    "qv_attn_prefill_tc": [_V, _I, _V, _I, _I, _V, _L, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _V, _V],
    "qv_attn_set_decode_variant": [_I],
    "qv_attn_set_error_word": [_V],
    "qv_attn_decode_bf16": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V, _V],
    "qv_embed_pair": [_V, _V, _V, _V, _V, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_add_rmsnorm2": [_V, _V, _V, _V, _V, _V, _I, _I, _F, _I, _I, _V],
    "qv_sum2": [_V, _V, _V, _L, _I, _I, _V],
    "qv_softcap": [_V, _L, _F, _V],
    "qv_latent_prepare": [_V, _I, _V, _I, _I, _V, _V, _F, _V, _I, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_latent_attention_generic": [_V, _I, _V, _I, _V, _I, _V, _V, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _V],
    "qv_latent_tc_workspace_bytes": [_I, _I, _I, _I, _I],
    "qv_latent_attention_tc": [_V, _I, _V, _I, _V, _I, _V, _V, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _V, _V],
    "qv_conv_state": [_V, _I, _V, _I, _V, _V, _V, _L, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_linear_scan_state_floats": [_I, _I, _I, _I],
    "qv_linear_scan": [_I, _V, _I, _V, _I, _I, _V, _I, _V, _I, _V, _I, _V, _I, _V, _V, _V, _F, _F, _V, _L, _V, _V, _I, _I, _I, _I, _I, _V],
    "qv_gated_group_norm": [_V, _I, _V, _I, _V, _I, _V, _I, _I, _I, _F, _I, _I, _V],
    "qv_moe_route": [_V, _V, _V, _V, _I, _V, _V, _V, _I, _I, _I, _I, _I, _I, _V],
    "qv_moe_max_tiles": [_I, _I, _I],
    "qv_moe_tile_rows": [_I],
    "qv_moe_group": [_V, _V, _V, _V, _V, _I, _I, _I, _I, _V],
    "qv_moe_experts_tc": [_I, _V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _V],
    "qv_moe_experts": [_I, _V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _V],
    "qv_moe_combine": [_V, _V, _V, _V, _V, _V, _V, _I, _I, _I, _I, _V, _V, _V],
    "qv_moe_route_table": [_V, _V, _V, _V, _I, _I, _I, _I, _V],
    "qv_scale_sum2": [_V, _V, _V, _V, _V, _I, _I, _I, _I, _V],
    "qv_stream_concat": [_V, _V, _V, _V, _I, _I, _I, _I, _V],
    "qv_add_vector": [_V, _V, _I, _I, _V],
    "qv_activation": [_V, _V, _L, _I, _I, _V],
    "qv_diff_prepare": [_V, _I, _V, _I, _V, _V, _V, _F, _V, _I, _V, _V, _V, _I, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_diff_partial_floats": [_I],
    "qv_diff_attention_tc": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F, _V, _I, _V],
    "qv_diff_attention_generic": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _F, _F, _F, _F, _I, _V],
    "qv_add_tanhnorm": [_V, _V, _V, _V, _V, _F, _V, _I, _I, _I, _I, _I, _V],
    "qv_embed_pos": [_V, _V, _V, _V, _V, _I, _I, _I, _I, _F, _V, _V, _F, _I, _V],
    "qv_glu_act": [_V, _V, _I, _I, _I, _I, _I, _V],
    "qv_sigmoid_gate": [_V, _V, _I, _V, _I, _V, _I, _I, _I, _V],
    "qv_depth_mix": [_V, _V, _V, _L, _V, _I, _V],
    "qv_scale": [_V, _L, _F, _V],
    "qv_channel_gates": [_V, _I, _V, _I, _V, _V, _I, _I, _I, _I, _I, _F, _V, _V],
    "qv_delta_operands": [_V, _V, _V, _V, _I, _V, _I, _V, _I, _V, _I, _I, _I, _I, _I, _F, _F, _V],
    "qv_post_rmsnorm_add": [_V, _V, _I, _V, _F, _V, _I, _I, _I, _I, _V],
    "qv_rmsnorm_rows": [_V, _I, _V, _I, _V, _F, _I, _I, _I, _I, _V],
    "qv_rot_norm_prepare": [_V, _I, _V, _I, _I, _I, _I, _V, _V, _I, _I, _I, _F, _V, _V, _I, _F, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _V],
    "qv_unit_keys": [_V, _V, _V, _I, _V, _I, _V, _I, _I, _I, _F, _V],
    "qv_channel_scan_state_floats": [_I, _I, _I],
    "qv_channel_scan": [_V, _I, _V, _I, _V, _I, _V, _I, _V, _I, _V, _I, _V, _I, _F, _V, _L, _V, _V, _I, _I, _I, _I, _I, _V],
    "qv_head_norm_gate": [_V, _I, _V, _I, _V, _I, _V, _I, _I, _I, _F, _I, _F, _I, _V],
    "qv_bias_attn_prepare": [_V, _I, _V, _I, _I, _I, _I, _V, _V, _V, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _V],
    "qv_bias_attention_generic": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _F, _V, _I, _V, _V, _I, _F, _I, _V],
    "qv_bias_attention_mma": [_V, _I, _V, _I, _V, _V, _V, _V, _I, _I, _I, _I, _I, _I, _I, _I, _F, _V, _I, _V, _I, _F, _V, _I, _I, _V],
    "qv_argmax": [_V, _V, _I, _I, _L, _V],
    "qv_sample": [_V, _V, _I, _I, _L, _V, _V, _V, _V, _V, _V, _I, _V, _V, _V, _V],
}
_RESTYPES = {"qv_error_string": ctypes.c_char_p, "qv_packed_weight_bytes": c_longlong, "qv_gemm_bf16_split_slot_bytes": c_longlong,
             "qv_linear_scan_state_floats": c_longlong, "qv_latent_tc_workspace_bytes": c_longlong, "qv_diff_partial_floats": c_longlong,
             "qv_channel_scan_state_floats": c_longlong}
_typed_libs = {}


def _lib(name: str):
    """The library `name` (compiled and loaded on first use) with its entry points' types declared."""
    lib = _typed_libs.get(name)
    if lib is None:
        lib = load_library(name)
        for fn, types in _ARGTYPES.items():
            if hasattr(lib, fn):
                f = getattr(lib, fn)
                f.argtypes = types
                f.restype = _RESTYPES.get(fn, c_int)
        _typed_libs[name] = lib
    return lib


def _ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (the raw getters cost a fraction of building a Stream object)."""
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must live on a CUDA device; there is no CPU path")


_launches = 0


def launch_count() -> int:
    """Kernels of this package launched so far (replays of captured steps add their kernels)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(rc: int, what: str):
    global _launches
    _launches += 1
    if rc != 0:
        lib = _lib("elementwise")
        msg = lib.qv_error_string(rc).decode()
        raise KernelError(f"{what}: {msg} (code {rc})")


def _i32(t, name):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------ elementwise

def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> None:
    """out[t] (float32) = table[ids[t]]."""
    _need_cuda(out, table, ids)
    _i32(ids, "ids")
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    assert table.shape[1] == d and ids.numel() >= T
    rc = _lib("elementwise").qv_embed(
        _ptr(out), _ptr(table), _ptr(ids), T, d, table.shape[0], dt_code(table.dtype), _stream())
    _check(rc, "embed")


def add_rmsnorm(out, residual, delta, weight, eps: float, row_idx=None, write_residual=True) -> None:
    """x = residual[s] (+ delta[s]); residual[s] = x if write_residual; out[r] = rmsnorm(x) * weight
    with s = row_idx[r] if row_idx is given, else r.  residual and weight are float32."""
    _need_cuda(out, residual, delta, weight, row_idx)
    rows, d = out.shape
    assert residual.dtype == torch.float32 and weight.dtype == torch.float32
    assert residual.is_contiguous() and out.is_contiguous() and weight.numel() == d and residual.shape[1] == d
    if delta is not None:
        assert delta.is_contiguous() and delta.shape == residual.shape
    if row_idx is not None:
        _i32(row_idx, "row_idx")
        assert row_idx.numel() >= rows
        write_residual = False
    else:
        assert residual.shape[0] >= rows
    ddt = dt_code(delta.dtype) if delta is not None else dt_code(out.dtype)
    rc = _lib("elementwise").qv_add_rmsnorm(
        _ptr(out), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(row_idx), rows, d, eps, 1 if (write_residual and
        delta is not None) else 0, ddt, dt_code(out.dtype), _stream())
    _check(rc, "add_rmsnorm")


def rope_kv_write(qkv, cache_layer, cos_sin, tok_pos, tok_seg, block_table, H, Hkv, hd, rot, page) -> None:
    """Rotates q (in place) and k, writes k and v of every token into its cache slot.
    qkv [T, (H+2Hkv)*hd]; cache_layer [pages, 2, Hkv, page, hd] or None; cos_sin [rows, rot/2, 2] float32."""
    _need_cuda(qkv, cache_layer, cos_sin, tok_pos, tok_seg, block_table)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == (H + 2 * Hkv) * hd
    if cos_sin is None:
        assert rot == 0, "a rotation needs its cos/sin table"
    else:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == rot
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    if cache_layer is not None:
        assert cache_layer.dtype == qkv.dtype and cache_layer.is_contiguous()
        assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    rc = _lib("elementwise").qv_rope_kv_write(
        _ptr(qkv), qkv.stride(0), _ptr(cache_layer), _ptr(cos_sin), cos_sin.shape[0] if cos_sin is not None else 1,
        _ptr(tok_pos), _ptr(tok_seg), _ptr(block_table), block_table.shape[-1], T, H, Hkv, hd, rot, page,
        dt_code(qkv.dtype), _stream())
    _check(rc, "rope_kv_write")


def swiglu(out, gu, interleaved: bool = False) -> None:
    """gu [T, 2f] -> out [T, f] = silu(gate) * up.  gu is [gate | up], or with `interleaved` groups of
    32 columns: 16 gate values, then the 16 up values of the same features."""
    _need_cuda(out, gu)
    T, f = out.shape
    assert gu.shape == (T, 2 * f) and gu.is_contiguous() and out.is_contiguous() and gu.dtype == out.dtype
    rc = _lib("elementwise").qv_swiglu(
        _ptr(out), _ptr(gu), T, f, 1 if interleaved else 0, dt_code(out.dtype), _stream())
    _check(rc, "swiglu")


def cast(out, src) -> None:
    _need_cuda(out, src)
    assert out.numel() == src.numel() and out.is_contiguous() and src.is_contiguous()
    rc = _lib("elementwise").qv_cast(
        _ptr(out), _ptr(src), src.numel(), dt_code(src.dtype), dt_code(out.dtype), _stream())
    _check(rc, "cast")


def cast_rows(out, src) -> None:
    """out[r, c] = src[r, c] for 2-D tensors whose rows are contiguous (any row stride), float32 or
    bfloat16 each: a dense copy of a slice, with a change of type if the two differ."""
    _need_cuda(out, src)
    assert out.dim() == 2 and out.shape == src.shape and out.stride(1) == 1 and src.stride(1) == 1
    rc = _lib("elementwise").qv_cast_rows(_ptr(out), out.stride(0), _ptr(src), src.stride(0), src.shape[0], src.shape[1],
                                          dt_code(src.dtype), dt_code(out.dtype), _stream())
    _check(rc, "cast_rows")


def embed_pair(out, table, pair, ids, ctx, last_token, buckets: int, mul_prev: int, mul_cur: int) -> None:
    """out[t] (float32) = table[ids[t]] + pair[hash of (token before, token)]; the request's first token takes
    pair's last row.  last_token [slots] int32 keeps each request's latest token between steps."""
    _need_cuda(out, table, pair, ids, last_token)
    _i32(ids, "ids"); _i32(last_token, "last_token")
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous() and pair.is_contiguous()
    assert table.shape[1] == d and pair.shape == (buckets + 1, d) and pair.dtype == table.dtype
    rc = _lib("elementwise").qv_embed_pair(
        _ptr(out), _ptr(table), _ptr(pair), _ptr(ids), _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(ctx.seg_q_start),
        _ptr(ctx.seg_slot), _ptr(last_token), T, d, table.shape[0], buckets, mul_prev, mul_cur, dt_code(table.dtype), _stream())
    _check(rc, "embed_pair")


def add_rmsnorm2(out1, out2, residual, delta, w1, w2, eps: float) -> None:
    """residual (float32) += delta; out1 = rmsnorm(residual) * w1 and out2 = rmsnorm(residual) * w2 (out2 and
    w2 may be None): the two norms of a block whose parts read the same stream, in one pass."""
    _need_cuda(out1, out2, residual, delta, w1, w2)
    rows, d = out1.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and residual.shape == (rows, d)
    assert out1.is_contiguous() and w1.dtype == torch.float32 and w1.numel() == d
    if out2 is not None:
        assert out2.is_contiguous() and out2.shape == out1.shape and out2.dtype == out1.dtype and w2.dtype == torch.float32
    if delta is not None:
        assert delta.is_contiguous() and delta.shape == residual.shape
    ddt = dt_code(delta.dtype) if delta is not None else dt_code(out1.dtype)
    rc = _lib("elementwise").qv_add_rmsnorm2(_ptr(out1), _ptr(out2), _ptr(residual), _ptr(delta), _ptr(w1), _ptr(w2), rows, d,
                                             eps, ddt, dt_code(out1.dtype), _stream())
    _check(rc, "add_rmsnorm2")


def sum2(out, a, b) -> None:
    """out (float32) = a + b, elementwise."""
    _need_cuda(out, a, b)
    assert out.dtype == torch.float32 and out.is_contiguous() and a.is_contiguous() and b.is_contiguous()
    assert a.numel() == out.numel() == b.numel()
    _check(_lib("elementwise").qv_sum2(_ptr(out), _ptr(a), _ptr(b), out.numel(), dt_code(a.dtype), dt_code(b.dtype), _stream()), "sum2")


def softcap(x, cap: float) -> None:
    """x = cap * tanh(x / cap) in place (float32)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_lib("elementwise").qv_softcap(_ptr(x), x.numel(), float(cap), _stream()), "softcap")


def scale_sum2(out, a, sa, b=None, sb=None) -> None:
    """out (float32 [T, d]) = a * sa + b * sb with per-feature factors sa, sb (float32 [d] or None); b may be None."""
    _need_cuda(out, a, sa, b, sb)
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and a.is_contiguous() and a.shape == out.shape
    assert b is None or (b.is_contiguous() and b.shape == out.shape)
    for sc in (sa, sb):
        assert sc is None or (sc.dtype == torch.float32 and sc.is_contiguous() and sc.numel() == d)
    rc = _lib("elementwise").qv_scale_sum2(_ptr(out), _ptr(a), _ptr(sa), _ptr(b), _ptr(sb), T, d, dt_code(a.dtype),
                                           dt_code(b.dtype) if b is not None else dt_code(a.dtype), _stream())
    _check(rc, "scale_sum2")


def stream_concat(out, residual, delta, x0) -> None:
    """out [T, 2d] (compute type) = [residual + delta (float32 sum; delta may be None) | x0], residual and x0 float32 [T, d]."""
    _need_cuda(out, residual, delta, x0)
    T, d = residual.shape
    assert out.shape == (T, 2 * d) and out.is_contiguous() and residual.dtype == x0.dtype == torch.float32
    assert residual.is_contiguous() and x0.is_contiguous() and x0.shape == residual.shape
    assert delta is None or (delta.is_contiguous() and delta.shape == residual.shape)
    rc = _lib("elementwise").qv_stream_concat(_ptr(out), _ptr(residual), _ptr(delta), _ptr(x0), T, d,
                                              dt_code(delta.dtype) if delta is not None else F32, dt_code(out.dtype), _stream())
    _check(rc, "stream_concat")


def add_vector(x, v) -> None:
    """x[t, :] += v (both float32), in place."""
    _need_cuda(x, v)
    assert x.dtype == v.dtype == torch.float32 and x.is_contiguous() and v.is_contiguous() and v.numel() == x.shape[1]
    _check(_lib("elementwise").qv_add_vector(_ptr(x), _ptr(v), x.shape[0], x.shape[1], _stream()), "add_vector")


ACT_RELU2, ACT_GELU_TANH = 0, 1


def activation(out, x, kind: int = ACT_RELU2) -> None:
    """out = act(x) elementwise (out may be x); kind ACT_RELU2: the square of relu, ACT_GELU_TANH: the tanh form of GELU."""
    _need_cuda(out, x)
    assert out.dtype == x.dtype and out.is_contiguous() and x.is_contiguous() and out.numel() == x.numel()
    _check(_lib("elementwise").qv_activation(_ptr(out), _ptr(x), x.numel(), kind, dt_code(x.dtype), _stream()), "activation")


def add_tanhnorm(out, residual, delta, weight, bias, alpha: float, row_idx=None) -> None:
    """residual (float32) += delta (None: nothing added); out = tanh(alpha * residual) * weight + bias.  With row_idx only
    those rows of residual + delta are normed and the residual is left as it is."""
    _need_cuda(out, residual, delta, weight, bias, row_idx)
    d = residual.shape[1]
    rows = residual.shape[0] if row_idx is None else row_idx.numel()
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (rows, d)
    assert weight.dtype == torch.float32 and weight.numel() == d and (bias is None or (bias.dtype == torch.float32 and bias.numel() == d))
    assert delta is None or (delta.is_contiguous() and delta.shape == residual.shape)
    if row_idx is not None:
        _i32(row_idx, "row_idx")
    rc = _lib("elementwise").qv_add_tanhnorm(_ptr(out), _ptr(residual), _ptr(delta), _ptr(weight), _ptr(bias), float(alpha), _ptr(row_idx),
                                             rows, d, 0 if row_idx is not None else 1, dt_code(delta.dtype) if delta is not None else F32,
                                             dt_code(out.dtype), _stream())
    _check(rc, "add_tanhnorm")


def embed_pos(out, table, pos_table, ids, tok_pos, pos_scale: float = 1.0, weight=None, bias=None, alpha: float = 1.0) -> None:
    """out[t] (float32) = table[ids[t]] + pos_scale * pos_table[tok_pos[t]]; with weight also tanh(alpha * out) * weight + bias."""
    _need_cuda(out, table, pos_table, ids, tok_pos, weight, bias)
    _i32(ids, "ids"); _i32(tok_pos, "tok_pos")
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous() and pos_table.is_contiguous()
    assert table.dtype == pos_table.dtype and table.shape[1] == d == pos_table.shape[1]
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == d and (bias is None or bias.dtype == torch.float32))
    rc = _lib("elementwise").qv_embed_pos(_ptr(out), _ptr(table), _ptr(pos_table), _ptr(ids), _ptr(tok_pos), T, d, table.shape[0],
                                          pos_table.shape[0], float(pos_scale), _ptr(weight), _ptr(bias), float(alpha),
                                          dt_code(table.dtype), _stream())
    _check(rc, "embed_pos")


GLU_SILU, GLU_GELU_TANH = 0, 1


def glu_act(out, gu, act: int, interleaved: bool = False) -> None:
    """out[t, i] = act(gate_i) * up_i; act GLU_SILU or GLU_GELU_TANH; gu is [gate | up], or with `interleaved` groups of
    32 columns: 16 gate values, then the 16 up values of the same features."""
    _need_cuda(out, gu)
    T, f = out.shape
    assert out.dtype == gu.dtype and out.is_contiguous() and gu.is_contiguous() and tuple(gu.shape) == (T, 2 * f)
    _check(_lib("elementwise").qv_glu_act(_ptr(out), _ptr(gu), T, f, act, 1 if interleaved else 0, dt_code(out.dtype), _stream()), "glu_act")


def sigmoid_gate(out, y, g, bias) -> None:
    """out (float32 [T, d]) = y * sigmoid(g + bias): y float32 or the compute type, g float32 (column slices are fine)."""
    _need_cuda(out, y, g, bias)
    T, d = out.shape
    assert out.dtype == g.dtype == torch.float32 and out.is_contiguous() and y.stride(1) == 1 and g.stride(1) == 1
    assert tuple(y.shape) == tuple(g.shape) == (T, d) and (bias is None or (bias.dtype == torch.float32 and bias.numel() == d))
    rc = _lib("elementwise").qv_sigmoid_gate(_ptr(out), _ptr(y), y.stride(0), _ptr(g), g.stride(0), _ptr(bias), T, d, dt_code(y.dtype),
                                             _stream())
    _check(rc, "sigmoid_gate")


def depth_mix(x, delta, stack, weights, count: int) -> None:
    """stack[count - 1] = x + delta (float32; delta may be None); x = sum over j < count of weights[j] * stack[j]."""
    _need_cuda(x, delta, stack, weights)
    n = x.numel()
    assert x.dtype == stack.dtype == weights.dtype == torch.float32 and x.is_contiguous() and stack.is_contiguous()
    assert stack.shape[0] >= count and stack[0].numel() == n and weights.numel() >= count
    assert delta is None or (delta.dtype == torch.float32 and delta.is_contiguous() and delta.numel() == n)
    _check(_lib("elementwise").qv_depth_mix(_ptr(x), _ptr(delta), _ptr(stack), n, _ptr(weights), count, _stream()), "depth_mix")


def scale(x, s: float) -> None:
    """x *= s in place (float32)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _check(_lib("elementwise").qv_scale(_ptr(x), x.numel(), float(s), _stream()), "scale")


def post_rmsnorm_add(residual, y, weight, eps: float, cast=None) -> None:
    """residual (float32 [T, d]) += y / rms(y) * weight, the root mean square over a row of y with eps under the root; y in the
    compute type or float32 (rows may be strided); `cast`, if given, receives the new residual in its own type."""
    _need_cuda(residual, y, weight, cast)
    T, d = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and tuple(y.shape) == (T, d) and y.stride(1) == 1
    assert weight.dtype == torch.float32 and weight.numel() == d and (cast is None or (cast.is_contiguous() and cast.shape == residual.shape))
    rc = _lib("elementwise").qv_post_rmsnorm_add(_ptr(residual), _ptr(y), y.stride(0), _ptr(weight), float(eps), _ptr(cast), T, d,
                                                 dt_code(y.dtype), dt_code(cast.dtype) if cast is not None else F32, _stream())
    _check(rc, "post_rmsnorm_add")


def rmsnorm_rows(out, x, weight, eps: float) -> None:
    """out[t] = x[t] / rms(x[t]) * weight (weight float32 or None), rows of either may be column slices; float32 arithmetic."""
    _need_cuda(out, x, weight)
    T, n = x.shape
    assert tuple(out.shape) == (T, n) and out.stride(1) == 1 and x.stride(1) == 1
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == n)
    rc = _lib("elementwise").qv_rmsnorm_rows(_ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(weight), float(eps), T, n,
                                             dt_code(x.dtype), dt_code(out.dtype), _stream())
    _check(rc, "rmsnorm_rows")


# ------------------------------------------------------------------ differential attention

def diff_prepare(q_out, proj, bias, q_weight, k_weight, eps, cos_sin, ctx, block_table, cache_layer, H, G, n, dv, rot, page) -> None:
    """Per token of proj (float32 or the compute type; columns [q: H*2n | k: G*2n | v: G*dv]): bias added, every map of q and
    k RMS-normed over n with its weight and rotated over its first `rot` entries (pairs i, i + rot/2); q -> q_out [T, H*2n],
    k and v -> the token's row of cache_layer [pages, page, G*(2n+dv)]."""
    _need_cuda(q_out, proj, bias, q_weight, k_weight, cos_sin, block_table, cache_layer)
    T = proj.shape[0]
    assert proj.stride(1) == 1 and proj.shape[1] == (H + G) * 2 * n + G * dv and q_out.stride(1) == 1 and q_out.shape == (T, H * 2 * n)
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (2 * n + dv)) and cache_layer.dtype == q_out.dtype
    assert q_weight.dtype == k_weight.dtype == torch.float32 and q_weight.numel() == k_weight.numel() == n
    assert bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == proj.shape[1])
    if rot:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == rot
    _i32(block_table, "block_table")
    rc = _lib("diff_attention").qv_diff_prepare(
        _ptr(q_out), q_out.stride(0), _ptr(proj), proj.stride(0), _ptr(bias), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos_sin),
        cos_sin.shape[0] if cos_sin is not None else 1, _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table), block_table.shape[-1],
        _ptr(cache_layer), T, H, G, n, dv, rot, page, dt_code(proj.dtype), dt_code(q_out.dtype), _stream())
    _check(rc, "diff_prepare")


def diff_attention_generic(out, q, cache_layer, ctx, block_table, H, G, n, dv, page, window, scale, lam, eps, post) -> None:
    """out[t, h*dv:(h+1)*dv] = (a1 - lam * a2) / rms * post for every token and head, a1 and a2 the head's two softmax
    maps over its request's cache rows; float32 arithmetic, any sizes (value size up to 512)."""
    _need_cuda(out, q, cache_layer, block_table)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (2 * n + dv))
    _i32(block_table, "block_table")
    rc = _lib("diff_attention").qv_diff_attention_generic(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table),
        block_table.shape[-1], T, H, G, n, dv, page, int(window), float(scale), float(lam), float(eps), float(post), dt_code(q.dtype),
        _stream())
    _check(rc, "diff_attention_generic")


def diff_attention_tc(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, G, n, dv, page, window, scale, lam,
                      eps, post, splits: int = 1) -> bool:
    """Differential attention on the tensor cores (bfloat16; map sizes up to 128 and value sizes up to 256, multiples of 8)
    for S segments that start at rows seg_q_start[s]; single tokens share a tile among the query heads of a key/value
    head, and splits > 1 (single tokens only) cuts every token's keys into slices that a second launch merges.  False, nothing written, for sizes it does not take."""
    if q.dtype != torch.bfloat16 or n % 8 or dv % 8 or n > 128 or dv > 256 or q.stride(0) % 8:
        return False
    _need_cuda(out, q, cache_layer, seg_q_start, seg_pos0, block_table)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == cache_layer.dtype == torch.bfloat16
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (2 * n + dv))
    _i32(block_table, "block_table")
    lib = _lib("diff_attention")
    partial = None
    if splits > 1:
        assert max_q_len == 1
        partial = torch.empty(S * H * splits * int(lib.qv_diff_partial_floats(dv)), device=q.device, dtype=torch.float32)
    rc = lib.qv_diff_attention_tc(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(seg_q_start), _ptr(seg_pos0),
                                  _ptr(block_table), block_table.shape[-1], S, max_q_len, H, G, n, dv, page, int(window), float(scale),
                                  float(lam), float(eps), float(post), _ptr(partial), splits, _stream())
    if rc == -2:
        return False
    _check(rc, "diff_attention_tc")
    if splits > 1:
        add_launches(1)                              # the merge of the slices
    return True


def diff_attention_splits(tokens: int, H: int, G: int, window: int, max_ctx: int) -> int:
    """Into how many slices the keys of single query tokens are cut so that a step fills the SMs (a CTA serves a token
    and a key/value head): a function of the step's shape only (a captured step keeps it).  One, where a key/value
    head has more than 16 query heads (those do not share a tile)."""
    if H // G > 16:
        return 1
    keys = min(window, max_ctx) if window > 0 else max_ctx
    blocks = max(1, -(-keys // 32))                  # the kernel's blocks of keys
    # about one CTA an SM, at least two blocks a slice, at most twelve slices (the merge reads them one after another)
    return max(1, min(sm_count() // max(tokens * G, 1), blocks // 2, 12))


def diff_attention(out, q, cache_layer, ctx, block_table, H, G, n, dv, page, window, scale, lam, eps, post) -> None:
    """Differential attention of every token of the step over its request's cache rows.  bfloat16: the tensor-core
    kernel where it takes the sizes (single tokens, which come first in a step, with tiles of 16 rows and their keys in
    slices; portions with tiles of 64 rows); float32 and other sizes: the CUDA-core kernel."""
    if q.dtype == torch.bfloat16:
        S = ctx.num_segments
        n1 = 0                                        # leading segments of one token (decoded tokens)
        while n1 < S and ctx.seg_len[n1] == 1:
            n1 += 1
        args = (H, G, n, dv, page, window, scale, lam, eps, post)
        ok = True
        if n1:
            splits = diff_attention_splits(n1, H, G, window, ctx.max_ctx_len)
            ok = diff_attention_tc(out, q, cache_layer, ctx.seg_q_start, ctx.seg_pos0, block_table, n1, 1, *args, splits=splits)
        if ok and n1 < S:
            ok = diff_attention_tc(out, q, cache_layer, ctx.seg_q_start[n1:], ctx.seg_pos0[n1:], block_table[n1:], S - n1,
                                   max(ctx.seg_len[n1:]), *args)
        if ok:
            return
    diff_attention_generic(out, q, cache_layer, ctx, block_table, H, G, n, dv, page, window, scale, lam, eps, post)


# ------------------------------------------------------------------ latent attention

def latent_prepare(proj, q, kv_off: int, cache_layer, norm_w, eps, cos_sin, ctx, block_table, H, dn, dr, rank, rot, page,
                   split_half: bool = False) -> None:
    """Per token of proj (rows [.. down: rank+dr at kv_off ..]): the latent part of the down projection RMS-normed, the
    shared key part rotated (pairs 2i, 2i+1, or i, i + rot/2 with split_half), both written to the token's row of
    cache_layer [pages, page, rank+dr]; every head's rotated query part of q [T, H*(dn+dr)] (columns of proj or a tensor
    of its own) rotated in place."""
    _need_cuda(proj, q, cache_layer, norm_w, cos_sin, block_table)
    assert proj.stride(1) == 1 and cache_layer.is_contiguous() and cache_layer.dtype == proj.dtype == q.dtype
    assert q.stride(1) == 1 and q.shape[0] == proj.shape[0] and q.shape[1] == H * (dn + dr)
    assert tuple(cache_layer.shape[1:]) == (page, rank + dr) and norm_w.dtype == torch.float32 and norm_w.numel() == rank
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == rot
    _i32(block_table, "block_table")
    rc = _lib("latent_attention").qv_latent_prepare(
        _ptr(proj), proj.stride(0), _ptr(q), q.stride(0), kv_off, _ptr(cache_layer), _ptr(norm_w), eps, _ptr(cos_sin), cos_sin.shape[0],
        _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table), block_table.shape[-1], proj.shape[0], H, dn, dr, rank, rot, page,
        1 if split_half else 0, dt_code(proj.dtype), _stream())
    _check(rc, "latent_prepare")


def latent_attention_generic(out, q, gate, cache_layer, wuk, wuv, ctx, block_table, H, dn, dr, dv, rank, page, window, scale) -> None:
    """out[t, h*dv:(h+1)*dv] = gate * Wuv_h (softmax-weighted latent) for every token and head, the query carried
    into the latent space by Wuk_h; float32 arithmetic, any sizes.  q: [T, H*(dn+dr)] (a column slice is fine)."""
    _need_cuda(out, q, gate, cache_layer, wuk, wuv, block_table)
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, rank + dr)
    assert wuk.is_contiguous() and tuple(wuk.shape) == (H * dn, rank) and wuv.is_contiguous() and tuple(wuv.shape) == (H * dv, rank)
    assert wuk.dtype == wuv.dtype
    if gate is not None:
        assert gate.stride(1) == 1 and gate.dtype == out.dtype
    _i32(block_table, "block_table")
    rc = _lib("latent_attention").qv_latent_attention_generic(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(cache_layer),
        _ptr(wuk), _ptr(wuv), _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table), block_table.shape[-1], q.shape[0], H, dn, dr,
        dv, rank, page, window, scale, dt_code(q.dtype), dt_code(wuk.dtype), _stream())
    _check(rc, "latent_attention_generic")


def latent_attention_splits(ctx, H: int) -> int:
    """Into how many slices the keys of a tile of 32 (token, head) rows are cut so that a step fills the SMs (one CTA
    each): a function of the step's shape only (a captured step keeps it)."""
    tiles = sum(-(-n * H // 32) for n in ctx.seg_len)
    blocks = max(1, -(-int(ctx.max_ctx_len) // 64))
    return max(1, min(sm_count() // max(tiles, 1), blocks))


def latent_attention_tc(out, q, gate, cache_layer, wuk_t, wuv, ctx, block_table, H, dn, dr, dv, rank, page, window, scale) -> bool:
    """Latent attention on the tensor cores (bfloat16; rank a multiple of 64 up to 512, rotated part a multiple of 16,
    unrotated part a multiple of 8).  wuk_t: the heads' key matrices transposed, [H, rank, dn].  False, nothing
    written, for other sizes."""
    if (q.dtype != torch.bfloat16 or wuk_t is None or wuk_t.dtype != torch.bfloat16 or wuv.dtype != torch.bfloat16 or rank % 64
            or rank > 512 or rank // 64 in (5, 7) or dr % 16 or dn % 8 or q.stride(0) % 8
            or (gate is not None and gate.dtype != torch.bfloat16)):
        return False
    _need_cuda(out, q, gate, cache_layer, wuk_t, wuv, block_table)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == cache_layer.dtype == torch.bfloat16
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, rank + dr)
    assert wuk_t.is_contiguous() and tuple(wuk_t.shape) == (H, rank, dn) and wuv.is_contiguous() and tuple(wuv.shape) == (H * dv, rank)
    _i32(block_table, "block_table")
    T = q.shape[0]
    splits = latent_attention_splits(ctx, H)
    lib = _lib("latent_attention")
    ws = torch.empty(int(lib.qv_latent_tc_workspace_bytes(T, H, dr, rank, splits)), device=q.device, dtype=torch.uint8)
    rc = lib.qv_latent_attention_tc(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(cache_layer),
        _ptr(wuk_t), _ptr(wuv), _ptr(ctx.seg_q_start), _ptr(ctx.seg_pos0), _ptr(block_table), block_table.shape[-1], T,
        ctx.num_segments, ctx.max_q_len, H, dn, dr, dv, rank, page, window, scale, splits, _ptr(ws), _stream())
    if rc == -2:
        return False
    _check(rc, "latent_attention_tc")
    add_launches(3)                                  # the queries' move into the latent space, the merge, the value matrices
    return True


def latent_attention(out, q, gate, cache_layer, wuk, wuv, ctx, block_table, H, dn, dr, dv, rank, page, window, scale, wuk_t=None) -> None:
    """Latent attention of every token of the step: the tensor-core kernels for bfloat16 where they take the sizes (and
    the transposed key matrices wuk_t [H, rank, dn] are given), else (and for float32) the CUDA-core kernel."""
    if q.dtype == torch.bfloat16 and latent_attention_tc(out, q, gate, cache_layer, wuk_t, wuv, ctx, block_table, H, dn, dr, dv, rank,
                                                         page, window, scale):
        return
    latent_attention_generic(out, q, gate, cache_layer, wuk, wuv, ctx, block_table, H, dn, dr, dv, rank, page, window, scale)


# ------------------------------------------------------------------ recurrent mixers

SCAN_GATED_MAX, SCAN_DECAY = 0, 1


def conv_state(out, x, w, bias, tail, ctx, act: bool = True, add_input: bool = False) -> None:
    """out = f(causal convolution of x along each request's tokens + bias), per channel, f SiLU or (act False) the
    identity; with add_input the current input is added (out = x + f(conv)); w [channels, taps] float32 with the
    current token's tap last; tail [slots, (taps-1)*channels] float32 keeps each request's last inputs and is brought
    up to date.  x and out may differ in type (float32 or bfloat16 each)."""
    _need_cuda(out, x, w, bias, tail)
    T, C = x.shape
    assert out.shape == x.shape and out.stride(1) == 1 and x.stride(1) == 1
    assert w.dtype == torch.float32 and w.is_contiguous() and w.shape[0] == C and tail.dtype == torch.float32
    taps = w.shape[1]
    assert tail.stride(-1) == 1 and tail.shape[-1] >= (taps - 1) * C
    rc = _lib("recurrent").qv_conv_state(
        _ptr(out), out.stride(0), _ptr(x), x.stride(0), _ptr(w), _ptr(bias), _ptr(tail), tail.stride(0), _ptr(ctx.seg_q_start),
        _ptr(ctx.seg_slot), ctx.num_segments, ctx.max_q_len, C, taps, dt_code(x.dtype), dt_code(out.dtype), 1 if act else 0,
        1 if add_input else 0, _stream())
    _check(rc, "conv_state")


def linear_scan_state_floats(kind: int, H: int, dk: int, dv: int) -> int:
    """How many float32 values linear_scan keeps per request for H heads of dk x dv."""
    return int(_lib("recurrent").qv_linear_scan_state_floats(kind, H, dk, dv))


def linear_scan(kind, out, q, k, v, g1, g2, p1, p2, p3, cap, q_scale, state, ctx, H, dk, dv, q_group=1) -> None:
    """Per request and head: S = a S + b k v^T, out = S^T q (see csrc/recurrent.cu for the two kinds of gates);
    state [slots, n] float32 is read and left up to date.  q, k: [T, (H/q_group)*dk], v: [T, H*dv] (column slices
    are fine), g1/g2: float32 [T, >=H] pre-activations, p1..p3: float32 [H] or None; out float32 [T, H*dv]."""
    _need_cuda(out, q, k, v, g1, g2, p1, p2, p3, state)
    assert out.dtype == torch.float32 and out.stride(1) == 1 and q.dtype == k.dtype == v.dtype
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and g1.dtype == torch.float32 and g1.stride(1) == 1
    assert state.dtype == torch.float32 and state.stride(-1) == 1
    for p in (p1, p2, p3):
        assert p is None or (p.dtype == torch.float32 and p.numel() >= H)
    rc = _lib("recurrent").qv_linear_scan(
        kind, _ptr(out), out.stride(0), _ptr(q), q.stride(0), q_group, _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(g1),
        g1.stride(0), _ptr(g2), g2.stride(0) if g2 is not None else 0, _ptr(p1), _ptr(p2), _ptr(p3), float(cap), float(q_scale),
        _ptr(state), state.stride(0), _ptr(ctx.seg_q_start), _ptr(ctx.seg_slot), ctx.num_segments, H, dk, dv, dt_code(q.dtype),
        _stream())
    _check(rc, "linear_scan")


def gated_group_norm(out, y, gate, w, groups: int, eps: float, gate_first: bool) -> None:
    """out = unit norm of y (float32) in `groups` equal parts of a row, times w, with the gate applied behind the
    norm as a sigmoid (gate_first False) or ahead of it as a SiLU (True)."""
    _need_cuda(out, y, gate, w)
    T, W = y.shape
    assert y.dtype == torch.float32 and y.stride(1) == 1 and out.stride(1) == 1 and gate.stride(1) == 1
    assert out.dtype == gate.dtype and w.dtype == torch.float32 and w.numel() == W
    rc = _lib("recurrent").qv_gated_group_norm(_ptr(out), out.stride(0), _ptr(y), y.stride(0), _ptr(gate), gate.stride(0), _ptr(w),
                                               T, W, groups, eps, 1 if gate_first else 0, dt_code(out.dtype), _stream())
    _check(rc, "gated_group_norm")


# ------------------------------------------------------------------ recurrences with a decay per key channel

GATE_POW_SIGMOID, GATE_EXP_NEG_SIGMOID, GATE_EXP_NEG_SOFTPLUS, GATE_LINEAR = 0, 1, 2, 3
HEAD_GATE_SIGMOID, HEAD_GATE_SILU = 0, 1


def channel_gates(out, x1, w2t, bias, pre_tanh: bool, kind: int, p: float, rate=None) -> None:
    """out[t, c] (float32) = g(sum_r f(x1[t, r]) w2t[r, c] + bias[c]): f the identity or tanh; g(z) = sigmoid(z)^p
    (GATE_POW_SIGMOID), exp(-p sigmoid(z)) (GATE_EXP_NEG_SIGMOID), exp(-rate[c] softplus(z)) (GATE_EXP_NEG_SOFTPLUS, rate
    float32 [N]) or z (GATE_LINEAR).  x1 float32 [T, R] (a column slice is fine), w2t float32 [R, N]: the up matrix
    transposed, so that neighbouring channels lie side by side."""
    _need_cuda(out, x1, w2t, bias, rate)
    assert rate is None or (rate.dtype == torch.float32 and rate.is_contiguous() and rate.numel() == w2t.shape[1])
    T, R = x1.shape
    N = w2t.shape[1]
    assert out.dtype == x1.dtype == w2t.dtype == torch.float32 and out.stride(1) == 1 and x1.stride(1) == 1 and w2t.is_contiguous()
    assert tuple(out.shape) == (T, N) and w2t.shape[0] == R and (bias is None or (bias.dtype == torch.float32 and bias.numel() == N))
    rc = _lib("channel_scan").qv_channel_gates(_ptr(out), out.stride(0), _ptr(x1), x1.stride(0), _ptr(w2t), _ptr(bias), T, N, R,
                                               1 if pre_tanh else 0, kind, float(p), _ptr(rate), _stream())
    _check(rc, "channel_gates")


def delta_operands(qh, kb, ug, q, k, b, g, H: int, G: int, n: int, eps: float, q_scale: float) -> None:
    """The scan's operands for a delta rule whose removal reads the decayed state: per token and head (head h reads group
    h // (H // G) of q and k) qh = q / |q| * q_scale, kb = sigmoid(b) k / |k|, ug = g * k / |k|, |x| = sqrt(sum x^2 + eps); q, k
    float32 [T, G*n], b float32 [T, H], g float32 [T, H*n] (column slices are fine); qh, kb, ug dense float32 [T, H*n]."""
    _need_cuda(qh, kb, ug, q, k, b, g)
    T = q.shape[0]
    for x in (qh, kb, ug):
        assert x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (T, H * n)
    for x in (q, k, b, g):
        assert x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[0] == T
    rc = _lib("channel_scan").qv_delta_operands(_ptr(qh), _ptr(kb), _ptr(ug), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(b), b.stride(0),
                                                _ptr(g), g.stride(0), T, H, G, n, float(eps), float(q_scale), _stream())
    _check(rc, "delta_operands")


def unit_keys(u, au, k, a, a_bias, H: int, n: int, eps: float) -> None:
    """Per token and head: u = k / sqrt(sum(k^2) + eps), au = sigmoid(a + a_bias) * u; k, a float32 [T, H*n] (column
    slices are fine), u, au dense float32 [T, H*n]."""
    _need_cuda(u, au, k, a, a_bias)
    T = k.shape[0]
    assert k.dtype == a.dtype == u.dtype == au.dtype == torch.float32 and k.stride(1) == 1 and a.stride(1) == 1
    assert u.is_contiguous() and au.is_contiguous() and tuple(u.shape) == tuple(au.shape) == (T, H * n)
    assert a_bias is None or (a_bias.dtype == torch.float32 and a_bias.numel() == H * n)
    rc = _lib("channel_scan").qv_unit_keys(_ptr(u), _ptr(au), _ptr(k), k.stride(0), _ptr(a), a.stride(0), _ptr(a_bias), T, H, n,
                                           float(eps), _stream())
    _check(rc, "unit_keys")


def channel_scan_state_floats(H: int, dk: int, dv: int) -> int:
    """How many float32 values channel_scan keeps per request for H heads of dk x dv."""
    return int(_lib("channel_scan").qv_channel_scan_state_floats(H, dk, dv))


def channel_scan(out, q, k, v, w, au, u, q_scale: float, state, ctx, H: int, dk: int, dv: int) -> None:
    """Per request and head: S = diag(w) S - au (u^T S) + k v^T (au, u None: no removal), out = S^T q * q_scale; all
    operands float32, q, k, w, au, u [T, H*dk] and v [T, H*dv] (column slices are fine); state [slots, n] float32 is
    read and left up to date."""
    _need_cuda(out, q, k, v, w, au, u, state)
    for x in (out, q, k, v, w, au, u):
        assert x is None or (x.dtype == torch.float32 and x.stride(1) == 1)
    assert state.dtype == torch.float32 and state.stride(-1) == 1 and state.shape[-1] >= channel_scan_state_floats(H, dk, dv)
    rc = _lib("channel_scan").qv_channel_scan(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(w), w.stride(0), _ptr(au),
        au.stride(0) if au is not None else 0, _ptr(u), u.stride(0) if u is not None else 0, float(q_scale), _ptr(state),
        state.stride(0), _ptr(ctx.seg_q_start), _ptr(ctx.seg_slot), ctx.num_segments, int(ctx.max_q_len), H, dk, dv, _stream())
    _check(rc, "channel_scan")


def head_norm_gate(out, y, gate, w, H: int, eps: float, gate_kind: int, factor: float = 1.0) -> None:
    """out = y over its root mean square per head, times w (float32 [H*dv]), times sigmoid or SiLU of gate (float32),
    times factor; y float32 [T, H*dv]; out (compute type) and gate may be column slices."""
    _need_cuda(out, y, gate, w)
    T, W = y.shape
    assert W % H == 0 and y.dtype == gate.dtype == w.dtype == torch.float32 and w.numel() == W
    assert y.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == T and out.shape[1] == W
    rc = _lib("channel_scan").qv_head_norm_gate(_ptr(out), out.stride(0), _ptr(y), y.stride(0), _ptr(gate), gate.stride(0), _ptr(w), T, H,
                                                W // H, float(eps), gate_kind, float(factor), dt_code(out.dtype), _stream())
    _check(rc, "head_norm_gate")


# ------------------------------------------------------------------ attention with a learned distance bias

def bias_attn_prepare(q_out, proj, q_off, k_off, v_off, bq, bk, bv, cache_layer, ctx, block_table, H, G, n, dv, page, coef, every) -> None:
    """From a float32 product's row [.. q .. k .. v ..]: q_out = (q + bq) * (1 + coef ln(floor((pos + 1) / every) + 1)) in the
    compute type; k + bk and v + bv go into the token's cache row [G*n | G*dv]."""
    _need_cuda(q_out, proj, bq, bk, bv, cache_layer, block_table)
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.stride(1) == 1 and q_out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (n + dv))
    for b, size in ((bq, H * n), (bk, G * n), (bv, G * dv)):
        assert b is None or (b.dtype == torch.float32 and b.numel() == size)
    _i32(block_table, "block_table")
    rc = _lib("bias_attention").qv_bias_attn_prepare(
        _ptr(q_out), q_out.stride(0), _ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(bq), _ptr(bk), _ptr(bv), _ptr(cache_layer),
        _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table), block_table.shape[-1], T, H, G, n, dv, page, float(coef), int(every),
        dt_code(q_out.dtype), _stream())
    _check(rc, "bias_attn_prepare")


def rot_norm_prepare(q_out, proj, q_off, k_off, v_off, cache_layer, cos_sin, rot, unit, eps, head_temp, v_first, lam, ctx, block_table,
                     H, G, n, dv, page) -> None:
    """From a float32 product's row [.. q .. k .. v ..]: q and k heads rotated over their first `rot` entries (pairs i, i + rot/2,
    cos_sin [rows, rot/2, 2] float32), then, with `unit`, divided by their root mean square (eps under the root); q times
    head_temp[h] (float32 [H] or None) -> q_out (compute type); v, blended as (1 - lam) v + lam v_first[t] where v_first (float32
    [T, G*dv], a column slice is fine) is given, and k go into the token's cache row [G*n | G*dv]."""
    _need_cuda(q_out, proj, cache_layer, cos_sin, head_temp, v_first, block_table)
    T = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and q_out.stride(1) == 1 and q_out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (n + dv))
    assert head_temp is None or (head_temp.dtype == torch.float32 and head_temp.numel() == H)
    assert v_first is None or (v_first.dtype == torch.float32 and v_first.stride(1) == 1 and tuple(v_first.shape) == (T, G * dv))
    if rot:
        assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous() and cos_sin.shape[1] * 2 == rot
    _i32(block_table, "block_table")
    rc = _lib("bias_attention").qv_rot_norm_prepare(
        _ptr(q_out), q_out.stride(0), _ptr(proj), proj.stride(0), q_off, k_off, v_off, _ptr(cache_layer), _ptr(cos_sin) if rot else None,
        cos_sin.shape[0] if rot else 1, int(rot), 1 if unit else 0, float(eps), _ptr(head_temp), _ptr(v_first),
        v_first.stride(0) if v_first is not None else 0, float(lam), _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table),
        block_table.shape[-1], T, H, G, n, dv, page, dt_code(q_out.dtype), _stream())
    _check(rc, "rot_norm_prepare")


def bias_attention_generic(out, q, cache_layer, ctx, block_table, H, G, n, dv, page, scale, bucket, bias, gate, factor) -> None:
    """out[t, h] = softmax_j((q_t,h . k_j) * scale + bias[bucket[min(i - j, len(bucket) - 1)], h]) v_j over the request's pages,
    times sigmoid(gate[t, h]) (float32, or None) and factor."""
    _need_cuda(out, q, cache_layer, block_table, bucket, bias, gate)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (n + dv))
    assert (bias is None) == (bucket is None), "a bias table comes with the buckets of its distances"
    if bias is not None:
        assert bucket.dtype == torch.int32 and bucket.is_contiguous() and bias.dtype == torch.float32 and bias.is_contiguous() and bias.shape[1] == H
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    _i32(block_table, "block_table")
    rc = _lib("bias_attention").qv_bias_attention_generic(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(ctx.tok_pos), _ptr(ctx.tok_seg), _ptr(block_table),
        block_table.shape[-1], T, H, G, n, dv, page, float(scale), _ptr(bucket), bucket.numel() - 1 if bucket is not None else 0, _ptr(bias), _ptr(gate),
        gate.stride(0) if gate is not None else 0, float(factor), dt_code(q.dtype), _stream())
    _check(rc, "bias_attention_generic")


def bias_attention_table(bucket, bias):
    """The bias per head and distance, times log2 e, for the tensor-core kernel: [H, len(bucket)] float32 from the
    buckets of the distances (int32) and the table [rows, H]."""
    return (bias.float()[bucket.long()] * math.log2(math.e)).t().contiguous()


def bias_attention_tc(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, G, n, dv, page, scale, table, gate, factor,
                      slices: int = 1, slice_keys: int = 0) -> bool:
    """Attention with a distance bias on the tensor cores (bfloat16; key and value sizes up to 128, multiples of 8) for S
    segments that start at rows seg_q_start[s]; single tokens (max_q_len 1) share a tile among the query heads of a
    key/value head, and slices > 1 cuts every token's keys into slices of slice_keys that a second launch joins.
    table: bias_attention_table(...).  False, nothing written, for sizes it does not take."""
    if q.dtype != torch.bfloat16 or n % 8 or dv % 8 or n > 128 or dv > 128 or q.stride(0) % 8 or out.stride(0) % 2:
        return False
    if q.data_ptr() % 16 or out.data_ptr() % 4:        # 16-byte copies of q, paired stores of the outputs
        return False
    if max_q_len == 1 and H // G > 16:
        return False
    _need_cuda(out, q, cache_layer, seg_q_start, seg_pos0, block_table, table, gate)
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == cache_layer.dtype == torch.bfloat16
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (page, G * (n + dv))
    assert table.dtype == torch.float32 and table.is_contiguous() and table.shape[0] == H
    assert gate is None or (gate.dtype == torch.float32 and gate.stride(1) == 1)
    _i32(block_table, "block_table")
    lib = _lib("bias_attention")
    partial = None
    if slices > 1:
        assert max_q_len == 1
        partial = torch.empty(S * H * slices * (2 + dv), device=q.device, dtype=torch.float32)
    rc = lib.qv_bias_attention_mma(_ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(seg_q_start), _ptr(seg_pos0),
                                   _ptr(block_table), block_table.shape[-1], S, max_q_len, H, G, n, dv, page, float(scale), _ptr(table),
                                   table.shape[1] - 1, _ptr(gate), gate.stride(0) if gate is not None else 0, float(factor), _ptr(partial),
                                   slices, slice_keys, _stream())
    if rc == -2:
        return False
    _check(rc, "bias_attention_mma")
    if slices > 1:
        add_launches(1)                              # the kernel that joins the slices
    return True


def bias_attention_slices(tokens: int, G: int, max_ctx: int):
    """(slices, keys a slice) for single query tokens (a warp serves a token, a key/value head and a slice): the keys a
    slice follow from the step's shape, so that few tokens still fill the SMs, and the slices cover the longest context
    the step may hold (in a captured step: the longest a request may reach; slices past a token's position cost a launch
    of a warp that leaves at once)."""
    work = tokens * G
    keys = 64 if work <= 128 else 128 if work <= 512 else 256
    return max(1, -(-max_ctx // keys)), keys


def bias_attention(out, q, cache_layer, ctx, block_table, H, G, n, dv, page, scale, bucket, bias, gate, factor, table_of_distances=None) -> None:
    """Attention with a distance bias for every token of the step (see bias_attention_generic).  bfloat16: the
    tensor-core kernel where it takes the sizes and the table per distance is given (single tokens, which come first in a
    step, with their keys in slices; portions with tiles of 64 rows); float32 and other sizes: the CUDA-core kernel."""
    if q.dtype == torch.bfloat16 and table_of_distances is not None:
        S = ctx.num_segments
        n1 = 0                                        # leading segments of one token (decoded tokens)
        while n1 < S and ctx.seg_len[n1] == 1:
            n1 += 1
        args = (H, G, n, dv, page, scale, table_of_distances)
        ok = True
        if n1:
            slices, keys = bias_attention_slices(n1, G, ctx.max_ctx_len)
            ok = bias_attention_tc(out, q, cache_layer, ctx.seg_q_start, ctx.seg_pos0, block_table, n1, 1, *args, gate, factor,
                                   slices=slices, slice_keys=keys)
        if ok and n1 < S:
            ok = bias_attention_tc(out, q, cache_layer, ctx.seg_q_start[n1:], ctx.seg_pos0[n1:], block_table[n1:], S - n1,
                                   max(ctx.seg_len[n1:]), *args, gate, factor)
        if ok:
            return
    bias_attention_generic(out, q, cache_layer, ctx, block_table, H, G, n, dv, page, scale, bucket, bias, gate, factor)


# ------------------------------------------------------------------ routed feed-forward

def moe_route(top_idx, top_w, gate_out, h, w_router, w_gate) -> None:
    """Per token: router logits in float32, the top choices (top_idx int32 [T, top]) and their weights (softmax
    over the chosen logits, top_w float32 [T, top]); gate_out [T] = sigmoid(w_gate . h) when w_gate is given."""
    _need_cuda(top_idx, top_w, gate_out, h, w_router, w_gate)
    T, d = h.shape
    E, top = w_router.shape[0], top_idx.shape[1]
    assert h.stride(1) == 1 and w_router.is_contiguous() and w_router.shape[1] == d and top_idx.is_contiguous() and top_w.is_contiguous()
    # the logits in a launch of their own: few tokens spread over more SMs, many share the router's rows in groups of eight
    few = T <= 256 or (d % 4 == 0 and 8 * d * 4 <= 160 * 1024)
    ws = torch.empty(T * (E + 1), device=h.device, dtype=torch.float32) if few else None
    rc = _lib("moe").qv_moe_route(_ptr(top_idx), _ptr(top_w), _ptr(gate_out), _ptr(h), h.stride(0), _ptr(w_router), _ptr(w_gate),
                                  _ptr(ws), T, d, E, top, dt_code(h.dtype), dt_code(w_router.dtype), _stream())
    _check(rc, "moe_route")
    if few:
        add_launches(1)


def moe_tile_rows(tensor_cores: bool) -> int:
    """Rows of a tile of grouped rows: what the tile table is made for (the two experts' kernels differ)."""
    return int(_lib("moe").qv_moe_tile_rows(1 if tensor_cores else 0))


def moe_max_tiles(rows: int, experts: int, tile_rows: int) -> int:
    return int(_lib("moe").qv_moe_max_tiles(rows, experts, tile_rows))


def moe_group(row_token, slot_row, tiles, top_idx, scratch, experts: int, tile_rows: int) -> None:
    """Sorts the (token, choice) pairs by expert on the device and lists the tiles of `tile_rows` rows; see csrc/moe.cu."""
    _need_cuda(row_token, slot_row, tiles, top_idx, scratch)
    T, top = top_idx.shape
    rc = _lib("moe").qv_moe_group(_ptr(row_token), _ptr(slot_row), _ptr(tiles), _ptr(top_idx), _ptr(scratch), T, top, experts,
                                  tile_rows, _stream())
    _check(rc, "moe_group")


def moe_pack_experts(w: torch.Tensor) -> torch.Tensor:
    """Experts' matrices [E, N, K] (bfloat16) as tiles of 64 rows x 64 k, [E, ceil(N/64), ceil(K/64), 64, 64],
    zero-padded at the edges: the layout the tensor-core kernel copies a stage from in one piece."""
    E, N, K = w.shape
    Np, Kp = -(-N // 64) * 64, -(-K // 64) * 64
    if (Np, Kp) != (N, K):
        w = torch.nn.functional.pad(w, (0, Kp - K, 0, Np - N))
    return w.view(E, Np // 64, 64, Kp // 64, 64).permute(0, 1, 3, 2, 4).contiguous()


def moe_experts_tc(up, out, a, p1, p2, row_token, tiles) -> None:
    """The experts' products on the tensor cores (bfloat16); up as for moe_experts.  p1, p2: matrices packed by moe_pack_experts; the sizes
    follow from out [R, N] and a [., K]; the tile table was made for tiles of moe_tile_rows(True) rows."""
    _need_cuda(out, a, p1, p2, row_token, tiles)
    R, N = out.shape
    K = a.shape[1]
    E = p1.shape[0]
    assert a.dtype == p1.dtype == torch.bfloat16 and a.stride(1) == 1 and out.stride(1) == 1 and a.stride(0) % 8 == 0
    assert p1.is_contiguous() and tuple(p1.shape[1:]) == (-(-N // 64), -(-K // 64), 64, 64) and R == row_token.numel()
    assert out.dtype == (torch.bfloat16 if up else torch.float32)
    rc = _lib("moe").qv_moe_experts_tc(int(up), _ptr(out), out.stride(0), _ptr(a), a.stride(0), _ptr(p1), _ptr(p2),
                                       _ptr(row_token), _ptr(tiles), R, E, N, K, _stream())
    _check(rc, "moe_experts_tc")


def moe_experts(up, out, a, w1, w2, row_token, tiles) -> None:
    """The experts' products over the grouped rows on the CUDA cores (float32 multiply-adds, k ascending).
    up True or 1: out[r] = silu(w1[e] x) * (w2[e] x) with x = a[row_token[r]]; 2: out[r] = relu(w1[e] x)^2 (ungated
    experts, w2 None); False or 0: out[r] (float32) = w1[e] a[r].
    w1, w2: [E, N, K]; the tile table was made for tiles of moe_tile_rows(False) rows."""
    _need_cuda(out, a, w1, w2, row_token, tiles)
    R = row_token.numel()
    E, N, K = w1.shape
    assert w1.is_contiguous() and a.stride(1) == 1 and out.stride(1) == 1 and a.shape[1] == K and out.shape == (R, N)
    assert out.dtype == (a.dtype if up else torch.float32)
    rc = _lib("moe").qv_moe_experts(int(up), _ptr(out), out.stride(0), _ptr(a), a.stride(0), _ptr(w1), _ptr(w2),
                                    _ptr(row_token), _ptr(tiles), R, E, N, K, dt_code(a.dtype), dt_code(w1.dtype), _stream())
    _check(rc, "moe_experts")


def moe_route_table(top_idx, top_w, table, ids, experts: int) -> None:
    """Experts without a router: top_idx[t] = table[ids[t]] (int32 [vocab, top]), top_w = 1/top."""
    _need_cuda(top_idx, top_w, table, ids)
    _i32(table, "table"); _i32(ids, "ids"); _i32(top_idx, "top_idx")
    T, top = top_idx.shape
    assert table.shape[1] == top and top_w.is_contiguous() and top_w.dtype == torch.float32 and ids.numel() >= T
    rc = _lib("moe").qv_moe_route_table(_ptr(top_idx), _ptr(top_w), _ptr(table), _ptr(ids), T, top, table.shape[0], int(experts), _stream())
    _check(rc, "moe_route_table")


def moe_combine(delta, mix, y, slot_row, top_w, shared, gate, mix_scale=None, ff_scale=None) -> None:
    """delta (float32) = mix * mix_scale + (sum_j top_w[t, j] * y[slot_row[t, j]] + gate[t] * shared[t]) * ff_scale; mix,
    shared, gate and the per-feature scales (float32 [d]) may be None."""
    _need_cuda(delta, mix, y, slot_row, top_w, shared, gate, mix_scale, ff_scale)
    for sc in (mix_scale, ff_scale):
        assert sc is None or (sc.dtype == torch.float32 and sc.is_contiguous() and sc.numel() == delta.shape[1])
    T, d = delta.shape
    assert delta.dtype == torch.float32 and delta.is_contiguous() and y.dtype == torch.float32 and y.is_contiguous()
    ref = mix if mix is not None else shared
    for t in (mix, shared):
        assert t is None or (t.is_contiguous() and t.shape == delta.shape and t.dtype == ref.dtype)
    rc = _lib("moe").qv_moe_combine(_ptr(delta), _ptr(mix), _ptr(y), _ptr(slot_row), _ptr(top_w), _ptr(shared), _ptr(gate), T, d,
                                    top_w.shape[1], dt_code(ref.dtype) if ref is not None else F32, _ptr(mix_scale), _ptr(ff_scale),
                                    _stream())
    _check(rc, "moe_combine")


# ------------------------------------------------------------------ matrix products

def gemm_simt(c, a, w, accumulate=False) -> None:
    """c[M,N] (+)= a[M,K] @ w[N,K]^T with float32 multiply-adds on the CUDA cores."""
    _need_cuda(c, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and c.shape == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    rc = _lib("gemm_simt").qv_gemm_simt(
        _ptr(c), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), dt_code(a.dtype),
        dt_code(w.dtype), dt_code(c.dtype), 1 if accumulate else 0, _stream())
    _check(rc, "gemm_simt")


_tc_state = {}


def _tc_buffers(device):
    """Per device: the error word of the tensor-core kernels."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _tc_state.get(key)
    if st is None:
        st = dict(err=torch.zeros(1, dtype=torch.int32, device=device))
        _tc_state[key] = st
    return st


_split_registered = [None]      # the workspace the library knows (its address), 0 after it was told to share no tiles
_split_enabled = [os.environ.get("QORVIX_SHARE_TILES", "1") != "0"]


def _gemm_buffers(device):
    """`_tc_buffers` plus, for the products: the workspace through which CTAs of the many-token
    kernel hand the partial sums of a tile they share to its owner (one slot and one flag per SM),
    registered with the library once; products run on one stream at a time."""
    st = _tc_buffers(device)
    if not _split_enabled[0]:
        return st
    if "split_slots" not in st:
        ctas = sm_count()
        st["split_slots"] = torch.empty(ctas * int(_lib("gemm_bf16").qv_gemm_bf16_split_slot_bytes()) // 4, dtype=torch.float32, device=device)
        st["split_flags"] = torch.zeros(ctas, dtype=torch.int32, device=device)
    key = st["split_slots"].data_ptr()
    if _split_registered[0] != key:
        _lib("gemm_bf16").qv_gemm_bf16_set_split_workspace(_ptr(st["split_slots"]), _ptr(st["split_flags"]), st["split_flags"].numel())
        _split_registered[0] = key
    return st


def prepare_products(device) -> None:
    """Allocates and registers what the bfloat16 products need beside their operands (error word, workspace
    of shared tiles), so that no first call inside a stream capture has to."""
    _gemm_buffers(torch.device(device))


def gemm_share_tiles(enabled: bool) -> None:
    """Switches the sharing of tiles between CTAs of the many-token kernel off, or on again (for comparison)."""
    _split_enabled[0] = bool(enabled)
    if not enabled and _split_registered[0]:
        _lib("gemm_bf16").qv_gemm_bf16_set_split_workspace(None, None, 0)
        _split_registered[0] = 0


def gemm_bf16_tc(c, a, w, force_splits: int = 0, swiglu: bool = False) -> bool:
    """c[M,N] (bf16 or f32) = a[M,K] @ w[N,K]^T on the tcgen05 tensor cores.  With `swiglu`, w holds
    gate and up rows interleaved in groups of 16 and c[M,N/2] = silu(gate) * up.  False when the
    shape is one the kernel refuses (K not a multiple of 8, unaligned rows); nothing is written then."""
    _need_cuda(c, a, w)
    M, K = a.shape
    N = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == K
    assert c.shape == ((M, N // 2) if swiglu else (M, N))
    assert a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    st = _gemm_buffers(a.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_tc(
        _ptr(c), _ptr(a), _ptr(w), M, N, K, a.stride(0), w.stride(0), c.stride(0), dt_code(c.dtype),
        _ptr(st["err"]), force_splits, int(swiglu), _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_bf16_tc")
    return True


def pack_weight(w: torch.Tensor) -> torch.Tensor:
    """The bfloat16 matrix w [N, K] as the 16 KB tiles (128 rows x 64 k, in the shared-memory layout of
    the MMA) that gemm_bf16_packed streams with contiguous copies.  K must be a multiple of 8."""
    _need_cuda(w)
    assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1
    N, K = w.shape
    lib = _lib("gemm_bf16")
    out = torch.empty(lib.qv_packed_weight_bytes(N, K) // 2, device=w.device, dtype=torch.bfloat16)
    _check(lib.qv_pack_weight_tiles(_ptr(out), _ptr(w), N, K, w.stride(0), _stream()), "pack_weight_tiles")
    return out


def gemm_bf16_packed(c, a, packed, N: int, force_splits: int = 0, swiglu: bool = False) -> bool:
    """As gemm_bf16_tc, with the weights given by pack_weight (for any number of rows of a)."""
    _need_cuda(c, a, packed)
    M, K = a.shape
    assert a.dtype == torch.bfloat16 and packed.dtype == torch.bfloat16
    assert c.shape == ((M, N // 2) if swiglu else (M, N)) and a.stride(1) == 1 and c.stride(1) == 1
    st = _gemm_buffers(a.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_packed(
        _ptr(c), _ptr(a), _ptr(packed), M, N, K, a.stride(0), c.stride(0), dt_code(c.dtype), _ptr(st["err"]),
        force_splits, int(swiglu), _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_bf16_packed")
    return True


def gemm_bf16_norm(c, a, packed, N: int, swiglu: bool = False, residual=None, norm_weight=None, ssq_out=None,
                   ssq_in=None, stream_width: int = 0, eps: float = 0.0) -> bool:
    """A product of up to 64 tokens with the neighbouring RMS norm folded in.
    residual (float32 [M, N]) given: residual += a w^T; c (bfloat16) = residual * norm_weight; ssq_out
    (float32 [ceil(N/128), 64]) = sums of squares of the updated rows per tile of 128 features.
    ssq_in (such sums of a stream of `stream_width` features) given: row t of a w^T is scaled by
    rsqrt(sum(ssq_in[:, t]) / stream_width + eps) before it is stored (or goes through SwiGLU).
    False, with nothing written, when the kernel does not take the product."""
    _need_cuda(c, a, packed, residual, norm_weight, ssq_out, ssq_in)
    M, K = a.shape
    if M > 64 or a.dtype != torch.bfloat16 or packed is None:
        return False
    assert c.shape == ((M, N // 2) if swiglu else (M, N)) and a.stride(1) == 1 and c.stride(1) == 1
    tiles_in = 0
    if residual is not None:
        assert residual.dtype == torch.float32 and residual.stride(1) == 1 and tuple(residual.shape) == (M, N)
        assert norm_weight.dtype == torch.float32 and norm_weight.numel() == N
        assert ssq_out.dtype == torch.float32 and ssq_out.is_contiguous() and tuple(ssq_out.shape) == (-(-N // 128), 64)
    if ssq_in is not None:
        assert ssq_in.dtype == torch.float32 and ssq_in.is_contiguous() and ssq_in.shape[1] == 64 and stream_width > 0
        tiles_in = ssq_in.shape[0]
    st = _gemm_buffers(a.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_norm(
        _ptr(c), _ptr(a), _ptr(packed), M, N, K, a.stride(0), c.stride(0), dt_code(c.dtype), _ptr(st["err"]),
        int(swiglu), _ptr(residual), residual.stride(0) if residual is not None else 0, _ptr(norm_weight),
        _ptr(ssq_out), _ptr(ssq_in), tiles_in, 1.0 / stream_width if stream_width else 0.0, eps, _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_bf16_norm")
    return True


def new_norm_stats(features: int, device) -> torch.Tensor:
    """The buffer gemm_bf16_norm leaves a stream's sums of squares in (per tile of 128 features of the
    few-token kernel, for its 64 token columns); what it holds is between the producing and the
    consuming launch of that kernel."""
    return torch.empty((-(-features // 128), 64), device=device, dtype=torch.float32)


def _rules():
    """The kernel-choice rules live in C++ (csrc/host/dispatch.hpp), one statement for this module and
    for the native executor; they are reached through the host runtime library."""
    from ..cache import native
    return native.lib()


def folded_norm_enabled(tokens: int) -> bool:
    """Whether the RMS norms of a step of `tokens` tokens ride in the epilogues of the products around
    them: up to 16 tokens, unless QORVIX_FOLDED_NORM=0 (never) or =64 (up to 64 tokens; for comparison)."""
    return bool(_rules().qvh_folded_norm_enabled(int(tokens)))


def fused_rope_enabled(tokens: int) -> bool:
    """Whether the QKV projection of a step of `tokens` tokens takes the rotation and the cache write
    into its epilogue: above 64 tokens, unless QORVIX_FUSED_ROPE=0 (for comparison)."""
    return bool(_rules().qvh_fused_rope_enabled(int(tokens)))


def gemm_qkv_rope(qkv, x, packed, cache_layer, cos_sin, tok_pos, tok_seg, block_table, H, Hkv, hd, page) -> bool:
    """The QKV projection of more than 64 tokens with the rotation of q and k and the cache write of k
    and v in the product's epilogue: qkv[:, :H*hd] gets the rotated queries, the key and value columns
    of qkv are not written.  False (nothing written) when the sizes are not ones it takes: head sizes
    other than 64 and 128, a partial rotation, no packed weights, 64 tokens or fewer."""
    if x.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or packed is None or cos_sin is None:
        return False
    M, K = x.shape
    if cos_sin.shape[1] * 2 != hd or cache_layer.dtype != torch.bfloat16:
        return False
    _need_cuda(qkv, x, packed, cache_layer, cos_sin, tok_pos, tok_seg, block_table)
    assert x.stride(1) == 1 and qkv.stride(1) == 1 and qkv.shape == (M, (H + 2 * Hkv) * hd)
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    assert cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    st = _gemm_buffers(x.device)
    rc = _lib("gemm_bf16").qv_gemm_bf16_qkv_rope(
        _ptr(qkv), _ptr(x), _ptr(packed), M, K, x.stride(0), qkv.stride(0), _ptr(st["err"]), _ptr(cos_sin),
        cos_sin.shape[0], _ptr(tok_pos), _ptr(tok_seg), _ptr(block_table), block_table.shape[-1], _ptr(cache_layer),
        H, Hkv, hd, page, _stream())
    if rc == -2:
        return False
    _check(rc, "gemm_qkv_rope")
    return True


def gemm_bf16_set_prefill_tile_width(bn: int) -> None:
    """Columns of the persistent kernel's tiles: 0 (default) lets each product choose, else a multiple
    of 16 (32 with the fused activation) up to 256.  For comparison and tests."""
    _lib("gemm_bf16").qv_gemm_bf16_set_prefill_bn(bn)


def check_kernel_errors() -> None:
    """Raises if a kernel gave up on a bounded wait since the last check (synchronises)."""
    for key, st in _tc_state.items():
        code = int(st["err"].item())
        if code:
            st["err"].zero_()
            raise KernelError(f"a tensor-core kernel on device {key} gave up waiting on a barrier (code {code})")


# ------------------------------------------------------------------ attention

def attention_generic(out, q, cache_layer, tok_pos, tok_seg, block_table, H, Hkv, hd, page, window, scale) -> None:
    """out[t, h*hd:(h+1)*hd] = causal GQA attention of query (t, h) over its request's pages.
    q may be a column slice of the qkv buffer (row stride given by its stride)."""
    _need_cuda(out, q, cache_layer, tok_pos, tok_seg, block_table)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == cache_layer.dtype
    assert cache_layer.is_contiguous() and tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    rc = _lib("attention_generic").qv_attention_generic(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(tok_pos), _ptr(tok_seg),
        _ptr(block_table), block_table.shape[-1], T, H, Hkv, hd, page, window, scale, dt_code(q.dtype), _stream())
    _check(rc, "attention_generic")


# ------------------------------------------------------------------ dispatch

def packed_weights_enabled() -> bool:
    """Whether bfloat16 weight matrices are stored as packed tiles (QORVIX_PACKED_WEIGHTS=0: as rows)."""
    import os
    return os.environ.get("QORVIX_PACKED_WEIGHTS", "1") != "0"


def gemm(out, x, w, packed=None, n: int = 0) -> None:
    """out = x @ w^T with the kernel that fits the dtypes and the shape.  w is the matrix as rows
    [n, K] (or None when only its packed tiles are kept, `packed` with `n` rows): bfloat16 operands
    go to the tensor-core kernels (over the packed tiles when there are any), everything else to the
    CUDA-core kernel."""
    if x.dtype == torch.bfloat16 and packed is not None and gemm_bf16_packed(out, x, packed, n or w.shape[0]):
        return
    if w is None:
        # Only the packed tiles are kept and the kernel that reads them refused x as it is (float32
        # values, rows that do not start on 16 bytes, a row stride that is no multiple of 8): an
        # aligned bfloat16 copy of x, which that kernel takes.
        xb = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
        cast_rows(xb, x)
        if packed is not None and gemm_bf16_packed(out, xb, packed, n):
            return
        raise KernelError("the product's shape is one the tensor-core kernel refuses and the weight rows were not kept")
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and gemm_bf16_tc(out, x, w):
        return
    gemm_simt(out, x, w)


def glu_epilogue(act: int) -> int:
    """The value of the products' `swiglu` argument that applies `act` (GLU_SILU or GLU_GELU_TANH) in the epilogue."""
    return 2 if act == GLU_GELU_TANH else 1


def gemm_swiglu(out, x, w_interleaved, packed=None, n: int = 0, act: int = 0) -> None:
    """out[M,f] = act(x Wg^T) * (x Wu^T) (act GLU_SILU or GLU_GELU_TANH) with gate and up rows interleaved in groups
    of 16 in w_interleaved [2f, K]: one tensor-core kernel when it takes the shape, else the product followed
    by the activation kernel."""
    n = n or w_interleaved.shape[0]
    if x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16:
        if packed is not None and gemm_bf16_packed(out, x, packed, n, swiglu=glu_epilogue(act)):
            return
        if (w_interleaved is not None and w_interleaved.dtype == torch.bfloat16
                and gemm_bf16_tc(out, x, w_interleaved, swiglu=glu_epilogue(act))):
            return
    gu = torch.empty((x.shape[0], n), device=x.device, dtype=out.dtype)
    gemm(gu, x, w_interleaved, packed, n)
    glu_act(out, gu, act, interleaved=True)


def attention_prefill_bf16(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd, page,
                           window, scale, variant: int = 0) -> bool:
    """Flash attention of prompt portions (any mix of segments) over the paged bfloat16 cache.
    False when the kernel refuses the sizes."""
    _need_cuda(out, q, cache_layer, seg_q_start, seg_pos0, block_table)
    assert q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache_layer.is_contiguous()
    assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(seg_q_start, "seg_q_start"); _i32(seg_pos0, "seg_pos0"); _i32(block_table, "block_table")
    rc = _lib("attention_bf16").qv_attn_prefill_bf16(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(seg_q_start), _ptr(seg_pos0),
        _ptr(block_table), block_table.shape[-1], S, max_q_len, H, Hkv, hd, page, window, scale, variant, _stream())
    if rc == -2:
        return False
    _check(rc, "attention_prefill_bf16")
    return True


def attention_prefill_tc(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd, page,
                         window, scale, max_ctx_len: int = 0) -> bool:
    """Flash attention of prompt portions with tcgen05 tensor-core products (head sizes 64 and 128).
    max_ctx_len: the longest context (cached + new tokens) among the portions, where the host knows it; it
    only steers how the kernel cuts its work.  False when the kernel refuses the sizes."""
    _need_cuda(out, q, cache_layer, seg_q_start, seg_pos0, block_table)
    assert q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache_layer.is_contiguous()
    assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(seg_q_start, "seg_q_start"); _i32(seg_pos0, "seg_pos0"); _i32(block_table, "block_table")
    st = _tc_buffers(q.device)
    rc = _lib("attention_tc").qv_attn_prefill_tc(
        _ptr(out), out.stride(0), _ptr(q), q.stride(0), q.shape[0], _ptr(cache_layer), cache_layer.shape[0],
        _ptr(seg_q_start), _ptr(seg_pos0), _ptr(block_table), block_table.shape[-1], S, max_q_len, int(max_ctx_len), H, Hkv,
        hd, page, window, scale, _ptr(st["err"]), _stream())
    if rc == -2:
        return False
    _check(rc, "attention_prefill_tc")
    return True


_decode_variant_forced = None
_sm_count = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once); without a device, as on a
    machine that only plans steps, the B200's 148."""
    global _sm_count
    if _sm_count is None:
        _sm_count = 148
        if torch.cuda.is_available():
            _sm_count = int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return _sm_count


def decode_variant(T: int, Hkv: int) -> int:
    """Which decode kernel a step of T tokens takes: 0 reads keys and values through a ring in shared
    memory that bulk copies fill (the faster one when many (token, kv head) pairs stream long key
    ranges), 1 through per-thread loads (less set-up; better when there are few pairs)."""
    if _decode_variant_forced is not None:
        return _decode_variant_forced
    return _rules().qvh_decode_variant(int(T), int(Hkv))


def decode_splits(T: int, Hkv: int, max_ctx: int, known: bool = True) -> int:
    """How many slices of the keys each (token, kv head) is cut into: the count whose waves of CTAs
    take the least time when max_ctx is the step's real longest context (`known`), else the count that
    fills one wave.  A function of the step's shape only (a captured step keeps it)."""
    return _rules().qvh_decode_splits(int(T), int(Hkv), int(max_ctx), 1 if known else 0, decode_variant(T, Hkv), sm_count())


def attention_decode_bf16(out, q, cache_layer, tok_pos, tok_seg, block_table, H, Hkv, hd, page, window, scale,
                          splits: int = 1) -> bool:
    """Attention of single query tokens (split over `splits` slices of the keys).  False when refused."""
    _need_cuda(out, q, cache_layer, tok_pos, tok_seg, block_table)
    T = q.shape[0]
    assert q.dtype == out.dtype == cache_layer.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and cache_layer.is_contiguous()
    assert tuple(cache_layer.shape[1:]) == (2, Hkv, page, hd)
    _i32(tok_pos, "tok_pos"); _i32(tok_seg, "tok_seg"); _i32(block_table, "block_table")
    partial = None
    if splits > 1:
        partial = torch.empty(T * H * splits * (hd + 2), dtype=torch.float32, device=q.device)
    lib = _lib("attention_bf16")
    lib.qv_attn_set_decode_variant(decode_variant(T, Hkv))
    if not getattr(lib, "_qv_err_set", False):
        # the word that the kernel's bounded waits report into (see check_kernel_errors)
        lib.qv_attn_set_error_word(_ptr(_tc_buffers(q.device)["err"]))
        lib._qv_err_set = True
    rc = lib.qv_attn_decode_bf16(_ptr(
        out), out.stride(0), _ptr(q), q.stride(0), _ptr(cache_layer), _ptr(tok_pos), _ptr(tok_seg),
        _ptr(block_table), block_table.shape[-1], T, H, Hkv, hd, page, window, scale, splits, _ptr(partial),
        _stream())
    if rc == -2:
        return False
    _check(rc, "attention_decode_bf16")
    if splits > 1:
        add_launches(1)                              # the merge of the slices
    return True


def attention_set_decode_variant(variant) -> None:
    """Forces the decode kernel (0: bulk copies into shared memory, 1: per-thread loads) or, with
    None, gives the choice back to decode_variant().  For comparison and tests."""
    global _decode_variant_forced
    _decode_variant_forced = variant


def _attention_portions_bf16(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd, page,
                             window, scale, max_ctx_len=0) -> bool:
    """Prompt portions: tcgen05 kernel for long portions at head sizes 64/128, else mma.sync kernels."""
    if max_q_len >= 32 and attention_prefill_tc(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len,
                                                H, Hkv, hd, page, window, scale, max_ctx_len):
        return True
    return attention_prefill_bf16(out, q, cache_layer, seg_q_start, seg_pos0, block_table, S, max_q_len, H, Hkv, hd,
                                  page, window, scale)


def attention(out, q, cache_layer, ctx, block_table, H, Hkv, hd, page, window, scale) -> None:
    """Attention of every token of the step over its request's pages.  bfloat16: the tensor-core
    kernels when they take the sizes (split-KV for single tokens, flash attention for portions; a
    step whose single-token segments come first is served by both, each on its part); float32,
    and sizes they refuse: the CUDA-core kernel."""
    if q.dtype == torch.bfloat16:
        T = q.shape[0]
        if ctx.max_q_len == 1:
            splits = decode_splits(T, Hkv, ctx.max_ctx_len, known=not ctx.captured)
            if attention_decode_bf16(out, q, cache_layer, ctx.tok_pos, ctx.tok_seg, block_table, H, Hkv, hd, page,
                                     window, scale, splits):
                return
        else:
            n1 = 0                                    # leading segments of one token (decoded tokens)
            while n1 < ctx.num_segments and ctx.seg_len[n1] == 1:
                n1 += 1
            S = ctx.num_segments
            # the longest context among the segments of more than one token (what the flash kernel cuts its work by)
            deep = max((p0 + n for p0, n in zip(ctx.seg_start_pos, ctx.seg_len) if n > 1), default=0)
            if n1 >= 4 and n1 < S:
                rest_q = max(ctx.seg_len[n1:])
                splits = decode_splits(n1, Hkv, ctx.max_ctx_len, known=not ctx.captured)
                ok = attention_decode_bf16(out[:n1], q[:n1], cache_layer, ctx.tok_pos, ctx.tok_seg, block_table, H, Hkv,
                                           hd, page, window, scale, splits)
                if ok and _attention_portions_bf16(out, q, cache_layer, ctx.seg_q_start[n1:], ctx.seg_pos0[n1:],
                                                   block_table[n1:], S - n1, rest_q, H, Hkv, hd, page, window, scale, deep):
                    return
            elif _attention_portions_bf16(out, q, cache_layer, ctx.seg_q_start, ctx.seg_pos0, block_table, S,
                                          ctx.max_q_len, H, Hkv, hd, page, window, scale, deep):
                return
    attention_generic(out, q, cache_layer, ctx.tok_pos, ctx.tok_seg, block_table, H, Hkv, hd, page, window, scale)


# ------------------------------------------------------------------ sampling

def argmax(out_ids, logits) -> None:
    """out_ids[r] = index of the first maximum of logits[r] (float32)."""
    _need_cuda(out_ids, logits)
    _i32(out_ids, "out_ids")
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out_ids.numel() >= logits.shape[0]
    rc = _lib("sampling").qv_argmax(
        _ptr(out_ids), _ptr(logits), logits.shape[0], logits.shape[1], logits.stride(0), _stream())
    _check(rc, "argmax")


def sample(out_ids, logits, temperature, top_k, top_p, min_p, uniform, recent=None, rep_pen=None,
           freq_pen=None, pres_pen=None) -> None:
    """One token per row of logits (float32; rewritten in place by the penalties).  Per-row
    parameters are device tensors: temperature/top_p/min_p/uniform float32, top_k int32; recent is
    int32 [rows, n] of the tokens the penalties look at (-1: empty)."""
    _need_cuda(out_ids, logits, temperature, top_k, top_p, min_p, uniform, recent, rep_pen, freq_pen, pres_pen)
    _i32(out_ids, "out_ids"); _i32(top_k, "top_k")
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    for t in (temperature, top_p, min_p, uniform):
        assert t.dtype == torch.float32 and t.is_contiguous() and t.numel() >= rows
    recent_n = 0
    if recent is not None:
        _i32(recent, "recent")
        recent_n = recent.shape[1]
        for t in (rep_pen, freq_pen, pres_pen):
            assert t is not None and t.dtype == torch.float32 and t.numel() >= rows
    rc = _lib("sampling").qv_sample(
        _ptr(out_ids), _ptr(logits), rows, V, logits.stride(0), _ptr(temperature), _ptr(top_k), _ptr(top_p),
        _ptr(min_p), _ptr(uniform), _ptr(recent), recent_n, _ptr(rep_pen), _ptr(freq_pen), _ptr(pres_pen),
        _stream())
    _check(rc, "sample")
