"""MLA prolog (quant) entry points for B200.

Same names, positional argument order (14 input tensors, 7 output tensors, 5 non-tensor arguments) and layouts
as models/deepseek_v32_exp/mla_prolog_quant_impl.py (mla_prolog_quant_d :848-875, _p :751-778).  Weights are
plain row-major matrices (the reference passes NZ-format views of the same logical matrices).  Caches are
updated in place at rows `cache_index`; the cache "out" arguments must be the same tensors as the cache inputs,
as in the reference tests.

The four projections (x.w_dq, int8 q_norm.w_uq_qr, per-head q_nope.w_uk, x.w_dkv_kr) and everything between
them -- RMSNorm, int8 quantisation, dequantisation, de-interleaved RoPE, four-group cache quantisation and the
cache scatter -- run in the kernels of libdsv32_b200.so; one call of dsv32_mla_prolog enqueues the operator.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib
from . import _runtime as rt

H, Q_LORA, N_HEADS, NOPE, ROPE, KV_LORA = 7168, 1536, 128, 128, 64, 512


@dataclass
class MlaTileConfig:
    """Ascend tile sizes of the reference (mla_prolog_quant_impl.py:57-93); accepted and ignored."""
    tile_bs: int = 8
    m_tile: int = 16
    mv_tile: int = 8
    extra: dict = field(default_factory=dict)


@dataclass
class RopeTileShapeConfig:
    two_dim: list = None
    three_dim: list = None
    four_dim: list = None


def validate(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index,
             kv_cache, kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out, query_rope_out,
             kv_cache_out, kr_cache_out, k_scale_cache_out, cache_mode):
    """Checks dtypes, shapes, contiguity, aliasing of the in-place caches and that everything lives on one
    device; returns that device."""
    rt.require_cuda()
    bf16 = torch.bfloat16
    rt.check_tensor(token_x, "token_x", bf16, (None, H))
    t = token_x.shape[0]
    rt.check_tensor(w_dq, "w_dq", bf16, (H, Q_LORA))
    rt.check_tensor(w_uq_qr, "w_uq_qr", torch.int8, (Q_LORA, N_HEADS * (NOPE + ROPE)))
    if dequant_scale.numel() != N_HEADS * (NOPE + ROPE):
        raise ValueError(f"dequant_scale: expected {N_HEADS * (NOPE + ROPE)} scales, got {tuple(dequant_scale.shape)}")
    rt.check_tensor(dequant_scale, "dequant_scale", torch.float32)
    rt.check_tensor(w_uk, "w_uk", bf16, (N_HEADS, NOPE, KV_LORA))
    rt.check_tensor(w_dkv_kr, "w_dkv_kr", bf16, (H, KV_LORA + ROPE))
    rt.check_tensor(gamma_cq, "gamma_cq", bf16, (Q_LORA,))
    rt.check_tensor(gamma_ckv, "gamma_ckv", bf16, (KV_LORA,))
    rt.check_tensor(cos, "cos", bf16, (t, ROPE))
    rt.check_tensor(sin, "sin", bf16, (t, ROPE))
    rt.check_tensor(cache_index, "cache_index", torch.int64, (t,))
    rt.check_tensor(kv_cache, "kv_cache", torch.int8, (None, None, 1, KV_LORA))
    blocks, bs = kv_cache.shape[0], kv_cache.shape[1]
    rt.check_tensor(kr_cache, "kr_cache", bf16, (blocks, bs, 1, ROPE))
    rt.check_tensor(k_scale_cache, "k_scale_cache", torch.float32, (blocks, bs, 1, 4))
    rt.check_tensor(q_norm_out, "q_norm_out", torch.int8, (t, Q_LORA))
    rt.check_tensor(q_norm_scale_out, "q_norm_scale_out", torch.float32, (t, 1))
    rt.check_tensor(query_nope_out, "query_nope_out", bf16, (t, N_HEADS, KV_LORA))
    rt.check_tensor(query_rope_out, "query_rope_out", bf16, (t, N_HEADS, ROPE))
    for name, a, b in (("kv_cache_out", kv_cache_out, kv_cache), ("kr_cache_out", kr_cache_out, kr_cache),
                       ("k_scale_cache_out", k_scale_cache_out, k_scale_cache)):
        if a.data_ptr() != b.data_ptr():
            raise ValueError(f"{name} must be the same tensor as its input cache (in-place update)")
    if str(cache_mode) not in ("PA_BSND", "BSND", "PA_NZ"):
        raise ValueError(f"cache_mode={cache_mode!r} is not supported")
    dev = rt.same_device(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin,
                         cache_index, kv_cache, kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out,
                         query_rope_out)
    return dev


def mla_prolog(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index,
               kv_cache, kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out, query_rope_out,
               kv_cache_out, kr_cache_out, k_scale_cache_out, epsilon_cq, epsilon_ckv, cache_mode):
    """Validates the arguments and runs the MLA prolog on the current stream of the tensors' device."""
    dev = validate(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index,
                   kv_cache, kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out, query_rope_out,
                   kv_cache_out, kr_cache_out, k_scale_cache_out, cache_mode)
    if token_x.shape[0] == 0:
        return None
    a, keep = mla_args(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index,
                       kv_cache, kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out, query_rope_out,
                       epsilon_cq, epsilon_ckv, dev)
    with torch.cuda.device(dev):
        rt.check(_lib.load().dsv32_mla_prolog(C.byref(a), rt.stream_ptr(dev)), "mla_prolog_quant")
    del keep
    return None


def mla_args(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index, kv_cache,
             kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out, query_rope_out, epsilon_cq,
             epsilon_ckv, dev):
    """(Dsv32MlaPrologArgs, keep-alive list) for already validated tensors."""
    lib = _lib.load()
    t = token_x.shape[0]
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_mla_prolog_workspace_bytes(t)
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.MlaPrologArgs(
            rt.ptr(token_x), rt.ptr(w_dq), rt.ptr(w_uq_qr), rt.ptr(dequant_scale), rt.ptr(w_uk), rt.ptr(w_dkv_kr),
            rt.ptr(gamma_cq), rt.ptr(gamma_ckv), rt.ptr(cos), rt.ptr(sin), rt.ptr(cache_index), rt.ptr(kv_cache),
            rt.ptr(kr_cache), rt.ptr(k_scale_cache), rt.ptr(q_norm_out), rt.ptr(q_norm_scale_out), rt.ptr(query_nope_out),
            rt.ptr(query_rope_out), rt.ptr(ws), int(ws_bytes), rt.ptr(rt.status_word(dev)),
            kv_cache.shape[0] * kv_cache.shape[1], t, float(epsilon_cq), float(epsilon_ckv))
    return a, [ws]


def _entry(name, args):
    if len(args) != 26:
        raise ValueError(f"{name} takes 26 positional arguments, got {len(args)}")
    return mla_prolog(*args[:24])


def mla_prolog_quant_d(*args):
    """Decode entry (mla_prolog_quant_impl.py:848-875): 14 input tensors, 7 output tensors, then epsilon_cq,
    epsilon_ckv, cache_mode, tile_config, rope_cfg (the last two are Ascend tiling and are ignored)."""
    return _entry("mla_prolog_quant_d", args)


def mla_prolog_quant_p(*args):
    """Prefill entry (mla_prolog_quant_impl.py:751-778); same math, any number of tokens."""
    return _entry("mla_prolog_quant_p", args)
