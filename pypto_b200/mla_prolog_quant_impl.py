"""MLA prolog (quant) entry points for B200.

Same names, positional argument order (14 input tensors, 7 output tensors, 5 non-tensor arguments) and layouts
as models/deepseek_v32_exp/mla_prolog_quant_impl.py (mla_prolog_quant_d :848-875, _p :751-778).  Weights are
plain row-major matrices (the reference passes NZ-format views of the same logical matrices).  Caches are
updated in place at rows `cache_index`; the cache "out" arguments must be the same tensors as the cache inputs,
as in the reference tests.

The four plain projections (x.w_dq, int8 q_norm.w_uq_qr, per-head q_nope.w_uk, x.w_dkv_kr) are library GEMMs
(cuBLAS through torch); everything between them -- RMSNorm, int8 quantisation, dequantisation, de-interleaved
RoPE, four-group cache quantisation and the cache scatter -- runs in the fused CUDA stages of
libdsv32_b200.so (dsv32_mla_prolog_stage).
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


def _int8_gemm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """int8 [m,k] x int8 [k,n] -> int32 [m', n] with m' >= m (the library kernel wants more than 16 rows)."""
    m = a.shape[0]
    if m <= 16:
        pad = torch.zeros((32, a.shape[1]), dtype=torch.int8, device=a.device)
        pad[:m] = a
        a = pad
    return torch._int_mm(a, b)


def mla_prolog(token_x, w_dq, w_uq_qr, dequant_scale, w_uk, w_dkv_kr, gamma_cq, gamma_ckv, cos, sin, cache_index,
               kv_cache, kr_cache, k_scale_cache, q_norm_out, q_norm_scale_out, query_nope_out, query_rope_out,
               kv_cache_out, kr_cache_out, k_scale_cache_out, epsilon_cq, epsilon_ckv, cache_mode):
    """Validates the arguments and runs the MLA prolog on the current stream of the tensors' device."""
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
    if t == 0:
        return None
    lib = _lib.load()
    with torch.cuda.device(dev):
        stream = rt.stream_ptr(dev)
        status = rt.status_word(dev)
        q_nope_tmp = torch.empty((N_HEADS, t, NOPE), dtype=bf16, device=dev)

        def stage(n, **kw):
            a = _lib.MlaStageArgs()
            a.t, a.status = t, status.data_ptr()
            a.eps_cq, a.eps_ckv = float(epsilon_cq), float(epsilon_ckv)
            for k, v in kw.items():
                setattr(a, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
            rt.check(lib.dsv32_mla_prolog_stage(C.byref(a), n, stream), f"mla_prolog_quant (stage {n})")

        # ---- q path ---------------------------------------------------------------------------------------
        q_a = torch.matmul(token_x, w_dq)                                         # library GEMM, bf16 out
        stage(0, q_a=q_a, gamma_cq=gamma_cq, q_norm=q_norm_out, q_norm_scale=q_norm_scale_out)
        q_b = _int8_gemm(q_norm_out, w_uq_qr)                                     # library GEMM, int32 out
        stage(1, q_b=q_b, q_b_ld=q_b.shape[1], q_norm_scale=q_norm_scale_out, w_qb_scale=dequant_scale,
              q_nope_tmp=q_nope_tmp, q_rope=query_rope_out, cos=cos, sin=sin)
        query_nope_out.copy_(torch.bmm(q_nope_tmp, w_uk).permute(1, 0, 2))       # library GEMM, [128, t, 512]
        # ---- kv path --------------------------------------------------------------------------------------
        kv_a = torch.matmul(token_x, w_dkv_kr)                                    # library GEMM, bf16 out
        stage(2, kv_a=kv_a, gamma_ckv=gamma_ckv, cos=cos, sin=sin, cache_index=cache_index, kv_cache=kv_cache,
              kr_cache=kr_cache, k_scale_cache=k_scale_cache, cache_rows=blocks * bs)
    return None


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
