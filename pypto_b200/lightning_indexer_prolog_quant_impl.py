"""Indexer prolog (quant) entry point for B200.

Same name, positional argument order and layouts as the reference operator file
models/deepseek_v32_exp/lightning_indexer_prolog_quant_impl.py
(lightning_indexer_prolog_quant :325-349; dataclasses :71-119).  The weights are taken as plain
row-major [K, N] matrices (the reference feeds an NZ-format view of the same logical matrices).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List

import torch

from . import _lib
from . import _runtime as rt


@dataclass
class IndexerPrologQuantInput:
    x: torch.Tensor
    q_norm: torch.Tensor
    q_norm_scale: torch.Tensor
    w_qb: torch.Tensor
    w_qb_scale: torch.Tensor
    wk: torch.Tensor
    w_proj: torch.Tensor
    ln_gamma_k: torch.Tensor
    ln_beta_k: torch.Tensor
    cos_idx_rope: torch.Tensor
    sin_idx_rope: torch.Tensor
    hadamard_q: torch.Tensor
    hadamard_k: torch.Tensor
    k_cache: torch.Tensor
    k_cache_scale: torch.Tensor
    k_cache_index: torch.Tensor


@dataclass
class IndexerPrologQuantOutput:
    q_int8: torch.Tensor
    q_scale: torch.Tensor
    k_int8: torch.Tensor
    k_scale: torch.Tensor
    weights: torch.Tensor


@dataclass
class IndexerPrologQuantAttr:
    eps: float = 1e-6
    layerout_query: str = "TND"
    layerout_key: str = "PA_BSND"


@dataclass
class IndexerPrologQuantConfigs:
    """Ascend tile shapes; accepted and ignored."""
    q_linear: List[int] = field(default_factory=list)
    q_hd: List[int] = field(default_factory=list)
    k_linear: List[int] = field(default_factory=list)
    w_linear: List[int] = field(default_factory=list)
    unroll_list: List[int] = field(default_factory=list)
    cube_l1_reuse_setting: dict = field(default_factory=dict)
    block_size: int = 128
    t_sub_tile: int = 1
    chunk_size: int = 1
    vec_nbuffer_setting: dict = field(default_factory=dict)


def prolog_args(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, ln_gamma_k_in,
                ln_beta_k_in, cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_int8_in, k_scale_in,
                k_cache_index_in, q_int8_out, q_scale_out, k_int8_out, k_scale_out, weights_out, attrs=None):
    """Validates the operator's tensors and returns (Dsv32PrologArgs, device, keep-alive list): the argument block
    of dsv32_indexer_prolog, also embedded in the fused MLA + indexer prolog call."""
    rt.require_cuda()
    bf16 = torch.bfloat16
    rt.check_tensor(x_in, "x", bf16, (None, 7168))
    t = x_in.shape[0]
    rt.check_tensor(q_norm_in, "q_norm", torch.int8, (t, 1536))
    rt.check_tensor(q_norm_scale_in, "q_norm_scale", torch.float32, (t, 1))
    rt.check_tensor(w_qb_in, "w_qb", torch.int8, (1536, 8192))
    rt.check_tensor(w_qb_scale_in, "w_qb_scale", torch.float32, (8192, 1))
    rt.check_tensor(wk_in, "wk", bf16, (7168, 128))
    rt.check_tensor(w_proj_in, "w_proj", bf16, (7168, 64))
    rt.check_tensor(ln_gamma_k_in, "ln_gamma_k", bf16, (128,))
    rt.check_tensor(ln_beta_k_in, "ln_beta_k", bf16, (128,))
    rt.check_tensor(cos_idx_rope_in, "cos_idx_rope", bf16, (t, 64))
    rt.check_tensor(sin_idx_rope_in, "sin_idx_rope", bf16, (t, 64))
    rt.check_tensor(hadamard_q_in, "hadamard_q", bf16, (128, 128))
    rt.check_tensor(hadamard_k_in, "hadamard_k", bf16, (128, 128))
    rt.check_tensor(k_int8_in, "k_int8", torch.int8, (None, None, 1, 128))
    rows = k_int8_in.shape[0] * k_int8_in.shape[1]
    rt.check_tensor(k_scale_in, "k_scale", torch.float16, (k_int8_in.shape[0], k_int8_in.shape[1], 1, 1))
    rt.check_tensor(k_cache_index_in, "k_cache_index", torch.int64, (t,))
    rt.check_tensor(q_int8_out, "q_int8_out", torch.int8, (t, 64, 128))
    rt.check_tensor(q_scale_out, "q_scale_out", torch.float16, (t, 64, 1))
    rt.check_tensor(weights_out, "weights_out", torch.float16, (t, 64))
    if k_int8_out.data_ptr() != k_int8_in.data_ptr() or k_scale_out.data_ptr() != k_scale_in.data_ptr():
        raise ValueError("k_int8_out / k_scale_out must be the same tensors as k_int8_in / k_scale_in (in-place cache)")
    dev = rt.same_device(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, ln_gamma_k_in,
                         ln_beta_k_in, cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_int8_in,
                         k_scale_in, k_cache_index_in, q_int8_out, q_scale_out, weights_out)
    eps = float(attrs.eps) if attrs is not None and getattr(attrs, "eps", None) is not None else 1e-6
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_prolog_workspace_bytes(t)
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.PrologArgs(
            rt.ptr(x_in), rt.ptr(q_norm_in), rt.ptr(q_norm_scale_in), rt.ptr(w_qb_in), rt.ptr(w_qb_scale_in),
            rt.ptr(wk_in), rt.ptr(w_proj_in), rt.ptr(ln_gamma_k_in), rt.ptr(ln_beta_k_in), rt.ptr(cos_idx_rope_in),
            rt.ptr(sin_idx_rope_in), rt.ptr(hadamard_q_in), rt.ptr(hadamard_k_in), rt.ptr(k_cache_index_in),
            rt.ptr(q_int8_out), rt.ptr(q_scale_out), rt.ptr(k_int8_in), rt.ptr(k_scale_in), rt.ptr(weights_out),
            rt.ptr(ws), int(ws_bytes), rt.ptr(rt.status_word(dev)), rows, t, eps)
    return a, dev, [ws]


def lightning_indexer_prolog_quant(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in,
                                   ln_gamma_k_in, ln_beta_k_in, cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in,
                                   hadamard_k_in, k_int8_in, k_scale_in, k_cache_index_in, q_int8_out, q_scale_out,
                                   k_int8_out, k_scale_out, weights_out, configs=None, attrs=None):
    """lightning_indexer_prolog_quant_impl.py:325-349.  k_int8_out / k_scale_out must alias
    k_int8_in / k_scale_in (the reference tests pass the same tensors): the cache is updated in place at
    rows k_cache_index_in and no other row is touched."""
    a, dev, keep = prolog_args(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, ln_gamma_k_in,
                               ln_beta_k_in, cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_int8_in,
                               k_scale_in, k_cache_index_in, q_int8_out, q_scale_out, k_int8_out, k_scale_out,
                               weights_out, attrs)
    with torch.cuda.device(dev):
        rt.check(_lib.load().dsv32_indexer_prolog(C.byref(a), rt.stream_ptr(dev)), "lightning_indexer_prolog_quant")
    del keep
    return None
