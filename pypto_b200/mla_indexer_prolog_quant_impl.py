"""Fused MLA prolog + indexer prolog (quant) entry points for B200.

Same names, positional argument order (24 input tensors, 10 output tensors, 7 non-tensor arguments) and
layouts as models/deepseek_v32_exp/mla_indexer_prolog_quant_impl.py (mla_indexer_prolog_quant_d :486-528,
_p :327-369).  The MLA half writes the int8 q_norm and q_norm_scale into device scratch that feeds the indexer
half, as in the reference (:112-211); both halves are enqueued by ONE call of dsv32_mla_indexer_prolog.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import _runtime as rt
from .lightning_indexer_prolog_quant_impl import (IndexerPrologQuantAttr, IndexerPrologQuantConfigs,  # noqa: F401
                                                  prolog_args)
from .mla_prolog_quant_impl import MlaTileConfig, RopeTileShapeConfig, Q_LORA, mla_args, validate  # noqa: F401


def _mla_indexer_prolog(token_x, mla_w_dq, mla_w_uq_qr, mla_dequant_scale, mla_w_uk, mla_w_dkv_kr, mla_gamma_cq,
                        mla_gamma_ckv, cos, sin, cache_index, mla_kv_cache, mla_kr_cache, mla_k_scale_cache,
                        ip_w_qb_in, ip_w_qb_scale_in, ip_wk_in, ip_w_proj_in, ip_ln_gamma_k_in, ip_ln_beta_k_in,
                        ip_hadamard_q_in, ip_hadamard_k_in, ip_k_cache, ip_k_cache_scale, mla_query_nope_out,
                        mla_query_rope_out, mla_kv_cache_out, mla_kr_cache_out, mla_k_scale_cache_out, ip_q_int8_out,
                        ip_q_scale_out, ip_k_int8_out, ip_k_scale_out, ip_weights_out, mla_epsilon_cq,
                        mla_epsilon_ckv, mla_cache_mode, mla_tile_config, ip_attrs, ip_configs, rope_cfg):
    t = token_x.shape[0]
    q_norm = torch.empty((t, Q_LORA), dtype=torch.int8, device=token_x.device)
    q_norm_scale = torch.empty((t, 1), dtype=torch.float32, device=token_x.device)
    dev = validate(token_x, mla_w_dq, mla_w_uq_qr, mla_dequant_scale, mla_w_uk, mla_w_dkv_kr, mla_gamma_cq, mla_gamma_ckv,
                   cos, sin, cache_index, mla_kv_cache, mla_kr_cache, mla_k_scale_cache, q_norm, q_norm_scale,
                   mla_query_nope_out, mla_query_rope_out, mla_kv_cache_out, mla_kr_cache_out, mla_k_scale_cache_out,
                   mla_cache_mode)
    ip, ip_dev, keep_ip = prolog_args(token_x, q_norm, q_norm_scale, ip_w_qb_in, ip_w_qb_scale_in.reshape(-1, 1), ip_wk_in,
                                      ip_w_proj_in, ip_ln_gamma_k_in, ip_ln_beta_k_in, cos, sin, ip_hadamard_q_in,
                                      ip_hadamard_k_in, ip_k_cache, ip_k_cache_scale, cache_index, ip_q_int8_out,
                                      ip_q_scale_out, ip_k_int8_out, ip_k_scale_out, ip_weights_out, ip_attrs)
    if ip_dev != dev:
        raise RuntimeError(f"all tensors must live on one device: {dev} vs {ip_dev}")
    if t == 0:
        return None
    mla, keep_mla = mla_args(token_x, mla_w_dq, mla_w_uq_qr, mla_dequant_scale, mla_w_uk, mla_w_dkv_kr, mla_gamma_cq,
                             mla_gamma_ckv, cos, sin, cache_index, mla_kv_cache, mla_kr_cache, mla_k_scale_cache, q_norm,
                             q_norm_scale, mla_query_nope_out, mla_query_rope_out, mla_epsilon_cq, mla_epsilon_ckv, dev)
    fused = _lib.FusedPrologArgs(mla, ip)
    with torch.cuda.device(dev):
        rt.check(_lib.load().dsv32_mla_indexer_prolog(C.byref(fused), rt.stream_ptr(dev)), "mla_indexer_prolog_quant")
    del keep_ip, keep_mla
    return None


def mla_indexer_prolog_quant_d(*args):
    """Decode entry (mla_indexer_prolog_quant_impl.py:486-528): 24 input tensors, 10 output tensors, then
    mla_epsilon_cq, mla_epsilon_ckv, mla_cache_mode, mla_tile_config, ip_attrs, ip_configs, rope_cfg."""
    if len(args) != 41:
        raise ValueError(f"mla_indexer_prolog_quant_d takes 41 positional arguments, got {len(args)}")
    return _mla_indexer_prolog(*args)


def mla_indexer_prolog_quant_p(*args):
    """Prefill entry (mla_indexer_prolog_quant_impl.py:327-369); same math, any number of tokens."""
    if len(args) != 41:
        raise ValueError(f"mla_indexer_prolog_quant_p takes 41 positional arguments, got {len(args)}")
    return _mla_indexer_prolog(*args)
