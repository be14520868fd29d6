"""Sparse flash attention (quant) entry points for B200.

Same names, positional argument order, tensor layouts and page-table conventions as the reference
operator file models/deepseek_v32_exp/sparse_flash_attention_quant_impl.py
(sparse_flash_attention_quant_d :655-674, _p :734, _d_950 :572).  Outputs are written in place,
the call returns None and only enqueues work on the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from . import _runtime as rt


@dataclass
class SaTileShapeConfig:
    """Ascend tile shapes of the reference (sparse_flash_attention_quant_impl.py:34-42).
    Accepted for signature compatibility; the CUDA kernels have fixed tiling."""
    g_tile: int = 128
    s_kv_tile: int = 2048
    gather_vec_tile_shape: list = None
    c1_tile_shape: list = None
    v1_tile_shape: list = None
    c2_tile_shape: list = None
    v2_tile_shape: list = None


def _sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices, block_table, kv_act_seqs,
         attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config, kv_splits=0):
    rt.require_cuda()
    if int(n_kv) != 1:
        raise ValueError(f"n_kv={n_kv}: the latent cache has one shared KV head")
    bf16 = torch.bfloat16
    rt.check_tensor(query_nope, "query_nope", bf16, (None, 512))
    rt.check_tensor(query_rope, "query_rope", bf16, (query_nope.shape[0], 64))
    # int8 cache with per-group scales, or the bf16 cache of the reference's non-quantised branch (:216-259)
    quant = key_nope_2d.dtype == torch.int8
    if not quant and key_nope_2d.dtype != bf16:
        raise ValueError(f"key_nope_2d: expected the int8 quantized cache or a bf16 cache, got {key_nope_2d.dtype}")
    rt.check_tensor(key_nope_2d, "key_nope_2d", torch.int8 if quant else bf16, (None, 512))
    rows = key_nope_2d.shape[0]
    rt.check_tensor(key_rope_2d, "key_rope_2d", bf16, (rows, 64))
    if quant:
        rt.check_tensor(k_nope_scales, "k_nope_scales", torch.float32, (rows, 4))
    rt.check_tensor(topk_indices, "topk_indices", torch.int32, (None, int(n_kv) * int(topk)))
    rt.check_tensor(block_table, "block_table", torch.int32, (None, int(max_blocknum_perbatch)))
    b = block_table.shape[0]
    rt.check_tensor(kv_act_seqs, "kv_act_seqs", torch.int32, (b,))
    t = topk_indices.shape[0]
    if b == 0 or t % b != 0:
        if b == 0 and t == 0:
            return None
        raise ValueError(f"topk_indices rows ({t}) must be a multiple of the batch ({b})")
    s1 = t // b
    if query_nope.shape[0] != t * int(nq):
        raise ValueError(f"query_nope rows {query_nope.shape[0]} != t*nq = {t * int(nq)}")
    rt.check_tensor(attention_out, "attention_out", bf16, (b, s1, int(nq), 512))
    dev = rt.same_device(query_nope, query_rope, key_nope_2d, key_rope_2d, topk_indices, block_table, kv_act_seqs,
                         attention_out, *([k_nope_scales] if quant else []))
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_sfa_workspace_bytes(b, s1, int(nq), int(topk), int(kv_splits))
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.SfaArgs(
            rt.ptr(query_nope), rt.ptr(query_rope), rt.ptr(key_nope_2d), rt.ptr(key_rope_2d),
            rt.ptr(k_nope_scales) if quant else None,
            rt.ptr(topk_indices), rt.ptr(block_table), rt.ptr(kv_act_seqs), rt.ptr(attention_out), rt.ptr(ws),
            int(ws_bytes), rt.ptr(rt.status_word(dev)), rows, b, s1, int(nq), int(topk), int(block_size),
            int(max_blocknum_perbatch), int(kv_splits), float(softmax_scale))
        fn = lib.dsv32_sfa_quant if quant else lib.dsv32_sfa_bf16_cache
        rt.check(fn(C.byref(a), rt.stream_ptr(dev)), "sparse_flash_attention_quant")
    return None


def sparse_flash_attention_quant_d(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                   block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk,
                                   block_size, max_blocknum_perbatch, tile_config=None):
    """Decode entry (sparse_flash_attention_quant_impl.py:655-674)."""
    return _sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices, block_table,
                kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                tile_config)


def sparse_flash_attention_quant_p(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                   block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk,
                                   block_size, max_blocknum_perbatch, tile_config=None):
    """Prefill entry (sparse_flash_attention_quant_impl.py:734-803); same math, any s1."""
    return _sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices, block_table,
                kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                tile_config)


def sparse_flash_attention_quant_d_950(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices,
                                       block_table, kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk,
                                       block_size, max_blocknum_perbatch, tile_config=None):
    """Ascend-950 decode entry of the reference (sparse_flash_attention_quant_impl.py:572-641); same math."""
    return _sfa(query_nope, query_rope, key_nope_2d, key_rope_2d, k_nope_scales, topk_indices, block_table,
                kv_act_seqs, attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                tile_config)
