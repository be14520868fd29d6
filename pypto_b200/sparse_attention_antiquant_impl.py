"""Sparse attention over the fused int8 cache ("store 8, compute 16") entry points for B200.

Same names, positional argument order and layouts as the reference operator file
models/deepseek_v32_exp/sparse_attention_antiquant_impl.py (sparse_attention_antiquant_d :287-356,
_p :358-420, _d_950 :739-768).  One cache row is 656 bytes: 512 int8 latent dims, 64 bf16 rope dims, 4 fp32
scales (deepseekv32_sparse_attention_antiquant.py:262-272), so a selected key is one contiguous gather instead
of three.  The arithmetic is that of sparse_flash_attention_quant; the kernels are the same with another row
stride.  Outputs are written in place, the call returns None and only enqueues work on the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import _runtime as rt
from .sparse_flash_attention_quant_impl import SaTileShapeConfig  # noqa: F401  (same tile-shape type)

ROW_BYTES = 656


def _sa_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs, attention_out, nq, n_kv,
                  softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config, kv_splits=0):
    rt.require_cuda()
    if int(n_kv) != 1:
        raise ValueError(f"n_kv={n_kv}: the latent cache has one shared KV head")
    bf16 = torch.bfloat16
    rt.check_tensor(query_nope, "query_nope", bf16, (None, 512))
    rt.check_tensor(query_rope, "query_rope", bf16, (query_nope.shape[0], 64))
    rt.check_tensor(nope_cache, "nope_cache", torch.int8, (None, ROW_BYTES))
    rows = nope_cache.shape[0]
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
    if attention_out.dim() == 2:  # the reference tests pass the output as [t*nq, 512]
        rt.check_tensor(attention_out, "attention_out", bf16, (t * int(nq), 512))
    else:
        rt.check_tensor(attention_out, "attention_out", bf16, (b, s1, int(nq), 512))
    dev = rt.same_device(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs, attention_out)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_sfa_workspace_bytes(b, s1, int(nq), int(topk), int(kv_splits))
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.SaAntiquantArgs(
            rt.ptr(query_nope), rt.ptr(query_rope), rt.ptr(nope_cache), rt.ptr(topk_indices), rt.ptr(block_table),
            rt.ptr(kv_act_seqs), rt.ptr(attention_out), rt.ptr(ws), int(ws_bytes), rt.ptr(rt.status_word(dev)), rows,
            b, s1, int(nq), int(topk), int(block_size), int(max_blocknum_perbatch), int(kv_splits),
            float(softmax_scale))
        rt.check(lib.dsv32_sparse_attention_antiquant(C.byref(a), rt.stream_ptr(dev)), "sparse_attention_antiquant")
    return None


def sparse_attention_antiquant_d(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                 attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                 tile_config=None):
    """Decode entry (sparse_attention_antiquant_impl.py:287-356)."""
    return _sa_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs, attention_out, nq,
                         n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config)


def sparse_attention_antiquant_p(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                 attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                 tile_config=None):
    """Prefill entry (sparse_attention_antiquant_impl.py:358-420); same math, any s1."""
    return _sa_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs, attention_out, nq,
                         n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config)


def sparse_attention_antiquant_d_950(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs,
                                     attention_out, nq, n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch,
                                     tile_config=None):
    """Ascend-950 decode entry (sparse_attention_antiquant_impl.py:739-768); same contract on B200."""
    return _sa_antiquant(query_nope, query_rope, nope_cache, topk_indices, block_table, kv_act_seqs, attention_out, nq,
                         n_kv, softmax_scale, topk, block_size, max_blocknum_perbatch, tile_config)


def pack_cache_rows(key_nope_2d, key_rope_2d, k_nope_scales):
    """[rows,512] int8, [rows,64] bf16, [rows,4] fp32 -> [rows,656] int8 in the fused layout."""
    rows = key_nope_2d.shape[0]
    out = torch.empty((rows, ROW_BYTES), dtype=torch.int8, device=key_nope_2d.device)
    out[:, :512] = key_nope_2d
    out[:, 512:640] = key_rope_2d.contiguous().view(torch.int8).reshape(rows, 128)
    out[:, 640:] = k_nope_scales.contiguous().view(torch.int8).reshape(rows, 16)
    return out
