"""DeepSeek-V4 sparse compress attention entry points for B200.

Same names, positional argument order and layouts as the reference operator file
models/deepseek_v4/sparse_compress_flash_attention_impl.py (sparse_compress_flash_attention_kernel :172-213,
npu_sparse_compress_flash_attention :240-299, sparse_compress_flash_attention_graph :371-401).  Every query
token attends to the last `win_size` positions of its request in the un-compressed bf16 cache `ori_kv` and to the
rows of the compressed bf16 cache `cmp_kv` that `cmp_sparse_indices` selects; a 512-dim cache row is key and
value at once, and one attention sink per head is added to the softmax denominator (:98-163).  The kernel is the
tcgen05 sparse-attention kernel of the DeepSeek-V3.2 path with another key-list builder.  The kernel entry writes
`attention_out` in place and returns None; the `npu_` / `_graph` entries allocate and return it, as the
reference's do.  Work is only enqueued on the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from . import _runtime as rt

MAX_S2 = 131072


@dataclass
class SCFATileShapeConfig:
    """Ascend tile sizes (sparse_compress_flash_attention_impl.py:38-44); carried for signature parity only."""
    g_tile: int
    c1_tile_shape: list
    v1_tile_shape: list
    c2_tile_shape: list


SELECTED, ALL_COMPRESSED = 0, 1   # DSV32_SCFA_SELECTED / DSV32_SCFA_ALL_COMPRESSED


def run_window_compress_attention(query, actual_seq_q, ori_kv, cmp_kv, ori_block_table, cmp_block_table, atten_sink,
                                  seqused_kv, cmp_sparse_indices, attention_out, nq, softmax_scale, topk, block_size,
                                  win_size, cmp_ratio, cmp_mode=SELECTED):
    """Validate and launch.  `topk` == 0 leaves the window alone (cmp_kv / cmp_block_table / cmp_sparse_indices may
    be None); `cmp_mode` ALL_COMPRESSED takes every compressed position below cur_len // cmp_ratio (at most `topk`)
    and needs no index tensor.  2-D caches [rows, 512]; query and attention_out [tokens * nq, 512]."""
    rt.require_cuda()
    bf16 = torch.bfloat16
    nq, topk = int(nq), int(topk)
    rt.check_tensor(query, "query", bf16, (None, 512))
    rt.check_tensor(ori_kv, "ori_kv", bf16, (None, 512))
    rt.check_tensor(ori_block_table, "ori_block_table", torch.int32, (None, None))
    b = ori_block_table.shape[0]
    rt.check_tensor(actual_seq_q, "actual_seq_q", torch.int32, (b + 1,))
    rt.check_tensor(seqused_kv, "seqused_kv", torch.int32, (b,))
    rt.check_tensor(atten_sink, "atten_sink", torch.float32, (nq,))
    if nq < 1 or query.shape[0] % nq != 0:
        raise ValueError(f"query rows {query.shape[0]} are not a multiple of nq = {nq}")
    t = query.shape[0] // nq
    tensors = [query, actual_seq_q, ori_kv, ori_block_table, atten_sink, seqused_kv, attention_out]
    if topk > 0:
        rt.check_tensor(cmp_kv, "cmp_kv", bf16, (None, 512))
        rt.check_tensor(cmp_block_table, "cmp_block_table", torch.int32, (b, None))
        tensors += [cmp_kv, cmp_block_table]
        if cmp_mode == SELECTED:
            rt.check_tensor(cmp_sparse_indices, "cmp_sparse_indices", torch.int32, (t, topk))
            tensors.append(cmp_sparse_indices)
    rt.check_tensor(attention_out, "attention_out", bf16, (t * nq, 512))
    if t == 0 or b == 0:
        return None
    dev = rt.same_device(*tensors)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_scfa_workspace_bytes(t, topk, int(win_size))
        ws = rt.workspace(ws_bytes, dev)
        has_cmp = topk > 0
        a = _lib.ScfaArgs(
            rt.ptr(query), rt.ptr(actual_seq_q), rt.ptr(ori_kv), rt.ptr(cmp_kv) if has_cmp else None,
            rt.ptr(ori_block_table), rt.ptr(cmp_block_table) if has_cmp else None, rt.ptr(atten_sink),
            rt.ptr(seqused_kv), rt.ptr(cmp_sparse_indices) if has_cmp and cmp_mode == SELECTED else None,
            rt.ptr(attention_out), rt.ptr(ws), int(ws_bytes), rt.ptr(rt.status_word(dev)), ori_kv.shape[0],
            cmp_kv.shape[0] if has_cmp else 0, t, b, nq, topk, int(block_size), int(win_size), int(cmp_ratio),
            ori_block_table.shape[1], cmp_block_table.shape[1] if has_cmp else 0, int(cmp_mode), float(softmax_scale))
        rt.check(lib.dsv32_sparse_compress_attention(C.byref(a), rt.stream_ptr(dev)), "sparse_compress_flash_attention")
    return None


def sparse_compress_flash_attention_kernel(query, actual_seq_q, ori_kv, cmp_kv, ori_block_table, cmp_block_table,
                                           atten_sink, seqused_kv, cmp_sparse_indices, attention_out, nq, n_kv,
                                           softmax_scale, topk, block_size, win_size, cmp_ratio, tile_config=None):
    """sparse_compress_flash_attention_impl.py:172-213: 10 tensors, then nq, n_kv, softmax_scale, topk, block_size,
    win_size, cmp_ratio, tile_config."""
    if int(n_kv) != 1:
        raise ValueError(f"n_kv={n_kv}: the caches have one shared KV head")
    if int(topk) < 1:
        raise ValueError(f"topk={topk} must be >= 1")
    if isinstance(cmp_sparse_indices, torch.Tensor) and cmp_sparse_indices.dim() == 2 and \
            query.shape[0] != cmp_sparse_indices.shape[0] * int(nq):
        raise ValueError(f"query rows {query.shape[0]} != tokens * nq = {cmp_sparse_indices.shape[0] * int(nq)}")
    return run_window_compress_attention(query, actual_seq_q, ori_kv, cmp_kv, ori_block_table, cmp_block_table,
                                         atten_sink, seqused_kv, cmp_sparse_indices, attention_out, nq, softmax_scale,
                                         topk, block_size, win_size, cmp_ratio, SELECTED)


def npu_sparse_compress_flash_attention(query_npu, q_act_seqs_npu, ori_kv_npu, cmp_kv_npu, ori_block_table_npu,
                                        cmp_block_table_npu, atten_sink_npu, seqused_kv_npu, cmp_sparse_indices_npu,
                                        softmax_scale, win_size, cmp_ratio):
    """sparse_compress_flash_attention_impl.py:240-299: derives nq and topk from the shapes (block size 128),
    allocates the [t*nq, 512] output and returns it."""
    if cmp_sparse_indices_npu.dim() != 2 or cmp_sparse_indices_npu.shape[0] == 0:
        raise ValueError("cmp_sparse_indices must be a non-empty 2-D tensor")
    attention_out = torch.zeros_like(query_npu)
    nq = query_npu.shape[0] // cmp_sparse_indices_npu.shape[0]
    sparse_compress_flash_attention_kernel(query_npu, q_act_seqs_npu, ori_kv_npu, cmp_kv_npu, ori_block_table_npu,
                                           cmp_block_table_npu, atten_sink_npu, seqused_kv_npu,
                                           cmp_sparse_indices_npu, attention_out, nq, 1, softmax_scale,
                                           cmp_sparse_indices_npu.shape[1], 128, win_size, cmp_ratio, None)
    return attention_out


def sparse_compress_flash_attention_graph(query_npu, q_act_seqs_npu, ori_kv_npu, cmp_kv_npu, ori_block_table_npu,
                                          cmp_block_table_npu, atten_sink_npu, seqused_kv_npu, cmp_sparse_indices_npu,
                                          softmax_scale, win_size, cmp_ratio):
    """sparse_compress_flash_attention_impl.py:371-401 (the torch.ops route of the reference): same call."""
    return npu_sparse_compress_flash_attention(query_npu, q_act_seqs_npu, ori_kv_npu, cmp_kv_npu, ori_block_table_npu,
                                               cmp_block_table_npu, atten_sink_npu, seqused_kv_npu,
                                               cmp_sparse_indices_npu, softmax_scale, win_size, cmp_ratio)
