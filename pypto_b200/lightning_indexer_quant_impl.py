"""Lightning indexer (quant) decode entry point for B200.

Same name, positional argument order and layouts as the reference operator file
models/deepseek_v32_exp/lightning_indexer_quant_impl.py (lightning_indexer_decode :226-275).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib
from . import _runtime as rt

INT32_MAX = 2 ** 31 - 1


@dataclass
class LightningIndexerConfigs:
    """Tiling knobs of the reference (deepseekv32_lightning_indexer_quant.py:26-43).  Accepted for
    signature compatibility; `extend_param` documents the fixed 2^-11 scale + ReLU of the score epilogue."""
    mg_copy_in_upper_bound: int = 2 * 1024 * 1024
    cube_l1_reuse_setting: dict = field(default_factory=lambda: {0: 16})
    vec_merge_mode: int = 2
    vec_nbuffer_setting: dict = field(default_factory=lambda: {-1: 16})
    s1_tile: int = 2
    topk_tile: int = 8192
    c1_tile: list = field(default_factory=lambda: [64, 64, 128, 128, 128, 128])
    c2_tile: list = field(default_factory=lambda: [128, 128, 64, 64, 128, 128])
    extend_param: dict = field(default_factory=lambda: {"scale": 1 / 2048.0, "relu_type": "RELU"})


def indexer_scores_topk(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                        block_table, topk_res=None, selected_count=2048, *, topk_scores=None, scores_out=None,
                        dots_out=None, key_begin=0, key_end=INT32_MAX, scatter=None):
    """Scores + top-k with the optional extra outputs of the C ABI (see include/dsv32_b200.h):
    `topk_scores` (scores of the selected keys), `scores_out` (full fp32 score rows), `dots_out`
    (raw int32 dot products, verification only) and a logical key range for key-range sharding.
    `scatter` = (world, rank, tokens_per_rank, idx_ptrs, score_ptrs): the rows go to the owning ranks' peer-mapped
    candidate buffers instead of topk_res (dsv32_indexer_topk_scatter)."""
    rt.require_cuda()
    rt.check_tensor(idx_query, "idx_query", torch.int8, (None, 64, 128))
    t = idx_query.shape[0]
    if idx_query_scale.dim() == 3:
        idx_query_scale = idx_query_scale.reshape(t, 64)
    rt.check_tensor(idx_query_scale, "idx_query_scale", torch.float16, (t, 64))
    rt.check_tensor(idx_key_cache, "idx_key_cache", torch.int8, (None, 128, 1, 128))
    nblk = idx_key_cache.shape[0]
    if idx_key_scale.dim() == 4:
        idx_key_scale = idx_key_scale.reshape(nblk, 128, 1)
    rt.check_tensor(idx_key_scale, "idx_key_scale", torch.float16, (nblk, 128, 1))
    rt.check_tensor(idx_weight, "idx_weight", torch.float16, (t, 64))
    rt.check_tensor(act_seq_key, "act_seq_key", torch.int32, ndim=1)
    b = act_seq_key.shape[0]
    rt.check_tensor(block_table, "block_table", torch.int32, (b, None))
    if b == 0 and t == 0:
        return None
    if b == 0 or t % b != 0:
        raise ValueError(f"idx_query tokens ({t}) must be a multiple of the batch ({b})")
    s1 = t // b
    max_blocks = block_table.shape[1]
    ld = max_blocks * 128
    tensors = [idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key, block_table]
    if topk_res is not None:
        rt.check_tensor(topk_res, "topk_res", torch.int32, (t, 1, int(selected_count)))
        tensors.append(topk_res)
    if topk_scores is not None:
        rt.check_tensor(topk_scores, "topk_scores", torch.float32, (t, int(selected_count)))
        tensors.append(topk_scores)
    if scores_out is not None:
        rt.check_tensor(scores_out, "scores_out", torch.float32, (t, None))  # rows may be longer than the page table
        if scores_out.shape[1] < ld:
            raise ValueError(f"scores_out: rows of {scores_out.shape[1]} scores, need at least {ld}")
        ld = scores_out.shape[1]
        tensors.append(scores_out)
    if dots_out is not None:
        rt.check_tensor(dots_out, "dots_out", torch.int32, (t, 64, ld))
        tensors.append(dots_out)
    dev = rt.same_device(*tensors)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = 0 if scores_out is not None else lib.dsv32_indexer_workspace_bytes(b, s1, max_blocks, 128)
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.IndexerArgs(
            rt.ptr(idx_query), rt.ptr(idx_query_scale), rt.ptr(idx_key_cache), rt.ptr(idx_key_scale),
            rt.ptr(idx_weight), rt.ptr(act_seq_key), rt.ptr(block_table), rt.ptr(topk_res), rt.ptr(topk_scores),
            rt.ptr(scores_out), rt.ptr(dots_out), rt.ptr(ws), int(ws_bytes), rt.ptr(rt.status_word(dev)), nblk, b, s1,
            128, max_blocks, int(selected_count), ld, int(key_begin), int(min(key_end, INT32_MAX)))
        if scatter is not None:
            world, rank, per, idx_ptrs, score_ptrs = scatter
            sca = _lib.TopkScatter(int(world), int(rank), int(per), 0)
            for r in range(int(world)):
                sca.idx_ptrs[r] = int(idx_ptrs[r])
                sca.score_ptrs[r] = int(score_ptrs[r])
            rt.check(lib.dsv32_indexer_topk_scatter(C.byref(a), C.byref(sca), rt.stream_ptr(dev)),
                     "lightning_indexer_decode (scatter)")
        else:
            rt.check(lib.dsv32_indexer_topk(C.byref(a), rt.stream_ptr(dev)), "lightning_indexer_decode")
    return None


def lightning_indexer_decode(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                             block_table, topk_res, unroll_list=None, configs=None, selected_count=2048):
    """Decode entry (lightning_indexer_quant_impl.py:226-238).  `unroll_list` and `configs` are Ascend
    tiling inputs and are ignored.  topk_res [t,1,selected_count] is written in place."""
    if topk_res is None:
        raise ValueError("topk_res: output tensor required")
    return indexer_scores_topk(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                               block_table, topk_res, selected_count)


def topk_select(scores, counts, k, ids=None, id_base=0, out_idx=None, out_scores=None):
    """Row-wise top-k (descending score, ties by ascending id, -1 pads) over fp32 `scores` [rows, ld];
    `counts` int32 [rows] gives the valid prefix of each row.  With `ids` the entries carry explicit ids
    (candidate merge).  Returns (out_idx, out_scores)."""
    rt.require_cuda()
    rt.check_tensor(scores, "scores", torch.float32, ndim=2)
    rows, ld = scores.shape
    rt.check_tensor(counts, "counts", torch.int32, (rows,))
    if ids is not None:
        rt.check_tensor(ids, "ids", torch.int32, (rows, ld))
    dev = scores.device
    if out_idx is None:
        out_idx = torch.empty((rows, k), dtype=torch.int32, device=dev)
    if out_scores is None:
        out_scores = torch.empty((rows, k), dtype=torch.float32, device=dev)
    rt.check_tensor(out_idx, "out_idx", torch.int32, (rows, k))
    rt.check_tensor(out_scores, "out_scores", torch.float32, (rows, k))
    lib = _lib.load()
    with torch.cuda.device(dev):
        a = _lib.TopkArgs(rt.ptr(scores), rt.ptr(ids), rt.ptr(counts), rt.ptr(out_idx), rt.ptr(out_scores), rows, ld,
                          int(k), int(id_base))
        rt.check(lib.dsv32_topk_select(C.byref(a), rt.stream_ptr(dev)), "topk_select")
    return out_idx, out_scores
