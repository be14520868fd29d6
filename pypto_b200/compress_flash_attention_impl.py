"""DeepSeek-V4 compressed flash attention (decode) entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/compress_flash_attention_impl.py (cfa_attention
:60-112, cfa_graph :243-248; compute c128_decode_impl :119-219).  Token i of a request with s1 = tokens / batch
query tokens sees vld_len = seqused_kv - (s1 - 1 - i) positions: it attends to the last min(vld_len, 128) rows of
the un-compressed cache `ori_kv` (the window) and to EVERY compressed row [0, vld_len // cmp_ratio) of `cmp_kv`;
a 512-dim row is key and value at once, the softmax scale is 512**-0.5 and one sink per head joins the softmax
denominator.  The reference assembles at most four compressed pages (512 rows); here every page of
`cmp_block_table` may be used.  The kernel is the tcgen05 sparse-attention kernel with a key list of window rows
followed by all compressed rows.  Returns a new tensor shaped like `q`; work is enqueued on the current stream.
"""
from __future__ import annotations

import torch

from . import _runtime as rt
from .sparse_compress_flash_attention_impl import ALL_COMPRESSED, run_window_compress_attention

WIN_SIZE = 128


def check_args(q, cmp_kv, sinks, cmp_block_table, seqused_kv, ori_kv, ori_block_table):
    """Shape rules of compress_flash_attention_impl.py:30-57, as exceptions (head count up to 128 here)."""
    if q.dim() != 3 or q.size(2) != 512 or not 1 <= q.size(1) <= 128:
        raise ValueError(f"q: expected [tokens, heads <= 128, 512], got {tuple(q.shape)}")
    for name, kv in (("cmp_kv", cmp_kv), ("ori_kv", ori_kv)):
        if kv.dim() != 4 or kv.size(2) != 1 or kv.size(3) != 512:
            raise ValueError(f"{name}: expected [blocks, block_size, 1, 512], got {tuple(kv.shape)}")
    if cmp_kv.size(1) != ori_kv.size(1):
        raise ValueError("cmp_kv and ori_kv must have the same block size")
    if sinks.dim() != 1 or sinks.size(0) != q.size(1):
        raise ValueError(f"sinks: expected [{q.size(1)}], got {tuple(sinks.shape)}")
    if cmp_block_table.dim() != 2 or ori_block_table.dim() != 2 or seqused_kv.dim() != 1:
        raise ValueError("cmp_block_table / ori_block_table must be 2-D and seqused_kv 1-D")


def cfa_attention(q, cmp_kv, sinks, cmp_block_table, seqused_kv, ori_kv, ori_block_table, cmp_ratio: int = 128):
    """compress_flash_attention_impl.py:60-112.  q [tokens, heads, 512] bf16 -> attention_out of the same shape."""
    rt.require_cuda()
    for name, x in (("q", q), ("cmp_kv", cmp_kv), ("sinks", sinks), ("cmp_block_table", cmp_block_table),
                    ("seqused_kv", seqused_kv), ("ori_kv", ori_kv), ("ori_block_table", ori_block_table)):
        if not isinstance(x, torch.Tensor):
            raise ValueError(f"{name}: expected a torch.Tensor, got {type(x).__name__}")
    check_args(q, cmp_kv, sinks, cmp_block_table, seqused_kv, ori_kv, ori_block_table)
    t, nq, d = q.shape
    b = seqused_kv.shape[0]
    if b == 0 or t % b != 0:
        raise ValueError(f"q tokens ({t}) must be a positive multiple of the batch ({b})")
    s1 = t // b
    block_size = cmp_kv.size(1)
    out = torch.empty((t * nq, d), dtype=q.dtype, device=q.device)
    seq_q = torch.arange(0, (b + 1) * s1, s1, dtype=torch.int32, device=q.device)
    run_window_compress_attention(q.reshape(t * nq, d), seq_q, ori_kv.reshape(-1, d), cmp_kv.reshape(-1, d),
                                  ori_block_table, cmp_block_table, sinks, seqused_kv, None, out, nq, d ** -0.5,
                                  cmp_block_table.shape[1] * block_size, block_size, WIN_SIZE, cmp_ratio,
                                  ALL_COMPRESSED)
    return out.reshape(q.shape)


def cfa_graph(q, cmp_kv, sinks, cmp_block_table, seqused_kv, ori_kv, ori_block_table, cmp_ratio):
    """compress_flash_attention_impl.py:243-248 (the torch.ops route of the reference): same call."""
    return cfa_attention(q, cmp_kv, sinks, cmp_block_table, seqused_kv, ori_kv, ori_block_table, cmp_ratio)
