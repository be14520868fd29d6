"""DeepSeek-V4 sliding-window attention entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/win_attention_impl.py (deepseekv4_win_atten
:263-289, sliding_win_atten_graph :309-322, get_mask :325-333; compute win_atten_main_tnd_mask :78-260).  Token i
of a request with s1 = cu_seqlens_q[r+1] - cu_seqlens_q[r] query tokens stands at cur_loc = seqused_kv[r] - s1 + i + 1
and attends to the last min(cur_loc, win_size) rows of the paged bf16 cache before cur_loc; a 512-dim row is key and
value at once, the softmax scale is 512**-0.5 and one sink per head joins the softmax denominator.  The reference
handles four tokens at a time with a boolean mask tensor; here every token has its own key list, so `mask` is
accepted and ignored.  The kernel is the tcgen05 sparse-attention kernel with a key list of window rows only.
Returns a new tensor shaped like `q`; work is enqueued on the current stream.
"""
from __future__ import annotations

import torch

from . import _runtime as rt
from .sparse_compress_flash_attention_impl import SELECTED, run_window_compress_attention


def deepseekv4_win_atten(q, ori_block_table, ori_kv, seqused_kv, sinks, win_size, mask=None, cu_seqlens_q=None):
    """win_attention_impl.py:263-289.  q [tokens, heads, 512] bf16; ori_kv [blocks, block_size, 1, 512] bf16."""
    rt.require_cuda()
    for name, x in (("q", q), ("ori_block_table", ori_block_table), ("ori_kv", ori_kv), ("seqused_kv", seqused_kv),
                    ("sinks", sinks), ("cu_seqlens_q", cu_seqlens_q)):
        if not isinstance(x, torch.Tensor):
            raise ValueError(f"{name}: expected a torch.Tensor, got {type(x).__name__}")
    if q.dim() != 3 or q.size(2) != 512 or not 1 <= q.size(1) <= 128:
        raise ValueError(f"q: expected [tokens, heads <= 128, 512], got {tuple(q.shape)}")
    if ori_kv.dim() != 4 or ori_kv.size(2) != 1 or ori_kv.size(3) != 512:
        raise ValueError(f"ori_kv: expected [blocks, block_size, 1, 512], got {tuple(ori_kv.shape)}")
    if int(win_size) < 1:
        raise ValueError(f"win_size={win_size} must be >= 1")
    t, nq, d = q.shape
    out = torch.empty((t * nq, d), dtype=q.dtype, device=q.device)
    run_window_compress_attention(q.reshape(t * nq, d), cu_seqlens_q, ori_kv.reshape(-1, d), None, ori_block_table,
                                  None, sinks, seqused_kv, None, out, nq, d ** -0.5, 0, ori_kv.size(1), win_size, 1,
                                  SELECTED)
    return out.reshape(q.shape)


def sliding_win_atten_graph(q, ori_block_table, ori_kv, seqused_kv, sinks, win_size, mask, cu_seqlens_q):
    """win_attention_impl.py:309-322 (the torch.ops route of the reference): same call."""
    return deepseekv4_win_atten(q, ori_block_table, ori_kv, seqused_kv, sinks, win_size, mask, cu_seqlens_q)


def get_mask(s_q, n_q, device, block_size):
    """The boolean band mask the reference operator takes (win_attention_impl.py:325-333): row r of token s keeps
    columns [128 + s, 256 + s).  Provided so call sites keep working; the kernel here does not read it."""
    left = torch.zeros((s_q * n_q, 128), dtype=torch.bool, device=device)
    rows = torch.arange(s_q, device=device).unsqueeze(1)
    cols = torch.arange(block_size * 2, device=device).unsqueeze(0)
    right = ((cols >= rows) & (cols < rows + 128)).unsqueeze(1).expand(-1, n_q, -1).reshape(s_q * n_q, block_size * 2)
    return torch.cat([left, right, left.clone()], dim=-1)
