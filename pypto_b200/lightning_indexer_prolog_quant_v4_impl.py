"""DeepSeek-V4 lightning indexer prolog (quant) entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/lightning_indexer_prolog_quant_v4_impl.py
(npu_quant_lightning_indexer_prolog :78-115, quant_lightning_indexer_prolog_kernel :118-266).  Per token:
  q       = per-(token, head) int8 quantisation of bf16([nope | irope(rope)] @ hadamard), where
            [nope | rope] = bf16(int32(qr @ idx_wq_b) * qr_scale * idx_wq_b_scale) split 64 + 64 per head and irope is
            the interleaved inverse rotary embedding (common.py:67-120; golden apply_rotary_pos_emb,
            utils/golden/common_func.py:45-69);
  q_scale = the dequantisation scale (1 / (127 / amax)) as fp16;
  weights = fp16(float(bf16(x @ weights_proj)) * 64**-0.5 * 128**-0.5).
There is no key path in this operator.  Weights are plain row-major [K, N] (the reference passes NZ-formatted
views of the same matrices).  The query path is the tcgen05 kernel of the DeepSeek-V3.2 indexer prolog with a
reduction length of 1024 and the other rotary form; work is only enqueued on the current CUDA stream.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib
from . import _runtime as rt

Q_LORA_RANK, IDX_NQ, HEAD_DIM, ROPE_DIM = 1024, 64, 128, 64


@dataclass
class IndexerPrologQuantConfig:
    """Ascend loop-unroll list (lightning_indexer_prolog_quant_v4_impl.py:36-38); carried for signature parity only."""
    unroll_list: list = field(default_factory=lambda: [128, 64, 32, 16, 8, 1])


def quant_lightning_indexer_prolog_kernel(qr, idx_wq_b, x, weights_proj, cos, sin, hadamard, qr_scale, idx_wq_b_scale, q,
                                          weights, q_scale, tile_config=None):
    """lightning_indexer_prolog_quant_v4_impl.py:118-266: 9 inputs, 3 outputs written in place, tile_config.
    Returns None."""
    rt.require_cuda()
    bf16 = torch.bfloat16
    rt.check_tensor(qr, "qr", torch.int8, (None, Q_LORA_RANK))
    t = qr.shape[0]
    rt.check_tensor(idx_wq_b, "idx_wq_b", torch.int8, (Q_LORA_RANK, IDX_NQ * HEAD_DIM))
    rt.check_tensor(x, "x", bf16, (t, None))
    h = x.shape[1]
    rt.check_tensor(weights_proj, "weights_proj", bf16, (h, IDX_NQ))
    rt.check_tensor(cos, "cos", bf16, (t, ROPE_DIM))
    rt.check_tensor(sin, "sin", bf16, (t, ROPE_DIM))
    rt.check_tensor(hadamard, "hadamard", bf16, (HEAD_DIM, HEAD_DIM))
    rt.check_tensor(qr_scale, "qr_scale", torch.float32, (t, 1))
    rt.check_tensor(idx_wq_b_scale, "idx_wq_b_scale", torch.float32, (IDX_NQ * HEAD_DIM, 1))
    if q.dim() == 2:  # the operator's table lists q as (t, idx_nq * head_dim); its callers pass (t, idx_nq, head_dim)
        rt.check_tensor(q, "q", torch.int8, (t, IDX_NQ * HEAD_DIM))
    else:
        rt.check_tensor(q, "q", torch.int8, (t, IDX_NQ, HEAD_DIM))
    rt.check_tensor(weights, "weights", torch.float16, (t, IDX_NQ))
    rt.check_tensor(q_scale, "q_scale", torch.float16, (t, IDX_NQ))
    if t == 0:
        return None
    dev = rt.same_device(qr, idx_wq_b, x, weights_proj, cos, sin, hadamard, qr_scale, idx_wq_b_scale, q, weights, q_scale)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_prolog_v4_workspace_bytes(t, h)
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.PrologV4Args(rt.ptr(qr), rt.ptr(idx_wq_b), rt.ptr(x), rt.ptr(weights_proj), rt.ptr(cos), rt.ptr(sin),
                              rt.ptr(hadamard), rt.ptr(qr_scale), rt.ptr(idx_wq_b_scale), rt.ptr(q), rt.ptr(weights),
                              rt.ptr(q_scale), rt.ptr(ws), int(ws_bytes), rt.ptr(rt.status_word(dev)), t, h)
        rt.check(lib.dsv32_indexer_prolog_v4(C.byref(a), rt.stream_ptr(dev)), "quant_lightning_indexer_prolog")
    return None


def npu_quant_lightning_indexer_prolog(qr, idx_wq_b, x, weights_proj, cos, sin, hadamard, qr_scale, idx_wq_b_scale):
    """lightning_indexer_prolog_quant_v4_impl.py:78-115: allocates and returns (q int8 [t, 64, 128],
    weights fp16 [t, 64], q_scale fp16 [t, 64])."""
    if not isinstance(qr, torch.Tensor) or qr.dim() != 2:
        raise ValueError("qr: expected a 2-D tensor")
    t = qr.shape[0]
    q = torch.empty((t, IDX_NQ, HEAD_DIM), dtype=torch.int8, device=qr.device)
    weights = torch.empty((t, IDX_NQ), dtype=torch.float16, device=qr.device)
    q_scale = torch.empty((t, IDX_NQ), dtype=torch.float16, device=qr.device)
    quant_lightning_indexer_prolog_kernel(qr, idx_wq_b, x, weights_proj, cos, sin, hadamard, qr_scale, idx_wq_b_scale,
                                          q, weights, q_scale, IndexerPrologQuantConfig())
    return q, weights, q_scale
