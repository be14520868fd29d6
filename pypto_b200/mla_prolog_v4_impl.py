"""DeepSeek-V4 MLA prolog without quantisation: entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/mla_prolog_v4_impl.py (mla_prolog_v4 :393-412,
mla_prolog_v4_in :415-455, mla_prolog_pypto :479-480; compute mla_prolog_v4_compute :310-390).  Per token:
  qr = bf16(RMSNorm(bf16(x @ wq_a)) * gamma_cq)
  q  = bf16(RMSNorm_per_head(bf16(qr @ wq_b))), heads of 512 dims, interleaved rotary embedding on the last 64
  kv = bf16(RMSNorm(bf16(x @ wkv)) * gamma_ckv), rotary embedding on its last 64 dims
The three projections run on this library's tcgen05 GEMM kernel (dsv32_gemm_bf16, fp32 accumulation, one rounding to
bf16); the stages between them are the kernels of
the quantised operator (mla_prolog_quant_v4_impl) instantiated without the quantisation.  Work is enqueued on the
current CUDA stream and, for the independent kv branch, on a second stream of the device that is forked from and
joined back into it by events (also when the q branch raises).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List

import torch

from . import _lib
from . import _runtime as rt

Q_LORA_RANK, HEAD_DIM, ROPE_DIM = 1024, 512, 64


@dataclass
class MlaPrologV4Attrs:
    """mla_prolog_v4_impl.py:94-98: the RMSNorm epsilon is the only field that carries math."""
    eps: float = 1e-6
    layout_query: str = "TND"
    layout_key: str = "PA_BSND"


@dataclass
class MlaPrologV4Configs:
    """Ascend pass knobs (mla_prolog_v4_impl.py:101-109); carried for signature parity only."""
    unroll_list: List[int] = field(default_factory=lambda: [128, 64, 32, 16, 1])
    cube_l1_reuse_setting: dict = field(default_factory=dict)
    mg_copyin_upper_bound: int = 2 * 1024 * 1024
    pg_upper_bound: int = 8192
    block_size: int = 128
    t_sub_tile: int = 1
    chunk_size: int = 2


def mla_prolog_v4(token_x, wq_a, wq_b, wkv, gamma_cq, gamma_ckv, rope_cos, rope_sin, q_out, kv_out, qr_out, attrs=None,
                  configs=None):
    """mla_prolog_v4_impl.py:393-412: 8 inputs (gamma before cos / sin), 3 outputs written in place, attrs, configs.
    Returns None."""
    rt.require_cuda()
    bf16 = torch.bfloat16
    rt.check_tensor(token_x, "token_x", bf16, (None, None))
    t, h = token_x.shape
    rt.check_tensor(wq_a, "wq_a", bf16, (h, Q_LORA_RANK))
    rt.check_tensor(wq_b, "wq_b", bf16, (Q_LORA_RANK, None))
    if wq_b.shape[1] == 0 or wq_b.shape[1] % HEAD_DIM != 0:
        raise ValueError(f"wq_b: {wq_b.shape[1]} columns are not a positive multiple of the head size {HEAD_DIM}")
    heads = wq_b.shape[1] // HEAD_DIM
    rt.check_tensor(wkv, "wkv", bf16, (h, HEAD_DIM))
    rt.check_tensor(gamma_cq, "gamma_cq", bf16, (Q_LORA_RANK,))
    rt.check_tensor(gamma_ckv, "gamma_ckv", bf16, (HEAD_DIM,))
    rt.check_tensor(rope_cos, "rope_cos", bf16, (t, ROPE_DIM))
    rt.check_tensor(rope_sin, "rope_sin", bf16, (t, ROPE_DIM))
    rt.check_tensor(q_out, "q_out", bf16, (t, heads, HEAD_DIM))
    rt.check_tensor(kv_out, "kv_out", bf16, (t, HEAD_DIM))
    rt.check_tensor(qr_out, "qr_out", bf16, (t, Q_LORA_RANK))
    if t == 0:
        return None
    eps = float(attrs.eps) if attrs is not None else 1e-6
    dev = rt.same_device(token_x, wq_a, wq_b, wkv, gamma_cq, gamma_ckv, rope_cos, rope_sin, q_out, kv_out, qr_out)
    lib = _lib.load()
    with torch.cuda.device(dev):
        a = _lib.MlaV4StageArgs(None, rt.ptr(gamma_cq), rt.ptr(qr_out), None, None, None, rt.ptr(q_out), None,
                                rt.ptr(gamma_ckv), rt.ptr(kv_out), rt.ptr(rope_cos), rt.ptr(rope_sin), t, heads, 0, 0,
                                eps)
        # the kv branch (one GEMM + one stage kernel) is independent of the q branch: it runs on a second stream
        fork = rt.side_stream(dev)
        with fork:
            kv_a = rt.gemm_bf16(token_x, wkv, torch.bfloat16)             # [t, 512] bf16
            a.kv_a = rt.ptr(kv_a)
            rt.check(lib.dsv32_mla_prolog_v4_stage(C.byref(a), 2, rt.stream_ptr(dev)), "mla_prolog_v4 (kv norm + rope)")
        try:   # whatever happens on this branch, the caller's stream must wait for the side branch
            stream = rt.stream_ptr(dev)
            q_a = rt.gemm_bf16(token_x, wq_a, torch.bfloat16)                 # [t, 1024] bf16
            a.q_a = rt.ptr(q_a)
            rt.check(lib.dsv32_mla_prolog_v4_stage(C.byref(a), 0, stream), "mla_prolog_v4 (q norm)")
            q_b = rt.gemm_bf16(qr_out, wq_b, torch.bfloat16)                  # [t, heads * 512] bf16
            a.q_b, a.q_b_ld = rt.ptr(q_b), q_b.shape[1]
            rt.check(lib.dsv32_mla_prolog_v4_stage(C.byref(a), 1, stream), "mla_prolog_v4 (q norm + rope)")
        finally:
            fork.join()
    return None


def mla_prolog_v4_in(token_x, wq_a, wq_b, wkv, rope_cos, rope_sin, gamma_cq, gamma_ckv):
    """mla_prolog_v4_impl.py:415-455: allocates and returns (q bf16 [t, heads, 512], kv bf16 [t, 512],
    qr bf16 [t, 1024])."""
    for name, x in (("token_x", token_x), ("wq_b", wq_b), ("gamma_cq", gamma_cq), ("gamma_ckv", gamma_ckv)):
        if not isinstance(x, torch.Tensor):
            raise ValueError(f"{name}: expected a torch.Tensor, got {type(x).__name__}")
    if token_x.dim() != 2 or wq_b.dim() != 2 or gamma_ckv.dim() != 1 or gamma_cq.dim() != 1 or gamma_ckv.shape[0] == 0:
        raise ValueError("token_x / wq_b must be 2-D and gamma_cq / gamma_ckv 1-D")
    t, dev = token_x.shape[0], token_x.device
    q = torch.zeros((t, wq_b.shape[1] // gamma_ckv.shape[0], gamma_ckv.shape[0]), dtype=token_x.dtype, device=dev)
    kv = torch.zeros((t, gamma_ckv.shape[0]), dtype=token_x.dtype, device=dev)
    qr = torch.zeros((t, gamma_cq.shape[0]), dtype=token_x.dtype, device=dev)
    mla_prolog_v4(token_x, wq_a, wq_b, wkv, gamma_cq, gamma_ckv, rope_cos, rope_sin, q, kv, qr, MlaPrologV4Attrs(),
                  MlaPrologV4Configs())
    return q, kv, qr


def mla_prolog_pypto(token_x, wq_a, wq_b, wkv, rope_cos, rope_sin, gamma_cq, gamma_ckv):
    """mla_prolog_v4_impl.py:479-480 (the torch.ops route of the reference): same call."""
    return mla_prolog_v4_in(token_x, wq_a, wq_b, wkv, rope_cos, rope_sin, gamma_cq, gamma_ckv)
