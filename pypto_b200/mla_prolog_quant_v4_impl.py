"""DeepSeek-V4 MLA prolog (quant) entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/mla_prolog_quant_v4_impl.py (mla_prolog_v4 :528-564,
mla_prolog_v4_in :567-629, mla_prolog_quant_pypto :655-658; compute mla_prolog_v4_compute :406-517).  Per token:
  qr, qr_scale = per-token int8 quant of RMSNorm(x @ wq_a) * gamma_cq            (feeds the V4 indexer prolog)
  q            = bf16(RMSNorm_per_head(int32(qr @ wq_b) * qr_scale * wq_b_scale)), heads of 512 dims, interleaved
                 rotary embedding on the last 64 dims of each head                (the query of the V4 attention)
  kv           = bf16(RMSNorm(x @ wkv) * gamma_ckv), rotary embedding on its last 64 dims   (the new cache row)
The three projections run on this library's tcgen05 GEMM kernel (dsv32_gemm_bf16: bf16 operands, fp32 accumulation and
fp32 results, which is the reference golden's fp32 product of the widened operands up to summation order;
dsv32_gemm_i8: int8 with exact int32 accumulation); everything between them is one fused CUDA kernel per stage.
Weights are plain row-major [K, N].  Work is enqueued on the current CUDA stream and, for the
independent kv branch, on a second stream of the device that is forked from and joined back into it by events
(also when the q branch raises).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from . import _lib
from . import _runtime as rt

Q_LORA_RANK, HEAD_DIM, ROPE_DIM = 1024, 512, 64


@dataclass
class MlaTileConfigs:
    """Ascend vector tile shapes (mla_prolog_quant_v4_impl.py:76-82); carried for signature parity only."""
    two_dim_tile: list = field(default_factory=lambda: [1, 64])
    three_dim_tile: list = field(default_factory=lambda: [1, 64, 64])
    four_dim_tile: list = field(default_factory=lambda: [1, 64, 64, 64])
    vec_tile: list = field(default_factory=lambda: [1, 64])


@dataclass
class MlaPrologV4Attrs:
    """mla_prolog_quant_v4_impl.py:91-94: the RMSNorm epsilon is the only field that carries math."""
    eps: float = 1e-6


@dataclass
class MlaPrologV4Configs:
    """Ascend pass knobs (mla_prolog_quant_v4_impl.py:96-105); carried for signature parity only."""
    unroll_list: list = field(default_factory=lambda: [128, 64, 32, 16, 1])
    cube_l1_reuse_setting: dict = field(default_factory=dict)
    mg_copyin_upper_bound: int = 2 * 1024 * 1024
    pg_upper_bound: int = 8192
    block_size: int = 128
    t_sub_tile: int = 1
    chunk_size: int = 2



def mla_prolog_v4(token_x, wq_a, wq_b, wkv, gamma_cq, gamma_ckv, rope_cos, rope_sin, wq_b_scale, q_out, kv_out, qr_out,
                  qr_scale_out, attrs=None, configs=None, tile_configs=None):
    """mla_prolog_quant_v4_impl.py:528-564: 9 inputs (note gamma before cos / sin here), 4 outputs written in place,
    then attrs, configs, tile_configs.  Returns None."""
    rt.require_cuda()
    bf16 = torch.bfloat16
    rt.check_tensor(token_x, "token_x", bf16, (None, None))
    t, h = token_x.shape
    rt.check_tensor(wq_a, "wq_a", bf16, (h, Q_LORA_RANK))
    rt.check_tensor(wq_b, "wq_b", torch.int8, (Q_LORA_RANK, None))
    if wq_b.shape[1] == 0 or wq_b.shape[1] % HEAD_DIM != 0:
        raise ValueError(f"wq_b: {wq_b.shape[1]} columns are not a positive multiple of the head size {HEAD_DIM}")
    heads = wq_b.shape[1] // HEAD_DIM
    rt.check_tensor(wkv, "wkv", bf16, (h, HEAD_DIM))
    rt.check_tensor(gamma_cq, "gamma_cq", bf16, (Q_LORA_RANK,))
    rt.check_tensor(gamma_ckv, "gamma_ckv", bf16, (HEAD_DIM,))
    rt.check_tensor(rope_cos, "rope_cos", bf16, (t, ROPE_DIM))
    rt.check_tensor(rope_sin, "rope_sin", bf16, (t, ROPE_DIM))
    if wq_b_scale.dim() == 2 and wq_b_scale.shape[0] == 1:    # the reference generator makes it [1, heads * 512]
        rt.check_tensor(wq_b_scale, "wq_b_scale", torch.float32, (1, heads * HEAD_DIM))
    elif wq_b_scale.dim() == 2:
        rt.check_tensor(wq_b_scale, "wq_b_scale", torch.float32, (heads * HEAD_DIM, 1))
    else:
        rt.check_tensor(wq_b_scale, "wq_b_scale", torch.float32, (heads * HEAD_DIM,))
    rt.check_tensor(q_out, "q_out", bf16, (t, heads, HEAD_DIM))
    rt.check_tensor(kv_out, "kv_out", bf16, (t, HEAD_DIM))
    rt.check_tensor(qr_out, "qr_out", torch.int8, (t, Q_LORA_RANK))
    rt.check_tensor(qr_scale_out, "qr_scale_out", torch.float32, (t, 1))
    if t == 0:
        return None
    eps = float(attrs.eps) if attrs is not None else 1e-6
    dev = rt.same_device(token_x, wq_a, wq_b, wkv, gamma_cq, gamma_ckv, rope_cos, rope_sin, wq_b_scale, q_out, kv_out,
                         qr_out, qr_scale_out)
    lib = _lib.load()
    with torch.cuda.device(dev):
        a = _lib.MlaV4StageArgs(None, rt.ptr(gamma_cq), rt.ptr(qr_out), rt.ptr(qr_scale_out), None,
                                rt.ptr(wq_b_scale), rt.ptr(q_out), None, rt.ptr(gamma_ckv), rt.ptr(kv_out),
                                rt.ptr(rope_cos), rt.ptr(rope_sin), t, heads, 0, 1, eps)
        # the kv branch (one GEMM + one stage kernel) is independent of the q branch: it runs on a second stream
        fork = rt.side_stream(dev)
        with fork:
            kv_a = rt.gemm_bf16_fp32(token_x, wkv)                               # [t, 512] fp32
            a.kv_a = rt.ptr(kv_a)
            rt.check(lib.dsv32_mla_prolog_v4_stage(C.byref(a), 2, rt.stream_ptr(dev)), "mla_prolog_v4 (kv norm + rope)")
        try:   # whatever happens on this branch, the caller's stream must wait for the side branch
            stream = rt.stream_ptr(dev)
            q_a = rt.gemm_bf16_fp32(token_x, wq_a)                                   # [t, 1024] fp32
            a.q_a = rt.ptr(q_a)
            rt.check(lib.dsv32_mla_prolog_v4_stage(C.byref(a), 0, stream), "mla_prolog_v4 (q norm + quant)")
            q_b = rt.gemm_i8(qr_out, wq_b)                                       # [t, heads * 512] int32, exact
            a.q_b, a.q_b_ld = rt.ptr(q_b), q_b.shape[1]
            rt.check(lib.dsv32_mla_prolog_v4_stage(C.byref(a), 1, stream), "mla_prolog_v4 (q dequant + norm + rope)")
        finally:
            fork.join()
    return None


def mla_prolog_v4_in(token_x, wq_a, wq_b, wkv, rope_cos, rope_sin, gamma_cq, gamma_ckv, wq_b_scale):
    """mla_prolog_quant_v4_impl.py:567-629: allocates and returns (q bf16 [t, heads, 512], kv bf16 [t, 512],
    qr int8 [t, 1024], qr_scale fp32 [t, 1])."""
    for name, x in (("token_x", token_x), ("wq_b", wq_b), ("gamma_cq", gamma_cq), ("gamma_ckv", gamma_ckv)):
        if not isinstance(x, torch.Tensor):
            raise ValueError(f"{name}: expected a torch.Tensor, got {type(x).__name__}")
    if token_x.dim() != 2 or wq_b.dim() != 2 or gamma_ckv.dim() != 1 or gamma_cq.dim() != 1 or gamma_ckv.shape[0] == 0:
        raise ValueError("token_x / wq_b must be 2-D and gamma_cq / gamma_ckv 1-D")
    t, dev = token_x.shape[0], token_x.device
    q = torch.empty((t, wq_b.shape[1] // gamma_ckv.shape[0], gamma_ckv.shape[0]), dtype=token_x.dtype, device=dev)
    kv = torch.empty((t, gamma_ckv.shape[0]), dtype=token_x.dtype, device=dev)
    qr = torch.empty((t, gamma_cq.shape[0]), dtype=torch.int8, device=dev)
    qr_scale = torch.empty((t, 1), dtype=torch.float32, device=dev)
    mla_prolog_v4(token_x, wq_a, wq_b, wkv, gamma_cq, gamma_ckv, rope_cos, rope_sin, wq_b_scale, q, kv, qr, qr_scale,
                  MlaPrologV4Attrs(eps=1e-6), MlaPrologV4Configs(), MlaTileConfigs())
    return q, kv, qr, qr_scale


def mla_prolog_quant_pypto(token_x, wq_a, wq_b, wkv, rope_cos, rope_sin, gamma_cq, gamma_ckv, wq_b_scale):
    """mla_prolog_quant_v4_impl.py:655-658 (the torch.ops route of the reference): same call."""
    return mla_prolog_v4_in(token_x, wq_a, wq_b, wkv, rope_cos, rope_sin, gamma_cq, gamma_ckv, wq_b_scale)
