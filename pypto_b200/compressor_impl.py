"""DeepSeek-V4 KV compressor entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/compressor_impl.py (npu_compressor :139-226,
compressor_pypto :101-136; kernels compressor_ratio_4_kernel :428-588, compressor_ratio_4_rotate_kernel :598-778,
compressor_ratio_128_kernel :788-923).  Every `ratio` (4 or 128) tokens of a request are compressed into one
cache row: per token kv = x @ wkv.T and score = x @ wgate.T + ape[pos % ratio] are stored into paged fp32 states;
when a window is complete its kv rows are summed with softmax(score rows) weights per column (ratio 4 mixes the
first halves of the previous window with the second halves of the current one), RMS-normalised, given the
interleaved rotary embedding on the last 64 dims and, with `rotate`, multiplied by a hadamard matrix.
The two projections and the hadamard product run on this library's tcgen05 GEMM kernel (dsv32_gemm_bf16; bf16 operands
with fp32 accumulation, i.e. the reference golden's fp32 product up to summation order; the weights are read as they
are held, one row per output column); the state update and the compression are one CUDA kernel.  `kv_state` and `score_state` are
updated in place and returned with the new rows, as the reference does.  Work is only enqueued on the current stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import _runtime as rt

PAGE, ROPE_DIM, EPS = 128, 64, 1e-6


def npu_compressor(x, kv_state, score_state, kv_block_table, score_block_table, sin, cos, wkv, wgate, ape, weight,
                   hadamard, start_pos, ratio, rope_head_dim, rotate):
    """compressor_impl.py:139-226.  Returns (out bf16 [min(b*s1, b*s1 // ratio + b), d], kv_state, score_state)."""
    rt.require_cuda()
    ratio = int(ratio)
    if ratio not in (4, 128):
        raise ValueError(f"ratio={ratio}: expected 4 or 128")
    if int(rope_head_dim) != ROPE_DIM:
        raise ValueError(f"rope_head_dim={rope_head_dim}: expected {ROPE_DIM}")
    if not isinstance(rotate, bool):
        raise ValueError(f"rotate: expected a bool, got {type(rotate).__name__}")
    coff = 2 if ratio == 4 else 1
    bf16, f32 = torch.bfloat16, torch.float32
    rt.check_tensor(weight, "weight", f32, (None,))
    d = weight.shape[0]
    if d < ROPE_DIM or d > 512 or d % 2:
        raise ValueError(f"weight: {d} output dims, expected an even number in [64, 512]")
    rt.check_tensor(x, "x", bf16, (None, None, None))
    b, s1, h = x.shape
    rt.check_tensor(kv_state, "kv_state", f32, (None, PAGE, coff * d))
    rt.check_tensor(score_state, "score_state", f32, (None, PAGE, coff * d))
    rt.check_tensor(kv_block_table, "kv_block_table", torch.int32, (b, None))
    rt.check_tensor(score_block_table, "score_block_table", torch.int32, (b, None))
    rows = min(b * s1, b * s1 // ratio + b)
    rt.check_tensor(sin, "sin", bf16, (rows, ROPE_DIM))
    rt.check_tensor(cos, "cos", bf16, (rows, ROPE_DIM))
    rt.check_tensor(wkv, "wkv", bf16, (coff * d, h))
    rt.check_tensor(wgate, "wgate", bf16, (coff * d, h))
    rt.check_tensor(ape, "ape", f32, (ratio, coff * d))
    rt.check_tensor(hadamard, "hadamard", bf16, (d, d))
    rt.check_tensor(start_pos, "start_pos", torch.int32, (b,))
    out = torch.zeros((rows, d), dtype=x.dtype, device=x.device)
    if b == 0 or s1 == 0:
        return out, kv_state, score_state
    dev = rt.same_device(x, kv_state, score_state, kv_block_table, score_block_table, sin, cos, wkv, wgate, ape, weight,
                         hadamard, start_pos)
    lib = _lib.load()
    with torch.cuda.device(dev):
        x2 = x.reshape(b * s1, h)
        kv_total = rt.gemm_bf16_fp32(x2, wkv.t())              # [b*s1, coff*d] fp32
        score_total = rt.gemm_bf16_fp32(x2, wgate.t())
        a = _lib.CompressorArgs(rt.ptr(kv_total), rt.ptr(score_total), rt.ptr(ape), rt.ptr(weight), rt.ptr(kv_state),
                                rt.ptr(score_state), rt.ptr(kv_block_table), rt.ptr(score_block_table), rt.ptr(sin),
                                rt.ptr(cos), rt.ptr(start_pos), rt.ptr(out), rt.ptr(rt.status_word(dev)),
                                kv_state.shape[0], score_state.shape[0], b, s1, d, ratio, kv_block_table.shape[1],
                                score_block_table.shape[1], EPS)
        rt.check(lib.dsv32_compressor_update(C.byref(a), rt.stream_ptr(dev)), "compressor")
        if rotate:
            out = rt.gemm_bf16(out, hadamard, torch.bfloat16)  # rows of requests that did not compress stay zero
    return out, kv_state, score_state


def compressor_pypto(x, kv_state, score_state, kv_block_table, score_block_table, sin, cos, wkv, wgate, ape, weight,
                     hadamard, start_pos, ratio, rope_head_dim, rotate):
    """compressor_impl.py:101-136 (the torch.ops route of the reference): same call."""
    return npu_compressor(x, kv_state, score_state, kv_block_table, score_block_table, sin, cos, wkv, wgate, ape, weight,
                          hadamard, start_pos, ratio, rope_head_dim, rotate)
