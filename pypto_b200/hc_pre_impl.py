"""DeepSeek-V4 hyper-connection pre-mix entry points for B200.

Same names, argument order and layouts as models/deepseek_v4/hc_pre_impl.py (hc_pre_kernel :100-206,
hc_pre_kernel_prefill :216-309, npu_hc_pre :371-392, hc_pre_pypto :366-367).  Per token, x holds 4 residual
streams of 4096 values:
  mix  = x.reshape(16384) @ hc_fn.T / sqrt(mean(x^2) + 1e-6)                       (24 values, fp32)
  pre  = sigmoid(mix[0:4] * hc_scale[0] + hc_base[0:4]) + hc_eps
  post = 2 * sigmoid(mix[4:8] * hc_scale[1] + hc_base[4:8])
  comb = Sinkhorn normalisation of the 4x4 matrix mix[8:24] * hc_scale[2] + hc_base[8:24]
  y    = bf16(sum_h pre[h] * x[h])
Two CUDA kernels: the 24 mixing dot products with hc_fn staged in shared memory and shared by a tile of tokens,
then a per-token finish (Sinkhorn on 16 lanes of a warp, weighted sum of the streams).  The decode and the prefill
kernel of the reference compute the same function, so both names run it.  Work is only enqueued on the current stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import _runtime as rt

HC_MULT, D, NORM_EPS = 4, 4096, 1e-6


def hc_pre_kernel(x, hc_fn, hc_scale, hc_base, y, post, comb, hc_mult=4, hc_split_sinkhorn_iters=20, hc_eps=1e-6):
    """hc_pre_impl.py:100-206: 4 inputs, 3 outputs written in place, then hc_mult, iterations, epsilon.  Returns None."""
    rt.require_cuda()
    if int(hc_mult) != HC_MULT:
        raise ValueError(f"hc_mult={hc_mult}: only {HC_MULT} residual streams are supported")
    if int(hc_split_sinkhorn_iters) < 1:
        raise ValueError(f"hc_split_sinkhorn_iters={hc_split_sinkhorn_iters} must be >= 1")
    mix = (2 + HC_MULT) * HC_MULT
    rt.check_tensor(x, "x", torch.bfloat16, (None, HC_MULT, D))
    t = x.shape[0]
    rt.check_tensor(hc_fn, "hc_fn", torch.float32, (mix, HC_MULT * D))
    rt.check_tensor(hc_scale, "hc_scale", torch.float32, (3,))
    rt.check_tensor(hc_base, "hc_base", torch.float32, (mix,))
    rt.check_tensor(y, "y", torch.bfloat16, (t, D))
    rt.check_tensor(post, "post", torch.float32, (t, HC_MULT))
    rt.check_tensor(comb, "comb", torch.float32, (t, HC_MULT, HC_MULT))
    if t == 0:
        return None
    dev = rt.same_device(x, hc_fn, hc_scale, hc_base, y, post, comb)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_hc_pre_workspace_bytes(t)
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.HcPreArgs(rt.ptr(x), rt.ptr(hc_fn), rt.ptr(hc_scale), rt.ptr(hc_base), rt.ptr(y), rt.ptr(post),
                           rt.ptr(comb), rt.ptr(ws), int(ws_bytes), t, HC_MULT, D, int(hc_split_sinkhorn_iters),
                           NORM_EPS, float(hc_eps))
        rt.check(lib.dsv32_hc_pre(C.byref(a), rt.stream_ptr(dev)), "hc_pre")
    return None


def hc_pre_kernel_prefill(x, hc_fn, hc_scale, hc_base, y, post, comb, hc_mult=4, hc_split_sinkhorn_iters=20, hc_eps=1e-6):
    """hc_pre_impl.py:216-309: the reference's transposed formulation for many tokens; same function."""
    return hc_pre_kernel(x, hc_fn, hc_scale, hc_base, y, post, comb, hc_mult, hc_split_sinkhorn_iters, hc_eps)


def npu_hc_pre(x, hc_fn, hc_scale, hc_base, hc_mult: int = 4, hc_split_sinkhorn_iters: int = 20, hc_eps: float = 1e-6):
    """hc_pre_impl.py:371-392: allocates and returns (y bf16 [t, 4096], post fp32 [t, 4], comb fp32 [t, 4, 4])."""
    if not isinstance(x, torch.Tensor) or x.dim() != 3:
        raise ValueError("x: expected a 3-D tensor [t, hc_mult, 4096]")
    y = torch.empty((x.shape[0], x.shape[2]), dtype=x.dtype, device=x.device)
    post = torch.empty((x.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
    comb = torch.empty((x.shape[0], x.shape[1], x.shape[1]), dtype=torch.float32, device=x.device)
    hc_pre_kernel(x, hc_fn, hc_scale, hc_base, y, post, comb, hc_mult, hc_split_sinkhorn_iters, hc_eps)
    return y, post, comb


def hc_pre_pypto(x, hc_fn, hc_scale, hc_base, hc_mult, hc_sinkhorn_iters, hc_eps):
    """hc_pre_impl.py:366-367 (the torch.ops route of the reference): same call."""
    return npu_hc_pre(x, hc_fn, hc_scale, hc_base, hc_mult, hc_sinkhorn_iters, hc_eps)
