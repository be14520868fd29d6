"""Shared host side of the two page-grouped 8-bit-float indexer prologs (MXFP8 and HiF8): argument checks and the
one C call.  The public entry points live in lightning_indexer_prolog_quant_mxfp8_impl.py and
lightning_indexer_prolog_quant_hif8_impl.py."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import _runtime as rt

HEAD_DIM, ROPE_DIM = 128, 64
FORMAT_MXFP8, FORMAT_HIF8 = 0, 1
_CODE_DTYPES = {FORMAT_MXFP8: (torch.float8_e4m3fn, torch.uint8), FORMAT_HIF8: (torch.uint8,)}


def _check_codes(t, name, fmt, shape):
    if not isinstance(t, torch.Tensor) or t.dtype not in _CODE_DTYPES[fmt]:
        raise ValueError(f"{name}: expected dtype in {_CODE_DTYPES[fmt]}, got {getattr(t, 'dtype', type(t).__name__)}")
    rt.check_tensor(t, name, t.dtype, shape)


def _paged_view(cache, name, dtype_ok, last, elem_bytes):
    """A cache argument is [pages, block_size, 1, last] with contiguous pages that may sit `stride(0)` elements
    apart (a view into a page-grouped buffer).  Returns (pages, block_size, page stride in bytes)."""
    if not isinstance(cache, torch.Tensor) or cache.dtype not in dtype_ok:
        raise ValueError(f"{name}: expected dtype in {dtype_ok}, got {getattr(cache, 'dtype', type(cache).__name__)}")
    if not cache.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor, got device {cache.device}")
    if cache.dim() != 4 or cache.shape[2] != 1 or cache.shape[3] != last:
        raise ValueError(f"{name}: expected shape (pages, block_size, 1, {last}), got {tuple(cache.shape)}")
    pages, bs = int(cache.shape[0]), int(cache.shape[1])
    if cache.stride(3) != 1 or cache.stride(2) != last or cache.stride(1) != last or (pages > 1 and cache.stride(0) < bs * last):
        raise ValueError(f"{name}: pages must be contiguous [block_size, 1, {last}] blocks, got strides {cache.stride()}")
    return pages, bs, (cache.stride(0) if pages > 1 else bs * last) * elem_bytes


def pg_prolog(fmt, x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, gamma_k_in, cos_idx_rope_in,
              sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_quant_in, k_scale_in, k_cache_index_in,
              k_scale_cache_index_in, q_quant_out, q_scale_out, k_quant_out, k_scale_out, weights_out, eps=1e-6):
    rt.require_cuda()
    bf16 = torch.bfloat16
    rt.check_tensor(x_in, "x_in", bf16, ndim=2)
    t, h = int(x_in.shape[0]), int(x_in.shape[1])
    _check_codes(q_norm_in, "q_norm_in", fmt, (t, None))
    q_lora = int(q_norm_in.shape[1])
    _check_codes(w_qb_in, "w_qb_in", fmt, (q_lora, None))
    n = int(w_qb_in.shape[1])
    rt.check_tensor(w_proj_in, "w_proj_in", bf16, (h, None))
    heads = int(w_proj_in.shape[1])
    if n != heads * HEAD_DIM:
        raise ValueError(f"w_qb_in: expected {heads} heads x {HEAD_DIM} = {heads * HEAD_DIM} columns, got {n}")
    if fmt == FORMAT_MXFP8:
        for name, s, numel in (("q_norm_scale_in", q_norm_scale_in, t * (q_lora // 32)), ("w_qb_scale_in", w_qb_scale_in, (q_lora // 32) * n)):
            if not isinstance(s, torch.Tensor) or s.dtype not in (torch.float8_e8m0fnu, torch.uint8):
                raise ValueError(f"{name}: expected E8M0 scales (torch.float8_e8m0fnu or uint8 codes)")
            rt.check_tensor(s, name, s.dtype)
            if s.numel() != numel:
                raise ValueError(f"{name}: expected {numel} scales (one per 32 reduction elements), got {s.numel()}")
        if w_qb_scale_in.dim() != 3 or tuple(w_qb_scale_in.shape) != (q_lora // 64, n, 2):
            raise ValueError(f"w_qb_scale_in: expected shape ({q_lora // 64}, {n}, 2), got {tuple(w_qb_scale_in.shape)}")
    else:
        rt.check_tensor(q_norm_scale_in, "q_norm_scale_in", torch.float32, (t, 1))
        rt.check_tensor(w_qb_scale_in, "w_qb_scale_in", torch.float32, (1, n))
    rt.check_tensor(wk_in, "wk_in", bf16, (h, HEAD_DIM))
    rt.check_tensor(gamma_k_in, "gamma_k_in", bf16)
    if gamma_k_in.numel() != HEAD_DIM:
        raise ValueError(f"gamma_k_in: expected {HEAD_DIM} elements, got shape {tuple(gamma_k_in.shape)}")
    rt.check_tensor(cos_idx_rope_in, "cos_idx_rope_in", bf16, (t, ROPE_DIM))
    rt.check_tensor(sin_idx_rope_in, "sin_idx_rope_in", bf16, (t, ROPE_DIM))
    rt.check_tensor(hadamard_q_in, "hadamard_q_in", bf16, (HEAD_DIM, HEAD_DIM))
    rt.check_tensor(hadamard_k_in, "hadamard_k_in", bf16, (HEAD_DIM, HEAD_DIM))
    rt.check_tensor(k_cache_index_in, "k_cache_index_in", torch.int64, (t, 1))
    rt.check_tensor(k_scale_cache_index_in, "k_scale_cache_index_in", torch.int64, (t, 1))
    _check_codes(q_quant_out, "q_quant_out", fmt, (t * heads, HEAD_DIM))
    rt.check_tensor(q_scale_out, "q_scale_out", torch.float32, (t * heads, 1))
    rt.check_tensor(weights_out, "weights_out", bf16, (t, heads))
    # the caches are updated in place: the operator's *_in and *_out arguments name the same storage
    for a, b, name in ((k_quant_in, k_quant_out, "k_quant"), (k_scale_in, k_scale_out, "k_scale")):
        if a.data_ptr() != b.data_ptr() or a.stride() != b.stride() or a.shape != b.shape:
            raise ValueError(f"{name}_in and {name}_out must be the same cache view (the update is in place)")
    pages, bs, k_stride = _paged_view(k_quant_out, "k_quant_out", _CODE_DTYPES[fmt], HEAD_DIM, 1)
    pages_s, bs_s, ks_stride = _paged_view(k_scale_out, "k_scale_out", (torch.float32,), 1, 4)
    if (pages_s, bs_s) != (pages, bs):
        raise ValueError(f"k_scale_out: expected {pages} pages of {bs} rows like k_quant_out, got {pages_s} x {bs_s}")
    if t == 0:
        return None
    dev = rt.same_device(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, gamma_k_in,
                         cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_quant_out, k_scale_out,
                         k_cache_index_in, k_scale_cache_index_in, q_quant_out, q_scale_out, weights_out)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_pg_indexer_prolog_workspace_bytes(t, h, q_lora, heads)
        ws = rt.workspace(ws_bytes, dev)
        a = _lib.PgPrologArgs(
            rt.ptr(x_in), rt.ptr(q_norm_in), rt.ptr(q_norm_scale_in), rt.ptr(w_qb_in), rt.ptr(w_qb_scale_in), rt.ptr(wk_in),
            rt.ptr(w_proj_in), rt.ptr(gamma_k_in), rt.ptr(cos_idx_rope_in), rt.ptr(sin_idx_rope_in), rt.ptr(hadamard_q_in),
            rt.ptr(hadamard_k_in), rt.ptr(k_cache_index_in), rt.ptr(k_scale_cache_index_in), rt.ptr(q_quant_out),
            rt.ptr(q_scale_out), rt.ptr(k_quant_out), rt.ptr(k_scale_out), rt.ptr(weights_out), rt.ptr(ws), int(ws_bytes),
            rt.ptr(rt.status_word(dev)), pages * bs, int(k_stride), int(ks_stride), t, h, q_lora, heads, bs, fmt, float(eps))
        rt.check(lib.dsv32_pg_indexer_prolog(C.byref(a), rt.stream_ptr(dev)), "lightning_indexer_prolog_quant (page-grouped)")
    return None
