"""Page-grouped lightning indexer prolog, HiF8 form, for B200.

Same name, argument order and layouts as lightning_indexer_prolog_quant of
python/tests/st/operator/pg/lightning_indexer_prolog_quant_hif8_impl.py:230-406.  q_norm / w_qb are HiF8 codes (uint8;
bit layout framework/src/interface/machine/device/tilefwk/aicore_print_base.h:361-484) with one fp32 scale per token
(q_norm_scale [t, 1]) and per output column (w_qb_scale [1, heads * 128]); query and key rows leave as HiF8 codes
with an fp32 scale amax / 32768 each.  `hif8_encode` / `hif8_decode` convert CUDA arrays.  Work is only enqueued on
the current CUDA stream.
"""
from __future__ import annotations

import torch

from . import _lib, _pg_prolog
from . import _runtime as rt


def lightning_indexer_prolog_quant(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, gamma_k_in,
                                   cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_quant_in, k_scale_in,
                                   k_cache_index_in, k_scale_cache_index_in, q_quant_out, q_scale_out, k_quant_out,
                                   k_scale_out, weights_out):
    """lightning_indexer_prolog_quant_hif8_impl.py:230-406.  Returns None; outputs are written in place."""
    return _pg_prolog.pg_prolog(_pg_prolog.FORMAT_HIF8, x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in,
                                w_proj_in, gamma_k_in, cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in,
                                k_quant_in, k_scale_in, k_cache_index_in, k_scale_cache_index_in, q_quant_out, q_scale_out,
                                k_quant_out, k_scale_out, weights_out)


def _convert(direction, src, dst_dtype):
    rt.require_cuda()
    rt.check_tensor(src, "input", torch.float32 if direction == 0 else torch.uint8)
    out = torch.empty(src.shape, dtype=dst_dtype, device=src.device)
    if src.numel():
        with torch.cuda.device(src.device):
            rt.check(_lib.load().dsv32_hif8_convert(direction, rt.ptr(src), rt.ptr(out), src.numel(), rt.stream_ptr(src.device)),
                     "hif8 conversion")
    return out


def hif8_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 CUDA tensor -> HiF8 codes (uint8): nearest value, ties away from zero, saturating at 2^15."""
    return _convert(0, x, torch.uint8)


def hif8_decode(codes: torch.Tensor) -> torch.Tensor:
    """HiF8 codes (uint8 CUDA tensor) -> fp32."""
    return _convert(1, codes, torch.float32)
