"""Page-grouped lightning indexer prolog, MXFP8 form, for B200.

Same name, argument order and layouts as lightning_indexer_prolog_quant of
python/tests/st/operator/pg/lightning_indexer_prolog_quant_mxfp8_impl.py:230-401: sixteen inputs, five outputs
written in place.  q_norm / w_qb are float8 E4M3 codes with one E8M0 scale per 32 reduction elements
(q_norm_scale [t, q_lora / 32], w_qb_scale [q_lora / 64, heads * 128, 2]); the query and key rows leave as E4M3
codes with an fp32 scale amax / 448 each; the key cache and its scale cache are page-grouped views (pages may sit
further apart than their own size, test_pg_lightning_indexer_prolog_quant_mxfp8.py:196-201).  The float8 tensors
may be passed as torch.float8_e4m3fn / torch.float8_e8m0fnu or as uint8 codes.  Work is only enqueued on the
current CUDA stream.
"""
from __future__ import annotations

from . import _pg_prolog


def lightning_indexer_prolog_quant(x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in, w_proj_in, gamma_k_in,
                                   cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in, k_quant_in, k_scale_in,
                                   k_cache_index_in, k_scale_cache_index_in, q_quant_out, q_scale_out, k_quant_out,
                                   k_scale_out, weights_out):
    """lightning_indexer_prolog_quant_mxfp8_impl.py:230-401.  Returns None; q_quant_out [t * heads, 128],
    q_scale_out [t * heads, 1], weights_out [t, heads] and the cache rows named by the two index tensors are written."""
    return _pg_prolog.pg_prolog(_pg_prolog.FORMAT_MXFP8, x_in, q_norm_in, q_norm_scale_in, w_qb_in, w_qb_scale_in, wk_in,
                                w_proj_in, gamma_k_in, cos_idx_rope_in, sin_idx_rope_in, hadamard_q_in, hadamard_k_in,
                                k_quant_in, k_scale_in, k_cache_index_in, k_scale_cache_index_in, q_quant_out, q_scale_out,
                                k_quant_out, k_scale_out, weights_out)
