"""pypto_b200 -- B200-native (sm_100a) drop-in for the DeepSeek-V3.2 quantized sparse-attention decode
operators of hicann/pypto (models/deepseek_v32_exp).  The modules mirror the reference operator files:

    sparse_flash_attention_quant_impl     sparse_flash_attention_quant_d / _p / _d_950
    lightning_indexer_quant_impl          lightning_indexer_decode
    lightning_indexer_prolog_quant_impl   lightning_indexer_prolog_quant

All compute runs in libdsv32_b200.so (hand-written CUDA, C ABI in include/dsv32_b200.h).
"""
from ._runtime import check_status  # noqa: F401
from ._lib import Dsv32Error, launch_count  # noqa: F401

__all__ = ["check_status", "Dsv32Error", "launch_count"]
