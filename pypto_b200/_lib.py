"""ctypes binding of libdsv32_b200.so (the C ABI declared in include/dsv32_b200.h).

There is no CPU fallback: if the shared library is missing or a call is rejected the
functions here raise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("DSV32_B200_LIB", os.path.join(HERE, "libdsv32_b200.so"))

c_void_p, c_i32, c_i64, c_size_t, c_float = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float


class SfaArgs(C.Structure):
    _fields_ = [
        ("query_nope", c_void_p), ("query_rope", c_void_p), ("key_nope", c_void_p), ("key_rope", c_void_p),
        ("k_nope_scales", c_void_p), ("topk_indices", c_void_p), ("block_table", c_void_p), ("kv_act_seqs", c_void_p),
        ("attention_out", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("status", c_void_p),
        ("rows", c_i64), ("b", c_i32), ("s1", c_i32), ("n_q", c_i32), ("topk", c_i32), ("block_size", c_i32),
        ("max_blocks", c_i32), ("kv_splits", c_i32), ("softmax_scale", c_float),
    ]


class SaAntiquantArgs(C.Structure):
    _fields_ = [
        ("query_nope", c_void_p), ("query_rope", c_void_p), ("nope_cache", c_void_p), ("topk_indices", c_void_p),
        ("block_table", c_void_p), ("kv_act_seqs", c_void_p), ("attention_out", c_void_p), ("workspace", c_void_p),
        ("workspace_bytes", c_size_t), ("status", c_void_p), ("rows", c_i64), ("b", c_i32), ("s1", c_i32),
        ("n_q", c_i32), ("topk", c_i32), ("block_size", c_i32), ("max_blocks", c_i32), ("kv_splits", c_i32),
        ("softmax_scale", c_float),
    ]


class ScfaArgs(C.Structure):
    _fields_ = [
        ("query", c_void_p), ("actual_seq_q", c_void_p), ("ori_kv", c_void_p), ("cmp_kv", c_void_p),
        ("ori_block_table", c_void_p), ("cmp_block_table", c_void_p), ("atten_sink", c_void_p),
        ("seqused_kv", c_void_p), ("cmp_sparse_indices", c_void_p), ("attention_out", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("status", c_void_p), ("ori_rows", c_i64),
        ("cmp_rows", c_i64), ("t", c_i32), ("b", c_i32), ("n_q", c_i32), ("topk", c_i32), ("block_size", c_i32),
        ("win_size", c_i32), ("cmp_ratio", c_i32), ("ori_max_blocks", c_i32), ("cmp_max_blocks", c_i32),
        ("cmp_mode", c_i32), ("softmax_scale", c_float),
    ]


class MlaV4StageArgs(C.Structure):
    _fields_ = [
        ("q_a", c_void_p), ("gamma_cq", c_void_p), ("qr", c_void_p), ("qr_scale", c_void_p), ("q_b", c_void_p),
        ("wq_b_scale", c_void_p), ("q_out", c_void_p), ("kv_a", c_void_p), ("gamma_ckv", c_void_p), ("kv_out", c_void_p),
        ("cos", c_void_p), ("sin", c_void_p), ("t", c_i32), ("heads", c_i32), ("q_b_ld", c_i32), ("quant", c_i32),
        ("eps", c_float),
    ]


class CompressorArgs(C.Structure):
    _fields_ = [
        ("kv_total", c_void_p), ("score_total", c_void_p), ("ape", c_void_p), ("weight", c_void_p),
        ("kv_state", c_void_p), ("score_state", c_void_p), ("kv_block_table", c_void_p),
        ("score_block_table", c_void_p), ("sin", c_void_p), ("cos", c_void_p), ("start_pos", c_void_p),
        ("out", c_void_p), ("status", c_void_p), ("kv_blocks", c_i64), ("score_blocks", c_i64), ("b", c_i32),
        ("s1", c_i32), ("d", c_i32), ("ratio", c_i32), ("kv_cols", c_i32), ("score_cols", c_i32), ("eps", c_float),
    ]


class HcPreArgs(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("hc_fn", c_void_p), ("hc_scale", c_void_p), ("hc_base", c_void_p), ("y", c_void_p),
        ("post", c_void_p), ("comb", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("t", c_i32),
        ("hc_mult", c_i32), ("d", c_i32), ("iters", c_i32),
        ("norm_eps", c_float), ("hc_eps", c_float),
    ]


class PrologV4Args(C.Structure):
    _fields_ = [
        ("qr", c_void_p), ("idx_wq_b", c_void_p), ("x", c_void_p), ("weights_proj", c_void_p), ("cos", c_void_p),
        ("sin", c_void_p), ("hadamard", c_void_p), ("qr_scale", c_void_p), ("idx_wq_b_scale", c_void_p),
        ("q", c_void_p), ("weights", c_void_p), ("q_scale", c_void_p), ("workspace", c_void_p),
        ("workspace_bytes", c_size_t), ("status", c_void_p), ("t", c_i32), ("h", c_i32),
    ]


class PgPrologArgs(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("q_norm", c_void_p), ("q_norm_scale", c_void_p), ("w_qb", c_void_p), ("w_qb_scale", c_void_p),
        ("wk", c_void_p), ("w_proj", c_void_p), ("gamma_k", c_void_p), ("cos_idx_rope", c_void_p),
        ("sin_idx_rope", c_void_p), ("hadamard_q", c_void_p), ("hadamard_k", c_void_p), ("k_cache_index", c_void_p),
        ("k_scale_cache_index", c_void_p), ("q_quant", c_void_p), ("q_scale", c_void_p), ("k_cache", c_void_p),
        ("k_scale_cache", c_void_p), ("weights", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("status", c_void_p), ("cache_rows", c_i64), ("k_block_stride", c_i64), ("k_scale_block_stride", c_i64),
        ("t", c_i32), ("h", c_i32), ("q_lora", c_i32), ("heads", c_i32), ("block_size", c_i32), ("format", c_i32),
        ("eps", C.c_float),
    ]


class GemmBf16Args(C.Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("c", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("status", c_void_p), ("t", c_i32), ("k", c_i32), ("n", c_i32), ("b_layout", c_i32), ("c_dtype", c_i32),
    ]


class GemmI8Args(C.Structure):
    _fields_ = [("a", c_void_p), ("b", c_void_p), ("c", c_void_p), ("status", c_void_p), ("t", c_i32), ("k", c_i32),
                ("n", c_i32)]


class TopkScatter(C.Structure):
    _fields_ = [("world", c_i32), ("rank", c_i32), ("tokens_per_rank", c_i32), ("reserved", c_i32),
                ("idx_ptrs", c_void_p * 8), ("score_ptrs", c_void_p * 8)]


class IndexerArgs(C.Structure):
    _fields_ = [
        ("idx_query", c_void_p), ("idx_query_scale", c_void_p), ("idx_key_cache", c_void_p),
        ("idx_key_scale", c_void_p), ("idx_weight", c_void_p), ("act_seq_key", c_void_p), ("block_table", c_void_p),
        ("topk_res", c_void_p), ("topk_scores", c_void_p), ("scores_out", c_void_p), ("dots_out", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("status", c_void_p), ("num_blocks", c_i64),
        ("b", c_i32), ("s1", c_i32), ("block_size", c_i32), ("max_blocks", c_i32), ("selected_count", c_i32),
        ("score_ld", c_i32), ("key_begin", c_i32), ("key_end", c_i32),
    ]


class TopkArgs(C.Structure):
    _fields_ = [
        ("scores", c_void_p), ("ids", c_void_p), ("counts", c_void_p), ("out_idx", c_void_p), ("out_scores", c_void_p),
        ("rows", c_i32), ("ld", c_i32), ("k", c_i32), ("id_base", c_i32),
    ]


class PrologArgs(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("q_norm", c_void_p), ("q_norm_scale", c_void_p), ("w_qb", c_void_p), ("w_qb_scale", c_void_p),
        ("wk", c_void_p), ("w_proj", c_void_p), ("ln_gamma_k", c_void_p), ("ln_beta_k", c_void_p),
        ("cos_idx_rope", c_void_p), ("sin_idx_rope", c_void_p), ("hadamard_q", c_void_p), ("hadamard_k", c_void_p),
        ("k_cache_index", c_void_p), ("q_int8", c_void_p), ("q_scale", c_void_p), ("k_cache", c_void_p),
        ("k_scale_cache", c_void_p), ("weights", c_void_p), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("status", c_void_p), ("cache_rows", c_i64), ("t", c_i32), ("ln_eps", c_float),
    ]


class MlaPrologArgs(C.Structure):
    _fields_ = [
        ("x", c_void_p), ("w_dq", c_void_p), ("w_uq_qr", c_void_p), ("w_qb_scale", c_void_p), ("w_uk", c_void_p),
        ("w_dkv_kr", c_void_p), ("gamma_cq", c_void_p), ("gamma_ckv", c_void_p), ("cos", c_void_p), ("sin", c_void_p),
        ("cache_index", c_void_p), ("kv_cache", c_void_p), ("kr_cache", c_void_p), ("k_scale_cache", c_void_p),
        ("q_norm", c_void_p), ("q_norm_scale", c_void_p), ("query_nope", c_void_p), ("query_rope", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("status", c_void_p), ("cache_rows", c_i64),
        ("t", c_i32), ("eps_cq", c_float), ("eps_ckv", c_float),
    ]


class AdvanceArgs(C.Structure):
    _fields_ = [("act_seq", c_void_p), ("block_table", c_void_p), ("cache_index", c_void_p), ("status", c_void_p),
                ("b", c_i32), ("s1", c_i32), ("grow", c_i32), ("block_size", c_i32), ("max_blocks", c_i32)]


class FusedPrologArgs(C.Structure):
    _fields_ = [("mla", MlaPrologArgs), ("indexer", PrologArgs)]


# every symbol include/dsv32_b200.h declares: name -> (restype, argtypes)
EXPORTS = {
    "dsv32_abi_version": (c_i32, []),
    "dsv32_last_error": (C.c_char_p, []),
    "dsv32_launch_count": (C.c_uint64, []),
    "dsv32_sfa_workspace_bytes": (c_size_t, [c_i32, c_i32, c_i32, c_i32, c_i32]),
    "dsv32_sfa_quant": (c_i32, [C.POINTER(SfaArgs), c_void_p]),
    "dsv32_sfa_bf16_cache": (c_i32, [C.POINTER(SfaArgs), c_void_p]),
    "dsv32_sparse_attention_antiquant": (c_i32, [C.POINTER(SaAntiquantArgs), c_void_p]),
    "dsv32_sparse_compress_attention": (c_i32, [C.POINTER(ScfaArgs), c_void_p]),
    "dsv32_scfa_workspace_bytes": (c_size_t, [c_i32, c_i32, c_i32]),
    "dsv32_indexer_workspace_bytes": (c_size_t, [c_i32, c_i32, c_i32, c_i32]),
    "dsv32_indexer_topk": (c_i32, [C.POINTER(IndexerArgs), c_void_p]),
    "dsv32_indexer_topk_noalloc": (c_i32, [C.POINTER(IndexerArgs), c_void_p]),
    "dsv32_indexer_topk_scatter": (c_i32, [C.POINTER(IndexerArgs), C.POINTER(TopkScatter), c_void_p]),
    "dsv32_topk_select": (c_i32, [C.POINTER(TopkArgs), c_void_p]),
    "dsv32_indexer_prolog_v4": (c_i32, [C.POINTER(PrologV4Args), c_void_p]),
    "dsv32_prolog_v4_workspace_bytes": (c_size_t, [c_i32, c_i32]),
    "dsv32_mla_prolog_v4_stage": (c_i32, [C.POINTER(MlaV4StageArgs), c_i32, c_void_p]),
    "dsv32_compressor_update": (c_i32, [C.POINTER(CompressorArgs), c_void_p]),
    "dsv32_hc_pre": (c_i32, [C.POINTER(HcPreArgs), c_void_p]),
    "dsv32_hc_pre_workspace_bytes": (c_size_t, [c_i32]),
    "dsv32_prolog_workspace_bytes": (c_size_t, [c_i32]),
    "dsv32_indexer_prolog": (c_i32, [C.POINTER(PrologArgs), c_void_p]),
    "dsv32_mla_prolog": (c_i32, [C.POINTER(MlaPrologArgs), c_void_p]),
    "dsv32_mla_prolog_workspace_bytes": (c_size_t, [c_i32]),
    "dsv32_mla_indexer_prolog": (c_i32, [C.POINTER(FusedPrologArgs), c_void_p]),
    "dsv32_decode_advance": (c_i32, [C.POINTER(AdvanceArgs), c_void_p]),
    "dsv32_wait_selftest": (c_i32, [c_void_p, c_i64, c_void_p]),
    "dsv32_pg_indexer_prolog": (c_i32, [C.POINTER(PgPrologArgs), c_void_p]),
    "dsv32_pg_indexer_prolog_workspace_bytes": (c_size_t, [c_i32, c_i32, c_i32, c_i32]),
    "dsv32_hif8_convert": (c_i32, [c_i32, c_void_p, c_void_p, c_i64, c_void_p]),
    "dsv32_gemm_bf16": (c_i32, [C.POINTER(GemmBf16Args), c_void_p]),
    "dsv32_gemm_bf16_workspace_bytes": (c_size_t, [c_i32, c_i32, c_i32]),
    "dsv32_gemm_i8": (c_i32, [C.POINTER(GemmI8Args), c_void_p]),
}

ABI_VERSION = 2
_lib = None


class Dsv32Error(RuntimeError):
    """A call into libdsv32_b200.so was rejected (host-side validation or CUDA launch error)."""


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise Dsv32Error(
            f"{LIB_PATH} not found: build it with `python -m pypto_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    if lib.dsv32_abi_version() != ABI_VERSION:
        raise Dsv32Error(f"ABI mismatch: library {lib.dsv32_abi_version()}, binding {ABI_VERSION}")
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != 0:
        msg = load().dsv32_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        raise Dsv32Error(f"{what} failed (code {rc}): {msg}")


def launch_count() -> int:
    return int(load().dsv32_launch_count())
