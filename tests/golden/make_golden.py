#!/usr/bin/env python3
"""Generate the golden fixtures in this directory from the UNMODIFIED reference goldens.

Run where the reference checkout is available, with its root as the argument (or in
$DSV32_REFERENCE_ROOT):

    python tests/golden/make_golden.py <reference root>

The reference's torch-CPU golden functions live in its operator test files.  Those
files import `pypto` and `torch_npu` at module level; both are replaced here by
permissive stand-in modules (every attribute access, call, subscript and decorator
use succeeds), which is enough to import the files and call the pure-torch goldens.

Outputs (small .npz files; bf16/fp16 tensors stored as int16 bit patterns):
  sfa_small.npz      inputs + output of compute_attention_no_flash
  indexer_small.npz  inputs + topk_res of lightning_indexer_compute (+ oracle scores)
  prolog_small.npz   seed + input digests + outputs of indexer_prolog
  mla_small.npz      seed + input digests + outputs of mla_prolog_quant_v32_compute
  sfa_bf16_small.npz inputs + output of compute_attention_no_flash with a bf16 (not quantised) cache
  sa_antiquant_small.npz  inputs + output of compute_attention_aq (fused 656-byte cache rows)
  scfa_small.npz     inputs + output of the DeepSeek-V4 sparse compress attention golden
                     (models/deepseek_v4/test_sparse_compress_flash_attention.py: window keys + selected
                     compressed keys + attention sinks)
  cfa_small.npz      a query + the output of the DeepSeek-V4 compress flash attention golden (ifa_golden,
                     models/deepseek_v4/test_compress_flash_attention.py) on the caches of scfa_small.npz
  win_small.npz      the output of the DeepSeek-V4 sliding-window attention golden (win_atten_calc_tnd,
                     models/deepseek_v4/test_win_attention.py) on the inputs of scfa_small.npz
  prolog_v4_small.npz  token count + input digests + outputs of the DeepSeek-V4 indexer prolog golden
                     (compute_quant_lightning_indexer_prolog, models/deepseek_v4/test_lightning_indexer_prolog_quant_v4.py)
  mla_v4_small.npz   token count + input digests + outputs of the DeepSeek-V4 MLA prolog golden
                     (mla_prolog_compute, models/deepseek_v4/test_mla_prolog_quant_v4.py)
  mla_v4_bf16_small.npz  outputs of the DeepSeek-V4 MLA prolog golden without quantisation (mla_prolog_compute,
                     models/deepseek_v4/test_mla_prolog_v4.py) on the un-quantised inputs of mla_v4_small.npz
  hc_pre_small.npz   token count + input digests + outputs of the DeepSeek-V4 hyper-connection pre-mix golden
                     (gen_hc_pre, models/deepseek_v4/test_hc_pre.py)
  compressor_small.npz  outputs and touched state rows of the DeepSeek-V4 compressor golden (golden_compress,
                     models/deepseek_v4/test_compressor.py) for three cases: ratio 128, ratio 4, ratio 4 + hadamard
  pg_prolog_mxfp8_small.npz  seed + input digests + outputs of the page-grouped MXFP8 indexer prolog golden
                     (indexer_prolog, python/tests/st/operator/pg/test_pg_lightning_indexer_prolog_quant_mxfp8.py)
  kat.json           the two interpreter known-answer tests, restated as data

Nothing at test time reads the reference: the tests only read these files.
"""
import hashlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DSV32_REFERENCE_ROOT", "")
MODEL_DIR = os.path.join(REF, "models", "deepseek_v32_exp")


class _Anything:
    """Stand-in object: any attribute, call, item or decorator use succeeds."""

    def __init__(self, name="stub"):
        self.__dict__["_name"] = name

    def __getattr__(self, item):
        if item.startswith("__") and item.endswith("__"):
            raise AttributeError(item)
        return _Anything(f"{self._name}.{item}")

    def __call__(self, *args, **kwargs):
        if len(args) == 1 and not kwargs and callable(args[0]) and not isinstance(args[0], _Anything):
            return args[0]  # used as a bare decorator
        return _Anything(f"{self._name}()")

    def __getitem__(self, item):
        return _Anything(f"{self._name}[]")

    def __iter__(self):
        return iter(())

    def __eq__(self, other):
        return False

    def __hash__(self):
        return id(self)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


class _StubModule(types.ModuleType):
    def __getattr__(self, item):
        if item.startswith("__") and item.endswith("__"):
            raise AttributeError(item)
        return _Anything(f"{self.__name__}.{item}")


def install_reference_stubs():
    for name in ("torch_npu", "pypto", "pypto.experimental", "pypto.operation", "pypto.pypto_impl",
                 "pypto.frontend", "pypto.platform"):
        mod = _StubModule(name)
        mod.__path__ = []
        sys.modules[name] = mod
    if MODEL_DIR not in sys.path:
        sys.path.insert(0, MODEL_DIR)


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy()


def digest(t: torch.Tensor) -> str:
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        raw = t.view(torch.int16).numpy().tobytes()
    else:
        raw = t.numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()


def make_sfa():
    import deepseekv32_sparse_flash_attention_quant as ref  # noqa: reference module
    b, nq, nkv, s1 = 3, 128, 1, 2
    act_seq = [2600, 700, 15]
    input_params, data, atten_out = ref.gen_gather_select_attention_golden(torch.bfloat16, (b, nq, nkv, s1), 1, act_seq)
    q_nope, q_rope, kn, kr, kn_scales, topk_indices, block_table, _ = data
    np.savez_compressed(
        os.path.join(HERE, "sfa_small.npz"),
        b=b, s1=s1, nq=nq, softmax_scale=np.float64(input_params[-1]), act_seq=np.array(act_seq, dtype=np.int32),
        q_nope=bits16(q_nope), q_rope=bits16(q_rope), k_nope=kn.numpy(), k_rope=bits16(kr),
        k_scales=kn_scales.numpy(), topk_indices=topk_indices.numpy(), block_table=block_table.numpy(),
        out=bits16(atten_out))
    print("sfa_small: out", tuple(atten_out.shape))


def make_sfa_bf16():
    import deepseekv32_sparse_flash_attention_quant as ref  # noqa: reference module
    torch.manual_seed(31)
    b, nq, nkv, s1 = 2, 128, 1, 2
    act_seq = [2200, 130]
    input_params, data, atten_out = ref.gen_gather_select_attention_golden(torch.bfloat16, (b, nq, nkv, s1), 0, act_seq)
    q_nope, q_rope, kn, kr, _, topk_indices, block_table, _ = data
    assert kn.dtype == torch.bfloat16
    np.savez_compressed(
        os.path.join(HERE, "sfa_bf16_small.npz"),
        b=b, s1=s1, nq=nq, softmax_scale=np.float64(input_params[-1]), act_seq=np.array(act_seq, dtype=np.int32),
        q_nope=bits16(q_nope), q_rope=bits16(q_rope), k_nope=bits16(kn), k_rope=bits16(kr),
        topk_indices=topk_indices.numpy(), block_table=block_table.numpy(), out=bits16(atten_out))
    print("sfa_bf16_small: out", tuple(atten_out.shape))


def make_sa_antiquant():
    import deepseekv32_sparse_attention_antiquant as ref  # noqa: reference module
    torch.manual_seed(21)
    b, nq, nkv, s1 = 3, 128, 1, 2
    act_seq = [2300, 900, 40]
    input_params, data, atten_out = ref.gen_gather_select_attention_golden_aq(torch.bfloat16, (b, nq, nkv, s1), 1, act_seq)
    q_nope, q_rope, nope_cache_2d, topk_indices, block_table, _ = data
    np.savez_compressed(
        os.path.join(HERE, "sa_antiquant_small.npz"),
        b=b, s1=s1, nq=nq, softmax_scale=np.float64(input_params[-1]), act_seq=np.array(act_seq, dtype=np.int32),
        q_nope=bits16(q_nope), q_rope=bits16(q_rope), nope_cache=nope_cache_2d.numpy(),
        topk_indices=topk_indices.numpy(), block_table=block_table.numpy(), out=bits16(atten_out))
    print("sa_antiquant_small: out", tuple(atten_out.shape))


def make_indexer():
    import deepseekv32_lightning_indexer_quant as ref  # noqa: reference module
    torch.manual_seed(11)
    np.random.seed(11)
    b, s1, n1, d, bs = 3, 2, 64, 128, 128
    act_seq = [3000, 971, 2049]
    s2 = max(act_seq)
    block_num = sum((s + bs - 1) // bs for s in act_seq)
    params = dict(b=b, s1=s1, n1=n1, n2=1, d=d, dtype=torch.float16, s2=s2, act_seq=act_seq, block_size=bs,
                  block_num=block_num, max_block_num=(s2 + bs - 1) // bs, selected_count=2048)
    m = ref.gen_data_for_compute(params, is_quant=True)
    # The stock generator draws randn->int8 (mostly 0/+-1), which makes thousands of exact
    # score ties.  Replace values (not shapes/layout) by full-range data so the top-k is well defined.
    g = torch.Generator().manual_seed(12)
    m["query"] = torch.randint(-127, 128, m["query"].shape, generator=g, dtype=torch.int8)
    m["key"] = torch.randint(-127, 128, m["key"].shape, generator=g, dtype=torch.int8)
    m["q_scale"] = (torch.rand(m["q_scale"].shape, generator=g) * 0.019 + 0.001).to(torch.float16)
    m["k_scale"] = (torch.rand(m["k_scale"].shape, generator=g) * 0.019 + 0.001).to(torch.float16)
    topk_res = ref.lightning_indexer_compute(m, params)
    np.savez_compressed(
        os.path.join(HERE, "indexer_small.npz"),
        b=b, s1=s1, act_seq=np.array(act_seq, dtype=np.int32),
        query=m["query"].reshape(b * s1, n1, d).numpy(), q_scale=bits16(m["q_scale"].reshape(b * s1, n1)),
        key=m["key"].numpy(), k_scale=bits16(m["k_scale"].reshape(block_num, bs, 1)),
        weights=bits16(m["weights"].reshape(b * s1, n1)), block_table=m["block_table"].numpy(),
        topk_res=topk_res.numpy())
    print("indexer_small: topk_res", tuple(topk_res.shape))


def prolog_inputs(seed, b, s1, s2):
    """Restates the call order of the reference generator
    (deepseekv32_lightning_indexer_prolog_quant.py:105-158) so that the same seed gives the
    same tensors without the reference being present."""
    import deepseekv32_lightning_indexer_prolog_quant as ref  # noqa: reference module
    torch.manual_seed(seed)
    dims = ref.gen_dims({"b": b, "s1": s1, "s2": s2})
    inputs = ref.gen_inputs(dims, torch.bfloat16)
    return ref, dims, inputs


def make_prolog():
    seed, b, s1, s2 = 7, 2, 2, 512
    ref, dims, inputs = prolog_inputs(seed, b, s1, s2)
    out = ref.indexer_prolog(inputs, dims)
    t = b * s1
    digests = {k: digest(v) for k, v in inputs.items() if isinstance(v, torch.Tensor)}
    np.savez_compressed(
        os.path.join(HERE, "prolog_small.npz"),
        seed=seed, b=b, s1=s1, s2=s2, digests=json.dumps(digests),
        q_int8=out["query"].reshape(t, 64, 128).numpy(), q_scale=bits16(out["query_scale"].reshape(t, 64, 1)),
        k_cache=out["idx_k_cache_out"].numpy(), k_scale_cache=bits16(out["idx_k_scale_cache_out"]),
        weights=bits16(out["weights"].reshape(t, 64)))
    print("prolog_small: q_int8", tuple(out["query"].shape))


def make_mla():
    import deepseekv32_mla_indexer_prolog_quant as ref  # noqa: reference module
    seed, b, s1, s2 = 6, 2, 2, 256
    torch.manual_seed(seed)
    params = dict(n1=128, n2=1, h=7168, num_heads=128, idx_n_heads=64, q_lora_rank=1536, qk_nope_head_dim=128,
                  idx_head_dim=128, qk_rope_head_dim=64, rope_head_dim=64, kv_lora_rank=512, block_size=128,
                  dtype=torch.bfloat16, b=b, s=s1, t=b * s1, s1=s1, s2=s2,
                  actual_seq=torch.tensor([s2] * b, dtype=torch.int32).unsqueeze(-1))
    (x, w_dq, w_uqqr, _, scale_data, w_dkvkr, w_uk, gamma_cq, gamma_ckv, cos, sin, cache_index, kv_cache, kr_cache,
     ks_cache, _, _) = ref.gen_mla_prolog_quant_v32_inputs(params, (torch.bfloat16, torch.bfloat16),
                                                          params["actual_seq"], (False, True), False, False, 128,
                                                          "PA_BSND")
    inputs = dict(dtype=torch.bfloat16, is_quant_a=False, is_quant_b=True, has_smooth=False, cache_mode="PA_BSND",
                  gamma_cq=gamma_cq, gamma_ckv=gamma_ckv, x=x, w_dq=w_dq, w_uqqr=w_uqqr, w_uk=w_uk, w_dkvkr=w_dkvkr,
                  cos=cos, sin=sin, kv_cache=kv_cache, kr_cache=kr_cache, kv_quant_scale_cache=ks_cache,
                  cache_index=cache_index, w_qb_scale=scale_data["w_uqqr"])
    q_nope, q_rope, q_norm, q_norm_scale, kv_out, kr_out, ks_out = ref.mla_prolog_quant_v32_compute(inputs)
    t = b * s1
    named = dict(x=x, w_dq=w_dq, w_uqqr=w_uqqr, w_qb_scale=scale_data["w_uqqr"], w_uk=w_uk, w_dkvkr=w_dkvkr,
                 gamma_cq=gamma_cq, gamma_ckv=gamma_ckv, cos=cos, sin=sin, cache_index=cache_index, kv_cache=kv_cache,
                 kr_cache=kr_cache, ks_cache=ks_cache)
    digests = {k: digest(v) for k, v in named.items()}
    np.savez_compressed(
        os.path.join(HERE, "mla_small.npz"), seed=seed, b=b, s1=s1, s2=s2, digests=json.dumps(digests),
        q_nope=bits16(q_nope.reshape(t, 128, 512)), q_rope=bits16(q_rope.reshape(t, 128, 64)),
        q_norm=q_norm.reshape(t, 1536).numpy(), q_norm_scale=q_norm_scale.reshape(t, 1).numpy(),
        kv_cache=kv_out.numpy(), kr_cache=bits16(kr_out), ks_cache=ks_out.numpy())
    print("mla_small: q_nope", tuple(q_nope.shape))


def make_scfa():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        import test_sparse_compress_flash_attention as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    b, nq, nkv, cmp_ratio = 3, 64, 1, 4
    actual_seq_q = [0, 2, 3, 5]
    ori_seq = [2100, 130, 700]   # compressed lengths 525 (> top-k 512: random selection), 32, 175
    input_params, data, atten_out = ref.gen_sparse_compress_attention_golden(
        torch.bfloat16, (b, nq, nkv, 2), actual_seq_q, ori_seq, cmp_ratio)
    q, cmp_kv, ori_kv, topk_indices, cmp_bt, ori_bt, seq_q, seq_kv, sink = data
    block_size, win_size, topk, scalar = input_params[7], input_params[8], input_params[9], input_params[10]
    np.savez_compressed(
        os.path.join(HERE, "scfa_small.npz"),
        b=b, nq=nq, cmp_ratio=cmp_ratio, block_size=block_size, win_size=win_size, topk=topk,
        softmax_scale=np.float64(scalar), actual_seq_q=np.array(seq_q, dtype=np.int32),
        seqused_kv=seq_kv.numpy(), q=bits16(q), cmp_kv=bits16(cmp_kv), ori_kv=bits16(ori_kv),
        cmp_sparse_indices=topk_indices.numpy(), cmp_block_table=cmp_bt.numpy(), ori_block_table=ori_bt.numpy(),
        atten_sink=sink.numpy(), out=bits16(atten_out))
    print("scfa_small: out", tuple(atten_out.shape))


def _load_scfa_inputs():
    z = np.load(os.path.join(HERE, "scfa_small.npz"))
    bf = lambda a: torch.from_numpy(a).view(torch.bfloat16)  # noqa: E731
    return z, bf


def make_cfa():
    """compress flash attention: window + every compressed row.  Reuses the caches, page tables and sequence
    lengths of scfa_small.npz (cmp_ratio 4) with a fresh query of two tokens per request."""
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        import test_compress_flash_attention as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    z, bf = _load_scfa_inputs()
    b, nq, s1, cmp_ratio = int(z["b"]), int(z["nq"]), 2, int(z["cmp_ratio"])
    torch.manual_seed(4242)
    q = torch.empty((b * s1, nq, 512), dtype=torch.bfloat16).uniform_(-1, 1)
    cmp_kv = bf(z["cmp_kv"]).reshape(-1, 128, 1, 512)
    ori_kv = bf(z["ori_kv"]).reshape(-1, 128, 1, 512)
    out = torch.zeros_like(q)
    ref.ifa_golden(q, cmp_kv, torch.from_numpy(z["atten_sink"]), torch.from_numpy(z["cmp_block_table"]),
                   torch.from_numpy(z["seqused_kv"]), out, None, enable_flash=False, cmp_ratio=cmp_ratio,
                   is_new_sink=True, ori_kv=ori_kv, ori_block_table=torch.from_numpy(z["ori_block_table"]))
    np.savez_compressed(os.path.join(HERE, "cfa_small.npz"), s1=s1, q=bits16(q), out=bits16(out))
    print("cfa_small: out", tuple(out.shape))


class _NpuDeviceAsCpu:
    """The window-attention golden allocates its result with device='npu:<id>'; while it runs, torch.zeros places
    such tensors on the CPU instead.  The golden itself is not modified."""

    def __enter__(self):
        self._zeros = torch.zeros

        def zeros(*args, **kwargs):
            if str(kwargs.get("device", "")).startswith("npu"):
                kwargs["device"] = "cpu"
            return self._zeros(*args, **kwargs)

        torch.zeros = zeros
        return self

    def __exit__(self, *exc):
        torch.zeros = self._zeros
        return False


def make_win():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        import test_win_attention as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    z, bf = _load_scfa_inputs()
    nq, win = int(z["nq"]), int(z["win_size"])
    seq_q = [int(x) for x in z["actual_seq_q"]]
    t = seq_q[-1]
    q = bf(z["q"]).reshape(t, nq, 512)
    kv_cache = bf(z["ori_kv"]).reshape(-1, 128, 1, 512)
    params = [t, 1, nq, 512, win, 512 ** -0.5]
    with _NpuDeviceAsCpu():
        out = ref.win_atten_calc_tnd(params, [int(x) for x in z["seqused_kv"]], torch.from_numpy(z["atten_sink"]), q,
                                     kv_cache, torch.from_numpy(z["ori_block_table"]), seq_q, 0)
    np.savez_compressed(os.path.join(HERE, "win_small.npz"), out=bits16(out))
    print("win_small: out", tuple(out.shape))


class _TolerateNpuDispatchKey:
    """Some reference operator files register a torch.library implementation for the dispatch key "NPU" at import
    time without guarding it; this torch build has no such key.  While such a file is imported, a registration
    for that key is skipped (the decorated function is returned as it is); nothing else changes."""

    def __enter__(self):
        self._impl = torch.library.impl

        def impl(lib, name, dispatch_key=""):
            if dispatch_key == "NPU":
                return lambda fn: fn
            return self._impl(lib, name, dispatch_key)

        torch.library.impl = impl
        return self

    def __exit__(self, *exc):
        torch.library.impl = self._impl
        return False


def make_prolog_v4():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        with _TolerateNpuDispatchKey():
            import test_lightning_indexer_prolog_quant_v4 as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    t = 37
    params = {"t": t, "idx_nq": 64, "head_dim": 128, "rope_dim": 64, "q_lora_rank": 1024, "h": 4096}
    inputs, q, weights, q_scale = ref.gen_quant_attention_post_golden(params)   # seeds torch with 42 itself
    names = ["qr", "idx_wq_b", "x", "weights_proj", "cos", "sin", "hadamard", "qr_scale", "idx_wq_b_scale"]
    digests = {n: digest(v) for n, v in zip(names, inputs)}
    np.savez_compressed(os.path.join(HERE, "prolog_v4_small.npz"), t=t, digests=json.dumps(digests),
                        q=q.reshape(t, 64, 128).numpy(), weights=bits16(weights), q_scale=bits16(q_scale))
    print("prolog_v4_small: q", tuple(q.shape))


def make_mla_v4():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        with _TolerateNpuDispatchKey():
            import test_mla_prolog_quant_v4 as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    t = 5
    params = {"t": t, "num_heads": 64, "h": 4096, "q_lora_rank": 1024, "head_dim": 512, "qk_rope_head_dim": 64}
    torch.manual_seed(5)   # the reference module seeds with 5 when it is imported; repeated here for a fixed start
    inputs, outputs = ref.gen_mla_prolog_data(params, torch.bfloat16, True, False)
    names = ["x", "wq_a", "wq_b", "w_kv", "cos", "sin", "gamma_cq", "gamma_ckv", "wq_b_scale"]
    digests = {n: digest(inputs[n]) for n in names}
    np.savez_compressed(os.path.join(HERE, "mla_v4_small.npz"), t=t, digests=json.dumps(digests),
                        q=bits16(outputs["q_golden"]), kv=bits16(outputs["kv_golden"]),
                        qr=outputs["qr_golden"].numpy(), qr_scale=outputs["qr_scale_golden"].numpy())
    print("mla_v4_small: q", tuple(outputs["q_golden"].shape))


def make_mla_v4_bf16():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        with _TolerateNpuDispatchKey():
            import test_mla_prolog_v4 as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    t = 5
    params = {"t": t, "num_heads": 64, "h": 4096, "q_lora_rank": 1024, "head_dim": 512, "qk_rope_head_dim": 64}
    torch.manual_seed(5)   # as the reference module does when it is imported
    x, wq_a, wq_b, w_kv, gamma_cq, gamma_ckv, cos, sin = ref.gen_mla_prolog_input_data(params, torch.bfloat16)
    inputs = {"x": x, "wq_a": wq_a, "wq_b": wq_b, "w_kv": w_kv, "cos": cos, "sin": sin, "gamma_cq": gamma_cq,
              "gamma_ckv": gamma_ckv}
    q, kv, qr = ref.mla_prolog_compute(inputs)
    digests = {n: digest(v) for n, v in inputs.items()}
    np.savez_compressed(os.path.join(HERE, "mla_v4_bf16_small.npz"), t=t, digests=json.dumps(digests), q=bits16(q),
                        kv=bits16(kv), qr=bits16(qr))
    print("mla_v4_bf16_small: q", tuple(q.shape))


def make_hc_pre():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        with _TolerateNpuDispatchKey():
            import test_hc_pre as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    t = 16
    x, hc_fn, hc_scale, hc_base, y, post, comb, _ = ref.gen_hc_pre_data(t)    # seeds torch with 42 itself
    digests = {"x": digest(x), "hc_fn": digest(hc_fn), "hc_scale": digest(hc_scale), "hc_base": digest(hc_base)}
    np.savez_compressed(os.path.join(HERE, "hc_pre_small.npz"), t=t, digests=json.dumps(digests), y=bits16(y),
                        post=post.numpy(), comb=comb.numpy())
    print("hc_pre_small: y", tuple(y.shape))


COMPRESSOR_CASES = {   # name: (ratio, rotate, d, batch, tokens per request, start positions)
    "r128": (128, False, 512, 3, 2, [254, 126, 300]),
    "r4": (4, False, 512, 4, 2, [255, 2, 6, 9]),
    "r4_rot": (4, True, 128, 4, 2, [255, 3, 10, 1]),
}


def make_compressor():
    v4_dir = os.path.join(REF, "models", "deepseek_v4")
    sys.path.insert(0, v4_dir)
    try:
        with _TolerateNpuDispatchKey():
            import test_compressor as ref  # noqa: reference module
    finally:
        sys.path.remove(v4_dir)
    saved = {}
    for name, (ratio, rotate, d, bsz, seq, starts) in COMPRESSOR_CASES.items():
        x, sin, cos, wkv, wgate, ape, weight, kv_state, score_state, table, hadamard = ref.gen_inputs(
            bsz, seq, 4096, d, 64, ratio, "cpu")          # seeds torch with 42 itself
        # the generator leaves the states zero; give them history so that the rows of earlier positions matter
        g = torch.Generator().manual_seed(7)
        kv_state.copy_(torch.rand(kv_state.shape, generator=g))
        score_state.copy_(torch.rand(score_state.shape, generator=g))
        st = torch.tensor(starts, dtype=torch.int32)
        digests = {n: digest(v) for n, v in (("x", x), ("sin", sin), ("cos", cos), ("wkv", wkv), ("wgate", wgate),
                                             ("ape", ape), ("hadamard", hadamard), ("kv_state", kv_state),
                                             ("score_state", score_state), ("table", table))}
        out = ref.golden_compress(x, sin, cos, wkv, wgate, ape, weight, kv_state, score_state, table, table, hadamard,
                                  ratio, st, 64, rotate)
        saved[name + "_digests"] = json.dumps(digests)
        saved[name + "_out"] = bits16(out)
        saved[name + "_kv_state_sum"] = kv_state.double().sum(-1).numpy()       # [blocks, 128] row checksums
        saved[name + "_score_state_sum"] = score_state.double().sum(-1).numpy()
        print("compressor", name, "out", tuple(out.shape))
    np.savez_compressed(os.path.join(HERE, "compressor_small.npz"), **saved)


def make_pg_prolog_mxfp8():
    pg_dir = os.path.join(REF, "python", "tests", "st", "operator", "pg")
    sys.path.insert(0, pg_dir)
    had_npu = hasattr(torch.Tensor, "npu")
    if not had_npu:
        torch.Tensor.npu = lambda self, *a, **k: self   # the generator parks two tensors on the device
    try:
        with _TolerateNpuDispatchKey():
            import test_pg_lightning_indexer_prolog_quant_mxfp8 as ref  # noqa: reference module
        seed, b, s1, s2 = 11, 2, 2, 256
        torch.manual_seed(seed)
        dims = ref.gen_dims({"b": b, "s1": s1, "s2": s2})
        inputs = ref.gen_inputs(dims, torch.bfloat16)
        out = ref.indexer_prolog(inputs, dims, "cpu")
    finally:
        sys.path.remove(pg_dir)
        if not had_npu:
            del torch.Tensor.npu
    t = b * s1

    def raw(v):
        v = v.contiguous()
        if v.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
            return v.view(torch.uint8)
        if v.dtype in (torch.bfloat16, torch.float16):
            return v.view(torch.int16)
        return v

    digests = {k: hashlib.sha256(raw(v).numpy().tobytes()).hexdigest() for k, v in inputs.items()}
    index = inputs["idx_k_cache_index"].reshape(-1)
    k_rows = out["idx_k_cache_out"].reshape(-1, 128)[index]          # fp32 values of the rows the operator wrote
    k_scales = out["idx_k_scale_cache_out"].reshape(-1)[index]
    np.savez_compressed(
        os.path.join(HERE, "pg_prolog_mxfp8_small.npz"),
        seed=seed, b=b, s1=s1, s2=s2, digests=json.dumps(digests),
        q=out["query"].reshape(t, 24, 128).view(torch.uint8).numpy(), q_scale=out["query_scale"].reshape(t, 24, 1).numpy(),
        k=k_rows.to(torch.float8_e4m3fn).view(torch.uint8).numpy(), k_scale=k_scales.numpy(),
        weights=out["weights"].reshape(t, 24).numpy(), cache_index=index.numpy())
    print("pg_prolog_mxfp8_small: q", tuple(out["query"].shape))


def make_kat():
    kat = {
        "topk_ties": {  # test_interp_calc_matmul_sort.cpp:510-524
            "input": [5, 4, 5, 3, 5, 2], "k": 3, "values": [5, 5, 5], "indices": [0, 2, 4]},
        "paged_gather": {  # test_interp_calc_matmul_sort.cpp:830-863
            "rows": 8, "cols": 4, "row_rule": "params[r][c] = 10*r + c", "indices": [0, 2, 5, 3],
            "page_table": [2, 0, 1], "block_size": 2, "expected_rows": [4, 0, 3, 1]},
    }
    with open(os.path.join(HERE, "kat.json"), "w") as f:
        json.dump(kat, f, indent=1)


if __name__ == "__main__":
    if not os.path.isdir(MODEL_DIR):
        sys.exit(f"reference checkout not found at {MODEL_DIR}")
    install_reference_stubs()
    make_kat()
    make_sfa()
    make_sfa_bf16()
    make_sa_antiquant()
    make_indexer()
    make_prolog()
    make_mla()
    make_scfa()
    make_cfa()
    make_win()
    make_prolog_v4()
    make_mla_v4()
    make_mla_v4_bf16()
    make_hc_pre()
    make_compressor()
    make_pg_prolog_mxfp8()
