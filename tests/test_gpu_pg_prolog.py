"""GPU parity of the page-grouped 8-bit-float indexer prologs (MXFP8, HiF8) through the C ABI.

Bars.  The 8-bit codes are compared under the reference's own three-way accuracy rule
(python/tests/st/operator/pg/compare_2_1.py:92-133, restated by oracle.pg_prolog_oracle.triple_compare): the errors
of the CUDA output against the fp32 golden may not exceed 2x (maximum relative error) / 1.2x (mean relative error,
RMSE) those of the bf16-rounding restatement of the operator, nor twice its count of small-value errors (codes and
head weights; a row scale is one bf16-valued maximum, so a single flipped rounding moves it by 0.4 %).  On top of
that the CUDA output is compared with that restatement directly: at least 97 % of the codes identical (the rest
follow from a different fp32 summation order flipping a bf16 rounding), row scales within 1 %.  Cache rows that no
index names stay byte-identical.
"""
import numpy as np
import pytest
import torch

import helpers
from oracle import pg_prolog_oracle as pgo

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ARG_NAMES = ("x", "q_norm", "q_norm_scale", "w_qb", "w_qb_scale", "wk", "w_proj", "gamma_k", "cos", "sin", "hadamard_q",
             "hadamard_k")


def _impl(fmt):
    if fmt == "mxfp8":
        from pypto_b200 import lightning_indexer_prolog_quant_mxfp8_impl as m
    else:
        from pypto_b200 import lightning_indexer_prolog_quant_hif8_impl as m
    return m


def _run(inp, fmt):
    """Runs the operator on the CUDA copies of `inp`; returns (q codes, q scales, pages after, weights)."""
    import pypto_b200
    c = {k: v.to(DEV) for k, v in inp.items() if isinstance(v, torch.Tensor)}
    t = c["x"].shape[0]
    heads = c["w_proj"].shape[1]
    k_cache, k_scale_cache = helpers.pg_cache_views(c["pages"], fmt)
    code_dtype = torch.float8_e4m3fn if fmt == "mxfp8" else torch.uint8
    q = torch.zeros((t * heads, 128), dtype=torch.uint8, device=DEV).view(code_dtype)
    q_scale = torch.zeros((t * heads, 1), dtype=torch.float32, device=DEV)
    weights = torch.zeros((t, heads), dtype=torch.bfloat16, device=DEV)
    _impl(fmt).lightning_indexer_prolog_quant(
        c["x"], c["q_norm"], c["q_norm_scale"], c["w_qb"], c["w_qb_scale"], c["wk"], c["w_proj"], c["gamma_k"], c["cos"],
        c["sin"], c["hadamard_q"], c["hadamard_k"], k_cache, k_scale_cache, c["cache_index"], c["cache_index"], q, q_scale,
        k_cache, k_scale_cache, weights)
    pypto_b200.check_status(DEV)
    return q.view(torch.uint8).cpu(), q_scale.cpu(), c["pages"].cpu(), weights.cpu()


def _oracle_args(inp):
    a = {k: inp[k] for k in ARG_NAMES}
    for k in ("q_norm_scale", "w_qb_scale"):
        if a[k].dtype == torch.float8_e8m0fnu:
            a[k] = a[k].view(torch.uint8)
    return a


def _values(codes_u8, fmt):
    return codes_u8.view(torch.float8_e4m3fn).float() if fmt == "mxfp8" else pgo.hif8_decode(codes_u8)


def _check(inp, fmt, got, golden=None):
    q, q_scale, pages_after, weights = got
    t = inp["x"].shape[0]
    heads = inp["w_proj"].shape[1]
    args = _oracle_args(inp)
    bq, bqs, bk, bks, bw = pgo.pg_prolog(fmt=fmt, **args)
    if golden is None:
        golden = pgo.pg_prolog_golden(fmt=fmt, **args)
    gq, gqs, gk, gks, gw = golden
    as_u8 = lambda v: v.view(torch.uint8) if v.dtype != torch.uint8 else v  # noqa: E731
    # rows the operator wrote, read back through the page-grouped views
    k_cache, k_scale_cache = helpers.pg_cache_views(pages_after, fmt)
    idx = inp["cache_index"].reshape(-1)
    k_rows = k_cache.reshape(-1, 128)[idx].view(torch.uint8) if fmt == "mxfp8" else k_cache.reshape(-1, 128)[idx]
    k_scales = k_scale_cache.reshape(-1)[idx]
    # every other byte of the page-grouped buffer is untouched
    before = inp["pages"].clone()
    kb, ksb = helpers.pg_cache_views(before, fmt)
    pg, slot = idx // helpers.PG_BS, idx % helpers.PG_BS
    kb[pg, slot, 0] = k_cache[pg, slot, 0]
    ksb[pg, slot, 0, 0] = k_scales
    assert torch.equal(before, pages_after), "bytes outside the named cache rows changed"
    checks = (
        ("q", _values(q.reshape(t, heads, 128), fmt), _values(as_u8(bq), fmt), _values(as_u8(gq).reshape(t, heads, 128), fmt), "fp8"),
        ("k", _values(k_rows, fmt), _values(as_u8(bk), fmt), _values(as_u8(gk), fmt), "fp8"),
        ("weights", weights.float(), bw.float(), gw.float(), "bf16"),
    )
    for name, out, bench, gold, kind in checks:
        ok, ratios = pgo.triple_compare(out, bench, gold, kind)
        assert ok, f"{name}: error ratios against the operator restatement {ratios}"
    same_q = float((q.reshape(-1) == as_u8(bq).reshape(-1)).float().mean())
    same_k = float((k_rows.reshape(-1) == as_u8(bk).reshape(-1)).float().mean())
    print(f"[pg prolog {fmt} t={t}] identical codes: q {same_q:.4f} k {same_k:.4f}")
    assert same_q >= 0.97 and same_k >= 0.97, (same_q, same_k)
    assert torch.allclose(q_scale.reshape(-1), bqs.reshape(-1), rtol=1e-2, atol=0)
    assert torch.allclose(k_scales, bks.reshape(-1), rtol=1e-2, atol=0)
    assert torch.allclose(weights.float(), bw.float(), rtol=2 ** -7, atol=1e-6)


def test_pg_prolog_mxfp8_reference_golden_fixture():
    g = helpers.load_pg_prolog_mxfp8_golden()
    ref = helpers.pg_prolog_reference_inputs(g["seed"], g["b"], g["s1"], g["s2"])
    t = g["b"] * g["s1"]
    inp = dict(x=ref["token_x"].reshape(t, -1), q_norm=ref["q_norm"].reshape(t, -1),
               q_norm_scale=ref["q_norm_scale"].reshape(t, -1), w_qb=ref["w_idx_qb"], w_qb_scale=ref["w_idx_qb_scale"],
               wk=ref["w_idx_k"], w_proj=ref["w_idx_proj"], gamma_k=ref["rms_norm_gamma"], cos=ref["cos_idx_rope"].reshape(t, -1),
               sin=ref["sin_idx_rope"].reshape(t, -1), hadamard_q=ref["hadamard_q"], hadamard_k=ref["hadamard_k"],
               pages=ref["pages"], cache_index=ref["idx_k_cache_index"].reshape(t, 1))
    golden = (g["q"], g["q_scale"], g["k"], g["k_scale"], g["weights"])
    _check(inp, "mxfp8", _run(inp, "mxfp8"), golden=golden)


@pytest.mark.parametrize("fmt", ["mxfp8", "hif8"])
@pytest.mark.parametrize("t", [1, 37, 300])
def test_pg_prolog_seeded_vs_oracle(fmt, t):
    inp = helpers.gen_pg_prolog_inputs(100 + t, t, fmt, nblocks=4)
    _check(inp, fmt, _run(inp, fmt))


def test_hif8_conversions_match_the_oracle_everywhere():
    from pypto_b200 import lightning_indexer_prolog_quant_hif8_impl as m
    table = pgo.hif8_decode_table()
    codes = torch.arange(256, dtype=torch.uint8)
    dec = m.hif8_decode(codes.to(DEV)).cpu().numpy()
    assert np.array_equal(np.isnan(dec), np.isnan(table))
    assert np.array_equal(dec[~np.isnan(table)], table[~np.isnan(table)])
    finite = np.sort(np.unique(np.abs(table[np.isfinite(table)]))).astype(np.float64)
    mids = (finite[1:] + finite[:-1]) / 2                                  # every tie point
    g = torch.Generator().manual_seed(3)
    rnd = torch.exp2(torch.rand(200000, generator=g) * 44 - 26) * torch.sign(torch.rand(200000, generator=g) - 0.5)
    pts = np.concatenate([finite, mids, np.nextafter(mids.astype(np.float32), 0), np.nextafter(mids.astype(np.float32), 1e9),
                          [0.0, -0.0, 1e9, -1e9, 40000.0, 2.0 ** -24, 2.0 ** -23, 1.2e-7, float("nan")]]).astype(np.float32)
    x = torch.cat([torch.from_numpy(pts), -torch.from_numpy(pts), rnd])
    got = m.hif8_encode(x.to(DEV)).cpu()
    want = pgo.hif8_encode(x)
    bad = (got != want).nonzero().flatten()
    assert bad.numel() == 0, [(float(x[i]), int(got[i]), int(want[i])) for i in bad[:8]]


def test_pg_prolog_rejects_bad_arguments_and_reports_bad_rows():
    import pypto_b200
    from pypto_b200 import _runtime as rt
    inp = helpers.gen_pg_prolog_inputs(9, 4, "mxfp8")
    c = {k: v.to(DEV) for k, v in inp.items()}
    k_cache, k_scale_cache = helpers.pg_cache_views(c["pages"], "mxfp8")
    q = torch.zeros((4 * 24, 128), dtype=torch.uint8, device=DEV)
    q_scale = torch.zeros((4 * 24, 1), dtype=torch.float32, device=DEV)
    weights = torch.zeros((4, 24), dtype=torch.bfloat16, device=DEV)
    fn = _impl("mxfp8").lightning_indexer_prolog_quant

    def call(**over):
        a = dict(x=c["x"], q_norm=c["q_norm"], q_norm_scale=c["q_norm_scale"], w_qb=c["w_qb"], w_qb_scale=c["w_qb_scale"],
                 wk=c["wk"], w_proj=c["w_proj"], gamma_k=c["gamma_k"], cos=c["cos"], sin=c["sin"], hq=c["hadamard_q"],
                 hk=c["hadamard_k"], k_in=k_cache, ks_in=k_scale_cache, idx=c["cache_index"], sidx=c["cache_index"], q=q,
                 qs=q_scale, k_out=k_cache, ks_out=k_scale_cache, w=weights)
        a.update(over)
        fn(a["x"], a["q_norm"], a["q_norm_scale"], a["w_qb"], a["w_qb_scale"], a["wk"], a["w_proj"], a["gamma_k"], a["cos"],
           a["sin"], a["hq"], a["hk"], a["k_in"], a["ks_in"], a["idx"], a["sidx"], a["q"], a["qs"], a["k_out"], a["ks_out"], a["w"])

    with pytest.raises(ValueError):
        call(q_norm=c["q_norm"].float())                       # not an 8-bit code tensor
    with pytest.raises(ValueError):
        call(w_qb_scale=c["w_qb_scale"].reshape(-1))           # scales not in the [q_lora / 64, n, 2] layout
    with pytest.raises(ValueError):
        call(k_out=k_cache.clone())                            # the update is in place: in and out must be one view
    with pytest.raises(ValueError):
        call(q=torch.zeros((4 * 24, 64), dtype=torch.uint8, device=DEV))
    with pytest.raises(RuntimeError):
        call(x=inp["x"])                                       # a CPU tensor
    # a row index past the caches: reported through the status word, nothing written for that token
    bad_idx = c["cache_index"].clone()
    bad_idx[2, 0] = 4 * 128
    pages_before = c["pages"].clone()
    call(idx=bad_idx, sidx=bad_idx)
    with pytest.raises(RuntimeError, match="out of range"):
        pypto_b200.check_status(DEV)
    k_after, _ = helpers.pg_cache_views(c["pages"], "mxfp8")
    k_before, _ = helpers.pg_cache_views(pages_before, "mxfp8")
    others = torch.ones(4 * 128, dtype=torch.bool, device=DEV)
    others[c["cache_index"].reshape(-1)[[0, 1, 3]]] = False
    assert torch.equal(k_after.reshape(-1, 128).view(torch.uint8)[others], k_before.reshape(-1, 128).view(torch.uint8)[others])
    rt.status_word(torch.device(DEV)).zero_()
