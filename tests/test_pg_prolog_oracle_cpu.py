"""CPU pins of the page-grouped 8-bit-float indexer prolog oracle: the fp32 golden restatement against the fixture
made from the reference's own golden, the operator restatement against that golden under the reference's three-way
accuracy rule, and the HiF8 codec against the facts the reference's decoder states."""
import math

import numpy as np
import torch

import helpers
from oracle import pg_prolog_oracle as pgo


def _golden_case():
    g = helpers.load_pg_prolog_mxfp8_golden()
    inp = helpers.pg_prolog_reference_inputs(g["seed"], g["b"], g["s1"], g["s2"])
    for name, want in g["digests"].items():
        assert helpers.pg_digest(inp[name]) == want, f"input {name} differs from the reference generator's"
    t = g["b"] * g["s1"]
    args = dict(
        x=inp["token_x"].reshape(t, -1), q_norm=inp["q_norm"].reshape(t, -1),
        q_norm_scale=inp["q_norm_scale"].reshape(t, -1).view(torch.uint8), w_qb=inp["w_idx_qb"],
        w_qb_scale=inp["w_idx_qb_scale"].view(torch.uint8), wk=inp["w_idx_k"], w_proj=inp["w_idx_proj"],
        gamma_k=inp["rms_norm_gamma"], cos=inp["cos_idx_rope"].reshape(t, -1), sin=inp["sin_idx_rope"].reshape(t, -1),
        hadamard_q=inp["hadamard_q"], hadamard_k=inp["hadamard_k"])
    return g, inp, args, t


def test_fp32_golden_restatement_equals_the_reference_golden_fixture():
    g, inp, args, t = _golden_case()
    q, qs, k, ks, w = pgo.pg_prolog_golden(**args)
    assert torch.equal(q.reshape(t, 24, 128).view(torch.uint8), g["q"])
    assert torch.equal(qs.reshape(t, 24, 1), g["q_scale"])
    assert torch.equal(k.view(torch.uint8), g["k"])
    assert torch.equal(ks.reshape(-1), g["k_scale"])
    assert torch.equal(w, g["weights"])
    assert torch.equal(inp["idx_k_cache_index"].reshape(-1), g["cache_index"])


def test_operator_restatement_meets_the_reference_accuracy_rule_against_its_golden():
    g, inp, args, t = _golden_case()
    q, qs, k, ks, w = pgo.pg_prolog(fmt="mxfp8", **args)
    gq = g["q"].view(torch.float8_e4m3fn).float()
    # the golden itself stands in as the benchmark: the ratios are then absolute errors over the small-value threshold
    for out, gold, kind in ((q.float(), gq, "fp8"), (qs, g["q_scale"], "fp32"), (k.float(), g["k"].view(torch.float8_e4m3fn).float(), "fp8"),
                            (ks.reshape(-1), g["k_scale"], "fp32"), (w.float(), g["weights"], "bf16")):
        d = (out.flatten() - gold.flatten()).abs()
        assert float((d / (gold.flatten().abs() + 1e-3)).mean()) < 0.02, kind
    # 8-bit codes: nearly all equal, the rest one code step away
    same = (q.view(torch.uint8) == g["q"]).float().mean()
    assert same > 0.9, float(same)


def test_hif8_decode_table_facts_and_round_trip():
    table = pgo.hif8_decode_table()
    assert table[0x00] == 0.0 and math.isnan(table[0x80])                 # no negative zero: 1_0000_000 is NaN
    assert np.isinf(table[0b0_11_0111_1]) and table[0b0_11_0111_1] > 0     # S_11_0111_1 is infinity
    assert table[0b0_11_0111_0] == 32768.0                                  # the largest finite value, 2^15
    assert table[0b0_0001_000] == 1.0 and table[0b0_0001_111] == 1.875      # exponent 0, three mantissa bits
    assert table[0b0_0000_001] == 2.0 ** -22 and table[0b0_0000_111] == 2.0 ** -16
    assert table[0b0_001_0_100] == 3.0 and table[0b0_001_1_000] == 0.5      # exponent +1 / -1
    assert table[0b0_01_00_000] == 4.0 and table[0b0_01_11_000] == 0.125    # exponent +-(2 + e)
    assert table[0b0_10_000_00] == 16.0 and table[0b0_10_111_11] == 2.0 ** -7 * 1.75
    assert table[0b0_11_1111_0] == 2.0 ** -15
    finite = [c for c in range(256) if np.isfinite(table[c])]
    vals = sorted(set(float(table[c]) for c in finite))
    assert len(vals) == len(finite)                                          # every finite code is a distinct value
    codes = torch.tensor(finite, dtype=torch.uint8)
    assert torch.equal(pgo.hif8_encode(pgo.hif8_decode(codes)), codes)       # encode inverts decode
    # nearest value, ties away from zero, saturation
    assert int(pgo.hif8_encode(torch.tensor([1.0625]))[0]) == 0b0_0001_001   # halfway between 1.0 and 1.125
    assert int(pgo.hif8_encode(torch.tensor([-1.0624]))[0]) == 0b1_0001_000
    assert int(pgo.hif8_encode(torch.tensor([1e9]))[0]) == 0b0_11_0111_0
    assert int(pgo.hif8_encode(torch.tensor([-0.0]))[0]) == 0


def test_hif8_operator_restatement_is_self_consistent():
    inp = helpers.gen_pg_prolog_inputs(5, 3, "hif8")
    args = {k: inp[k] for k in ("x", "q_norm", "q_norm_scale", "w_qb", "w_qb_scale", "wk", "w_proj", "gamma_k", "cos", "sin",
                                "hadamard_q", "hadamard_k")}
    q, qs, k, ks, w = pgo.pg_prolog(fmt="hif8", **args)
    assert q.dtype == torch.uint8 and q.shape == (3, 24, 128) and qs.shape == (3, 24, 1)
    # every row uses the whole range: its largest magnitude is the largest finite code
    top = pgo.hif8_decode(q).abs().amax(dim=-1)
    assert torch.all(top == 32768.0)
    assert torch.isfinite(w.float()).all() and ks.shape == (3, 1)
