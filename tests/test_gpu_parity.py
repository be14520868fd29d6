"""GPU parity tests: the CUDA path (through the Python entry points -> C ABI) against the CPU oracle
and against the committed reference-golden fixtures.  Tolerances:
  * indexer int32 dot products: bit-exact;
  * top-k index sets: equal, ties by lower index; entries within 1e-6 (relative) of the k-th score exempt;
  * attention output: rtol 1e-2, atol 1e-2 (bf16); max-abs / mean-abs error are reported.  The reference's
    own test rule (atol 1e-4, rtol 5e-3, <= 0.5 % of elements outside) cannot be met by an online softmax:
    it rounds P to bf16 before the final normalisation, the golden after it, which flips the last bf16 bit
    of 3-10 % of the outputs (emulating the online order with torch on the CPU gives the same fraction), and
    one bf16 ulp is up to 0.78 % > rtol 5e-3.  That fraction is reported and bounded at 15 % as a regression
    guard, and the mean absolute error must stay below 1 % of the mean output magnitude;
  * prolog: int8 outputs within 1 LSB, scales / weights atol 2.5e-5 (the reference's test tolerances).
"""
import math

import pytest
import torch

import helpers
from oracle import dsv32_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _cuda(d):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


# --------------------------------------------------------------------------------------------------
# top-k
# --------------------------------------------------------------------------------------------------
def _run_topk(scores, counts, k, ids=None, id_base=0):
    import pypto_b200
    from pypto_b200.lightning_indexer_quant_impl import topk_select
    oi, os_ = topk_select(scores.to(DEV), counts.to(DEV), k, ids=None if ids is None else ids.to(DEV), id_base=id_base)
    pypto_b200.check_status()
    return oi.cpu(), os_.cpu()


def test_topk_kat_ties_lower_index_first():
    kat = helpers.load_kat()["topk_ties"]
    sc = torch.tensor([kat["input"]], dtype=torch.float32)
    oi, os_ = _run_topk(sc, torch.tensor([len(kat["input"])], dtype=torch.int32), kat["k"])
    assert oi[0].tolist() == kat["indices"]
    assert os_[0].tolist() == [float(v) for v in kat["values"]]


@pytest.mark.parametrize("n,k", [(70000, 2048), (5000, 2048), (2048, 2048), (100, 2048), (1, 4), (131072, 2048)])
def test_topk_random_rows_exact_order(n, k):
    g = torch.Generator().manual_seed(n + k)
    rows = 3
    sc = torch.randn(rows, n, generator=g)
    sc[1] = torch.randint(0, 50, (n,), generator=g).float()  # heavy ties
    sc[2] = -sc[2].abs()  # all negative
    counts = torch.tensor([n, n, max(n - 3, 1)], dtype=torch.int32)
    oi, os_ = _run_topk(sc, counts, k)
    for r in range(rows):
        c = int(counts[r])
        ref = orc.topk_indices_ref(sc[r, :c], min(k, c))
        assert oi[r, :ref.numel()].tolist() == ref.tolist(), (r,)
        assert (oi[r, ref.numel():] == -1).all()
        assert torch.equal(os_[r, :ref.numel()], sc[r, ref])


@pytest.mark.parametrize("n,k", [(65536, 2048), (9000, 2048), (65536, 100)])
def test_topk_exact_order_across_score_distributions(n, k):
    """The output order comes from placing the winners by the top 12 key bits and ranking inside a bucket, with the
    bitonic sort as the fall-back for crowded buckets: rows whose winners spread over many octaves (hundreds of small
    buckets), over both signs, over one narrow bucket (the fall-back), a row with a plateau of equal scores across
    the threshold, and one with infinities."""
    g = torch.Generator().manual_seed(n * 3 + k)
    sc = torch.empty(6, n)
    sc[0] = torch.exp(torch.randn(n, generator=g) * 4)                       # many octaves
    sc[1] = torch.randn(n, generator=g) * torch.exp(torch.randn(n, generator=g) * 3)   # both signs, wide
    sc[2] = 1.0 + torch.rand(n, generator=g) * 0.01                          # one bucket
    sc[3] = torch.randn(n, generator=g)
    sc[3, torch.randperm(n, generator=g)[:min(3 * k, n // 2)]] = 0.75          # plateau around the threshold
    sc[4] = torch.randn(n, generator=g)
    sc[4, :7] = float("inf")
    sc[4, 7:19] = float("-inf")
    sc[5] = -torch.exp(torch.randn(n, generator=g) * 4)                      # all negative, many octaves
    counts = torch.full((6,), n, dtype=torch.int32)
    oi, os_ = _run_topk(sc, counts, k)
    for r in range(6):
        ref = orc.topk_indices_ref(sc[r], min(k, n))
        assert oi[r, :ref.numel()].tolist() == ref.tolist(), (r,)
        assert torch.equal(os_[r, :ref.numel()], sc[r, ref])


@pytest.mark.parametrize("rows,ld", [(2, 65536), (20, 65536), (40, 65536), (5, 65537), (3, 131072 + 36)])
def test_topk_rows_split_over_a_cluster(rows, ld):
    """While rows are few and long, a row is scanned by the 8, 4 or 2 CTAs of a cluster (fewer CTAs as rows grow).
    One launch mixes rows that are split with rows that are not: a short one, an empty one, rows whose start is
    not 16-byte aligned (odd row pitch), a row of one narrow bucket (the threshold bucket overflows the candidate
    list and the first CTA finishes alone) and a plateau across the threshold."""
    k = 2048
    g = torch.Generator().manual_seed(rows * 7 + ld)
    sc = torch.randn(rows, ld, generator=g)
    counts = torch.full((rows,), ld, dtype=torch.int32)
    counts[0] = ld - 5
    if rows > 2:
        counts[1] = 3000                                             # short: left to the first CTA
        sc[2] = 2.0 + torch.rand(ld, generator=g) * 0.001            # one bucket
    if rows > 4:
        counts[3] = 0
        sc[4, torch.randperm(ld, generator=g)[:3 * k]] = 1.25          # plateau around the threshold
    oi, os_ = _run_topk(sc, counts, k)
    for r in range(rows):
        c = int(counts[r])
        ref = orc.topk_indices_ref(sc[r, :c], min(k, c))
        assert oi[r, :ref.numel()].tolist() == ref.tolist(), (r,)
        assert (oi[r, ref.numel():] == -1).all()
        assert torch.equal(os_[r, :ref.numel()], sc[r, ref])


def test_topk_explicit_ids_merge_rule():
    g = torch.Generator().manual_seed(9)
    n, k = 4096, 512
    sc = torch.randint(0, 200, (2, n), generator=g).float()
    ids = torch.stack([torch.randperm(100000, generator=g)[:n] for _ in range(2)]).to(torch.int32)
    ids[0, 5:50] = -1  # ignored entries
    sc_cpu = sc.clone()
    sc_cpu[ids < 0] = float("-inf")
    oi, _ = _run_topk(sc, torch.tensor([n, n], dtype=torch.int32), k, ids=ids)
    ref = orc.merge_topk_candidates(sc_cpu, ids, k)
    assert torch.equal(oi, ref)


# --------------------------------------------------------------------------------------------------
# lightning indexer
# --------------------------------------------------------------------------------------------------
def _run_indexer(d, selected=2048, want_scores=True, want_dots=False, key_begin=0, key_end=2 ** 31 - 1):
    import pypto_b200
    from pypto_b200.lightning_indexer_quant_impl import indexer_scores_topk
    c = _cuda(d)
    t = d["query"].shape[0]
    ld = d["block_table"].shape[1] * 128
    res = torch.zeros((t, 1, selected), dtype=torch.int32, device=DEV)
    tsc = torch.zeros((t, selected), dtype=torch.float32, device=DEV)
    scores = torch.full((t, ld), float("nan"), dtype=torch.float32, device=DEV) if want_scores else None
    dots = torch.zeros((t, 64, ld), dtype=torch.int32, device=DEV) if want_dots else None
    indexer_scores_topk(c["query"], c["q_scale"], c["key"], c["k_scale"], c["weights"], c["act_seq"], c["block_table"],
                        res, selected, topk_scores=tsc, scores_out=scores, dots_out=dots, key_begin=key_begin,
                        key_end=key_end)
    pypto_b200.check_status()
    return res.cpu(), tsc.cpu(), None if scores is None else scores.cpu(), None if dots is None else dots.cpu()


def _check_indexer_against_oracle(d, res, scores_gpu, selected=2048):
    ref, ref_scores = orc.lightning_indexer(d["query"], d["q_scale"], d["key"], d["k_scale"], d["weights"],
                                            d["act_seq"], d["block_table"], selected, return_scores=True)
    s1 = d["s1"]
    for t in range(res.shape[0]):
        bi, si = divmod(t, s1)
        L = int(d["act_seq"][bi])
        eff = L - (s1 - 1 - si)
        sc_ref = ref_scores[bi][si]
        if scores_gpu is not None and L > 0:
            got = scores_gpu[t, :L]
            assert torch.allclose(got, sc_ref[:L], rtol=2e-6, atol=1e-7), (t, (got - sc_ref[:L]).abs().max())
        ok, ndiff, nexc = orc.topk_sets_match(res[t, 0], ref[t, 0], sc_ref if eff > 0 else sc_ref)
        assert ok, (t, ndiff, nexc)
        nvalid = max(min(eff, selected), 0)
        assert (res[t, 0, :nvalid] >= 0).all() and (res[t, 0, nvalid:] == -1).all()


def test_indexer_reference_golden_fixture():
    g = helpers.load_indexer_golden()
    res, _, scores, dots = _run_indexer(g, want_dots=True)
    # bit-exact int32 dot products
    for bi in range(g["b"]):
        L = int(g["act_seq"][bi])
        rows = orc.paged_rows(g["block_table"][bi], torch.arange(L), 128)
        keys = g["key"].reshape(-1, 128)[rows].to(torch.int32)
        for si in range(g["s1"]):
            t = bi * g["s1"] + si
            ref = g["query"][t].to(torch.int32) @ keys.t()
            assert torch.equal(dots[t, :, :L], ref)
    _check_indexer_against_oracle(g, res, scores)
    # and directly against the reference's own golden output
    _, ref_scores = orc.lightning_indexer(g["query"], g["q_scale"], g["key"], g["k_scale"], g["weights"],
                                          g["act_seq"], g["block_table"], 2048, return_scores=True)
    for t in range(res.shape[0]):
        ok, ndiff, _ = orc.topk_sets_match(res[t, 0], g["topk_res"][t, 0], ref_scores[t // g["s1"]][t % g["s1"]])
        assert ok, (t, ndiff)


@pytest.mark.parametrize("act_seq,s1", [([4101, 971, 2048, 129], 1), ([3000, 127, 2049], 2), ([1, 2, 5000], 2),
                                        ([700, 2500], 4), ([16511], 3)])
def test_indexer_ragged_vs_oracle(act_seq, s1):
    d = helpers.gen_indexer_inputs(100 + len(act_seq) + s1, act_seq, s1=s1, extra_blocks=3)
    res, tsc, scores, _ = _run_indexer(d)
    _check_indexer_against_oracle(d, res, scores)
    # rows are sorted by descending score and the reported scores are the scores of the reported keys
    for t in range(res.shape[0]):
        n = int((res[t, 0] >= 0).sum())
        if n:
            assert (tsc[t, :n - 1] >= tsc[t, 1:n]).all()
            assert torch.equal(tsc[t, :n], scores[t, res[t, 0, :n].long()])


def test_indexer_64k_context_properties_and_sampled_oracle():
    d = helpers.gen_indexer_inputs(7, [65536, 65536, 40000], s1=2)
    res, tsc, scores, _ = _run_indexer(d)
    _check_indexer_against_oracle(d, res, scores)
    for t in range(res.shape[0]):
        row = res[t, 0]
        assert row.min() >= 0 and row.unique().numel() == 2048
        assert (tsc[t, :-1] >= tsc[t, 1:]).all()
        eff = int(d["act_seq"][t // 2]) - (1 - t % 2)
        assert row.max() < eff
        # every unselected score is <= the smallest selected one
        mask = torch.ones(eff, dtype=torch.bool)
        mask[row.long()] = False
        assert scores[t, :eff][mask].max() <= tsc[t, -1]


def test_indexer_key_range_shards_merge_to_global_topk():
    import pypto_b200
    from pypto_b200.lightning_indexer_quant_impl import topk_select
    d = helpers.gen_indexer_inputs(21, [6000], s1=2)
    full, _, _, _ = _run_indexer(d)
    shards, k = 3, 2048
    cs, ci = [], []
    for s in range(shards):
        res, tsc, _, _ = _run_indexer(d, want_scores=False, key_begin=s * 2048, key_end=(s + 1) * 2048)
        cs.append(tsc)
        ci.append(res[:, 0])
    cand_s, cand_i = torch.cat(cs, 1), torch.cat(ci, 1).to(torch.int32)
    counts = torch.full((cand_s.shape[0],), cand_s.shape[1], dtype=torch.int32)
    oi, _ = topk_select(cand_s.to(DEV), counts.to(DEV), k, ids=cand_i.to(DEV))
    pypto_b200.check_status()
    assert torch.equal(oi.cpu(), full[:, 0])
    assert torch.equal(orc.merge_topk_candidates(cand_s, cand_i, k), full[:, 0])


@pytest.mark.parametrize("act_seq,s1", [([3000, 700], 8), ([5000], 64), ([260, 9000], 5)])
def test_indexer_many_query_tokens_per_request(act_seq, s1):
    """More than four query tokens per request (a prefill-style chunk): the kernel walks the tokens in groups of
    four (grid.z), the last group may be partial.  Checked like the ragged cases: scores, top-k sets, pads."""
    d = helpers.gen_indexer_inputs(300 + s1, act_seq, s1=s1, extra_blocks=2)
    res, tsc, scores, dots = _run_indexer(d, want_dots=True)
    _check_indexer_against_oracle(d, res, scores)
    for bi, L in enumerate(act_seq):   # bit-exact int32 dot products of the first and the last token of a request
        rows = orc.paged_rows(d["block_table"][bi], torch.arange(L), 128)
        keys = d["key"].reshape(-1, 128)[rows].to(torch.int32)
        for si in (0, s1 - 1):
            t = bi * s1 + si
            assert torch.equal(dots[t, :, :L], d["query"][t].to(torch.int32) @ keys.t())


def test_indexer_sequence_longer_than_page_table_is_clamped_and_reported():
    """act_seq beyond max_blocks * 128: status BAD_INDEX, nothing written past the page table's capacity (a guard
    region after every score row stays untouched), the keys the table does describe are still scored."""
    import pypto_b200
    from pypto_b200.lightning_indexer_quant_impl import indexer_scores_topk
    d = helpers.gen_indexer_inputs(12, [1100, 1152], s1=2)       # 9 blocks per request
    max_blocks = d["block_table"].shape[1]
    cap = max_blocks * 128
    good, _, good_scores, _ = _run_indexer(dict(d, act_seq=torch.tensor([cap, cap], dtype=torch.int32)))
    d["act_seq"] = torch.tensor([cap + 300, 1152], dtype=torch.int32)
    c = _cuda(d)
    t, guard = d["query"].shape[0], 64 * 128
    res = torch.zeros((t, 1, 2048), dtype=torch.int32, device=DEV)
    scores = torch.full((t, cap + guard), 12345.0, dtype=torch.float32, device=DEV)
    indexer_scores_topk(c["query"], c["q_scale"], c["key"], c["k_scale"], c["weights"], c["act_seq"], c["block_table"],
                        res, 2048, scores_out=scores)
    with pytest.raises(RuntimeError, match="status"):
        pypto_b200.check_status()
    sc = scores.cpu()
    assert (sc[:, cap:] == 12345.0).all()
    assert torch.equal(sc[:2, :cap], good_scores[:2, :cap])      # request 0: every key of its nine pages
    assert torch.equal(res.cpu()[1], good[1])                    # its last token sees all of them in both runs


def test_indexer_bad_page_table_sets_status_not_fault():
    import pypto_b200
    d = helpers.gen_indexer_inputs(3, [600], s1=1)
    d["block_table"][0, 1] = -1
    with pytest.raises(RuntimeError, match="status"):
        _run_indexer(d, want_scores=False)
    pypto_b200.check_status()  # cleared


# --------------------------------------------------------------------------------------------------
# sparse flash attention
# --------------------------------------------------------------------------------------------------
def _run_sfa(d, kv_splits=0, entry="d"):
    import pypto_b200
    from pypto_b200 import sparse_flash_attention_quant_impl as sfa
    c = _cuda(d)
    out = torch.full((d["b"], d["s1"], d["nq"], 512), float("nan"), dtype=torch.bfloat16, device=DEV)
    cfg = sfa.SaTileShapeConfig()
    if kv_splits:
        sfa._sfa(c["q_nope"], c["q_rope"], c["k_nope"], c["k_rope"], c["k_scales"], c["topk_indices"],
                 c["block_table"], c["act_seq"], out, d["nq"], 1, d["softmax_scale"], d.get("topk", 2048), 128,
                 d["block_table"].shape[1], cfg, kv_splits=kv_splits)
    else:
        fn = {"d": sfa.sparse_flash_attention_quant_d, "p": sfa.sparse_flash_attention_quant_p,
              "d950": sfa.sparse_flash_attention_quant_d_950}[entry]
        fn(c["q_nope"], c["q_rope"], c["k_nope"], c["k_rope"], c["k_scales"], c["topk_indices"], c["block_table"],
           c["act_seq"], out, d["nq"], 1, d["softmax_scale"], d.get("topk", 2048), 128, d["block_table"].shape[1], cfg)
    pypto_b200.check_status()
    return out.cpu()


def _sfa_oracle(d, tokens=None):
    return orc.sfa_quant(d["q_nope"], d["q_rope"], d["k_nope"], d["k_rope"], d["k_scales"], d["topk_indices"],
                         d["block_table"], d["act_seq"], d["nq"], d["softmax_scale"], d.get("topk", 2048), 128,
                         tokens=tokens)


def _assert_attention_close(out, ref, strict_frac=0.15):
    o, r = out.float(), ref.float()
    assert not torch.isnan(o).any()
    err = (o - r).abs()
    assert torch.allclose(o, r, rtol=1e-2, atol=1e-2), f"max-abs {err.max():.4g} mean-abs {err.mean():.4g}"
    strict = orc.reference_compare_count(out, ref, 1e-4, 5e-3)
    print(f"[attention] strict-rule outliers {strict / max(out.numel(), 1):.4f} of {out.numel()} (bound {strict_frac})")
    assert strict <= strict_frac * out.numel(), f"{strict} of {out.numel()} outside the reference's own last-bit rule"
    assert err.mean() <= 1e-2 * r.abs().mean() + 1e-6, f"mean-abs {err.mean():.4g} vs mean |ref| {r.abs().mean():.4g}"
    return float(err.max()), float(err.mean())


def test_sfa_reference_golden_fixture():
    g = helpers.load_sfa_golden()
    out = _run_sfa(g)
    _assert_attention_close(out, g["out"])
    _assert_attention_close(out, _sfa_oracle(g))


def test_sfa_bf16_cache_reference_golden_fixture_and_seeded():
    """The operator's branch for a cache that is not quantised (bf16 latent rows, no scales)."""
    g = helpers.load_sfa_bf16_golden()
    out = _run_sfa(g)
    _assert_attention_close(out, g["out"])
    _assert_attention_close(out, _sfa_oracle(g))
    d = helpers.gen_sfa_inputs(61, [3000, 64, 2049], s1=2, extra_blocks=1)
    d["k_nope"] = (d["k_nope"].float() * 0.01).to(torch.bfloat16)
    d["k_scales"] = None
    _assert_attention_close(_run_sfa(d), _sfa_oracle(d))
    _assert_attention_close(_run_sfa(d, kv_splits=3), _sfa_oracle(d))


# ---- DeepSeek-V4 sparse compress attention (window + selected compressed keys + sinks) -------------------------
def _run_scfa(d, entry="kernel"):
    import pypto_b200
    from pypto_b200 import sparse_compress_flash_attention_impl as scfa
    c = _cuda(d)
    args = (c["q"], c["actual_seq_q"], c["ori_kv"], c["cmp_kv"], c["ori_block_table"], c["cmp_block_table"],
            c["atten_sink"], c["seqused_kv"], c["cmp_sparse_indices"])
    if entry == "kernel":
        out = torch.full_like(c["q"], float("nan"))
        cfg = scfa.SCFATileShapeConfig(64, [64, 64, 128, 512, 128, 128], [32, 640], [64, 64, 128, 640, 256, 256])
        assert scfa.sparse_compress_flash_attention_kernel(*args, out, d["nq"], 1, d["softmax_scale"], d["topk"],
                                                           d["block_size"], d["win_size"], d["cmp_ratio"], cfg) is None
    else:
        fn = scfa.npu_sparse_compress_flash_attention if entry == "npu" else scfa.sparse_compress_flash_attention_graph
        out = fn(*args, d["softmax_scale"], d["win_size"], d["cmp_ratio"])
    pypto_b200.check_status()
    return out.cpu()


def _scfa_oracle(d):
    return orc.scfa(d["q"], d["actual_seq_q"], d["ori_kv"], d["cmp_kv"], d["ori_block_table"], d["cmp_block_table"],
                    d["atten_sink"], d["seqused_kv"], d["cmp_sparse_indices"], d["nq"], d["softmax_scale"],
                    d["win_size"], d["cmp_ratio"], d["block_size"])


def test_scfa_reference_golden_fixture():
    g = helpers.load_scfa_golden()
    out = _run_scfa(g)
    _assert_attention_close(out, g["out"].reshape(out.shape))
    _assert_attention_close(out, _scfa_oracle(g))
    assert torch.equal(_run_scfa(g, "npu"), out)
    assert torch.equal(_run_scfa(g, "graph"), out)


@pytest.mark.parametrize("seed,ori_seq,s1_list,nq,kw", [
    (1, [8192, 8192, 8192, 8192], [2, 2, 2, 2], 64, {}),                       # the reference's decode shape, 4 requests
    (2, [65536, 130, 700, 50], [16, 1, 3, 4], 64, {}),                         # ragged s1; a context shorter than the window
    (3, [3, 1, 2100, 0], [1, 3, 2, 2], 64, {}),                                # no compressed key; tokens with no key at all
    (4, [2100, 4000], [2, 1], 128, {"holes": 37}),                             # 128 heads; -1 entries among the selected
    (5, [5000, 300], [1, 2], 32, {"topk": 200, "win_size": 64, "cmp_ratio": 8, "scale": 3.0}),   # other sizes, peaked softmax
    (6, [900], [5], 64, {"topk": 64, "win_size": 300, "cmp_ratio": 2}),        # window longer than two pages
    (7, [5000], [1], 64, {}),                                                  # one token: fewer query rows than the 128-row tile
    (8, [300], [1], 32, {"topk": 64}),
    (9, [2100, 900, 3000], [2, 3, 4], 64, {"holes": 37}),                      # paired tokens with -1 entries among the selected
    (10, [2100, 300, 129], [2, 4, 3], 16, {}),                                 # 16 heads: both tokens of a pair in one warp
    (11, [900, 5000], [3, 2], 48, {"holes": 11}),                              # 48 heads: a warp with heads of both tokens
])
def test_scfa_seeded_cases(seed, ori_seq, s1_list, nq, kw):
    d = helpers.gen_scfa_inputs(700 + seed, ori_seq, s1_list, nq=nq, **kw)
    out = _run_scfa(d)
    ref = _scfa_oracle(d)
    # With a peaked softmax few keys carry the sum, so the bf16 rounding of the probabilities (un-normalised in the
    # kernel, normalised in the reference) shows in the last bit of more outputs; the 1e-2 bar is unchanged.
    _assert_attention_close(out, ref, strict_frac=0.35 if kw.get("scale", 1.0) > 1.0 else 0.15)
    # a token without any key (context shorter than its position) yields a zero row, as in the oracle
    assert torch.equal(out.float().abs().sum(-1) == 0, ref.float().abs().sum(-1) == 0)


def test_scfa_reference_decode_shape_sampled_tokens():
    """The reference's decode case (64 requests x 2 tokens, context 8192, 64 heads, 128 + 512 keys): sampled tokens
    against the oracle, every row finite, and the result independent of the order of the selected indices up to
    the rounding of another summation order."""
    d = helpers.gen_scfa_inputs(760, [8192] * 64, [2] * 64)
    out = _run_scfa(d)
    assert torch.isfinite(out.float()).all() and (out.float().abs().sum(-1) > 0).all()
    sample = [0, 1, 37, 64, 126, 127]
    ref = orc.scfa(d["q"], d["actual_seq_q"], d["ori_kv"], d["cmp_kv"], d["ori_block_table"], d["cmp_block_table"],
                   d["atten_sink"], d["seqused_kv"], d["cmp_sparse_indices"], d["nq"], d["softmax_scale"], d["win_size"],
                   d["cmp_ratio"], d["block_size"], tokens=sample)
    rows = torch.cat([torch.arange(t * 64, (t + 1) * 64) for t in sample])
    _assert_attention_close(out[rows], ref[rows])
    g = torch.Generator().manual_seed(1)
    shuffled = dict(d, cmp_sparse_indices=d["cmp_sparse_indices"][:, torch.randperm(512, generator=g)].contiguous())
    out2 = _run_scfa(shuffled)
    assert torch.allclose(out2.float(), out.float(), rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("shared", [512, 460, 1])
def test_scfa_paired_tokens_with_overlapping_selections(shared):
    """With at most 64 heads the two tokens of a request share a CTA and its key list is the union of both selections:
    identical, mostly identical and nearly disjoint selections must all match the oracle."""
    d = helpers.gen_scfa_inputs(790 + shared, [8192] * 6, [2] * 6)
    idx = d["cmp_sparse_indices"].clone()
    idx[1::2, :shared] = idx[0::2, :shared]
    if shared < 512:   # keep every row free of duplicates: the rest of the odd rows comes from the unused positions
        g = torch.Generator().manual_seed(shared)
        for t in range(1, idx.shape[0], 2):
            used = set(idx[t - 1].tolist())
            rest = [v for v in torch.randperm(2048, generator=g).tolist() if v not in used][:512 - shared]
            idx[t, shared:] = torch.tensor(rest, dtype=torch.int32)
    d = dict(d, cmp_sparse_indices=idx)
    _assert_attention_close(_run_scfa(d), _scfa_oracle(d))


def test_scfa_sink_and_window_matter():
    """The sink only enters the denominator; dropping it, or the window, must change the result."""
    d = helpers.gen_scfa_inputs(770, [1000, 600], [1, 2])
    out = _run_scfa(d)
    d2 = dict(d, atten_sink=torch.full_like(d["atten_sink"], -1e30))
    no_sink = _run_scfa(d2)
    _assert_attention_close(no_sink, _scfa_oracle(d2))
    assert not torch.allclose(out.float(), no_sink.float(), rtol=1e-2, atol=1e-4)
    big = dict(d, atten_sink=torch.full_like(d["atten_sink"], 30.0))   # a dominant sink drives the output to zero
    assert _run_scfa(big).float().abs().max() < 1e-6
    d3 = dict(d, win_size=0)
    _assert_attention_close(_run_scfa(d3), _scfa_oracle(d3))


def test_scfa_bad_arguments_and_bad_pages():
    import pypto_b200
    from pypto_b200 import sparse_compress_flash_attention_impl as scfa
    d = helpers.gen_scfa_inputs(780, [600, 300], [1, 1])
    c = _cuda(d)

    def call(**over):
        a = dict(c, **over)
        out = torch.zeros_like(a["q"])
        scfa.sparse_compress_flash_attention_kernel(
            a["q"], a["actual_seq_q"], a["ori_kv"], a["cmp_kv"], a["ori_block_table"], a["cmp_block_table"],
            a["atten_sink"], a["seqused_kv"], a["cmp_sparse_indices"], out, over.get("nq", d["nq"]), over.get("n_kv", 1),
            d["softmax_scale"], d["topk"], d["block_size"], d["win_size"], over.get("cmp_ratio", d["cmp_ratio"]), None)

    with pytest.raises(ValueError):
        call(q=c["q"].float())
    with pytest.raises(ValueError):
        call(n_kv=2)
    with pytest.raises(ValueError):
        call(actual_seq_q=c["actual_seq_q"][:-1].contiguous())
    with pytest.raises(ValueError):
        call(atten_sink=c["atten_sink"][:-1].contiguous())
    with pytest.raises(ValueError):
        call(cmp_ratio=0)
    with pytest.raises(RuntimeError):
        call(q=d["q"])                                    # host tensor
    bad = c["cmp_block_table"].clone()
    bad[0, 0] = -1                                        # a selected key on a page that is not mapped
    call(cmp_block_table=bad)
    with pytest.raises(RuntimeError):
        pypto_b200.check_status()
    bad = c["ori_block_table"].clone()
    bad[1, 2] = 10 ** 6                                   # a window row past the end of the cache
    call(ori_block_table=bad)
    with pytest.raises(RuntimeError):
        pypto_b200.check_status()
    call()                                                # the context stays usable
    pypto_b200.check_status()


# ---- DeepSeek-V4 compress flash attention (window + every compressed row) and sliding-window attention ---------
def _run_cfa(d, graph=False):
    import pypto_b200
    from pypto_b200 import compress_flash_attention_impl as cfa
    c = _cuda(d)
    fn = cfa.cfa_graph if graph else cfa.cfa_attention
    out = fn(c["q"], c["cmp_kv"], c["atten_sink"], c["cmp_block_table"], c["seqused_kv"], c["ori_kv"],
             c["ori_block_table"], d["cmp_ratio"])
    pypto_b200.check_status()
    assert out.shape == d["q"].shape
    return out.cpu()


def _cfa_oracle(d):
    return orc.cfa(d["q"], d["cmp_kv"], d["atten_sink"], d["cmp_block_table"], d["seqused_kv"], d["ori_kv"],
                   d["ori_block_table"], d["cmp_ratio"])


def _as_cfa_inputs(d, s1):
    """Seeded sparse-compress inputs in the 3-D / 4-D layouts of the compress flash attention operator."""
    t = d["b"] * s1
    return dict(d, q=d["q"].reshape(t, d["nq"], 512), cmp_kv=d["cmp_kv"].reshape(-1, 128, 1, 512),
                ori_kv=d["ori_kv"].reshape(-1, 128, 1, 512))


def test_cfa_reference_golden_fixture():
    g = helpers.load_cfa_golden()
    out = _run_cfa(g)
    _assert_attention_close(out, g["out"])
    _assert_attention_close(out, _cfa_oracle(g))
    assert torch.equal(_run_cfa(g, graph=True), out)


@pytest.mark.parametrize("seed,ori_seq,s1,nq,cmp_ratio", [
    (1, [8192] * 4, 2, 64, 128),          # the reference's decode shape (64 compressed rows), 4 requests
    (2, [65536, 130, 700, 50], 2, 64, 128),   # 512 compressed rows; a context shorter than the window
    (3, [3000, 5, 1, 2], 3, 64, 4),       # compression ratio 4: 750 compressed rows; tokens with no key at all
    (4, [2100, 4000], 1, 128, 4),         # 128 heads
    (5, [2100, 130, 9], 2, 16, 4),        # 16 heads: both tokens of a pair in one warp
    (6, [700, 3000], 3, 48, 128),         # 48 heads: a warp with heads of both tokens
])
def test_cfa_seeded_cases(seed, ori_seq, s1, nq, cmp_ratio):
    d = _as_cfa_inputs(helpers.gen_scfa_inputs(800 + seed, ori_seq, [s1] * len(ori_seq), nq=nq, cmp_ratio=cmp_ratio), s1)
    out = _run_cfa(d)
    ref = _cfa_oracle(d)
    _assert_attention_close(out, ref)
    assert torch.equal(out.float().abs().sum(-1) == 0, ref.float().abs().sum(-1) == 0)


def _run_win(d, graph=False):
    import pypto_b200
    from pypto_b200 import win_attention_impl as wa
    c = _cuda(d)
    mask = wa.get_mask(4, d["nq"], DEV, 128)
    fn = wa.sliding_win_atten_graph if graph else wa.deepseekv4_win_atten
    out = fn(c["q"], c["ori_block_table"], c["ori_kv"], c["seqused_kv"], c["atten_sink"], d["win_size"], mask,
             c["actual_seq_q"])
    pypto_b200.check_status()
    assert out.shape == d["q"].shape
    return out.cpu()


def _win_oracle(d):
    return orc.win_attention(d["q"], d["ori_block_table"], d["ori_kv"], d["seqused_kv"], d["atten_sink"], d["win_size"],
                             d["actual_seq_q"])


def test_win_attention_reference_golden_fixture():
    g = helpers.load_win_golden()
    out = _run_win(g)
    _assert_attention_close(out, g["out"])
    _assert_attention_close(out, _win_oracle(g))
    assert torch.equal(_run_win(g, graph=True), out)


@pytest.mark.parametrize("seed,ori_seq,s1_list,nq,win", [
    (1, [8192] * 4, [2, 2, 2, 2], 64, 128),         # the reference's decode shape, 4 requests
    (2, [300, 129, 128, 7, 1], [5, 4, 1, 9, 3], 64, 128),   # ragged query counts; windows cut by the start of the context
    (3, [1000, 40], [2, 1], 128, 300),              # 128 heads; a window over more than two pages
    (4, [1, 2, 3, 200], [2, 2, 2, 7], 64, 128),     # paired tokens: the first of a pair without any key; an odd count
    (5, [500, 600], [2, 4], 32, 128),               # 32 heads, two tokens per CTA
    (6, [500, 3, 129], [2, 4, 3], 16, 128),         # 16 heads: both tokens of a pair in one warp
    (7, [260, 90], [3, 2], 48, 128),                # 48 heads: a warp with heads of both tokens
])
def test_win_attention_seeded_cases(seed, ori_seq, s1_list, nq, win):
    d = helpers.gen_scfa_inputs(900 + seed, ori_seq, s1_list, nq=nq, win_size=win)
    t = int(d["actual_seq_q"][-1])
    d = dict(d, q=d["q"].reshape(t, nq, 512), ori_kv=d["ori_kv"].reshape(-1, 128, 1, 512))
    out = _run_win(d)
    ref = _win_oracle(d)
    _assert_attention_close(out, ref)
    assert torch.equal(out.float().abs().sum(-1) == 0, ref.float().abs().sum(-1) == 0)


def test_cfa_and_win_attention_bad_arguments():
    from pypto_b200 import compress_flash_attention_impl as cfa
    from pypto_b200 import win_attention_impl as wa
    d = _as_cfa_inputs(helpers.gen_scfa_inputs(990, [600, 300], [2, 2]), 2)
    c = _cuda(d)
    args = [c["q"], c["cmp_kv"], c["atten_sink"], c["cmp_block_table"], c["seqused_kv"], c["ori_kv"], c["ori_block_table"]]
    with pytest.raises(ValueError):
        cfa.cfa_attention(c["q"].reshape(-1, 512), *args[1:])          # 2-D query
    with pytest.raises(ValueError):
        cfa.cfa_attention(args[0], c["cmp_kv"].reshape(-1, 512), *args[2:])   # 2-D cache
    with pytest.raises(ValueError):
        cfa.cfa_attention(c["q"][:3].contiguous(), *args[1:])          # tokens not a multiple of the batch
    with pytest.raises(ValueError):
        cfa.cfa_attention(*args, cmp_ratio=0)
    with pytest.raises(ValueError):
        cfa.cfa_attention(args[0], args[1], c["atten_sink"][:5].contiguous(), *args[3:])
    with pytest.raises(RuntimeError):
        cfa.cfa_attention(d["q"], *args[1:])                           # host tensor
    with pytest.raises(ValueError):
        wa.deepseekv4_win_atten(c["q"], c["ori_block_table"], c["ori_kv"], c["seqused_kv"], c["atten_sink"], 0, None,
                                c["actual_seq_q"])
    with pytest.raises(ValueError):
        wa.deepseekv4_win_atten(c["q"], c["ori_block_table"], c["ori_kv"], c["seqused_kv"], c["atten_sink"], 128, None,
                                None)


def _run_sa_antiquant(d, cache, entry="d", flat_out=False):
    import pypto_b200
    from pypto_b200 import sparse_attention_antiquant_impl as sa
    c = _cuda(d)
    shape = (d["b"] * d["s1"] * d["nq"], 512) if flat_out else (d["b"], d["s1"], d["nq"], 512)
    out = torch.full(shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    fn = {"d": sa.sparse_attention_antiquant_d, "p": sa.sparse_attention_antiquant_p,
          "d950": sa.sparse_attention_antiquant_d_950}[entry]
    fn(c["q_nope"], c["q_rope"], cache.to(DEV), c["topk_indices"], c["block_table"], c["act_seq"], out, d["nq"], 1,
       d["softmax_scale"], d.get("topk", 2048), 128, d["block_table"].shape[1], sa.SaTileShapeConfig())
    pypto_b200.check_status()
    return out.cpu().reshape(d["b"], d["s1"], d["nq"], 512)


def test_sa_antiquant_reference_golden_fixture():
    g = helpers.load_sa_antiquant_golden()
    out = _run_sa_antiquant(g, g["nope_cache"], flat_out=True)  # the reference test passes a [t*nq, 512] output
    _assert_attention_close(out, g["out"])
    _assert_attention_close(out, orc.sa_antiquant(g["q_nope"], g["q_rope"], g["nope_cache"], g["topk_indices"],
                                                  g["block_table"], g["act_seq"], g["nq"], g["softmax_scale"]))


@pytest.mark.parametrize("entry,act_seq,s1", [("d", [2600, 700, 15, 0], 2), ("p", [5000, 2049], 4), ("d950", [64, 2048], 1)])
def test_sa_antiquant_fused_rows_equal_split_arrays(entry, act_seq, s1):
    """The fused 656-byte row holds the same bytes as the three arrays: the two operators return the same bits."""
    from pypto_b200.sparse_attention_antiquant_impl import pack_cache_rows
    d = helpers.gen_sfa_inputs(300 + s1, act_seq, s1=s1, extra_blocks=1)
    cache = pack_cache_rows(d["k_nope"], d["k_rope"], d["k_scales"])
    kn, kr, sc = orc.unpack_cache_rows(cache)
    assert torch.equal(kn, d["k_nope"]) and torch.equal(kr, d["k_rope"]) and torch.equal(sc, d["k_scales"])
    fused = _run_sa_antiquant(d, cache, entry=entry)
    assert torch.equal(fused, _run_sfa(d))
    _assert_attention_close(fused, _sfa_oracle(d))


def test_sa_antiquant_rejects_bad_arguments():
    from pypto_b200 import sparse_attention_antiquant_impl as sa
    d = helpers.gen_sfa_inputs(9, [300], s1=1)
    c = _cuda(d)
    out = torch.empty((1, 1, 128, 512), dtype=torch.bfloat16, device=DEV)
    cache = sa.pack_cache_rows(c["k_nope"], c["k_rope"], c["k_scales"])
    with pytest.raises(ValueError):  # wrong row width
        sa.sparse_attention_antiquant_d(c["q_nope"], c["q_rope"], cache[:, :640].contiguous(), c["topk_indices"],
                                        c["block_table"], c["act_seq"], out, 128, 1, 0.04, 2048, 128,
                                        d["block_table"].shape[1], None)
    with pytest.raises(ValueError):  # more than one KV head
        sa.sparse_attention_antiquant_d(c["q_nope"], c["q_rope"], cache, c["topk_indices"], c["block_table"],
                                        c["act_seq"], out, 128, 2, 0.04, 2048, 128, d["block_table"].shape[1], None)


@pytest.mark.parametrize("entry", ["d", "p", "d950"])
def test_sfa_config0_seeded_vs_oracle(entry):
    g = torch.Generator().manual_seed(1000)
    act = torch.randint(2048, 8193, (4,), generator=g).tolist()
    d = helpers.gen_sfa_inputs(1000, act, s1=1)
    _assert_attention_close(_run_sfa(d, entry=entry), _sfa_oracle(d))


@pytest.mark.parametrize("act_seq,s1", [([15, 666, 2048, 2049], 1), ([1, 33, 5000], 2), ([2047, 100], 4),
                                        ([0, 300], 1)])
def test_sfa_ragged_edges_vs_oracle(act_seq, s1):
    d = helpers.gen_sfa_inputs(77 + s1, act_seq, s1=s1, extra_blocks=2)
    _assert_attention_close(_run_sfa(d), _sfa_oracle(d))


@pytest.mark.parametrize("seed,act_seq,s1,scale_mul", [(1000, [5000, 3000], 1, 1.0), (1001, [2049, 77, 4000], 2, 1.0),
                                                       (1002, [6000], 2, 6.0)])
def test_sfa_holds_to_its_own_online_order_tightly(seed, act_seq, s1, scale_mul):
    """Against the oracle's emulation of the kernel's OWN order of operations (64-key tiles, reference maximum raised
    only past 2^8, P rounded to bf16 before P V) the output may differ in the last bf16 bit of at most 0.5 % of the
    elements under the reference's strict rule (atol 1e-4, rtol 5e-3) -- the differences left are fp32 summation
    order and the hardware exponential; measured 0.01-0.05 %.  A wrong or missing rescale of O or of the row sum fails this by a wide
    margin, where the 15 % allowance against the reference's order would only see a shifted fraction.  The third
    case has a softmax scale six times the model's, so that new maxima keep arriving and the rescale path runs."""
    d = helpers.gen_sfa_inputs(seed, act_seq, s1=s1)
    d["softmax_scale"] = d["softmax_scale"] * scale_mul
    out = _run_sfa(d, kv_splits=1)
    own = orc.sfa_quant_online(d["q_nope"], d["q_rope"], d["k_nope"], d["k_rope"], d["k_scales"], d["topk_indices"],
                               d["block_table"], d["act_seq"], d["nq"], d["softmax_scale"])
    strict = orc.reference_compare_count(out, own, 1e-4, 5e-3)
    ref = _sfa_oracle(d)
    print(f"[attention] vs own order: {strict / out.numel():.4f} outside the strict rule; own order vs reference order: "
          f"{orc.reference_compare_count(own, ref, 1e-4, 5e-3) / out.numel():.4f}")
    assert strict <= 0.005 * out.numel(), strict / out.numel()
    assert torch.allclose(out.float(), own.float(), rtol=1e-2, atol=2e-3)


@pytest.mark.parametrize("nq,topk,act_seq", [(64, 2048, [2600, 90]), (128, 512, [3000, 300]), (128, 1024, [1024, 5000]),
                                             (64, 1024, [700])])
def test_sfa_other_head_counts_and_selection_sizes(nq, topk, act_seq):
    """64 heads fill half of the 128-row tile; a smaller top-k shortens every index row."""
    d = helpers.gen_sfa_inputs(40 + nq + topk, act_seq, s1=2, nq=nq, topk=topk)
    _assert_attention_close(_run_sfa(d), _sfa_oracle(d))


@pytest.mark.parametrize("nq,act_seq,s1", [(16, [2600, 90], 2), (48, [700], 3), (1, [300], 1), (96, [2100], 2)])
def test_sfa_head_counts_below_the_tile(nq, act_seq, s1):
    """Fewer than 128 heads: the heads of a token are the first rows of the 128-row tile, the rest idle."""
    d = helpers.gen_sfa_inputs(140 + nq, act_seq, s1=s1, nq=nq)
    _assert_attention_close(_run_sfa(d), _sfa_oracle(d))
    _assert_attention_close(_run_sfa(d, kv_splits=3), _sfa_oracle(d))


def test_sfa_negative_index_inside_prefix_is_skipped():
    d = helpers.gen_sfa_inputs(5, [3000], s1=1)
    d["topk_indices"][0, 10:200] = -1
    _assert_attention_close(_run_sfa(d), _sfa_oracle(d))


@pytest.mark.parametrize("splits", [1, 2, 5, 16])
def test_sfa_kv_split_invariance(splits):
    d = helpers.gen_sfa_inputs(11, [5000, 700], s1=2)
    ref = _sfa_oracle(d)
    _assert_attention_close(_run_sfa(d, kv_splits=splits), ref)


def test_sfa_full_size_properties_batch64_ctx64k():
    # BASELINE shapes (batch 64, 64K context, s1=2): the oracle is checked on sampled tokens, the rest
    # through order-independence (softmax attention does not depend on the order of the selected keys).
    b, s1, ctx = 64, 2, 65536
    g = torch.Generator(device=DEV).manual_seed(2)
    blocks = b * ctx // 128
    rows = blocks * 128
    k_nope = torch.randint(-127, 128, (rows, 512), generator=g, dtype=torch.int8, device=DEV)
    k_rope = torch.randn((rows, 64), generator=g, device=DEV).to(torch.bfloat16)
    k_scales = torch.rand((rows, 4), generator=g, device=DEV) * 0.019 + 0.001
    q_nope = torch.randn((b * s1 * 128, 512), generator=g, device=DEV).to(torch.bfloat16)
    q_rope = torch.randn((b * s1 * 128, 64), generator=g, device=DEV).to(torch.bfloat16)
    block_table = torch.randperm(blocks, generator=g, device=DEV).to(torch.int32).reshape(b, ctx // 128)
    act = torch.full((b,), ctx, dtype=torch.int32, device=DEV)
    idx = torch.stack([torch.randperm(ctx - 1, generator=g, device=DEV)[:2048] for _ in range(b * s1)]).to(torch.int32)
    from pypto_b200.sparse_flash_attention_quant_impl import sparse_flash_attention_quant_d as sfa_d
    import pypto_b200
    scale = 576 ** -0.5
    out1 = torch.empty((b, s1, 128, 512), dtype=torch.bfloat16, device=DEV)
    out2 = torch.empty_like(out1)
    sfa_d(q_nope, q_rope, k_nope, k_rope, k_scales, idx, block_table, act, out1, 128, 1, scale, 2048, 128, ctx // 128)
    idx2 = idx.flip(1).contiguous()
    sfa_d(q_nope, q_rope, k_nope, k_rope, k_scales, idx2, block_table, act, out2, 128, 1, scale, 2048, 128, ctx // 128)
    pypto_b200.check_status()
    assert not torch.isnan(out1.float()).any()
    assert torch.allclose(out1.float(), out2.float(), rtol=1e-2, atol=1e-2)
    # sampled oracle: gather the few rows the sampled tokens touch into a compact CPU cache
    for tok in (0, 77, 127):
        bi = tok // s1
        ids = idx[tok].long()
        phys = block_table[bi][ids // 128].long() * 128 + ids % 128
        sub = dict(q_nope=q_nope[tok * 128:(tok + 1) * 128].cpu(), q_rope=q_rope[tok * 128:(tok + 1) * 128].cpu(),
                   k_nope=k_nope[phys].cpu(), k_rope=k_rope[phys].cpu(), k_scales=k_scales[phys].cpu(),
                   topk_indices=torch.arange(2048, dtype=torch.int32).reshape(1, -1),
                   block_table=torch.arange(16, dtype=torch.int32).reshape(1, -1),
                   act_seq=torch.tensor([2048], dtype=torch.int32), b=1, s1=1, nq=128, softmax_scale=scale)
        ref = _sfa_oracle(sub)
        _assert_attention_close(out1[bi, tok % s1].cpu().reshape(1, 1, 128, 512), ref)


def test_sfa_rejects_bad_arguments():
    from pypto_b200.sparse_flash_attention_quant_impl import sparse_flash_attention_quant_d as sfa_d
    d = _cuda(helpers.gen_sfa_inputs(1, [300], s1=1))
    out = torch.empty((1, 1, 128, 512), dtype=torch.bfloat16, device=DEV)
    args = [d["q_nope"], d["q_rope"], d["k_nope"], d["k_rope"], d["k_scales"], d["topk_indices"], d["block_table"],
            d["act_seq"], out, 128, 1, d["softmax_scale"], 2048, 128, d["block_table"].shape[1], None]
    bad = list(args)
    bad[0] = d["q_nope"].float()
    with pytest.raises(ValueError):
        sfa_d(*bad)
    bad = list(args)
    bad[2] = d["k_nope"].t()
    with pytest.raises(ValueError):
        sfa_d(*bad)
    bad = list(args)
    bad[5] = d["topk_indices"].cpu()
    with pytest.raises(RuntimeError):
        sfa_d(*bad)


# --------------------------------------------------------------------------------------------------
# indexer prolog
# --------------------------------------------------------------------------------------------------
def _run_prolog(inp, eps=1e-6):
    import pypto_b200
    from pypto_b200 import lightning_indexer_prolog_quant_impl as pl
    c = _cuda(inp)
    t = inp["token_x"].shape[0]
    q_int8 = torch.zeros((t, 64, 128), dtype=torch.int8, device=DEV)
    q_scale = torch.zeros((t, 64, 1), dtype=torch.float16, device=DEV)
    weights = torch.zeros((t, 64), dtype=torch.float16, device=DEV)
    kc, ksc = c["idx_k_cache"].clone(), c["idx_k_scale_cache"].clone()
    pl.lightning_indexer_prolog_quant(
        c["token_x"], c["q_norm"], c["q_norm_scale"], c["w_idx_qb"], c["w_idx_qb_scale"], c["w_idx_k"],
        c["w_idx_proj"], c["layer_norm_gamma"], c["layer_norm_beta"], c["cos_idx_rope"], c["sin_idx_rope"],
        c["hadamard_q"], c["hadamard_k"], kc, ksc, c["idx_k_cache_index"], q_int8, q_scale, kc, ksc, weights,
        pl.IndexerPrologQuantConfigs(), pl.IndexerPrologQuantAttr(eps=eps))
    pypto_b200.check_status()
    return q_int8.cpu(), q_scale.cpu(), kc.cpu(), ksc.cpu(), weights.cpu()


def _assert_prolog_close(got, ref, cache_index):
    q_i8, q_s, kc, ksc, w = got
    rq_i8, rq_s, rkc, rksc, rw = ref
    assert (q_i8.int() - rq_i8.reshape(q_i8.shape).int()).abs().max() <= 1
    assert (q_i8 != rq_i8.reshape(q_i8.shape)).float().mean() < 0.02
    assert torch.allclose(q_s.float().reshape(-1), rq_s.float().reshape(-1), atol=2.5e-5, rtol=2e-3)
    assert (kc.int() - rkc.int()).abs().max() <= 1
    assert torch.allclose(ksc.float(), rksc.float(), atol=2.5e-5, rtol=2e-3)
    assert torch.allclose(w.float(), rw.float().reshape(w.shape), atol=2.5e-5, rtol=4e-3)
    # untouched cache rows are bit-identical
    mask = torch.ones(kc.reshape(-1, 128).shape[0], dtype=torch.bool)
    mask[cache_index] = False
    assert torch.equal(kc.reshape(-1, 128)[mask], rkc.reshape(-1, 128)[mask])


def test_prolog_reference_golden_fixture():
    g = helpers.load_prolog_golden()
    inp = helpers.prolog_reference_inputs(g["seed"], g["b"], g["s1"], g["s2"])
    got = _run_prolog(inp)
    _assert_prolog_close(got, (g["q_int8"], g["q_scale"], g["k_cache"], g["k_scale_cache"], g["weights"]),
                         inp["idx_k_cache_index"])


@pytest.mark.parametrize("t", [1, 16, 37])
def test_prolog_config1_distributions_vs_oracle(t):
    g = torch.Generator().manual_seed(1001 + t)
    bf = torch.bfloat16
    x = torch.randn((t, 7168), generator=g).to(bf)
    qr = torch.randn((t, 1536), generator=g)
    amax = qr.abs().amax(-1, keepdim=True)
    q_norm = torch.round(qr * (127 / amax)).to(torch.int8)
    q_norm_scale = (amax / 127).float()
    wq = torch.randn((1536, 8192), generator=g) * 0.02
    wamax = wq.abs().amax(0, keepdim=True)
    w_qb = torch.round(wq * (127 / wamax)).to(torch.int8)
    w_qb_scale = (wamax / 127).reshape(8192, 1).float()
    wk = (torch.randn((7168, 128), generator=g) * 0.02).to(bf)
    w_proj = (torch.randn((7168, 64), generator=g) * 0.02).to(bf)
    ang = torch.rand((t, 64), generator=g) * 2 * math.pi
    had = torch.ones((1, 1))
    while had.shape[0] < 128:
        had = torch.cat([torch.cat([had, had], 1), torch.cat([had, -had], 1)], 0)
    had = (had / math.sqrt(128)).to(bf)
    nblk = 8
    inp = {
        "token_x": x, "q_norm": q_norm, "q_norm_scale": q_norm_scale, "w_idx_qb": w_qb, "w_idx_qb_scale": w_qb_scale,
        "w_idx_k": wk, "w_idx_proj": w_proj, "layer_norm_gamma": (1 + 0.1 * torch.randn(128, generator=g)).to(bf),
        "layer_norm_beta": (0.1 * torch.randn(128, generator=g)).to(bf), "cos_idx_rope": torch.cos(ang).to(bf),
        "sin_idx_rope": torch.sin(ang).to(bf), "hadamard_q": had, "hadamard_k": had,
        "idx_k_cache": torch.randint(-127, 128, (nblk, 128, 1, 128), generator=g, dtype=torch.int8),
        "idx_k_scale_cache": (torch.rand((nblk, 128, 1, 1), generator=g) * 0.02).to(torch.float16),
        "idx_k_cache_index": torch.randperm(nblk * 128, generator=g)[:t].to(torch.int64),
    }
    ref = orc.indexer_prolog(inp["token_x"], inp["q_norm"], inp["q_norm_scale"], inp["w_idx_qb"], inp["w_idx_qb_scale"],
                             inp["w_idx_k"], inp["w_idx_proj"], inp["layer_norm_gamma"], inp["layer_norm_beta"],
                             inp["cos_idx_rope"], inp["sin_idx_rope"], inp["hadamard_q"], inp["hadamard_k"],
                             inp["idx_k_cache"], inp["idx_k_scale_cache"], inp["idx_k_cache_index"])
    _assert_prolog_close(_run_prolog(inp), ref, inp["idx_k_cache_index"])


# --------------------------------------------------------------------------------------------------
# DeepSeek-V4 indexer prolog (query path + head weights)
# --------------------------------------------------------------------------------------------------
def _run_prolog_v4(inp, entry="npu"):
    import pypto_b200
    from pypto_b200 import lightning_indexer_prolog_quant_v4_impl as pv4
    c = _cuda(inp)
    args = [c[k] for k in ("qr", "idx_wq_b", "x", "weights_proj", "cos", "sin", "hadamard", "qr_scale", "idx_wq_b_scale")]
    if entry == "npu":
        q, w, qs = pv4.npu_quant_lightning_indexer_prolog(*args)
    else:
        t = inp["qr"].shape[0]
        q = torch.zeros((t, 64 * 128), dtype=torch.int8, device=DEV)      # the operator's table lists q as 2-D
        w = torch.zeros((t, 64), dtype=torch.float16, device=DEV)
        qs = torch.zeros((t, 64), dtype=torch.float16, device=DEV)
        assert pv4.quant_lightning_indexer_prolog_kernel(*args, q, w, qs, pv4.IndexerPrologQuantConfig()) is None
        q = q.reshape(t, 64, 128)
    pypto_b200.check_status()
    return q.cpu(), w.cpu(), qs.cpu()


def _assert_prolog_v4_close(got, ref):
    q, w, qs = got
    rq, rw, rqs = ref
    assert (q.int() - rq.int()).abs().max() <= 1
    assert (q != rq).float().mean() < 0.02
    # the reference's own tolerances (test_lightning_indexer_prolog_quant_v4.py:158-160)
    assert torch.allclose(w.float(), rw.float(), atol=1e-4, rtol=0.007825)
    assert torch.allclose(qs.float(), rqs.float(), atol=1e-4, rtol=0.007825)


def test_prolog_v4_reference_golden_fixture():
    g = helpers.load_prolog_v4_golden()
    inp = helpers.prolog_v4_reference_inputs(g["t"])
    got = _run_prolog_v4(inp)
    _assert_prolog_v4_close(got, (g["q"], g["weights"], g["q_scale"]))
    again = _run_prolog_v4(inp, entry="kernel")
    assert all(torch.equal(a, b) for a, b in zip(got, again))


@pytest.mark.parametrize("t,h", [(1, 4096), (37, 4096), (128, 4096), (200, 4096), (16, 7168), (5, 1000)])
def test_prolog_v4_seeded_vs_oracle(t, h):
    inp = helpers.gen_prolog_v4_inputs(1100 + t, t, h)
    got = _run_prolog_v4(inp)
    ref = orc.indexer_prolog_v4(**inp)
    _assert_prolog_v4_close(got, ref)
    # the int32 products are exact and the order of the roundings is the reference's: expect (near) bit equality
    assert (got[0] != ref[0]).float().mean() < 2e-3
    assert (got[2] != ref[2]).float().mean() < 2e-3


def test_prolog_v4_bad_arguments():
    from pypto_b200 import lightning_indexer_prolog_quant_v4_impl as pv4
    inp = helpers.gen_prolog_v4_inputs(1, 4)
    c = _cuda(inp)
    order = ("qr", "idx_wq_b", "x", "weights_proj", "cos", "sin", "hadamard", "qr_scale", "idx_wq_b_scale")

    def call(**over):
        a = dict(c, **over)
        return pv4.npu_quant_lightning_indexer_prolog(*[a[k] for k in order])

    with pytest.raises(ValueError):
        call(qr=c["qr"][:, :512].contiguous())
    with pytest.raises(ValueError):
        call(idx_wq_b=c["idx_wq_b"].to(torch.int32))
    with pytest.raises(ValueError):
        call(x=c["x"][:3].contiguous())
    with pytest.raises(ValueError):
        call(weights_proj=c["weights_proj"][:100].contiguous())
    with pytest.raises(ValueError):
        call(cos=c["cos"].float())
    with pytest.raises(ValueError):
        call(idx_wq_b_scale=c["idx_wq_b_scale"].reshape(-1))
    with pytest.raises(RuntimeError):
        call(hadamard=inp["hadamard"])
    call()


# --------------------------------------------------------------------------------------------------
# --------------------------------------------------------------------------------------------------
# DeepSeek-V4 MLA prolog (q / kv / qr) and its hand-over to the V4 indexer prolog
# --------------------------------------------------------------------------------------------------
def _run_mla_v4(inp, entry="in"):
    import pypto_b200
    from pypto_b200 import mla_prolog_quant_v4_impl as m4
    c = _cuda(inp)
    if entry == "in":
        out = m4.mla_prolog_v4_in(c["x"], c["wq_a"], c["wq_b"], c["w_kv"], c["cos"], c["sin"], c["gamma_cq"],
                                  c["gamma_ckv"], c["wq_b_scale"])
    else:
        t, heads = inp["x"].shape[0], inp["wq_b"].shape[1] // 512
        q = torch.zeros((t, heads, 512), dtype=torch.bfloat16, device=DEV)
        kv = torch.zeros((t, 512), dtype=torch.bfloat16, device=DEV)
        qr = torch.zeros((t, 1024), dtype=torch.int8, device=DEV)
        qs = torch.zeros((t, 1), dtype=torch.float32, device=DEV)
        assert m4.mla_prolog_v4(c["x"], c["wq_a"], c["wq_b"], c["w_kv"], c["gamma_cq"], c["gamma_ckv"], c["cos"], c["sin"],
                                c["wq_b_scale"], q, kv, qr, qs, m4.MlaPrologV4Attrs(eps=1e-6), m4.MlaPrologV4Configs(),
                                m4.MlaTileConfigs()) is None
        out = (q, kv, qr, qs)
    pypto_b200.check_status()
    return tuple(o.cpu() for o in out)


def _mla_v4_oracle(inp, qr_override=None):
    return orc.mla_prolog_v4(inp["x"], inp["wq_a"], inp["wq_b"], inp["w_kv"], inp["gamma_cq"], inp["gamma_ckv"],
                             inp["cos"], inp["sin"], inp["wq_b_scale"])


def _assert_mla_v4_close(got, ref, inp):
    q, kv, qr, qs = got
    rq, rkv, rqr, rqs = ref
    # the reference's own tolerances (test_mla_prolog_quant_v4.py:344-350): q / kv atol 1e-4 rtol 2^-7 with 0.5 % of
    # the elements allowed outside, qr within one step, qr_scale atol 2.5e-5 rtol 5e-3
    assert (qr.int() - rqr.int()).abs().max() <= 1
    assert (qr != rqr).float().mean() < 0.02
    assert torch.allclose(qs, rqs, atol=2.5e-5, rtol=0.005)
    assert torch.allclose(kv.float(), rkv.float(), atol=1e-4, rtol=0.0078125) or \
        orc.reference_compare_count(kv, rkv, 1e-4, 0.0078125) <= 0.005 * kv.numel()
    # q depends on qr: where the library GEMM's summation order flips a last bit of qr, q moves by up to the weight
    # of one quantisation step; judge q against the oracle run on the device's own qr (tight), and against the
    # reference value with the reference's outlier allowance
    x, heads = inp["x"], inp["wq_b"].shape[1] // 512
    q_b = torch.matmul(qr.to(torch.int32), inp["wq_b"].to(torch.int32)).to(torch.float32) * qs
    q_b = (q_b * inp["wq_b_scale"].reshape(1, -1)).reshape(x.shape[0], heads, 512)
    qn = (q_b / torch.sqrt((q_b * q_b * (1.0 / 512)).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    q_own = torch.cat([qn[:, :, :-64], orc.rope_interleaved_inverse(qn[:, :, -64:], inp["cos"], -inp["sin"])], dim=-1)
    assert orc.reference_compare_count(q, q_own, 1e-4, 0.0078125) <= 0.001 * q.numel()
    assert orc.reference_compare_count(q, rq, 1e-4, 0.0078125) <= 0.02 * q.numel()


def test_mla_v4_reference_golden_fixture():
    g = helpers.load_mla_v4_golden()
    inp = helpers.mla_v4_reference_inputs(g["t"])
    got = _run_mla_v4(inp)
    _assert_mla_v4_close(got, (g["q"], g["kv"], g["qr"], g["qr_scale"]), inp)
    again = _run_mla_v4(inp, entry="kernel")
    assert all(torch.equal(a, b) for a, b in zip(got, again))


@pytest.mark.parametrize("t,heads,h", [(1, 64, 4096), (37, 64, 4096), (128, 64, 4096), (20, 8, 1024)])
def test_mla_v4_seeded_vs_oracle(t, heads, h):
    inp = helpers.gen_mla_v4_inputs(1200 + t, t, heads, h)
    _assert_mla_v4_close(_run_mla_v4(inp), _mla_v4_oracle(inp), inp)


def test_mla_v4_feeds_the_v4_indexer_prolog():
    """qr / qr_scale of the MLA prolog are the first inputs of the indexer prolog: chain both on the device and compare
    with the oracle chain run on the device's qr."""
    t = 9
    m = helpers.gen_mla_v4_inputs(1300, t)
    p = helpers.gen_prolog_v4_inputs(1301, t)
    q, kv, qr, qs = _run_mla_v4(m)
    p = dict(p, qr=qr, qr_scale=qs, x=m["x"], cos=m["cos"], sin=m["sin"])
    _assert_prolog_v4_close(_run_prolog_v4(p), orc.indexer_prolog_v4(**p))


def _run_mla_v4_bf16(inp, entry="in"):
    import pypto_b200
    from pypto_b200 import mla_prolog_v4_impl as m4
    c = _cuda(inp)
    if entry == "in":
        out = m4.mla_prolog_v4_in(c["x"], c["wq_a"], c["wq_b"], c["w_kv"], c["cos"], c["sin"], c["gamma_cq"], c["gamma_ckv"])
    else:
        t, heads = inp["x"].shape[0], inp["wq_b"].shape[1] // 512
        q = torch.zeros((t, heads, 512), dtype=torch.bfloat16, device=DEV)
        kv = torch.zeros((t, 512), dtype=torch.bfloat16, device=DEV)
        qr = torch.zeros((t, 1024), dtype=torch.bfloat16, device=DEV)
        assert m4.mla_prolog_v4(c["x"], c["wq_a"], c["wq_b"], c["w_kv"], c["gamma_cq"], c["gamma_ckv"], c["cos"], c["sin"],
                                q, kv, qr, m4.MlaPrologV4Attrs(), m4.MlaPrologV4Configs()) is None
        out = (q, kv, qr)
    pypto_b200.check_status()
    return tuple(o.cpu() for o in out)


def _assert_mla_v4_bf16_close(got, ref, inp):
    q, kv, qr = got
    rq, rkv, rqr = ref
    # the reference's rule for all three outputs (test_mla_prolog_v4.py:309-313): atol 1e-4, rtol 2^-7, 0.5 % of the
    # elements may fall outside.  A last-bit difference of the bf16 GEMM results (another summation order) is one
    # bf16 step = 2^-8 relative, inside the rule; q is two GEMMs deep, so it is also judged from the device's own qr.
    for name, a, b in (("kv", kv, rkv), ("qr", qr, rqr)):
        bad = orc.reference_compare_count(a, b, 1e-4, 0.0078125)
        assert bad <= 0.005 * a.numel(), f"{name}: {bad} of {a.numel()} outside the reference's rule"
    heads = inp["wq_b"].shape[1] // 512
    qb = torch.matmul(qr, inp["wq_b"]).reshape(qr.shape[0], heads, 512).float()
    qn = (qb / torch.sqrt((qb * qb * (1.0 / 512)).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    q_own = torch.cat([qn[:, :, :-64], orc.rope_interleaved_inverse(qn[:, :, -64:], inp["cos"], -inp["sin"])], dim=-1)
    assert orc.reference_compare_count(q, q_own, 1e-4, 0.0078125) <= 0.005 * q.numel()
    assert orc.reference_compare_count(q, rq, 1e-4, 0.0078125) <= 0.03 * q.numel()
    assert torch.allclose(q.float(), rq.float(), atol=0.02, rtol=0.05)


def test_mla_v4_bf16_reference_golden_fixture():
    g = helpers.load_mla_v4_bf16_golden()
    inp = helpers.mla_v4_bf16_reference_inputs(g["t"])
    got = _run_mla_v4_bf16(inp)
    _assert_mla_v4_bf16_close(got, (g["q"], g["kv"], g["qr"]), inp)
    again = _run_mla_v4_bf16(inp, entry="kernel")
    assert all(torch.equal(a, b) for a, b in zip(got, again))


@pytest.mark.parametrize("t,heads,h", [(1, 64, 4096), (37, 64, 4096), (128, 64, 4096), (20, 8, 1024)])
def test_mla_v4_bf16_seeded_vs_oracle(t, heads, h):
    inp = helpers.gen_mla_v4_inputs(1400 + t, t, heads, h)
    inp = dict(inp, wq_b=(inp["wq_b"].float() * inp["wq_b_scale"]).to(torch.bfloat16))
    ref = orc.mla_prolog_v4_bf16(inp["x"], inp["wq_a"], inp["wq_b"], inp["w_kv"], inp["gamma_cq"], inp["gamma_ckv"],
                                 inp["cos"], inp["sin"])
    _assert_mla_v4_bf16_close(_run_mla_v4_bf16(inp), ref, inp)


def test_mla_v4_bad_arguments():
    from pypto_b200 import mla_prolog_quant_v4_impl as m4
    inp = helpers.gen_mla_v4_inputs(5, 3, heads=4, h=512)
    c = _cuda(inp)
    order = ("x", "wq_a", "wq_b", "w_kv", "cos", "sin", "gamma_cq", "gamma_ckv", "wq_b_scale")

    def call(**over):
        a = dict(c, **over)
        return m4.mla_prolog_v4_in(*[a[k] for k in order])

    with pytest.raises(ValueError):
        call(x=c["x"].float())
    with pytest.raises(ValueError):
        call(wq_a=c["wq_a"][:, :512].contiguous())
    with pytest.raises(ValueError):
        call(wq_b=c["wq_b"][:, :700].contiguous())
    with pytest.raises(ValueError):
        call(cos=c["cos"][:2].contiguous())
    with pytest.raises(ValueError):
        call(wq_b_scale=c["wq_b_scale"][:, :100].contiguous())
    with pytest.raises(RuntimeError):
        call(gamma_cq=inp["gamma_cq"])
    q, kv, qr, qs = call()
    assert q.shape == (3, 4, 512) and kv.shape == (3, 512) and qr.shape == (3, 1024) and qs.shape == (3, 1)


# --------------------------------------------------------------------------------------------------
# DeepSeek-V4 hyper-connection pre-mix
# --------------------------------------------------------------------------------------------------
def _run_hc_pre(inp, entry="npu", iters=20, eps=1e-6):
    import pypto_b200
    from pypto_b200 import hc_pre_impl as hp
    c = _cuda(inp)
    if entry == "npu":
        out = hp.npu_hc_pre(c["x"], c["hc_fn"], c["hc_scale"], c["hc_base"], 4, iters, eps)
    else:
        t = inp["x"].shape[0]
        y = torch.zeros((t, 4096), dtype=torch.bfloat16, device=DEV)
        post = torch.zeros((t, 4), dtype=torch.float32, device=DEV)
        comb = torch.zeros((t, 4, 4), dtype=torch.float32, device=DEV)
        fn = hp.hc_pre_kernel if entry == "kernel" else hp.hc_pre_kernel_prefill
        assert fn(c["x"], c["hc_fn"], c["hc_scale"], c["hc_base"], y, post, comb, 4, iters, eps) is None
        out = (y, post, comb)
    pypto_b200.check_status()
    return tuple(o.cpu() for o in out)


def _assert_hc_pre_close(got, ref):
    # the reference's own tolerances (test_hc_pre.py:203-208)
    y, post, comb = got
    ry, rpost, rcomb = ref
    assert orc.reference_compare_count(y, ry, 1e-4, 0.0078125) <= 0.005 * y.numel()
    assert torch.allclose(post, rpost, atol=2.5e-5, rtol=0.005)
    assert torch.allclose(comb, rcomb, atol=2.5e-5, rtol=0.005)


def test_hc_pre_reference_golden_fixture():
    g = helpers.load_hc_pre_golden()
    inp = helpers.hc_pre_reference_inputs(g["t"])
    got = _run_hc_pre(inp)
    _assert_hc_pre_close(got, (g["y"], g["post"], g["comb"]))
    for entry in ("kernel", "prefill"):
        assert all(torch.equal(a, b) for a, b in zip(got, _run_hc_pre(inp, entry)))


@pytest.mark.parametrize("t,iters,eps", [(1, 20, 1e-6), (37, 20, 1e-6), (512, 20, 1e-6), (9, 1, 1e-6), (9, 3, 1e-3)])
def test_hc_pre_seeded_vs_oracle(t, iters, eps):
    inp = helpers.gen_hc_pre_inputs(1500 + t + iters, t)
    got = _run_hc_pre(inp, iters=iters, eps=eps)
    _assert_hc_pre_close(got, orc.hc_pre(**inp, iters=iters, hc_eps=eps))
    if iters == 20:  # converged Sinkhorn: doubly stochastic
        assert torch.allclose(got[2].sum(-2), torch.ones(t, 4), atol=1e-4)


def test_hc_pre_bad_arguments():
    from pypto_b200 import hc_pre_impl as hp
    inp = helpers.gen_hc_pre_inputs(7, 2)
    c = _cuda(inp)
    with pytest.raises(ValueError):
        hp.npu_hc_pre(c["x"][:, :2].contiguous(), c["hc_fn"], c["hc_scale"], c["hc_base"])
    with pytest.raises(ValueError):
        hp.npu_hc_pre(c["x"], c["hc_fn"].to(torch.bfloat16), c["hc_scale"], c["hc_base"])
    with pytest.raises(ValueError):
        hp.npu_hc_pre(c["x"], c["hc_fn"], c["hc_scale"][:2].contiguous(), c["hc_base"])
    with pytest.raises(ValueError):
        hp.npu_hc_pre(c["x"], c["hc_fn"], c["hc_scale"], c["hc_base"], 8)
    with pytest.raises(ValueError):
        hp.npu_hc_pre(c["x"], c["hc_fn"], c["hc_scale"], c["hc_base"], 4, 0)
    with pytest.raises(RuntimeError):
        hp.npu_hc_pre(inp["x"], c["hc_fn"], c["hc_scale"], c["hc_base"])
    y, post, comb = hp.npu_hc_pre(c["x"], c["hc_fn"], c["hc_scale"], c["hc_base"])
    assert y.shape == (2, 4096) and post.shape == (2, 4) and comb.shape == (2, 4, 4)


# --------------------------------------------------------------------------------------------------
# DeepSeek-V4 KV compressor
# --------------------------------------------------------------------------------------------------
def _run_compressor(inp, kv_table=None, score_table=None):
    import pypto_b200
    from pypto_b200 import compressor_impl as cp
    c = _cuda(inp)
    kv_state, score_state = c["kv_state"].clone(), c["score_state"].clone()
    out, kv2, sc2 = cp.npu_compressor(c["x"], kv_state, score_state, c["table"] if kv_table is None else kv_table.to(DEV),
                                      c["table"] if score_table is None else score_table.to(DEV), c["sin"], c["cos"],
                                      c["wkv"], c["wgate"], c["ape"], c["weight"], c["hadamard"], c["start_pos"],
                                      inp["ratio"], 64, inp["rotate"])
    pypto_b200.check_status()
    assert kv2 is kv_state and sc2 is score_state          # updated in place and handed back
    return out.cpu(), kv_state.cpu(), score_state.cpu()


def _compressor_oracle(inp):
    kv_state, score_state = inp["kv_state"].clone(), inp["score_state"].clone()
    out = orc.compressor(inp["x"], kv_state, score_state, inp["table"], inp["table"], inp["sin"], inp["cos"], inp["wkv"],
                         inp["wgate"], inp["ape"], inp["weight"], inp["hadamard"], inp["start_pos"], inp["ratio"], 64,
                         inp["rotate"])
    return out, kv_state, score_state


def _assert_compressor_close(got, ref):
    out, kv_state, score_state = got
    rout, rkv, rsc = ref
    # states: fp32 GEMM rows (another summation order than the CPU's) -- relative 1e-4 of the row scale
    assert torch.allclose(kv_state, rkv, rtol=1e-4, atol=1e-4 * float(rkv.abs().max()))
    assert torch.allclose(score_state, rsc, rtol=1e-4, atol=1e-4 * float(rsc.abs().max()))
    # out: the reference's own rule (test_compressor.py: atol 1e-4, rtol 2^-7, 0.5 % of the elements may fall outside)
    assert orc.reference_compare_count(out, rout, 1e-4, 0.0078125) <= 0.005 * out.numel()
    assert torch.equal(out.float().abs().sum(-1) == 0, rout.float().abs().sum(-1) == 0)   # rows that did not compress


@pytest.mark.parametrize("name", list(helpers.COMPRESSOR_CASES))
def test_compressor_reference_golden_fixture(name):
    g = helpers.load_compressor_golden(name)
    inp = helpers.compressor_reference_inputs(name)
    out, kv_state, score_state = _run_compressor(inp)
    assert orc.reference_compare_count(out, g["out"], 1e-4, 0.0078125) <= 0.005 * out.numel()
    assert torch.allclose(kv_state.double().sum(-1), g["kv_state_sum"], rtol=1e-5, atol=1e-2)
    assert torch.allclose(score_state.double().sum(-1), g["score_state_sum"], rtol=1e-5, atol=1e-2)
    _assert_compressor_close((out, kv_state, score_state), _compressor_oracle(inp))


@pytest.mark.parametrize("ratio,rotate,d,starts,s1", [
    (4, False, 512, [3, 4, 7, 8, 123, 124, 127, 128, 0], 1),       # every residue; windows that span two pages
    (4, False, 512, [0, 1, 5, 250], 4),                             # four tokens per request: two compressions in one call
    (128, False, 512, [127, 255, 383, 100], 1),
    (128, False, 512, [125, 126, 254], 3),
    (4, True, 128, [255, 3, 4, 11], 2),
])
def test_compressor_seeded_vs_oracle(ratio, rotate, d, starts, s1):
    g = torch.Generator().manual_seed(1600 + ratio + d + s1)
    bf = torch.bfloat16
    b, coff, h = len(starts), (2 if ratio == 4 else 1), 4096
    pages = 4
    perm = torch.randperm(b * pages, generator=g).to(torch.int32).reshape(b, pages)
    rows = min(b * s1, b * s1 // ratio + b)
    ang = torch.rand((rows, 32), generator=g) * 6.2831853
    inp = dict(
        x=torch.randn((b, s1, h), generator=g).to(bf), sin=torch.sin(ang).repeat_interleave(2, -1).to(bf),
        cos=torch.cos(ang).repeat_interleave(2, -1).to(bf), wkv=(torch.randn((coff * d, h), generator=g) * 0.02).to(bf),
        wgate=(torch.randn((coff * d, h), generator=g) * 0.02).to(bf), ape=torch.randn((ratio, coff * d), generator=g) * 0.5,
        weight=1 + 0.1 * torch.randn(d, generator=g), kv_state=torch.randn((b * pages, 128, coff * d), generator=g),
        score_state=torch.randn((b * pages, 128, coff * d), generator=g), table=perm,
        hadamard=(torch.randn((d, d), generator=g) * d ** -0.5).to(bf), start_pos=torch.tensor(starts, dtype=torch.int32),
        ratio=ratio, rotate=rotate, d=d)
    _assert_compressor_close(_run_compressor(inp), _compressor_oracle(inp))


def test_compressor_bad_arguments_and_bad_pages():
    import pypto_b200
    from pypto_b200 import compressor_impl as cp
    inp = helpers.compressor_reference_inputs("r4")
    c = _cuda(inp)

    def call(**over):
        a = dict(c, **over)
        return cp.npu_compressor(a["x"], a["kv_state"].clone(), a["score_state"].clone(), a["table"], a["table"], a["sin"],
                                 a["cos"], a["wkv"], a["wgate"], a["ape"], a["weight"], a["hadamard"], a["start_pos"],
                                 over.get("ratio", 4), over.get("rope", 64), over.get("rotate", False))

    with pytest.raises(ValueError):
        call(ratio=8)
    with pytest.raises(ValueError):
        call(rope=32)
    with pytest.raises(ValueError):
        call(rotate=1)
    with pytest.raises(ValueError):
        call(x=c["x"].float())
    with pytest.raises(ValueError):
        call(ape=c["ape"][:2].contiguous())
    with pytest.raises(ValueError):
        call(start_pos=c["start_pos"].long())
    with pytest.raises(RuntimeError):
        call(weight=inp["weight"])
    bad = c["table"].clone()
    bad[0, 1] = 10 ** 6                                   # request 0 writes position 255 -> page slot 1
    call(table=bad)
    with pytest.raises(RuntimeError):
        pypto_b200.check_status()
    call(start_pos=torch.tensor([128 * 100, 2, 6, 9], dtype=torch.int32, device=DEV))   # past the table's last column
    with pytest.raises(RuntimeError):
        pypto_b200.check_status()
    call()
    pypto_b200.check_status()


# --------------------------------------------------------------------------------------------------
# fused MLA prolog + indexer prolog
# --------------------------------------------------------------------------------------------------
def _run_mla(inp, ip):
    """Runs the stand-alone MLA entry (for q_norm) and the fused entry on copies of the same caches."""
    import pypto_b200
    from pypto_b200 import mla_indexer_prolog_quant_impl as mla
    from pypto_b200 import mla_prolog_quant_impl as mlp
    from pypto_b200 import lightning_indexer_prolog_quant_impl as pl
    c, ci = _cuda(inp), _cuda(ip)
    t = inp["x"].shape[0]
    bf = torch.bfloat16
    scale = c["w_qb_scale"].reshape(-1, 1).contiguous()
    # stand-alone MLA prolog: exposes q_norm / q_norm_scale
    q_norm = torch.zeros((t, 1536), dtype=torch.int8, device=DEV)
    q_norm_scale = torch.zeros((t, 1), dtype=torch.float32, device=DEV)
    q_nope0 = torch.zeros((t, 128, 512), dtype=bf, device=DEV)
    q_rope0 = torch.zeros((t, 128, 64), dtype=bf, device=DEV)
    kv0, kr0, ks0 = c["kv_cache"].clone(), c["kr_cache"].clone(), c["ks_cache"].clone()
    mlp.mla_prolog_quant_d(c["x"], c["w_dq"], c["w_uqqr"], scale, c["w_uk"], c["w_dkvkr"], c["gamma_cq"], c["gamma_ckv"],
                           c["cos"], c["sin"], c["cache_index"], kv0, kr0, ks0, q_norm, q_norm_scale, q_nope0, q_rope0,
                           kv0, kr0, ks0, 1e-6, 1e-6, "PA_BSND", mlp.MlaTileConfig(), mlp.RopeTileShapeConfig())
    # fused entry
    q_nope = torch.zeros((t, 128, 512), dtype=bf, device=DEV)
    q_rope = torch.zeros((t, 128, 64), dtype=bf, device=DEV)
    kv, kr, ks = c["kv_cache"].clone(), c["kr_cache"].clone(), c["ks_cache"].clone()
    q_int8 = torch.zeros((t, 64, 128), dtype=torch.int8, device=DEV)
    q_scale = torch.zeros((t, 64, 1), dtype=torch.float16, device=DEV)
    weights = torch.zeros((t, 64), dtype=torch.float16, device=DEV)
    ikc, iksc = ci["idx_k_cache"].clone(), ci["idx_k_scale_cache"].clone()
    mla.mla_indexer_prolog_quant_d(
        c["x"], c["w_dq"], c["w_uqqr"], scale, c["w_uk"], c["w_dkvkr"], c["gamma_cq"],
        c["gamma_ckv"], c["cos"], c["sin"], c["cache_index"], kv, kr, ks, ci["w_idx_qb"], ci["w_idx_qb_scale"],
        ci["w_idx_k"], ci["w_idx_proj"], ci["layer_norm_gamma"], ci["layer_norm_beta"], ci["hadamard_q"],
        ci["hadamard_k"], ikc, iksc, q_nope, q_rope, kv, kr, ks, q_int8, q_scale, ikc, iksc, weights,
        1e-6, 1e-6, "PA_BSND", mla.MlaTileConfig(), pl.IndexerPrologQuantAttr(eps=1e-6), pl.IndexerPrologQuantConfigs(),
        mla.RopeTileShapeConfig())
    pypto_b200.check_status()
    # both entries run the same kernels on the same inputs: identical results
    for a, b in ((q_nope0, q_nope), (q_rope0, q_rope), (kv0, kv), (kr0, kr), (ks0, ks)):
        assert torch.equal(a, b)
    return dict(q_nope=q_nope.cpu(), q_rope=q_rope.cpu(), kv=kv.cpu(), kr=kr.cpu(), ks=ks.cpu(), q_int8=q_int8.cpu(),
                q_scale=q_scale.cpu(), weights=weights.cpu(), ikc=ikc.cpu(), iksc=iksc.cpu(), q_norm=q_norm.cpu(),
                q_norm_scale=q_norm_scale.cpu())


def _indexer_side_inputs(seed, t, nblk):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    return {
        "w_idx_qb": torch.randint(-128, 128, (1536, 8192), generator=g, dtype=torch.int8),
        "w_idx_qb_scale": (torch.rand((8192, 1), generator=g) * 2e-3 + 1e-4),
        "w_idx_k": (torch.randn((7168, 128), generator=g) * 0.02).to(bf),
        "w_idx_proj": (torch.randn((7168, 64), generator=g) * 0.02).to(bf),
        "layer_norm_gamma": torch.ones(128, dtype=bf), "layer_norm_beta": torch.zeros(128, dtype=bf),
        "hadamard_q": (torch.rand((128, 128), generator=g) * 2 - 1).to(bf),
        "hadamard_k": (torch.rand((128, 128), generator=g) * 2 - 1).to(bf),
        "idx_k_cache": torch.randint(-127, 128, (nblk, 128, 1, 128), generator=g, dtype=torch.int8),
        "idx_k_scale_cache": (torch.rand((nblk, 128, 1, 1), generator=g) * 0.02).to(torch.float16),
    }


def _check_mla(out, ref, ip, inp, ratio=0.005, scale_ratio=0.005):
    q_nope, q_rope, q_norm, q_norm_scale, kv, kr, ks = ref
    bad = []

    def points(name, got, want, atol, rtol, allowed):
        n = orc.reference_compare_count(got, want, atol, rtol)
        if n > allowed:
            bad.append(f"{name}: {n} of {want.numel()} elements outside atol={atol} rtol={rtol} (allowed {allowed:.1f})")

    def lsb(name, got, want, steps):
        d = int((got.int() - want.int()).abs().max())
        if d > steps:
            bad.append(f"{name}: max int8 difference {d} > {steps}")

    # the reference's own tolerances for the fused operator (deepseekv32_mla_indexer_prolog_quant.py:808-828);
    # `ratio` is its allowance of error points (0.5 % there)
    points("q_nope", out["q_nope"], q_nope, 0.005, 0.0078125, ratio * q_nope.numel())
    points("q_rope", out["q_rope"], q_rope, 0.005, 0.0078125, ratio * q_rope.numel())
    lsb("kv", out["kv"], kv, 1)
    points("kr", out["kr"], kr, 1e-4, 0.0078125, 0.005 * kr.numel())
    # a scale is 1/127 of a bf16 maximum: one bf16 step of that maximum is the resolution of the comparison
    points("k_scale", out["ks"], ks, 2.5e-5, 0.008, 0)
    lsb("q_norm", out["q_norm"], q_norm, 1)
    points("q_norm_scale", out["q_norm_scale"], q_norm_scale, 0, 0.008, 0)
    # tight: the oracle continued from the q_norm the device produced -- int32 GEMM, dequantisation and RoPE
    # are then exact, the w_uk projection differs only by the library's accumulation order
    x_nope, x_rope = orc.mla_prolog(inp["x"], inp["w_dq"], inp["w_uqqr"], inp["w_qb_scale"], inp["w_uk"], inp["w_dkvkr"],
                                    inp["gamma_cq"], inp["gamma_ckv"], inp["cos"], inp["sin"], inp["cache_index"],
                                    inp["kv_cache"], inp["kr_cache"], inp["ks_cache"],
                                    q_norm_in=(out["q_norm"], out["q_norm_scale"]))[:2]
    if not torch.equal(out["q_rope"], x_rope):
        bad.append(f"q_rope from the device q_norm: {(out['q_rope'] != x_rope).sum()} elements differ")
    points("q_nope from the device q_norm", out["q_nope"], x_nope, 0.005, 0.0078125, 0.0005 * x_nope.numel())
    ipargs = (ip["w_idx_qb"], ip["w_idx_qb_scale"], ip["w_idx_k"], ip["w_idx_proj"], ip["layer_norm_gamma"],
              ip["layer_norm_beta"], inp["cos"], inp["sin"], ip["hadamard_q"], ip["hadamard_k"], ip["idx_k_cache"],
              ip["idx_k_scale_cache"], inp["cache_index"])
    # indexer half, tight: the oracle fed with the q_norm the device produced
    iq, iqs, ikc, iksc, w = orc.indexer_prolog(inp["x"], out["q_norm"], out["q_norm_scale"], *ipargs)
    lsb("idx q_int8 (device q_norm)", out["q_int8"], iq.reshape(out["q_int8"].shape), 1)
    points("idx q_scale (device q_norm)", out["q_scale"].reshape(-1), iqs.reshape(-1), 2.5e-5, 2e-3, 0.001 * iqs.numel())
    lsb("idx k_int8", out["ikc"], ikc, 1)
    points("idx k_scale", out["iksc"], iksc, 2.5e-5, 2e-3, 0)
    points("idx weights", out["weights"], w.reshape(out["weights"].shape), 2.5e-5, 4e-3, 0.001 * w.numel())
    # indexer half, end to end: the oracle chain with the reference's tolerances (:825-829)
    iq, iqs, ikc, iksc, w = orc.indexer_prolog(inp["x"], q_norm, q_norm_scale, *ipargs)
    points("idx q_int8", out["q_int8"], iq.reshape(out["q_int8"].shape), 2, 0, ratio * iq.numel())
    points("idx q_scale", out["q_scale"].reshape(-1), iqs.reshape(-1), 2.5e-5, 0.006, max(1, scale_ratio * iqs.numel()))
    assert not bad, "\n".join(bad)


def test_mla_indexer_prolog_reference_golden_fixture():
    g = helpers.load_mla_golden()
    inp = helpers.mla_reference_inputs(g["seed"], g["b"], g["s1"], g["s2"])
    ip = _indexer_side_inputs(3, inp["x"].shape[0], inp["kv_cache"].shape[0])
    out = _run_mla(inp, ip)
    ref = (g["q_nope"], g["q_rope"], g["q_norm"], g["q_norm_scale"], g["kv_cache"], g["kr_cache"], g["ks_cache"])
    _check_mla(out, ref, ip, inp)


@pytest.mark.parametrize("t", [1, 37, 128])
def test_mla_indexer_prolog_seeded_vs_oracle(t):
    g = torch.Generator().manual_seed(500 + t)
    bf = torch.bfloat16
    nblk = 6
    u = lambda shape, a: ((torch.rand(shape, generator=g) * 2 - 1) * a)  # noqa: E731
    w_uqqr_f = u((1536, 128 * 192), 0.1)
    wamax = w_uqqr_f.abs().amax(0, keepdim=True)
    ang = torch.rand((t, 64), generator=g) * 2 * math.pi
    inp = dict(
        x=u((t, 7168), 1.0).to(bf), w_dq=u((7168, 1536), 0.1).to(bf), w_uqqr=torch.round(w_uqqr_f * (127 / wamax)).to(torch.int8),
        w_qb_scale=(wamax / 127).reshape(-1).float().contiguous(), w_uk=u((128, 128, 512), 0.1).to(bf),
        w_dkvkr=u((7168, 576), 0.1).to(bf), gamma_cq=u((1536,), 1.0).to(bf), gamma_ckv=u((512,), 1.0).to(bf),
        cos=torch.cos(ang).to(bf), sin=torch.sin(ang).to(bf),
        cache_index=torch.randperm(nblk * 128, generator=g)[:t].to(torch.int64),
        kv_cache=torch.randint(-127, 128, (nblk, 128, 1, 512), generator=g, dtype=torch.int8),
        kr_cache=u((nblk, 128, 1, 64), 1.0).to(bf), ks_cache=torch.rand((nblk, 128, 1, 4), generator=g) * 0.02)
    ip = _indexer_side_inputs(600 + t, t, nblk)
    ref = orc.mla_prolog(inp["x"], inp["w_dq"], inp["w_uqqr"], inp["w_qb_scale"], inp["w_uk"], inp["w_dkvkr"],
                         inp["gamma_cq"], inp["gamma_ckv"], inp["cos"], inp["sin"], inp["cache_index"], inp["kv_cache"],
                         inp["kr_cache"], inp["ks_cache"])
    # these value distributions are not the reference generator's: one-LSB differences of q_norm (library GEMM
    # accumulation order) move a few more elements past the reference tolerance, so allow 1.5 % error points;
    # the indexer's per-head scale is a maximum over 128 sums of those differences and moves with them (5 %)
    _check_mla(_run_mla(inp, ip), ref, ip, inp, ratio=0.015, scale_ratio=0.05)


# --------------------------------------------------------------------------------------------------
# decode loop with host I/O on separate streams
# --------------------------------------------------------------------------------------------------
def test_host_pipelined_decode_matches_serial_steps():
    """Six steps with two alternating sets of host activations through the three-stream loop give, step by step,
    the outputs of the serial host path (copy in, run, copy out on one stream)."""
    from pypto_b200 import synth
    from pypto_b200.decode_chain import HostPipelinedDecode, SparseDecodeStep
    w = synth.make_decode_workload([3000, 700, 2600, 129], 2, 77, DEV)
    step = SparseDecodeStep(w)
    step.enable_host_io()
    from pypto_b200.decode_chain import PackedTensors
    set_a = step.host_pack            # the step's activations as one pinned buffer
    g = torch.Generator().manual_seed(5)
    other = dict(set_a.views)
    for name in ("q_nope", "q_rope", "x"):
        other[name] = (torch.randn(other[name].shape, generator=g) * 0.5).to(other[name].dtype)
    set_b = PackedTensors(other, "cpu", pin=True)
    want = {}
    for tag, hs in (("a", set_a), ("b", set_b)):
        step.host_pack = hs
        want[tag] = step.step_from_host().clone()
        torch.cuda.synchronize()
        want[tag] = step.host_out.clone()
    assert not torch.equal(want["a"], want["b"])
    pipe = HostPipelinedDecode(step)
    outs = []
    for k in range(6):
        tag = "ab"[k % 2] if k < 4 else "ba"[k % 2]
        buf = pipe.submit(set_a if tag == "a" else set_b)
        if k >= 1:  # the output of the previous step may be read once its copy has completed
            pipe.out_done[(k - 1) & 1].synchronize()
            outs.append((prev_tag, pipe.host_out[(k - 1) & 1].clone()))
        prev_tag = tag
    pipe.drain()
    torch.cuda.synchronize()
    outs.append((prev_tag, buf.clone()))
    import pypto_b200
    pypto_b200.check_status()
    assert len(outs) == 6
    for tag, o in outs:
        assert torch.equal(o, want[tag])


def test_captured_step_matches_eager_step():
    """The step replayed from CUDA graphs (whole, per stage, and inside the host-pipelined loop) writes the same
    bits as the eager step."""
    import pypto_b200
    from pypto_b200 import synth
    from pypto_b200.decode_chain import HostPipelinedDecode, SparseDecodeStep
    w = synth.make_decode_workload([2500, 300, 4100], 2, 78, DEV)
    step = SparseDecodeStep(w)
    want = step.step().clone()
    want_topk = step.topk_res.clone()
    torch.cuda.synchronize()
    for per_stage in (False, True):
        step.capture(per_stage=per_stage)
        step.out.zero_()
        step.topk_res.zero_()
        got = step.replay()
        torch.cuda.synchronize()
        assert torch.equal(got, want) and torch.equal(step.topk_res, want_topk)
    step.enable_host_io()
    pipe = HostPipelinedDecode(step, use_graphs=True)
    bufs = [pipe.submit(step.host_pack) for _ in range(3)]
    pipe.drain()
    torch.cuda.synchronize()
    pypto_b200.check_status()
    assert torch.equal(bufs[-1], want.cpu()) and torch.equal(bufs[-2], want.cpu())


# --------------------------------------------------------------------------------------------------
# multi-step decode: every step appends its tokens to both caches and the next step sees them
# --------------------------------------------------------------------------------------------------
def test_decode_loop_appends_to_both_caches_across_pages():
    """Four decode steps of a small ragged batch through fused prolog -> indexer + top-k -> attention -> advance,
    replayed from ONE captured CUDA graph.  Request 1 crosses a page boundary between steps, request 2 inside a
    step.  After every step: the position state follows the reference's cache-index rule; exactly the rows of the
    step's tokens changed in both caches, to the oracle's values; the top-k (on the device's own prolog outputs and
    caches) and the attention (on the device's own queries, caches and top-k) match the oracle -- so the keys a step
    appends are scored and attended to by the steps after it."""
    import pypto_b200
    from pypto_b200 import synth
    from pypto_b200.decode_chain import FullDecodeStep
    ctx, s1, steps = [300, 126, 255], 2, 4
    w = synth.make_full_decode_workload(ctx, s1, s1 * steps, 41, DEV)
    step = FullDecodeStep(w)
    t = w.t
    cpu = lambda x: x.detach().cpu()  # noqa: E731
    wc = {k: cpu(v) for k, v in vars(w).items() if isinstance(v, torch.Tensor)}
    step.set_inputs(**synth.make_full_step_activations(t, 899, DEV))   # the capture's warm-up run uses other inputs
    step.capture()
    for k in range(steps):
        acts = synth.make_full_step_activations(t, 900 + k, "cpu")
        step.set_inputs(**acts)
        before = {n: cpu(getattr(w, n)).clone() for n in ("kv_cache", "kr_cache", "k_scale_cache", "idx_k", "idx_k_scale",
                                                          "act_seq", "cache_index")}
        step.graph.replay()
        pypto_b200.check_status()
        act, ci = before["act_seq"], before["cache_index"]
        assert act.tolist() == [c + k * s1 for c in ctx]
        assert torch.equal(ci, synth.cache_index_for(act, wc["block_table"], s1))
        # ---- position state after the step ---------------------------------------------------------------
        assert cpu(w.act_seq).tolist() == [c + (k + 1) * s1 for c in ctx]
        assert torch.equal(cpu(w.cache_index), synth.cache_index_for(cpu(w.act_seq), wc["block_table"], s1))
        # ---- caches: the oracle's rows at cache_index, every other row untouched ------------------------------
        q_nope, q_rope, q_norm, q_norm_scale, kv_ref, kr_ref, ks_ref = orc.mla_prolog(
            acts["x"], wc["w_dq"], wc["w_uq_qr"], wc["w_uq_qr_scale"], wc["w_uk"], wc["w_dkv_kr"], wc["gamma_cq"],
            wc["gamma_ckv"], acts["cos"], acts["sin"], ci, before["kv_cache"], before["kr_cache"], before["k_scale_cache"])
        _, _, ik_ref, iks_ref, _ = orc.indexer_prolog(
            acts["x"], q_norm, q_norm_scale, wc["w_qb"], wc["w_qb_scale"], wc["wk"], wc["w_proj"], wc["ln_gamma"],
            wc["ln_beta"], acts["cos"], acts["sin"], wc["hadamard"], wc["hadamard"], before["idx_k"],
            before["idx_k_scale"].reshape(-1, 128, 1), ci)
        kv, kr, ks = cpu(w.kv_cache), cpu(w.kr_cache), cpu(w.k_scale_cache)
        ik, iks = cpu(w.idx_k), cpu(w.idx_k_scale)
        rows = torch.zeros(kv.shape[0] * 128, dtype=torch.bool)
        rows[ci] = True
        for name, got, ref, old, width in (("kv", kv, kv_ref, before["kv_cache"], 512), ("kr", kr, kr_ref, before["kr_cache"], 64),
                                           ("ks", ks, ks_ref, before["k_scale_cache"], 4), ("ik", ik, ik_ref, before["idx_k"], 128),
                                           ("iks", iks, iks_ref.reshape(iks.shape), before["idx_k_scale"], 1)):
            g2, r2, o2 = got.reshape(-1, width), ref.reshape(-1, width), old.reshape(-1, width)
            assert torch.equal(g2[~rows], o2[~rows]), name          # no other row is touched
            assert not torch.equal(g2[rows], o2[rows]), name        # the step's rows were written
            if got.dtype == torch.int8:
                assert (g2[rows].int() - r2[rows].int()).abs().max() <= 1, name
            else:   # the reference's tolerances for these outputs; the rope rows may hold a few last-bit outliers
                bad = orc.reference_compare_count(g2[rows], r2[rows], 1e-4 if name == "kr" else 2.5e-5, 0.008)
                assert bad <= (0.02 * g2[rows].numel() if name == "kr" else 0), (name, bad)
        # ---- queries against the oracle's (the reference's tolerances for the fused operator) -----------------
        for name, got, ref in (("q_nope", cpu(step.q_nope), q_nope), ("q_rope", cpu(step.q_rope), q_rope)):
            assert orc.reference_compare_count(got, ref, 0.005, 0.0078125) <= 0.015 * ref.numel(), name
        # ---- indexer + top-k on the device's own prolog outputs and caches -----------------------------------------
        ref_idx, ref_scores = orc.lightning_indexer(cpu(step.q_int8), cpu(step.q_scale).reshape(-1, 64), ik,
                                                    iks.reshape(-1, 128, 1), cpu(step.weights), act, wc["block_table"], 2048,
                                                    return_scores=True)
        got_idx = cpu(step.topk_res)
        for tok in range(t):
            ok, nd, _ = orc.topk_sets_match(got_idx[tok, 0], ref_idx[tok, 0], ref_scores[tok // s1][tok % s1])
            assert ok, (k, tok, nd)
            eff = int(act[tok // s1]) - (s1 - 1 - tok % s1)      # fewer than 2048 keys: all of them, the newest included
            assert sorted(got_idx[tok, 0, :eff].tolist()) == list(range(eff)) and (got_idx[tok, 0, eff:] == -1).all()
        # ---- attention on the device's own queries, caches and top-k ------------------------------------------------
        ref_out = orc.sfa_quant(cpu(step.q_nope).reshape(-1, 512), cpu(step.q_rope).reshape(-1, 64), kv.reshape(-1, 512),
                                kr.reshape(-1, 64), ks.reshape(-1, 4), got_idx.reshape(-1, 2048), wc["block_table"], act, 128,
                                576 ** -0.5)
        _assert_attention_close(cpu(step.out), ref_out)


def test_decode_advance_reports_positions_beyond_the_page_table():
    import pypto_b200
    from pypto_b200.decode_chain import decode_advance
    bt = torch.tensor([[3, 1], [0, -1]], dtype=torch.int32, device=DEV)
    act = torch.tensor([254, 100], dtype=torch.int32, device=DEV)
    ci = torch.zeros(4, dtype=torch.int64, device=DEV)
    decode_advance(act, bt, ci, 2)                         # request 0: positions 254, 255 -> page 1 rows 126, 127
    pypto_b200.check_status()
    assert act.tolist() == [256, 102] and ci.tolist() == [128 + 126, 128 + 127, 100, 101]
    decode_advance(act, bt, ci, 2)                         # request 0 runs past its two pages
    with pytest.raises(RuntimeError, match="status"):
        pypto_b200.check_status()
    assert ci.tolist()[:2] == [-1, -1] and ci.tolist()[2:] == [102, 103]
    act[1] = 127
    decode_advance(act, bt, ci, 2)                         # request 1 steps onto a page that is not assigned
    with pytest.raises(RuntimeError, match="status"):
        pypto_b200.check_status()
    assert ci.tolist()[2:] == [127, -1]


def test_bounded_wait_runs_out_with_a_status_word_and_a_clean_return():
    """A device-side wait whose barrier never completes gives up after its cycle budget: status TIMEOUT with the
    wait's location id, the kernel returns, the context stays usable (nothing asynchronous is in flight in this
    diagnostic kernel; the production kernels use the same wait with a budget of about a second)."""
    import ctypes as C
    import time
    import pypto_b200
    from pypto_b200 import _lib, _runtime as rt
    lib = _lib.load()
    dev = torch.device(DEV)
    pypto_b200.check_status(dev)
    st = rt.status_word(dev)
    t0 = time.perf_counter()
    _lib.check(lib.dsv32_wait_selftest(C.c_void_p(st.data_ptr()), 200000, rt.stream_ptr(dev)), "wait selftest")
    with pytest.raises(RuntimeError, match="timed out"):
        pypto_b200.check_status(dev)
    assert time.perf_counter() - t0 < 5.0
    pypto_b200.check_status(dev)                          # cleared; the device still works
    x = torch.arange(10, device=DEV)
    assert int(x.sum()) == 45
    assert lib.dsv32_wait_selftest(None, 10, None) == -1 and lib.dsv32_wait_selftest(C.c_void_p(st.data_ptr()), -1, None) == -1
