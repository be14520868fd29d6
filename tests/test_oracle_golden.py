"""The CPU oracle against the fixtures produced by the unmodified reference goldens."""
import pytest
import torch

import helpers
from oracle import dsv32_oracle as orc


def test_kat_topk_ties_lower_index_first():
    kat = helpers.load_kat()["topk_ties"]
    idx = orc.topk_indices_ref(torch.tensor(kat["input"], dtype=torch.float32), kat["k"])
    assert idx.tolist() == kat["indices"]


def test_kat_paged_gather():
    kat = helpers.load_kat()["paged_gather"]
    params = torch.tensor([[10 * r + c for c in range(kat["cols"])] for r in range(kat["rows"])])
    got = orc.paged_gather(params, torch.tensor(kat["indices"]), torch.tensor(kat["page_table"]), kat["block_size"])
    assert got.tolist() == [params[r].tolist() for r in kat["expected_rows"]]


def test_sfa_oracle_matches_reference_golden():
    g = helpers.load_sfa_golden()
    out = orc.sfa_quant(g["q_nope"], g["q_rope"], g["k_nope"], g["k_rope"], g["k_scales"], g["topk_indices"],
                        g["block_table"], g["act_seq"], g["nq"], g["softmax_scale"])
    assert out.shape == g["out"].shape
    # same torch ops on the same data: bit-exact on the generating machine, a bf16 ulp elsewhere
    assert torch.allclose(out.float(), g["out"].float(), rtol=1e-2, atol=1e-3)
    assert orc.reference_compare_count(out, g["out"], 1e-4, 5e-3) <= 0.005 * out.numel()


def test_sfa_oracle_matches_reference_golden_bf16_cache():
    g = helpers.load_sfa_bf16_golden()
    out = orc.sfa_quant(g["q_nope"], g["q_rope"], g["k_nope"], g["k_rope"], None, g["topk_indices"], g["block_table"],
                        g["act_seq"], g["nq"], g["softmax_scale"])
    assert torch.allclose(out.float(), g["out"].float(), rtol=1e-2, atol=1e-3)
    assert orc.reference_compare_count(out, g["out"], 1e-4, 5e-3) <= 0.005 * out.numel()


def test_scfa_oracle_matches_reference_golden():
    g = helpers.load_scfa_golden()
    out = orc.scfa(g["q"], g["actual_seq_q"], g["ori_kv"], g["cmp_kv"], g["ori_block_table"], g["cmp_block_table"],
                   g["atten_sink"], g["seqused_kv"], g["cmp_sparse_indices"], g["nq"], g["softmax_scale"],
                   g["win_size"], g["cmp_ratio"], g["block_size"])
    ref = g["out"].reshape(out.shape)
    assert torch.allclose(out.float(), ref.float(), rtol=1e-2, atol=1e-3)
    assert orc.reference_compare_count(out, ref, 1e-4, 5e-3) <= 0.005 * out.numel()
    # the window and the selected compressed keys both matter: dropping either changes the result
    no_sel = orc.scfa(g["q"], g["actual_seq_q"], g["ori_kv"], g["cmp_kv"], g["ori_block_table"], g["cmp_block_table"],
                      g["atten_sink"], g["seqused_kv"], g["cmp_sparse_indices"][:, :0], g["nq"], g["softmax_scale"],
                      g["win_size"], g["cmp_ratio"], g["block_size"])
    assert not torch.allclose(no_sel.float(), ref.float(), rtol=1e-2, atol=1e-3)


def test_cfa_oracle_matches_reference_golden():
    g = helpers.load_cfa_golden()
    out = orc.cfa(g["q"], g["cmp_kv"], g["atten_sink"], g["cmp_block_table"], g["seqused_kv"], g["ori_kv"],
                  g["ori_block_table"], g["cmp_ratio"])
    assert out.shape == g["out"].shape
    assert torch.allclose(out.float(), g["out"].float(), rtol=1e-2, atol=1e-3)
    assert orc.reference_compare_count(out, g["out"], 1e-4, 5e-3) <= 0.005 * out.numel()


def test_win_attention_oracle_matches_reference_golden():
    g = helpers.load_win_golden()
    out = orc.win_attention(g["q"], g["ori_block_table"], g["ori_kv"], g["seqused_kv"], g["atten_sink"], g["win_size"],
                            g["actual_seq_q"])
    assert out.shape == g["out"].shape
    assert torch.allclose(out.float(), g["out"].float(), rtol=1e-2, atol=1e-3)
    assert orc.reference_compare_count(out, g["out"], 1e-4, 5e-3) <= 0.005 * out.numel()


def test_prolog_v4_oracle_matches_reference_golden():
    g = helpers.load_prolog_v4_golden()
    inp = helpers.prolog_v4_reference_inputs(g["t"])
    for name, tensor in inp.items():
        assert helpers.digest(tensor) == g["digests"][name], f"regenerated input {name} differs from the reference's"
    q, w, qs = orc.indexer_prolog_v4(**inp)
    assert (q.int() - g["q"].int()).abs().max() <= 1 and (q != g["q"]).float().mean() < 0.01
    assert torch.allclose(w.float(), g["weights"].float(), atol=1e-4, rtol=0.007825)
    assert torch.allclose(qs.float(), g["q_scale"].float(), atol=1e-4, rtol=0.007825)
    # the interleaved inverse rotation undoes the forward one: x -> rope -> inverse rope == x (up to bf16 rounding)
    x = torch.randn(3, 5, 64).to(torch.bfloat16)
    ang = torch.rand(3, 64 // 2) * 6.28
    cos = torch.cos(ang).repeat_interleave(2, -1).to(torch.bfloat16)
    sin = torch.sin(ang).repeat_interleave(2, -1).to(torch.bfloat16)
    fwd = orc.rope_interleaved_inverse(x, cos, -sin)
    assert torch.allclose(orc.rope_interleaved_inverse(fwd, cos, sin).float(), x.float(), atol=0.05)


def test_mla_v4_oracle_matches_reference_golden():
    g = helpers.load_mla_v4_golden()
    inp = helpers.mla_v4_reference_inputs(g["t"])
    for name, tensor in inp.items():
        assert helpers.digest(tensor) == g["digests"][name], f"regenerated input {name} differs from the reference's"
    q, kv, qr, qs = orc.mla_prolog_v4(inp["x"], inp["wq_a"], inp["wq_b"], inp["w_kv"], inp["gamma_cq"], inp["gamma_ckv"],
                                      inp["cos"], inp["sin"], inp["wq_b_scale"])
    # the reference's own tolerances (test_mla_prolog_quant_v4.py:344-350)
    assert torch.allclose(q.float(), g["q"].float(), atol=1e-4, rtol=0.0078125)
    assert torch.allclose(kv.float(), g["kv"].float(), atol=1e-4, rtol=0.0078125)
    assert (qr.int() - g["qr"].int()).abs().max() <= 1
    assert torch.allclose(qs, g["qr_scale"], atol=2.5e-5, rtol=0.005)


def test_mla_v4_bf16_oracle_matches_reference_golden():
    g = helpers.load_mla_v4_bf16_golden()
    inp = helpers.mla_v4_bf16_reference_inputs(g["t"])
    for name, tensor in inp.items():
        assert helpers.digest(tensor) == g["digests"][name], f"regenerated input {name} differs from the reference's"
    q, kv, qr = orc.mla_prolog_v4_bf16(inp["x"], inp["wq_a"], inp["wq_b"], inp["w_kv"], inp["gamma_cq"], inp["gamma_ckv"],
                                       inp["cos"], inp["sin"])
    for got, ref in ((q, g["q"]), (kv, g["kv"]), (qr, g["qr"])):   # the reference's own tolerance for all three
        assert torch.allclose(got.float(), ref.float(), atol=1e-4, rtol=0.0078125)


def test_hc_pre_oracle_matches_reference_golden():
    g = helpers.load_hc_pre_golden()
    inp = helpers.hc_pre_reference_inputs(g["t"])
    for name, tensor in inp.items():
        assert helpers.digest(tensor) == g["digests"][name], f"regenerated input {name} differs from the reference's"
    y, post, comb = orc.hc_pre(**inp)
    # the reference's own tolerances (test_hc_pre.py:203-208)
    assert torch.allclose(y.float(), g["y"].float(), atol=1e-4, rtol=0.0078125)
    assert torch.allclose(post, g["post"], atol=2.5e-5, rtol=0.005)
    assert torch.allclose(comb, g["comb"], atol=2.5e-5, rtol=0.005)
    # Sinkhorn leaves a (nearly) doubly stochastic matrix
    y, post, comb = orc.hc_pre(**helpers.gen_hc_pre_inputs(3, 5))
    assert torch.allclose(comb.sum(-2), torch.ones(5, 4), atol=1e-4) and torch.allclose(comb.sum(-1), torch.ones(5, 4), atol=1e-3)


@pytest.mark.parametrize("name", list(helpers.COMPRESSOR_CASES))
def test_compressor_oracle_matches_reference_golden(name):
    g = helpers.load_compressor_golden(name)
    inp = helpers.compressor_reference_inputs(name)
    for key, want in g["digests"].items():
        assert helpers.digest(inp[key]) == want, f"regenerated input {key} differs from the reference's"
    out = orc.compressor(inp["x"], inp["kv_state"], inp["score_state"], inp["table"], inp["table"], inp["sin"], inp["cos"],
                         inp["wkv"], inp["wgate"], inp["ape"], inp["weight"], inp["hadamard"], inp["start_pos"],
                         inp["ratio"], 64, inp["rotate"])
    assert torch.allclose(out.float(), g["out"].float(), atol=1e-4, rtol=0.0078125)
    # the state rows written by this call (row checksums of every page position)
    assert torch.allclose(inp["kv_state"].double().sum(-1), g["kv_state_sum"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(inp["score_state"].double().sum(-1), g["score_state_sum"], rtol=1e-6, atol=1e-6)


def test_sa_antiquant_oracle_matches_reference_golden():
    g = helpers.load_sa_antiquant_golden()
    out = orc.sa_antiquant(g["q_nope"], g["q_rope"], g["nope_cache"], g["topk_indices"], g["block_table"], g["act_seq"],
                           g["nq"], g["softmax_scale"])
    assert out.shape == g["out"].shape
    assert torch.allclose(out.float(), g["out"].float(), rtol=1e-2, atol=1e-3)
    assert orc.reference_compare_count(out, g["out"], 1e-4, 5e-3) <= 0.005 * out.numel()
    # the fused row is the three arrays side by side
    kn, kr, sc = orc.unpack_cache_rows(g["nope_cache"])
    assert kn.shape[1] == 512 and kr.dtype == torch.bfloat16 and sc.dtype == torch.float32
    assert float(sc.min()) > 0 and float(kr.float().abs().max()) <= 1.0


def test_indexer_oracle_matches_reference_golden():
    g = helpers.load_indexer_golden()
    res, scores = orc.lightning_indexer(g["query"], g["q_scale"], g["key"], g["k_scale"], g["weights"], g["act_seq"],
                                        g["block_table"], 2048, return_scores=True)
    assert res.shape == g["topk_res"].shape
    s1 = g["s1"]
    for t in range(res.shape[0]):
        ok, ndiff, _ = orc.topk_sets_match(res[t, 0], g["topk_res"][t, 0], scores[t // s1][t % s1])
        assert ok, (t, ndiff)
        # pads: -1 exactly where the reference has them
        assert ((res[t, 0] < 0) == (g["topk_res"][t, 0] < 0)).all()


def test_indexer_dots_exact_in_fp32():
    g = helpers.gen_indexer_inputs(5, [300], s1=2)
    rows = orc.paged_rows(g["block_table"][0], torch.arange(300), 128)
    keys = g["key"].reshape(-1, 128)[rows]
    _, dots = orc.indexer_request_scores(g["query"], g["q_scale"], g["weights"], keys,
                                         g["k_scale"].reshape(-1)[rows], return_dots=True)
    ref = torch.matmul(g["query"].reshape(128, 128).to(torch.int32), keys.t().to(torch.int32)).reshape(2, 64, -1)
    assert torch.equal(dots, ref)


def test_prolog_inputs_reproduce_and_oracle_matches_reference_golden():
    g = helpers.load_prolog_golden()
    inp = helpers.prolog_reference_inputs(g["seed"], g["b"], g["s1"], g["s2"])
    for name, d in g["digests"].items():
        if name in inp:
            assert helpers.digest(inp[name]) == d, name
    q_i8, q_s, kc, ksc, w = orc.indexer_prolog(
        inp["token_x"], inp["q_norm"], inp["q_norm_scale"], inp["w_idx_qb"], inp["w_idx_qb_scale"], inp["w_idx_k"],
        inp["w_idx_proj"], inp["layer_norm_gamma"], inp["layer_norm_beta"], inp["cos_idx_rope"], inp["sin_idx_rope"],
        inp["hadamard_q"], inp["hadamard_k"], inp["idx_k_cache"], inp["idx_k_scale_cache"], inp["idx_k_cache_index"])
    assert (q_i8.int() - g["q_int8"].int()).abs().max() <= 1
    assert torch.allclose(q_s.float(), g["q_scale"].float(), atol=2.5e-5, rtol=1e-3)
    assert (kc.int() - g["k_cache"].int()).abs().max() <= 1
    assert torch.allclose(ksc.float(), g["k_scale_cache"].float(), atol=2.5e-5, rtol=1e-3)
    assert torch.allclose(w.float(), g["weights"].float(), atol=2.5e-5, rtol=1e-3)


def test_merge_topk_candidates_equals_global_topk():
    gen = torch.Generator().manual_seed(3)
    scores = torch.randn(2, 4000, generator=gen)
    scores[0, 100] = scores[0, 3000]  # a tie across shards
    k, shards = 256, 4
    cs, ci = [], []
    for s in range(shards):
        lo, hi = s * 1000, (s + 1) * 1000
        part = scores[:, lo:hi]
        idx = torch.stack([orc.topk_indices_ref(part[i], k) for i in range(2)])
        cs.append(torch.gather(part, 1, idx))
        ci.append((idx + lo).to(torch.int32))
    merged = orc.merge_topk_candidates(torch.cat(cs, 1), torch.cat(ci, 1), k)
    for i in range(2):
        assert merged[i].tolist() == orc.topk_indices_ref(scores[i], k).tolist()


def test_mla_inputs_reproduce_and_oracle_matches_reference_golden():
    g = helpers.load_mla_golden()
    inp = helpers.mla_reference_inputs(g["seed"], g["b"], g["s1"], g["s2"])
    for name, d in g["digests"].items():
        assert helpers.digest(inp[name].reshape(-1)) == d, name
    q_nope, q_rope, q_norm, q_norm_scale, kv, kr, ks = orc.mla_prolog(
        inp["x"], inp["w_dq"], inp["w_uqqr"], inp["w_qb_scale"], inp["w_uk"], inp["w_dkvkr"], inp["gamma_cq"],
        inp["gamma_ckv"], inp["cos"], inp["sin"], inp["cache_index"], inp["kv_cache"], inp["kr_cache"], inp["ks_cache"])
    # the reference's own test tolerances (deepseekv32_mla_indexer_prolog_quant.py:808-828)
    assert orc.reference_compare_count(q_nope, g["q_nope"], 0.005, 0.0078125) <= 0.005 * q_nope.numel()
    assert orc.reference_compare_count(q_rope, g["q_rope"], 0.005, 0.0078125) <= 0.005 * q_rope.numel()
    assert (q_norm.int() - g["q_norm"].int()).abs().max() <= 1
    assert torch.allclose(q_norm_scale, g["q_norm_scale"], rtol=1e-3)
    assert (kv.int() - g["kv_cache"].int()).abs().max() <= 1
    assert orc.reference_compare_count(kr, g["kr_cache"], 1e-4, 0.0078125) <= 0.005 * kr.numel()
    assert torch.allclose(ks, g["ks_cache"], rtol=1e-3, atol=1e-6)
