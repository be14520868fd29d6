"""Host-side multi-rank logic on CPU ranks (gloo, world_size 2): request partitioning, the key-range
sharded indexer with candidate all-gather + merge, and what the healthy rank sees when a peer dies before
the collective.  The CUDA kernels are replaced by the CPU oracle here; the same flow runs on GPUs in
tests/test_gpu_parity.py::test_indexer_key_range_shards_merge_to_global_topk."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers
from oracle import dsv32_oracle as orc
from pypto_b200 import sharding


def test_split_even_and_key_ranges():
    assert sharding.split_even(10, 4) == [[0, 1, 2], [3, 4, 5], [6, 7], [8, 9]]
    assert sum(len(x) for x in sharding.split_even(64, 8)) == 64
    ranges = [sharding.key_range_for_rank(131072, r, 8) for r in range(8)]
    assert ranges[0] == (0, 16384) and ranges[7][0] == 7 * 16384 and ranges[7][1] == sharding.INT32_MAX
    # ragged: 1000 keys = 8 blocks over 3 ranks -> 3/3/2 blocks
    assert [sharding.key_range_for_rank(1000, r, 3)[0] for r in range(3)] == [0, 384, 768]


def test_lpt_balances_ragged_batches():
    g = torch.Generator().manual_seed(4)
    ctx = torch.exp(torch.rand(256, generator=g) * (torch.log(torch.tensor(131072.0)) - torch.log(torch.tensor(1024.0)))
                    + torch.log(torch.tensor(1024.0))).long().tolist()
    costs = [sharding.request_cost(c, 2) for c in ctx]
    bins = sharding.lpt_assign(costs, 8)
    assert sorted(i for b in bins for i in b) == list(range(256))
    loads = [sum(costs[i] for i in b) for b in bins]
    assert max(loads) / (sum(loads) / 8) < 1.05


def test_token_slices_and_long_request_generator():
    from pypto_b200 import synth
    assert [sharding.token_slice_for_rank(4096, r, 8) for r in (0, 7)] == [(0, 512), (3584, 4096)]
    assert [sharding.token_slice_for_rank(5, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 5), (5, 5)]
    full = synth.make_long_request(1000, 6, 9, "cpu")
    part = synth.make_long_request(1000, 6, 9, "cpu", token_slice=(2, 5))
    # the shared state and the index-side queries are the same bits on every rank; attention queries follow the slice
    for k in ("block_table", "idx_k", "k_nope", "k_scales", "q_int8", "weights"):
        assert torch.equal(full[k], part[k])
    assert torch.equal(part["q_nope"], full["q_nope"][2 * 128:5 * 128])
    smp = synth.make_long_request(1000, 6, 9, "cpu", sample=3)
    assert smp["tokens"] == [0, 2, 5] and smp["eff"].tolist() == [995, 997, 1000]
    assert torch.equal(smp["q_int8"], full["q_int8"][[0, 2, 5]])
    assert torch.equal(smp["q_rope"][128:256], full["q_rope"][2 * 128:3 * 128])


def test_packed_tensors_views_share_one_buffer():
    from pypto_b200.decode_chain import PackedTensors
    src = {"a": torch.arange(10, dtype=torch.int32), "b": torch.randn(3, 5).to(torch.bfloat16), "c": torch.tensor([7], dtype=torch.int64)}
    pk = PackedTensors(src, "cpu")
    for k, v in src.items():
        assert torch.equal(pk.views[k], v) and pk.offsets[k] % 256 == 0
    other = PackedTensors({k: torch.zeros_like(v) for k, v in src.items()}, "cpu")
    other.buf.copy_(pk.buf)            # one copy moves every tensor
    assert all(torch.equal(other.views[k], v) for k, v in src.items())


def test_ragged_contexts_of_the_bench():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    ctx = bench.ragged_contexts(256, 1004)
    assert len(ctx) == 256 and min(ctx) >= 64 and max(ctx) <= 131072
    assert sum(c < 2048 for c in ctx) >= 26                      # every tenth request is forced below the top-k size
    assert ctx == bench.ragged_contexts(256, 1004)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_local(q, qs, kc, ks, w, act, bt, k, begin, end):
    t, b = q.shape[0], act.shape[0]
    s1 = t // b
    scores = orc.indexer_scores(q, qs, kc, ks, w, act, bt, key_offset=begin, key_limit=end)
    idx = torch.full((t, k), -1, dtype=torch.int32)
    sc = torch.full((t, k), float("-inf"))
    for bi in range(b):
        for si in range(s1):
            eff = int(act[bi]) - (s1 - 1 - si)
            n = max(min(eff, end) - begin, 0)
            if n <= 0:
                continue
            row = scores[bi][si, :n]
            sel = orc.topk_indices_ref(row, min(k, n))
            idx[bi * s1 + si, :sel.numel()] = (sel + begin).to(torch.int32)
            sc[bi * s1 + si, :sel.numel()] = row[sel]
    return idx, sc


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        d = helpers.gen_indexer_inputs(21, [6000], s1={"own": 3, "own1": 1}.get(mode, 2))
        if mode == "die" and rank == 1:
            raise RuntimeError("rank 1 fails before the collective")
        if mode in ("own", "own1"):   # three tokens over two ranks: slices of two and one token, the second padded on the
            # wire; one token: the second rank owns nothing and gets an empty result
            out = sharding.sharded_indexer_topk_own_slice(d["query"], d["q_scale"], d["key"], d["k_scale"], d["weights"],
                                                          d["act_seq"], d["block_table"], 2048, local_fn=_oracle_local,
                                                          merge_fn=orc.merge_topk_candidates)
            ref = orc.lightning_indexer(d["query"], d["q_scale"], d["key"], d["k_scale"], d["weights"], d["act_seq"],
                                        d["block_table"], 2048)
            t0, t1 = sharding.token_slice_for_rank(ref.shape[0], rank, world)
            ret[rank] = "ok" if (out.shape[0] == t1 - t0 and torch.equal(out, ref[t0:t1, 0])) else "mismatch"
            return
        out = sharding.sharded_indexer_topk(d["query"], d["q_scale"], d["key"], d["k_scale"], d["weights"], d["act_seq"],
                                            d["block_table"], 2048, local_fn=_oracle_local,
                                            merge_fn=orc.merge_topk_candidates)
        ref = orc.lightning_indexer(d["query"], d["q_scale"], d["key"], d["k_scale"], d["weights"], d["act_seq"],
                                    d["block_table"], 2048)
        ret[rank] = "ok" if torch.equal(out, ref[:, 0]) else "mismatch"
    except Exception as e:  # noqa: BLE001
        ret[rank] = f"error: {type(e).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(mode):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert not p.is_alive()
    return dict(ret)


def test_key_range_sharded_indexer_equals_unsharded_world2():
    assert _run("ok") == {0: "ok", 1: "ok"}


def test_own_slice_exchange_equals_unsharded_rows_world2():
    """The all-to-all form: every rank gets the global top-k of its own token slice only."""
    assert _run("own") == {0: "ok", 1: "ok"}


def test_own_slice_exchange_with_a_rank_that_owns_no_token_world2():
    assert _run("own1") == {0: "ok", 1: "ok"}


def test_rank_failure_surfaces_as_error_on_the_healthy_rank():
    ret = _run("die")
    assert ret[1].startswith("error: RuntimeError")
    assert ret[0].startswith("error")  # the collective ends with an error (peer gone / timeout), it does not hang
