"""The allocation-free lightning-indexer entry point (dsv32_indexer_topk_noalloc), called through the
C ABI, against the regular entry point.

It exists for callers that cannot allocate device memory when they run the operator (a serving loop
whose memory pool owns the whole device, a host that forbids cudaMalloc inside operator calls): its
score scratch is a fixed array inside the library.  This file sorts last on purpose so that a run that
stops at the first failure has already executed every other test; it also passes when run alone.
"""
import ctypes as C

import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _args(lib_mod, d, res, tsc, workspace):
    ptr = lambda t: C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)  # noqa: E731
    t = d["query"].shape[0]
    b = d["act_seq"].shape[0]
    max_blocks = d["block_table"].shape[1]
    ws_bytes = workspace.numel() if workspace is not None else 0
    return lib_mod.IndexerArgs(
        ptr(d["query"]), ptr(d["q_scale"]), ptr(d["key"]), ptr(d["k_scale"]), ptr(d["weights"]), ptr(d["act_seq"]),
        ptr(d["block_table"]), ptr(res), ptr(tsc), C.c_void_p(0), C.c_void_p(0), ptr(workspace), ws_bytes,
        C.c_void_p(0), d["key"].shape[0], b, t // b, 128, max_blocks, 2048, 0, 0, 2 ** 31 - 1)


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    from pypto_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, act_seq, s1 in ((31, [5000, 971, 2049], 2), (32, [16000, 300], 1)):
        d = {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v)
             for k, v in helpers.gen_indexer_inputs(seed, act_seq, s1=s1, extra_blocks=2).items()}
        t = d["query"].shape[0]
        ws = torch.empty(lib.dsv32_indexer_workspace_bytes(len(act_seq), s1, d["block_table"].shape[1], 128),
                         dtype=torch.uint8, device=DEV)
        ref_idx = torch.zeros((t, 1, 2048), dtype=torch.int32, device=DEV)
        ref_sc = torch.zeros((t, 2048), dtype=torch.float32, device=DEV)
        _lib.check(lib.dsv32_indexer_topk(C.byref(_args(_lib, d, ref_idx, ref_sc, ws)), stream), "regular")
        for call in range(2):  # two calls in a row share the built-in scratch
            idx = torch.full((t, 1, 2048), -7, dtype=torch.int32, device=DEV)
            sc = torch.zeros((t, 2048), dtype=torch.float32, device=DEV)
            args = _args(_lib, d, idx, sc, None)
            torch.cuda.synchronize()
            free0, held0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
            _lib.check(lib.dsv32_indexer_topk_noalloc(C.byref(args), stream), "noalloc")
            torch.cuda.synchronize()
            if seed != 31 or call > 0:   # what the entry point is for: after the device's first call, no allocation
                assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == held0
            assert torch.equal(idx, ref_idx)
            assert torch.equal(sc, ref_sc)


def test_noalloc_entry_rejects_sizes_beyond_its_scratch():
    from pypto_b200 import _lib
    lib = _lib.load()
    a = _lib.IndexerArgs()
    a.b, a.s1, a.block_size, a.max_blocks = 64, 2, 128, 512  # 8.4 M scores > 2 M
    assert lib.dsv32_indexer_topk_noalloc(C.byref(a), None) == -2
    assert b"exceed the built-in scratch" in lib.dsv32_last_error()
