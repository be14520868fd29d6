"""No-GPU checks of the drop-in boundary: the shared library builds/loads, exports every symbol the
public header declares, and rejects bad arguments on the host without touching a device."""
import ctypes as C
import os
import re

import pytest
import torch

import helpers
from pypto_b200 import _lib


def _header_symbols():
    with open(os.path.join(helpers.ROOT, "include", "dsv32_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsv32_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from pypto_b200 import build
        build.build()
    return _lib.load()


def test_header_and_binding_agree():
    assert _header_symbols() == sorted(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in _header_symbols():
        assert hasattr(lib, name), name
    assert lib.dsv32_abi_version() == _lib.ABI_VERSION


def test_workspace_queries(lib):
    # the row id of every selected key; key-split partials only when there are too few CTAs for one split
    assert lib.dsv32_sfa_workspace_bytes(64, 2, 128, 2048, 0) == 64 * 2 * 2048 * 4
    assert lib.dsv32_sfa_workspace_bytes(4, 1, 128, 2048, 0) > 4 * 2048 * 4
    assert lib.dsv32_indexer_workspace_bytes(2, 2, 4, 128) == 2 * 2 * 4 * 128 * 4
    assert lib.dsv32_prolog_workspace_bytes(16) > 0
    assert lib.dsv32_prolog_workspace_bytes(0) == 0


def test_host_side_rejections(lib):
    assert lib.dsv32_sfa_quant(None, None) == -1
    assert b"NULL" in lib.dsv32_last_error()
    a = _lib.SfaArgs()
    a.b, a.s1, a.n_q, a.topk, a.block_size, a.max_blocks = 1, 1, 129, 2048, 128, 1
    assert lib.dsv32_sfa_quant(C.byref(a), None) == -1
    assert b"n_q" in lib.dsv32_last_error()
    i = _lib.IndexerArgs()
    i.b, i.s1, i.block_size, i.max_blocks = 1, 1, 64, 1
    assert lib.dsv32_indexer_topk(C.byref(i), None) == -1
    assert b"block_size" in lib.dsv32_last_error()
    t = _lib.TopkArgs()
    t.rows, t.ld, t.k = 1, 8, 4096
    assert lib.dsv32_topk_select(C.byref(t), None) == -1
    # the sharded form of the indexer: one request, at most eight ranks, a buffer pair for every rank
    sc = _lib.TopkScatter()
    i2 = _lib.IndexerArgs()
    i2.b, i2.s1, i2.block_size, i2.max_blocks, i2.selected_count = 2, 4, 128, 1, 2048
    sc.world, sc.rank, sc.tokens_per_rank = 2, 0, 2
    assert lib.dsv32_indexer_topk_scatter(C.byref(i2), C.byref(sc), None) == -1
    assert b"one request" in lib.dsv32_last_error()
    i2.b = 1
    sc.world = 9
    assert lib.dsv32_indexer_topk_scatter(C.byref(i2), C.byref(sc), None) == -1
    assert b"at most 8" in lib.dsv32_last_error()
    sc.world, sc.tokens_per_rank = 2, 1
    assert lib.dsv32_indexer_topk_scatter(C.byref(i2), C.byref(sc), None) == -1
    assert b"does not cover" in lib.dsv32_last_error()
    sc.tokens_per_rank = 2
    assert lib.dsv32_indexer_topk_scatter(C.byref(i2), C.byref(sc), None) == -1
    assert b"buffer of rank 0" in lib.dsv32_last_error()
    assert lib.dsv32_indexer_topk_scatter(C.byref(i2), None, None) == -1
    p = _lib.PrologArgs()
    p.t = -1
    assert lib.dsv32_indexer_prolog(C.byref(p), None) == -1


def test_python_entry_points_fail_loudly_without_gpu():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from pypto_b200.sparse_flash_attention_quant_impl import sparse_flash_attention_quant_d
    z = torch.zeros(1)
    with pytest.raises(RuntimeError):
        sparse_flash_attention_quant_d(z, z, z, z, z, z, z, z, z, 128, 1, 1.0, 2048, 128, 1, None)


def test_missing_library_is_an_error(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.Dsv32Error):
        _lib.load()


def test_every_module_of_the_package_imports():
    """An entry module that cannot be imported would only show on a GPU box otherwise."""
    import importlib
    import pkgutil
    import pypto_b200
    for m in pkgutil.iter_modules(pypto_b200.__path__):
        if not m.name.startswith("lib"):   # the shared library sits in the package directory
            importlib.import_module(f"pypto_b200.{m.name}")
