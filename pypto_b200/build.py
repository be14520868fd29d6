"""In-tree build of libdsv32_b200.so with nvcc for sm_100a.

    python -m pypto_b200.build [--verbose] [--force]

The shared library is written next to this file (pypto_b200/libdsv32_b200.so) so that it ships
with a source snapshot of the tree; it is not installed anywhere else.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libdsv32_b200.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
SOURCES = ["api.cu", "topk.cu", "indexer_tc.cu", "sfa_tc.cu", "sfa_combine.cu", "prolog.cu", "prolog_tc.cu", "mla_prolog.cu", "mla_prolog_tc.cu", "pg_prolog.cu",
           "mla_prolog_v4.cu", "hc_pre.cu", "compressor.cu", "decode_advance.cu", "noalloc.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return cand


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _newest_source_mtime() -> float:
    m = 0.0
    for root in (CSRC, os.path.join(os.path.dirname(HERE), "include")):
        for f in os.listdir(root):
            m = max(m, os.path.getmtime(os.path.join(root, f)))
    return m


def is_stale() -> bool:
    return not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < _newest_source_mtime()


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    objs = []
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    common = [nvcc_path(), *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in _sources():
        obj = os.path.join(build_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)} ---\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    link = [nvcc_path(), *ARCH_FLAGS, "-shared", "-o", LIB_PATH, *objs, "-lcudart"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(verbose=a.verbose, force=a.force))
