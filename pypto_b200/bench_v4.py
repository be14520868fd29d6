"""Timings of the DeepSeek-V4 operators at the reference's decode shapes (64 requests x 2 tokens, 64 heads).

    python -m pypto_b200.bench_v4 [--batch 64] [--s1 2] [--ctx 8192] [--reps 15]

Every operator is called through its reference-named entry point, captured once in a CUDA graph and replayed
`reps` times with a buffer larger than L2 written between replays; the time is the median of CUDA-event
durations.  One JSON line per operator on stdout.  Inputs are seeded synthetic tensors (uniform [-1, 1) caches and
queries as in the reference's test generators, random page assignment, random selections).
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from . import (compress_flash_attention_impl as cfa, compressor_impl as comp, hc_pre_impl as hcp,
               lightning_indexer_prolog_quant_v4_impl as ipv4, mla_prolog_quant_v4_impl as mlaq, mla_prolog_v4_impl as mlab,
               sparse_compress_flash_attention_impl as scfa, win_attention_impl as win)
from ._runtime import check_status

DEV = "cuda"
BF = torch.bfloat16


def _uni(shape, g, scale=1.0, dtype=BF):
    return ((torch.rand(shape, generator=g, device=DEV) * 2 - 1) * scale).to(dtype)


def _pages(b, blocks_each, g):
    perm = torch.randperm(b * blocks_each, generator=g, device=DEV).to(torch.int32)
    return perm.reshape(b, blocks_each).contiguous()


def _timeit(fn, reps, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    times = []
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2] * 1000.0


def attention_inputs(b, s1, ctx, nq, cmp_ratio, topk, g, shared_selection):
    t = b * s1
    ori_blocks, cmp_len = math.ceil(ctx / 128), ctx // cmp_ratio
    cmp_blocks = max(math.ceil(cmp_len / 128), 1)
    idx = torch.full((t, topk), -1, dtype=torch.int32, device=DEV)
    n = min(cmp_len, topk)
    for tok in range(t):
        if shared_selection and tok % s1:
            idx[tok] = idx[tok - 1]
        else:
            idx[tok, :n] = torch.randperm(cmp_len, generator=g, device=DEV)[:n].to(torch.int32)
    return dict(
        q=_uni((t * nq, 512), g), ori_kv=_uni((b * ori_blocks * 128, 512), g), cmp_kv=_uni((b * cmp_blocks * 128, 512), g),
        ori_bt=_pages(b, ori_blocks, g), cmp_bt=_pages(b, cmp_blocks, g), sink=_uni((nq,), g, dtype=torch.float32),
        seq_q=torch.arange(0, t + 1, s1, dtype=torch.int32, device=DEV),
        seq_kv=torch.full((b,), ctx, dtype=torch.int32, device=DEV), idx=idx)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--s1", type=int, default=2)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--reps", type=int, default=15)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_v4 needs a CUDA device")
    b, s1, ctx, nq, t = args.batch, args.s1, args.ctx, 64, args.batch * args.s1
    g = torch.Generator(device=DEV).manual_seed(4)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    rows = []

    def report(name, us, **extra):
        rows.append(dict(operator=name, us=round(us, 1), tokens=t, **extra))

    for shared in (False, True):
        a = attention_inputs(b, s1, ctx, nq, 4, 512, g, shared)
        us = _timeit(lambda: scfa.npu_sparse_compress_flash_attention(
            a["q"], a["seq_q"], a["ori_kv"], a["cmp_kv"], a["ori_bt"], a["cmp_bt"], a["sink"], a["seq_kv"], a["idx"],
            512 ** -0.5, 128, 4), args.reps, flush)
        report("sparse_compress_flash_attention", us, keys=128 + 512, ctx=ctx,
               selections="shared by the tokens of a request" if shared else "independent random")
    a = attention_inputs(b, s1, ctx, nq, 128, 1, g, False)
    q3 = a["q"].reshape(t, nq, 512)
    ok4, ck4 = a["ori_kv"].reshape(-1, 128, 1, 512), a["cmp_kv"].reshape(-1, 128, 1, 512)
    us = _timeit(lambda: cfa.cfa_attention(q3, ck4, a["sink"], a["cmp_bt"], a["seq_kv"], ok4, a["ori_bt"], 128), args.reps, flush)
    report("cfa_attention", us, keys=128 + ctx // 128, ctx=ctx)
    us = _timeit(lambda: win.deepseekv4_win_atten(q3, a["ori_bt"], ok4, a["seq_kv"], a["sink"], 128, None, a["seq_q"]),
                 args.reps, flush)
    report("deepseekv4_win_atten", us, keys=128, ctx=ctx)

    # prologs (h 4096, q_lora_rank 1024, 64 heads of 512 / 64 index heads of 128)
    x = _uni((t, 4096), g)
    ang = torch.rand((t, 32), generator=g, device=DEV) * 2 * math.pi
    cos, sin = torch.cos(ang).repeat_interleave(2, -1).to(BF), torch.sin(ang).repeat_interleave(2, -1).to(BF)
    wq_a, wkv = _uni((4096, 1024), g, 0.03), _uni((4096, 512), g, 0.03)
    wq_b = torch.randint(-127, 128, (1024, 64 * 512), generator=g, device=DEV, dtype=torch.int8)
    wq_b_scale = torch.rand((1, 64 * 512), generator=g, device=DEV) * 1e-3 + 1e-4
    gam_q, gam_kv = 1 + _uni((1024,), g, 0.1), 1 + _uni((512,), g, 0.1)
    us = _timeit(lambda: mlaq.mla_prolog_v4_in(x, wq_a, wq_b, wkv, cos, sin, gam_q, gam_kv, wq_b_scale), args.reps, flush)
    report("mla_prolog_v4 (quant)", us)
    wq_b16 = (wq_b.float() * wq_b_scale).to(BF)
    us = _timeit(lambda: mlab.mla_prolog_v4_in(x, wq_a, wq_b16, wkv, cos, sin, gam_q, gam_kv), args.reps, flush)
    report("mla_prolog_v4 (bf16)", us)
    qr = torch.randint(-127, 128, (t, 1024), generator=g, device=DEV, dtype=torch.int8)
    iw = torch.randint(-127, 128, (1024, 8192), generator=g, device=DEV, dtype=torch.int8)
    w_proj, had_q = _uni((4096, 64), g, 0.03), _uni((128, 128), g)
    qr_scale = torch.rand((t, 1), generator=g, device=DEV) * 0.02
    iw_scale = torch.rand((8192, 1), generator=g, device=DEV) * 0.002
    us = _timeit(lambda: ipv4.npu_quant_lightning_indexer_prolog(qr, iw, x, w_proj, cos, sin, had_q, qr_scale, iw_scale),
                 args.reps, flush)
    report("quant_lightning_indexer_prolog (v4)", us)
    xh = torch.randn((t, 4, 4096), generator=g, device=DEV).to(BF)
    hc_fn = torch.randn((24, 16384), generator=g, device=DEV) * 0.02
    hc_scale, hc_base = torch.rand((3,), generator=g, device=DEV) + 0.5, torch.randn((24,), generator=g, device=DEV) * 0.5
    us = _timeit(lambda: hcp.npu_hc_pre(xh, hc_fn, hc_scale, hc_base), args.reps, flush)
    report("hc_pre", us)
    for ratio, d, rotate, start in ((4, 512, False, 255), (4, 128, True, 255), (128, 512, False, 254)):
        coff = 2 if ratio == 4 else 1
        out_rows = min(t, t // ratio + b)
        xs = _uni((b, s1, 4096), g)
        table = torch.arange(b * 4, dtype=torch.int32, device=DEV).reshape(b, 4)
        kv_state = torch.randn((b * 4, 128, coff * d), generator=g, device=DEV)
        sc_state = torch.randn((b * 4, 128, coff * d), generator=g, device=DEV)
        wk, wg = _uni((coff * d, 4096), g, 0.03), _uni((coff * d, 4096), g, 0.03)
        ape, weight = torch.randn((ratio, coff * d), generator=g, device=DEV), torch.ones(d, device=DEV)
        csin, ccos = _uni((out_rows, 64), g), _uni((out_rows, 64), g)
        had = _uni((d, d), g, d ** -0.5)
        st = torch.full((b,), start, dtype=torch.int32, device=DEV)
        us = _timeit(lambda: comp.npu_compressor(xs, kv_state, sc_state, table, table, csin, ccos, wk, wg, ape, weight, had,
                                                 st, ratio, 64, rotate), args.reps, flush)
        report("compressor", us, ratio=ratio, d=d, rotate=rotate, note="every request closes a window in this call")
    check_status()
    for r in rows:
        print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
