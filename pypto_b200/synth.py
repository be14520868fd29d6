"""Seeded synthetic decode workloads (device-resident) for the benchmark and the smoke check.

Distributions: queries/activations N(0,1) bf16, latent cache int8 U{-127..127} with four fp32 scales per
row U(0.001,0.02), rope parts N(0,1) bf16, index keys int8 U{-127..127} with fp16 scales U(0.001,0.02),
weights N(0,0.02); pages are a random permutation of the pool; RoPE angles U(0,2pi); the 128x128
"Hadamard" input is the Sylvester matrix / sqrt(128).  No dataset is involved.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class DecodeWorkload:
    b: int
    s1: int
    ctx: list            # per-request context length (python ints)
    block_table: torch.Tensor
    act_seq: torch.Tensor
    # latent KV cache
    k_nope: torch.Tensor
    k_rope: torch.Tensor
    k_scales: torch.Tensor
    # index key cache
    idx_k: torch.Tensor
    idx_k_scale: torch.Tensor
    # weights of the indexer prolog
    w_qb: torch.Tensor
    w_qb_scale: torch.Tensor
    wk: torch.Tensor
    w_proj: torch.Tensor
    ln_gamma: torch.Tensor
    ln_beta: torch.Tensor
    hadamard: torch.Tensor
    # per-step activations (host or device)
    x: torch.Tensor
    q_norm: torch.Tensor
    q_norm_scale: torch.Tensor
    cos: torch.Tensor
    sin: torch.Tensor
    cache_index: torch.Tensor
    q_nope: torch.Tensor
    q_rope: torch.Tensor

    @property
    def t(self):
        return self.b * self.s1

    @property
    def max_blocks(self):
        return self.block_table.shape[1]


def sylvester_hadamard(n=128, dtype=torch.bfloat16, device="cpu"):
    h = torch.ones((1, 1))
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h / math.sqrt(n)).to(dtype).to(device)


def make_decode_workload(ctx, s1, seed, device, nq=128, block_size=128):
    """ctx: list of per-request context lengths.  Everything is created on `device`."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    b = len(ctx)
    t = b * s1
    bf = torch.bfloat16
    nblk = [math.ceil(c / block_size) for c in ctx]
    blocks = sum(nblk)
    rows = blocks * block_size
    perm = torch.randperm(blocks, generator=g, device=dev).to(torch.int32)
    block_table = torch.full((b, max(nblk)), -1, dtype=torch.int32, device=dev)
    pos = 0
    for i, n in enumerate(nblk):
        block_table[i, :n] = perm[pos:pos + n]
        pos += n
    act_seq = torch.tensor(ctx, dtype=torch.int32, device=dev)

    def randint8(shape):
        return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8, device=dev)

    def randn(shape, std=1.0, dtype=bf):
        return (torch.randn(shape, generator=g, device=dev) * std).to(dtype)

    k_nope = randint8((rows, 512))
    k_rope = randn((rows, 64))
    k_scales = torch.rand((rows, 4), generator=g, device=dev) * 0.019 + 0.001
    idx_k = randint8((blocks, block_size, 1, 128))
    idx_k_scale = (torch.rand((blocks, block_size, 1), generator=g, device=dev) * 0.019 + 0.001).to(torch.float16)
    wq = torch.randn((1536, 8192), generator=g, device=dev) * 0.02
    wamax = wq.abs().amax(0, keepdim=True)
    w_qb = torch.round(wq * (127 / wamax)).to(torch.int8)
    w_qb_scale = (wamax / 127).reshape(8192, 1).float().contiguous()
    wk = randn((7168, 128), 0.02)
    w_proj = randn((7168, 64), 0.02)
    x = randn((t, 7168))
    qr = torch.randn((t, 1536), generator=g, device=dev)
    amax = qr.abs().amax(-1, keepdim=True)
    q_norm = torch.round(qr * (127 / amax)).to(torch.int8)
    q_norm_scale = (amax / 127).float().contiguous()
    ang = torch.rand((t, 64), generator=g, device=dev) * 2 * math.pi
    bt_cpu = block_table.cpu()
    ci = []
    for bi, c in enumerate(ctx):
        for si in range(s1):
            p = max(c - s1 + si, 0)
            ci.append(int(bt_cpu[bi, p // block_size]) * block_size + p % block_size)
    cache_index = torch.tensor(ci, dtype=torch.int64, device=dev)
    return DecodeWorkload(
        b=b, s1=s1, ctx=list(ctx), block_table=block_table, act_seq=act_seq, k_nope=k_nope, k_rope=k_rope,
        k_scales=k_scales, idx_k=idx_k, idx_k_scale=idx_k_scale, w_qb=w_qb, w_qb_scale=w_qb_scale, wk=wk, w_proj=w_proj,
        ln_gamma=torch.ones(128, dtype=bf, device=dev), ln_beta=torch.zeros(128, dtype=bf, device=dev),
        hadamard=sylvester_hadamard(128, bf, dev), x=x, q_norm=q_norm, q_norm_scale=q_norm_scale,
        cos=torch.cos(ang).to(bf), sin=torch.sin(ang).to(bf), cache_index=cache_index,
        q_nope=randn((t * nq, 512)), q_rope=randn((t * nq, 64)))


def make_step_activations(w: DecodeWorkload, seed, nq=128):
    """Another set of per-step activations for the same workload (same shapes, distributions and cache positions,
    different values): rotating between sets keeps a timed loop from replaying the same queries and top-k rows."""
    dev = w.k_nope.device
    g = torch.Generator(device=dev).manual_seed(seed)
    t, bf = w.t, torch.bfloat16

    def randn(shape):
        return torch.randn(shape, generator=g, device=dev).to(bf)

    qr = torch.randn((t, 1536), generator=g, device=dev)
    amax = qr.abs().amax(-1, keepdim=True)
    ang = torch.rand((t, 64), generator=g, device=dev) * 2 * math.pi
    return dict(x=randn((t, 7168)), q_norm=torch.round(qr * (127 / amax)).to(torch.int8),
                q_norm_scale=(amax / 127).float().contiguous(), cos=torch.cos(ang).to(bf), sin=torch.sin(ang).to(bf),
                cache_index=w.cache_index.clone(), q_nope=randn((t * nq, 512)), q_rope=randn((t * nq, 64)))


def make_long_request(ctx, s1, seed, device, token_slice=None, sample=None, block_size=128, nq=128):
    """One long request (prefill-style chunk): `ctx` keys in both paged caches and `s1` query tokens, the i-th of
    which sees ctx - s1 + 1 + i keys.  Everything is drawn from CPU generators (the same bits on every rank and in
    the CPU tests) and then moved to `device`.  The index-side query tensors cover all s1 tokens; the attention
    queries only `token_slice` = (first, last + 1) (default: all).  With `sample` = n the query side is cut down
    to n tokens spread evenly over the chunk and `eff` holds their valid-key counts (CPU baseline / oracle checks).
    Returns a dict."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    blocks = math.ceil(ctx / block_size)
    rows = blocks * block_size
    block_table = torch.randperm(blocks, generator=g).to(torch.int32).reshape(1, blocks)
    idx_k = torch.randint(-127, 128, (blocks, block_size, 1, 128), generator=g, dtype=torch.int8)
    idx_k_scale = (torch.rand((blocks, block_size, 1), generator=g) * 0.019 + 0.001).to(torch.float16)
    k_nope = torch.randint(-127, 128, (rows, 512), generator=g, dtype=torch.int8)
    k_rope = torch.randn((rows, 64), generator=g).to(bf)
    k_scales = torch.rand((rows, 4), generator=g) * 0.019 + 0.001
    q_int8 = torch.randint(-127, 128, (s1, 64, 128), generator=g, dtype=torch.int8)
    q_scale = (torch.rand((s1, 64), generator=g) * 0.019 + 0.001).to(torch.float16)
    weights = (torch.randn((s1, 64), generator=g) * 0.1).to(torch.float16)
    if sample is not None:
        pick = sorted({int(round(j * (s1 - 1) / max(sample - 1, 1))) for j in range(sample)})
    else:
        t0, t1 = token_slice if token_slice is not None else (0, s1)
        pick = list(range(t0, t1))
    qn, qr = [], []
    for i in pick:   # per-token generators: a token's attention query does not depend on which rank draws it
        gi = torch.Generator().manual_seed(seed * 1000003 + i)
        qn.append(torch.randn((nq, 512), generator=gi).to(bf))
        qr.append(torch.randn((nq, 64), generator=gi).to(bf))
    q_nope = torch.cat(qn) if qn else torch.empty((0, 512), dtype=bf)
    q_rope = torch.cat(qr) if qr else torch.empty((0, 64), dtype=bf)
    out = dict(block_table=block_table, act_seq=torch.tensor([ctx], dtype=torch.int32), idx_k=idx_k,
               idx_k_scale=idx_k_scale, k_nope=k_nope, k_rope=k_rope, k_scales=k_scales, q_int8=q_int8, q_scale=q_scale,
               weights=weights, q_nope=q_nope, q_rope=q_rope, tokens=pick)
    if sample is not None:
        sel = torch.tensor(pick, dtype=torch.long)
        out.update(q_int8=q_int8[sel], q_scale=q_scale[sel], weights=weights[sel],
                   eff=torch.tensor([ctx - s1 + 1 + i for i in pick], dtype=torch.int32))
    dev = torch.device(device)
    return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in out.items()}


@dataclass
class FullDecodeWorkload:
    """State of a multi-step decode loop through the fused MLA + indexer prolog: both paged caches (sharing one
    page table with room to grow), the weights of both prolog halves, and the batch's position state."""
    b: int
    s1: int
    block_table: torch.Tensor     # int32 [b, max_blocks], -1 = not assigned
    act_seq: torch.Tensor         # int32 [b]: length including the current step's s1 tokens
    cache_index: torch.Tensor     # int64 [b * s1]: cache rows of the current step's tokens
    kv_cache: torch.Tensor        # int8 [blocks, 128, 1, 512]
    kr_cache: torch.Tensor        # bf16 [blocks, 128, 1, 64]
    k_scale_cache: torch.Tensor   # fp32 [blocks, 128, 1, 4]
    idx_k: torch.Tensor           # int8 [blocks, 128, 1, 128]
    idx_k_scale: torch.Tensor     # fp16 [blocks, 128, 1, 1]
    w_dq: torch.Tensor
    w_uq_qr: torch.Tensor
    w_uq_qr_scale: torch.Tensor
    w_uk: torch.Tensor
    w_dkv_kr: torch.Tensor
    gamma_cq: torch.Tensor
    gamma_ckv: torch.Tensor
    w_qb: torch.Tensor
    w_qb_scale: torch.Tensor
    wk: torch.Tensor
    w_proj: torch.Tensor
    ln_gamma: torch.Tensor
    ln_beta: torch.Tensor
    hadamard: torch.Tensor

    @property
    def t(self):
        return self.b * self.s1

    @property
    def max_blocks(self):
        return self.block_table.shape[1]


def cache_index_for(act_seq, block_table, s1, block_size=128):
    """The reference's rule (deepseekv32_mla_indexer_prolog_quant.py:184-194) on the host: rows of the s1 newest
    positions of every request."""
    bt = block_table.cpu()
    out = []
    for bi, cur in enumerate(act_seq.cpu().tolist()):
        for j in range(s1):
            pos = cur - s1 + j
            out.append(int(bt[bi, pos // block_size]) * block_size + pos % block_size if pos >= 0 else -1)
    return torch.tensor(out, dtype=torch.int64)


def make_full_decode_workload(ctx, s1, grow_tokens, seed, device, block_size=128):
    """ctx: per-request lengths including the first step's s1 tokens; every request gets pages for
    ctx + grow_tokens positions.  Caches hold random history, weights follow the distributions of the single-step
    workloads.  Drawn from a CPU generator (the same bits on any device)."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    b = len(ctx)
    nblk = [math.ceil((c + grow_tokens) / block_size) for c in ctx]
    blocks = sum(nblk)
    perm = torch.randperm(blocks, generator=g).to(torch.int32)
    block_table = torch.full((b, max(nblk)), -1, dtype=torch.int32)
    pos = 0
    for i, n in enumerate(nblk):
        block_table[i, :n] = perm[pos:pos + n]
        pos += n
    act_seq = torch.tensor(ctx, dtype=torch.int32)

    def randn(shape, std=1.0, dtype=bf):
        return (torch.randn(shape, generator=g) * std).to(dtype)

    def randint8(shape):
        return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)

    wq = torch.randn((1536, 128 * 192), generator=g) * 0.02
    wq_amax = wq.abs().amax(0, keepdim=True)
    wi = torch.randn((1536, 8192), generator=g) * 0.02
    wi_amax = wi.abs().amax(0, keepdim=True)
    w = FullDecodeWorkload(
        b=b, s1=s1, block_table=block_table, act_seq=act_seq, cache_index=cache_index_for(act_seq, block_table, s1),
        kv_cache=randint8((blocks, block_size, 1, 512)), kr_cache=randn((blocks, block_size, 1, 64)),
        k_scale_cache=torch.rand((blocks, block_size, 1, 4), generator=g) * 0.019 + 0.001,
        idx_k=randint8((blocks, block_size, 1, 128)),
        idx_k_scale=(torch.rand((blocks, block_size, 1, 1), generator=g) * 0.019 + 0.001).to(torch.float16),
        w_dq=randn((7168, 1536), 0.02), w_uq_qr=torch.round(wq * (127 / wq_amax)).to(torch.int8),
        w_uq_qr_scale=(wq_amax / 127).reshape(-1, 1).float().contiguous(), w_uk=randn((128, 128, 512), 0.05),
        w_dkv_kr=randn((7168, 576), 0.02), gamma_cq=(1 + randn((1536,), 0.1, torch.float32)).to(bf),
        gamma_ckv=(1 + randn((512,), 0.1, torch.float32)).to(bf),
        w_qb=torch.round(wi * (127 / wi_amax)).to(torch.int8), w_qb_scale=(wi_amax / 127).reshape(8192, 1).float().contiguous(),
        wk=randn((7168, 128), 0.02), w_proj=randn((7168, 64), 0.02), ln_gamma=torch.ones(128, dtype=bf),
        ln_beta=torch.zeros(128, dtype=bf), hadamard=sylvester_hadamard(128, bf))
    dev = torch.device(device)
    for k, v in list(vars(w).items()):
        if isinstance(v, torch.Tensor):
            setattr(w, k, v.to(dev))
    return w


def make_full_step_activations(t, seed, device):
    """Hidden states and rotary tables of one decode step: x bf16 [t, 7168], cos / sin bf16 [t, 64]."""
    g = torch.Generator().manual_seed(seed)
    ang = torch.rand((t, 64), generator=g) * 2 * math.pi
    dev = torch.device(device)
    return dict(x=torch.randn((t, 7168), generator=g).to(torch.bfloat16).to(dev), cos=torch.cos(ang).to(torch.bfloat16).to(dev),
                sin=torch.sin(ang).to(torch.bfloat16).to(dev))
