"""Shared helpers for the test-suite: fixture loading, seeded synthetic inputs."""
import hashlib
import json
import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def from_bits16(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).view(dtype)


def digest(t: torch.Tensor) -> str:
    t = t.contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        raw = t.view(torch.int16).numpy().tobytes()
    else:
        raw = t.numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()


def load_sfa_golden():
    z = np.load(os.path.join(GOLDEN, "sfa_small.npz"))
    bf = torch.bfloat16
    return dict(
        b=int(z["b"]), s1=int(z["s1"]), nq=int(z["nq"]), softmax_scale=float(z["softmax_scale"]),
        act_seq=torch.from_numpy(z["act_seq"]), q_nope=from_bits16(z["q_nope"], bf), q_rope=from_bits16(z["q_rope"], bf),
        k_nope=torch.from_numpy(z["k_nope"]), k_rope=from_bits16(z["k_rope"], bf),
        k_scales=torch.from_numpy(z["k_scales"]), topk_indices=torch.from_numpy(z["topk_indices"]),
        block_table=torch.from_numpy(z["block_table"]), out=from_bits16(z["out"], bf))


def load_sfa_bf16_golden():
    z = np.load(os.path.join(GOLDEN, "sfa_bf16_small.npz"))
    bf = torch.bfloat16
    return dict(
        b=int(z["b"]), s1=int(z["s1"]), nq=int(z["nq"]), softmax_scale=float(z["softmax_scale"]),
        act_seq=torch.from_numpy(z["act_seq"]), q_nope=from_bits16(z["q_nope"], bf), q_rope=from_bits16(z["q_rope"], bf),
        k_nope=from_bits16(z["k_nope"], bf), k_rope=from_bits16(z["k_rope"], bf), k_scales=None,
        topk_indices=torch.from_numpy(z["topk_indices"]), block_table=torch.from_numpy(z["block_table"]),
        out=from_bits16(z["out"], bf))


def load_scfa_golden():
    """DeepSeek-V4 sparse compress attention fixture (window keys + selected compressed keys + sinks)."""
    z = np.load(os.path.join(GOLDEN, "scfa_small.npz"))
    bf = torch.bfloat16
    return dict(
        b=int(z["b"]), nq=int(z["nq"]), cmp_ratio=int(z["cmp_ratio"]), block_size=int(z["block_size"]),
        win_size=int(z["win_size"]), topk=int(z["topk"]), softmax_scale=float(z["softmax_scale"]),
        actual_seq_q=torch.from_numpy(z["actual_seq_q"]), seqused_kv=torch.from_numpy(z["seqused_kv"]),
        q=from_bits16(z["q"], bf), cmp_kv=from_bits16(z["cmp_kv"], bf), ori_kv=from_bits16(z["ori_kv"], bf),
        cmp_sparse_indices=torch.from_numpy(z["cmp_sparse_indices"]),
        cmp_block_table=torch.from_numpy(z["cmp_block_table"]), ori_block_table=torch.from_numpy(z["ori_block_table"]),
        atten_sink=torch.from_numpy(z["atten_sink"]), out=from_bits16(z["out"], bf))


def load_cfa_golden():
    """DeepSeek-V4 compress flash attention fixture: its own query (two tokens per request) and output; caches,
    page tables, sinks and sequence lengths are those of the sparse compress attention fixture."""
    g = load_scfa_golden()
    z = np.load(os.path.join(GOLDEN, "cfa_small.npz"))
    bf = torch.bfloat16
    q = from_bits16(z["q"], bf)
    return dict(g, s1=int(z["s1"]), q=q, out=from_bits16(z["out"], bf),
                cmp_kv=g["cmp_kv"].reshape(-1, 128, 1, 512), ori_kv=g["ori_kv"].reshape(-1, 128, 1, 512))


def load_win_golden():
    """DeepSeek-V4 sliding-window attention fixture: the inputs of the sparse compress attention fixture (query,
    un-compressed cache, its page table, sinks, ragged query counts) with the window-only golden output."""
    g = load_scfa_golden()
    z = np.load(os.path.join(GOLDEN, "win_small.npz"))
    t = int(g["actual_seq_q"][-1])
    return dict(g, q=g["q"].reshape(t, g["nq"], 512), ori_kv=g["ori_kv"].reshape(-1, 128, 1, 512),
                out=from_bits16(z["out"], torch.bfloat16))


def load_sa_antiquant_golden():
    z = np.load(os.path.join(GOLDEN, "sa_antiquant_small.npz"))
    bf = torch.bfloat16
    return dict(
        b=int(z["b"]), s1=int(z["s1"]), nq=int(z["nq"]), softmax_scale=float(z["softmax_scale"]),
        act_seq=torch.from_numpy(z["act_seq"]), q_nope=from_bits16(z["q_nope"], bf), q_rope=from_bits16(z["q_rope"], bf),
        nope_cache=torch.from_numpy(z["nope_cache"]), topk_indices=torch.from_numpy(z["topk_indices"]),
        block_table=torch.from_numpy(z["block_table"]), out=from_bits16(z["out"], bf))


def load_indexer_golden():
    z = np.load(os.path.join(GOLDEN, "indexer_small.npz"))
    h = torch.float16
    return dict(
        b=int(z["b"]), s1=int(z["s1"]), act_seq=torch.from_numpy(z["act_seq"]), query=torch.from_numpy(z["query"]),
        q_scale=from_bits16(z["q_scale"], h), key=torch.from_numpy(z["key"]), k_scale=from_bits16(z["k_scale"], h),
        weights=from_bits16(z["weights"], h), block_table=torch.from_numpy(z["block_table"]),
        topk_res=torch.from_numpy(z["topk_res"]))


def load_prolog_golden():
    z = np.load(os.path.join(GOLDEN, "prolog_small.npz"))
    return dict(
        seed=int(z["seed"]), b=int(z["b"]), s1=int(z["s1"]), s2=int(z["s2"]), digests=json.loads(str(z["digests"])),
        q_int8=torch.from_numpy(z["q_int8"]), q_scale=from_bits16(z["q_scale"], torch.float16),
        k_cache=torch.from_numpy(z["k_cache"]), k_scale_cache=from_bits16(z["k_scale_cache"], torch.float16),
        weights=from_bits16(z["weights"], torch.float16))


def load_kat():
    with open(os.path.join(GOLDEN, "kat.json")) as f:
        return json.load(f)


# --------------------------------------------------------------------------
# seeded synthetic inputs
# --------------------------------------------------------------------------
def make_block_table(act_seq, block_size, gen, extra_blocks=0):
    """Random page assignment; unused slots are -1.  Returns (block_num, table)."""
    nblk = [math.ceil(int(s) / block_size) for s in act_seq]
    total = sum(nblk) + extra_blocks
    perm = torch.randperm(total, generator=gen).to(torch.int32)
    width = max(max(nblk), 1)
    table = torch.full((len(act_seq), width), -1, dtype=torch.int32)
    pos = 0
    for i, n in enumerate(nblk):
        table[i, :n] = perm[pos:pos + n]
        pos += n
    return total, table


def prolog_reference_inputs(seed, b, s1, s2):
    """Same RNG call order as the reference generator
    (deepseekv32_lightning_indexer_prolog_quant.py:105-158), so the same seed reproduces
    the tensors whose digests are stored in prolog_small.npz."""
    torch.manual_seed(seed)
    bf = torch.bfloat16
    h, qr, d, n, rd, bs = 7168, 1536, 128, 64, 64, 128
    x = torch.empty((b, s1, h), dtype=bf).uniform_(-1, 1)
    q_norm = torch.randint(low=-128, high=128, size=(b, s1, qr), dtype=torch.int8)
    q_norm_scale = torch.empty((b, s1, 1), dtype=torch.float32).uniform_(-1, 1)
    w_qb = torch.randint(low=-128, high=128, size=(qr, n * d), dtype=torch.int8)
    w_qb_scale = torch.empty((n * d, 1), dtype=torch.float32).uniform_(-1, 1)
    wk = torch.empty((h, d), dtype=bf).uniform_(-1, 1)
    w_proj = torch.empty((h, n), dtype=bf).uniform_(-1, 1)
    ln_gamma = torch.ones((d,), dtype=bf)
    ln_beta = torch.zeros((d,), dtype=bf)
    ang = torch.rand(b, s1, rd, dtype=torch.float32) * 2 * torch.pi
    cos = torch.cos(ang).to(bf)
    sin = torch.sin(ang).to(bf)
    hq = torch.empty((d, d), dtype=bf).uniform_(-1, 1)
    hk = torch.empty((d, d), dtype=bf).uniform_(-1, 1)
    k_bsnd = torch.randint(low=-128, high=128, size=(b, s2, 1, d), dtype=torch.int8)
    ks_bsnd = torch.empty((b, s2, 1, 1), dtype=torch.float16).uniform_(-1, 1)
    nblk_each = math.ceil(s2 / bs)
    block_num = nblk_each * b
    perm = torch.arange(0, block_num, 1)
    perm = perm[torch.randperm(perm.size(0))].to(torch.int32)
    block_table = perm.reshape(b, nblk_each).clone()
    cache_index = torch.empty((b, s1), dtype=torch.int64)
    for i in range(b):
        for j in range(s1):
            pos = s2 - s1 + j
            cache_index[i, j] = int(block_table[i, pos // bs]) * bs + pos % bs
    k_cache = torch.zeros((block_num, bs, 1, d), dtype=torch.int8)
    k_scale_cache = torch.zeros((block_num, bs, 1, 1), dtype=torch.float16)
    for i in range(b):
        for j in range(nblk_each):
            k_cache[block_table[i, j]] = k_bsnd[i, j * bs:(j + 1) * bs]
            k_scale_cache[block_table[i, j]] = ks_bsnd[i, j * bs:(j + 1) * bs]
    t = b * s1
    return {
        "token_x": x.reshape(t, h), "q_norm": q_norm.reshape(t, qr), "q_norm_scale": q_norm_scale.reshape(t, 1),
        "w_idx_qb": w_qb, "w_idx_qb_scale": w_qb_scale, "w_idx_k": wk, "w_idx_proj": w_proj,
        "layer_norm_gamma": ln_gamma, "layer_norm_beta": ln_beta, "cos_idx_rope": cos.reshape(t, rd),
        "sin_idx_rope": sin.reshape(t, rd), "hadamard_q": hq, "hadamard_k": hk, "idx_k_cache": k_cache,
        "idx_k_scale_cache": k_scale_cache, "idx_k_cache_index": cache_index.reshape(t),
        "idx_block_table": block_table,
    }


def gen_sfa_inputs(seed, act_seq, s1=1, nq=128, topk=2048, block_size=128, pad_short=True, extra_blocks=0):
    """Seeded synthetic SFA inputs in the operator's layouts: standard-normal bf16 queries and rope keys, full-range
    int8 latent keys, scales uniform in [0.001, 0.02]."""
    g = torch.Generator().manual_seed(seed)
    b = len(act_seq)
    t = b * s1
    bf = torch.bfloat16
    block_num, block_table = make_block_table(act_seq, block_size, g, extra_blocks)
    rows = block_num * block_size
    q_nope = torch.randn((t * nq, 512), generator=g).to(bf)
    q_rope = torch.randn((t * nq, 64), generator=g).to(bf)
    k_nope = torch.randint(-127, 128, (rows, 512), generator=g, dtype=torch.int8)
    k_rope = torch.randn((rows, 64), generator=g).to(bf)
    k_scales = torch.rand((rows, 4), generator=g) * 0.019 + 0.001
    topk_indices = torch.full((t, topk), -1, dtype=torch.int32)
    for bi, L in enumerate(act_seq):
        for si in range(s1):
            eff = max(int(L) - (s1 - 1 - si), 0)
            if eff >= topk:
                topk_indices[bi * s1 + si] = torch.randperm(eff, generator=g)[:topk].to(torch.int32)
            elif eff > 0:
                topk_indices[bi * s1 + si, :eff] = torch.randperm(eff, generator=g).to(torch.int32)
    return dict(q_nope=q_nope, q_rope=q_rope, k_nope=k_nope, k_rope=k_rope, k_scales=k_scales,
                topk_indices=topk_indices, block_table=block_table,
                act_seq=torch.tensor(act_seq, dtype=torch.int32), b=b, s1=s1, nq=nq,
                softmax_scale=576 ** -0.5, topk=topk, block_size=block_size)


def load_prolog_v4_golden():
    z = np.load(os.path.join(GOLDEN, "prolog_v4_small.npz"))
    return dict(t=int(z["t"]), digests=json.loads(str(z["digests"])), q=torch.from_numpy(z["q"]),
                weights=from_bits16(z["weights"], torch.float16), q_scale=from_bits16(z["q_scale"], torch.float16))


def prolog_v4_reference_inputs(t):
    """Same RNG call order and arithmetic as the reference generator of the DeepSeek-V4 indexer prolog test
    (models/deepseek_v4/test_lightning_indexer_prolog_quant_v4.py:77-110 with gen_uniform_data and quant_golden of
    utils/golden/common_func.py:16-35,72-82), so the tensors reproduce the digests stored in prolog_v4_small.npz."""
    torch.manual_seed(42)
    bf = torch.bfloat16

    def uni(shape, lo, hi, dtype):
        if dtype == torch.int8:
            return torch.randint(low=lo, high=hi, size=shape, dtype=dtype)
        return lo + (hi - lo) * torch.rand(shape, dtype=dtype)

    def quant(x):
        xf = x.to(torch.float32)
        s = 127.0 / torch.amax(torch.abs(xf), dim=-1, keepdim=True)
        y = torch.round(xf * s).to(torch.int32)
        return torch.trunc(y.to(x.dtype)).to(torch.int8), 1.0 / s

    qr_ori = uni([t, 1024], -1, 1, torch.int8)
    wq_ori = uni([1024, 8192], -1, 1, torch.int8)
    x = uni([t, 4096], -1, 1, bf)
    weights_proj = uni([4096, 64], -0.1, 0.1, bf)
    cos = uni([t, 64], -1, 1, bf)
    sin = uni([t, 64], -1, 1, bf)
    hadamard = uni([128, 128], -1, 1, bf)
    qr, qr_scale = quant(qr_ori)
    wq, wq_scale = quant(wq_ori.t())
    return dict(qr=qr, idx_wq_b=wq.t().contiguous(), x=x, weights_proj=weights_proj, cos=cos, sin=sin, hadamard=hadamard,
                qr_scale=qr_scale, idx_wq_b_scale=wq_scale)


def gen_prolog_v4_inputs(seed, t, h=4096):
    """Seeded full-range inputs of the DeepSeek-V4 indexer prolog (the reference generator only produces the int8
    values -127 and 0): uniform int8 operands, scales of realistic size, unit-circle cos / sin, a random hadamard."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    ang = torch.rand((t, 64), generator=g) * 2 * torch.pi
    return dict(
        qr=torch.randint(-127, 128, (t, 1024), generator=g, dtype=torch.int8),
        idx_wq_b=torch.randint(-127, 128, (1024, 8192), generator=g, dtype=torch.int8),
        x=torch.randn((t, h), generator=g).to(bf), weights_proj=(torch.randn((h, 64), generator=g) * 0.02).to(bf),
        cos=torch.cos(ang).to(bf), sin=torch.sin(ang).to(bf),
        hadamard=(torch.rand((128, 128), generator=g) * 2 - 1).to(bf),
        qr_scale=torch.rand((t, 1), generator=g) * 0.02 + 0.001,
        idx_wq_b_scale=torch.rand((8192, 1), generator=g) * 0.002 + 0.0001)


def load_mla_v4_golden():
    z = np.load(os.path.join(GOLDEN, "mla_v4_small.npz"))
    bf = torch.bfloat16
    return dict(t=int(z["t"]), digests=json.loads(str(z["digests"])), q=from_bits16(z["q"], bf),
                kv=from_bits16(z["kv"], bf), qr=torch.from_numpy(z["qr"]), qr_scale=torch.from_numpy(z["qr_scale"]))


def mla_v4_reference_inputs(t, heads=64, h=4096):
    """Same RNG call order as the reference generator of the DeepSeek-V4 MLA prolog test
    (models/deepseek_v4/test_mla_prolog_quant_v4.py:192-233, seed 5), so the tensors reproduce the digests stored in
    mla_v4_small.npz."""
    torch.manual_seed(5)
    bf = torch.bfloat16
    x = torch.empty([t, h], dtype=bf).uniform_(-1, 1)
    wq_a = torch.empty([h, 1024], dtype=bf).uniform_(-0.1, 0.1)
    wq_b = torch.empty([1024, heads * 512], dtype=bf).uniform_(-0.1, 0.1)
    w_kv = torch.empty([h, 512], dtype=bf).uniform_(-0.1, 0.1)
    wf = wq_b.to(torch.float32)                       # per-column int8 quantisation of wq_b
    s = 127 / torch.max(torch.abs(wf), dim=-2, keepdim=True)[0]
    wq_b_i8 = torch.trunc(torch.round(wf * s).to(torch.int32).to(torch.float16)).to(torch.int8)
    gamma_cq = torch.empty([1024], dtype=bf).uniform_(-1, 1)
    gamma_ckv = torch.empty([512], dtype=bf).uniform_(-1, 1)
    cos = torch.empty([t, 64], dtype=bf).uniform_(-1, 1)
    sin = torch.empty([t, 64], dtype=bf).uniform_(-1, 1)
    return dict(x=x, wq_a=wq_a, wq_b=wq_b_i8, w_kv=w_kv, cos=cos, sin=sin, gamma_cq=gamma_cq, gamma_ckv=gamma_ckv,
                wq_b_scale=1 / s)


def load_mla_v4_bf16_golden():
    z = np.load(os.path.join(GOLDEN, "mla_v4_bf16_small.npz"))
    bf = torch.bfloat16
    return dict(t=int(z["t"]), digests=json.loads(str(z["digests"])), q=from_bits16(z["q"], bf),
                kv=from_bits16(z["kv"], bf), qr=from_bits16(z["qr"], bf))


def mla_v4_bf16_reference_inputs(t, heads=64, h=4096):
    """The reference generator of the MLA prolog test without quantisation
    (models/deepseek_v4/test_mla_prolog_v4.py:161-199, seed 5): the same draws as mla_v4_reference_inputs, with
    wq_b kept in bf16."""
    torch.manual_seed(5)
    bf = torch.bfloat16
    x = torch.empty([t, h], dtype=bf).uniform_(-1, 1)
    wq_a = torch.empty([h, 1024], dtype=bf).uniform_(-0.1, 0.1)
    wq_b = torch.empty([1024, heads * 512], dtype=bf).uniform_(-0.1, 0.1)
    w_kv = torch.empty([h, 512], dtype=bf).uniform_(-0.1, 0.1)
    gamma_cq = torch.empty([1024], dtype=bf).uniform_(-1, 1)
    gamma_ckv = torch.empty([512], dtype=bf).uniform_(-1, 1)
    cos = torch.empty([t, 64], dtype=bf).uniform_(-1, 1)
    sin = torch.empty([t, 64], dtype=bf).uniform_(-1, 1)
    return dict(x=x, wq_a=wq_a, wq_b=wq_b, w_kv=w_kv, cos=cos, sin=sin, gamma_cq=gamma_cq, gamma_ckv=gamma_ckv)


def load_hc_pre_golden():
    z = np.load(os.path.join(GOLDEN, "hc_pre_small.npz"))
    return dict(t=int(z["t"]), digests=json.loads(str(z["digests"])), y=from_bits16(z["y"], torch.bfloat16),
                post=torch.from_numpy(z["post"]), comb=torch.from_numpy(z["comb"]))


def hc_pre_reference_inputs(t):
    """The reference generator of the hyper-connection pre-mix test (models/deepseek_v4/test_hc_pre.py:141-149,
    seed 42): reproduces the digests stored in hc_pre_small.npz."""
    torch.manual_seed(42)
    x = torch.empty((t, 4, 4096), dtype=torch.bfloat16).uniform_(-1, 1)
    hc_fn = torch.empty((24, 4 * 4096), dtype=torch.float32).uniform_(-1, 1)
    hc_scale = torch.empty((3,), dtype=torch.float32).uniform_(-1, 1)
    hc_base = torch.empty((24,), dtype=torch.float32).uniform_(-1, 1)
    return dict(x=x, hc_fn=hc_fn, hc_scale=hc_scale, hc_base=hc_base)


def gen_hc_pre_inputs(seed, t, fn_scale=0.02):
    """Seeded inputs with mixing logits of order one (the reference generator's saturate every sigmoid)."""
    g = torch.Generator().manual_seed(seed)
    return dict(x=torch.randn((t, 4, 4096), generator=g).to(torch.bfloat16),
                hc_fn=torch.randn((24, 4 * 4096), generator=g) * fn_scale,
                hc_scale=torch.rand((3,), generator=g) + 0.5, hc_base=torch.randn((24,), generator=g) * 0.5)


COMPRESSOR_CASES = {   # name: (ratio, rotate, d, batch, tokens per request, start positions) -- as in make_golden.py
    "r128": (128, False, 512, 3, 2, [254, 126, 300]),
    "r4": (4, False, 512, 4, 2, [255, 2, 6, 9]),
    "r4_rot": (4, True, 128, 4, 2, [255, 3, 10, 1]),
}


def compressor_reference_inputs(name):
    """The reference generator of the compressor test (models/deepseek_v4/test_compressor.py:190-236, seed 42) with
    the state history make_golden.py adds (seed 7); reproduces the digests stored in compressor_small.npz."""
    ratio, rotate, d, bsz, seq, starts = COMPRESSOR_CASES[name]
    torch.manual_seed(42)
    bf = torch.bfloat16
    coff = 2 if ratio == 4 else 1
    x = torch.rand((bsz, seq, 4096), dtype=bf)
    rows = min(bsz * seq, bsz * seq // ratio + bsz)
    sin = torch.rand((rows, 64), dtype=bf)
    cos = torch.rand((rows, 64), dtype=bf)
    wkv = torch.rand((coff * d, 4096), dtype=bf)
    wgate = torch.rand((coff * d, 4096), dtype=bf)
    ape = torch.rand((ratio, coff * d), dtype=torch.float32)
    weight = torch.ones(d, dtype=torch.float32)
    if ratio == 4:
        table = torch.ones(bsz, 100, dtype=torch.int32) + torch.arange(bsz, dtype=torch.int32).view(-1, 1) * 2
    else:
        table = torch.arange(100, dtype=torch.int32) % 2 + 1 + torch.arange(bsz, dtype=torch.int32).view(-1, 1) * 2
    nblk = int(table.max()) + 1
    hadamard = torch.rand((d, d), dtype=bf) * (d ** -0.5)
    g = torch.Generator().manual_seed(7)
    kv_state = torch.rand((nblk, 128, coff * d), generator=g)
    score_state = torch.rand((nblk, 128, coff * d), generator=g)
    return dict(x=x, sin=sin, cos=cos, wkv=wkv, wgate=wgate, ape=ape, weight=weight, kv_state=kv_state,
                score_state=score_state, table=table, hadamard=hadamard,
                start_pos=torch.tensor(starts, dtype=torch.int32), ratio=ratio, rotate=rotate, d=d)


def load_compressor_golden(name):
    z = np.load(os.path.join(GOLDEN, "compressor_small.npz"))
    return dict(digests=json.loads(str(z[name + "_digests"])), out=from_bits16(z[name + "_out"], torch.bfloat16),
                kv_state_sum=torch.from_numpy(z[name + "_kv_state_sum"]),
                score_state_sum=torch.from_numpy(z[name + "_score_state_sum"]))


def gen_mla_v4_inputs(seed, t, heads=64, h=4096):
    """Seeded inputs of the DeepSeek-V4 MLA prolog with realistic distributions: normal activations and weights,
    gamma near one, unit-circle cos / sin repeated per rotary pair."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    wq = torch.randn((1024, heads * 512), generator=g) * 0.03
    s = 127 / wq.abs().amax(0, keepdim=True)
    ang = torch.rand((t, 32), generator=g) * 2 * torch.pi
    return dict(
        x=torch.randn((t, h), generator=g).to(bf), wq_a=(torch.randn((h, 1024), generator=g) * 0.02).to(bf),
        wq_b=torch.round(wq * s).to(torch.int8), w_kv=(torch.randn((h, 512), generator=g) * 0.02).to(bf),
        cos=torch.cos(ang).repeat_interleave(2, -1).to(bf), sin=torch.sin(ang).repeat_interleave(2, -1).to(bf),
        gamma_cq=(1 + 0.1 * torch.randn(1024, generator=g)).to(bf),
        gamma_ckv=(1 + 0.1 * torch.randn(512, generator=g)).to(bf), wq_b_scale=(1 / s).float())


def gen_scfa_inputs(seed, ori_seq, s1_list, nq=64, topk=512, win_size=128, cmp_ratio=4, block_size=128, holes=0,
                    scale=1.0):
    """Seeded synthetic inputs of the DeepSeek-V4 sparse compress attention in the operator's layouts: queries,
    both caches and the sinks uniform in [-scale, scale) (the reference test uses [-1, 1)), pages randomly
    permuted, selected indices a random subset of each request's compressed positions.  `holes`: this many
    entries of every index row are replaced by -1."""
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    b = len(ori_seq)
    seq_q = [0]
    for s1 in s1_list:
        seq_q.append(seq_q[-1] + s1)
    t = seq_q[-1]
    cmp_seq = [int(L) // cmp_ratio for L in ori_seq]
    ori_blocks, ori_bt = make_block_table([max(int(L), 1) for L in ori_seq], block_size, g, 1)
    cmp_blocks, cmp_bt = make_block_table([max(L, 1) for L in cmp_seq], block_size, g, 1)

    def uni(shape):
        return ((torch.rand(shape, generator=g) * 2 - 1) * scale).to(bf)

    q = uni((t * nq, 512))
    ori_kv = uni((ori_blocks * block_size, 512))
    cmp_kv = uni((cmp_blocks * block_size, 512))
    sink = (torch.rand((nq,), generator=g) * 2 - 1) * scale
    idx = torch.full((t, topk), -1, dtype=torch.int32)
    for bi in range(b):
        for si in range(s1_list[bi]):
            tok = seq_q[bi] + si
            n = min(cmp_seq[bi], topk)
            if n > 0:
                idx[tok, :n] = torch.randperm(cmp_seq[bi], generator=g)[:n].to(torch.int32)
            if holes:
                idx[tok, torch.randperm(topk, generator=g)[:holes]] = -1
    return dict(q=q, ori_kv=ori_kv, cmp_kv=cmp_kv, atten_sink=sink, cmp_sparse_indices=idx, ori_block_table=ori_bt,
                cmp_block_table=cmp_bt, actual_seq_q=torch.tensor(seq_q, dtype=torch.int32),
                seqused_kv=torch.tensor(ori_seq, dtype=torch.int32), b=b, nq=nq, topk=topk, win_size=win_size,
                cmp_ratio=cmp_ratio, block_size=block_size, softmax_scale=512 ** -0.5)


def gen_indexer_inputs(seed, act_seq, s1=1, block_size=128, extra_blocks=0):
    g = torch.Generator().manual_seed(seed)
    b = len(act_seq)
    t = b * s1
    block_num, block_table = make_block_table(act_seq, block_size, g, extra_blocks)
    query = torch.randint(-127, 128, (t, 64, 128), generator=g, dtype=torch.int8)
    q_scale = (torch.rand((t, 64), generator=g) * 0.019 + 0.001).to(torch.float16)
    weights = (torch.randn((t, 64), generator=g) * 0.1).to(torch.float16)
    key = torch.randint(-127, 128, (block_num, block_size, 1, 128), generator=g, dtype=torch.int8)
    k_scale = (torch.rand((block_num, block_size, 1), generator=g) * 0.019 + 0.001).to(torch.float16)
    return dict(query=query, q_scale=q_scale, weights=weights, key=key, k_scale=k_scale, block_table=block_table,
                act_seq=torch.tensor(act_seq, dtype=torch.int32), b=b, s1=s1)


def load_mla_golden():
    z = np.load(os.path.join(GOLDEN, "mla_small.npz"))
    bf = torch.bfloat16
    return dict(
        seed=int(z["seed"]), b=int(z["b"]), s1=int(z["s1"]), s2=int(z["s2"]), digests=json.loads(str(z["digests"])),
        q_nope=from_bits16(z["q_nope"], bf), q_rope=from_bits16(z["q_rope"], bf), q_norm=torch.from_numpy(z["q_norm"]),
        q_norm_scale=torch.from_numpy(z["q_norm_scale"]), kv_cache=torch.from_numpy(z["kv_cache"]),
        kr_cache=from_bits16(z["kr_cache"], bf), ks_cache=torch.from_numpy(z["ks_cache"]))


def _per_row_quant(t, dim):
    """quant() of the MLA golden (deepseekv32_mla_indexer_prolog_quant.py:35-53) along `dim`."""
    f = t.to(torch.float32)
    amax = torch.max(torch.abs(f), dim=dim, keepdim=True)[0]
    s = 127 / amax
    q = torch.trunc(torch.round(f * s).to(torch.int32).to(torch.float16)).to(torch.int8)
    return q, 1 / s


def mla_reference_inputs(seed, b, s1, s2):
    """Same RNG call order as the reference generator (deepseekv32_mla_indexer_prolog_quant.py:161-333,
    is_quant = (False, True), no smoothing), so the same seed reproduces the tensors whose digests are stored
    in mla_small.npz."""
    torch.manual_seed(seed)
    bf = torch.bfloat16
    h, qr, n, nope, rope, lora, bs = 7168, 1536, 128, 128, 64, 512, 128
    nblk_each = math.ceil(s2 / bs)
    block_num = nblk_each * b
    perm = torch.arange(0, block_num, 1)
    perm = perm[torch.randperm(perm.size(0))].to(torch.int32)
    block_table = perm.reshape(b, nblk_each).clone()
    cache_index = torch.empty((b, s1), dtype=torch.int64)
    for i in range(b):
        for j in range(s1):
            pos = s2 - s1 + j
            cache_index[i, j] = int(block_table[i, pos // bs]) * bs + pos % bs
    x = torch.empty([b, s1, h]).uniform_(-1, 1).to(bf)
    w_dq = torch.empty([h, qr]).uniform_(-0.1, 0.1).to(bf)
    w_uqqr = torch.empty([qr, n * (nope + rope)]).uniform_(-0.1, 0.1).to(bf)
    w_dkvkr = torch.empty([h, lora + rope]).uniform_(-0.1, 0.1).to(bf)
    w_uqqr, w_qb_scale = _per_row_quant(w_uqqr, -2)
    w_uk = torch.empty([n, nope, lora]).uniform_(-0.1, 0.1).to(bf)
    gamma_cq = torch.empty([qr]).uniform_(-1, 1).to(bf)
    gamma_ckv = torch.empty([lora]).uniform_(-1, 1).to(bf)
    cos = torch.empty([b, s1, rope]).uniform_(-0.1, 0.1).to(bf)
    sin = torch.empty([b, s1, rope]).uniform_(-0.1, 0.1).to(bf)
    k_bsnd = torch.empty([b, s2, 1, lora + rope]).uniform_(-1, 1).to(bf)
    k_pad = torch.zeros((b, nblk_each * bs, 1, lora + rope)).to(bf)
    k_pad[:, :s2] = k_bsnd
    k_cache = torch.zeros([block_num, bs, 1, lora + rope]).to(bf)
    for i in range(b):
        for j in range(nblk_each):
            k_cache[block_table[i, j]] = k_pad[i, j * bs:(j + 1) * bs]
    kv_cache = k_cache[:, :, :, :lora]
    kr_cache = k_cache[:, :, :, lora:].contiguous()
    kv_q, kv_s = _per_row_quant(kv_cache.reshape(-1, 4, lora // 4), -1)
    t = b * s1
    return dict(x=x.reshape(t, h), w_dq=w_dq, w_uqqr=w_uqqr, w_qb_scale=w_qb_scale, w_uk=w_uk, w_dkvkr=w_dkvkr,
                gamma_cq=gamma_cq, gamma_ckv=gamma_ckv, cos=cos.reshape(t, rope), sin=sin.reshape(t, rope),
                cache_index=cache_index.reshape(t), kv_cache=kv_q.reshape(block_num, bs, 1, lora), kr_cache=kr_cache,
                ks_cache=kv_s.reshape(block_num, bs, 1, 4), block_table=block_table)


# --------------------------------------------------------------------------
# page-grouped 8-bit-float indexer prologs (python/tests/st/operator/pg/ in the reference)
# --------------------------------------------------------------------------
PG_H, PG_QLORA, PG_HEADS, PG_D, PG_ROPE, PG_BS = 2560, 1024, 24, 128, 64, 128
PG_GROUP = 41    # caches of this many row widths share one page of the page-grouped buffer


def load_pg_prolog_mxfp8_golden():
    z = np.load(os.path.join(GOLDEN, "pg_prolog_mxfp8_small.npz"))
    return dict(seed=int(z["seed"]), b=int(z["b"]), s1=int(z["s1"]), s2=int(z["s2"]), digests=json.loads(str(z["digests"])),
                q=torch.from_numpy(z["q"]), q_scale=torch.from_numpy(z["q_scale"]), k=torch.from_numpy(z["k"]),
                k_scale=torch.from_numpy(z["k_scale"]), weights=torch.from_numpy(z["weights"]),
                cache_index=torch.from_numpy(z["cache_index"]))


def pg_prolog_reference_inputs(seed, b, s1, s2):
    """Same RNG call order as the reference generator (test_pg_lightning_indexer_prolog_quant_mxfp8.py:160-222), so the
    same seed reproduces the tensors whose digests are stored in pg_prolog_mxfp8_small.npz.  The key cache and its
    scale cache are strided views into one page-grouped byte buffer, as the reference builds them."""
    torch.manual_seed(seed)
    bf, f8, e8 = torch.bfloat16, torch.float8_e4m3fn, torch.float8_e8m0fnu
    h, qr, d, n, rd, bs = PG_H, PG_QLORA, PG_D, PG_HEADS, PG_ROPE, PG_BS
    x = torch.empty((b, s1, h), dtype=bf).uniform_(-1, 1)
    q_norm = torch.empty((b, s1, qr), dtype=torch.float32).uniform_(-10, 10).to(f8)
    q_norm_scale = torch.empty((b, s1, qr // 32), dtype=torch.float32).uniform_(0, 1).to(e8)
    w_qb = torch.empty((qr, n * d), dtype=torch.float32).uniform_(-10, 10).to(f8)
    w_qb_scale = torch.empty((qr // 64, n * d, 2), dtype=torch.float32).uniform_(0, 1).to(e8)
    wk = torch.empty((h, d), dtype=bf).uniform_(-1, 1)
    w_proj = torch.empty((h, n), dtype=bf).uniform_(-1, 1)
    gamma = torch.ones((d,), dtype=bf)
    ang = torch.rand(b, s1, rd, dtype=torch.float32) * 2 * torch.pi
    cos, sin = torch.cos(ang).to(bf), torch.sin(ang).to(bf)
    hq = torch.empty((d, d), dtype=bf).uniform_(-1, 1)
    hk = torch.empty((d, d), dtype=bf).uniform_(-1, 1)
    k_bsnd = torch.empty((b, s2, 1, d), dtype=torch.float32).uniform_(-10, 10).to(f8)
    ks_bsnd = torch.empty((b, s2, 1, 1), dtype=torch.float32).uniform_(-1, 1)
    nblk_each = math.ceil(s2 / bs)
    block_num = nblk_each * b
    perm = torch.arange(0, block_num, 1)
    perm = perm[torch.randperm(perm.size(0))].to(torch.int32)
    block_table = perm.reshape(b, nblk_each).clone()
    cache_index = torch.empty((b, s1), dtype=torch.int64)
    for i in range(b):
        for j in range(s1):
            pos = s2 - s1 + j
            cache_index[i, j] = int(block_table[i, pos // bs]) * bs + pos % bs
    pages = torch.randint(0, 256, (block_num, bs * d * PG_GROUP), dtype=torch.uint8)
    k_cache = pages.view(f8)[:, bs * d:2 * bs * d].view(block_num, bs, 1, d)
    off = 2 * bs * d // 4
    k_scale_cache = pages.view(torch.float32)[:, off:off + bs].view(block_num, bs, 1, 1)
    for i in range(b):
        for j in range(nblk_each):
            k_cache[block_table[i, j]] = k_bsnd[i, j * bs:(j + 1) * bs]
            k_scale_cache[block_table[i, j]] = ks_bsnd[i, j * bs:(j + 1) * bs]
    return {
        "token_x": x, "q_norm": q_norm, "q_norm_scale": q_norm_scale, "w_idx_qb": w_qb, "w_idx_qb_scale": w_qb_scale,
        "w_idx_k": wk, "w_idx_proj": w_proj, "rms_norm_gamma": gamma, "cos_idx_rope": cos, "sin_idx_rope": sin,
        "hadamard_q": hq, "hadamard_k": hk, "idx_k_cache": k_cache, "idx_k_scale_cache": k_scale_cache,
        "idx_k_cache_index": cache_index, "idx_block_table": block_table, "act_seq": torch.tensor([s2] * b),
        "pages": pages,
    }


def pg_digest(v: torch.Tensor) -> str:
    v = v.contiguous()
    if v.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
        v = v.view(torch.uint8)
    elif v.dtype in (torch.bfloat16, torch.float16):
        v = v.view(torch.int16)
    return hashlib.sha256(v.numpy().tobytes()).hexdigest()


def gen_pg_prolog_inputs(seed, t, fmt, nblocks=4):
    """Seeded inputs of the page-grouped prolog in either format, as the operator's 2-D arguments (CPU tensors).
    fmt "mxfp8": float8_e4m3fn codes with E8M0 scales per 32 reduction elements; fmt "hif8": uint8 HiF8 codes with
    an fp32 scale per token / per output column.  The caches are strided views into a page-grouped byte buffer."""
    from oracle import pg_prolog_oracle as pgo
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    h, qr, d, n, rd, bs = PG_H, PG_QLORA, PG_D, PG_HEADS, PG_ROPE, PG_BS
    u = lambda shape, a, lo=None: torch.empty(shape, dtype=torch.float32).uniform_(-a if lo is None else lo, a, generator=g)  # noqa: E731
    x = u((t, h), 1.0).to(bf)
    if fmt == "mxfp8":
        q_norm = u((t, qr), 10.0).to(torch.float8_e4m3fn)
        q_norm_scale = u((t, qr // 32), 1.0, 0.0).to(torch.float8_e8m0fnu)
        w_qb = u((qr, n * d), 10.0).to(torch.float8_e4m3fn)
        w_qb_scale = u((qr // 64, n * d, 2), 1.0, 0.0).to(torch.float8_e8m0fnu)
    else:
        q_norm = pgo.hif8_encode(u((t, qr), 10.0))
        q_norm_scale = u((t, 1), 1.0, 0.05)
        w_qb = pgo.hif8_encode(u((qr, n * d), 10.0))
        w_qb_scale = u((1, n * d), 1.0, 0.05)
    wk = u((h, d), 1.0).to(bf)
    w_proj = u((h, n), 1.0).to(bf)
    gamma = u((1, d), 1.5, 0.5).to(bf)
    ang = torch.rand((t, rd), generator=g) * 2 * torch.pi
    cos, sin = torch.cos(ang).to(bf), torch.sin(ang).to(bf)
    hq, hk = u((d, d), 1.0).to(bf), u((d, d), 1.0).to(bf)
    pages = torch.randint(0, 256, (nblocks, bs * d * PG_GROUP), dtype=torch.uint8, generator=g)
    cache_index = torch.randperm(nblocks * bs, generator=g)[:t].to(torch.int64).reshape(t, 1)
    return dict(x=x, q_norm=q_norm, q_norm_scale=q_norm_scale, w_qb=w_qb, w_qb_scale=w_qb_scale, wk=wk, w_proj=w_proj,
                gamma_k=gamma, cos=cos, sin=sin, hadamard_q=hq, hadamard_k=hk, pages=pages, cache_index=cache_index)


def pg_cache_views(pages: torch.Tensor, fmt: str):
    """(key cache [blocks, 128, 1, 128], key scale cache [blocks, 128, 1, 1] fp32) as strided views into `pages`."""
    bs, d = PG_BS, PG_D
    blocks = pages.shape[0]
    kc = pages.view(torch.float8_e4m3fn) if fmt == "mxfp8" else pages
    k_cache = kc[:, bs * d:2 * bs * d].view(blocks, bs, 1, d)
    off = 2 * bs * d // 4
    k_scale_cache = pages.view(torch.float32)[:, off:off + bs].view(blocks, bs, 1, 1)
    return k_cache, k_scale_cache
