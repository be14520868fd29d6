"""CPU oracle for the page-grouped lightning-indexer prologs with 8-bit float formats (MXFP8 and HiF8).

TEST INFRASTRUCTURE ONLY: imported by the test-suite; the product package never imports it.

Reference files (relative to the reference project root, under python/tests/st/operator/pg/):
  lightning_indexer_prolog_quant_mxfp8_impl.py:230-401   the operator (rounding points restated by `pg_prolog`)
  lightning_indexer_prolog_quant_hif8_impl.py:230-406    the HiF8 form of it
  test_pg_lightning_indexer_prolog_quant_mxfp8.py:272-345 the fp32 torch-CPU golden (restated by `pg_prolog_golden`)
  compare_2_1.py:92-133                                   the three-way accuracy rule (restated by `triple_compare`)
HiF8 bit layout: framework/src/interface/machine/device/tilefwk/aicore_print_base.h:361-484 (DecodeHf8), restated
by `hif8_decode_table`.

Parity pins.  MXFP8: `pg_prolog_golden` is pinned bit for bit by tests/golden/pg_prolog_mxfp8_small.npz, made by
tests/golden/make_golden.py from the unmodified reference golden.  HiF8: the reference's golden converts to and from
HiF8 with an NPU library call (torch_npu.npu_dtype_cast), which cannot run here; the DECODE direction follows the
reference's own decoder line by line, the ENCODE direction (round to the nearest representable value, ties away from
zero, magnitudes above the largest finite value saturate to it) is this file's reading of the published format:
parity unpinned for the encode rounding of HiF8.
"""
from __future__ import annotations

import math

import numpy as np
import torch

HEAD_DIM = 128
ROPE_DIM = 64
FP8_MAX = 448.0      # float8_e4m3fn
HIF8_MAX = 32768.0   # 2^15, the largest finite HiF8 value


# ----------------------------------------------------------------------------
# HiF8
# ----------------------------------------------------------------------------
def hif8_decode_table() -> np.ndarray:
    """float32 value of every HiF8 code (aicore_print_base.h:361-484).  Bit 7 is the sign; the lower seven bits are
    a prefix-coded exponent width, a sign-magnitude exponent with an implied leading one, and the mantissa:
      0000mmm  2^(m-23) for m = 1..7; m = 0 is zero (sign 0) or NaN (sign 1)
      0001mmm  exponent 0, 3 mantissa bits
      001emmm  exponent +1 / -1 (e = 0 / 1), 3 mantissa bits
      01semmm  exponent +-(2 + e), 3 mantissa bits
      10seemm  exponent +-(4 + ee), 2 mantissa bits
      11seeem  exponent +-(8 + eee), 1 mantissa bit; exponent +15 with mantissa 1 is infinity."""
    out = np.zeros(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        low = code & 0x7F
        if (low >> 3) == 0:
            m = low & 7
            if m == 0:
                out[code] = np.nan if code & 0x80 else 0.0
            else:
                out[code] = sign * 2.0 ** (m - 23)
            continue
        if (low >> 3) == 1:
            ev, mant, bits = 0, low & 7, 3
        elif (low >> 4) == 1:
            ev, mant, bits = (-1 if (low >> 3) & 1 else 1), low & 7, 3
        elif (low >> 5) == 1:
            eb = (low >> 3) & 3
            ev, mant, bits = (2 + (eb & 1)) * (-1 if eb >> 1 else 1), low & 7, 3
        elif (low >> 5) == 2:
            eb = (low >> 2) & 7
            ev, mant, bits = (4 + (eb & 3)) * (-1 if eb >> 2 else 1), low & 3, 2
        else:
            eb = (low >> 1) & 15
            ev, mant, bits = (8 + (eb & 7)) * (-1 if eb >> 3 else 1), low & 1, 1
            if ev == 15 and mant == 1:
                out[code] = sign * np.inf
                continue
        out[code] = sign * 2.0 ** ev * (1.0 + mant / (1 << bits))
    return out


def hif8_decode(codes: torch.Tensor) -> torch.Tensor:
    table = torch.from_numpy(hif8_decode_table())
    return table[codes.to(torch.int64) & 0xFF]


def hif8_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> HiF8 code (uint8): nearest representable magnitude, ties away from zero, saturating at 2^15; the
    smallest magnitudes round between zero and 2^-22; NaN gives the NaN code 0x80."""
    table = hif8_decode_table()
    pos_codes = np.array([c for c in range(128) if np.isfinite(table[c])], dtype=np.int64)
    pos_vals = table[pos_codes].astype(np.float64)
    order = np.argsort(pos_vals, kind="stable")
    pos_codes, pos_vals = pos_codes[order], pos_vals[order]          # ascending magnitudes, 0 first
    xf = x.detach().to(torch.float32).cpu().numpy()
    mag = np.minimum(np.abs(xf).astype(np.float64), HIF8_MAX)
    hi = np.clip(np.searchsorted(pos_vals, mag, side="left"), 0, len(pos_vals) - 1)
    lo = np.clip(hi - 1, 0, len(pos_vals) - 1)
    take_hi = (pos_vals[hi] - mag) <= (mag - pos_vals[lo])           # a tie goes to the larger magnitude
    idx = np.where(take_hi, hi, lo)
    code = pos_codes[idx]
    neg = np.signbit(xf) & (pos_vals[idx] != 0.0)                     # there is no negative zero
    code = np.where(neg, code | 0x80, code)
    code = np.where(np.isnan(xf), 0x80, code)
    return torch.from_numpy(code.astype(np.uint8)).reshape(x.shape)


# ----------------------------------------------------------------------------
# shared pieces
# ----------------------------------------------------------------------------
def e8m0_to_float(s: torch.Tensor) -> torch.Tensor:
    """E8M0 scale code (uint8 view of float8_e8m0fnu) -> 2^(code - 127) as fp32 (code 255 is NaN)."""
    e = s.to(torch.int32) - 127
    return torch.ldexp(torch.ones(e.shape, dtype=torch.float32), e)


def expand_mx_scales(q_norm_scale_u8: torch.Tensor, w_qb_scale_u8: torch.Tensor, q_lora: int, n: int):
    """Per-element fp32 scales of the two MXFP8 operands: one scale per 32 consecutive reduction elements.
    q_norm_scale [t, q_lora/32]; w_qb_scale [q_lora/64, n, 2] -- block kb of column c is w_qb_scale[kb // 2, c, kb % 2]
    (test_pg_lightning_indexer_prolog_quant_mxfp8.py:291-295)."""
    qs = e8m0_to_float(q_norm_scale_u8).repeat_interleave(32, dim=-1)
    ws = e8m0_to_float(w_qb_scale_u8).transpose(1, 2).reshape(q_lora // 32, n).repeat_interleave(32, dim=0)
    return qs, ws


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(torch.float32)


def _quant(x: torch.Tensor, fmt: str):
    """Per-row dynamic quantisation as the operator does it (lightning_indexer_prolog_quant_mxfp8_impl.py:111-147,
    hif8 form :111-147): scale = amax * fl(1 / max), codes = cast(x / scale)."""
    amax = x.abs().amax(dim=-1, keepdim=True)
    if fmt == "mxfp8":
        scale = amax * np.float32(1.0 / FP8_MAX)
        y = (x / scale).clamp(-FP8_MAX, FP8_MAX)           # saturating cast
        return y.to(torch.float8_e4m3fn), scale
    scale = amax * np.float32(1.0 / HIF8_MAX)
    return hif8_encode(x / scale), scale


def codes_to_float(codes: torch.Tensor, fmt: str) -> torch.Tensor:
    if fmt == "mxfp8":
        return codes.view(torch.float8_e4m3fn).to(torch.float32) if codes.dtype == torch.uint8 else codes.to(torch.float32)
    return hif8_decode(codes)


# ----------------------------------------------------------------------------
# the operator with its rounding points
# ----------------------------------------------------------------------------
def pg_prolog(x, q_norm, q_norm_scale, w_qb, w_qb_scale, wk, w_proj, gamma_k, cos, sin, hadamard_q, hadamard_k,
              fmt: str, eps: float = 1e-6):
    """lightning_indexer_prolog_quant_{mxfp8,hif8}_impl.py:330-401 on CPU tensors.
    x bf16 [t, h]; q_norm codes [t, q_lora] (float8_e4m3fn, or uint8 HiF8 codes); q_norm_scale uint8 E8M0 codes
    [t, q_lora/32] (mxfp8) or fp32 [t, 1] (hif8); w_qb codes [q_lora, n]; w_qb_scale uint8 [q_lora/64, n, 2] (mxfp8)
    or fp32 [1, n] (hif8).  Returns (q codes [t, heads, 128], q_scale fp32 [t, heads, 1], k codes [t, 128],
    k_scale fp32 [t, 1], weights bf16 [t, heads]); the caller scatters k / k_scale into the caches."""
    t = x.shape[0]
    q_lora, n = w_qb.shape
    heads = n // HEAD_DIM
    x32 = x.to(torch.float32)
    cos32, sin32 = cos.to(torch.float32), sin.to(torch.float32)
    if fmt == "mxfp8":
        qs, ws = expand_mx_scales(q_norm_scale, w_qb_scale, q_lora, n)
        q_mm = _bf((codes_to_float(q_norm, fmt) * qs) @ (codes_to_float(w_qb, fmt) * ws))            # :339
    else:
        q_mm = codes_to_float(q_norm, fmt) @ codes_to_float(w_qb, fmt)                              # hif8 :339
        q_mm = _bf((q_mm * q_norm_scale.reshape(t, 1)) * w_qb_scale.reshape(1, n))                   # hif8 :343-345
    q3 = q_mm.reshape(t, heads, HEAD_DIM)
    q_rope, q_nope = q3[..., :ROPE_DIM], q3[..., ROPE_DIM:]
    c3, s3 = cos32.reshape(t, 1, ROPE_DIM), sin32.reshape(t, 1, ROPE_DIM)
    q_roped = _bf(q_rope * c3 + rotate_half(q_rope) * s3)                                            # rope_3d :191-224
    q_cat = torch.cat([q_roped, q_nope], dim=-1).reshape(t * heads, HEAD_DIM)
    q_had = _bf(q_cat @ hadamard_q.to(torch.float32))                                                # :356
    q_codes, q_scale = _quant(q_had, fmt)                                                            # :360
    # key path
    k_proj = _bf(x32 @ wk.to(torch.float32))                                                         # :368
    ms = (k_proj * k_proj * np.float32(1.0 / HEAD_DIM)).sum(dim=-1, keepdim=True)
    k_norm = _bf((k_proj / torch.sqrt(ms + eps)) * gamma_k.to(torch.float32).reshape(1, HEAD_DIM))   # quant_rms_norm :40-72
    k_rope, k_nope = k_norm[:, :ROPE_DIM], k_norm[:, ROPE_DIM:]
    k_roped = _bf(k_rope * cos32 + rotate_half(k_rope) * sin32)                                      # quant_rope_2d :75-108
    k_had = _bf(torch.cat([k_roped, k_nope], dim=-1) @ hadamard_k.to(torch.float32))                 # :384
    k_codes, k_scale = _quant(k_had, fmt)                                                            # :388
    # weights
    w = _bf(x32 @ w_proj.to(torch.float32))
    w = _bf(w * np.float32(heads ** -0.5))
    w = (w * np.float32(HEAD_DIM ** -0.5)).to(torch.bfloat16)                                        # :398-400
    return (q_codes.reshape(t, heads, HEAD_DIM), q_scale.reshape(t, heads, 1), k_codes, k_scale, w)


# ----------------------------------------------------------------------------
# the reference's fp32 golden
# ----------------------------------------------------------------------------
def pg_prolog_golden(x, q_norm, q_norm_scale, w_qb, w_qb_scale, wk, w_proj, gamma_k, cos, sin, hadamard_q,
                     hadamard_k, fmt: str = "mxfp8", eps: float = 1e-6):
    """test_pg_lightning_indexer_prolog_quant_mxfp8.py:272-345 (platform "cpu"): every input widened to fp32 and no
    intermediate rounding; quantisation as quant_fp8e4m3 (:238-248).  Same returns as `pg_prolog`, the MXFP8 codes as
    float8_e4m3fn, the weights as fp32.  With fmt "hif8" the same computation with the HiF8 operands, scales and
    codec of this file (test_pg_lightning_indexer_prolog_quant_hif8.py:240-250, whose casts are NPU calls): a
    yardstick of this file's making, not a pinned golden."""
    t = x.shape[0]
    q_lora, n = w_qb.shape
    heads = n // HEAD_DIM
    f = lambda v: v.to(torch.float32)  # noqa: E731
    if fmt == "mxfp8":
        qs, ws = expand_mx_scales(q_norm_scale, w_qb_scale, q_lora, n)
        q_mm = torch.matmul(f(q_norm) * qs, f(w_qb) * ws)
    else:
        q_mm = torch.matmul(hif8_decode(q_norm), hif8_decode(w_qb)) * q_norm_scale.reshape(t, 1) * w_qb_scale.reshape(1, n)
    q3 = q_mm.reshape(t, heads, HEAD_DIM)
    c3, s3 = f(cos).reshape(t, 1, ROPE_DIM), f(sin).reshape(t, 1, ROPE_DIM)
    q_rope = q3[..., :ROPE_DIM] * c3 + rotate_half(q3[..., :ROPE_DIM]) * s3
    q_had = torch.matmul(torch.cat([q_rope, q3[..., ROPE_DIM:]], dim=-1), f(hadamard_q))

    def quant(v):
        amax = torch.amax(torch.abs(v), dim=-1, keepdim=True)
        if fmt == "mxfp8":
            sq = FP8_MAX / amax
            return (v * sq).to(torch.float8_e4m3fn), 1.0 / sq
        sq = HIF8_MAX / amax
        return hif8_encode(v * sq), 1.0 / sq

    q_codes, q_scale = quant(q_had)
    k_proj = torch.matmul(f(x), f(wk))
    rms = torch.sqrt(torch.mean(k_proj ** 2, dim=-1, keepdim=True) + eps)
    k_norm = (k_proj / rms) * f(gamma_k).reshape(1, HEAD_DIM)
    k_rope = k_norm[:, :ROPE_DIM] * f(cos) + rotate_half(k_norm[:, :ROPE_DIM]) * f(sin)
    k_had = torch.matmul(torch.cat([k_rope, k_norm[:, ROPE_DIM:]], dim=-1), f(hadamard_k))
    k_codes, k_scale = quant(k_had)
    w = torch.matmul(f(x), f(w_proj)) * (heads ** -0.5) * (HEAD_DIM ** -0.5)
    return q_codes, q_scale, k_codes, k_scale, w


# ----------------------------------------------------------------------------
# the reference's accuracy rule
# ----------------------------------------------------------------------------
_SMALL_VALUE = {"fp8": 2.0 ** -4, "bf16": 2.0 ** -8, "fp32": 2.0 ** -14}
_SMALL_ERROR = {"fp8": 2.0 ** -6, "bf16": 2.0 ** -16, "fp32": 2.0 ** -30}


def triple_compare(out, bench, golden, kind: str, thres=(2.0, 1.2, 1.2)):
    """compare_2_1.py:92-133: the errors of `out` against `golden` (max and mean relative error and RMSE over the
    entries whose golden magnitude reaches the small-value threshold, and the count of small entries that are off by
    more than the small-error threshold) may not exceed `thres` times (twice, for the count) those of `bench`.
    `kind` names the output's type ("fp8" for both 8-bit formats, "bf16", "fp32").  Returns (passed, ratios)."""
    out, bench, golden = (v.to(torch.float32).flatten() for v in (out, bench, golden))
    small_thres = _SMALL_VALUE[kind]
    large = golden.abs() >= small_thres

    def small_errors(v):
        return int(((v[~large] - golden[~large]).abs() > _SMALL_ERROR[kind]).sum()) if (~large).any() else 0

    def large_errors(v):
        if not large.any():
            return 0.0, 0.0, 0.0
        d = (v[large] - golden[large]).abs()
        rel = d / (golden[large].abs() + 1e-7)
        return float(rel.max()), float(rel.mean()), float(torch.sqrt((d * d).mean()))

    def ratio(a, b):
        if math.isinf(b) or math.isnan(b):
            return 1.0
        if math.isinf(a) or math.isnan(a):
            return 1000.0
        return a / max(b, small_thres)

    small_ratio = small_errors(out) / max(small_errors(bench), 1)
    ratios = tuple(ratio(a, b) for a, b in zip(large_errors(out), large_errors(bench)))
    passed = small_ratio <= 2 and all(r <= th for r, th in zip(ratios, thres))
    return passed, ratios + (small_ratio,)
