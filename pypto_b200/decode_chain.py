"""One decode step of the sparse-attention chain as the reference model files define it
(models/deepseek_v32_exp/README_en.md data flow): indexer prolog -> lightning indexer + top-k ->
sparse flash attention, all through the operator entry points of this package.

The latent cache, the index-key cache and the weights are device-resident state; the per-step
activations may be given as pinned host tensors, in which case the step copies them to the device
and copies the attention output back (the end-to-end path).
"""
from __future__ import annotations

import torch

import ctypes as C

from . import _lib
from . import _runtime as rt
from .lightning_indexer_prolog_quant_impl import (IndexerPrologQuantAttr, IndexerPrologQuantConfigs,
                                                  lightning_indexer_prolog_quant)
from .lightning_indexer_quant_impl import LightningIndexerConfigs, lightning_indexer_decode
from .sparse_flash_attention_quant_impl import SaTileShapeConfig, _sfa, sparse_flash_attention_quant_d

STEP_INPUTS = ("x", "q_norm", "q_norm_scale", "cos", "sin", "cache_index", "q_nope", "q_rope")


class PackedTensors:
    """A set of named tensors laid out back to back (256-byte aligned) in ONE byte buffer, on a device or in
    pinned host memory, so that the whole set moves with a single copy.  `views[name]` are typed views."""

    def __init__(self, like: dict, device, pin=False):
        self.offsets, pos = {}, 0
        for k, v in like.items():
            self.offsets[k] = pos
            pos += (v.numel() * v.element_size() + 255) // 256 * 256
        self.nbytes = pos
        self.buf = torch.empty(pos, dtype=torch.uint8, device=device)
        if pin:
            self.buf = self.buf.pin_memory()
        self.views = {}
        for k, v in like.items():
            n = v.numel() * v.element_size()
            self.views[k] = self.buf[self.offsets[k]:self.offsets[k] + n].view(v.dtype).view(v.shape)
            self.views[k].copy_(v)


class SparseDecodeStep:
    def __init__(self, w, nq=128, topk=2048, acts=None):
        """`w`: a synth.DecodeWorkload (caches, page table, weights: device-resident state).  `acts`: the per-step
        activations (a dict with the STEP_INPUTS names); default: the ones that come with the workload."""
        self.w = w
        dev = w.k_nope.device
        t = w.t
        self.nq, self.topk = nq, topk
        self.q_int8 = torch.empty((t, 64, 128), dtype=torch.int8, device=dev)
        self.q_scale = torch.empty((t, 64, 1), dtype=torch.float16, device=dev)
        self.weights = torch.empty((t, 64), dtype=torch.float16, device=dev)
        self.topk_res = torch.empty((t, 1, topk), dtype=torch.int32, device=dev)
        self.out = torch.empty((w.b, w.s1, nq, 512), dtype=torch.bfloat16, device=dev)
        self.idx_k_scale4 = w.idx_k_scale.reshape(w.idx_k_scale.shape[0], 128, 1, 1)
        self.softmax_scale = 576 ** -0.5
        self.kv_splits = 0   # key splits of the attention kernel: 0 = the library's choice (profiling may fix it)
        self._cfg = (IndexerPrologQuantConfigs(), IndexerPrologQuantAttr(eps=1e-6), LightningIndexerConfigs(),
                     SaTileShapeConfig())
        acts = acts if acts is not None else {k: getattr(w, k) for k in STEP_INPUTS}
        self.dev_pack = PackedTensors({k: acts[k] for k in STEP_INPUTS}, dev)
        self._dev_in = self.dev_pack.views
        self.host_pack = None
        self.host_in = None
        self.host_out = None

    # ---- end-to-end staging -----------------------------------------------------------------------
    def enable_host_io(self):
        """Keep a pinned host copy of the per-step activations (one contiguous buffer: one copy per step) and a
        pinned output buffer.  Returns the bytes per step in each direction."""
        self.host_pack = PackedTensors(self._dev_in, "cpu", pin=True)
        self.host_in = self.host_pack.views
        self.host_out = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        d2h = self.host_out.numel() * self.host_out.element_size()
        return self.host_pack.nbytes, d2h

    # ---- stages -------------------------------------------------------------------------------------
    def prolog(self):
        w, d = self.w, self._dev_in
        pc, pa, _, _ = self._cfg
        lightning_indexer_prolog_quant(
            d["x"], d["q_norm"], d["q_norm_scale"], w.w_qb, w.w_qb_scale, w.wk, w.w_proj, w.ln_gamma, w.ln_beta,
            d["cos"], d["sin"], w.hadamard, w.hadamard, w.idx_k, self.idx_k_scale4, d["cache_index"], self.q_int8,
            self.q_scale, w.idx_k, self.idx_k_scale4, self.weights, pc, pa)

    def indexer(self):
        w = self.w
        lightning_indexer_decode(self.q_int8, self.q_scale.reshape(-1, 64), w.idx_k, w.idx_k_scale, self.weights,
                                 w.act_seq, w.block_table, self.topk_res, None, self._cfg[2], self.topk)

    def attention(self):
        w, d = self.w, self._dev_in
        # (the operator entry sparse_flash_attention_quant_d with the key split of the C ABI exposed: 0 = automatic)
        _sfa(d["q_nope"], d["q_rope"], w.k_nope, w.k_rope, w.k_scales, self.topk_res.reshape(-1, self.topk),
             w.block_table, w.act_seq, self.out, self.nq, 1, self.softmax_scale, self.topk, 128, w.max_blocks,
             self._cfg[3], kv_splits=self.kv_splits)

    def step(self):
        """Device-resident step: prolog -> indexer + top-k -> attention on the current stream."""
        self.prolog()
        self.indexer()
        self.attention()
        return self.out

    # ---- CUDA graphs ------------------------------------------------------------------------------------
    def capture(self, per_stage=False):
        """Capture the step on its current input / output buffers into CUDA graphs (one graph, or one per stage
        so that events can be recorded between the stages).  Returns the list of graphs; `replay()` runs them
        in order on the current stream.  The buffers captured are the ones the step points at now."""
        dev = self.out.device
        cur = torch.cuda.current_stream(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(cur)
        with torch.cuda.stream(side):  # warm-up outside capture: lazy initialisation, tensor maps, allocator
            self.step()
        cur.wait_stream(side)
        stages = (self.prolog, self.indexer, self.attention) if per_stage else (self.step,)
        graphs = []
        for fn in stages:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            graphs.append(g)
        self.graphs = graphs
        return graphs

    def replay(self):
        for g in self.graphs:
            g.replay()
        return self.out

    def step_from_host(self):
        """End-to-end step: pinned host activations -> device, the three stages, output -> pinned host."""
        self.dev_pack.buf.copy_(self.host_pack.buf, non_blocking=True)
        self.step()
        self.host_out.copy_(self.out, non_blocking=True)
        return self.host_out


class HostPipelinedDecode:
    """End-to-end decode loop with the host traffic overlapped with compute.

    Every step still copies its own activations from pinned host memory and returns its own attention
    output to pinned host memory, but on separate streams: while step k runs, the inputs of step k+1 are
    copied in and the output of step k-1 is copied out (two device buffers per direction, events between the
    three streams).  `submit(host_pack)` (a pinned PackedTensors of the step's activations) enqueues one step and returns the pinned tensor its output will land
    in; `drain()` makes the current stream wait for everything submitted so far.
    """

    def __init__(self, step: SparseDecodeStep, use_graphs=False):
        self.step = step
        dev = step.out.device
        self.dev = dev
        self.s_in = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self.dev_packs = [step.dev_pack, PackedTensors(step._dev_in, dev)]  # both sets valid from the start
        self.dev_in = [p.views for p in self.dev_packs]
        self.dev_out = [step.out, torch.empty_like(step.out)]
        self.host_out = [torch.empty(step.out.shape, dtype=step.out.dtype).pin_memory() for _ in range(2)]
        self.in_ready = [torch.cuda.Event() for _ in range(2)]
        self.run_done = [torch.cuda.Event() for _ in range(2)]
        self.out_done = [torch.cuda.Event() for _ in range(2)]
        self.k = 0
        self.graphs = None
        if use_graphs:  # one captured step per buffer pair
            self.graphs = []
            for p in range(2):
                step._dev_in, step.out = self.dev_in[p], self.dev_out[p]
                self.graphs.append(step.capture()[0])

    def submit(self, host_pack: PackedTensors):
        step, p = self.step, self.k & 1
        run = torch.cuda.current_stream(self.dev)
        if self.k >= 2:
            self.s_in.wait_event(self.run_done[p])      # the step two back has finished reading this input buffer
        else:
            self.s_in.wait_stream(run)                   # everything enqueued before the first steps
        with torch.cuda.stream(self.s_in):
            self.dev_packs[p].buf.copy_(host_pack.buf, non_blocking=True)   # all activations of the step: one copy
            self.in_ready[p].record(self.s_in)
        run.wait_event(self.in_ready[p])
        if self.k >= 2:
            run.wait_event(self.out_done[p])             # its output buffer has been copied out
        step._dev_in, step.out = self.dev_in[p], self.dev_out[p]
        if self.graphs is not None:
            self.graphs[p].replay()
        else:
            step.step()
        self.run_done[p].record(run)
        self.s_out.wait_event(self.run_done[p])
        with torch.cuda.stream(self.s_out):
            self.host_out[p].copy_(self.dev_out[p], non_blocking=True)
            self.out_done[p].record(self.s_out)
        self.k += 1
        return self.host_out[p]

    def drain(self):
        run = torch.cuda.current_stream(self.dev)
        for e in self.out_done[: min(self.k, 2)]:
            run.wait_event(e)


def decode_advance(act_seq, block_table, cache_index, s1, grow=None, block_size=128):
    """Prepare the next decode step on the device (dsv32_decode_advance): act_seq += grow (default s1) and the cache
    rows of the step's tokens by the reference's rule (deepseekv32_mla_indexer_prolog_quant.py:184-194).  In place,
    on the current stream, capturable."""
    rt.require_cuda()
    rt.check_tensor(act_seq, "act_seq", torch.int32, ndim=1)
    b = act_seq.shape[0]
    rt.check_tensor(block_table, "block_table", torch.int32, (b, None))
    rt.check_tensor(cache_index, "cache_index", torch.int64, (b * int(s1),))
    dev = rt.same_device(act_seq, block_table, cache_index)
    a = _lib.AdvanceArgs(rt.ptr(act_seq), rt.ptr(block_table), rt.ptr(cache_index), rt.ptr(rt.status_word(dev)), b, int(s1),
                         int(s1 if grow is None else grow), int(block_size), block_table.shape[1])
    with torch.cuda.device(dev):
        rt.check(_lib.load().dsv32_decode_advance(C.byref(a), rt.stream_ptr(dev)), "decode_advance")


class FullDecodeStep:
    """A decode loop that appends: every step runs the fused MLA + indexer prolog on the step's hidden states (which
    writes the s1 new rows of both caches at `cache_index`), the lightning indexer + top-k over the grown context and
    the sparse attention; `advance()` then moves the batch to the next positions on the device.  `w` is a
    synth.FullDecodeWorkload; x / cos / sin of a step are copied into fixed buffers so that the loop can be captured."""

    def __init__(self, w, nq=128, topk=2048):
        from .mla_indexer_prolog_quant_impl import MlaTileConfig, RopeTileShapeConfig
        self.w = w
        dev = w.kv_cache.device
        t = w.t
        self.nq, self.topk = nq, topk
        bf = torch.bfloat16
        self.x = torch.zeros((t, 7168), dtype=bf, device=dev)
        self.cos = torch.zeros((t, 64), dtype=bf, device=dev)
        self.sin = torch.zeros((t, 64), dtype=bf, device=dev)
        self.q_nope = torch.empty((t, nq, 512), dtype=bf, device=dev)
        self.q_rope = torch.empty((t, nq, 64), dtype=bf, device=dev)
        self.q_int8 = torch.empty((t, 64, 128), dtype=torch.int8, device=dev)
        self.q_scale = torch.empty((t, 64, 1), dtype=torch.float16, device=dev)
        self.weights = torch.empty((t, 64), dtype=torch.float16, device=dev)
        self.topk_res = torch.empty((t, 1, topk), dtype=torch.int32, device=dev)
        self.out = torch.empty((w.b, w.s1, nq, 512), dtype=bf, device=dev)
        self._cfg = (MlaTileConfig(), IndexerPrologQuantAttr(eps=1e-6), IndexerPrologQuantConfigs(), RopeTileShapeConfig(),
                     LightningIndexerConfigs(), SaTileShapeConfig())
        self.graph = None

    def set_inputs(self, x, cos, sin):
        self.x.copy_(x, non_blocking=True)
        self.cos.copy_(cos, non_blocking=True)
        self.sin.copy_(sin, non_blocking=True)

    def prolog(self):
        from .mla_indexer_prolog_quant_impl import mla_indexer_prolog_quant_d
        w = self.w
        mla_cfg, ip_attr, ip_cfg, rope_cfg = self._cfg[:4]
        mla_indexer_prolog_quant_d(
            self.x, w.w_dq, w.w_uq_qr, w.w_uq_qr_scale, w.w_uk, w.w_dkv_kr, w.gamma_cq, w.gamma_ckv, self.cos, self.sin,
            w.cache_index, w.kv_cache, w.kr_cache, w.k_scale_cache, w.w_qb, w.w_qb_scale, w.wk, w.w_proj, w.ln_gamma,
            w.ln_beta, w.hadamard, w.hadamard, w.idx_k, w.idx_k_scale, self.q_nope, self.q_rope, w.kv_cache, w.kr_cache,
            w.k_scale_cache, self.q_int8, self.q_scale, w.idx_k, w.idx_k_scale, self.weights, 1e-6, 1e-6, "PA_BSND",
            mla_cfg, ip_attr, ip_cfg, rope_cfg)

    def indexer(self):
        w = self.w
        lightning_indexer_decode(self.q_int8, self.q_scale.reshape(-1, 64), w.idx_k,
                                 w.idx_k_scale.reshape(w.idx_k_scale.shape[0], 128, 1), self.weights, w.act_seq,
                                 w.block_table, self.topk_res, None, self._cfg[4], self.topk)

    def attention(self):
        w = self.w
        sparse_flash_attention_quant_d(self.q_nope.reshape(-1, 512), self.q_rope.reshape(-1, 64),
                                       w.kv_cache.reshape(-1, 512), w.kr_cache.reshape(-1, 64),
                                       w.k_scale_cache.reshape(-1, 4), self.topk_res.reshape(-1, self.topk), w.block_table,
                                       w.act_seq, self.out, self.nq, 1, 576 ** -0.5, self.topk, 128, w.max_blocks,
                                       self._cfg[5])

    def step(self):
        self.prolog()
        self.indexer()
        self.attention()
        return self.out

    def advance(self):
        decode_advance(self.w.act_seq, self.w.block_table, self.w.cache_index, self.w.s1)

    def capture(self):
        """One CUDA graph of step() followed by advance(): every replay is the next decode step (new hidden states
        are copied into `x`, `cos`, `sin` before it)."""
        dev = self.out.device
        cur = torch.cuda.current_stream(dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(cur)
        saved = (self.w.act_seq.clone(), self.w.cache_index.clone())
        with torch.cuda.stream(side):   # warm-up outside capture (lazy initialisation); undone below
            self.step()
        cur.wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
            self.advance()
        self.w.act_seq.copy_(saved[0])
        self.w.cache_index.copy_(saved[1])
        self.graph = g
        return g
