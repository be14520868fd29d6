#!/usr/bin/env python3
"""Benchmark of the sparse-attention decode chain (indexer prolog -> lightning indexer + top-2048 ->
sparse flash attention over the int8 paged cache) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config 2|3|4] [--scaling strong|weak] [--workload chain|v4]
                    [--batch 64] [--ctx 65536] [--s1 2]

config 2 (default)  full decode chain, batch 64, context 64K, 2 query tokens per request.  With N > 1 (torchrun,
                    one rank per GPU, no collective on the data path) the 64 requests are SPLIT over the ranks
                    ("strong"); the figure with 64 requests on every rank is printed beside it as "weak".
config 3            one request, 128K keys, a 4096-token query chunk: the index-key range is sharded over the ranks,
                    every rank sends each peer its top-2048 candidates for that peer's query slice (one NCCL all-to-all), the
                    candidates are re-selected, attention runs on the rank that owns each query slice.
config 4            ragged production decode, batch 256, context lengths log-uniform in [1K, 128K] (10 % below 2048),
                    requests assigned to ranks by longest-processing-time-first on their cost.
One step = one pass of the chain over the batch.  The metric is decode tokens/s (whole job, all ranks).  Every
figure is the median over rounds of exactly K steps, each round bracketed by a barrier and a device
synchronisation, timed with CUDA events, maximum over ranks.  Prints ONE JSON line on rank 0.
`--workload v4` times the DeepSeek-V4 operators instead (one JSON line per operator, N = 1); `--workload mla` the
MLA prolog and the fused MLA + indexer prolog.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "SFA-quant decode tokens/s per GPU @64K ctx, top-k 2048 (indexer prolog + lightning indexer + top-k + SFA chain)"
UNIT = "tokens/s"
TOPK = 2048
NVLINK_PEER_GBS = 770.0   # measured peer copy per direction on this pool (nominal 900)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_ncu_traffic():
    """DRAM traffic per unit of the dominant kernels, from the ncu captures summarised under profiles/ (a small
    JSON written beside the summaries: bytes per token / per request, the case captured and the kernel sources'
    digest at capture time).  None when the file is missing or the kernel sources have changed since."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(p) as f:
            d = json.load(f)
        import hashlib
        out = {}
        for name, e in d.items():
            h = hashlib.sha256()
            for src in e["sources"]:
                with open(os.path.join(ROOT, src), "rb") as sf:
                    h.update(sf.read())
            out[name] = e["bytes_per_unit"] if h.hexdigest()[:16] == e["sources_sha16"] else None
        return out
    except Exception:
        return {}


# ---- algorithmic work per unit ---------------------------------------------------------------------------
def sfa_flops_per_token(k):        # 2*128*K*(576+512)
    return 278528.0 * k


def sfa_bytes_per_token(k, ctx):   # gathered rows + indices + Q + O + page table
    return k * (512 + 16 + 128) + k * 4 + 147456 + 131072 + ((ctx + 127) // 128) * 4


def indexer_bytes_per_request(ctx, s1):
    return ctx * 130 + ((ctx + 127) // 128) * 4 + s1 * (8192 + 128 + 128) + s1 * 8192


def prolog_bytes_per_call(t):
    return 15433728 + t * (14336 + 1536 + 4 + 256 + 8) + t * (8192 + 128 + 130 + 128)


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
                 str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 9:
                        continue
                    try:
                        if float(c[3]) < 250.0:  # idle sample (power draw in W): not under load
                            continue
                        sm.append(float(c[1]))
                        mx.append(float(c[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         c[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


class numa_local:
    """While active, the calling thread runs on the CPUs of the NUMA node its GPU hangs off (when the box has more
    than one node), so that pinned staging buffers allocated inside the block sit next to the GPU; the thread's
    affinity is put back on exit.  Best effort: `node` is the node used, or None."""

    def __init__(self, local_rank):
        self.local_rank, self.node, self.saved = local_rank, None, None

    def __enter__(self):
        try:
            nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node")]
            if len(nodes) < 2:
                return self
            pr = torch.cuda.get_device_properties(self.local_rank)
            path = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0/numa_node"
            with open(path) as f:
                node = int(f.read().strip())
            if node < 0:
                return self
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            saved = os.sched_getaffinity(0)
            if cpus & saved:
                os.sched_setaffinity(0, cpus & saved)
                self.saved, self.node = saved, node
        except Exception:
            pass
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            try:
                os.sched_setaffinity(0, self.saved)
            except Exception:
                pass
        return False


# ---- workloads ------------------------------------------------------------------------------------------------
def ragged_contexts(n, seed):
    """Config 4: context lengths log-uniform over [1K, 128K]; every tenth request is forced below 2048 keys
    (its index rows are padded with -1)."""
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(n, generator=g)
    ctx = torch.exp(math.log(1024.0) + u * (math.log(131072.0) - math.log(1024.0))).long().clamp(1024, 131072)
    short = torch.randint(64, 2048, (n,), generator=g)
    ctx[::10] = short[::10]
    return [int(c) for c in ctx]


def requests_of_rank(args, rank, world):
    """Context length of every request this rank serves."""
    from pypto_b200 import sharding
    if args.config == 4:
        ctx = ragged_contexts(args.batch, 1004)
        bins = sharding.lpt_assign([sharding.request_cost(c, args.s1) for c in ctx], world)
        return [ctx[i] for i in bins[rank]]
    if args.scaling == "weak":
        return [args.ctx] * args.batch
    return [args.ctx] * len(sharding.split_even(args.batch, world)[rank])


def workload_config(args, world):
    if args.config == 3:
        return {"workload": f"config 3: one request, {args.ctx} keys, {args.s1}-token query chunk, 128 heads, top-k {TOPK}: "
                            f"lightning indexer over a sharded key range + candidate merge + SFA",
                "ctx": args.ctx, "s1": args.s1, "topk": TOPK, "global_batch": 1,
                "parallelism": f"index-key range sharded over {world} GPU(s); one all-to-all of (score, index) "
                               f"candidates (each rank receives those of its own query slice); attention on the "
                               f"rank that owns each query slice",
                "l2_policy": "L2 flushed between steps (a 256 MB buffer is overwritten)"}
    name = "config 2: full decode chain" if args.config == 2 else \
        "config 4: ragged decode chain (ctx log-uniform 1K..128K, 10 % below 2048, LPT assignment)"
    per_rank = args.batch if (args.scaling == "weak" and args.config == 2) else None
    return {"workload": f"{name}, batch {args.batch}, ctx {args.ctx if args.config == 2 else 'ragged'}, "
                        f"MTP s1={args.s1}, 128 heads, top-k {TOPK}",
            "global_batch": args.batch * (world if per_rank else 1), "ctx": args.ctx if args.config == 2 else None,
            "s1": args.s1, "topk": TOPK,
            "parallelism": f"requests sharded over {world} GPU(s), no collective",
            "l2_policy": "inputs larger than L2 (per-GPU working set of caches well above 126 MB); two sets of per-step "
                         "activations alternate",
            "launch": "one CUDA graph per step, captured from the operator entry points"}


# ---- CPU reference arm ------------------------------------------------------------------------------------
def cpu_chain_sample(ctx_list, s1, seed, steps=1, warmup=0):
    """Time the CPU oracle (the reference goldens' algorithm) on a bounded sample of the workload: the requests
    in `ctx_list`, whole chain.  Returns (tokens/s, seconds per step, threads)."""
    from oracle import dsv32_oracle as orc
    from pypto_b200 import synth
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    w = synth.make_decode_workload(list(ctx_list), s1, seed, "cpu")

    def one():
        q_i8, q_s, kc, ksc, wts = orc.indexer_prolog(w.x, w.q_norm, w.q_norm_scale, w.w_qb, w.w_qb_scale, w.wk, w.w_proj,
                                                     w.ln_gamma, w.ln_beta, w.cos, w.sin, w.hadamard, w.hadamard,
                                                     w.idx_k, w.idx_k_scale, w.cache_index)
        idx = orc.lightning_indexer(q_i8, q_s.reshape(-1, 64), kc, ksc.reshape(ksc.shape[0], 128, 1), wts, w.act_seq,
                                    w.block_table, TOPK)
        return orc.sfa_quant(w.q_nope, w.q_rope, w.k_nope, w.k_rope, w.k_scales, idx.reshape(-1, TOPK), w.block_table,
                             w.act_seq, 128, 576 ** -0.5)

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return len(ctx_list) * s1 / dt, dt, threads


def cpu_config3_sample(ctx, s1, n_tokens, seed, steps=1):
    """Config 3 on the CPU oracle: `n_tokens` query tokens sampled evenly from the chunk, each scored against all
    of its keys, top-2048, attention.  Returns (tokens/s, seconds per step, threads)."""
    from oracle import dsv32_oracle as orc
    from pypto_b200 import synth
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    d = synth.make_long_request(ctx, s1, seed, "cpu", token_slice=None, sample=n_tokens)
    # every sampled token becomes a request of its own that shares the page table (its context = its valid keys)
    bt = d["block_table"].expand(n_tokens, -1).contiguous()

    def one():
        idx = orc.lightning_indexer(d["q_int8"], d["q_scale"], d["idx_k"], d["idx_k_scale"], d["weights"], d["eff"], bt, TOPK)
        return orc.sfa_quant(d["q_nope"], d["q_rope"], d["k_nope"], d["k_rope"], d["k_scales"], idx.reshape(-1, TOPK), bt,
                             d["eff"], 128, 576 ** -0.5)

    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return n_tokens / dt, dt, threads


def cpu_sample_for(args, steps, warmup=0):
    """(tokens/s, seconds per step, threads, description) of the CPU arm's bounded sample for this config."""
    if args.config == 3:
        n = args.cpu_requests
        v, dt, th = cpu_config3_sample(args.ctx, args.s1, n, 1003, steps=steps)
        return v, dt, th, f"{n} query tokens sampled evenly from the {args.s1}-token chunk, {args.ctx} keys, indexer + top-k + attention"
    if args.config == 4:
        ctx = ragged_contexts(args.batch, 1004)[:args.cpu_requests]
        v, dt, th = cpu_chain_sample(ctx, args.s1, 1004, steps=steps, warmup=warmup)
        return v, dt, th, f"the first {len(ctx)} requests of the ragged batch x {args.s1} tokens, whole chain"
    v, dt, th = cpu_chain_sample([args.ctx] * args.cpu_requests, args.s1, 1002, steps=steps, warmup=warmup)
    return v, dt, th, f"{args.cpu_requests} requests x {args.s1} tokens at ctx {args.ctx} per step (same chain, same distributions)"


def run_reference(args, rank, world):
    if rank != 0:
        return
    val, dt, threads, sample = cpu_sample_for(args, args.steps, warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, world),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit_json(line)


# ---- timing helpers ---------------------------------------------------------------------------------------------
class Timer:
    """Rounds of exactly `steps` calls, each bracketed by barrier + synchronize, CUDA events, max over ranks."""

    def __init__(self, dev, world):
        self.dev, self.world = dev, world

    def barrier(self):
        import torch.distributed as dist
        torch.cuda.synchronize(self.dev)
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize(self.dev)

    def one_round(self, fn, steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        start.record()
        for i in range(steps):
            fn(i)
        end.record()
        self.barrier()
        return start.elapsed_time(end)

    def rounds(self, fn, steps, min_total_ms=500.0, min_rounds=3, max_rounds=200, after_round=None):
        """Keeps timing rounds until `min_total_ms` of timed region have accumulated.  Returns per-round ms
        (already the max over ranks)."""
        import torch.distributed as dist
        first = self.one_round(fn, steps)
        if self.world > 1:  # every rank must run the same number of rounds
            t = torch.tensor([first], dtype=torch.float64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            first = float(t.item())
        n = int(min(max(math.ceil(min_total_ms / max(first, 1e-3)), min_rounds), max_rounds))
        ms = [first]
        for _ in range(n - 1):
            if after_round is not None:
                after_round()
            ms.append(self.one_round(fn, steps))
        if self.world > 1:
            t = torch.tensor(ms, dtype=torch.float64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = [first] + [float(v) for v in t.tolist()[1:]]
        return ms


def spread(ms_rounds, steps):
    per = sorted(m / steps for m in ms_rounds)
    return {"median": statistics.median(per), "min": per[0], "max": per[-1], "rounds": len(per),
            "timed_ms_total": sum(ms_rounds)}


def host_link_probe(dev, h2d_bytes, d2h_bytes, timer, iters=20, host_in=None, host_out=None):
    """Concurrent H2D + D2H cudaMemcpyAsync of the step's buffer sizes on two streams, all ranks at once: the
    bandwidth the end-to-end loop could reach if nothing but its copies ran.  `host_in` / `host_out` are the loop's
    own pinned buffers (byte views), so that the probe sees the same host pages as the loop; the best round counts,
    as a bound should.  Returns seconds per (H2D + D2H) pair."""
    hin = host_in if host_in is not None else torch.empty(max(h2d_bytes, 1), dtype=torch.uint8).pin_memory()
    hout = host_out if host_out is not None else torch.empty(max(d2h_bytes, 1), dtype=torch.uint8).pin_memory()
    din = torch.empty(hin.numel(), dtype=torch.uint8, device=dev)
    dout = torch.empty(hout.numel(), dtype=torch.uint8, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def pair(i):
        # both directions are queued back to back on their own streams, as in the decode loop; the timed stream
        # joins them after the last copy of the round
        cur = torch.cuda.current_stream(dev)
        if i == 0:
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            din.copy_(hin, non_blocking=True)
        with torch.cuda.stream(s_out):
            hout.copy_(dout, non_blocking=True)
        if i == iters - 1:
            cur.wait_stream(s_in)
            cur.wait_stream(s_out)

    for i in range(iters):
        pair(i)
    ms = timer.rounds(pair, iters, min_total_ms=50.0, min_rounds=5, max_rounds=10)
    return min(ms) / iters * 1e-3


# ---- config 2 / 4: the decode chain, requests sharded over ranks ------------------------------------------------------
def build_steps(ctx_list, s1, seed, dev, kv_splits=0):
    from pypto_b200 import synth
    from pypto_b200.decode_chain import SparseDecodeStep
    w = synth.make_decode_workload(ctx_list, s1, seed, dev)
    a = SparseDecodeStep(w)
    b = SparseDecodeStep(w, acts=synth.make_step_activations(w, seed + 7919))
    a.kv_splits = b.kv_splits = kv_splits
    return w, a, b


def run_chain(args, rank, world, local_rank):
    import torch.distributed as dist
    import pypto_b200
    from pypto_b200.decode_chain import HostPipelinedDecode

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    timer = Timer(dev, world)
    ctx_list = requests_of_rank(args, rank, world)
    tokens_rank = len(ctx_list) * args.s1
    w, step_a, step_b = build_steps(ctx_list, args.s1, 1002 + rank, dev, args.kv_splits)
    steps = (step_a, step_b)
    with numa_local(local_rank) as nl:
        h2d, d2h = step_a.enable_host_io()
        step_b.enable_host_io()
    numa = nl.node

    def total_tokens_per_step():
        if world == 1:
            return tokens_rank
        t = torch.tensor([tokens_rank], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        return int(t.item())

    tokens_step = total_tokens_per_step()
    gpu_index = local_rank
    try:
        gpu_index = int(os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[local_rank])
    except (ValueError, IndexError):
        pass
    sampler = ClockSampler(gpu_index)
    if rank == 0:
        sampler.start()
    # warm-up (at least 3 steps; kept going for ~1 s so that the clock sampler sees the GPU under this load)
    t_warm = time.perf_counter()
    n_warm = 0
    while n_warm < max(args.warmup, 3) or time.perf_counter() - t_warm < (1.0 if args.min_timed_ms > 0 else 0.0):
        steps[n_warm & 1].step()
        n_warm += 1
        if n_warm % 8 == 0:
            torch.cuda.synchronize(dev)
    pypto_b200.check_status(dev)
    launches0 = pypto_b200.launch_count()
    step_a.step()
    launches_per_step = pypto_b200.launch_count() - launches0  # counted on an eager step: graph replays do not pass
    whole = [s.capture(per_stage=False)[0] for s in steps]     # through the library's launch counter
    for i in range(4):
        whole[i & 1].replay()
    ms_rounds = timer.rounds(lambda i: whole[i & 1].replay(), args.steps, min_total_ms=args.min_timed_ms)
    dev_stats = spread(ms_rounds, args.steps)
    # stage times: the three stages of step A replayed from their own graphs, an event between them
    stage_graphs = step_a.capture(per_stage=True)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]

    def staged(i):
        for j in range(3):
            ev[i][j].record()
            stage_graphs[j].replay()
        ev[i][3].record()

    staged(0)
    timer.one_round(staged, args.steps)
    stages = [statistics.median(e[j].elapsed_time(e[j + 1]) for e in ev) for j in range(3)]
    # end-to-end: pinned host activations in, attention output back, every step -- on one stream ...
    for i in range(2):
        steps[i].step_from_host()
    ser_rounds = timer.rounds(lambda i: steps[i & 1].step_from_host(), args.steps, min_total_ms=min(200.0, args.min_timed_ms))
    # ... and with the copies of steps k+1 / k-1 overlapping the compute of step k (three streams)
    with numa_local(local_rank):
        pipe = HostPipelinedDecode(step_a, use_graphs=True)
    packs = (step_a.host_pack, step_b.host_pack)
    for i in range(3):
        pipe.submit(packs[i & 1])
    pipe.drain()

    def e2e_round(i):
        pipe.submit(packs[i & 1])
        if i == args.steps - 1:
            pipe.drain()

    e2e_rounds = timer.rounds(e2e_round, args.steps, min_total_ms=args.min_timed_ms)
    e2e_stats = spread(e2e_rounds, args.steps)
    with numa_local(local_rank):
        link_s = host_link_probe(dev, h2d, d2h, timer, host_in=step_a.host_pack.buf,
                                 host_out=step_a.host_out.view(-1).view(torch.uint8))
    clocks = sampler.stop() if rank == 0 else None
    pypto_b200.check_status(dev)

    # the same chain with `batch` requests on every rank (weak scaling), for the record
    weak = None
    if world > 1 and args.config == 2 and args.scaling == "strong" and not args.no_weak:
        del pipe
        _, wa, wb = build_steps([args.ctx] * args.batch, args.s1, 2002 + rank, dev)
        for s in (wa, wb):
            s.step()
        wg = [s.capture(per_stage=False)[0] for s in (wa, wb)]
        for i in range(4):
            wg[i & 1].replay()
        wr = timer.rounds(lambda i: wg[i & 1].replay(), args.steps, min_total_ms=200.0)
        ws = spread(wr, args.steps)
        weak = {"value": args.batch * args.s1 * world / (ws["median"] * 1e-3), "unit": UNIT, "ms_per_step": ws["median"],
                "batch_per_gpu": args.batch, "global_batch": args.batch * world}

    h2d_total, d2h_total = _sum_bytes(h2d, d2h, world, dev)
    if rank == 0:
        peaks = load_peaks()
        traffic = load_ncu_traffic()
        ms_step = dev_stats["median"]
        value = tokens_step / (ms_step * 1e-3)
        e2e_value = tokens_step / (e2e_stats["median"] * 1e-3)
        t_prolog, t_index, t_sfa = [s * 1e-3 for s in stages]  # seconds per step (rank 0)
        sfa_flops = sum(sfa_flops_per_token(min(TOPK, max(c - args.s1 + 1 + i, 0))) for c in ctx_list for i in range(args.s1))
        sfa_bytes = sum(sfa_bytes_per_token(min(TOPK, max(c - args.s1 + 1 + i, 0)), c) for c in ctx_list for i in range(args.s1))
        idx_bytes = sum(indexer_bytes_per_request(c, args.s1) for c in ctx_list)
        stage_info = {
            "prolog": {"ms": t_prolog * 1e3, "achieved_gbs": prolog_bytes_per_call(tokens_rank) / t_prolog / 1e9,
                       "hbm_frac": prolog_bytes_per_call(tokens_rank) / t_prolog / 1e9 / peaks["hbm_gbs"]},
            "indexer_topk": {"ms": t_index * 1e3, "achieved_gbs": idx_bytes / t_index / 1e9,
                             "hbm_frac": idx_bytes / t_index / 1e9 / peaks["hbm_gbs"]},
            "sfa": {"ms": t_sfa * 1e3, "achieved_tflops": sfa_flops / t_sfa / 1e12,
                    "tensor_frac": sfa_flops / t_sfa / 1e12 / peaks["bf16_tflops_sustained"],
                    "achieved_gbs": sfa_bytes / t_sfa / 1e9, "hbm_frac": sfa_bytes / t_sfa / 1e9 / peaks["hbm_gbs"]},
        }
        uniform = args.config == 2 and args.ctx == 65536
        if t_sfa >= t_index:
            per = traffic.get("sfa_tc_kernel")
            roofline = {"kernel": "sfa_tc_kernel", "bound": "tensor", "achieved": sfa_flops / t_sfa / 1e12,
                        "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                        "frac": sfa_flops / t_sfa / 1e12 / peaks["bf16_tflops_sustained"],
                        "traffic": per * tokens_rank if (per and uniform) else None,
                        "algorithmic_bytes": sfa_bytes, "peak_source": peaks["source"] + " (sustained bf16)"}
        else:
            per = traffic.get("indexer_scores_tc_kernel")
            roofline = {"kernel": "indexer_scores_tc_kernel + topk_select_kernel", "bound": "hbm",
                        "achieved": idx_bytes / t_index / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": idx_bytes / t_index / 1e9 / peaks["hbm_gbs"],
                        "traffic": per * len(ctx_list) if (per and uniform) else None,
                        "algorithmic_bytes": idx_bytes, "peak_source": peaks["source"]}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cval, cdt, threads, sample = cpu_sample_for(args, args.cpu_passes)
            cpu = {"value": cval, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"{sample}; {args.cpu_passes} passes of {cdt:.1f} s"}
        link_gbs = (h2d + d2h) / link_s / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "warmup_steps_run": n_warm, "ms_per_step": ms_step,
            "ms_per_step_spread": dev_stats, "higher_is_better": True,
            "scaling": args.scaling if args.config == 2 else "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": dict(workload_config(args, world), batch_rank0=len(ctx_list)),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_total,
                    "d2h_bytes_per_step": d2h_total, "ms_per_step": e2e_stats["median"], "ms_per_step_spread": e2e_stats,
                    "serial_ms_per_step": statistics.median(ser_rounds) / args.steps,
                    "mode": "every step copies its activations from pinned host memory (one packed buffer, one copy) and "
                            "its output back; the copies of steps k+1 / k-1 run on their own streams under the compute "
                            "of step k (a CUDA graph)",
                    "roofline": {"bound": "host link", "rank0_bytes_per_step": h2d + d2h,
                                 "probe_gbs_rank0": link_gbs, "probe_ms_per_step": link_s * 1e3,
                                 "compute_ms_per_step": ms_step,
                                 "bound_ms_per_step": max(link_s * 1e3, ms_step),
                                 "frac": max(link_s * 1e3, ms_step) / e2e_stats["median"],
                                 "probe": "concurrent H2D + D2H cudaMemcpyAsync of the loop's own pinned buffers on two streams, "
                                          "all ranks at once, best of at least five rounds", "numa_node": numa}},
            "gpu_launches": int(launches_per_step * args.steps * dev_stats["rounds"]), "clocks": clocks,
            "roofline": roofline, "stages": stage_info, "cpu_baseline": cpu,
        }
        if weak is not None:
            line["weak"] = weak
        _emit_json(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _sum_bytes(h2d, d2h, world, dev):
    if world == 1:
        return h2d, d2h
    import torch.distributed as dist
    t = torch.tensor([h2d, d2h], dtype=torch.int64, device=dev)
    dist.all_reduce(t)
    return int(t[0].item()), int(t[1].item())


# ---- config 3: one long request, index-key range sharded over ranks ---------------------------------------------
def run_config3(args, rank, world, local_rank):
    import torch.distributed as dist
    import pypto_b200
    from pypto_b200 import sharding, synth
    from pypto_b200.lightning_indexer_quant_impl import indexer_scores_topk, topk_select
    from pypto_b200.sparse_flash_attention_quant_impl import sparse_flash_attention_quant_d

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    timer = Timer(dev, world)
    L, s1 = args.ctx, args.s1
    t0, t1 = sharding.token_slice_for_rank(s1, rank, world)
    d = synth.make_long_request(L, s1, 1003, dev, token_slice=(t0, t1))
    n_own = t1 - t0
    begin, end = sharding.key_range_for_rank(L, rank, world)
    res = torch.empty((s1, 1, TOPK), dtype=torch.int32, device=dev)
    sc = torch.empty((s1, TOPK), dtype=torch.float32, device=dev)
    per = math.ceil(s1 / world)
    # candidate exchange: the top-k kernel stores every token's row straight into the owning rank's symmetric-memory
    # buffer ("peer stores": no collective, a barrier), or one NCCL all-to-all where symmetric memory is unavailable
    bufs, exchange = None, "none"
    if world > 1:
        exchange = "nccl all-to-all"
        if args.c3_exchange == "peer":
            try:
                bufs = sharding.PeerCandidateBuffers(s1, TOPK, dev)
                exchange = "peer stores from the top-k kernel (symmetric memory), one barrier"
            except Exception as e:  # noqa: BLE001
                sys.stderr.write(f"config 3: symmetric memory unavailable ({type(e).__name__}: {e}); using the all-to-all\n")
        # every rank must take the same path
        flag = torch.tensor([1 if bufs is not None else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            bufs, exchange = None, "nccl all-to-all"
    a2a_send = torch.empty((world, 2, per, TOPK), dtype=torch.int32, device=dev) if world > 1 and bufs is None else None
    a2a_recv = torch.empty_like(a2a_send) if a2a_send is not None else None
    counts = torch.full((n_own,), world * TOPK, dtype=torch.int32, device=dev)
    merged = torch.empty((n_own, TOPK), dtype=torch.int32, device=dev)
    merged_sc = torch.empty((n_own, TOPK), dtype=torch.float32, device=dev)
    out = torch.empty((1, max(n_own, 1), 128, 512), dtype=torch.bfloat16, device=dev)
    # attention over a slice of the chunk: the same operator with the slice as the request's query tokens and the
    # sequence length cut so that every token keeps its own count of valid keys
    act_slice = torch.tensor([L - s1 + t1], dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ev = {k: [] for k in ("indexer", "gather", "merge", "sfa")}

    def step(i, record=True):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        e[0].record()
        if bufs is not None:
            bufs.barrier()   # nobody is still merging the previous step's candidates
            indexer_scores_topk(d["q_int8"], d["q_scale"], d["idx_k"], d["idx_k_scale"], d["weights"], d["act_seq"],
                                d["block_table"], None, TOPK, key_begin=begin, key_end=end, scatter=bufs.scatter_arg())
            e[1].record()
            bufs.barrier()
            e[2].record()
            cs, ci = bufs.own()
        else:
            indexer_scores_topk(d["q_int8"], d["q_scale"], d["idx_k"], d["idx_k_scale"], d["weights"], d["act_seq"],
                                d["block_table"], res, TOPK, topk_scores=sc, key_begin=begin, key_end=end)
            e[1].record()
        if world > 1:
            if bufs is None:
                # candidates of this rank's own query slice from every rank, one row per token: [n_own, world * topk]
                cs, ci = sharding.exchange_own_slice(sc, res.reshape(s1, TOPK), send=a2a_send, recv=a2a_recv)
                e[2].record()
            if n_own:
                topk_select(cs.contiguous(), counts, TOPK, ids=ci.contiguous(), out_idx=merged, out_scores=merged_sc)
            sel = merged
        else:
            e[2].record()
            sel = res.reshape(s1, TOPK)
        e[3].record()
        if n_own:
            sparse_flash_attention_quant_d(d["q_nope"], d["q_rope"], d["k_nope"], d["k_rope"], d["k_scales"], sel,
                                           d["block_table"], act_slice, out, 128, 1, 576 ** -0.5, TOPK, 128,
                                           d["block_table"].shape[1], None)
        e[4].record()
        if record:
            for k, j in zip(("indexer", "gather", "merge", "sfa"), range(4)):
                ev[k].append((e[j], e[j + 1]))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    n_warm = max(args.warmup, 3)
    launches0 = pypto_b200.launch_count()
    for i in range(n_warm):
        step(i, record=False)
    launches_per_step = (pypto_b200.launch_count() - launches0) // n_warm
    pypto_b200.check_status(dev)
    ms_rounds = timer.rounds(step, args.steps, min_total_ms=args.min_timed_ms, max_rounds=20, after_round=flush.zero_)
    stats = spread(ms_rounds, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    pypto_b200.check_status(dev)
    phase = {k: statistics.median(a.elapsed_time(b) for a, b in v) for k, v in ev.items()}
    if world > 1:
        t = torch.tensor([phase[k] for k in ("indexer", "gather", "merge", "sfa")], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phase = dict(zip(("indexer", "gather", "merge", "sfa"), [float(v) for v in t.tolist()]))
    if rank == 0:
        peaks = load_peaks()
        ms_step = stats["median"]
        value = s1 / (ms_step * 1e-3)
        sent = 2 * per * TOPK * 4 * (world - 1)   # bytes this rank sends to its peers (and receives from them)
        k_valid = [min(TOPK, max(L - s1 + 1 + i, 0)) for i in range(t0, t1)]
        sfa_flops = sum(sfa_flops_per_token(k) for k in k_valid)
        t_sfa = phase["sfa"] * 1e-3
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cval, cdt, threads, sample = cpu_sample_for(args, 1)
            cpu = {"value": cval, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"{sample}; one pass of {cdt:.1f} s"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": n_warm,
            "ms_per_step": ms_step, "ms_per_step_spread": stats, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
            "phases_ms": {"indexer_topk_local": phase["indexer"], "exchange": phase["gather"],
                          "merge_topk": phase["merge"], "sfa_own_slice": phase["sfa"],
                          "exchange_share": phase["gather"] / ms_step, "exchange_form": exchange},
            "nvlink": None if world == 1 else {
                "bytes_sent_per_rank": sent, "bytes_received_per_rank": sent,
                "achieved_gbs_per_direction": sent / (phase["gather"] * 1e-3) / 1e9,
                "peak_gbs_per_direction": NVLINK_PEER_GBS,
                "frac": sent / (phase["gather"] * 1e-3) / 1e9 / NVLINK_PEER_GBS,
                "note": ("with peer stores the bytes cross NVLink inside the top-k kernel of the indexer phase; the exchange "
                         "phase is the barrier alone, so achieved / frac are not a link bandwidth") if bufs is not None else
                        "the all-to-all phase also holds the packing copies into the send buffer"},
            "roofline": {"kernel": "sfa_tc_kernel", "bound": "tensor", "achieved": sfa_flops / t_sfa / 1e12 if t_sfa > 0 else None,
                         "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                         "frac": sfa_flops / t_sfa / 1e12 / peaks["bf16_tflops_sustained"] if t_sfa > 0 else None,
                         "traffic": None, "peak_source": peaks["source"] + " (sustained bf16)"},
            "e2e": None, "gpu_launches": int(launches_per_step * args.steps * stats["rounds"]), "clocks": clocks,
            "cpu_baseline": cpu,
        }
        _emit_json(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ---- DeepSeek-V4 operators ----------------------------------------------------------------------------------------
def run_v4(args):
    """Timings of the DeepSeek-V4 operators at the reference's decode shapes (64 requests x 2 tokens, 64 heads):
    every operator is called through its reference-named entry point, captured once in a CUDA graph and replayed
    with a buffer larger than L2 written between replays; median of CUDA-event durations, one JSON line each."""
    from pypto_b200 import (compress_flash_attention_impl as cfa, compressor_impl as comp, hc_pre_impl as hcp,
                            lightning_indexer_prolog_quant_v4_impl as ipv4, mla_prolog_quant_v4_impl as mlaq,
                            mla_prolog_v4_impl as mlab, sparse_compress_flash_attention_impl as scfa,
                            win_attention_impl as win)
    from pypto_b200 import check_status
    DEV, BF = "cuda", torch.bfloat16
    b, s1, ctx, nq, reps = args.batch, args.s1, min(args.ctx, 8192), 64, 15
    t = b * s1
    g = torch.Generator(device=DEV).manual_seed(4)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def uni(shape, scale=1.0, dtype=BF):
        return ((torch.rand(shape, generator=g, device=DEV) * 2 - 1) * scale).to(dtype)

    def pages(n, blocks_each):
        return torch.randperm(n * blocks_each, generator=g, device=DEV).to(torch.int32).reshape(n, blocks_each).contiguous()

    def timeit(fn):
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
        return statistics.median(times) * 1000.0

    def attention_inputs(cmp_ratio, topk, shared_selection):
        ori_blocks, cmp_len = math.ceil(ctx / 128), ctx // cmp_ratio
        cmp_blocks = max(math.ceil(cmp_len / 128), 1)
        idx = torch.full((t, topk), -1, dtype=torch.int32, device=DEV)
        n = min(cmp_len, topk)
        for tok in range(t):
            if shared_selection and tok % s1:
                idx[tok] = idx[tok - 1]
            else:
                idx[tok, :n] = torch.randperm(cmp_len, generator=g, device=DEV)[:n].to(torch.int32)
        return dict(q=uni((t * nq, 512)), ori_kv=uni((b * ori_blocks * 128, 512)), cmp_kv=uni((b * cmp_blocks * 128, 512)),
                    ori_bt=pages(b, ori_blocks), cmp_bt=pages(b, cmp_blocks), sink=uni((nq,), dtype=torch.float32),
                    seq_q=torch.arange(0, t + 1, s1, dtype=torch.int32, device=DEV),
                    seq_kv=torch.full((b,), ctx, dtype=torch.int32, device=DEV), idx=idx)

    rows = []

    def report(name, us, **extra):
        rows.append(dict(workload="v4", operator=name, us=round(us, 1), tokens=t, **extra))

    for shared in (False, True):
        a = attention_inputs(4, 512, shared)
        us = timeit(lambda: scfa.npu_sparse_compress_flash_attention(
            a["q"], a["seq_q"], a["ori_kv"], a["cmp_kv"], a["ori_bt"], a["cmp_bt"], a["sink"], a["seq_kv"], a["idx"],
            512 ** -0.5, 128, 4))
        report("sparse_compress_flash_attention", us, keys=128 + 512, ctx=ctx,
               selections="shared by the tokens of a request" if shared else "independent random")
    a = attention_inputs(128, 1, False)
    q3 = a["q"].reshape(t, nq, 512)
    ok4, ck4 = a["ori_kv"].reshape(-1, 128, 1, 512), a["cmp_kv"].reshape(-1, 128, 1, 512)
    report("cfa_attention", timeit(lambda: cfa.cfa_attention(q3, ck4, a["sink"], a["cmp_bt"], a["seq_kv"], ok4, a["ori_bt"], 128)),
           keys=128 + ctx // 128, ctx=ctx)
    report("deepseekv4_win_atten",
           timeit(lambda: win.deepseekv4_win_atten(q3, a["ori_bt"], ok4, a["seq_kv"], a["sink"], 128, None, a["seq_q"])),
           keys=128, ctx=ctx)
    # prologs (h 4096, q_lora_rank 1024, 64 heads of 512 / 64 index heads of 128)
    x = uni((t, 4096))
    ang = torch.rand((t, 32), generator=g, device=DEV) * 2 * math.pi
    cos, sin = torch.cos(ang).repeat_interleave(2, -1).to(BF), torch.sin(ang).repeat_interleave(2, -1).to(BF)
    wq_a, wkv = uni((4096, 1024), 0.03), uni((4096, 512), 0.03)
    wq_b = torch.randint(-127, 128, (1024, 64 * 512), generator=g, device=DEV, dtype=torch.int8)
    wq_b_scale = torch.rand((1, 64 * 512), generator=g, device=DEV) * 1e-3 + 1e-4
    gam_q, gam_kv = 1 + uni((1024,), 0.1), 1 + uni((512,), 0.1)
    report("mla_prolog_v4 (quant)", timeit(lambda: mlaq.mla_prolog_v4_in(x, wq_a, wq_b, wkv, cos, sin, gam_q, gam_kv, wq_b_scale)))
    wq_b16 = (wq_b.float() * wq_b_scale).to(BF)
    report("mla_prolog_v4 (bf16)", timeit(lambda: mlab.mla_prolog_v4_in(x, wq_a, wq_b16, wkv, cos, sin, gam_q, gam_kv)))
    qr = torch.randint(-127, 128, (t, 1024), generator=g, device=DEV, dtype=torch.int8)
    iw = torch.randint(-127, 128, (1024, 8192), generator=g, device=DEV, dtype=torch.int8)
    w_proj, had_q = uni((4096, 64), 0.03), uni((128, 128))
    qr_scale = torch.rand((t, 1), generator=g, device=DEV) * 0.02
    iw_scale = torch.rand((8192, 1), generator=g, device=DEV) * 0.002
    report("quant_lightning_indexer_prolog (v4)",
           timeit(lambda: ipv4.npu_quant_lightning_indexer_prolog(qr, iw, x, w_proj, cos, sin, had_q, qr_scale, iw_scale)))
    xh = torch.randn((t, 4, 4096), generator=g, device=DEV).to(BF)
    hc_fn = torch.randn((24, 16384), generator=g, device=DEV) * 0.02
    hc_scale, hc_base = torch.rand((3,), generator=g, device=DEV) + 0.5, torch.randn((24,), generator=g, device=DEV) * 0.5
    report("hc_pre", timeit(lambda: hcp.npu_hc_pre(xh, hc_fn, hc_scale, hc_base)))
    for ratio, dd, rotate, start in ((4, 512, False, 255), (4, 128, True, 255), (128, 512, False, 254)):
        coff = 2 if ratio == 4 else 1
        out_rows = min(t, t // ratio + b)
        xs = uni((b, s1, 4096))
        table = torch.arange(b * 4, dtype=torch.int32, device=DEV).reshape(b, 4)
        kv_state = torch.randn((b * 4, 128, coff * dd), generator=g, device=DEV)
        sc_state = torch.randn((b * 4, 128, coff * dd), generator=g, device=DEV)
        wk, wg = uni((coff * dd, 4096), 0.03), uni((coff * dd, 4096), 0.03)
        ape, weight = torch.randn((ratio, coff * dd), generator=g, device=DEV), torch.ones(dd, device=DEV)
        csin, ccos = uni((out_rows, 64)), uni((out_rows, 64))
        had = uni((dd, dd), dd ** -0.5)
        st = torch.full((b,), start, dtype=torch.int32, device=DEV)
        report("compressor", timeit(lambda: comp.npu_compressor(xs, kv_state, sc_state, table, table, csin, ccos, wk, wg, ape,
                                                                weight, had, st, ratio, 64, rotate)),
               ratio=ratio, d=dd, rotate=rotate, note="every request closes a window in this call")
    check_status()
    for r in rows:
        _emit_json(r)


def run_mla(args):
    """The fused MLA + indexer prolog (mla_indexer_prolog_quant_d) and the MLA prolog alone at `batch * s1` tokens,
    each replayed from a CUDA graph with a buffer larger than L2 written between replays (85 MB + 15 MB of weights
    would otherwise stay in L2); median of CUDA-event durations, one JSON line."""
    from pypto_b200 import check_status, synth
    from pypto_b200.decode_chain import FullDecodeStep
    from pypto_b200 import mla_prolog_quant_impl as mlp
    dev = "cuda"
    t = args.batch * args.s1
    w = synth.make_full_decode_workload([4096] * args.batch, args.s1, 0, 7, dev)
    step = FullDecodeStep(w)
    step.set_inputs(**synth.make_full_step_activations(t, 8, dev))
    q_norm = torch.empty((t, 1536), dtype=torch.int8, device=dev)
    q_norm_scale = torch.empty((t, 1), dtype=torch.float32, device=dev)

    def mla_only():
        mlp.mla_prolog_quant_d(step.x, w.w_dq, w.w_uq_qr, w.w_uq_qr_scale, w.w_uk, w.w_dkv_kr, w.gamma_cq, w.gamma_ckv,
                               step.cos, step.sin, w.cache_index, w.kv_cache, w.kr_cache, w.k_scale_cache, q_norm,
                               q_norm_scale, step.q_nope, step.q_rope, w.kv_cache, w.kr_cache, w.k_scale_cache, 1e-6, 1e-6,
                               "PA_BSND", mlp.MlaTileConfig(), mlp.RopeTileShapeConfig())

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {}
    for name, fn in (("mla_prolog_quant_d", mla_only), ("mla_indexer_prolog_quant_d", step.prolog)):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        times = []
        for _ in range(15):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        out[name] = round(statistics.median(times) * 1000.0, 1)
    check_status()
    weights = 7168 * 1536 * 2 + 1536 * 24576 + 128 * 128 * 512 * 2 + 7168 * 576 * 2
    _emit_json({"workload": "mla", "tokens": t, "us": out, "mla_weight_bytes": weights,
                "mla_weight_stream_gbs": weights / (out["mla_prolog_quant_d"] * 1e-6) / 1e9,
                "timing": "CUDA graph replays, L2 flushed between replays, median of 15 CUDA-event durations"})


_JSON_FD = None


def _reserve_stdout_for_json():
    """stdout carries the JSON line(s) only.  Native libraries write to file descriptor 1 directly (NCCL prints its
    version banner there when NCCL_DEBUG is set), so descriptor 1 is pointed at stderr for the rest of the run and
    the JSON goes out through a saved copy of the original descriptor."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def _emit_json(line):
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_JSON_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4])
    ap.add_argument("--workload", default="chain", choices=["chain", "v4", "mla"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--s1", type=int, default=None)
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--no-weak", action="store_true", help="skip the weak-scaling figure printed beside a strong run")
    ap.add_argument("--cpu-requests", type=int, default=None, help="requests (config 3: query tokens) in the bounded CPU sample")
    ap.add_argument("--cpu-passes", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--min-timed-ms", type=float, default=500.0, help="keep timing rounds of --steps until this much "
                    "timed region has accumulated (profiling runs pass 0: three rounds)")
    ap.add_argument("--c3-exchange", default="peer", choices=["peer", "a2a"],
                    help="config 3: how the ranks' top-k candidates reach the rank that owns a token")
    ap.add_argument("--kv-splits", type=int, default=0, help="fix the key splits of the attention kernel (0: automatic)")
    args = ap.parse_args()
    defaults = {2: (64, 65536, 2), 3: (1, 131072, 4096), 4: (256, None, 2)}[args.config]
    args.batch = args.batch if args.batch is not None else defaults[0]
    args.ctx = args.ctx if args.ctx is not None else defaults[1]
    args.s1 = args.s1 if args.s1 is not None else defaults[2]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    _reserve_stdout_for_json()
    if args.cpu_requests is None:
        if args.config == 3:
            args.cpu_requests = 8
        else:
            args.cpu_requests = min(args.batch, 64) if (args.impl == "ours" and args.config == 2) else 4
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode chain has no CPU fallback")
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (one process per GPU)")
    if args.workload in ("v4", "mla"):
        if rank == 0:
            if args.batch == 256:
                args.batch = 64
            (run_v4 if args.workload == "v4" else run_mla)(args)
        return
    if args.config == 3:
        run_config3(args, rank, world, local_rank)
    else:
        run_chain(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
