#!/usr/bin/env python3
"""Benchmark of the sparse-attention decode chain (indexer prolog -> lightning indexer + top-2048 ->
sparse flash attention over the int8 paged cache) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch 64] [--ctx 65536] [--s1 2] [--scaling weak|strong]

One step = one decode step of the whole chain for `batch` requests (batch*s1 query tokens).  The metric is
decode tokens/s (whole job, all ranks).  With N > 1 (torchrun, one rank per GPU) requests are sharded over
ranks with no collective on the data path; "weak" keeps `batch` requests per rank, "strong" splits them.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
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


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---- algorithmic work per unit ---------------------------------------------------------------------------
def sfa_flops_per_token(k):        # 2*128*K*(576+512)
    return 278528.0 * k


def sfa_bytes_per_token(k, ctx):   # gathered rows + indices + Q + O + page table
    return k * (512 + 16 + 128) + k * 4 + 147456 + 131072 + ((ctx + 127) // 128) * 4


def indexer_bytes_per_request(ctx, s1):
    return ctx * 130 + ((ctx + 127) // 128) * 4 + s1 * (8192 + 128 + 128) + s1 * 8192


# DRAM traffic per unit from the ncu capture summarised in profiles/tcgen05_kernels_b16_ctx64k.md
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch / units of that launch); it grows in proportion
# to the units, so a full launch is units x this figure.
NCU_SFA_TRAFFIC_PER_TOKEN = (51.868672e6 + 0.504832e6) / 32
NCU_INDEXER_TRAFFIC_PER_REQUEST = (136.643584e6 + 5.581312e6) / 16


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


# ---- CPU reference arm ------------------------------------------------------------------------------------
def cpu_chain_sample(n_req, ctx, s1, seed, steps=1, warmup=0):
    """Time the CPU oracle (the reference goldens' algorithm) on a bounded sample of the workload:
    `n_req` requests of the same shape, whole chain.  Returns (tokens/s, seconds per step, threads)."""
    from oracle import dsv32_oracle as orc
    from pypto_b200 import synth
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    w = synth.make_decode_workload([ctx] * n_req, s1, seed, "cpu")

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
    return n_req * s1 / dt, dt, threads


def run_reference(args, rank, world):
    if rank != 0:
        return
    n_req = args.cpu_requests
    val, dt, threads = cpu_chain_sample(n_req, args.ctx, args.s1, 1002, steps=args.steps, warmup=min(args.warmup, 1))
    sample = f"{n_req} requests x {args.s1} tokens at ctx {args.ctx} per step (same chain, same distributions)"
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


def workload_config(args, world):
    per_rank = args.batch if args.scaling == "weak" else max(args.batch // world, 1)
    return {"workload": f"config 2: full decode chain, batch {args.batch}, ctx {args.ctx}, MTP s1={args.s1}, "
                        f"128 heads, top-k {TOPK}",
            "batch_per_gpu": per_rank, "global_batch": per_rank * world, "ctx": args.ctx, "s1": args.s1, "topk": TOPK,
            "parallelism": f"requests sharded over {world} GPU(s), no collective",
            "l2_policy": "inputs larger than L2 (per-GPU working set > 3 GB at the default shape)",
            "launch": "each stage replayed from a CUDA graph captured from the operator entry points"}


# ---- our arm -------------------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    import pypto_b200
    from pypto_b200 import synth
    from pypto_b200.decode_chain import HostPipelinedDecode, SparseDecodeStep

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode chain has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    per_rank = args.batch if args.scaling == "weak" else max(args.batch // world, 1)
    w = synth.make_decode_workload([args.ctx] * per_rank, args.s1, 1002 + rank, dev)
    step = SparseDecodeStep(w)
    h2d, d2h = step.enable_host_io()
    tokens_per_rank = per_rank * args.s1

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, stage_events=False):
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)] if stage_events else None
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(steps):
            if stage_events:  # the three stages replayed from their CUDA graphs, an event between them
                ev[i][0].record()
                stage_graphs[0].replay()
                ev[i][1].record()
                stage_graphs[1].replay()
                ev[i][2].record()
                stage_graphs[2].replay()
                ev[i][3].record()
            else:
                fn()
        end.record()
        barrier()
        ms = start.elapsed_time(end)
        stages = None
        if stage_events:
            stages = [sum(e[j].elapsed_time(e[j + 1]) for e in ev) / steps for j in range(3)]
        return ms, stages

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
    while n_warm < max(args.warmup, 3) or time.perf_counter() - t_warm < 1.0:
        step.step()
        n_warm += 1
        if n_warm % 8 == 0:
            torch.cuda.synchronize(dev)
    pypto_b200.check_status(dev)
    launches0 = pypto_b200.launch_count()
    step.step()
    launches_per_step = pypto_b200.launch_count() - launches0  # counted on an eager step: graph replays do not pass
    stage_graphs = step.capture(per_stage=True)                # through the library's launch counter
    for _ in range(3):
        step.replay()
    ms, stages = timed(None, args.steps, stage_events=True)
    launches = launches_per_step * args.steps
    # end-to-end: pinned host activations in, attention output back, every step
    for _ in range(2):
        step.step_from_host()
    ms_e2e_serial, _ = timed(step.step_from_host, args.steps)
    # ... and with the copies of steps k+1 / k-1 overlapping the compute of step k (three streams)
    pipe = HostPipelinedDecode(step, use_graphs=True)
    for _ in range(3):
        pipe.submit(step.host_in)
    pipe.drain()

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        pipe.submit(step.host_in)
    pipe.drain()
    end.record()
    barrier()
    ms_e2e = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else None
    pypto_b200.check_status(dev)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = max_over_ranks(ms)
    ms_e2e = max_over_ranks(ms_e2e)
    ms_e2e_serial = max_over_ranks(ms_e2e_serial)
    total_tokens = tokens_per_rank * world * args.steps
    value = total_tokens / (ms * 1e-3)
    e2e_value = total_tokens / (ms_e2e * 1e-3)

    if rank == 0:
        peaks = load_peaks()
        t_prolog, t_index, t_sfa = [s * 1e-3 for s in stages]  # seconds per step (rank 0)
        sfa_flops = sfa_flops_per_token(min(TOPK, args.ctx)) * tokens_per_rank
        sfa_bytes = sfa_bytes_per_token(min(TOPK, args.ctx), args.ctx) * tokens_per_rank
        idx_bytes = indexer_bytes_per_request(args.ctx, args.s1) * per_rank
        stage_info = {
            "prolog": {"ms": t_prolog * 1e3, "achieved_gbs": prolog_bytes_per_call(tokens_per_rank) / t_prolog / 1e9,
                       "hbm_frac": prolog_bytes_per_call(tokens_per_rank) / t_prolog / 1e9 / peaks["hbm_gbs"]},
            "indexer_topk": {"ms": t_index * 1e3, "achieved_gbs": idx_bytes / t_index / 1e9,
                             "hbm_frac": idx_bytes / t_index / 1e9 / peaks["hbm_gbs"]},
            "sfa": {"ms": t_sfa * 1e3, "achieved_tflops": sfa_flops / t_sfa / 1e12,
                    "tensor_frac": sfa_flops / t_sfa / 1e12 / peaks["bf16_tflops_sustained"],
                    "achieved_gbs": sfa_bytes / t_sfa / 1e9, "hbm_frac": sfa_bytes / t_sfa / 1e9 / peaks["hbm_gbs"]},
        }
        if t_sfa >= t_index:
            roofline = {"kernel": "sfa_tc_kernel", "bound": "tensor", "achieved": sfa_flops / t_sfa / 1e12,
                        "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                        "frac": sfa_flops / t_sfa / 1e12 / peaks["bf16_tflops_sustained"],
                        "traffic": NCU_SFA_TRAFFIC_PER_TOKEN * tokens_per_rank if args.ctx == 65536 else None,
                        "algorithmic_bytes": sfa_bytes,
                        "peak_source": peaks["source"] + " (sustained bf16)"}
        else:
            roofline = {"kernel": "indexer_scores_tc_kernel + topk_select_kernel", "bound": "hbm",
                        "achieved": idx_bytes / t_index / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": idx_bytes / t_index / 1e9 / peaks["hbm_gbs"],
                        "traffic": NCU_INDEXER_TRAFFIC_PER_REQUEST * per_rank if args.ctx == 65536 else None,
                        "algorithmic_bytes": idx_bytes, "peak_source": peaks["source"]}
        # CPU baseline on a bounded sample of the same workload (rank 0, N=1 only)
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cval, cdt, threads = cpu_chain_sample(args.cpu_requests, args.ctx, args.s1, 1002, steps=args.cpu_passes)
            cpu = {"value": cval, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"{args.cpu_requests} requests x {args.s1} tokens at ctx {args.ctx}, whole chain, "
                             f"{args.cpu_passes} passes of {cdt:.1f} s"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "warmup_steps_run": n_warm,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(args, world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                    "ms_per_step": ms_e2e / args.steps, "serial_ms_per_step": ms_e2e_serial / args.steps,
                    "mode": "every step copies its inputs from pinned host memory and its output back; the copies "
                            "of steps k+1 / k-1 run on their own streams under the compute of step k (a CUDA graph)"},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline, "stages": stage_info,
            "cpu_baseline": cpu,
        }
        _emit_json(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_JSON_FD = None


def _reserve_stdout_for_json():
    """stdout carries the one JSON line only.  Native libraries write to file descriptor 1 directly (NCCL prints its
    version banner there when NCCL_DEBUG is set), so descriptor 1 is pointed at stderr for the rest of the run and
    the JSON line goes out through a saved copy of the original descriptor."""
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
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=65536)
    ap.add_argument("--s1", type=int, default=2)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--cpu-requests", type=int, default=None, help="requests in the bounded CPU sample")
    ap.add_argument("--cpu-passes", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    _reserve_stdout_for_json()
    if args.cpu_requests is None:
        args.cpu_requests = min(args.batch, 64) if args.impl == "ours" else 4
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (one process per GPU)")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
