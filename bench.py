#!/usr/bin/env python
"""Benchmark of the quantized TBE inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|c1..c5]

One "step" is one pooled lookup (``torch.ops.fbgemm.int_nbit_split_embedding_codegen_lookup_function``)
over one synthetic request batch.  At N=1 the workload is benchmark configuration 2 (26 INT8 tables of
1M x 128, B=2048, Poisson(30) bag lengths, Zipf(1.05) indices, int64, SUM -> fp16); at N>1 it is the
table-wise sharded configuration 4 (64 INT8 tables of 12M x 128 per rank, global B=65536, lookup ->
exchange of pooled rows over NVLink -> feature-order permutation), weak scaling.  Rank 0 prints one
JSON line.

``--impl reference`` times the CPU path the reference's tests compare against: the FBGEMM
EmbeddingSpMDM kernels (as shipped in libtorch_cpu.so) driven in the table-batched layout with all
host threads, on the same configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (workload, scale_e, scale_b) -> bytes
NCU_TRAFFIC_BYTES = {("c2", 1.0, 1.0): 155_366_912 + 33_108_992}
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "pooled_lookup_rows_per_s"
UNIT = "rows/s"


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        rows = [l.split(", ") for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or \
               [l.split(", ") for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.strip().lower() == "active":
                        reasons.add(name)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ---------------------------------------------------------------------------------------------
# CPU arm: the FBGEMM kernels (reference-side CPU path) or the C restatement, on host cores.
# ---------------------------------------------------------------------------------------------

def cpu_lookup_timer(ws, tables, batches, impl: str, budget_s: float, min_calls: int = 3):
    """Times oracle lookups on the host over the given batches for about ``budget_s`` seconds.
    Returns (rows per second, calls, seconds, threads)."""
    import numpy as np
    import oracle as O

    dev = tables.weights_dev.cpu().numpy()
    wo = tables.weights_offsets.cpu().numpy()
    wt = tables.weights_tys.cpu().numpy()
    do = tables.D_offsets.cpu().numpy()
    host = [(b.indices.cpu().numpy(), b.offsets.cpu().numpy(), None if b.weights is None else b.weights.cpu().numpy())
            for b in batches]
    out_ty = int(ws.output_dtype)
    O.tbe_lookup(dev, wo, wt, do, host[0][0], host[0][1], int(ws.pooling), host[0][2], out_ty, impl=impl)  # warm-up / JIT
    rows = 0
    calls = 0
    t0 = time.perf_counter()
    while True:
        idx, offs, w = host[calls % len(host)]
        O.tbe_lookup(dev, wo, wt, do, idx, offs, int(ws.pooling), w, out_ty, impl=impl)
        rows += idx.size
        calls += 1
        dt = time.perf_counter() - t0
        if calls >= min_calls and dt >= budget_s:
            break
    return rows / dt, calls, dt, O.num_threads(impl)


def run_reference_arm(args):
    """``--impl reference``: the CPU path on this box's host cores, same configuration and metric."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from fbgemm_ascend_b200 import workloads as W
    import oracle as O
    O.build()
    name = "c2" if args.workload == "auto" and args.gpus == 1 else ("c4" if args.workload == "auto" else args.workload)
    note = ""
    if name in ("c3", "c4", "c5"):
        # tables of 30-110 GB do not fit host memory next to the process: scale rows per table, keep the rest
        ws = W.spec(name, scale_E=1.0 / 16, scale_B=1.0 / 16)
        note = " (scaled-E: rows per table and batch / 16 to fit host memory)"
    else:
        ws = W.spec(name)
    dev = torch.device("cuda:0") if torch.cuda.is_available() else None
    if dev is None:
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device to generate the workload on"}))
        return
    tables = W.build_tables(ws, dev)
    batches = [W.make_batch(ws, dev, batch_seed=i) for i in range(2)]
    import numpy as np
    host = [(b.indices.cpu().numpy(), b.offsets.cpu().numpy(), None if b.weights is None else b.weights.cpu().numpy())
            for b in batches]
    hdev = tables.weights_dev.cpu().numpy()
    wo, wt, do = (tables.weights_offsets.cpu().numpy(), tables.weights_tys.cpu().numpy(), tables.D_offsets.cpu().numpy())
    del tables
    torch.cuda.empty_cache()

    def step(i):
        idx, offs, w = host[i % len(host)]
        O.tbe_lookup(hdev, wo, wt, do, idx, offs, int(ws.pooling), w, int(ws.output_dtype), impl="ref")
        return idx.size

    for i in range(args.warmup):
        step(i)
    t0 = time.perf_counter()
    rows = 0
    for i in range(args.steps):
        rows += step(i)
    dt = time.perf_counter() - t0
    value = rows / dt
    threads = O.num_threads("ref")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 rows, fp32 accumulate", "data": "synthetic",
        "config": {"workload": ws.name + note, "tables": ws.T, "rows_per_table": ws.E, "dim": ws.dims[0], "batch": ws.B,
                   "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "reference",
                         "sample": f"{args.steps} full {ws.name} batches, FBGEMM EmbeddingSpMDM kernels from libtorch_cpu.so, "
                                   f"{threads} OpenMP threads{note}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def time_region(fn, steps: int, stream: torch.cuda.Stream, barrier=None) -> float:
    """Device time (ms) of ``steps`` calls of fn(i), bracketed by barrier + synchronize."""
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(i)
    e1.record(stream)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def run_single_gpu(args):
    import fbgemm_ascend_b200  # noqa: F401  (fails loudly without the CUDA libraries)
    from fbgemm_ascend_b200 import workloads as W
    from fbgemm_ascend_b200.types import SparseType

    name = "c2" if args.workload == "auto" else args.workload
    ws = W.spec(name, scale_E=args.scale_e, scale_B=args.scale_b)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream()
    t_build = time.time()
    tables = W.build_tables(ws, dev)
    n_batches = args.batches
    batches = [W.make_batch(ws, dev, batch_seed=i) for i in range(n_batches)]
    torch.cuda.synchronize()
    t_build = time.time() - t_build

    def step(i):
        b = batches[i % n_batches]
        return tables.forward(b.indices, b.offsets, b.weights)

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    w0 = time.time()
    ms = time_region(step, args.steps, stream)
    w1 = time.time()
    rows = sum(batches[i % n_batches].num_rows for i in range(args.steps))
    value = rows / (ms * 1e-3)

    # per-launch duration of the lookup kernel, CUDA events around every launch on its stream
    evs = []
    for i in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        step(i)
        b.record(stream)
        evs.append((a, b))
    torch.cuda.synchronize()
    per_launch_ms = [a.elapsed_time(b) for a, b in evs]
    kern_ms = statistics.mean(per_launch_ms)
    clocks = sampler.stop(w0, time.time())
    acct = [W.algorithmic_bytes(ws, batches[i % n_batches]) for i in range(args.steps)]
    alg_bytes = statistics.mean(a["algorithmic"] for a in acct)
    peak, peak_kind = _peaks()
    achieved = alg_bytes / (kern_ms * 1e-3) / 1e9

    # end to end: host buffers in pinned memory, H2D of the request, lookup, D2H of the pooled output
    e2e = None if args.no_e2e else run_e2e(tables, batches, ws, args, stream)

    cpu = None
    if not args.no_cpu:
        try:
            import oracle as O
            O.build()
            v, calls, secs, threads = cpu_lookup_timer(ws, tables, batches[:2], "ref", args.cpu_seconds)
            cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "reference",
                   "sample": f"{calls} full {ws.name} batches in {secs:.1f} s; FBGEMM EmbeddingSpMDM CPU kernels "
                             f"(libtorch_cpu.so) in the table-batched layout, {threads} OpenMP threads"}
        except Exception as e:  # the CPU checker is not part of the product path
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": f"failed: {e}"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 rows (int8 codes, fp16 scale/bias), fp32 accumulate, fp16 out" if name in ("c1", "c2", "c4") else
                 "mixed quantized rows, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"{ws.name}: T={ws.T} x E={ws.E} x D={sorted(set(ws.dims))} "
                               f"{sorted(set(t.name for t in ws.tys))}, B={ws.B}, L={ws.length_dist}, idx={ws.index_dist} "
                               f"{str(ws.index_dtype).split('.')[-1]}, pool={ws.pooling.name}, out={SparseType(ws.output_dtype).name}",
                   "rows_per_step": rows / args.steps, "table_bytes": W.table_bytes(ws),
                   "scale_e": args.scale_e, "scale_b": args.scale_b,
                   "l2_policy": f"tables ({W.table_bytes(ws) / 1e9:.2f} GB) larger than L2; {n_batches} distinct request "
                                "batches rotate, so hot rows stay L2-resident as in steady-state serving",
                   "build_s": round(t_build, 1)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get((name, args.scale_e, args.scale_b)), "traffic_source": "ncu capture of one "
                     "launch of this workload (profiles/tbe_pooled_kernel_c2.md); null for workloads not captured",
                     "peak_kind": peak_kind, "kernel": "tbe_pooled_kernel",
                     "kernel_ms": kern_ms, "algorithmic_bytes_per_launch": alg_bytes,
                     "padded_bytes_per_launch": statistics.mean(a["padded"] for a in acct),
                     "sector_bytes_per_launch": statistics.mean(a["sector"] for a in acct),
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "cpu_baseline": cpu,
        "e2e": e2e,
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line))


def run_e2e(tables, batches, ws, args, stream, forward=None):
    """Same metric through the operator with HOST buffers: every step copies its request (indices,
    offsets, weights) from pinned host memory, runs the lookup and reads the pooled output back
    to pinned host memory.  Three streams keep copy-in, lookup and copy-out of consecutive steps
    in flight at once (double buffering), as a serving loop would."""
    dev = tables.device
    n = len(batches)
    forward = forward or tables.forward
    host_in = []
    for b in batches:
        host_in.append((b.indices.cpu().pin_memory(), b.offsets.cpu().pin_memory(),
                        None if b.weights is None else b.weights.cpu().pin_memory()))
    NBUF = 3
    out0 = forward(batches[0].indices, batches[0].offsets, batches[0].weights)
    max_idx = max(b.num_rows for b in batches)
    dbuf = [(torch.empty(max_idx, dtype=batches[0].indices.dtype, device=dev),
             torch.empty_like(batches[0].offsets),
             torch.empty(max_idx, dtype=torch.float32, device=dev) if ws.weighted else None) for _ in range(NBUF)]
    host_out = [torch.empty(out0.shape, dtype=out0.dtype).pin_memory() for _ in range(NBUF)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(NBUF)]
    ev_k = [torch.cuda.Event() for _ in range(NBUF)]
    ev_out = [torch.cuda.Event() for _ in range(NBUF)]
    h2d = d2h = 0

    def step(i):
        nonlocal h2d, d2h
        k = i % NBUF
        hi, ho, hw = host_in[i % n]
        di, do_, dw = dbuf[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_k[k])          # the lookup that last read this buffer is done
            di[:hi.numel()].copy_(hi, non_blocking=True)
            do_.copy_(ho, non_blocking=True)
            if hw is not None:
                dw[:hw.numel()].copy_(hw, non_blocking=True)
            ev_in[k].record(s_in)
        stream.wait_event(ev_in[k])
        # an output may live in a buffer that is rewritten two steps later (the sharded path double-buffers
        # its peer-visible result): the read-back of step i-2 must be over before step i runs
        stream.wait_event(ev_out[(i - 2) % NBUF])
        out = forward(di[:hi.numel()], do_, None if hw is None else dw[:hw.numel()])
        ev_k[k].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_k[k])
            s_out.wait_event(ev_out[k])
            host_out[k].copy_(out, non_blocking=True)
            ev_out[k].record(s_out)
            out.record_stream(s_out)
        return hi.numel() * hi.element_size() + ho.numel() * ho.element_size() + (hw.numel() * 4 if hw is not None else 0), \
            out.numel() * out.element_size()

    for i in range(3):
        step(i)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        a, b = step(i)
        h2d += a
        d2h += b
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    rows = sum(batches[i % n].num_rows for i in range(args.steps))
    return {"value": rows / dt, "unit": UNIT, "h2d_bytes_per_step": h2d / args.steps, "d2h_bytes_per_step": d2h / args.steps,
            "ms_per_step": dt / args.steps * 1e3, "pipelined": True}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--batches", type=int, default=8, help="distinct request batches that rotate")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--exchange", default="both", choices=["both", "direct", "nccl"],
                    help="multi-GPU: peer-store epilogue, NCCL all-to-all + permute kernel, or time both")
    ap.add_argument("--scale-e", type=float, default=1.0, help="scale rows per table (small cases for profiling)")
    ap.add_argument("--scale-b", type=float, default=1.0, help="scale the batch size (small cases for profiling)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--probe-gather", action="store_true",
                    help="run the row-gather ceiling probe (rows/s the memory system delivers for scattered rows, "
                         "no dequantisation) instead of the benchmark")
    ap.add_argument("--probe-max-gib", type=float, default=120.0, help="largest table the probe may allocate")
    args = ap.parse_args()
    if args.probe_gather:
        probe = os.path.join(ROOT, "fbgemm_ascend_b200", "lib", "tbe_b200_row_gather_probe")
        if not os.path.exists(probe):
            raise SystemExit(f"{probe} is missing: run `python -m fbgemm_ascend_b200.build`")
        raise SystemExit(subprocess.call([probe, str(args.probe_max_gib)]))
    if args.impl == "reference":
        run_reference_arm(args)
        return
    rank, world, local = dist_env()
    if args.gpus > 1 or world > 1:
        from fbgemm_ascend_b200.sharded_bench import run_sharded
        run_sharded(args)
        return
    run_single_gpu(args)


if __name__ == "__main__":
    main()
