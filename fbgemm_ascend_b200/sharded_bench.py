"""Multi-GPU leg of the benchmark: the table-wise sharded configuration (benchmark configuration 4).

Launched by ``bench.py --gpus N`` under ``torch.distributed.run`` (one rank per GPU, NCCL).  Per rank:
64 INT8 tables of 12M x 128 (about 110 GB of rows), the global batch of 65536 bags per table with
Poisson(32) bag lengths clipped to [1, 128] and Zipf(1.05) indices, SUM pooling, fp16 output; then the
exchange of pooled rows and the permutation into a seeded random feature order.  Per-GPU work is fixed
as N grows (weak scaling).  Rank 0 prints the JSON line.
"""
from __future__ import annotations

import json
import os
import random
import statistics
import time

import torch
import torch.distributed as dist


def _allreduce_max(x: float, device) -> float:
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _allreduce_sum(x: float, device) -> float:
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def _timed(fn, steps, device):
    """Device time (ms) of `steps` calls, barrier + synchronize on both sides, max over ranks."""
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    return _allreduce_max(e0.elapsed_time(e1), device)


def run_sharded(args) -> None:
    import bench as B   # the driver's entry script: shared helpers (clock sampler, peaks, metric names)
    import fbgemm_ascend_b200  # noqa: F401
    from fbgemm_ascend_b200 import workloads as W
    from fbgemm_ascend_b200.sharded import ShardPlan, TableWiseShardedLookup
    from fbgemm_ascend_b200.types import SparseType

    rank, world, local = B.dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    name = "c4" if args.workload == "auto" else args.workload
    ws = W.spec(name, scale_E=args.scale_e, scale_B=args.scale_b)
    T_loc = ws.T
    T_glob = T_loc * world
    if ws.B % world:
        raise SystemExit(f"global batch {ws.B} is not divisible by {world} ranks")
    order = list(range(T_glob))
    random.Random(ws.seed).shuffle(order)
    plan = ShardPlan(world=world, rank=rank, dims=[ws.dims[0]] * T_glob, feature_order=order, global_batch=ws.B)
    t0 = time.time()
    tables = W.build_tables(ws, dev, table_seed_offset=rank)
    n_batches = max(1, min(args.batches, 2))
    batches = [W.make_batch(ws, dev, batch_seed=i, table_ids=plan.local_tables) for i in range(n_batches)]
    torch.cuda.synchronize()
    build_s = time.time() - t0

    results = {}
    modes = ["direct", "nccl"] if args.exchange == "both" else [args.exchange]
    sh = {}
    for mode in modes:
        try:
            sh[mode] = TableWiseShardedLookup(plan, tables, group=dist.group.WORLD, exchange=mode, device=dev)
        except Exception as e:  # e.g. symmetric memory not available: the NCCL path still stands
            results[mode] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    rows_step = [b.num_rows for b in batches]
    sampler = B.ClockSampler(local)
    clocks = None
    for mode, obj in sh.items():
        def step(i, obj=obj):
            b = batches[i % n_batches]
            return obj(b.indices, b.offsets, b.weights)
        for i in range(max(args.warmup, 3)):
            step(i)
        if rank == 0 and clocks is None:
            sampler.start()
            time.sleep(0.3)
        w0 = time.time()
        ms = _timed(step, args.steps, dev)
        if rank == 0 and clocks is None:
            clocks = sampler.stop(w0, time.time())
        rows = _allreduce_sum(float(sum(rows_step[i % n_batches] for i in range(args.steps))), dev)
        results[mode] = {"value": rows / (ms * 1e-3), "ms_per_step": ms / args.steps}

    # the lookup kernel alone on every rank (no exchange, no permute): the per-GPU base of the weak scaling
    def lookup_only(i):
        b = batches[i % n_batches]
        return tables.forward(b.indices, b.offsets, b.weights)
    for i in range(3):
        lookup_only(i)
    ms_lk = _timed(lookup_only, args.steps, dev)
    acct = W.algorithmic_bytes(ws, batches[0])
    peak, peak_kind = B._peaks()
    kern_ms = ms_lk / args.steps
    achieved = acct["algorithmic"] / (kern_ms * 1e-3) / 1e9

    # cross-check the two exchange paths against each other on this rank
    agree = None
    if "direct" in sh and "nccl" in sh:
        b = batches[0]
        a = sh["direct"](b.indices, b.offsets, b.weights).clone()
        c = sh["nccl"](b.indices, b.offsets, b.weights)
        agree = bool(torch.equal(a, c))
        agree = bool(_allreduce_sum(0.0 if agree else 1.0, dev) == 0.0)

    main = "direct" if "value" in results.get("direct", {}) else "nccl"
    e2e = None
    if not args.no_e2e:
        e2e = B.run_e2e(tables, batches, ws, args, torch.cuda.current_stream(), forward=lambda i, o, w: sh[main](i, o, w))
        e2e["value"] = _allreduce_sum(e2e["value"], dev)   # rows/s of all ranks (each rank timed its own pipeline)
    if rank == 0:
        line = {
            "metric": B.METRIC, "value": results[main]["value"], "unit": B.UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": results[main]["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": "u8 rows (int8 codes, fp16 scale/bias), fp32 accumulate, fp16 out", "data": "synthetic",
            "config": {"workload": f"{ws.name} table-wise sharded: {T_loc} tables/rank x E={ws.E} x D={ws.dims[0]} INT8, "
                                   f"global B={ws.B}, L={ws.length_dist}, idx={ws.index_dist} int64, SUM -> fp16, exchange="
                                   f"{main}, then feature-order permute",
                       "world": world, "rows_per_step_per_rank": rows_step[0], "table_bytes_per_rank": W.table_bytes(ws),
                       "scale_e": args.scale_e, "scale_b": args.scale_b, "build_s": round(build_s, 1),
                       "l2_policy": "tables far larger than L2; request batches rotate"},
            "exchange": results, "exchange_paths_agree": agree,
            "weak_scaling_base": {"what": "lookup kernel only, per rank, no exchange", "ms_per_step": kern_ms,
                                  "rows_per_s_per_gpu": rows_step[0] / (kern_ms * 1e-3)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "tbe_pooled_kernel", "kernel_ms": kern_ms,
                         "algorithmic_bytes_per_launch": acct["algorithmic"], "frac_of_nominal_8TBs": achieved / 8000.0},
            "cpu_baseline": None, "e2e": e2e,
            "gpu_launches": args.steps * (1 if main == "direct" else 2), "clocks": clocks,
        }
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
