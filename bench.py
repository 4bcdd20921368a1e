#!/usr/bin/env python
"""Benchmark of the tree-ensemble inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic rows.  Prints ONE
JSON line (rank 0).  At N > 1 (launched under torch.distributed.run, one rank per GPU)
rows are sharded across GPUs with no collective ("weak" scaling: every GPU gets the
full batch of the workload); ``--shard trees`` partitions the trees instead and sums
per-row partials with an NCCL reduce.

``--impl reference`` times the reference's CPU implementation of the same path on the
host cores (the reference's own DecisionForest.h through oracle/_ref when that shim is
present, else the C restatement of its parallel CPU schedule), on bounded samples.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from treebeard_b200 import synth  # noqa: E402

HBM_FALLBACK_GBS = 6650.0

# DRAM bytes per row (dram__bytes_read.sum + dram__bytes_write.sum) of the walk kernel, from
# one ncu capture per workload on a reduced batch (see profiles/); traffic grows in
# proportion to the rows, so a launch's traffic is this figure times its rows.
NCU_DRAM_BYTES_PER_ROW = {"c3": 8189.0, "c2": 118.2, "c4": 76.3}


def bytes_per_row(cfg):
    """Algorithmic HBM bytes per predicted row: features in + prediction out."""
    return 4 * cfg["F"] + (1 if cfg["classes"] > 0 else 4)


def visits_per_row(cfg):
    """Node visits of the fixed-depth walk: trees x decision levels."""
    return cfg["T"] * cfg["D"]


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_threads():
    """Host threads this process may use.  torch.distributed.run exports OMP_NUM_THREADS=1
    for its workers; the CPU arms size their OpenMP teams from the affinity mask instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# ---------------------------------------------------------------------------
# reference arm: the CPU implementation of the path on the host cores


def run_reference(args, cfg):
    rank, _, world = dist_env()
    if rank != 0:
        return
    # before the OpenMP runtime starts: the reference's walker takes its team size from here
    os.environ["OMP_NUM_THREADS"] = str(host_threads())
    from oracle import oracle
    forest, marg, n_full = synth.make_config(args.workload, rows=args.rows)
    n_full = args.rows or n_full
    use_ref = oracle.ref_lib() is not None and not args.port
    threads = host_threads()
    if use_ref:
        engine = oracle.RefForest(forest)
        run = engine.predict
        kind = "reference"
    else:
        engine = oracle.CpuBaseline(forest)
        run = lambda x: engine.predict(x, threads)  # noqa: E731
        kind = "port"
    pilot_rows = max(threads * 8, 256)
    X = synth.config_rows(args.workload, marg, min(n_full, 1 << 16))
    t0 = time.perf_counter()
    run(X[:pilot_rows])
    pilot = time.perf_counter() - t0
    budget = 120.0 / max(1, args.steps + args.warmup)           # seconds per step
    sample = int(min(len(X), max(pilot_rows, pilot_rows * min(budget, 4.0) / max(pilot, 1e-6))))
    Xs = np.ascontiguousarray(X[:sample])
    for _ in range(args.warmup):
        run(Xs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run(Xs)
    dt = (time.perf_counter() - t0) / args.steps
    value = sample / dt
    desc = (f"first {sample} rows of the {args.workload} batch ({n_full} rows) per step, "
            f"{threads} OpenMP threads, " +
            ("reference DecisionForest::Predict_Float via oracle/_ref" if use_ref else
             "C restatement of the reference's parallel CPU schedule"))
    line = {"impl": "reference", "metric": "rows_per_second", "value": value, "unit": "rows/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, cfg, n_full, world),
            "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": kind,
                             "sample": desc},
            "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, n_rows, world):
    return {"workload": f"{args.workload}: {cfg['desc']}, {n_rows} rows per GPU",
            "trees": cfg["T"], "levels": cfg["D"], "features": cfg["F"], "classes": cfg["classes"],
            "rows_per_gpu": n_rows, "sharding": args.shard if world > 1 else "none",
            "representation": args.representation, "tile_size": args.tile_size,
            "l2": "inputs larger than L2 (no flush needed)"
                  if n_rows * cfg["F"] * 4 > (126 << 20) else "L2 flushed between timed steps"}


# ---------------------------------------------------------------------------
# the B200 arm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(synth.CONFIGS))
    ap.add_argument("--rows", type=int, default=None, help="rows per GPU (default: the workload's)")
    ap.add_argument("--trees", type=int, default=None)
    ap.add_argument("--shard", default="rows", choices=["rows", "trees"])
    ap.add_argument("--representation", default="auto")
    ap.add_argument("--tile-size", type=int, default=1)
    ap.add_argument("--rows-per-block", type=int, default=0)
    ap.add_argument("--rows-per-thread", type=int, default=0)
    ap.add_argument("--tree-threads", type=int, default=0)
    ap.add_argument("--tree-chunks", type=int, default=0)
    ap.add_argument("--cache-trees", type=int, default=0)
    ap.add_argument("--port", action="store_true", help="reference arm: force the C restatement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    cfg = dict(synth.CONFIGS[args.workload])
    if args.trees:
        cfg["T"] = args.trees
    if args.impl == "reference":
        return run_reference(args, cfg)

    import torch
    import torch.distributed as dist
    from treebeard_b200 import kernels

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    forest, marg, n_rows = synth.make_config(args.workload, trees=args.trees, rows=args.rows)
    rep = args.representation
    tree_sharded = world > 1 and args.shard == "trees"
    my_forest = forest
    if tree_sharded:
        T = forest.num_trees
        my_forest = forest.tree_slice(rank * T // world, (rank + 1) * T // world)
    df = kernels.DeviceForest(my_forest, device=local_rank, batch_hint=n_rows, representation=rep,
                              tile_size=args.tile_size, rows_per_block=args.rows_per_block,
                              rows_per_thread=args.rows_per_thread, tree_threads=args.tree_threads,
                              tree_chunks=args.tree_chunks, cache_trees=args.cache_trees)

    # seeded synthetic rows, generated on the host; a tree-sharded run needs the same rows
    # on every rank, a row-sharded run gives every rank its own batch
    X_host = synth.config_rows(args.workload, marg, n_rows, offset=0 if tree_sharded else rank)
    x_pinned = torch.from_numpy(X_host).pin_memory()
    X = x_pinned.to(dev, non_blocking=False)
    int8 = forest.num_classes > 0
    out = torch.empty(n_rows, device=dev, dtype=torch.int8 if int8 else torch.float32)
    partial = torch.empty((n_rows, max(1, forest.num_classes)), device=dev) if tree_sharded else None
    flush = None
    if n_rows * cfg["F"] * 4 <= (126 << 20):
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        if tree_sharded:
            df.predict_partial(X, out=partial)
            dist.reduce(partial, dst=0, op=dist.ReduceOp.SUM)
            if rank == 0:
                df.finalize(partial, out=out, int8=int8)
        else:
            df.predict(X, out=out, int8=int8)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    df.check_status()
    launches0 = df.launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.25)
    stream = torch.cuda.current_stream()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    t_wall = time.perf_counter()
    for i in range(args.steps):
        if flush is not None:
            flush.fill_(i & 0xFF)
        starts[i].record(stream)
        step()
        ends[i].record(stream)
    barrier()
    t_wall = time.perf_counter() - t_wall
    per_step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    clocks = sampler.stop()
    launches = df.launch_count() - launches0
    df.check_status()

    total_ms = sum(per_step_ms)
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    rows_per_step = n_rows if tree_sharded else n_rows * world
    value = rows_per_step / (ms_per_step * 1e-3)

    # roofline of the walk kernel: algorithmic bytes per launch over its device time
    peak, peak_src = measured_peak()
    kernel_ms = statistics.mean(per_step_ms)
    bpr = bytes_per_row(cfg)
    achieved = n_rows * bpr / (kernel_ms * 1e-3) / 1e9
    per_row = NCU_DRAM_BYTES_PER_ROW.get(args.workload) if not args.trees else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": per_row * n_rows if per_row else None,
                "traffic_source": "ncu dram bytes per row on a reduced batch x rows" if per_row else None,
                "peak_source": f"hbm_gbs of {peak_src}",
                "algorithmic_bytes_per_row": bpr, "kernel_ms": kernel_ms,
                "node_visits_per_s": n_rows * visits_per_row(cfg) / (kernel_ms * 1e-3)}

    # end to end through the host-buffer entry point: pinned host rows in, host results out
    e2e = None
    if not args.no_e2e and not tree_sharded:
        res = torch.empty(n_rows, dtype=torch.int8 if int8 else torch.float32).pin_memory()
        xin, rout = x_pinned.numpy(), res.numpy()
        df.predict_host(xin, rout, int8=int8)
        barrier()
        t0 = time.perf_counter()
        reps = max(2, min(args.steps, 5))
        for _ in range(reps):
            df.predict_host(xin, rout, int8=int8)
        dt = torch.tensor([(time.perf_counter() - t0) / reps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": n_rows * world / float(dt.item()), "unit": "rows/s",
               "h2d_bytes_per_step": n_rows * cfg["F"] * 4,
               "d2h_bytes_per_step": n_rows * (1 if int8 else 4),
               "steps": reps, "ms_per_step": float(dt.item()) * 1e3,
               "via": "tbk_predict_host (chunked H2D / walk / D2H on two streams)"}
        # chunked launches may group trees differently: same leaves, fp32 sums within rounding
        e2e["max_abs_diff_vs_device_path"] = float(np.abs(
            rout[:4096].astype(np.float64) - out[:4096].float().cpu().numpy()).max())

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle
        threads = host_threads()
        base = oracle.CpuBaseline(forest)
        pilot = max(256, threads * 8)
        t0 = time.perf_counter()
        base.predict(X_host[:pilot], threads)
        dt = time.perf_counter() - t0
        sample = int(min(n_rows, max(pilot, pilot * 10.0 / max(dt, 1e-6))))
        t0 = time.perf_counter()
        ref_out = base.predict(X_host[:sample], threads)
        dt = time.perf_counter() - t0
        gpu_out = out[:sample].float().cpu().numpy()
        cpu = {"value": sample / dt, "unit": "rows/s", "cores": threads, "kind": "port",
               "sample": f"first {sample} of {n_rows} rows, one pass, C restatement of the "
                         f"reference's parallel CPU schedule ({threads} OpenMP threads)",
               "max_abs_diff_vs_gpu": float(np.abs(ref_out - gpu_out).max())}

    if rank == 0:
        info = df.info()
        line = {"metric": "rows_per_second", "value": value, "unit": "rows/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong" if tree_sharded else "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(args, cfg, n_rows, world),
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
                "clocks": clocks, "wall_ms_per_step": t_wall * 1e3 / args.steps,
                "schedule": {"rows_per_block": info.schedule.rows_per_block,
                             "rows_per_thread": info.schedule.rows_per_thread,
                             "tree_threads": info.schedule.tree_threads,
                             "tree_chunks": info.schedule.tree_chunks,
                             "staged": info.staged, "smem_bytes": info.smem_bytes,
                             "threads": info.threads_per_block, "packed_bytes": info.packed_bytes}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
