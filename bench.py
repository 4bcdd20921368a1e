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
# proportion to the rows, so a launch's traffic is this figure times its rows.  Each figure
# belongs to the kernel sources it was captured on: it is reported only while the hash of the
# code of the headers that make up the workload's kernel (kernel_source_hash) still matches.
KERNEL_SOURCES = {"c3": ("walk_kernels.cuh", "walk_quant.cuh"),
                  "c2": ("walk_kernels.cuh", "walk_quant.cuh", "walk_quant_batch.cuh"),
                  "c4": ("walk_kernels.cuh", "walk_quant.cuh", "walk_quant_batch.cuh")}
NCU_DRAM_BYTES_PER_ROW = {"c3": (8718.9, "9818290bfb5d6a18"), "c2": (131.6, "e10befea55613438"), "c4": (106.9, "e10befea55613438")}


def kernel_source_hash(workload):
    """Hash of the CODE of the workload's kernel headers: comments and blank space do not
    count, so that an edit of a comment does not disown an ncu figure."""
    import hashlib
    import re
    h = hashlib.sha256()
    for name in KERNEL_SOURCES.get(workload, ()):
        with open(os.path.join(ROOT, "treebeard_b200", "csrc", name), "r", encoding="utf-8") as fh:
            for line in fh:
                code = re.sub(r"\s+", " ", line.split("//", 1)[0]).strip()
                if code:
                    h.update(code.encode() + b"\n")
    return h.hexdigest()[:16]


def ncu_traffic(workload, n_rows, custom):
    """(bytes per launch or None, where the figure comes from / why there is none)."""
    if custom or workload not in NCU_DRAM_BYTES_PER_ROW:
        return None, "no ncu capture for this workload"
    per_row, captured_on = NCU_DRAM_BYTES_PER_ROW[workload]
    now = kernel_source_hash(workload)
    if captured_on != now:
        return None, f"kernel sources changed since the ncu capture (captured on {captured_on or 'an earlier build'}, now {now})"
    return per_row * n_rows, "ncu dram bytes per row on a reduced batch x rows (profiles/)"


def bytes_per_row(cfg):
    """Algorithmic HBM bytes per predicted row: features in + prediction out."""
    return 4 * cfg["F"] + (1 if cfg["classes"] > 0 else 4)


def visits_per_row(cfg):
    """Node visits of the fixed-depth walk: trees x decision levels."""
    return cfg["T"] * cfg["D"]


def useful_visits_per_row(forest, leaf_ids):
    """Node visits a walk that stops at its leaf needs: the depth of the selected leaf, summed
    over trees, averaged over the sampled rows (leaf_ids: [rows, trees] node ids from the
    GPU's leaf-id pass)."""
    depth = synth.node_depths(forest)
    glob = leaf_ids.astype(np.int64) + forest.tree_off[:-1][None, :]
    return float(depth[glob].sum(axis=1).mean())


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


def tree_sharded_c5(args, torch, dist, kernels, rank, world, dev):
    """The large forest (T=16 000, D=12, F=128) over all 4 194 304 rows with its trees
    partitioned evenly across the ranks: every rank walks its trees over ALL rows into per-row
    partial sums, one NCCL reduce (fp32, 16 MiB per rank, onto rank 0) adds them, rank 0 adds
    the initial value.  Beside it the row-sharded run of the same forest (every rank the whole
    forest and 1/world of the rows, no collective).  Device times, max over ranks."""
    steps, warmup = 5, 3
    forest, marg, n_rows = synth.make_config("c5", trees=args.c5_trees, rows=args.c5_rows)
    X = torch.from_numpy(synth.config_rows("c5", marg, n_rows)).to(dev)
    T = forest.num_trees
    mine = forest.tree_slice(rank * T // world, (rank + 1) * T // world)
    df = kernels.DeviceForest(mine, device=dev.index, batch_hint=n_rows, representation="auto")
    partial = torch.empty((n_rows, 1), device=dev)
    out = torch.empty(n_rows, device=dev)
    stream = torch.cuda.current_stream()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, marks):
        for _ in range(warmup):
            fn(None)
        sync()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(marks)] for _ in range(steps)]
        for i in range(steps):
            fn(ev[i])
        sync()
        spans = np.array([[ev[i][j].elapsed_time(ev[i][j + 1]) for j in range(marks - 1)] for i in range(steps)])
        t = torch.tensor(spans.mean(axis=0).tolist() + [spans.sum(axis=1).mean()], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def tree_step(ev):
        if ev: ev[0].record(stream)
        df.predict_partial(X, out=partial)
        if ev: ev[1].record(stream)
        if world > 1:
            dist.reduce(partial, dst=0, op=dist.ReduceOp.SUM)
        if ev: ev[2].record(stream)
        if rank == 0:
            df.finalize(partial, out=out)
        if ev: ev[3].record(stream)

    walk_ms, reduce_ms, finalize_ms, total_ms = timed(tree_step, 4)
    df.check_status()
    res = {"workload": f"c5: {synth.CONFIGS['c5']['desc']}, {n_rows} rows, {T} trees over {world} GPU(s)",
           "ms_per_step": total_ms, "rows_per_s": n_rows / (total_ms * 1e-3), "walk_ms": walk_ms,
           "reduce_ms": reduce_ms, "finalize_ms": finalize_ms, "steps": steps, "warmup": warmup,
           "collective": (f"ncclReduce fp32 {n_rows * 4 / 2**20:.0f} MiB -> rank 0" if world > 1 else "none (one GPU)"),
           "row_sharded_ms": None}
    if world > 1:
        del df
        full = kernels.DeviceForest(forest, device=dev.index, batch_hint=n_rows // world, representation="auto")
        lo, hi = rank * n_rows // world, (rank + 1) * n_rows // world
        # rank 0 holds the tree-sharded predictions (the sum of every rank's partial sums): its
        # own row range, recomputed below with the whole forest on one GPU, must agree
        tree_pred = out[lo:hi].clone() if rank == 0 else None
        Xs, outs = X[lo:hi], out[lo:hi]

        def row_step(ev):
            if ev: ev[0].record(stream)
            full.predict(Xs, out=outs)
            if ev: ev[1].record(stream)

        res["row_sharded_ms"] = timed(row_step, 2)[-1]
        full.check_status()
        if rank == 0:
            diff = (outs - tree_pred).abs()
            tol = 1e-6 + 1e-5 * outs.abs()
            res["tree_vs_row_sharded"] = {"rows_compared": int(hi - lo), "max_abs_diff": float(diff.max()),
                                          "within_tolerance": bool((diff <= tol).all())}
    return res


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
    ap.add_argument("--no-c5", action="store_true", help="skip the tree-sharded large-forest section")
    ap.add_argument("--c5-trees", type=int, default=None)
    ap.add_argument("--c5-rows", type=int, default=None)
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

    # roofline of the walk kernel on ONE GPU (this rank's launch): algorithmic bytes per launch
    # over its device time
    peak, peak_src = measured_peak()
    kernel_ms = statistics.mean(per_step_ms)
    bpr = bytes_per_row(cfg)
    achieved = n_rows * bpr / (kernel_ms * 1e-3) / 1e9
    traffic, traffic_src = ncu_traffic(args.workload, n_rows, bool(args.trees) or tree_sharded)
    sample = min(n_rows, 2048)
    useful = useful_visits_per_row(my_forest, df.predict_leaf_ids(X[:sample]).cpu().numpy())
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src,
                "peak_source": f"hbm_gbs of {peak_src}", "per": "GPU",
                "algorithmic_bytes_per_row": bpr, "kernel_ms": kernel_ms,
                "node_visits_per_s": n_rows * my_forest.num_trees * cfg["D"] / (kernel_ms * 1e-3),
                "useful_node_visits_per_s": n_rows * useful / (kernel_ms * 1e-3),
                "useful_visits_per_row": useful}

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

    info = df.info()
    c5 = None
    if not args.no_c5 and args.workload == "c3" and not args.trees and not args.rows and not tree_sharded:
        del df, X, out
        torch.cuda.empty_cache()
        c5 = tree_sharded_c5(args, torch, dist, kernels, rank, world, dev)

    if rank == 0:
        line = {"metric": "rows_per_second", "value": value, "unit": "rows/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong" if tree_sharded else "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(args, cfg, n_rows, world),
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "tree_sharded": c5,
                "gpu_launches": launches,
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
