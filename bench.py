#!/usr/bin/env python
"""Benchmark of the boosting hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--rows R]

Workload (N = 1): the binary-classification configuration the headline metric is
quoted on -- 10 M rows x 28 fp32 features (21 ~ N(0,1) plus 7 derived ones), label
~ Bernoulli(sigmoid(w.x + 0.3 * sum of pair products)), hist_size 255, reg:logistic,
max_depth 8, eta 0.1, min_child_weight 1.  The data are seeded synthetic stand-ins
(there is no public data set behind the metric).  One step = one boosting round
(AGrowTree).  For N > 1 the same rows are sharded over one process per GPU (strong
scaling) and every level's histogram is summed with ncclAllReduce.

`value` is rounds/s with the binned matrix resident in HBM; `e2e` is rounds/s of the
whole job through the C ABI from host buffers: DMatrix construction (host->device
copy, quantisation), K rounds, read-back of the training predictions.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FULL_ROWS = 10_000_000
FEATURES = 28
CONFIG = {"objective": 1, "method": 1,
          "internals": {"double_precision": False, "compute_overlap": 2, "seed": 0,
                        "use_hist_subtraction_trick": True, "upload_features": True,
                        "hist_size": 255},
          "verbose": {"gpu": False, "booster": False, "data": False},
          "tree": {"eta": 0.1, "max_depth": 8, "min_child_weight": 1.0, "min_leaf_size": 1,
                   "lambda": 1.0, "alpha": 0.0, "colsample_bytree": 1.0, "colsample_bylevel": 1.0}}
# DRAM bytes moved per algorithmic byte by the launches the roofline times (the histogram
# kernel's), over one boosting round of this very workload in the ncu capture named below:
# 2326 MB moved for 34.6 M scanned rows x 36 B (with the reduction of the kernel's planes:
# 2689 MB, 2.16).
HIST_TRAFFIC_RATIO = 1.87
HIST_TRAFFIC_SOURCE = ("profiles/level_kernels_bench10M.md: ncu SpeedOfLight + MemoryWorkloadAnalysis of the 57 "
                       "launches of one round of this workload (10 M x 28); dram__bytes.sum.per_second x "
                       "gpu__time_duration.sum of the 8 hist_u8_kernel launches / (rows scanned x 36 B); a "
                       "ratio, applied to this run's algorithmic bytes per launch")


def make_rows(n, seed):
    """Rows of the 10M x 28 logistic configuration; weights are fixed by seed 2."""
    wrng = np.random.default_rng(2)
    w = wrng.normal(size=FEATURES).astype(np.float32)
    rng = np.random.default_rng([2, seed])
    X = np.empty((n, FEATURES), dtype=np.float32)
    X[:, :21] = rng.standard_normal((n, 21), dtype=np.float32)
    X[:, 21] = X[:, 0] * X[:, 1]
    X[:, 22] = X[:, 2] * X[:, 3]
    X[:, 23] = X[:, 4] * X[:, 5]
    X[:, 24] = X[:, 6] * X[:, 7]
    X[:, 25] = np.abs(X[:, 8] - X[:, 9])
    X[:, 26] = np.abs(X[:, 10] + X[:, 11])
    X[:, 27] = np.abs(X[:, 12] * X[:, 13])
    logit = X @ w
    for j in range(7):
        logit += 0.3 * X[:, 2 * j] * X[:, 2 * j + 1]
    y = (rng.random(n, dtype=np.float32) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
    return X, y


def _cfg(objective, max_depth, eta, **kw):
    c = json.loads(json.dumps(CONFIG))
    c["objective"] = objective
    c["tree"]["max_depth"] = max_depth
    c["tree"]["eta"] = eta
    for k, v in kw.items():
        (c["internals"] if k in ("chunk_rows", "resident_chunks") else c["tree"])[k] = v
    return c


def make_c1(n, seed):  # small regression: y = w.x + 0.5 x0 x1 + N(0, 0.1)
    rng = np.random.default_rng([1, seed])
    X = rng.standard_normal((n, 28), dtype=np.float32)
    w = np.random.default_rng(1).normal(size=28).astype(np.float32)
    y = X @ w + 0.5 * X[:, 0] * X[:, 1] + rng.normal(0, 0.1, n).astype(np.float32)
    return X, y.astype(np.float32), None


_C3_CACHE = {}


def _c3(n, seed):
    """Wide table: 1990 log-normal columns with 20 % of the cells missing and 10 categorical
    columns (cardinality 50 .. 1000, Zipf-distributed codes); the target is the sum of 30
    column effects plus noise."""
    key = (n, seed)
    if key in _C3_CACHE:
        return _C3_CACHE[key]
    rng = np.random.default_rng([3, seed])
    F, n_cat = 2000, 10
    Fd = F - n_cat
    prm = np.random.default_rng(3)
    cols = prm.choice(F, 30, replace=False)
    coef = prm.normal(size=30).astype(np.float32)
    cards = prm.integers(50, 1001, size=n_cat)
    offsets = [prm.normal(size=int(c)).astype(np.float32) for c in cards]
    X = np.empty((n, Fd), dtype=np.float32)
    y = rng.normal(0, 0.5, n).astype(np.float32)
    for lo in range(0, Fd, 100):  # column blocks keep the temporaries small
        w = min(100, Fd - lo)
        blk = np.exp(rng.standard_normal((n, w), dtype=np.float32))
        for k, c in enumerate(cols):
            if lo <= c < lo + w:
                y += coef[k] * np.log1p(blk[:, c - lo])
        blk[rng.random((n, w), dtype=np.float32) < 0.2] = np.nan
        X[:, lo:lo + w] = blk
    cat = np.empty((n, n_cat), dtype=np.uint32)
    for j in range(n_cat):
        cat[:, j] = np.minimum(rng.zipf(1.2, n), cards[j]) - 1
        for k, c in enumerate(cols):
            if c == Fd + j:
                y += offsets[j][cat[:, j]]
    _C3_CACHE.clear()
    _C3_CACHE[key] = (X, cat, y.astype(np.float32))
    return _C3_CACHE[key]


def make_c3(n, seed):
    X, _, y = _c3(n, seed)
    return X, y, None


def make_c3_categories(n, seed):
    return _c3(n, seed)[1]


# workloads whose rows come with categorical columns: name -> generator of the codes
CATEGORIES = {"c3": make_c3_categories}


def make_c4(n, seed):  # 10 classes by argmax of random projections plus Gumbel noise
    rng = np.random.default_rng([4, seed])
    X = rng.standard_normal((n, 50), dtype=np.float32)
    W = np.random.default_rng(4).normal(size=(50, 10)).astype(np.float32)
    labels = np.argmax(X @ W + rng.gumbel(size=(n, 10)).astype(np.float32), axis=1).astype(np.uint8)
    return X, None, labels


def make_c5(n, seed):  # pre-binned uint8, uniform bins, logistic label from 10 active features
    rng = np.random.default_rng([5, seed])
    bins = rng.integers(0, 255, size=(n, 100), dtype=np.uint8)
    prm = np.random.default_rng(5)
    active = prm.choice(100, 10, replace=False)
    c = prm.normal(0, 2, 10).astype(np.float32)
    logit = ((bins[:, active].astype(np.float32) / 255.0 - 0.5) * c).sum(axis=1)
    y = (rng.random(n, dtype=np.float32) < 1.0 / (1.0 + np.exp(-logit))).astype(np.float32)
    return bins, y, None


def make_c2(n, seed):
    X, y = make_rows(n, seed)
    return X, y, None


# name -> (default rows, features, generator, configuration, description); the bench
# line of the driver is c2; the others are the remaining configurations at full size
WORKLOADS = {
    "c1": (100_000, 28, make_c1, _cfg(0, 6, 0.1),
           "regression %d x 28 fp32, reg:linear, max_depth 6, eta 0.1 (configs[0])"),
    "c2": (FULL_ROWS, FEATURES, make_c2, CONFIG,
           "binary classification %d x 28 fp32, hist_size 255, reg:logistic, max_depth 8, eta 0.1 "
           "(configs[1])"),
    "c3": (1_000_000, 2000, make_c3, _cfg(0, 6, 0.1, colsample_bytree=0.5),
           "wide table %d x (1990 fp32 with 20%% NaN + 10 categorical), colsample_bytree 0.5, "
           "max_depth 6 (configs[2])"),
    "c4": (5_000_000, 50, make_c4, _cfg(3, 6, 0.2, labels_count=10),
           "multi:softmax %d x 50 fp32, 10 classes, max_depth 6, eta 0.2 (configs[3])"),
    "c5": (50_000_000, 100, make_c5, _cfg(1, 8, 0.1),
           "pre-binned uint8 %d x 100, reg:logistic, max_depth 8, in HBM (configs[4] shape)"),
    "c5a": (50_000_000, 100, make_c5, _cfg(1, 8, 0.1, chunk_rows=8_000_000, resident_chunks=0),
            "pre-binned uint8 %d x 100, reg:logistic, max_depth 8, every chunk streamed from pinned "
            "host memory (configs[4] mode a)"),
}


# boosting rounds of a whole job as the configurations state them (BASELINE.json)
JOB_ROUNDS = {"c1": 100, "c2": 500, "c3": 200, "c4": 100, "c5": 100, "c5a": 100}


class ClockSampler(object):
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
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
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(smax)) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "span": "every 50 ms from the end-to-end jobs through the timed and the profiled rounds"}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def _pin_host_threads():
    """All host cores for the CPU port, whatever the launcher put in the environment
    (torchrun sets OMP_NUM_THREADS=1 for its workers); to be called before the oracle's
    library is loaded."""
    cores = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(cores)
    return cores


def oracle_rounds_per_s(rows, rounds, warmup, workload="c2"):
    """The CPU port of the path on `rows` rows of the workload: rounds/s."""
    from oracle import oracle as orc
    _, features, gen, cfg, _ = WORKLOADS[workload]
    X, y, labels = gen(rows, 1000)
    cat = CATEGORIES[workload](rows, 1000) if workload in CATEGORIES else None
    o = orc.Oracle(cfg, missing_bin=True)
    if X.dtype == np.uint8:
        thr = np.tile(np.arange(255, dtype=np.float32) + 0.5, (features, 1))
        o.set_binned(np.ascontiguousarray(X.T).astype(np.uint16), thr, np.full(features, 255, dtype=np.int32))
    else:
        o.set_dense(X, categories=cat)
    if labels is not None:
        o.set_label(labels)
    else:
        o.set_y(y)
    o.grow(warmup)
    t0 = time.perf_counter()
    o.grow(rounds)
    return rounds / (time.perf_counter() - t0)


# rows the CPU port is timed on in the reference arm, per workload: everything for the
# headline configuration; the wider or longer ones are cut so that the arm ends in minutes
REFERENCE_ARM_ROWS = {"c1": 100_000, "c2": FULL_ROWS, "c3": 100_000, "c4": 1_000_000, "c5": 5_000_000,
                      "c5a": 5_000_000}


def run_reference(args, rank, world):
    """Reference arm.  arboretum has no CPU training path, so this times the CPU port of its
    algorithm (oracle/) with all host threads -- on all rows of the headline workload; the
    reference's own CUDA build is timed by the other arm's `ref_cuda` record."""
    if rank != 0:
        return
    cores = _pin_host_threads()
    rows = min(args.rows, REFERENCE_ARM_ROWS[args.workload])
    value = oracle_rounds_per_s(rows, max(1, args.steps), max(0, args.warmup), args.workload)
    cfg = workload_config(args, world)
    cfg["rows"] = rows  # what was timed, nothing scaled
    cfg["rows_per_gpu"] = None
    cfg["parallelism"] = "host threads x%d" % cores
    cfg["workload"] = WORKLOADS[args.workload][4] % rows
    line = {"impl": "reference", "metric": "boosting_rounds_per_sec", "value": value,
            "unit": "rounds/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": "rounds/s", "cores": cores, "kind": "port",
                             "sample": "all %d rows, %d rounds timed after %d (nothing scaled)"
                                       % (rows, args.steps, args.warmup)},
            "e2e": {"value": value, "unit": "rounds/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def reference_cuda_record(workload, rows):
    """The reference's own CUDA build (oracle/_ref, compiled from its sources by
    oracle/build_ref_cuda.py) on the same seeded rows, in a child process: rounds/s of
    `for round: AGrowTree` on this GPU."""
    from oracle import ref_cuda
    if not ref_cuda.available():
        return {"unavailable": "oracle/_ref/libarboretum_ref.so is not built"}
    if workload not in ("c1", "c2"):
        return {"unavailable": "the reference trains dense fp32 with reg:linear / reg:logistic only"}
    cmd = [sys.executable, os.path.join(ROOT, "oracle", "ref_cuda.py"), "time", "--workload", workload,
           "--rows", str(rows), "--rounds", "10", "--warmup", "2", "--double", "0"]
    try:
        out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
        rec = json.loads(out.stdout.strip().splitlines()[-1])
    except Exception as e:  # a reference that misbehaves must not take the bench line with it
        return {"unavailable": "the reference run failed: %r" % (e,)}
    return {"value": rec["value"], "unit": rec["unit"], "config": rec["workload"],
            "ms_per_round": rec["ms_per_round"], "double_precision": rec["double_precision"],
            "first_round_with_quantisation_s": rec["first_round_with_quantisation_s"], "how": rec["how"]}


def run_c5b(rows_per_gpu, steps, warmup, rank, world, local_rank, base_cfg):
    """The out-of-core-scale configuration's sharded mode: rows pre-binned to uint8 x 100
    features, `rows_per_gpu` of them generated ON every GPU (never on the host), a logistic
    label from 10 active features, max_depth 8; rows sharded over the ranks with the
    per-level histogram exchange.  Weak scaling: the per-GPU work is fixed, so rounds/s at N
    GPUs against rounds/s at 1 GPU is the scaling of the row throughput.  Returns the
    sub-record of the bench line (rank 0) or None."""
    import torch
    import torch.distributed as dist
    import arboretum_b200 as arboretum
    from arboretum_b200 import distributed as adist
    F = 100
    dev = torch.device("cuda", local_rank)
    ok = torch.ones(1, device=dev)
    model = None
    try:
        gen = torch.Generator(device=dev)
        gen.manual_seed(5000 + rank)
        bins = torch.randint(0, 255, (rows_per_gpu, F), dtype=torch.uint8, device=dev, generator=gen)
        prm = np.random.default_rng(5)
        active = torch.as_tensor(prm.choice(F, 10, replace=False), device=dev)
        coef = torch.as_tensor(prm.normal(0, 2, 10).astype(np.float32), device=dev)
        logit = torch.zeros(rows_per_gpu, device=dev)
        for j in range(10):  # column by column: no rows x 10 float temporary
            logit += (bins[:, active[j]].float() / 255.0 - 0.5) * coef[j]
        y = (torch.rand(rows_per_gpu, device=dev, generator=gen) < torch.sigmoid(logit)).float()
        del logit
        torch.cuda.synchronize()
        data = arboretum.DMatrix.from_device_bins(bins.data_ptr(), rows_per_gpu, F, 255, y.data_ptr())
        del bins, y
        torch.cuda.empty_cache()
        cfg = json.loads(json.dumps(base_cfg))
        cfg["internals"]["device"] = local_rank
        model = arboretum.Garden(cfg)
        model.data = data
        if world > 1:
            adist.init_nccl(model, rank, world)
    except Exception as e:  # e.g. not enough memory for this many rows
        ok.zero_()
        err = repr(e)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if ok.item() == 0:  # every rank leaves together, before any exchange
        return {"unavailable": "set-up failed on a rank" + (": " + err if "err" in dir() else "")} if rank == 0 else None
    for _ in range(max(1, warmup)):
        model.grow_tree()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        model.grow_tree()
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([ev0.elapsed_time(ev1) / 1000.0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_s = float(t.item()) / steps
    model.set_profile(True)
    model.grow_tree()
    tm = model.timings()
    del model, data
    if rank != 0:
        return None
    return {"workload": "pre-binned uint8 %d rows per GPU x 100 features, reg:logistic, max_depth 8, rows sharded "
                        "over the GPUs (configs[4] mode b), generated on the devices" % rows_per_gpu,
            "rows_per_gpu": rows_per_gpu, "rows_total": rows_per_gpu * world, "n_gpus": world,
            "scaling": "weak", "value": 1.0 / step_s, "unit": "rounds/s", "ms_per_step": 1000.0 * step_s,
            "steps": steps, "warmup": max(1, warmup),
            "rows_x_features_per_s": rows_per_gpu * world * F / step_s,
            "hist_rows_x_features_per_s_per_gpu": tm["hist_rows"] * F / (tm["hist_ms"] * 1e-3) if tm["hist_ms"] > 0 else None,
            "hist_frac_of_hbm_peak": (tm["hist_bytes"] / (tm["hist_ms"] * 1e-3) / 1e9 / measured_peak()[0]) if tm["hist_ms"] > 0 else None,
            "level_exchange": tm.get("level_exchange"),
            "phase_ms_per_round": {k: tm[k] for k in ("grad_ms", "partition_ms", "plan_ms", "hist_ms", "allreduce_ms",
                                                      "subtract_ms", "split_ms", "update_ms")}}


def shared_atomics(t, features):
    """The histogram pass against the ceiling of its inner loop: (g, h) pair updates per
    second of the two shared-memory reductions alone, measured by the library on this GPU
    (every scanned row updates one pair per feature slot, 32 slots per tile of features)."""
    from arboretum_b200 import core
    peak = core.shared_atomic_peak(2000)
    # the columns the histograms cover (the sampled ones when a tree samples its columns)
    cols = int(round(t["hist_row_features"] / max(1, t["hist_launches"]))) if t.get("hist_row_features") else features
    slots = (cols + 31) // 32 * 32
    achieved = t["hist_rows"] * slots / ((t.get("hist_kernel_ms") or t["hist_ms"]) * 1e-3)
    return {"achieved": achieved, "peak": peak, "frac": achieved / peak, "unit": "(g, h) updates/s",
            "note": "histogram kernel time of all levels; feature slots padded to 32 per tile"}


def workload_config(args, world):
    _, features, _, cfg, desc = WORKLOADS[args.workload]
    pitch = (features + 31) // 32 * 32
    return {"workload": desc % args.rows, "rows": args.rows, "features": features,
            "max_depth": cfg["tree"]["max_depth"],
            "rows_per_gpu": args.rows // world, "parallelism": "rows sharded x%d" % world,
            "l2": "inputs (bins %.0f MB + gradients %.0f MB per GPU) exceed the 126 MB L2"
                  % (args.rows // world * pitch / 1e6, args.rows // world * 8 / 1e6)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--rows", type=int, default=0)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true",
                    help="skip the run of the reference's own CUDA build (the `ref_cuda` record)")
    ap.add_argument("--no-full-job", action="store_true",
                    help="skip the one job with the configuration's full number of rounds")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the end-to-end jobs (profiling runs: fewer launches before the timed rounds)")
    ap.add_argument("--internals", default="", help='JSON merged into the "internals" configuration')
    ap.add_argument("--predict-rows", type=int, default=0,
                    help="also time inference (APredict) of the trained model on this many of the rows")
    ap.add_argument("--c5b-rows-per-gpu", type=int, default=250_000_000,
                    help="rows per GPU of the sharded out-of-core-scale sub-record (0: skip it)")
    args = ap.parse_args()
    if args.rows <= 0:
        args.rows = WORKLOADS[args.workload][0]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import arboretum_b200 as arboretum
    from arboretum_b200 import distributed as adist

    args.warmup = max(args.warmup, 3)
    n_local = args.rows // world
    _, features, gen, base_cfg, _ = WORKLOADS[args.workload]
    X, y, labels = gen(n_local, rank)
    cat = CATEGORIES[args.workload](n_local, rank) if args.workload in CATEGORIES else None
    binned = X.dtype == np.uint8
    xp = torch.from_numpy(X).pin_memory()  # the job's host buffers are pinned
    Xh = xp.numpy()
    target = labels if labels is not None else y
    yp = torch.from_numpy(target).pin_memory()
    yh = yp.numpy()
    cfg = json.loads(json.dumps(base_cfg))
    cfg["internals"]["device"] = local_rank
    if args.internals:
        cfg["internals"].update(json.loads(args.internals))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def new_model():
        kw = {"binned_hist_size": 255} if binned else {}
        if cat is not None:
            kw["data_category"] = cat
        if labels is not None:
            data = arboretum.DMatrix(Xh, labels=yh, **kw)
        else:
            data = arboretum.DMatrix(Xh, y=yh, **kw)
        model = arboretum.Garden(cfg)
        model.data = data
        model.labels_count = data.labels_count
        if world > 1:  # the ranks then quantise their shards together, at the first round
            adist.init_nccl(model, rank, world)
        return model, data

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- end to end: host buffers -> model -> predictions on the host --------------
    # A small job first, so that the timed runs do not pay for loading the kernels and for
    # the allocator's first calls; then the whole job five times, the median is reported.
    warm_rows = min(n_local, 200_000)
    Xw, yw, lw = gen(warm_rows, 10_000 + rank)
    kw = {"binned_hist_size": 255} if binned else {}
    if cat is not None:
        kw["data_category"] = CATEGORIES[args.workload](warm_rows, 10_000 + rank)
    wd = arboretum.DMatrix(Xw, labels=lw, **kw) if lw is not None else arboretum.DMatrix(Xw, y=yw, **kw)
    wm = arboretum.Garden(cfg)
    wm.data = wd
    wm.labels_count = wd.labels_count
    if world > 1:  # the process's communicator is made here, once; the timed jobs attach it
        adist.init_nccl(wm, rank, world)
    wm.grow_tree()
    wm.train_yhat()
    del wm, wd
    # clocks and throttle reasons are sampled from here to the end of the profiled rounds: the
    # timed region alone (tens of milliseconds) is shorter than the sampler's start-up
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e2e_runs, e2e_parts = [], []
    for _ in range(0 if args.no_e2e else 5):
        model = data = None
        barrier()
        t0 = time.perf_counter()
        model, data = new_model()
        t1 = time.perf_counter()
        model.grow_tree()  # quantises the matrix first
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        for _ in range(args.steps - 1):
            model.grow_tree()
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        yhat = model.train_yhat()
        t4 = time.perf_counter()
        barrier()
        e2e_runs.append(max_over_ranks(time.perf_counter() - t0))
        e2e_parts.append([round(b - a, 4) for a, b in ((t0, t1), (t1, t2), (t2, t3), (t3, t4))])
    if args.no_e2e:
        model, data = new_model()
        model.grow_tree()
        yhat = model.train_yhat()
        e2e_runs = [float("nan")]
    e2e_s = sorted(e2e_runs)[len(e2e_runs) // 2]
    e2e = {"value": None if args.no_e2e else args.steps / e2e_s, "unit": "rounds/s",
           "h2d_bytes_per_step": int((Xh.nbytes + yh.nbytes + (cat.nbytes if cat is not None else 0))
                                     * world / args.steps),
           "d2h_bytes_per_step": int(yhat.nbytes * world / args.steps),
           "runs_s": [] if args.no_e2e else [round(t, 4) for t in e2e_runs],
           "parts_s": {"order": ["DMatrix (host to device)", "quantise + first round", "other rounds",
                                 "predictions to host"],
                       "per_run": e2e_parts},
           "what": "median of %d: DMatrix from pinned host memory + quantise + %d rounds + "
                   "predictions to host; CUDA context, kernel images and (N > 1) the NCCL "
                   "communicator exist before the timed jobs" % (len(e2e_runs), args.steps)}

    # ---- device-resident rounds (the model above is already bound and warm) ---------
    for _ in range(args.warmup):
        model.grow_tree()
    launches0 = model.timings()["kernel_launches"]
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.grow_tree()
    ev1.record()
    barrier()
    wall_s = time.perf_counter() - t0
    step_s = max_over_ranks(ev0.elapsed_time(ev1) / 1000.0)
    launches = model.timings()["kernel_launches"] - launches0

    # ---- roofline of the dominant kernel: CUDA events on the library's own stream ----
    model.set_profile(True)
    prof_rounds = 3
    for _ in range(prof_rounds):
        model.grow_tree()
    t = model.timings()
    model.set_profile(False)
    clocks = sampler.stop() if rank == 0 else None
    peak, peak_src = measured_peak()
    if t["hist_ms"] > 0:
        # the dominant kernel's own launches (one per level), timed by events on the library's
        # stream directly before and behind each; the reduction of its planes is reported beside it
        kernel_ms = t.get("hist_kernel_ms") or t["hist_ms"]
        hist_gbs = t["hist_bytes"] / (kernel_ms * 1e-3) / 1e9
        per_launch_bytes = t["hist_bytes"] / max(1, t["hist_launches"])
        roofline = {"bound": "hbm", "kernel": "hist_u8_kernel", "achieved": hist_gbs, "peak": peak,
                    "unit": "GB/s", "frac": hist_gbs / peak, "peak_source": peak_src,
                    "frac_of_nominal_8TBs": hist_gbs / 8000.0,
                    "with_plane_reduction": {"achieved": t["hist_bytes"] / (t["hist_ms"] * 1e-3) / 1e9,
                                             "frac": t["hist_bytes"] / (t["hist_ms"] * 1e-3) / 1e9 / peak,
                                             "what": "the same bytes over histogram + reduce_kernel time"},
                    "traffic": None if HIST_TRAFFIC_RATIO is None or args.workload != "c2"
                    else per_launch_bytes * HIST_TRAFFIC_RATIO,
                    "traffic_source": HIST_TRAFFIC_SOURCE if args.workload == "c2" else None,
                    "algorithmic_bytes_per_launch": per_launch_bytes,
                    "avg_launch_ms": kernel_ms / max(1, t["hist_launches"]),
                    "rows_x_features_per_s_per_gpu": t["hist_rows"] * features / (kernel_ms * 1e-3),
                    "smem_atomic_updates_per_s": 2.0 * t["hist_rows"] * features / (kernel_ms * 1e-3),
                    "tree_ms": t["tree_ms"] / max(1, t["trees"]),
                    "shared_atomics": shared_atomics(t, features),
                    "phase_ms_per_round": {k: t[k] / prof_rounds for k in
                                           ("grad_ms", "partition_ms", "plan_ms", "hist_ms", "allreduce_ms",
                                            "subtract_ms", "split_ms", "update_ms")}}
        roofline["phase_ms_per_round"]["hist_kernel_ms"] = (t.get("hist_kernel_ms") or 0.0) / prof_rounds
    else:
        # row chunks streamed from the host: the level loop is bound by the host link, and
        # the phases of the chunks interleave, so only the whole tree is timed
        link_gbs = t["h2d_bytes"] / (t["tree_ms"] * 1e-3) / 1e9
        roofline = {"bound": "host link", "kernel": "chunk copies + hist_u8_kernel", "achieved": link_gbs,
                    "peak": None, "unit": "GB/s", "frac": None, "traffic": None,
                    "h2d_bytes_per_round": t["h2d_bytes"] / prof_rounds,
                    "tree_ms": t["tree_ms"] / max(1, t["trees"]),
                    "rows_streamed_per_s": t["h2d_bytes"] / ((features + 31) // 32 * 32) / (t["tree_ms"] * 1e-3)}

    # ---- inference on the device (RegTree::Predict of the reference runs on the host) ---------
    predict = None
    if args.predict_rows > 0 and not binned:
        kw_p = {"data_category": cat[:args.predict_rows]} if cat is not None else {}
        pd = arboretum.DMatrix(np.ascontiguousarray(Xh[:args.predict_rows]), **kw_p)
        model.predict(pd)  # uploads the forest
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model.predict(pd)
        dt = time.perf_counter() - t0
        trees = len(json.loads(model.dump())["model"])
        predict = {"rows": int(pd.rows), "trees": trees, "seconds": dt, "rows_x_trees_per_s": pd.rows * trees / dt,
                   "what": "APredict on a resident matrix: tree walk over raw fp32 rows, link function, "
                           "result copied to the host"}
        del pd, out

    # one whole job as the configuration states it (all its boosting rounds), timed the same
    # way, when the jobs above say that it ends within a quarter of a minute
    full_job = None
    if not args.no_e2e and not args.no_full_job:
        rounds = JOB_ROUNDS[args.workload]
        # the same figure on every rank, so that all of them take the same decision
        per_round = max_over_ranks(sorted(p[2] for p in e2e_parts)[len(e2e_parts) // 2] / max(1, args.steps - 1))
        if 3 * rounds * per_round < 30.0:
            jobs = []
            for _ in range(3):
                barrier()
                t0 = time.perf_counter()
                job_model, job_data = new_model()
                for _ in range(rounds):
                    job_model.grow_tree()
                job_model.train_yhat()
                barrier()
                jobs.append(max_over_ranks(time.perf_counter() - t0))
                del job_model, job_data
            job_s = sorted(jobs)[1]
            full_job = {"rounds": rounds, "seconds": job_s, "value": rounds / job_s, "unit": "rounds/s",
                        "runs_s": [round(t, 4) for t in jobs],
                        "what": "median of 3 jobs with the configuration's own number of boosting rounds, "
                                "host buffers to predictions on the host"}
    e2e["full_job"] = full_job

    # ---- the 2 B-row configuration's sharded mode, per-GPU share fixed (weak scaling) ------
    c5b = None
    if args.c5b_rows_per_gpu > 0 and args.workload == "c2":
        del model, data, yhat, xp, Xh, X
        arboretum.release_cached_memory()
        torch.cuda.empty_cache()
        c5b = run_c5b(args.c5b_rows_per_gpu, 5, 2, rank, world, local_rank, WORKLOADS["c5"][3])

    if rank == 0:
        line = {"metric": "boosting_rounds_per_sec", "value": args.steps / step_s, "unit": "rounds/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": 1000.0 * step_s / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "int64 fixed-point sums of f32 gradients",
                "data": "synthetic", "config": workload_config(args, world), "clocks": clocks,
                "e2e": e2e, "gpu_launches": int(launches), "wall_ms_per_step": 1000.0 * wall_s / args.steps,
                "level_exchange": t.get("level_exchange"),
                "exchange_ms_per_round": None if "exchanges" not in t else {
                    "waiting for the peers' buffers": t["exchange_wait_peers_ms"] / prof_rounds,
                    "summing and storing this rank's slice": t["exchange_move_ms"] / prof_rounds,
                    "waiting for the peers' slices": t["exchange_wait_done_ms"] / prof_rounds,
                    "exchanges": t["exchanges"] / prof_rounds},
                "roofline": roofline}
        if c5b is not None:
            line["c5b"] = c5b
        if predict is not None:
            line["predict"] = predict
        if world == 1 and not args.no_ref_cuda:
            line["ref_cuda"] = reference_cuda_record(args.workload, args.rows)
        if world == 1 and not args.no_cpu_baseline:
            sample = min(args.rows, max(20_000, 14_000_000 // features))
            cores = os.cpu_count() or 1
            rps = oracle_rounds_per_s(sample, 2, 1, args.workload) * sample / args.rows
            line["cpu_baseline"] = {"value": rps, "unit": "rounds/s", "cores": cores, "kind": "port",
                                    "sample": "%d of %d rows, 2 rounds timed after 1, rounds/s scaled "
                                              "by rows" % (sample, args.rows)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
