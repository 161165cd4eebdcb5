"""Worker of tests/test_gpu_multi.py: one process per GPU (torchrun).  Trains the same
data sharded over all ranks and, on rank 0, unsharded on one GPU; the trees must be
bit-identical because every histogram is an exact integer sum."""
import json
import os
import sys
import zlib

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import arboretum_b200 as arboretum  # noqa: E402
from arboretum_b200 import distributed as adist  # noqa: E402


def run_sharded_quantizer_case(rank, world, local):
    """No thresholds are handed in: the ranks quantise their shards together, and both the
    thresholds and the trees must equal those of the unsharded matrix on one GPU."""
    rng = np.random.default_rng(321)
    n, F, rounds = 50001, 37, 3  # shards of unequal length, two column blocks
    X = rng.normal(size=(n, F)).astype(np.float32)
    X[:, 5] = np.round(X[:, 5] * 3)          # few distinct values
    X[rng.random(n) < 0.1, 7] = np.nan       # missing values
    y = (X[:, 0] + 0.5 * X[:, 1] * X[:, 2] + rng.normal(0, 0.1, n)).astype(np.float32)
    cfg = {"objective": 0, "method": 1,
           "internals": {"hist_size": 255, "seed": 0, "device": local},
           "verbose": {"gpu": False, "booster": False, "data": False},
           "tree": {"eta": 0.1, "max_depth": 5, "lambda": 1.0, "min_child_weight": 1.0}}
    lo, hi = adist.shard_rows(n, rank, world)
    data = arboretum.DMatrix(X[lo:hi], y=y[lo:hi])
    model = arboretum.Garden(cfg)
    model.data = data
    adist.init_nccl(model, rank, world)
    for _ in range(rounds):
        model.grow_tree()
    sharded = json.loads(model.dump())["model"]
    thr, size, _ = data.quantize(255, True, want_bins=False)  # what the shards agreed on
    ok = True
    if rank == 0:
        full = arboretum.DMatrix(X, y=y)
        thr1, size1, _ = full.quantize(255, True, want_bins=False)
        single = json.loads(arboretum.train(cfg, full, rounds).dump())["model"]
        ok = bool(np.array_equal(thr.view(np.uint32), thr1.view(np.uint32))) and \
            bool(np.array_equal(size, size1)) and single == sharded
    digest = torch.tensor([zlib.crc32(json.dumps(sharded).encode()) % (2 ** 31)], device="cuda")
    gathered = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    same = all(int(g.item()) == int(digest.item()) for g in gathered)
    return ok, same


def run_case(rank, world, local, objective):
    rng = np.random.default_rng(123)
    n, F, rounds = 60000, 28, 4
    X = rng.normal(size=(n, F)).astype(np.float32)
    w = rng.normal(size=F)
    if objective == 1:
        y = (rng.random(n) < 1 / (1 + np.exp(-(X @ w * 0.5 + 0.3 * X[:, 0] * X[:, 1])))).astype(np.float32)
    else:
        y = (X @ w + rng.normal(0, 0.1, n)).astype(np.float32)
        y[-5:] += 300.0  # the largest |gradient| lives in the last shard only
    cfg = {"objective": objective, "method": 1,
           "internals": {"hist_size": 255, "seed": 0, "device": local},
           "verbose": {"gpu": False, "booster": False, "data": False},
           "tree": {"eta": 0.1, "max_depth": 6, "lambda": 1.0, "min_child_weight": 1.0}}
    # thresholds of the WHOLE matrix, computed on rank 0, shared with everybody
    thr = size = None
    if rank == 0:
        thr, size, _ = arboretum.DMatrix(X).quantize(255, True, want_bins=False)
    lo, hi = adist.shard_rows(n, rank, world)
    data = arboretum.DMatrix(X[lo:hi], y=y[lo:hi])
    thr, size = adist.share_thresholds(data, 255, rank, world, thresholds=thr, sizes=size)
    model = arboretum.Garden(cfg)
    model.data = data
    adist.init_nccl(model, rank, world)
    for _ in range(rounds):
        model.grow_tree()
    sharded = json.loads(model.dump())["model"]
    ok = True
    if rank == 0:
        full = arboretum.DMatrix(X, y=y)
        full.set_thresholds(thr, size)
        single = json.loads(arboretum.train(cfg, full, rounds).dump())["model"]
        ok = single == sharded
    # every rank must hold the same model
    digest = torch.tensor([zlib.crc32(json.dumps(sharded).encode()) % (2 ** 31)], device="cuda")
    gathered = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    same = all(int(g.item()) == int(digest.item()) for g in gathered)
    return ok, same


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ok = same = True
    for objective in (1, 0):
        o, s = run_case(rank, world, local, objective)
        ok, same = ok and o, same and s
    o, s = run_sharded_quantizer_case(rank, world, local)
    if rank == 0 and not o:
        print("SHARDED_QUANTIZER_DIFFERS", flush=True)
    ok, same = ok and o, same and s
    if rank == 0:
        print("MULTI_GPU_TREES_IDENTICAL" if ok else "MULTI_GPU_TREES_DIFFER", flush=True)
        print("MULTI_GPU_RANKS_AGREE" if same else "MULTI_GPU_RANKS_DISAGREE", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if (ok and same) else 1)


if __name__ == "__main__":
    main()
