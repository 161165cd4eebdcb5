"""Host-side logic of the row-sharded multi-GPU path on CPU ranks (gloo, world 2):
the shard arithmetic, the byte broadcast used for thresholds and the ncclUniqueId,
and the property the design rests on -- per-shard fixed-point histograms summed by
an integer all-reduce equal the histogram of all rows, exactly."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_shard_rows_cover_everything_once():
    from arboretum_b200.distributed import shard_rows
    for n in (0, 1, 7, 1000, 10_000_001):
        for world in (1, 2, 3, 8):
            edges = [shard_rows(n, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            for a, b in zip(edges, edges[1:]):
                assert a[1] == b[0]
            sizes = [e[1] - e[0] for e in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import torch
    from arboretum_b200.distributed import _broadcast_bytes, shard_rows
    # 1. byte broadcast (thresholds, communicator id)
    buf = np.arange(128, dtype=np.uint8) if rank == 0 else np.zeros(128, dtype=np.uint8)
    _broadcast_bytes(buf, 0)
    ok = bool((buf == np.arange(128, dtype=np.uint8)).all())
    # 2. sharded fixed-point histogram + integer all-reduce == histogram of all rows
    rng = np.random.default_rng(5)
    n, hist_size, qb = 20000, 64, 17
    bins = rng.integers(0, hist_size, size=n).astype(np.uint16)
    g = rng.normal(size=n).astype(np.float32)
    h = rng.uniform(0.01, 0.25, size=n).astype(np.float32)
    sg = 2.0 ** (qb - np.frexp(np.abs(g).max())[1])
    sh = 2.0 ** (qb - np.frexp(h.max())[1])
    gq = np.rint(g * np.float32(sg)).astype(np.int64)
    hq = np.maximum(1, np.rint(h * np.float32(sh))).astype(np.int64)
    lo, hi = shard_rows(n, rank, world)
    part = np.zeros((2, hist_size), dtype=np.int64)
    np.add.at(part[0], bins[lo:hi], gq[lo:hi])
    np.add.at(part[1], bins[lo:hi], hq[lo:hi])
    t = torch.from_numpy(part)
    dist.all_reduce(t)
    full = np.zeros((2, hist_size), dtype=np.int64)
    np.add.at(full[0], bins, gq)
    np.add.at(full[1], bins, hq)
    ok = ok and bool((t.numpy() == full).all())
    # ... and agrees with the oracle's double sums to the quantisation
    og, oh, oc = orc.hist(bins, g, h, [0, n], hist_size)
    ok = ok and bool(np.allclose(full[0] / sg, og, atol=1e-5 * np.abs(g).sum()))
    ok = ok and bool(np.allclose(full[1] / sh, oh, rtol=1e-4))
    out[rank] = ok
    dist.destroy_process_group()


def test_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert all(out[r] for r in range(world))


def _failing_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import arboretum_b200
    from arboretum_b200.distributed import guarded

    def step():
        if rank == 1:
            raise MemoryError("no room for the level buffers")  # a set-up step that fails on one rank
        return "ready"

    try:
        guarded(step, "building the level buffers")
        out[rank] = "went on"
    except arboretum_b200.ArboretumError as e:
        out[rank] = str(e)
    # a step that works everywhere goes through on every rank
    out[(rank, "second")] = guarded(lambda: rank * 10, "a step that works")
    dist.destroy_process_group()


def test_a_rank_that_fails_during_set_up_stops_all_ranks():
    """One rank's set-up raises: every rank gets an error instead of entering the next
    exchange, where the others would wait for the one that never comes."""
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_failing_worker, args=(world, port, out), nprocs=world, join=True)
        assert "another rank" in out[0]
        assert "this rank" in out[1] and "no room" in out[1]
        assert out[(0, "second")] == 0 and out[(1, "second")] == 10
