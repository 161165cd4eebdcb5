"""Host-side plumbing of row-sharded multi-GPU training (one process per GPU).

Every exchange of the data path is done by the library with NCCL on its own stream: the
per-level histogram sums, the per-round gradient scale and, at the first round, the
all-gather of the quantizer (the ranks find the thresholds of the whole data set together,
each sorting its share of the columns).  What this module does on the host, through
``torch.distributed`` (NCCL or gloo), is the set-up around it:

* ``shard_rows``      -- the contiguous row range of a rank;
* ``init_nccl``       -- rank 0 creates the ncclUniqueId, the others receive it, and
                         every rank joins the communicator of its Garden;
* ``share_thresholds``-- optional: hand thresholds computed elsewhere to every rank
                         (the Gardens then skip their own quantizer).
"""
import ctypes

import numpy as np


def shard_rows(n_rows, rank, world):
    """[begin, end) of the rows rank `rank` owns out of `n_rows`."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    return (n_rows * rank) // world, (n_rows * (rank + 1)) // world


def _broadcast_bytes(buf, src=0):
    """Broadcast a numpy uint8 array in place from rank `src`."""
    import torch
    import torch.distributed as dist
    t = torch.from_numpy(buf)
    if dist.get_backend() == "nccl":
        d = t.cuda()
        dist.broadcast(d, src)
        buf[:] = d.cpu().numpy()
    else:
        dist.broadcast(t, src)
    return buf


def share_thresholds(data, hist_size, rank, world, thresholds=None, sizes=None, src=0):
    """Give every rank's DMatrix the same thresholds.

    With `thresholds` / `sizes` given on rank `src` (computed from the whole data
    set before sharding) they are used as they are; otherwise rank `src` quantises
    its own shard and shares the result (an approximation: 1/world of the rows).
    """
    F = data.columns
    quantized_here = False
    if rank == src and thresholds is None:
        thresholds, sizes, _ = data.quantize(hist_size, True, want_bins=False)
        quantized_here = True  # this DMatrix is binned with these thresholds already
    thr = np.zeros((F, hist_size), dtype=np.float32)
    size = np.zeros(F, dtype=np.int32)
    if rank == src:
        thr[:] = thresholds
        size[:] = sizes
    _broadcast_bytes(thr.view(np.uint8).reshape(-1), src)
    _broadcast_bytes(size.view(np.uint8).reshape(-1), src)
    if not quantized_here:
        data.set_thresholds(thr, size)
    return thr, size


def all_ranks_ok(ok, what="set-up"):
    """Every rank says whether its own step went well; all return True only if all did.
    A rank that failed before a collective must not leave the others waiting inside it: call
    this (``torch.distributed``, any backend) after the step and before the next exchange,
    and raise on every rank when it returns False."""
    import torch
    import torch.distributed as dist
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    if dist.get_backend() == "nccl":
        flag = flag.cuda()
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(int(flag.item()) == 1)


def guarded(step, what="set-up"):
    """Runs ``step()`` on this rank, then agrees with the other ranks: if it raised anywhere,
    it raises here too (``ArboretumError``), and no rank goes on to the next exchange."""
    from . import core
    err = None
    try:
        result = step()
    except Exception as e:  # noqa: BLE001  (reported below, on every rank)
        err, result = e, None
    if not all_ranks_ok(err is None, what):
        raise core.ArboretumError("%s failed on %s" % (what, "this rank: %r" % (err,) if err is not None
                                                       else "another rank"))
    return result


_PROCESS_COMM = None  # (rank, world) of the communicator this process keeps


def init_nccl(garden, rank, world, src=0, reuse=True):
    """Give the Garden a communicator; must precede its first grow_tree.

    The first call of a process makes one (rank ``src`` draws the ncclUniqueId, the others
    receive it through torch.distributed) and the library keeps it; later calls with the
    same rank and world size attach that one (``reuse=False`` makes a new one).  Every rank
    must take the same path, which they do when they make the same sequence of calls."""
    global _PROCESS_COMM
    from . import core
    garden._ensure_init()
    if reuse and _PROCESS_COMM == (rank, world):
        core._call_and_throw_if_error(core.lib().AInitNccl(garden.handle, rank, world, None))
        return
    uid = np.zeros(128, dtype=np.uint8)
    if rank == src:
        core._call_and_throw_if_error(core.lib().ANcclUniqueId(uid.ctypes.data_as(ctypes.c_void_p)))
    _broadcast_bytes(uid, src)
    core._call_and_throw_if_error(core.lib().AInitNccl(garden.handle, rank, world,
                                                      uid.ctypes.data_as(ctypes.c_void_p)))
    if _PROCESS_COMM is None:
        _PROCESS_COMM = (rank, world)
