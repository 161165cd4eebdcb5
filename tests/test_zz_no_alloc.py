"""AThresholdsNoAlloc: the threshold search for callers that may not allocate device
memory (their GPU memory belongs to one arena, or they run under a fixed budget):
its scratch is an array inside the library image instead of a cudaMalloc.  The test
hands it device buffers that the TEST allocates (with torch), calls it twice in a row
through the C ABI and compares with the thresholds of the existing entry point
(AQuantize), bit for bit.  The second call uses a shorter column, so leftovers of the
first call in the shared scratch array would show.  A process's first call on a device
may make the CUDA runtime load the library's kernels (which takes device memory once, like
any first launch); from the second call on the free device memory must not move, which
the test reads with cudaMemGetInfo around a repeat of both calls.  Collected last on
purpose."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _existing(col, hist_size):
    import arboretum_b200 as arboretum
    thr, size, _ = arboretum.DMatrix(col.reshape(-1, 1)).quantize(hist_size, False, want_bins=False)
    return thr[0]


def _no_alloc(col, hist_size):
    import torch
    import arboretum_b200 as arboretum
    dev = torch.device("cuda", 0)
    sorted_col = torch.sort(torch.from_numpy(col).to(dev)).values.contiguous()
    out = torch.empty(hist_size, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    err = arboretum.lib().AThresholdsNoAlloc(ctypes.c_void_p(sorted_col.data_ptr()),
                                             ctypes.c_longlong(col.size), ctypes.c_int(hist_size),
                                             ctypes.c_void_p(out.data_ptr()), None)
    assert err is None, err
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_no_alloc_thresholds_match_the_allocating_path_twice():
    rng = np.random.default_rng(17)
    first = rng.normal(size=300_000).astype(np.float32)
    second = np.round(rng.normal(size=41_000) * 20).astype(np.float32)  # many ties, shorter
    for col, hist_size in ((first, 255), (second, 64)):
        assert _no_alloc(col, hist_size).tobytes() == _existing(col, hist_size).tobytes()


def test_no_alloc_calls_leave_the_free_device_memory_unchanged():
    import torch
    rng = np.random.default_rng(18)
    cols = [(rng.normal(size=200_000).astype(np.float32), 255),
            (rng.normal(size=50_000).astype(np.float32), 32)]
    dev = torch.device("cuda", 0)
    staged = []
    for col, hist_size in cols:
        staged.append((torch.sort(torch.from_numpy(col).to(dev)).values.contiguous(),
                       torch.empty(hist_size, dtype=torch.float32, device=dev), col.size, hist_size))
    import arboretum_b200 as arboretum
    call = arboretum.lib().AThresholdsNoAlloc

    def run_all():
        for src, out, n, hist_size in staged:
            err = call(ctypes.c_void_p(src.data_ptr()), ctypes.c_longlong(n), ctypes.c_int(hist_size),
                       ctypes.c_void_p(out.data_ptr()), None)
            assert err is None, err
        torch.cuda.synchronize()

    run_all()  # whatever a first call loads is loaded now
    free_before, _ = torch.cuda.mem_get_info(dev)
    run_all()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before


@pytest.mark.parametrize("n", [0, 1])
def test_no_alloc_degenerate_columns_give_an_empty_table(n):
    import torch
    import arboretum_b200 as arboretum
    dev = torch.device("cuda", 0)
    src = torch.zeros(4, dtype=torch.float32, device=dev)
    out = torch.zeros(16, dtype=torch.float32, device=dev)
    err = arboretum.lib().AThresholdsNoAlloc(ctypes.c_void_p(src.data_ptr()), ctypes.c_longlong(n),
                                             ctypes.c_int(16), ctypes.c_void_p(out.data_ptr()), None)
    assert err is None, err
    torch.cuda.synchronize()
    assert bool(torch.isinf(out).all()) and bool((out > 0).all())  # no threshold: every slot +inf


def test_no_alloc_rejects_oversized_input():
    import arboretum_b200 as arboretum
    # the size check comes before any memory is touched, so dummy non-NULL pointers do
    err = arboretum.lib().AThresholdsNoAlloc(ctypes.c_void_p(256), ctypes.c_longlong((1 << 26) + 1),
                                             ctypes.c_int(255), ctypes.c_void_p(256), None)
    assert err is not None and b"limit" in err
