"""Driver of the reference's own CUDA build (``oracle/_ref/libarboretum_ref.so``, made by
``oracle/build_ref_cuda.py``): the second checker and the single-GPU baseline.

TEST INFRASTRUCTURE ONLY.  Nothing under ``arboretum_b200/`` imports this file.  Every
command runs the reference in THIS process; callers that must survive a reference that
calls ``exit()`` on a CUDA error (src/core/cuda_helpers.h:12-20) start it as a child:

    python oracle/ref_cuda.py kats [filter]      the reference's tests/cpp known-answer tests
    python oracle/ref_cuda.py iris               tests/py/test_hist_logregression.py goldens
    python oracle/ref_cuda.py train --workload c1 --rounds 100 --out result.npz
    python oracle/ref_cuda.py time  --workload c2 --rounds 20 --warmup 3

``train`` / ``time`` take the benchmark's seeded generators (``bench.WORKLOADS``) and print
one JSON line; ``train`` also saves the predictions and the dumped model.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "_ref", "libarboretum_ref.so")
KATS = os.path.join(HERE, "_ref", "ref_kats")
GOLDEN = os.path.join(ROOT, "tests", "golden", "iris_hist_golden.json")


def available():
    return os.path.exists(LIB)


class Ref(object):
    """The fourteen entry points of python-wrapper/arboretum_wrapper.h:4-39."""

    def __init__(self):
        L = ctypes.CDLL(LIB)
        for name in ("ACreateFromDenseMatrix", "ASetY", "AInitGarden", "AGrowTree", "APredict",
                     "ADumpModel", "ALoadModel", "AFreeDMatrix", "AFreeGarden", "ADeleteArray"):
            getattr(L, name).restype = ctypes.c_char_p
        self.L = L

    @staticmethod
    def _ok(ret):
        if ret is not None:
            raise RuntimeError("reference: %s" % ret.decode(errors="replace"))

    def dmatrix(self, X, y):
        X = np.ascontiguousarray(X, dtype=np.float32)
        h = ctypes.c_void_p()
        self._ok(self.L.ACreateFromDenseMatrix(
            X.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), None, ctypes.c_int(X.shape[0]),
            ctypes.c_int(X.shape[1]), ctypes.c_int(0), ctypes.c_float(np.nan), ctypes.byref(h)))
        if y is not None:
            y = np.ascontiguousarray(y, dtype=np.float32)
            self._ok(self.L.ASetY(h, y.ctypes.data_as(ctypes.POINTER(ctypes.c_float))))
        return h

    def garden(self, cfg):
        g = ctypes.c_void_p()
        self._ok(self.L.AInitGarden(ctypes.c_char_p(json.dumps(cfg).encode()), ctypes.byref(g)))
        return g

    def grow(self, g, d):
        self._ok(self.L.AGrowTree(g, d, None))

    def predict(self, g, d, rows, n_rounds=-1):
        out = ctypes.POINTER(ctypes.c_float)()
        self._ok(self.L.APredict(g, d, ctypes.byref(out), ctypes.c_int(n_rounds)))
        res = np.copy(np.ctypeslib.as_array(out, shape=(rows,)))
        self.L.ADeleteArray(out)
        return res

    def dump(self, g):
        s = ctypes.c_char_p()
        self._ok(self.L.ADumpModel(ctypes.byref(s), g))
        return s.value.decode()


def reference_config(cfg, double_precision=None):
    """A configuration of this repository's benchmarks as the reference parses it
    (src/core/json_conversion.h:108-167): every key it reads, none it does not."""
    t = cfg["tree"]
    out = {"objective": cfg["objective"], "method": 1,
           "internals": {"double_precision": bool(cfg["internals"].get("double_precision", False)
                                                  if double_precision is None else double_precision),
                         "compute_overlap": 2, "use_hist_subtraction_trick": True,
                         "dynamic_parallelism": True, "upload_features": True,
                         "hist_size": cfg["internals"].get("hist_size", 255),
                         "seed": cfg["internals"].get("seed", 0)},
           "verbose": {"gpu": False, "booster": False, "data": False},
           "tree": {"eta": t.get("eta", 0.1), "max_depth": t["max_depth"], "gamma": 0.0,
                    "min_child_weight": t.get("min_child_weight", 1.0),
                    "min_leaf_size": t.get("min_leaf_size", 1),
                    "colsample_bytree": t.get("colsample_bytree", 1.0),
                    "colsample_bylevel": t.get("colsample_bylevel", 1.0),
                    "lambda": t.get("lambda", 1.0), "alpha": t.get("alpha", 0.0)}}
    return out


def cmd_kats(args):
    if not os.path.exists(KATS):
        print(json.dumps({"kats": "unavailable", "why": "oracle/_ref/ref_kats is not built"}))
        return 2
    return subprocess.call([KATS] + ([args.filter] if args.filter else []))


def cmd_iris(args):
    from sklearn.datasets import load_iris
    iris = load_iris()
    X, y = iris.data.astype(np.float32), (iris.target != 2).astype(np.float32)
    gold = json.load(open(GOLDEN))
    ref = Ref()
    worst, close = 0.0, True
    for case, c in sorted(gold["hist_logregression"].items()):
        for dp in (True, False):
            cfg = json.loads(json.dumps(gold["config"]))
            cfg["tree"]["max_depth"] = c["max_depth"]
            cfg["internals"]["double_precision"] = dp
            d = ref.dmatrix(X, y)
            g = ref.garden(cfg)
            for _ in range(c["trees"]):
                ref.grow(g, d)
            for i in range(c["trees"]):
                p = ref.predict(g, d, len(y), i + 1)
                worst = max(worst, float(np.abs(p - np.asarray(c["predictions"][i])).max()))
                close = close and bool(np.allclose(p, c["predictions"][i]))  # the reference test's own check
            model = json.loads(ref.dump(g))
            for a, b in zip(c["model"]["model"], model["model"]):
                assert a["nodes"] == b["nodes"], (case, dp)
                assert np.allclose(a["weights"], b["weights"], rtol=1e-4, atol=1e-6), (case, dp)
    ok = close
    print(json.dumps({"iris_goldens": "ok" if ok else "FAILED", "max_abs_prediction_error": worst}))
    return 0 if ok else 1


def _workload(args):
    sys.path.insert(0, ROOT)
    import bench
    rows_default, features, gen, cfg, desc = bench.WORKLOADS[args.workload]
    rows = args.rows or rows_default
    X, y, labels = gen(rows, args.seed)
    assert labels is None and X.dtype == np.float32, "the reference trains dense fp32 with reg:linear / reg:logistic only"
    return X, y, reference_config(cfg, bool(args.double)), desc % rows


def cmd_train(args):
    X, y, cfg, desc = _workload(args)
    ref = Ref()
    d = ref.dmatrix(X, y)
    g = ref.garden(cfg)
    t0 = time.perf_counter()
    for _ in range(args.rounds):
        ref.grow(g, d)
    t1 = time.perf_counter()
    pred = ref.predict(g, d, len(y))
    np.savez_compressed(args.out, pred=pred, model=np.frombuffer(ref.dump(g).encode(), dtype=np.uint8))
    print(json.dumps({"workload": desc, "rounds": args.rounds, "train_s": t1 - t0, "out": args.out}))
    return 0


def cmd_time(args):
    import torch
    X, y, cfg, desc = _workload(args)
    ref = Ref()
    t0 = time.perf_counter()
    d = ref.dmatrix(X, y)
    g = ref.garden(cfg)
    ref.grow(g, d)  # quantises the matrix first (DataMatrix::InitHist, src/io/io.cu:342-435)
    torch.cuda.synchronize()
    first_s = time.perf_counter() - t0
    for _ in range(max(0, args.warmup - 1)):
        ref.grow(g, d)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    for _ in range(args.rounds):
        ref.grow(g, d)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t1
    print(json.dumps({"impl": "reference CUDA build (sm_100a, five compatibility edits)",
                      "workload": desc, "double_precision": bool(args.double),
                      "value": args.rounds / dt, "unit": "rounds/s", "ms_per_round": 1000.0 * dt / args.rounds,
                      "rounds": args.rounds, "warmup": args.warmup,
                      "first_round_with_quantisation_s": first_s,
                      "how": "wall clock around `for round: AGrowTree` with the matrix quantised and "
                             "resident (python-wrapper/arboretum_wrapper.cu:101-111); every round "
                             "synchronises the device itself", "host_cores": os.cpu_count()}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    k = sub.add_parser("kats")
    k.add_argument("filter", nargs="?", default="")
    sub.add_parser("iris")
    for name in ("train", "time"):
        p = sub.add_parser(name)
        p.add_argument("--workload", default="c1")
        p.add_argument("--rows", type=int, default=0)
        p.add_argument("--rounds", type=int, default=20)
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--double", type=int, default=0)
        p.add_argument("--seed", type=int, default=0)
        p.add_argument("--out", default="ref_cuda_result.npz")
    args = ap.parse_args()
    return {"kats": cmd_kats, "iris": cmd_iris, "train": cmd_train, "time": cmd_time}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
