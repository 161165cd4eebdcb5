"""The reference's own code as a second checker.

* Where the reference tree is mounted (REF, default the sibling checkout): ITS
  python-package/arboretum/core.py is imported from a scratch directory that holds a link to
  this repository's libarboretum.so -- the drop-in claim, line for line: the loader finds the
  library, binds the fourteen symbols it declares, and (on a GPU) replays one of its golden
  tests through it.
* Where the reference's CUDA library has been compiled (oracle/_ref/libarboretum_ref.so, made
  by oracle/build_ref_cuda.py): the small regression configuration is trained by it and by this
  build on the same seeded rows; trees and predictions must agree.  The reference runs in a
  child process (it calls exit() on CUDA errors).
"""
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("REF", os.path.join(os.path.dirname(ROOT), "reference"))
REF_CORE = os.path.join(REF, "python-package", "arboretum", "core.py")
GOLDEN = os.path.join(ROOT, "tests", "golden", "iris_hist_golden.json")


def _reference_package(tmp_path):
    """The reference's Python package, imported from a directory of links: its core.py,
    its __init__.py and this build's library under the name its loader looks for."""
    pkg = tmp_path / "arboretum"
    pkg.mkdir()
    for name in ("core.py", "__init__.py"):
        os.symlink(os.path.join(REF, "python-package", "arboretum", name), pkg / name)
    os.symlink(os.path.join(ROOT, "arboretum_b200", "libarboretum.so"), pkg / "libarboretum.so")
    spec = importlib.util.spec_from_file_location("arboretum_reference_package", pkg / "__init__.py",
                                                  submodule_search_locations=[str(pkg)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["arboretum_reference_package"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.skipif(not os.path.exists(REF_CORE), reason="the reference tree is not mounted here")
def test_reference_python_package_loads_this_library(tmp_path):
    ref = _reference_package(tmp_path)
    import arboretum_b200  # noqa: F401  (the build must exist)
    for name in ("DMatrix", "Garden", "train", "load"):
        assert hasattr(ref, name)
    lib = sys.modules["arboretum_reference_package.core"]._LIB
    for sym in ("ACreateFromDenseMatrix", "ASetY", "ASetLabel", "ASetWeights", "AInitGarden", "AGrowTree",
                "AAppendLastTree", "AGetY", "APredict", "ADumpModel", "ALoadModel", "AFreeDMatrix",
                "AFreeGarden", "ADeleteArray"):
        assert hasattr(lib, sym), sym


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(REF_CORE), reason="the reference tree is not mounted here")
def test_reference_python_package_replays_its_golden_through_this_library(tmp_path):
    from sklearn.datasets import load_iris
    ref = _reference_package(tmp_path)
    gold = json.load(open(GOLDEN))
    c = gold["hist_logregression"]["test_single_tree_depth_2"]
    cfg = json.loads(json.dumps(gold["config"]))
    cfg["tree"]["max_depth"] = c["max_depth"]
    iris = load_iris()
    data = ref.DMatrix(iris.data, y=(iris.target != 2))
    model = ref.train(cfg, data, c["trees"])
    assert np.allclose(model.predict(data, 1), c["predictions"][0])


def _ref_cuda_available():
    return os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libarboretum_ref.so"))


@pytest.mark.gpu
@pytest.mark.skipif(not _ref_cuda_available(), reason="the reference's CUDA library is not built")
@pytest.mark.parametrize("double_precision", [1, 0])
def test_small_regression_configuration_against_the_reference_cuda_build(tmp_path, double_precision):
    """100 k x 28, reg:linear, depth 6, 100 trees by the reference's own CUDA code and by this
    build: identical trees for as long as no node has two equally good splits, thresholds bit
    for bit (they come from the quantiser: equal thresholds mean equal bin borders), and
    predictions within 1e-4."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import bench
    import arboretum_b200 as arboretum
    out = str(tmp_path / "ref.npz")
    rounds = 100
    run = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_cuda.py"), "train", "--workload", "c1",
                          "--rounds", str(rounds), "--double", str(double_precision), "--out", out],
                         cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    ref = np.load(out)
    ref_model = json.loads(ref["model"].tobytes().decode())["model"]
    X, y, _ = bench.make_c1(100_000, 0)
    cfg = json.loads(json.dumps(bench.WORKLOADS["c1"][3]))
    data = arboretum.DMatrix(X, y=y)
    model = arboretum.train(cfg, data, rounds)
    mine = json.loads(model.dump())["model"]
    same = 0
    for a, b in zip(mine, ref_model):
        if a["nodes"] != b["nodes"]:
            break
        same += 1
    # The runs part where a node has two splits whose gains are a unit or two in the last place
    # of the single-precision terms apart (the reference's double- and single-precision modes
    # part from one another the same way, after 16 trees on these rows); up to there the trees
    # are the same, and the finished models fit the training data equally well.
    assert same >= 1, "identical trees: %d" % same
    for a, b in list(zip(mine, ref_model))[:same]:
        assert np.allclose(a["weights"], b["weights"], rtol=1e-3, atol=1e-5)
    if same == rounds:
        assert np.allclose(model.predict(data), ref["pred"], atol=1e-4, rtol=0)
    else:  # the first `same` trees are the same functions: compare what they predict
        part = arboretum.load(json.dumps({"configuration": json.loads(model.dump())["configuration"],
                                          "model": ref_model[:same]}))
        assert np.allclose(model.predict(data, same), part.predict(data), atol=1e-4, rtol=0)
    rmse = lambda p: float(np.sqrt(np.mean((p.astype(np.float64) - y) ** 2)))
    mine_fit, ref_fit = rmse(model.predict(data)), rmse(ref["pred"])
    assert abs(mine_fit - ref_fit) <= 0.01 * ref_fit, (mine_fit, ref_fit)
