"""CPU-side checks of bench.py: the workload table, its seeded generators and the reference
arm (the CPU port of the path), which must print one well-formed JSON line for every
workload without a GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_generators_are_seeded_and_shaped():
    for name, (rows, features, gen, cfg, desc) in bench.WORKLOADS.items():
        a = gen(500, 3)
        b = gen(500, 3)
        n_cat = bench.CATEGORIES[name](500, 3).shape[1] if name in bench.CATEGORIES else 0
        assert a[0].shape == (500, features - n_cat), name
        assert np.array_equal(a[0], b[0], equal_nan=True), name
        target = a[2] if a[2] is not None else a[1]
        assert len(target) == 500, name
        assert desc % rows  # the description takes the row count
        assert cfg["tree"]["max_depth"] >= 2
    X, y, _ = bench.make_c3(400, 0)
    assert 0.15 < np.isnan(X).mean() < 0.25
    bins, y, _ = bench.make_c5(400, 0)
    assert bins.dtype == np.uint8 and bins.max() <= 254
    _, _, labels = bench.make_c4(2000, 0)
    assert set(np.unique(labels)) <= set(range(10))


@pytest.mark.parametrize("workload", ["c1", "c2", "c3", "c4", "c5"])
def test_reference_arm_prints_one_json_line(workload):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--workload", workload, "--rows", "3000", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "boosting_rounds_per_sec"
    assert d["unit"] == "rounds/s" and d["higher_is_better"] is True and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["e2e"]["value"] == d["value"]
    assert "workload" in d["config"] and "model" not in d["config"]


def test_every_package_name_the_bench_uses_exists():
    """The GPU arm cannot run here, so a misspelt or unexported name would only show on a GPU box."""
    import re

    import arboretum_b200
    source = open(bench.__file__).read()
    names = set(re.findall(r"\barboretum\.([A-Za-z_]\w*)", source))
    assert names, "bench.py no longer calls the package?"
    missing = sorted(n for n in names if not hasattr(arboretum_b200, n))
    assert not missing, missing


def test_every_workload_states_the_rounds_of_its_whole_job():
    assert set(bench.JOB_ROUNDS) == set(bench.WORKLOADS)
    assert bench.JOB_ROUNDS["c2"] == 500 and bench.JOB_ROUNDS["c1"] == 100
