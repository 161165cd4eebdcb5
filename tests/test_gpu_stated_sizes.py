"""Parity with the CPU oracle at the sizes the benchmark configurations state, and on the
input shapes the smaller parity cases do not reach: the 10 M x 28 binary-classification
configuration level by level, the small regression configuration with all of its 100 trees,
a wide table with missing values, column sampling and categorical columns, heavy-tailed
regression targets, row-count limits on (gradient, hessian) objectives, and training that
continues from a dumped model."""
import json
import os
import sys

import numpy as np
import pytest

from oracle import oracle as orc
from test_gpu_parity import GAIN_GAP, PRED_ATOL, arb, compare_with_oracle, make_config, synth

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    import bench
    return bench


def _same_trees(model, o, rounds=None):
    md, od = json.loads(model.dump())["model"], o.model_dict()
    for a, b in list(zip(md, od))[:rounds]:
        assert a["nodes"] == b["nodes"]
        assert np.allclose(a["weights"], b["weights"], rtol=1e-4, atol=1e-6)


def test_binary_classification_at_full_size_matches_oracle_level_by_level():
    """10 M x 28, reg:logistic, depth 8 (the configuration the headline metric is quoted on):
    every level of two rounds against the oracle -- node row counts exact, split feature and bin
    identical, sums within the contract -- and the predictions of a slice within 1e-4."""
    bench = _bench()
    n = 10_000_000
    X, y = bench.make_rows(n, 0)
    cfg = json.loads(json.dumps(bench.CONFIG))
    cfg["internals"]["double_precision"] = True  # the oracle sums in double
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 2)
    if ambiguous == 0:
        sl = slice(0, n, 97)
        mine = model.train_yhat()[0][sl]
        assert np.allclose(mine, o.yhat()[0][sl], atol=PRED_ATOL, rtol=0)
        arboretum = arb()
        pred = arboretum.load(model.dump()).predict(arboretum.DMatrix(np.ascontiguousarray(X[sl])))
        assert np.allclose(pred, o.predict(np.ascontiguousarray(X[sl])), atol=PRED_ATOL, rtol=0)
        _same_trees(model, o)


def test_small_regression_configuration_all_100_trees():
    """100 k x 28, reg:linear, depth 6, eta 0.1, lambda 1, 100 trees.  Every level of every
    tree is compared until the two sides take different splits of a node, which must then be
    equally good within the tolerance: the reference's gain is a single-precision difference
    of single-precision terms a hundred times its size, so two neighbouring bins are often
    one or two units in the last place apart, and which one wins then hangs on the last bits
    of the sums.  The trees up to there are identical and predict the same within 1e-4; the
    100-tree models of both sides fit the training data equally well."""
    bench = _bench()
    X, y, _ = bench.make_c1(100_000, 0)
    cfg = json.loads(json.dumps(bench.WORKLOADS["c1"][3]))
    cfg["internals"]["double_precision"] = True
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 100)
    same = o.num_trees() - ambiguous  # rounds both sides grew identically
    assert same >= 1
    _same_trees(model, o, same)
    assert np.allclose(model.predict(data, same), o.predict(X, same), atol=PRED_ATOL, rtol=0)
    if ambiguous == 0:
        assert same == 100
        assert np.allclose(model.train_yhat()[0], o.yhat()[0], atol=PRED_ATOL, rtol=0)
    for _ in range(100 - o.num_trees()):
        model.grow_tree()
        o.grow(1)
    rmse = lambda p: float(np.sqrt(np.mean((p.astype(np.float64) - y) ** 2)))
    mine, theirs = rmse(model.train_yhat()[0]), rmse(o.yhat()[0])
    assert abs(mine - theirs) <= 0.01 * theirs, (mine, theirs)


def wide_table(n, seed, F=2000, n_cat=10):
    """The wide-table configuration's shape: F - n_cat log-normal columns with 20 % of the
    cells missing, n_cat categorical columns (cardinality 50 .. 1000, Zipf-distributed), a
    target made of 30 column effects plus noise."""
    rng = np.random.default_rng([3, seed])
    Fd = F - n_cat
    X = np.exp(rng.standard_normal((n, Fd), dtype=np.float32))
    cards = rng.integers(50, 1001, size=n_cat)
    cat = np.stack([np.minimum(rng.zipf(1.2, n), c) - 1 for c in cards], axis=1).astype(np.uint32)
    cols = rng.choice(F, 30, replace=False)
    y = rng.normal(0, 0.5, n)
    for c in cols:
        if c < Fd:
            y += rng.normal() * np.log1p(X[:, c])
        else:
            y += rng.normal(size=cards[c - Fd])[cat[:, c - Fd]]
    # two categorical effects that no dense column explains, so that category splits win nodes
    y += 1.5 * (cat[:, 0] == 0) - 1.0 * (cat[:, 1] == 2)
    X[rng.random((n, Fd), dtype=np.float32) < 0.2] = np.nan
    return X, cat, y.astype(np.float32)


def test_wide_table_with_missing_values_column_sampling_and_categories():
    """2000 features = 63 feature tiles, 20 % NaN, colsample_bytree 0.5 and ten categorical
    columns together; rows cut to what the oracle follows in seconds."""
    X, cat, y = wide_table(20_000, 0)
    cfg = make_config(0, 6, colsample_bytree=0.5)
    cfg["internals"]["seed"] = 3
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 3, categories=cat)
    used = [nd["fid"] for t in json.loads(model.dump())["model"] for nd in t["nodes"] if "category" in nd]
    assert used and min(used) >= X.shape[1]  # category splits were found, on categorical columns
    if ambiguous == 0:
        _same_trees(model, o)
        assert np.allclose(model.predict(data), o.predict(X, categories=cat), atol=PRED_ATOL, rtol=0)
        assert np.allclose(model.train_yhat()[0], o.yhat()[0], atol=PRED_ATOL, rtol=0)


def test_categorical_model_survives_dump_and_load():
    arboretum = arb()
    X, cat, y = wide_table(6000, 1, F=40, n_cat=4)
    cfg = make_config(0, 4)
    data = arboretum.DMatrix(X, data_category=cat, y=y)
    model = arboretum.train(cfg, data, 3)
    again = arboretum.load(model.dump())
    assert np.array_equal(again.predict(data), model.predict(data))
    assert json.loads(again.dump())["model"] == json.loads(model.dump())["model"]


def test_heavy_tailed_regression_target():
    """A few targets hundreds of times larger than the rest: the round's largest |gradient|
    says little about the others, and a fixed-point scale taken from it alone would leave the
    typical gradient a handful of bits.  The sums must still meet the contract."""
    X, y = synth("linear", 60_000, 20, seed=41)
    rng = np.random.default_rng(7)
    out = rng.choice(len(y), 5, replace=False)
    y[out] += 300.0 * np.abs(y).mean() * rng.choice([-1.0, 1.0], 5)
    cfg = make_config(0, 6, eta=0.3)
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 4)
    if ambiguous == 0:
        assert np.allclose(model.train_yhat()[0], o.yhat()[0], atol=PRED_ATOL * max(1.0, float(np.abs(y).mean())), rtol=1e-5)


@pytest.mark.parametrize("objective", [1, 3])
def test_min_leaf_size_with_gradient_hessian_objectives(objective):
    """min_leaf_size gates every candidate on row counts (gain.cu:125-134 of the reference);
    (gradient, hessian) objectives get them from a count histogram."""
    rng = np.random.default_rng(12)
    n, F = 15_000, 12
    X = rng.normal(size=(n, F)).astype(np.float32)
    if objective == 1:
        X, y = synth("logistic", n, F, seed=12)
        cfg = make_config(1, 6, eta=0.3, min_leaf_size=400, min_child_weight=0.5)
        model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 3)
    else:
        K = 3
        labels = np.argmax(X @ rng.normal(size=(F, K)) + rng.gumbel(size=(n, K)), axis=1).astype(np.uint8)
        cfg = make_config(3, 5, eta=0.3, labels_count=K, min_leaf_size=300, min_child_weight=0.5)
        model, data, o, ambiguous = compare_with_oracle(cfg, X, None, 2, labels=labels)
    # the limit binds: some node of the last level has no admissible split left
    last = model.level_stats(cfg["tree"]["max_depth"] - 1)
    sizes = np.diff(last["node_begin"].astype(np.int64))
    assert (last["fid"] < 0).any() or sizes.min() >= cfg["tree"]["min_leaf_size"]
    if ambiguous == 0:
        _same_trees(model, o)


def test_training_continues_from_a_dumped_model():
    """Six rounds in one go, and three rounds, dump, load, three more on the same matrix: the
    restored predictions, the position of the feature-sampling engine and the round counter
    make the second half identical."""
    arboretum = arb()
    X, y = synth("logistic", 30_000, 20, seed=17)
    cfg = make_config(1, 5, eta=0.3, colsample_bytree=0.6, colsample_bylevel=0.8)
    straight = arboretum.train(cfg, arboretum.DMatrix(X, y=y), 6)
    first = arboretum.train(cfg, arboretum.DMatrix(X, y=y), 3)
    resumed = arboretum.load(first.dump())
    resumed.data = arboretum.DMatrix(X, y=y)
    for _ in range(3):
        resumed.grow_tree()
    a, b = json.loads(straight.dump())["model"], json.loads(resumed.dump())["model"]
    assert len(a) == len(b) == 6
    for ta, tb in zip(a, b):
        assert ta["nodes"] == tb["nodes"]
        assert np.allclose(ta["weights"], tb["weights"], rtol=1e-5, atol=1e-7)
    assert np.allclose(straight.train_yhat(), resumed.train_yhat(), atol=1e-5, rtol=0)
