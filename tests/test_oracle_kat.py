"""Pins the CPU oracle against the reference's own known-answer tests.

Each test restates the inputs of one reference test (they are formulas, a few
lines each) and checks the oracle against the expected values that test asserts.
"""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "iris_hist_golden.json")


# --- quantizer: tests/cpp/test_datamatrix.cu -------------------------------------
def _bits(size):
    return int(size).bit_length()  # io.cu:411  32 - clz(size)


def test_hist_wide_range():  # test_datamatrix.cu:25-46
    col = np.array([128 - i for i in range(128)], dtype=np.float32)
    thr, size, bins = orc.quantize_column(col, 8)
    assert _bits(size) == 4
    assert (bins == np.array([8 - (i // 16) - 1 for i in range(128)])).all()


def test_hist_255():  # test_datamatrix.cu:48-71
    col = np.arange(1024, dtype=np.float32)
    thr, size, bins = orc.quantize_column(col, 255)
    assert _bits(size) == 8
    exp = np.array([i // (1024 // 255) if i < 1020 else 254 for i in range(1024)])
    assert (bins == exp).all()


def test_hist_skewed_range():  # test_datamatrix.cu:73-111
    col = np.array([10, 0, 11, 1, 0, 2, 3, 0, 0, 0, 0, 0], dtype=np.float32)
    thr, size, bins = orc.quantize_column(col, 4)
    assert _bits(size) == 3
    assert bins.tolist() == [3, 0, 3, 1, 0, 2, 3, 0, 0, 0, 0, 0]


def test_hist_tiny_range1():  # test_datamatrix.cu:113-152
    col = np.array([0, 0, 0, 1, 0, 2, 0, 0, 0, 0, 0, 0], dtype=np.float32)
    thr, size, bins = orc.quantize_column(col, 4)
    assert _bits(size) == 2
    assert bins.tolist() == [0, 0, 0, 1, 0, 2, 0, 0, 0, 0, 0, 0]


def test_hist_tiny_range2():  # test_datamatrix.cu:154-197
    col = np.array([10, 10, 10, 1, 10, 2, 10, 10, 10, 10, 10, 10], dtype=np.float32)
    thr, size, bins = orc.quantize_column(col, 4)
    assert _bits(size) == 1
    assert bins.tolist() == [0] * 12
    assert np.isinf(thr[0])


# --- partition index: tests/cpp/test_hist.cu:20-78 ---------------------------------
def test_partition_index():
    go_right = np.array([i % 2 for i in range(32)], dtype=np.uint8)
    idx = orc.partition_index(go_right, [0, 32])
    exp = [i // 2 if i % 2 == 0 else 31 - i // 2 for i in range(32)]
    assert idx.tolist() == exp


# --- naive histograms: tests/cpp/test_hist_sum.cu (grad[i]=i, bin=i%H patterns) ----
@pytest.mark.parametrize("hist_size,n", [(4, 32), (256, 1 << 12), (1024, 1 << 13)])
def test_hist_single_segment(hist_size, n):
    bins = np.arange(n) % hist_size
    g = np.arange(n, dtype=np.float32)
    og, oh, oc = orc.hist(bins, g, np.ones(n, dtype=np.float32), [0, n], hist_size)
    per = n // hist_size
    for b in range(hist_size):
        assert oc[b] == per
        assert og[b] == sum(range(b, n, hist_size))
        assert oh[b] == per


# --- split search: tests/cpp/test_hist.cu:80-127 (root), :129-260 (level 1) --------
def _best(lsum, lcnt, tot, tcnt, p):
    best = (0.0, 0)
    for i in range(len(lsum)):
        g = orc.lib().orc_gain_f2(lsum[i][0], lsum[i][1], tot[0], tot[1], lcnt[i], tcnt, p)
        if g > 0 and (g > best[0] or (g == best[0] and i > best[1])):
            best = (g, i)
    return best


def test_root_search_gain():  # expected (idx 1, gain 2048.0), test_hist.cu:124-126
    p = orc.gain_params()
    g = np.arange(32, dtype=np.float64)
    bins = np.arange(32) // 8
    ls = [(g[bins <= b].sum(), float((bins <= b).sum())) for b in range(4)]
    lc = [int((bins <= b).sum()) for b in range(4)]
    gain, idx = _best(ls, lc, (g.sum(), 32.0), 32, p)
    assert idx == 1
    assert gain == pytest.approx(2048.0, rel=1e-6)


def test_level1_search_gain():  # expected (4, 64026.672), (11, 565504), test_hist.cu:222-226
    p = orc.gain_params()
    g = np.array([i * i for i in range(32)], dtype=np.float64)
    bins = np.arange(32) // 4
    go_right = np.arange(32) % 2
    idx = orc.partition_index(go_right.astype(np.uint8), [0, 32])
    # the reference test partitions only the bin column (ProcessDenseFeature);
    # the gradients stay in their original positions
    g2 = g
    b2 = np.empty(32, dtype=np.int64)
    b2[idx] = bins
    # expected partitioned column, test_hist.cu:228-259
    assert b2.tolist() == [i // 2 for i in range(16)] + [7 - i // 2 for i in range(16)]
    og, oh, oc = orc.hist(b2, g2.astype(np.float32), np.ones(32, dtype=np.float32), [0, 16, 32], 8)
    assert og.tolist() == [1, 13, 41, 85, 145, 221, 313, 421,
                           1861, 1625, 1405, 1201, 1013, 841, 685, 545]  # test_hist.cu:188-220
    assert (oc == 2).all()
    for node, (eidx, egain) in enumerate([(4, 64026.672), (11, 565504.0)]):
        sl = slice(node * 8, node * 8 + 8)
        cg = np.cumsum(og[sl])
        cc = np.cumsum(oc[sl])
        ls = [(cg[b], float(cc[b])) for b in range(8)]
        gain, i = _best(ls, [int(c) for c in cc], (cg[-1], 16.0), 16, p)
        assert node * 8 + i == eidx
        assert gain == pytest.approx(egain, rel=1e-6)


# --- end to end: iris goldens (tests/py/test_hist_logregression.py) ------------------
def _iris():
    from sklearn.datasets import load_iris
    iris = load_iris()
    return iris.data.astype(np.float32), (iris.target != 2).astype(np.float32)


def _assert_model(true_model, trees, rtol=1e-4, atol=1e-6):  # tests/py/utils.py:4-12
    assert len(true_model["model"]) == len(trees)
    for t, c in zip(true_model["model"], trees):
        assert np.allclose(t["weights"], c["weights"], rtol=rtol, atol=atol)
        assert t["nodes"] == c["nodes"]


@pytest.mark.parametrize("case", ["test_single_tree_depth_2", "test_2trees_depth_1"])
@pytest.mark.parametrize("double_precision", [True, False])
@pytest.mark.parametrize("use_trick", [True, False])
def test_iris_golden(case, double_precision, use_trick):
    gold = json.load(open(GOLDEN))
    c = gold["hist_logregression"][case]
    cfg = json.loads(json.dumps(gold["config"]))
    cfg["tree"]["max_depth"] = c["max_depth"]
    cfg["internals"]["double_precision"] = double_precision
    cfg["internals"]["use_hist_subtraction_trick"] = use_trick
    X, y = _iris()
    o = orc.Oracle(cfg).set_dense(X).set_y(y).grow(c["trees"])
    _assert_model(c["model"], o.model_dict())
    for i in range(c["trees"]):
        assert np.allclose(o.predict(X, i + 1), c["predictions"][i])


@pytest.mark.parametrize("hist_size", [255, 256, 511, 512, 1023])
def test_iris_sklearn_golden(hist_size):  # tests/py/test_sklearn_classification.py:9-61
    gold = json.load(open(GOLDEN))
    cfg = json.loads(json.dumps(gold["config"]))
    cfg["tree"]["max_depth"] = 2
    cfg["internals"]["hist_size"] = hist_size
    X, y = _iris()
    o = orc.Oracle(cfg).set_dense(X).set_y(y).grow(1)
    assert np.allclose(o.predict(X), gold["sklearn_classification"]["predictions"][0])


# --- multi-node histogram sums: tests/cpp/test_hist_sum.cu:383-640 ---------------------
def multi_node_kats():
    """(name, bins, grad, node_begin, with_parent, expected counts, expected sums); None = unchecked.
    Inputs follow the reference tests' formulas (grad[i] = i, bin = i % 4 or 0, two nodes)."""
    size = 1280
    i = np.arange(size)
    g = i.astype(np.float32)
    b4 = (i % 4).astype(np.uint16)
    whole = np.array([np.bincount(b4, weights=g, minlength=4)]), np.array([np.bincount(b4, minlength=4)])
    return [
        ("2_NodesNoTrick", b4, g, [0, size // 2, size], None,           # :383-424
         [size // 8] * 8, None),
        ("2_NodesAsymmetricNoTrick", b4, g, [0, 10, size], None,        # :426-477
         [3, 3, 2, 2, 317, 317, 318, 318],
         [12.0, 15.0, 8.0, 10.0, 204148.0, 204465.0, 204792.0, 205110.0]),
        ("2_NodesAsymmetricWithTrick", b4, g, [0, 10, size], whole,     # :479-538
         [3, 3, 2, 2, 317, 317, 318, 318],
         [12.0, 15.0, 8.0, 10.0, 204148.0, 204465.0, 204792.0, 205110.0]),
        ("2_NodesAsymmetricWithTrick2", b4, g, [0, size - 10, size], whole,  # :540-599
         [318, 318, 317, 317, 2, 2, 3, 3],
         [201612.0, 201930.0, 200978.0, 201295.0, 2548.0, 2550.0, 3822.0, 3825.0]),
        ("SingleSegmentWithTrick", np.zeros(size, dtype=np.uint16), g, [0, size // 2, size],  # :601-650
         (np.array([[g.sum(), 0, 0, 0]]), np.array([[size, 0, 0, 0]])),
         [size // 2, 0, 0, 0, size // 2, 0, 0, 0],
         [float(g[:size // 2].sum()), 0, 0, 0, float(g[size // 2:].sum()), 0, 0, 0]),
    ]


@pytest.mark.parametrize("case", range(5))
def test_multi_node_hist_sum_kats(case):
    name, bins, g, node_begin, parent, counts, sums = multi_node_kats()[case]
    nb = np.array(node_begin, dtype=np.uint32)
    if parent is None:
        og, _, oc = orc.hist(bins, g, None, nb, 4)
    else:  # the smaller child is scanned (ties: the left one), the other is parent - scanned
        left_small = nb[1] - nb[0] <= nb[2] - nb[1]
        seg = nb[:2] if left_small else nb[1:]
        sg, _, sc = orc.hist(bins, g, None, np.array(seg, dtype=np.uint32), 4)
        rest_g, rest_c = parent[0][0] - sg, parent[1][0] - sc
        og = np.concatenate([sg, rest_g] if left_small else [rest_g, sg])
        oc = np.concatenate([sc, rest_c] if left_small else [rest_c, sc])
    assert oc.tolist() == counts
    if sums is not None:
        assert og.tolist() == sums
    if name == "2_NodesNoTrick":
        half = 1280 // 2
        assert og[:4].sum() == half * (half - 1) / 2
        assert og[4:].sum() == half * (half + 1280 - 1) / 2


# --- categorical columns (extension: one category against the rest) --------------------
def test_oracle_splits_on_a_category():
    rng = np.random.default_rng(5)
    n = 4000
    X = rng.normal(size=(n, 3)).astype(np.float32)
    cat = np.stack([rng.integers(0, 6, n), rng.integers(0, 400, n)], axis=1).astype(np.uint32)
    y = (2.0 * (cat[:, 0] == 4) + 0.1 * X[:, 0] + rng.normal(0, 0.05, n)).astype(np.float32)
    cfg = {"objective": 0, "method": 1, "internals": {"hist_size": 255, "seed": 0, "double_precision": True},
           "tree": {"max_depth": 2, "eta": 1.0, "lambda": 0.0, "min_child_weight": 1.0, "min_leaf_size": 1,
                    "initial_y": 0.0}}
    o = orc.Oracle(cfg, missing_bin=True).set_dense(X, categories=cat).set_y(y).grow(1)
    root = o.model_dict()[0]["nodes"][0]
    assert root["fid"] == 3 and root["category"] == 4 and root["threshold"] is None
    pred = o.predict(X, categories=cat)
    assert np.abs(pred - y).mean() < 0.1
    # 400 categories do not fit 255 bins: the 254 most frequent keep a bin, the rest share one
    bins, _, sizes = o.bins()
    assert sizes[4] == 255 and bins[4].max() == 254 and sizes[3] == 6
