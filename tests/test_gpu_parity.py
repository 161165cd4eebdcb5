"""Parity of the CUDA path (through the C ABI) with the CPU oracle and with the
reference's golden vectors.  Integer results (bins, node row counts, split
feature / bin) must match exactly; histogram sums within 1e-5 relative; tree
structures must be identical wherever the oracle's best and runner-up gains of a
node differ by more than 1e-6 relative; predictions within 1e-4."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "iris_hist_golden.json")
HIST_RTOL = 1e-5
GAIN_GAP = 1e-6
PRED_ATOL = 1e-4


def arb():
    import arboretum_b200
    return arboretum_b200


# ---------------------------------------------------------------------------------
# quantizer
# ---------------------------------------------------------------------------------
def _quantize_gpu(X, hist_size, missing_bin=False):
    d = arb().DMatrix(np.ascontiguousarray(X, dtype=np.float32))
    return d.quantize(hist_size, missing_bin)


KAT_COLUMNS = [  # tests/cpp/test_datamatrix.cu
    (np.array([128 - i for i in range(128)], dtype=np.float32), 8,
     [8 - (i // 16) - 1 for i in range(128)]),
    (np.arange(1024, dtype=np.float32), 255,
     [i // 4 if i < 1020 else 254 for i in range(1024)]),
    (np.array([10, 0, 11, 1, 0, 2, 3, 0, 0, 0, 0, 0], dtype=np.float32), 4,
     [3, 0, 3, 1, 0, 2, 3, 0, 0, 0, 0, 0]),
    (np.array([0, 0, 0, 1, 0, 2, 0, 0, 0, 0, 0, 0], dtype=np.float32), 4,
     [0, 0, 0, 1, 0, 2, 0, 0, 0, 0, 0, 0]),
    (np.array([10, 10, 10, 1, 10, 2, 10, 10, 10, 10, 10, 10], dtype=np.float32), 4, [0] * 12),
]


@pytest.mark.parametrize("case", range(len(KAT_COLUMNS)))
def test_quantizer_reference_kats(case):
    col, hist_size, expected = KAT_COLUMNS[case]
    thr, size, bins = _quantize_gpu(col.reshape(-1, 1), hist_size)
    assert bins[:, 0].tolist() == expected


@pytest.mark.parametrize("n,F,hist_size,kind", [
    (5000, 7, 255, "normal"), (20000, 28, 255, "normal"), (3000, 5, 16, "dups"),
    (4096, 3, 512, "normal"), (1500, 4, 1023, "normal"), (2000, 6, 255, "nan"),
    (700, 2, 255, "const"), (100003, 3, 255, "lognormal")])
def test_quantizer_matches_oracle_bit_exactly(n, F, hist_size, kind):
    rng = np.random.default_rng(n + F)
    X = rng.normal(size=(n, F)).astype(np.float32)
    missing = False
    if kind == "dups":
        X = np.round(X * 3).astype(np.float32)
    elif kind == "nan":
        X[rng.random(X.shape) < 0.2] = np.nan
        missing = True
    elif kind == "const":
        X[:, 0] = 3.5
    elif kind == "lognormal":
        X = np.exp(X).astype(np.float32)
    thr, size, bins = _quantize_gpu(X, hist_size, missing)
    for f in range(F):
        othr, osize, obins = orc.quantize_column(X[:, f], hist_size, missing)
        assert size[f] == osize
        assert thr[f].tobytes() == othr.tobytes()
        assert (bins[:, f] == obins).all()


# ---------------------------------------------------------------------------------
# histogram kernel
# ---------------------------------------------------------------------------------
def _oracle_hist(bins, g, h, rowid, node_begin, hw):
    n, F = bins.shape
    pos_bins = bins if rowid is None else bins[rowid]
    pg = g if rowid is None else g[rowid]
    ph = None if h is None else (h if rowid is None else h[rowid])
    nn = len(node_begin) - 1
    og = np.zeros((nn, F, hw))
    oh = np.zeros((nn, F, hw))
    for f in range(F):
        a, b, c = orc.hist(pos_bins[:, f], pg, ph, node_begin, hw)
        og[:, f, :] = a.reshape(nn, hw)
        oh[:, f, :] = (b if ph is not None else c.astype(np.float64)).reshape(nn, hw)
    return og, oh


@pytest.mark.parametrize("hist_size,n", [(4, 32), (255, 1 << 12), (256, 1 << 12), (1023, 1 << 13)])
@pytest.mark.parametrize("pair", [False, True])
def test_histogram_reference_pattern(hist_size, n, pair):
    # tests/cpp/test_hist_sum.cu: grad[i] = i, bin = i % hist_size, one segment
    dtype = np.uint8 if hist_size < 256 else np.uint16
    bins = (np.arange(n) % hist_size).astype(dtype).reshape(-1, 1)
    g = np.arange(n, dtype=np.float32)
    grad = np.stack([g, np.ones(n, dtype=np.float32)], axis=1) if pair else g
    og, oh = arb().build_histogram(bins, grad, hist_size, quant_bits=17)
    for b in range(hist_size):
        assert og[0, 0, b] == pytest.approx(float(sum(range(b, n, hist_size))), rel=HIST_RTOL)
        assert oh[0, 0, b] == len(range(b, n, hist_size))


@pytest.mark.parametrize("n,F,hist_size,nodes,pair", [
    (50000, 28, 255, 1, True), (50000, 28, 255, 8, True), (30000, 28, 255, 4, False),
    (20000, 70, 255, 3, True), (9000, 5, 600, 2, True), (7000, 33, 64, 5, False)])
def test_histogram_matches_oracle(n, F, hist_size, nodes, pair):
    rng = np.random.default_rng(n + F + nodes)
    dtype = np.uint8 if hist_size < 256 else np.uint16
    bins = rng.integers(0, hist_size + 1, size=(n, F)).astype(dtype)  # id hist_size = missing
    g = rng.normal(size=n).astype(np.float32)
    h = rng.uniform(0.01, 0.25, size=n).astype(np.float32)
    rowid = rng.permutation(n).astype(np.uint32)
    cuts = np.sort(rng.integers(0, n, size=nodes - 1)) if nodes > 1 else np.array([], dtype=np.int64)
    node_begin = np.concatenate([[0], cuts, [n]]).astype(np.uint32)
    grad = np.stack([g, h], axis=1) if pair else g
    og, oh = arb().build_histogram(bins, grad, hist_size, rowid=rowid, node_begin=node_begin)
    eg, eh = _oracle_hist(bins.astype(np.uint16), g, h if pair else None, rowid, node_begin, hist_size + 1)
    scale_g = np.abs(g).sum() / (hist_size + 1)
    assert np.allclose(og, eg, rtol=HIST_RTOL, atol=HIST_RTOL * scale_g)
    if pair:
        assert np.allclose(oh, eh, rtol=HIST_RTOL, atol=HIST_RTOL)
    else:
        assert (oh == eh).all()  # counts are exact


@pytest.mark.parametrize("n,F,nodes,pair", [(5000, 28, 4, True), (5000, 28, 4, False), (300, 28, 4, True),
                                             (40, 5, 3, True), (200000, 70, 8, True)])
def test_histogram_tma_gather_is_identical(n, F, nodes, pair, monkeypatch):
    """The rows a node names by id are fetched with cp.async or, with ARBORETUM_TMA_GATHER set,
    by the TMA unit (tile::gather4): the sums are integers, so the two must agree exactly."""
    rng = np.random.default_rng(n + nodes)
    bins = rng.integers(0, 256, size=(n, F)).astype(np.uint8)
    g = rng.normal(size=n).astype(np.float32)
    h = rng.uniform(0.01, 0.25, size=n).astype(np.float32)
    rowid = rng.permutation(n).astype(np.uint32)
    node_begin = np.concatenate([[0], np.sort(rng.integers(0, n, size=nodes - 1)), [n]]).astype(np.uint32)
    grad = np.stack([g, h], axis=1) if pair else g
    out = []
    for tma in (False, True):
        if tma:
            monkeypatch.setenv("ARBORETUM_TMA_GATHER", "1")
        else:
            monkeypatch.delenv("ARBORETUM_TMA_GATHER", raising=False)
        out.append(arb().build_histogram(bins, grad, 255, rowid=rowid, node_begin=node_begin))
    assert (out[0][0] == out[1][0]).all() and (out[0][1] == out[1][1]).all()


@pytest.mark.parametrize("case", range(5))
@pytest.mark.parametrize("dtype", [np.uint8, np.uint16])
def test_histogram_multi_node_reference_kats(case, dtype):
    """tests/cpp/test_hist_sum.cu:383-640: two nodes, even and asymmetric, scanned whole or
    with the subtraction trick (the smaller node scanned, the other parent - scanned)."""
    from test_oracle_kat import multi_node_kats
    name, bins, g, node_begin, parent, counts, sums = multi_node_kats()[case]
    nb = np.array(node_begin, dtype=np.uint32)
    kw = {}
    if parent is not None:
        pad = lambda a: np.concatenate([a, np.zeros((1, 1))], axis=1).reshape(1, 1, 5).astype(np.float64)
        kw["parents"] = (pad(parent[0]), pad(parent[1]))
    og, oh = arb().build_histogram(bins.astype(dtype).reshape(-1, 1), g, 4, node_begin=nb, **kw)
    assert oh[:, 0, :4].reshape(-1).tolist() == counts
    assert (oh[:, 0, 4] == 0).all() and (og[:, 0, 4] == 0).all()  # nothing in the missing-value bin
    if sums is not None:
        assert og[:, 0, :4].reshape(-1).tolist() == sums
    else:
        half = len(g) // 2
        assert og[0].sum() == half * (half - 1) / 2 and og[1].sum() == half * (half + len(g) - 1) / 2


# ---------------------------------------------------------------------------------
# end to end
# ---------------------------------------------------------------------------------
def _iris():
    from sklearn.datasets import load_iris
    iris = load_iris()
    return iris.data.astype(np.float32), (iris.target != 2).astype(np.float32)


def _assert_model(true_model, created, rtol=1e-4, atol=1e-6):  # tests/py/utils.py:4-12
    assert len(true_model["model"]) == len(created["model"])
    for t, c in zip(true_model["model"], created["model"]):
        assert np.allclose(t["weights"], c["weights"], rtol=rtol, atol=atol)
        assert t["nodes"] == c["nodes"]


@pytest.mark.parametrize("case", ["test_single_tree_depth_2", "test_2trees_depth_1"])
@pytest.mark.parametrize("double_precision", [True, False])
@pytest.mark.parametrize("use_trick", [True, False])
def test_iris_golden_through_the_abi(case, double_precision, use_trick):
    # tests/py/test_hist_logregression.py:10-66
    arboretum = arb()
    gold = json.load(open(GOLDEN))
    c = gold["hist_logregression"][case]
    cfg = json.loads(json.dumps(gold["config"]))
    cfg["tree"]["max_depth"] = c["max_depth"]
    cfg["internals"]["double_precision"] = double_precision
    cfg["internals"]["use_hist_subtraction_trick"] = use_trick
    X, y = _iris()
    data = arboretum.DMatrix(X, y=y)
    model = arboretum.train(cfg, data, c["trees"])
    for i in range(c["trees"]):
        assert np.allclose(model.predict(data, i + 1), c["predictions"][i])
    dumped = model.dump()
    _assert_model(c["model"], json.loads(dumped))
    restored = arboretum.load(dumped)
    for i in range(c["trees"]):
        assert np.allclose(restored.predict(data, i + 1), c["predictions"][i])


@pytest.mark.parametrize("hist_size", [255, 256, 511, 512, 1023])
def test_iris_sklearn_golden(hist_size):  # tests/py/test_sklearn_classification.py:9-61
    arboretum = arb()
    gold = json.load(open(GOLDEN))
    X, y = _iris()
    data = arboretum.DMatrix(X, y=y)
    model = arboretum.ArboretumClassifier(
        max_depth=2, learning_rate=0.2, n_estimators=1, verbosity=0, gamma_absolute=0.0,
        gamma_relative=0.0, min_child_weight=2.0, min_leaf_size=0, max_leaf_weight=0,
        colsample_bytree=1.0, colsample_bylevel=1.0, l1=0, l2=0, scale_pos_weight=1.0,
        initial_y=0.5, seed=0, double_precision=True, method='hist', hist_size=hist_size)
    model.fit(data, y)
    assert np.allclose(model.predict(data), gold["sklearn_classification"]["predictions"][0])


def make_config(objective, max_depth, eta=0.1, hist_size=255, **tree):
    t = {"eta": eta, "max_depth": max_depth, "lambda": 1.0, "alpha": 0.0, "min_child_weight": 1.0,
         "min_leaf_size": 1, "colsample_bytree": 1.0, "colsample_bylevel": 1.0}
    t.update(tree)
    return {"objective": objective, "method": 1,
            "internals": {"double_precision": True, "compute_overlap": 2, "seed": 0,
                          "use_hist_subtraction_trick": True, "upload_features": True,
                          "hist_size": hist_size},
            "verbose": {"gpu": False, "booster": False, "data": False}, "tree": t}


def synth(kind, n, F, seed):
    rng = np.random.default_rng(seed)
    X = rng.normal(size=(n, F)).astype(np.float32)
    w = rng.normal(size=F)
    if kind == "linear":  # the small regression config: y = w.x + 0.5 x0 x1 + noise
        y = X @ w + 0.5 * X[:, 0] * X[:, min(1, F - 1)] + rng.normal(0, 0.1, n)
    else:
        logit = X @ w * 0.5 + 0.3 * X[:, 0] * X[:, min(1, F - 1)]
        y = (rng.random(n) < 1 / (1 + np.exp(-logit))).astype(np.float64)
    return X, y.astype(np.float32)


CONTRACT_MIN_ROWS = 64  # nodes below this many rows are held to the rigorous bound only


def compare_with_oracle(cfg, X, y, rounds, labels=None, max_level=None, categories=None):
    """Grow `rounds` rounds on both sides, comparing every level of every tree (all
    `labels_count` trees of a multi:softmax round).  Returns (model, data, oracle, ambiguous):
    `ambiguous` counts the rounds in which the two sides took different, equally good splits
    (the comparison stops there: the trees below differ legitimately)."""
    arboretum = arb()
    if labels is None:
        data = arboretum.DMatrix(X, data_category=categories, y=y)
        o = orc.Oracle(cfg, missing_bin=True).set_dense(X, categories=categories).set_y(y)
    else:
        data = arboretum.DMatrix(X, data_category=categories, labels=labels)
        o = orc.Oracle(cfg, missing_bin=True).set_dense(X, categories=categories).set_label(labels)
    model = arboretum.Garden(cfg)
    model.data = data
    model.labels_count = data.labels_count
    K = cfg["tree"].get("labels_count", 1)
    depth = cfg["tree"]["max_depth"]
    lam = cfg["tree"].get("lambda", 1.0)
    ambiguous = 0
    for r in range(rounds):
        model.grow_tree()
        o.grow(1)
        step = model.gradient_step()[0]  # every gradient of the round is off by less than this
        diverged = False
        for k in range(K):
            if diverged:
                break
            t = o.num_trees() - K + k
            for l in range(min(depth, max_level or depth)):
                g = model.level_stats(l, k)
                e = o.level(t, l)
                if l > 0 and not diverged:
                    assert (g["node_begin"] == e["node_begin"]).all(), (r, k, l)
                for i in range(1 << l):
                    if diverged:
                        break
                    same = (g["fid"][i] == e["fid"][i]) and (g["bin"][i] == e["bin"][i] or e["fid"][i] < 0)
                    if not same:
                        gap = abs(e["gain"][i] - max(e["gain2"][i], g["gain"][i])) / max(abs(e["gain"][i]), 1e-30)
                        assert gap <= 10 * GAIN_GAP, (r, k, l, i, g["fid"][i], g["bin"][i], e["fid"][i], e["bin"][i], gap)
                        ambiguous += 1
                        diverged = True
                        continue
                    rows_i = float(e["node_begin"][i + 1] - e["node_begin"][i]) if l > 0 else float(len(X))
                    # (1) what the implementation guarantees: the dithered fixed-point sums are off by
                    #     less than one step per row
                    bound = step * max(rows_i, 1.0)
                    assert abs(g["tot_g"][i] - e["tot_g"][i]) <= bound, (r, k, l, i)
                    assert abs(g["left_g"][i] - e["left_g"][i]) <= bound, (r, k, l, i)
                    # (2) the contract: histogram sums within 1e-5 of the node's sum of |g|
                    contract = HIST_RTOL * max(e["abs_g"][i], 1e-3)
                    if rows_i >= CONTRACT_MIN_ROWS:
                        assert abs(g["tot_g"][i] - e["tot_g"][i]) <= contract, (r, k, l, i, rows_i)
                        assert abs(g["left_g"][i] - e["left_g"][i]) <= contract, (r, k, l, i, rows_i)
                    tol = max(contract, bound) if rows_i < CONTRACT_MIN_ROWS else contract
                    # the gain is a difference of terms G^2 / (H + lambda): an error of `tol` in a
                    # sum G moves a term by 2 |w| tol, with w = G / (H + lambda) the term's weight
                    hs = (e["tot_h"][i], e["left_h"][i], e["tot_h"][i] - e["left_h"][i])
                    gs = (e["tot_g"][i], e["left_g"][i], e["tot_g"][i] - e["left_g"][i])
                    if cfg["objective"] == 0:  # reg:linear: the hessian sum is the row count
                        lc = float(e["left_count"][i])
                        hs = (rows_i, lc, rows_i - lc)
                    wmax = max(abs(a) / (max(b, 0.0) + lam) for a, b in zip(gs, hs))
                    gain_tol = max(1e-4 * abs(e["gain"][i]), 1e-6, 8.0 * wmax * tol)
                    assert abs(g["gain"][i] - e["gain"][i]) <= gain_tol, (r, k, l, i)
        if diverged:
            break
    return model, data, o, ambiguous


@pytest.mark.parametrize("kind,objective,n,depth,rounds", [
    ("linear", 0, 20000, 6, 5), ("logistic", 1, 30000, 8, 5), ("logistic", 1, 5000, 4, 10),
    ("linear", 0, 3000, 3, 8)])
def test_training_matches_oracle(kind, objective, n, depth, rounds):
    X, y = synth(kind, n, 28, seed=depth)
    cfg = make_config(objective, depth)
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, rounds)
    if ambiguous == 0:
        pred = model.predict(data)
        assert np.allclose(pred, o.predict(X), atol=PRED_ATOL, rtol=0)
        assert np.allclose(model.train_yhat()[0], o.yhat()[0], atol=PRED_ATOL, rtol=0)
        md, od = json.loads(model.dump())["model"], o.model_dict()
        for a, b in zip(md, od):
            assert a["nodes"] == b["nodes"]
            assert np.allclose(a["weights"], b["weights"], rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("objective,tree", [
    (0, {"alpha": 0.5, "lambda": 3.0}),                      # L1 and a stronger L2 term
    (1, {"alpha": 0.05, "lambda": 0.1, "min_child_weight": 5.0}),
    (0, {"gamma_absolute": 2.0}),                            # splits must gain at least this much
    (1, {"gamma_relative": 0.05}),                           # ... or this share of the parent's gain
    (0, {"max_leaf_weight": 0.5}),                           # clamped leaf weights
    (1, {"max_leaf_weight": 0.3, "initial_y": 0.2}),
    (0, {"min_leaf_size": 40, "min_child_weight": 40.0}),    # reg:linear has a count plane
])
def test_regularisation_parameters_match_oracle(objective, tree):
    kind = "linear" if objective == 0 else "logistic"
    X, y = synth(kind, 12000, 16, seed=77 + objective)
    cfg = make_config(objective, 5, eta=0.3, **tree)
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 4)
    if ambiguous == 0:
        assert np.allclose(model.train_yhat()[0], o.yhat()[0], atol=PRED_ATOL, rtol=0)
        md, od = json.loads(model.dump())["model"], o.model_dict()
        for a, b in zip(md, od):
            assert a["nodes"] == b["nodes"]
            # (|G| - alpha) / (H + lambda) of a leaf of a few rows cancels when |G| is near
            # alpha: absolute agreement, at a tenth of the predictions' tolerance
            assert np.allclose(a["weights"], b["weights"], rtol=1e-3, atol=0.1 * PRED_ATOL)


def test_training_is_deterministic():
    arboretum = arb()
    X, y = synth("logistic", 40000, 28, seed=11)
    cfg = make_config(1, 6)
    dumps = []
    for _ in range(2):
        data = arboretum.DMatrix(X, y=y)
        dumps.append(arboretum.train(cfg, data, 4).dump())
    assert dumps[0] == dumps[1]


def test_trick_and_no_trick_give_identical_trees():
    arboretum = arb()
    X, y = synth("logistic", 25000, 28, seed=5)
    out = []
    for trick in (True, False):
        cfg = make_config(1, 6)
        cfg["internals"]["use_hist_subtraction_trick"] = trick
        out.append(json.loads(arboretum.train(cfg, arboretum.DMatrix(X, y=y), 3).dump())["model"])
    assert out[0] == out[1]


def test_colsample_follows_the_reference_rng():
    X, y = synth("linear", 8000, 28, seed=3)
    cfg = make_config(0, 4, colsample_bytree=0.5, colsample_bylevel=0.7)
    cfg["internals"]["seed"] = 7
    compare_with_oracle(cfg, X, y, 4)


@pytest.mark.parametrize("kind,objective,hist_size", [("linear", 0, 255), ("logistic", 1, 255), ("logistic", 1, 300)])
def test_sampled_columns_are_histogrammed_from_a_side_by_side_copy(kind, objective, hist_size, monkeypatch):
    """With colsample_bytree < 1 and more feature tiles than the sampled columns need, a tree's
    columns are copied side by side and the histograms and the split search cover those alone
    (70 features, 28 sampled: 3 tiles -> 1 for uint8 bins, 5 -> 2 for uint16).  The trees must
    follow the oracle, and be the very trees the full-width histograms give."""
    arboretum = arb()
    X, y = synth(kind, 9000, 70, seed=12)
    X[np.random.default_rng(2).random(X.shape) < 0.1] = np.nan
    cfg = make_config(objective, 5, hist_size=hist_size, colsample_bytree=0.4, colsample_bylevel=0.8)
    cfg["internals"]["seed"] = 3
    monkeypatch.delenv("ARBORETUM_NO_COLUMN_COPY", raising=False)
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 4)
    monkeypatch.setenv("ARBORETUM_NO_COLUMN_COPY", "1")
    full = arboretum.train(cfg, arboretum.DMatrix(X, y=y), 4)
    assert full.dump() == model.dump()


def test_missing_values_go_right():
    arboretum = arb()
    X, y = synth("linear", 6000, 8, seed=9)
    X[np.random.default_rng(1).random(X.shape) < 0.2] = np.nan
    cfg = make_config(0, 4)
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 3)
    if ambiguous == 0:
        assert np.allclose(model.predict(data), o.predict(X), atol=PRED_ATOL, rtol=0)


@pytest.mark.parametrize("kind,objective", [("linear", 0), ("logistic", 1)])
def test_deep_tree_beyond_the_shared_memory_node_tables(kind, objective):
    # 4096 nodes on the last level: the descend and list kernels leave their 2048-entry
    # shared-memory tables and count / rank through global memory
    X, y = synth(kind, 20000, 12, seed=31)
    cfg = make_config(objective, 14)
    # level by level against the oracle down to the nodes of a few hundred rows; below that
    # a node's gain is a small difference of large terms and the fixed-point step of the
    # gradients shows in it.  One round: the leaves of a tree this deep hold one or two rows,
    # their weights carry those rows' rounding whole, and a second round would start from
    # predictions that already differ by it.
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 1, max_level=7)
    model.grow_tree()
    # the leaf every training row was counted into is the leaf the finished trees send its
    # raw feature values to: the per-row node numbers against the fp32 tree walk
    internal = model.train_yhat()[0]
    pred = model.predict(data)
    if objective == 1:
        internal = 1.0 / (1.0 + np.exp(-internal.astype(np.float64)))
    assert np.allclose(internal, pred, atol=1e-5, rtol=0)
    # the same trees without the subtraction trick (every node gets a list)
    arboretum = arb()
    out = []
    for trick in (True, False):
        c = make_config(objective, 14)
        c["internals"]["use_hist_subtraction_trick"] = trick
        out.append(json.loads(arboretum.train(c, arboretum.DMatrix(X, y=y), 2).dump())["model"])
    assert out[0] == out[1]


@pytest.mark.parametrize("n,F,hist_size,depth,objective", [
    (33, 1, 255, 2, 0),        # fewer rows than a warp, one feature, a single split
    (2049, 3, 15, 3, 1),       # one row past a work item, 16 bins
    (5000, 33, 255, 4, 1),     # one feature past a tile of 32: two tiles, the second nearly empty
    (5000, 65, 255, 5, 0),     # three tiles
    (3000, 7, 2047, 4, 0),     # the largest table: uint16 bins, 4 features per tile
    (4000, 5, 256, 4, 1),      # the smallest uint16 table
    (70000, 28, 255, 9, 1),    # more rows than one CTA of any pass, 256 nodes on the last level
])
def test_edge_shapes_match_oracle(n, F, hist_size, depth, objective):
    X, y = synth("linear" if objective == 0 else "logistic", n, F, seed=n + F)
    cfg = make_config(objective, depth, hist_size=hist_size)
    model, data, o, ambiguous = compare_with_oracle(cfg, X, y, 3, max_level=7)
    internal = model.train_yhat()[0]
    if objective == 1:
        internal = 1.0 / (1.0 + np.exp(-internal.astype(np.float64)))
    assert np.allclose(internal, model.predict(data), atol=1e-5, rtol=0)
    if ambiguous == 0 and depth <= 7:
        assert np.allclose(model.train_yhat()[0], o.yhat()[0], atol=PRED_ATOL, rtol=0)


def test_uint16_bins_training():
    X, y = synth("logistic", 6000, 10, seed=21)
    cfg = make_config(1, 4, hist_size=600)
    compare_with_oracle(cfg, X, y, 3)


def test_append_last_tree_and_get_y():
    arboretum = arb()
    X, y = synth("logistic", 4000, 12, seed=2)
    cfg = make_config(1, 3)
    data = arboretum.DMatrix(X, y=y)
    ev = arboretum.DMatrix(X[:500])
    model = arboretum.Garden(cfg)
    model.data = data
    for _ in range(3):
        model.grow_tree()
        model.append_last_tree(ev)
    assert np.allclose(model.get_y(ev), model.predict(ev), atol=1e-6)


def test_softmax_rounds_match_oracle():
    rng = np.random.default_rng(4)
    n, F, K = 6000, 10, 4
    X = rng.normal(size=(n, F)).astype(np.float32)
    labels = np.argmax(X @ rng.normal(size=(F, K)) + rng.gumbel(size=(n, K)), axis=1).astype(np.uint8)
    cfg = make_config(3, 3, eta=0.2, labels_count=K)
    model, data, o, _ = compare_with_oracle(cfg, X, None, 2, labels=labels)
    pred = model.predict(data)
    assert pred.shape == (n, K)
    assert np.allclose(pred.sum(axis=1), 1.0, atol=1e-5)
    assert np.allclose(pred, o.predict(X), atol=PRED_ATOL, rtol=0)


def test_prebinned_input_equals_dense_input():
    arboretum = arb()
    X, y = synth("logistic", 8000, 12, seed=8)
    cfg = make_config(1, 4)
    dense = arboretum.DMatrix(X, y=y)
    thr, size, bins = dense.quantize(255, True)
    m1 = json.loads(arboretum.train(cfg, dense, 3).dump())["model"]
    pre = arboretum.DMatrix(bins.astype(np.uint8), y=y, binned_hist_size=255)
    m2 = json.loads(arboretum.train(cfg, pre, 3).dump())["model"]
    for a, b in zip(m1, m2):
        assert [n.get("fid") for n in a["nodes"]] == [n.get("fid") for n in b["nodes"]]
        assert a["weights"] == b["weights"]


def test_full_size_level_records_are_consistent():
    """The bench configuration at its full size (10 M x 28, depth 8), where the oracle is too slow
    to follow: properties that hold whatever the size.  Every level's node totals add up to
    the root's, a parent's left sum is its left child's total (all exact: the sums are
    integers), the prefix counts match the rows that went left, and the node every training
    row was counted into is where the finished trees send its raw values."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    arboretum = arb()
    n = 10_000_000
    X, y = bench.make_rows(n, 0)
    cfg = json.loads(json.dumps(bench.CONFIG))
    data = arboretum.DMatrix(X, y=y)
    model = arboretum.Garden(cfg)
    model.data = data
    depth = cfg["tree"]["max_depth"]
    for _ in range(2):
        model.grow_tree()
        prev = None
        for l in range(depth):
            g = model.level_stats(l)
            nb = g["node_begin"].astype(np.int64)
            assert nb[0] == 0 and nb[-1] == n and (np.diff(nb) >= 0).all()
            if prev is not None:
                pg, pnb = prev
                for k in ("tot_g", "tot_h"):
                    kids = g[k].reshape(-1, 2)
                    assert np.array_equal(kids.sum(axis=1), pg[k])           # children add up
                    assert np.array_equal(kids[:, 0], pg["left_" + k[-1]])   # left child = left sum
                assert np.array_equal(nb[1::2] - nb[0:-1:2], pg["left_count"].astype(np.int64))
                assert np.array_equal(nb[::2], pnb)
            split = g["fid"] >= 0
            assert (g["gain"][split] > 0).all() and (g["gain"][~split] == 0).all()
            prev = (g, nb)
    sl = slice(0, n, 10)  # every tenth row through the fp32 tree walk
    internal = model.train_yhat()[0][sl].astype(np.float64)
    pred_model = arboretum.load(model.dump())
    out = pred_model.predict(arboretum.DMatrix(np.ascontiguousarray(X[sl])))
    assert np.allclose(1.0 / (1.0 + np.exp(-internal)), out, atol=1e-5, rtol=0)


def test_freed_memory_is_kept_and_can_be_released():
    import torch
    from arboretum_b200 import core
    arboretum = arb()
    core.release_cached_memory()
    free0 = torch.cuda.mem_get_info()[0]
    X, y = synth("logistic", 400000, 28, seed=4)
    model = arboretum.train(make_config(1, 6), arboretum.DMatrix(X, y=y), 2)
    first = model.dump()
    del model
    kept = free0 - torch.cuda.mem_get_info()[0]
    assert kept > 50 * 2 ** 20  # the freed blocks stay with the pool ...
    again = arboretum.train(make_config(1, 6), arboretum.DMatrix(X, y=y), 2).dump()
    assert again == first  # ... a second model is built from them, to the same trees ...
    core.release_cached_memory()
    assert free0 - torch.cuda.mem_get_info()[0] < kept / 4  # ... and the driver gets them back on request


_OVERLAP_JOB = """
import hashlib, json, sys
import numpy as np
import arboretum_b200 as arboretum
rng = np.random.default_rng(77)
n, F = 1500000, 28
X = rng.standard_normal((n, F)).astype(np.float32)
w = rng.standard_normal(F)
y = (X @ w + rng.standard_normal(n) > 0).astype(np.float32)
cfg = {"objective": 1, "method": 1,
       "internals": {"double_precision": True, "compute_overlap": 2, "seed": 0,
                     "use_hist_subtraction_trick": True, "upload_features": True, "hist_size": 255},
       "verbose": {"gpu": False, "booster": False, "data": False},
       "tree": {"eta": 0.3, "max_depth": 8, "lambda": 1.0, "alpha": 0.0, "min_child_weight": 1.0,
                "min_leaf_size": 1, "colsample_bytree": 1.0, "colsample_bylevel": 1.0}}
model = arboretum.train(cfg, arboretum.DMatrix(X, y=y), 12)
h = hashlib.sha256(model.dump().encode())
h.update(np.ascontiguousarray(model.predict(arboretum.DMatrix(X[:100000]))).tobytes())
print("digest", h.hexdigest())
"""


def test_overlapped_launches_give_the_same_model():
    """The level kernels are launched so that each may start while the one before it drains
    and waits for it before touching global memory.  A kernel that read too early would
    change a sum somewhere in 12 rounds over 1.5 M rows: the model must be identical, byte
    for byte, to the one built with plain stream-ordered launches."""
    import subprocess
    import sys
    arb()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    digests = []
    for plain in (False, True, False):
        env = dict(os.environ)
        env.pop("ARBORETUM_NO_LAUNCH_OVERLAP", None)
        if plain:
            env["ARBORETUM_NO_LAUNCH_OVERLAP"] = "1"
        out = subprocess.run([sys.executable, "-c", _OVERLAP_JOB], cwd=root, env=env, check=True,
                             capture_output=True, text=True, timeout=600).stdout
        digests.append([l for l in out.splitlines() if l.startswith("digest")][0])
    assert digests[0] == digests[1] == digests[2]


def test_tma_row_gather_gives_the_same_model():
    """With ARBORETUM_TMA_GATHER=1 the uint8 histogram kernel fetches the rows of a node
    through the TMA unit below the root (four rows per gather instruction, completion on a
    per-warp mbarrier) instead of with cp.async.  Both must build the same model, byte for
    byte, on a large matrix and on a small one (few rows per node, most CTAs idle)."""
    import subprocess
    import sys
    arb()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for job in (_OVERLAP_JOB, _OVERLAP_JOB.replace("n, F = 1500000, 28", "n, F = 20000, 28")):
        digests = []
        for tma in (False, True):
            env = dict(os.environ)
            env.pop("ARBORETUM_TMA_GATHER", None)
            if tma:
                env["ARBORETUM_TMA_GATHER"] = "1"
            out = subprocess.run([sys.executable, "-c", job], cwd=root, env=env, check=True,
                                 capture_output=True, text=True, timeout=600).stdout
            digests.append([l for l in out.splitlines() if l.startswith("digest")][0])
        assert digests[0] == digests[1]


def test_bad_calls_return_errors():
    arboretum = arb()
    X, y = synth("linear", 100, 4, seed=1)
    with pytest.raises(arboretum.ArboretumError):
        arboretum.train(make_config(0, 3, colsample_bytree=0.01), arboretum.DMatrix(X, y=y), 1)
    with pytest.raises(arboretum.ArboretumError):
        arboretum.train(make_config(0, 3), arboretum.DMatrix(X), 1)  # no labels


# ---------------------------------------------------------------------------------
# out-of-core: row chunks streamed from pinned host memory
# ---------------------------------------------------------------------------------
@pytest.mark.parametrize("resident", [0, 1, -1])
@pytest.mark.parametrize("kind,objective", [("logistic", 1), ("linear", 0)])
def test_out_of_core_chunks_give_identical_trees(resident, kind, objective):
    """Histograms are exact integer sums, so cutting the rows into streamed chunks
    must not change a single bit of the model."""
    arboretum = arb()
    X, y = synth(kind, 30011, 28, seed=31)
    base = make_config(objective, 6)
    ref = arboretum.train(base, arboretum.DMatrix(X, y=y), 4)
    cfg = make_config(objective, 6)
    cfg["internals"]["chunk_rows"] = 7000
    cfg["internals"]["resident_chunks"] = resident
    data = arboretum.DMatrix(X, y=y)
    model = arboretum.train(cfg, data, 4)
    assert json.loads(model.dump())["model"] == json.loads(ref.dump())["model"]
    assert np.array_equal(model.train_yhat(), ref.train_yhat())
    assert (model.level_stats(3)["node_begin"] == ref.level_stats(3)["node_begin"]).all()


def test_out_of_core_prebinned_input():
    arboretum = arb()
    rng = np.random.default_rng(77)
    n, F = 40000, 100  # the pre-binned configuration's shape: 100 uint8 features
    bins = rng.integers(0, 255, size=(n, F)).astype(np.uint8)
    active = rng.choice(F, 10, replace=False)
    logit = ((bins[:, active] / 255.0 - 0.5) * rng.normal(0, 2, 10)).sum(axis=1)
    y = (rng.random(n) < 1 / (1 + np.exp(-logit))).astype(np.float32)
    base = make_config(1, 5)
    ref = arboretum.train(base, arboretum.DMatrix(bins, y=y, binned_hist_size=255), 3)
    cfg = make_config(1, 5)
    cfg["internals"]["chunk_rows"] = 9000
    cfg["internals"]["resident_chunks"] = 1
    ooc = arboretum.train(cfg, arboretum.DMatrix(bins, y=y, binned_hist_size=255), 3)
    assert json.loads(ooc.dump())["model"] == json.loads(ref.dump())["model"]
    o = orc.Oracle(base, missing_bin=True)
    thr = np.tile(np.arange(255, dtype=np.float32) + 0.5, (F, 1))
    o.set_binned(bins.T.astype(np.uint16), thr, np.full(F, 255, dtype=np.int32)).set_y(y).grow(3)
    got, exp = json.loads(ref.dump())["model"], o.model_dict()
    for a, b in zip(got, exp):
        assert [nd.get("fid") for nd in a["nodes"]] == [nd.get("fid") for nd in b["nodes"]]
        assert np.allclose(a["weights"], b["weights"], rtol=1e-4, atol=1e-6)


def test_sampled_columns_with_row_counts():
    """min_leaf_size > 1 with a (gradient, hessian) objective keeps a second histogram of row
    counts; with sampled columns both histograms run over the side-by-side copy."""
    X, y = synth("logistic", 12000, 70, seed=21)
    cfg = make_config(1, 5, colsample_bytree=0.4, min_leaf_size=40)
    cfg["internals"]["seed"] = 5
    compare_with_oracle(cfg, X, y, 3)


def test_out_of_core_with_two_byte_bins():
    """hist_size >= 256 makes the bins uint16; 20 columns are 40 bytes of a 64-byte padded row,
    so the host rows go without the padding."""
    arboretum = arb()
    X, y = synth("linear", 20000, 20, seed=8)
    base = make_config(0, 5, hist_size=400)
    ref = arboretum.train(base, arboretum.DMatrix(X, y=y), 3)
    cfg = make_config(0, 5, hist_size=400)
    cfg["internals"]["chunk_rows"] = 6000
    cfg["internals"]["resident_chunks"] = 1
    ooc = arboretum.train(cfg, arboretum.DMatrix(X, y=y), 3)
    assert json.loads(ooc.dump())["model"] == json.loads(ref.dump())["model"]
    assert np.array_equal(ooc.train_yhat(), ref.train_yhat())


@pytest.mark.parametrize("F", [100, 27, 64])
def test_out_of_core_prebinned_rows_from_device_memory(F):
    """Pre-binned rows handed over in device memory and trained out of core: the rows go to
    pinned host memory (without the padding to 32 bytes where that is an eighth of a row or
    more: 100 and 27 columns; with it for 64) and come back chunk by chunk.  Same trees as
    the matrix held in HBM."""
    import torch
    arboretum = arb()
    rng = np.random.default_rng(F)
    n = 30000
    bins = rng.integers(0, 255, size=(n, F)).astype(np.uint8)
    active = rng.choice(F, 8, replace=False)
    logit = ((bins[:, active] / 255.0 - 0.5) * rng.normal(0, 2, 8)).sum(axis=1)
    y = (rng.random(n) < 1 / (1 + np.exp(-logit))).astype(np.float32)
    d_bins = torch.from_numpy(bins).cuda()
    d_y = torch.from_numpy(y).cuda()
    base = make_config(1, 5)
    ref = arboretum.train(base, arboretum.DMatrix(bins, y=y, binned_hist_size=255), 3)
    cfg = make_config(1, 5)
    cfg["internals"]["chunk_rows"] = 7000
    cfg["internals"]["resident_chunks"] = 1
    data = arboretum.DMatrix.from_device_bins(d_bins.data_ptr(), n, F, 255, d_y.data_ptr())
    ooc = arboretum.train(cfg, data, 3)
    assert json.loads(ooc.dump())["model"] == json.loads(ref.dump())["model"]
    assert np.array_equal(ooc.train_yhat(), ref.train_yhat())


def test_a_wait_on_a_peer_that_never_answers_gives_up():
    """The exchange kernels between row shards wait for their peers with a time limit.  Here the
    same wait runs on a word that nothing sets: it gives up after the limit, the kernel returns
    normally, the status says so, and the device goes on working."""
    import ctypes
    from arboretum_b200 import core
    timed_out, waited = ctypes.c_int(-1), ctypes.c_double(0)
    assert core.lib().APeerWaitProbe(50.0, ctypes.byref(timed_out), ctypes.byref(waited)) is None
    assert timed_out.value == 1
    assert 45.0 <= waited.value < 1000.0
    assert core.shared_atomic_peak(50) > 0  # the context is intact


def test_matrix_and_targets_from_device_memory():
    """A float32 matrix and targets that already live on the GPU (anything with
    __cuda_array_interface__) train to the same model as the same values from host memory."""
    import torch
    arboretum = arb()
    X, y = synth("logistic", 20000, 12, seed=3)
    cfg = make_config(1, 5)
    host = arboretum.train(cfg, arboretum.DMatrix(X, y=y), 3).dump()
    Xd, yd = torch.from_numpy(X).cuda(), torch.from_numpy(y).cuda()
    dev = arboretum.train(cfg, arboretum.DMatrix(Xd, y=yd), 3).dump()
    assert dev == host
