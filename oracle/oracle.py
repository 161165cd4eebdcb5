"""ctypes front end of the CPU oracle (``oracle/oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline legs as the checker / the timed CPU port.  The
product package never imports it.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


class GainParams(ctypes.Structure):
    """GainFunctionParameters (src/core/gain.cuh:11-30)."""
    _fields_ = [("min_leaf_size", ctypes.c_uint), ("hess", ctypes.c_float),
                ("gamma_absolute", ctypes.c_float), ("gamma_relative", ctypes.c_float),
                ("lambda_", ctypes.c_float), ("alpha", ctypes.c_float),
                ("max_leaf_weight", ctypes.c_float)]


class Config(ctypes.Structure):
    _fields_ = [("objective", ctypes.c_int), ("depth", ctypes.c_int),
                ("min_child_weight", ctypes.c_float), ("min_leaf_size", ctypes.c_uint),
                ("colsample_bytree", ctypes.c_float), ("colsample_bylevel", ctypes.c_float),
                ("gamma_absolute", ctypes.c_float), ("gamma_relative", ctypes.c_float),
                ("lambda_", ctypes.c_float), ("alpha", ctypes.c_float),
                ("initial_y", ctypes.c_float), ("eta", ctypes.c_float),
                ("max_leaf_weight", ctypes.c_float), ("labels_count", ctypes.c_int),
                ("double_precision", ctypes.c_int), ("seed", ctypes.c_uint),
                ("use_trick", ctypes.c_int), ("hist_size", ctypes.c_int),
                ("missing_bin", ctypes.c_int)]


def build(force=False):
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or \
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "oracle.cpp")):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        f, d, u64, u32 = ctypes.c_float, ctypes.c_double, ctypes.c_uint64, ctypes.c_uint
        gp = ctypes.POINTER(GainParams)
        L.orc_gain_f.restype = f
        L.orc_gain_f.argtypes = [f, f, u64, u64, gp]
        L.orc_gain_d.restype = f
        L.orc_gain_d.argtypes = [d, d, u64, u64, gp]
        L.orc_gain_f2.restype = f
        L.orc_gain_f2.argtypes = [f, f, f, f, u64, u64, gp]
        L.orc_gain_d2.restype = f
        L.orc_gain_d2.argtypes = [d, d, d, d, u64, u64, gp]
        L.orc_weight_f.restype = f
        L.orc_weight_f.argtypes = [f, u32, gp]
        L.orc_weight_d.restype = f
        L.orc_weight_d.argtypes = [d, u32, gp]
        L.orc_weight_f2.restype = f
        L.orc_weight_f2.argtypes = [f, f, u32, gp]
        L.orc_weight_d2.restype = f
        L.orc_weight_d2.argtypes = [d, d, u32, gp]
        L.orc_quantize_column.restype = ctypes.c_int
        L.orc_quantize_column.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.orc_create.restype = ctypes.c_void_p
        L.orc_create.argtypes = [ctypes.POINTER(Config)]
        L.orc_error.restype = ctypes.c_char_p
        L.orc_error.argtypes = [ctypes.c_void_p]
        for name in ("orc_free", "orc_set_y", "orc_set_label", "orc_get_yhat"):
            getattr(L, name).restype = None
        L.orc_free.argtypes = [ctypes.c_void_p]
        L.orc_set_dense.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.orc_set_binned.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                     ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.orc_set_categories.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.orc_get_tree_categories.restype = None
        L.orc_get_tree_categories.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.orc_predict_cat.restype = None
        L.orc_predict_cat.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                      ctypes.c_int, ctypes.c_void_p]
        L.orc_set_y.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.orc_set_label.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.orc_get_bins.restype = None
        L.orc_get_bins.argtypes = [ctypes.c_void_p] * 4
        L.orc_keep_hist.restype = None
        L.orc_keep_hist.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.orc_init.argtypes = [ctypes.c_void_p]
        L.orc_grow.argtypes = [ctypes.c_void_p]
        L.orc_num_trees.argtypes = [ctypes.c_void_p]
        L.orc_get_tree.restype = None
        L.orc_get_tree.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 4
        L.orc_get_level.restype = None
        L.orc_get_level.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 11
        L.orc_get_hist.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 3
        L.orc_get_yhat.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.orc_predict.restype = None
        L.orc_predict.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                  ctypes.c_int, ctypes.c_void_p]
        L.orc_partition_index.restype = None
        L.orc_partition_index.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        L.orc_hist.restype = None
        L.orc_hist.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 3
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def gain_params(min_leaf_size=0, hess=0.0, gamma_absolute=0.0, gamma_relative=0.0,
                lambda_=0.0, alpha=0.0, max_leaf_weight=0.0):
    return GainParams(min_leaf_size, hess, gamma_absolute, gamma_relative, lambda_, alpha,
                      max_leaf_weight)


def quantize_column(col, hist_size, missing_bin=False):
    """Thresholds, number of bins in use and bin ids of one fp32 column."""
    col = np.ascontiguousarray(col, dtype=np.float32)
    thr = np.empty(hist_size, dtype=np.float32)
    bins = np.empty(col.size, dtype=np.uint16)
    size = lib().orc_quantize_column(_p(col), col.size, hist_size, int(missing_bin), _p(thr), _p(bins))
    return thr, size, bins


def partition_index(go_right, seg_begin):
    go_right = np.ascontiguousarray(go_right, dtype=np.uint8)
    seg_begin = np.ascontiguousarray(seg_begin, dtype=np.uint32)
    out = np.empty(go_right.size, dtype=np.uint32)
    lib().orc_partition_index(_p(go_right), _p(seg_begin), seg_begin.size - 1, _p(out))
    return out


def hist(bins, g, h, seg_begin, hw):
    bins = np.ascontiguousarray(bins, dtype=np.uint16)
    g = np.ascontiguousarray(g, dtype=np.float32)
    h = None if h is None else np.ascontiguousarray(h, dtype=np.float32)
    seg_begin = np.ascontiguousarray(seg_begin, dtype=np.uint32)
    nseg = seg_begin.size - 1
    og = np.zeros(nseg * hw)
    oh = np.zeros(nseg * hw)
    oc = np.zeros(nseg * hw, dtype=np.uint32)
    lib().orc_hist(_p(bins), _p(g), _p(h), _p(seg_begin), nseg, hw, _p(og), _p(oh), _p(oc))
    return og, oh, oc


def config_from_dict(config, missing_bin=False):
    """Nested arboretum configuration dict -> oracle Config (defaults param.h:20-60)."""
    tree = config.get("tree", {})
    internals = config.get("internals", {})
    return Config(
        objective=int(config["objective"]), depth=int(tree.get("max_depth", 7)) + 1,
        min_child_weight=tree.get("min_child_weight", 1.0),
        min_leaf_size=int(tree.get("min_leaf_size", 1)),
        colsample_bytree=tree.get("colsample_bytree", 1.0),
        colsample_bylevel=tree.get("colsample_bylevel", 1.0),
        gamma_absolute=tree.get("gamma_absolute", 0.0), gamma_relative=tree.get("gamma_relative", 0.0),
        lambda_=tree.get("lambda", 1.0), alpha=tree.get("alpha", 0.0),
        initial_y=tree.get("initial_y", 0.5), eta=tree.get("eta", 0.3),
        max_leaf_weight=tree.get("max_leaf_weight", 0.0),
        labels_count=int(tree.get("labels_count", 1)),
        double_precision=int(bool(internals.get("double_precision", False))),
        seed=int(internals.get("seed", 0)),
        use_trick=int(bool(internals.get("use_hist_subtraction_trick", True))),
        hist_size=int(internals.get("hist_size", 255)), missing_bin=int(missing_bin))


class Oracle(object):
    """One booster bound to one data set (Garden + DataMatrix of the reference)."""

    def __init__(self, config, missing_bin=False):
        self.cfg = config if isinstance(config, Config) else config_from_dict(config, missing_bin)
        self.h = lib().orc_create(ctypes.byref(self.cfg))
        self.n = 0
        self.F = 0

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_free(self.h)
            self.h = None

    def set_dense(self, X, categories=None):
        """Dense fp32 rows and, optionally, categorical columns (uint32 codes [rows][C]):
        features ``F .. F + C - 1`` of the trees (extension of this build)."""
        X = np.ascontiguousarray(X, dtype=np.float32)
        self.n, self.F = X.shape
        self.C = 0
        if categories is not None:
            categories = np.ascontiguousarray(categories, dtype=np.uint32)
            assert categories.shape[0] == self.n
            self.C = categories.shape[1]
            lib().orc_set_categories(self.h, _p(categories), self.n, self.C)
        lib().orc_set_dense(self.h, _p(X), self.n, self.F)
        return self

    def set_binned(self, bins_fm, mapping, fsize):
        bins_fm = np.ascontiguousarray(bins_fm, dtype=np.uint16)
        self.F, self.n = bins_fm.shape
        mapping = np.ascontiguousarray(mapping, dtype=np.float32)
        fsize = np.ascontiguousarray(fsize, dtype=np.int32)
        lib().orc_set_binned(self.h, _p(bins_fm), self.n, self.F, _p(mapping), _p(fsize))
        return self

    def set_y(self, y):
        y = np.ascontiguousarray(y, dtype=np.float32)
        assert y.size == self.n
        lib().orc_set_y(self.h, _p(y))
        return self

    def set_label(self, labels):
        labels = np.ascontiguousarray(labels, dtype=np.uint8)
        assert labels.size == self.n
        lib().orc_set_label(self.h, _p(labels))
        return self

    def bins(self):
        """(bins [F][n] uint16, thresholds [F][H] float32, bins in use [F])."""
        H = self.cfg.hist_size
        F = self.F + getattr(self, "C", 0)  # categorical columns follow the dense ones
        b = np.empty((F, self.n), dtype=np.uint16)
        m = np.empty((F, H), dtype=np.float32)
        s = np.empty(F, dtype=np.int32)
        lib().orc_get_bins(self.h, _p(b), _p(m), _p(s))
        return b, m, s

    def keep_hist(self, on=True):
        lib().orc_init(self.h)
        lib().orc_keep_hist(self.h, int(on))

    def grow(self, rounds=1):
        for _ in range(rounds):
            if lib().orc_grow(self.h) != 0:
                raise ValueError(lib().orc_error(self.h).decode())
        return self

    def num_trees(self):
        return lib().orc_num_trees(self.h)

    def tree(self, t):
        depth = self.cfg.depth
        nn = (1 << depth) - 1
        fid = np.empty(nn, dtype=np.int32)
        q = np.empty(nn, dtype=np.int32)
        thr = np.empty(nn, dtype=np.float32)
        w = np.empty(1 << (depth - 1), dtype=np.float32)
        lib().orc_get_tree(self.h, t, _p(fid), _p(q), _p(thr), _p(w))
        is_cat = np.empty(nn, dtype=np.int32)
        category = np.empty(nn, dtype=np.uint32)
        lib().orc_get_tree_categories(self.h, t, _p(is_cat), _p(category))
        return {"fid": fid, "quantized": q, "threshold": thr, "weights": w,
                "categorical": is_cat, "category": category}

    def level(self, t, l):
        L = 1 << l
        out = {"node_begin": np.empty(L + 1, dtype=np.uint32),
               "gain": np.empty(L, dtype=np.float32), "gain2": np.empty(L, dtype=np.float32),
               "fid": np.empty(L, dtype=np.int32), "bin": np.empty(L, dtype=np.int32),
               "left_g": np.empty(L), "left_h": np.empty(L), "tot_g": np.empty(L),
               "tot_h": np.empty(L), "left_count": np.empty(L, dtype=np.uint32),
               "abs_g": np.empty(L)}
        lib().orc_get_level(self.h, t, l, *[_p(out[k]) for k in
                                            ("node_begin", "gain", "gain2", "fid", "bin", "left_g",
                                             "left_h", "tot_g", "tot_h", "left_count", "abs_g")])
        return out

    def hist(self, level, fid):
        hw = self.cfg.hist_size + self.cfg.missing_bin
        L = 1 << level
        g = np.empty(L * hw)
        h = np.empty(L * hw)
        c = np.empty(L * hw, dtype=np.uint32)
        rc = lib().orc_get_hist(self.h, level, fid, _p(g), _p(h), _p(c))
        if rc != 0:
            return None
        return g.reshape(L, hw), h.reshape(L, hw), c.reshape(L, hw)

    def yhat(self):
        out = np.empty((self.cfg.labels_count, self.n), dtype=np.float32)
        lib().orc_get_yhat(self.h, _p(out))
        return out

    def predict(self, X, n_rounds=-1, categories=None):
        X = np.ascontiguousarray(X, dtype=np.float32)
        K = self.cfg.labels_count
        out = np.empty(X.shape[0] * K, dtype=np.float32)
        if categories is not None:
            categories = np.ascontiguousarray(categories, dtype=np.uint32)
        lib().orc_predict_cat(self.h, _p(X), _p(categories), X.shape[0], n_rounds, _p(out))
        return out if K == 1 else out.reshape(X.shape[0], K)

    def model_dict(self):
        """The ``model`` part of the reference's dump (json_conversion.h:13-49)."""
        depth = self.cfg.depth
        trees = []
        for t in range(self.num_trees()):
            tr = self.tree(t)
            nodes = []
            first_leaf = (1 << (depth - 1)) - 1
            for i in range((1 << depth) - 1):
                if i < first_leaf:
                    thr = float(tr["threshold"][i])
                    nodes.append({"fid": int(tr["fid"][i]), "id": i, "leaf": False,
                                  "left": 2 * i + 1, "right": 2 * i + 2,
                                  "threshold": None if np.isinf(thr) else thr})
                    if tr["categorical"][i]:
                        nodes[-1]["category"] = int(tr["category"][i])
                else:
                    nodes.append({"id": i, "idx": i - first_leaf, "leaf": True})
            trees.append({"depth": depth, "nodes": nodes,
                          "weights": [float(w) for w in tr["weights"]]})
        return trees
