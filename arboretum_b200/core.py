# coding: utf-8
"""Python surface of the B200 build: the same classes, functions, arguments and
error behaviour as the reference's ``python-package/arboretum/core.py`` (DMatrix
:51-120, Garden :123-294, train :297-319, load :322-339, the scikit-learn style
wrappers :342-732), talking to this repository's ``libarboretum.so`` through the
same fourteen C entry points.  There is no CPU path: importing this module
without the built library raises.
"""
import ctypes
import json
import os

import numpy as np

__all__ = ["ArboretumError", "DMatrix", "Garden", "train", "load",
           "ArboretumRegression", "ArboretumClassifier", "lib"]


class ArboretumError(Exception):
    pass


def _load_lib():
    here = os.path.dirname(os.path.abspath(os.path.expanduser(__file__)))
    path = os.path.join(here, "libarboretum.so")
    if not os.path.exists(path):
        raise ImportError(
            "%s is missing: build it with `python arboretum_b200/build.py` "
            "(there is no CPU fallback)" % path)
    lib = ctypes.cdll.LoadLibrary(path)
    for name in ("ACreateFromDenseMatrix", "ASetY", "AInitGarden", "AGrowTree", "APredict",
                 "AFreeDMatrix", "AFreeGarden", "AAppendLastTree", "AGetY", "ADeleteArray",
                 "ASetLabel", "ASetWeights", "ADumpModel", "ALoadModel",
                 # additive entry points of this build
                 "ACreateFromBinnedMatrix", "ASetThresholds", "AQuantize", "AGetTrainY",
                 "AGetLevelStats", "AGetLevelStatsOf", "AGetGradientStep", "APeerWaitProbe", "ASetProfile", "AGetTimings", "ABuildHistogram",
                 "ABuildHistogramFromParents", "ANcclUniqueId", "AInitNccl", "AThresholdsNoAlloc", "ASharedAtomicPeak",
                 "AReleaseCachedMemory"):
        getattr(lib, name).restype = ctypes.c_char_p
    lib.ADumpModel.argtypes = [ctypes.POINTER(ctypes.c_char_p), ctypes.c_void_p]
    lib.AFreeDMatrix.argtypes = [ctypes.c_void_p]
    lib.AFreeGarden.argtypes = [ctypes.c_void_p]
    lib.AGrowTree.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.AAppendLastTree.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.ALoadModel.argtypes = [ctypes.c_char_p, ctypes.c_void_p]
    lib.ASetY.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.ASetLabel.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.ASetWeights.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.APredict.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    lib.AGetY.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.ADeleteArray.argtypes = [ctypes.c_void_p]
    lib.ACreateFromDenseMatrix.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_float,
                                           ctypes.c_void_p]
    lib.ACreateFromBinnedMatrix.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_void_p]
    lib.ASetThresholds.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    lib.AQuantize.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                              ctypes.c_void_p, ctypes.c_void_p]
    lib.AGetTrainY.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.AGetLevelStats.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 9
    lib.AGetLevelStatsOf.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 9
    lib.AGetGradientStep.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_double),
                                     ctypes.POINTER(ctypes.c_double)]
    lib.APeerWaitProbe.argtypes = [ctypes.c_double, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double)]
    lib.ASetProfile.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.AGetTimings.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_char_p)]
    lib.ABuildHistogram.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                                    ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                    ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                    ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.ABuildHistogramFromParents.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                               ctypes.c_void_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 4
    lib.ASharedAtomicPeak.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    lib.AThresholdsNoAlloc.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                       ctypes.c_void_p, ctypes.c_void_p]
    lib.ANcclUniqueId.argtypes = [ctypes.c_void_p]
    lib.AInitNccl.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib


_LIB = _load_lib()


def lib():
    """The loaded C library (for callers that use the additive entry points)."""
    return _LIB


def _call_and_throw_if_error(ret):
    if ret is not None:
        raise ArboretumError(ValueError(ret))


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class DMatrix(object):
    """Data container: dense fp32 features plus ``y`` (regression / binary) or
    ``labels`` (multi-class).  ``binned`` (additive) takes rows that are already
    quantised to uint8 bin ids instead of ``data``."""

    def __init__(self, data, data_category=None, y=None, labels=None, weights=None, missing=0.0,
                 binned_hist_size=None):
        self.labels_count = 1
        self.rows = data.shape[0]
        self.columns = data.shape[1]
        if binned_hist_size is None:
            self._init_from_npy2d(data, missing, category=data_category)
        else:
            self._init_from_binned(data, binned_hist_size)

        if y is not None and labels is not None:
            raise ValueError(
                'y and labels both are not None. Specify labels only for multi label classification')
        if y is not None:
            assert data.shape[0] == (y.shape[0] if hasattr(y, "shape") else len(y))
            self._init_y(y)
        elif labels is not None:
            self.labels_count = int(np.max(labels)) + 1
            assert data.shape[0] == len(labels)
            self._init_labels(labels)

        if weights is not None:
            assert weights.shape[0] == self.rows
            assert weights.size == self.rows
            self._set_weight(weights)

    def __del__(self):
        handle = getattr(self, "handle", None)
        if handle is not None and _LIB is not None:
            _call_and_throw_if_error(_LIB.AFreeDMatrix(handle))
            self.handle = None

    def _set_weight(self, weights):
        data = np.array(weights.reshape(self.rows), dtype=np.float32)
        _call_and_throw_if_error(_LIB.ASetWeights(self.handle, _ptr(data)))

    def _init_from_npy2d(self, mat, missing, category=None):
        if len(mat.shape) != 2:
            raise ValueError('Input numpy.ndarray must be 2 dimensional')
        cai = getattr(mat, "__cuda_array_interface__", None)
        if cai is not None:
            # additive: a C-contiguous float32 matrix that already lives in device memory (torch,
            # cupy, numba ...) is copied device to device; nothing passes through the host
            if cai["typestr"] != "<f4" or cai.get("strides") not in (None, (4 * mat.shape[1], 4)):
                raise ValueError("device matrices must be C-contiguous float32")
            if category is not None and not np.issubdtype(category.dtype, np.integer):
                raise ValueError('Categoty''s type must be int like')
            self.handle = ctypes.c_void_p()
            cat = None if category is None else np.array(category.reshape(category.size), dtype=np.uint32)
            _call_and_throw_if_error(_LIB.ACreateFromDenseMatrix(
                ctypes.c_void_p(cai["data"][0]), _ptr(cat), ctypes.c_int(mat.shape[0]),
                ctypes.c_int(mat.shape[1]), ctypes.c_int(0 if category is None else category.shape[1]),
                ctypes.c_float(missing), ctypes.byref(self.handle)))
            return
        if category is not None and not np.issubdtype(category.dtype, np.integer):
            raise ValueError('Categoty''s type must be int like')
        # no host copy when the caller's matrix is already C-contiguous float32 (the library
        # copies it to the device during this call and does not keep the pointer)
        data = np.ascontiguousarray(mat, dtype=np.float32).reshape(mat.size)
        self.handle = ctypes.c_void_p()
        if category is None:
            data_category = None
            columns = 0
        else:
            columns = category.shape[1]
            data_category = np.array(category.reshape(category.size), dtype=np.uint32)
        _call_and_throw_if_error(_LIB.ACreateFromDenseMatrix(
            _ptr(data), _ptr(data_category), ctypes.c_int(mat.shape[0]), ctypes.c_int(mat.shape[1]),
            ctypes.c_int(columns), ctypes.c_float(missing), ctypes.byref(self.handle)))

    def _init_from_binned(self, mat, hist_size):
        if len(mat.shape) != 2:
            raise ValueError('Input numpy.ndarray must be 2 dimensional')
        data = np.ascontiguousarray(mat, dtype=np.uint8)
        self.handle = ctypes.c_void_p()
        _call_and_throw_if_error(_LIB.ACreateFromBinnedMatrix(
            _ptr(data), ctypes.c_int64(mat.shape[0]), ctypes.c_int(mat.shape[1]),
            ctypes.c_int(hist_size), ctypes.byref(self.handle)))

    def _init_y(self, y):
        cai = getattr(y, "__cuda_array_interface__", None)
        if cai is not None:  # additive: float32 targets in device memory
            if cai["typestr"] != "<f4" or int(np.prod(cai["shape"])) != self.rows:
                raise ValueError("device targets must be %d float32 values" % self.rows)
            _call_and_throw_if_error(_LIB.ASetY(self.handle, ctypes.c_void_p(cai["data"][0])))
            return
        data = np.ascontiguousarray(np.asarray(y).reshape(self.rows), dtype=np.float32)
        _call_and_throw_if_error(_LIB.ASetY(self.handle, _ptr(data)))

    def _init_labels(self, labels):
        data = np.array(np.asarray(labels).reshape(self.rows), dtype=np.uint8)
        _call_and_throw_if_error(_LIB.ASetLabel(self.handle, _ptr(data)))

    # ---- additive helpers -------------------------------------------------------
    @classmethod
    def from_device_bins(cls, bins_ptr, rows, columns, hist_size, y_ptr=None):
        """Rows that are already binned AND already in device memory: ``bins_ptr`` is the
        address of ``rows x columns`` uint8 bin ids (row-major), ``y_ptr`` of ``rows`` float32
        targets (e.g. ``tensor.data_ptr()`` of torch CUDA tensors, which must stay alive
        until this call returns)."""
        self = cls.__new__(cls)
        self.labels_count = 1
        self.rows, self.columns = int(rows), int(columns)
        self.handle = ctypes.c_void_p()
        _call_and_throw_if_error(_LIB.ACreateFromBinnedMatrix(
            ctypes.c_void_p(bins_ptr), ctypes.c_int64(rows), ctypes.c_int(columns),
            ctypes.c_int(hist_size), ctypes.byref(self.handle)))
        if y_ptr is not None:
            _call_and_throw_if_error(_LIB.ASetY(self.handle, ctypes.c_void_p(y_ptr)))
        return self

    def set_thresholds(self, thresholds, sizes):
        """Use thresholds computed elsewhere ([columns][hist_size], bins in use)."""
        thr = np.ascontiguousarray(thresholds, dtype=np.float32)
        size = np.ascontiguousarray(sizes, dtype=np.int32)
        assert thr.shape[0] == self.columns and size.size == self.columns
        _call_and_throw_if_error(_LIB.ASetThresholds(self.handle, _ptr(thr), _ptr(size),
                                                     ctypes.c_int(thr.shape[1])))

    def quantize(self, hist_size=255, missing_bin=True, want_bins=True):
        """Quantise now; returns (thresholds [columns][hist_size], sizes, bins [rows][columns])."""
        thr = np.empty((self.columns, hist_size), dtype=np.float32)
        size = np.empty(self.columns, dtype=np.int32)
        bins = np.empty((self.rows, self.columns), dtype=np.uint16) if want_bins else None
        _call_and_throw_if_error(_LIB.AQuantize(self.handle, hist_size, int(missing_bin), _ptr(thr),
                                                _ptr(size), _ptr(bins)))
        return thr, size, bins


class Garden(object):
    """Low level object to work with arboretum."""

    def __init__(self, config, data=None):
        if isinstance(config, str):  # additive: the reference takes a dict only
            config = json.loads(config)
        self.config = config
        self.data = data
        self._init = False
        if 'labels_count' in config.get('tree', {}):
            self.labels_count = config['tree']['labels_count']
        else:
            self.labels_count = 1
        self.config_str = json.dumps(config)

    def __del__(self):
        handle = getattr(self, "handle", None)
        if handle is not None and _LIB is not None:
            _call_and_throw_if_error(_LIB.AFreeGarden(handle))
            self.handle = None
        if hasattr(self, 'data'):
            del self.data

    def _ensure_init(self):
        if not self._init:
            self.handle = ctypes.c_void_p()
            _call_and_throw_if_error(_LIB.AInitGarden(
                ctypes.c_char_p(self.config_str.encode('UTF-8')), ctypes.byref(self.handle)))
            self._init = True

    def load(self, json_model_str):
        """Load model from json."""
        self._ensure_init()
        _call_and_throw_if_error(_LIB.ALoadModel(
            ctypes.c_char_p(json_model_str.encode('UTF-8')), self.handle))

    def grow_tree(self, grad=None):
        """Grows one boosting round (``labels_count`` trees)."""
        self._ensure_init()
        if grad is not None:
            assert len(grad) == self.data.rows
            data = np.array(grad.reshape(self.data.rows), dtype=np.float32)
            _call_and_throw_if_error(_LIB.AGrowTree(self.handle, self.data.handle, _ptr(data)))
        else:
            _call_and_throw_if_error(_LIB.AGrowTree(self.handle, self.data.handle, None))

    def append_last_tree(self, data):
        """Adds the last round's trees to the prediction kept for ``data``."""
        _call_and_throw_if_error(_LIB.AAppendLastTree(self.handle, data.handle))

    def _take(self, preds, length):
        if self.labels_count == 1:
            res = np.copy(np.ctypeslib.as_array(preds, shape=(length,)))
        else:
            res = np.copy(np.ctypeslib.as_array(preds, shape=(length, self.labels_count)))
        _call_and_throw_if_error(_LIB.ADeleteArray(preds))
        return res

    def get_y(self, data):
        """Prediction accumulated by ``append_last_tree`` calls."""
        preds = ctypes.POINTER(ctypes.c_float)()
        _call_and_throw_if_error(_LIB.AGetY(self.handle, data.handle, ctypes.byref(preds)))
        return self._take(preds, int(data.rows))

    def predict(self, data, n_rounds=-1):
        """Predict with the first ``n_rounds`` trees (-1: all)."""
        preds = ctypes.POINTER(ctypes.c_float)()
        _call_and_throw_if_error(_LIB.APredict(self.handle, data.handle, ctypes.byref(preds),
                                               n_rounds))
        return self._take(preds, int(data.rows))

    def dump(self):
        """Dumps the model as a json string."""
        json_p = ctypes.c_char_p()
        _call_and_throw_if_error(_LIB.ADumpModel(ctypes.byref(json_p), self.handle))
        return json_p.value.decode('utf-8')

    # ---- additive helpers -------------------------------------------------------
    def train_yhat(self):
        """Training-time predictions (internal scale), shape [labels][rows]."""
        out = np.empty((self.labels_count, self.data.rows), dtype=np.float32)
        _call_and_throw_if_error(_LIB.AGetTrainY(self.handle, _ptr(out)))
        return out

    def level_stats(self, level, tree_in_round=-1):
        """Split records of one level of a tree of the last round (-1: the last tree grown;
        multi:softmax grows ``labels_count`` trees per round, numbered from 0)."""
        L = 1 << level
        out = {"node_begin": np.empty(L + 1, dtype=np.uint32), "gain": np.empty(L, dtype=np.float32),
               "fid": np.empty(L, dtype=np.int32), "bin": np.empty(L, dtype=np.int32),
               "left_g": np.empty(L), "left_h": np.empty(L), "tot_g": np.empty(L),
               "tot_h": np.empty(L), "left_count": np.empty(L, dtype=np.uint32)}
        _call_and_throw_if_error(_LIB.AGetLevelStatsOf(
            self.handle, int(tree_in_round), level, *[_ptr(out[k]) for k in ("node_begin", "gain", "fid", "bin", "left_g",
                                                         "left_h", "tot_g", "tot_h", "left_count")]))
        return out

    def gradient_step(self):
        """(gradient step, hessian step) of the last round's fixed-point representation."""
        g, h = ctypes.c_double(0), ctypes.c_double(0)
        _call_and_throw_if_error(_LIB.AGetGradientStep(self.handle, ctypes.byref(g), ctypes.byref(h)))
        return g.value, h.value

    def set_profile(self, on=True):
        self._ensure_init()
        _call_and_throw_if_error(_LIB.ASetProfile(self.handle, int(on)))

    def timings(self):
        p = ctypes.c_char_p()
        _call_and_throw_if_error(_LIB.AGetTimings(self.handle, ctypes.byref(p)))
        return json.loads(p.value.decode('utf-8'))


def train(config, data, num_round):
    """Train ``num_round`` boosting rounds on ``data``; returns the Garden."""
    model = Garden(config)
    model.data = data
    model.labels_count = data.labels_count
    for _ in range(num_round):
        model.grow_tree(None)
    return model


def load(json_model_str):
    """Rebuild a model from the string ``Garden.dump`` returned."""
    json_model = json.loads(json_model_str)
    config = json_model['configuration']
    model = Garden(config)
    model.load(json_model_str)
    return model


def release_cached_memory():
    """Hand the device memory the library has freed but kept (its pool) back to the driver."""
    _call_and_throw_if_error(_LIB.AReleaseCachedMemory())


def shared_atomic_peak(steps=2000):
    """(g, h) pair updates per second of the histogram kernels' shared-memory reductions alone
    (``ASharedAtomicPeak``): the ceiling the histogram pass is measured against."""
    out = ctypes.c_double(0)
    _call_and_throw_if_error(_LIB.ASharedAtomicPeak(int(steps), ctypes.byref(out)))
    return out.value


def build_histogram(bins, grad, hist_size, rowid=None, node_begin=None, quant_bits=17, reps=0,
                    parents=None):
    """One histogram launch (kernel-level entry point ``ABuildHistogram``).

    bins: [rows][columns] uint8/uint16; grad: [rows] or [rows][2] float32.
    Returns (sum_g, sum_h) as [nodes][columns][hist_size + 1] doubles and, when
    ``reps`` > 0, the mean device time of one launch in milliseconds.
    ``parents`` = (sum_g, sum_h) of the nodes' parents switches the subtraction trick on
    (``ABuildHistogramFromParents``): only the smaller child of every pair is scanned.
    """
    bins = np.ascontiguousarray(bins)
    assert bins.dtype in (np.uint8, np.uint16)
    n, F = bins.shape
    grad = np.ascontiguousarray(grad, dtype=np.float32)
    pair = int(grad.ndim == 2)
    if node_begin is None:
        node_begin = np.array([0, n], dtype=np.uint32)
    node_begin = np.ascontiguousarray(node_begin, dtype=np.uint32)
    if rowid is not None:
        rowid = np.ascontiguousarray(rowid, dtype=np.uint32)
    nn = node_begin.size - 1
    og = np.zeros((nn, F, hist_size + 1))
    oh = np.zeros((nn, F, hist_size + 1))
    ms = ctypes.c_float(0)
    if parents is not None:
        pg = np.ascontiguousarray(parents[0], dtype=np.float64)
        ph = np.ascontiguousarray(parents[1], dtype=np.float64)
        assert pg.shape == (nn // 2, F, hist_size + 1) and ph.shape == pg.shape
        _call_and_throw_if_error(_LIB.ABuildHistogramFromParents(
            _ptr(bins), bins.dtype.itemsize, n, F, hist_size, _ptr(grad), pair, _ptr(rowid),
            _ptr(node_begin), nn, quant_bits, _ptr(pg), _ptr(ph), _ptr(og), _ptr(oh)))
        return og, oh
    _call_and_throw_if_error(_LIB.ABuildHistogram(
        _ptr(bins), bins.dtype.itemsize, n, F, hist_size, _ptr(grad), pair, _ptr(rowid),
        _ptr(node_begin), nn, quant_bits, _ptr(og), _ptr(oh), reps, ctypes.byref(ms)))
    return (og, oh, ms.value) if reps > 0 else (og, oh)


class _SklearnBase(object):
    _objective = 0

    def __init__(self, max_depth=6, learning_rate=0.1, n_estimators=100, verbosity=1,
                 gamma_absolute=0.0, gamma_relative=0.0, min_child_weight=1.0, min_leaf_size=0,
                 max_leaf_weight=0.0, colsample_bytree=0.8, colsample_bylevel=1.0, l1=1.0, l2=1.0,
                 scale_pos_weight=1.0, initial_y=0.5, seed=0, double_precision=False,
                 method='hist', hist_size=255, **kwargs):
        # key set and defaults of core.py:398-430 (regression) / :571-603 (classifier)
        config = {'objective': self._objective,
                  'method': 1 if method == 'hist' else 0,
                  'internals': {'double_precision': double_precision, 'compute_overlap': 2,
                                'use_hist_subtraction_trick': True, 'dynamic_parallelism': True,
                                'upload_features': True, 'hist_size': hist_size, 'seed': seed},
                  'verbose': {'gpu': verbosity > 0, 'booster': verbosity > 0, 'data': verbosity > 0},
                  'tree': {'eta': learning_rate, 'max_depth': max_depth,
                           'gamma_absolute': gamma_absolute, 'gamma_relative': gamma_relative,
                           'min_child_weight': min_child_weight, 'min_leaf_size': min_leaf_size,
                           'colsample_bytree': colsample_bytree,
                           'colsample_bylevel': colsample_bylevel,
                           'max_leaf_weight': max_leaf_weight, 'lambda': l2, 'alpha': l1}}
        self._config = config
        self.n_estimators = n_estimators
        self._garden = Garden(self._config)
        self.verbosity = verbosity

    def _default_metric(self):
        raise NotImplementedError

    def fit(self, X, y=None, eval_set=None, eval_labels=None, early_stopping_rounds=5,
            eval_metric=None):
        """Fit; with ``eval_set`` stop when the metric has not improved for
        ``early_stopping_rounds`` rounds (core.py:435-507)."""
        if eval_metric is None:
            eval_metric = self._default_metric()
        if isinstance(X, DMatrix):
            data = X
        elif isinstance(X, np.ndarray) and isinstance(y, np.ndarray):
            data = DMatrix(X, y=y)
        else:
            raise ctypes.ArgumentError("Only DMatrix and numpy array are supported")
        self._garden.data = data

        eval_data = None
        if eval_set is not None:
            if isinstance(eval_set, DMatrix):
                eval_data = eval_set
            elif isinstance(eval_set, np.ndarray):
                eval_data = DMatrix(eval_set)
            else:
                raise ctypes.ArgumentError("Only DMatrix and numpy array are supported")

        self.best_round = -1
        self.best_score = np.inf
        for i in range(self.n_estimators):
            self._garden.grow_tree()
            if eval_data is not None:
                self._garden.append_last_tree(eval_data)
                pred = self._garden.get_y(eval_data)
                score = eval_metric(eval_labels, pred)
                if score < self.best_score:
                    if self.verbosity > 0:
                        print("improved score {0} {1}->{2}".format(i, self.best_score, score))
                    self.best_score = score
                    self.best_round = i
                if early_stopping_rounds + self.best_round < i:
                    if self.verbosity > 0:
                        print("early stopping at {0} score {1}, use 'best_round' and 'best_score' "
                              "to get it".format(self.best_round, self.best_score))
                    break
        return self

    def predict(self, X, n_rounds=-1):
        if isinstance(X, DMatrix):
            data = X
        elif isinstance(X, np.ndarray):
            data = DMatrix(X)
        else:
            raise ctypes.ArgumentError("Only DMatrix and numpy array are supported")
        return self._garden.predict(data, n_rounds)


class ArboretumRegression(_SklearnBase):
    """Scikit-learn API like implementation for regression."""
    _objective = 0

    def _default_metric(self):
        from sklearn.metrics import mean_squared_error
        return mean_squared_error


class ArboretumClassifier(_SklearnBase):
    """Scikit-learn API like implementation for binary classification."""
    _objective = 1

    def _default_metric(self):
        from sklearn.metrics import roc_auc_score
        return lambda a, b: -roc_auc_score(a, b)
