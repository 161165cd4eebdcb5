"""CPU-side checks of the boundary: the library loads without a GPU, exports every
symbol that include/arboretum_b200.h declares, and rejects bad input with an error
string instead of crashing (no compute call is made here)."""
import ctypes
import json
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "arboretum_b200.h")).read()
    return sorted(set(re.findall(r"const char \*(A[A-Za-z]+)\(", text)))


def test_reference_abi_is_complete():
    # python-wrapper/arboretum_wrapper.h:4-39
    ref = {"ACreateFromDenseMatrix", "ASetY", "ASetLabel", "ASetWeights", "AInitGarden",
           "AGrowTree", "AAppendLastTree", "AGetY", "APredict", "ADumpModel", "ALoadModel",
           "AFreeDMatrix", "AFreeGarden", "ADeleteArray"}
    assert ref <= set(_declared())


def test_library_exports_every_declared_symbol():
    import arboretum_b200
    lib = arboretum_b200.lib()
    for name in _declared():
        assert hasattr(lib, name), name


def test_errors_are_strings_not_crashes():
    import arboretum_b200
    lib = arboretum_b200.lib()
    h = ctypes.c_void_p()
    assert lib.AInitGarden(b"{not json", ctypes.byref(h)) is not None
    assert b"objective" in lib.AInitGarden(json.dumps({"objective": 7, "method": 1}).encode(),
                                           ctypes.byref(h)).lower()
    assert b"exact" in lib.AInitGarden(json.dumps({"objective": 0, "method": 0}).encode(),
                                       ctypes.byref(h))
    # NULL handles are ignored by the free functions (core.py:147-150 frees unconditionally)
    assert lib.AFreeGarden(None) is None
    assert lib.AFreeDMatrix(None) is None
    assert lib.ADeleteArray(None) is None
    assert lib.ACreateFromDenseMatrix(None, None, 0, 0, 0, ctypes.c_float(0), ctypes.byref(h)) is not None


def test_python_surface_matches_reference():
    import arboretum_b200 as arboretum
    for name in ("DMatrix", "Garden", "train", "load", "ArboretumRegression", "ArboretumClassifier",
                 "ArboretumError"):
        assert hasattr(arboretum, name)
    for name in ("grow_tree", "append_last_tree", "get_y", "predict", "dump", "load"):
        assert hasattr(arboretum.Garden, name)


def _model_json(fid, depth=2):
    nodes = [{"id": 0, "leaf": False, "left": 1, "right": 2, "threshold": 0.5, "fid": fid},
             {"id": 1, "leaf": True, "idx": 0}, {"id": 2, "leaf": True, "idx": 1}]
    cfg = {"objective": 0, "method": 1, "tree": {"max_depth": depth - 1}}
    return cfg, json.dumps({"configuration": cfg, "model": [{"depth": depth, "nodes": nodes,
                                                             "weights": [0.25, -0.25]}]})


def test_loading_a_model_checks_what_inference_would_index():
    """A dumped model is input like any other: a feature id or a depth that the device-side
    tree walk would index out of range is refused when the model is loaded."""
    import arboretum_b200
    lib = arboretum_b200.lib()
    cfg, good = _model_json(1)
    h = ctypes.c_void_p()
    assert lib.AInitGarden(json.dumps(cfg).encode(), ctypes.byref(h)) is None
    assert lib.ALoadModel(good.encode(), h) is None
    out = ctypes.c_char_p()
    assert lib.ADumpModel(ctypes.byref(out), h) is None
    assert json.loads(out.value.decode())["model"][0]["nodes"][0]["fid"] == 1
    for bad in (_model_json(-3)[1], _model_json(70000)[1],
                good.replace('"depth": 2', '"depth": 99'), good.replace('"depth": 2', '"depth": 0')):
        msg = lib.ALoadModel(bad.encode(), h)
        assert msg is not None and (b"range" in msg or b"depth" in msg)
    assert lib.AFreeGarden(h) is None


def test_thresholds_and_histogram_arguments_are_validated():
    import numpy as np
    import arboretum_b200
    lib = arboretum_b200.lib()
    bins = np.zeros((8, 2), dtype=np.uint8)
    grad = np.ones(8, dtype=np.float32)
    og = np.zeros((1, 2, 5))
    oh = np.zeros((1, 2, 5))
    ms = ctypes.c_float(0)

    def call(b, rowid, node_begin, n_nodes=1):
        p = lambda a: None if a is None else a.ctypes.data_as(ctypes.c_void_p)
        return lib.ABuildHistogram(p(b), 1, 8, 2, 4, p(grad), 0, p(rowid), p(node_begin), n_nodes, 17,
                                   p(og), p(oh), 0, ctypes.byref(ms))
    nb = np.array([0, 8], dtype=np.uint32)
    assert b"exceeds" in call(bins, None, np.array([0, 9], dtype=np.uint32))
    assert b"non-decreasing" in call(bins, None, np.array([5, 2, 8], dtype=np.uint32), 2)
    assert b"rowid" in call(bins, np.array([0, 1, 2, 3, 4, 5, 6, 99], dtype=np.uint32), nb)
    too_big = bins.copy()
    too_big[3, 1] = 5
    assert b"bin id" in call(too_big, None, nb)
