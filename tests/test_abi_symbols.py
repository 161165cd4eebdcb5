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
