"""B200-native drop-in for the GPU engine of sh1ng/arboretum (hist method)."""
from .core import (ArboretumClassifier, ArboretumError, ArboretumRegression, DMatrix, Garden,
                   build_histogram, lib, load, release_cached_memory, shared_atomic_peak,
                   train)

__all__ = ["ArboretumClassifier", "ArboretumError", "ArboretumRegression", "DMatrix", "Garden",
           "build_histogram", "lib", "load", "release_cached_memory", "shared_atomic_peak", "train"]
