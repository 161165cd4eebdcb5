"""B200-native drop-in for the GPU engine of sh1ng/arboretum (hist method)."""
from .core import (ArboretumClassifier, ArboretumError, ArboretumRegression, DMatrix, Garden,
                   build_histogram, lib, load, train)

__all__ = ["ArboretumClassifier", "ArboretumError", "ArboretumRegression", "DMatrix", "Garden",
           "build_histogram", "lib", "load", "train"]
