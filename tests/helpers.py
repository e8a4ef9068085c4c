"""Shared helpers for the tests (package loading, metrics, seeded inputs)."""
import importlib
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
PKG_NAME = "int8-transformer-kernels_b200"


def pkg():
    return importlib.import_module(PKG_NAME)


def ext():
    return pkg().int8_ext


def cabi():
    return pkg().cabi


def cosine(a, b):
    """float64 cosine (validation/validate_int8.py:101-110 uses float64 too)."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    na, nb = np.linalg.norm(a), np.linalg.norm(b)
    if na < 1e-6 and nb < 1e-6:
        return 1.0
    if na < 1e-6 or nb < 1e-6:
        return 0.0
    return float(min(1.0, a @ b / (na * nb)))


def gold(name):
    return np.load(os.path.join(GOLD, name))
