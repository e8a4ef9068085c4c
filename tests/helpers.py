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


# ---- the reference's gate-1 metrics, restated in numpy (validation/validate_int8.py:101-165) ----
def top10_overlap(ref, act, max_rows=4096):
    """Mean per-row overlap of the ten largest-|value| indices along the last dimension
    (validate_int8.py:113-129); None when the rows are constant."""
    r = np.asarray(ref, dtype=np.float32).reshape(-1, ref.shape[-1])
    a = np.asarray(act, dtype=np.float32).reshape(-1, act.shape[-1])
    if r.shape[0] > max_rows:
        idx = np.linspace(0, r.shape[0] - 1, max_rows).astype(np.int64)
        r, a = r[idx], a[idx]
    k = min(10, r.shape[-1])
    if float(np.abs(r).std()) < 1e-6:
        return None
    rt = np.argsort(-np.abs(r), axis=-1, kind="stable")[:, :k]
    at = np.argsort(-np.abs(a), axis=-1, kind="stable")[:, :k]
    match = (rt[:, :, None] == at[:, None, :]).any(-1).astype(np.float32).mean()
    return float(match)


def outlier_ratio(ref, act, err_atol=0.1):
    """Fraction of elements whose error exceeds max(atol, 10 % relative), the atol floor scaled
    with the tensor's RMS (validate_int8.py:132-153)."""
    r = np.asarray(ref, dtype=np.float32)
    a = np.asarray(act, dtype=np.float32)
    atol = max(err_atol, 0.05 * float(np.sqrt(np.mean(np.square(r)))))
    tol = np.maximum(0.10 * np.abs(r), atol)
    return float((np.abs(r - a) > tol).mean())


def gate1(ref, act, thr, is_zero_dataset=False):
    """validate_int8.py:264-283: returns (metrics, list of failed conditions)."""
    fails = []
    res = {"nan_inf": bool(np.isfinite(act).all())}
    if not res["nan_inf"]:
        fails.append("NaN/Inf in kernel output")
    res["cosine"] = cosine(ref, act)
    if res["cosine"] < thr["cos_min"]:
        fails.append("cosine %.5f < %s" % (res["cosine"], thr["cos_min"]))
    ov = None if is_zero_dataset else top10_overlap(ref, act)
    res["top10"] = ov
    if ov is not None and ov < thr["top10_min"]:
        fails.append("top10 overlap %.3f < %s" % (ov, thr["top10_min"]))
    res["outlier_ratio"] = outlier_ratio(ref, act)
    if res["outlier_ratio"] > thr["outlier_ratio_max"]:
        fails.append("outlier ratio %.4f > %s" % (res["outlier_ratio"], thr["outlier_ratio_max"]))
    return res, fails


def gate4(ref, act, thr):
    """validate_int8.py:313-327: edge datasets -- no NaN/Inf, zero output for zero input, cosine floor."""
    fails = []
    if not np.isfinite(act).all():
        fails.append("NaN/Inf in edge-case output")
    if thr.get("zero_output"):
        m = float(np.abs(act).max())
        if m > 1e-3:
            fails.append("zeros dataset: |out| max %.5f > 1e-3" % m)
    else:
        c = cosine(ref, act)
        if c < thr.get("edge_cos_min", 0.99):
            fails.append("edge cosine %.5f < %s" % (c, thr.get("edge_cos_min", 0.99)))
    return fails
