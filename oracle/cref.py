"""ctypes loader for the C restatement (oracle/lloyd_ref.c).  TEST INFRASTRUCTURE."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liblloyd_ref.so")


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])
    return _SO


def load():
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(os.path.join(_HERE, "lloyd_ref.c")):
        build()
    return ctypes.CDLL(_SO)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def step(X, C_old):
    """One iteration in C.  Returns (C_new float64, labels int32, counts int64, n_moved)."""
    lib = load()
    X = np.ascontiguousarray(X)
    suf = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}[X.dtype]
    n, d = X.shape
    C_old = np.ascontiguousarray(C_old, dtype=np.float64)
    k = C_old.shape[0]
    C_new = np.empty((k, d), np.float64)
    labels = np.empty(n, np.int32)
    counts = np.empty(k, np.int64)
    fn = getattr(lib, "oracle_step_" + suf)
    fn.restype = ctypes.c_int
    moved = fn(_p(X), ctypes.c_size_t(n), ctypes.c_int(d), _p(C_old), ctypes.c_int(k),
               _p(C_new), _p(labels), _p(counts))
    return C_new, labels, counts, moved


def assign(X, C):
    lib = load()
    X = np.ascontiguousarray(X)
    suf = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}[X.dtype]
    n, d = X.shape
    C = np.ascontiguousarray(C, dtype=np.float64)
    labels = np.empty(n, np.int32)
    best = np.empty(n, np.float64)
    fn = getattr(lib, "oracle_assign_" + suf)
    fn.restype = None
    fn(_p(X), ctypes.c_size_t(n), ctypes.c_int(d), _p(C), ctypes.c_int(C.shape[0]), _p(labels), _p(best))
    return labels, best


def transform(X, C):
    lib = load()
    X = np.ascontiguousarray(X)
    suf = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}[X.dtype]
    n, d = X.shape
    C = np.ascontiguousarray(C, dtype=np.float64)
    out = np.empty(n * C.shape[0], np.float64)
    fn = getattr(lib, "oracle_transform_" + suf)
    fn.restype = None
    fn(_p(X), ctypes.c_size_t(n), ctypes.c_int(d), _p(C), ctypes.c_int(C.shape[0]), _p(out))
    return out
