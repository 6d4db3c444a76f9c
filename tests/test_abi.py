"""The C-ABI library without a GPU: it builds for sm_100a, loads, exports every
symbol the public header declares, and fails loudly (never computes) when no
device is present."""
import ctypes
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "h2o4gpu_kmeans.h")).read()
    c_part = text.split("#ifdef __cplusplus\n} /* extern \"C\" */")[0]
    names = set(re.findall(r"^(?:int|void|const char\*)\s+(\w+)\s*\(", c_part, re.M))
    return names


def test_exports_every_declared_symbol(built_lib):
    from h2o4gpu_b200.libs import lib_kmeans
    names = _declared()
    assert {"kmeans_fit_f32", "kmeans_predict_f64", "kmeans_transform_f32", "kmeans_create",
            "kmeans_fit_resident", "kmeans_free"} <= names
    lib = ctypes.CDLL(built_lib)
    for n in sorted(names):
        assert hasattr(lib, n), n
    assert names == set(lib_kmeans.SIGNATURES), names ^ set(lib_kmeans.SIGNATURES)


def test_reference_header_names_are_exported_with_cxx_linkage(built_lib):
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", built_lib], capture_output=True, text=True).stdout
    for n in ("make_ptr_float_kmeans", "make_ptr_double_kmeans", "kmeans_transform_float", "kmeans_transform_double"):
        assert re.search(r" T _Z\d+%s" % n, out), n


def test_no_device_is_an_error_not_a_fallback(built_lib):
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.cdll()
    if lib.kmeans_device_count() > 0:
        return
    X = np.zeros((8, 2), np.float32)
    pc, pl = ctypes.c_void_p(), ctypes.c_void_p()
    rc = lib.kmeans_fit_f32(0, 0, 0, 1, 8, 2, 2, 3, 0, 0.0, X.ctypes.data_as(ctypes.c_void_p), None,
                            ctypes.byref(pc), ctypes.byref(pl))
    assert rc == -4 and b"no CUDA device" in lib.kmeans_last_error()
    import pytest
    with pytest.raises(RuntimeError):
        lib_kmeans.get()


def test_wrapper_cpu_backend_and_params():
    import h2o4gpu_b200
    X = np.array([[1., 1.], [1., 4.], [1., 0.]])
    m = h2o4gpu_b200.KMeans(n_clusters=2, n_gpus=0, random_state=1234, init=X[:2].copy()).fit(X)
    assert m.cluster_centers_.shape == (2, 2) and len(m.labels_) == 3
    assert m.predict(X).shape == (3,) and m.transform(X).shape == (3, 2)
    os.environ["H2O4GPU_BACKEND"] = "sklearn"
    try:
        m2 = h2o4gpu_b200.KMeans(n_clusters=2)
        assert m2.do_sklearn
    finally:
        del os.environ["H2O4GPU_BACKEND"]
    est = h2o4gpu_b200.KMeansH2O(n_clusters=3, max_iter=7, n_gpus=0)
    p = est.get_params()
    assert p["n_clusters"] == 3 and p["max_iter"] == 7
    est.set_params(n_clusters=4)
    assert est.n_clusters == 4
    import pytest
    with pytest.raises(ValueError):
        est.set_params(bogus=1)
    with pytest.raises(ValueError):
        h2o4gpu_b200.KMeansH2O(init="nonsense")
