"""The reference's CPU k-means path.  TEST INFRASTRUCTURE, not product code.

``h2o4gpu.KMeans(n_gpus=0, ...)`` builds ``KMeansSklearn(n_clusters, init,
n_init, max_iter, tol, precompute_distances, verbose, random_state, copy_x,
n_jobs, algorithm)`` and forwards fit / predict / transform to it
(src/interface_py/h2o4gpu/solvers/kmeans.py:738-750, 775-814).  ``KMeansSklearn``
is scikit-learn's ``KMeans`` renamed at build time (scripts/prepare_sklearn.sh:30-37).
The two keyword arguments that later scikit-learn releases removed
(``precompute_distances``, ``n_jobs``) are dropped and ``algorithm='auto'|'full'``
maps to ``'lloyd'``.
"""
import time
import warnings

import numpy as np


def _make(n_clusters, init, max_iter, tol, random_state=0):
    from sklearn.cluster import KMeans
    return KMeans(n_clusters=n_clusters, init=init, n_init=1, max_iter=max_iter,
                  tol=tol, verbose=0, random_state=random_state, copy_x=True,
                  algorithm="lloyd")


def fit(X, init, max_iter, tol=0.0, sample_weight=None):
    """Run the reference CPU path from explicit initial centroids (optionally with the
    ``sample_weight`` the wrapper forwards, kmeans.py:800-804).

    Returns a dict with ``centers`` (k x d, dtype of X), ``labels`` (int32),
    ``n_iter`` and ``inertia``.
    """
    X = np.ascontiguousarray(X)
    init = np.ascontiguousarray(init, dtype=X.dtype)
    km = _make(init.shape[0], init, max_iter, tol)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        km.fit(X, sample_weight=sample_weight)
    return {"centers": km.cluster_centers_, "labels": km.labels_.astype(np.int32),
            "n_iter": int(km.n_iter_), "inertia": float(km.inertia_), "model": km}


def timed_fit(X, init, max_iter, tol=0.0):
    """fit() plus its wall time; throughput = n * n_iter / seconds."""
    t0 = time.perf_counter()
    out = fit(X, init, max_iter, tol)
    out["seconds"] = time.perf_counter() - t0
    out["points_iters_per_s"] = X.shape[0] * out["n_iter"] / out["seconds"]
    return out


def _with_centers(centers):
    from sklearn.cluster import KMeans
    centers = np.ascontiguousarray(centers)
    km = KMeans(n_clusters=centers.shape[0], init=centers, n_init=1, max_iter=1)
    km.cluster_centers_ = centers
    km._n_features_out = centers.shape[0]
    km._n_threads = 1
    km.n_features_in_ = centers.shape[1]
    return km


def predict(X, centers):
    """Nearest-centre labels as scikit-learn computes them (ties -> lowest index)."""
    return _with_centers(centers).predict(np.ascontiguousarray(X)).astype(np.int32)


def transform(X, centers):
    """Euclidean (not squared) distances n x k, as sklearn's transform returns."""
    return _with_centers(centers).transform(np.ascontiguousarray(X))


def thread_info():
    import os
    info = {"cpu_count": os.cpu_count()}
    try:
        from threadpoolctl import threadpool_info
        info["pools"] = [{"api": p.get("user_api"), "threads": p.get("num_threads"),
                          "lib": p.get("internal_api")} for p in threadpool_info()]
    except Exception:  # pragma: no cover
        info["pools"] = []
    return info
