"""sklearn-style k-means estimators over the B200 engine.

Mirrors the reference's Python interface for this path
(src/interface_py/h2o4gpu/solvers/kmeans.py): ``KMeansH2O`` (:18-588) calls the
native library, ``KMeans`` (:591-829) selects between it and scikit-learn.
Differences, all deliberate:

* an ndarray ``init`` runs on the GPU (``init_from_data=2``); the reference
  routes it to scikit-learn because its fit ABI drops the centroids argument
  (kmeans.py:713-721, src/gpu/kmeans/kmeans_h2o4gpu.cu:983-986);
* ``inertia_`` and ``n_iter_`` are set by the GPU path (the reference leaves
  ``inertia_`` None, kmeans.py:187), ``n_init > 1`` keeps the run with the
  lowest inertia (the reference ignores ``n_init`` on the GPU, kmeans.py:722-725)
  and ``score`` is computed on the GPU; ``fit(X, sample_weight=w)`` stays on the GPU too
  (the reference hands it to scikit-learn, kmeans.py:800-804);
* when the native library or a GPU is missing and the caller did not ask for
  CPU (``n_gpus=0`` / ``backend='sklearn'``), construction raises instead of
  silently falling back (kmeans.py:768-770 falls back);
* ``precompute_distances`` and ``n_jobs`` are accepted and not forwarded: the
  installed scikit-learn no longer takes them; ``algorithm`` 'auto'/'full' maps
  to 'lloyd'.
"""
import os
import sys

import numpy as np


def _get_data(X):
    """numpy 2-D view of the input (the part of solvers/utils.py:46-96 this path needs)."""
    if hasattr(X, "values") and not isinstance(X, np.ndarray):
        X = X.values
    X = np.asarray(X)
    if X.ndim == 1:
        X = X.reshape(-1, 1)
    if X.ndim != 2:
        raise ValueError("X must be 2-dimensional")
    return X


def _check_data_content(do_check, name, data):
    """solvers/utils.py:144-158: refuse NaN / Inf when do_checks is on."""
    if do_check == 1:
        if not np.isfinite(data).all():
            raise ValueError("%s contains Inf or NaN" % name)


def device_count(n_gpus=-1):
    """(n_gpus, devices) clamped to what is visible (src/interface_py/h2o4gpu/util/gpu.py:14-38)."""
    try:
        from ..libs import lib_kmeans
        devices = lib_kmeans.cdll().kmeans_device_count()
    except Exception:  # library not built / no driver
        devices = 0
    if n_gpus < 0 or n_gpus > devices:
        n_gpus = devices
    return n_gpus, devices


class KMeansH2O(object):
    """K-Means clustering on the GPU(s).

    Same constructor as the reference's ``KMeansH2O`` (kmeans.py:131-148):
    sklearn's arguments plus ``gpu_id``, ``n_gpus`` and ``do_checks``.
    ``init`` may be 'k-means++', 'random' or a (n_clusters, n_features) array.
    """

    def __init__(self, n_clusters=8, init='k-means++', n_init=1, max_iter=300, tol=1e-4,
                 precompute_distances='auto', verbose=0, random_state=None, copy_x=True, n_jobs=1,
                 algorithm='auto', gpu_id=0, n_gpus=-1, do_checks=1):
        if isinstance(tol, np.generic):
            tol = tol.item()
        if isinstance(init, str) and init not in ['random', 'k-means++']:
            raise ValueError("Invalid initialization method. Should be 'k-means++' or 'random' "
                             "but got '%s'." % init)
        self.init = init
        self._n_clusters = n_clusters
        self._gpu_id = gpu_id
        self._n_gpus_requested = n_gpus
        (self.n_gpus, self.devices) = device_count(n_gpus)
        self._max_iter = max_iter
        self.tol = tol
        self._did_sklearn_fit = 0
        self.verbose = verbose
        self.do_checks = do_checks
        self.n_init = n_init
        self.copy_x = copy_x
        self.algorithm = algorithm
        if random_state is None:
            import random
            self.random_state = random.randint(0, 32000)
        else:
            self.random_state = random_state
        self.cluster_centers_ = None
        self.labels_ = None
        self.inertia_ = None
        self.n_iter_ = None
        self.sklearn_model = None
        self.double_precision = 0

    # -- sklearn plumbing ---------------------------------------------------
    @classmethod
    def _get_param_names(cls):
        import inspect
        sig = inspect.signature(cls.__init__)
        return sorted(p.name for p in sig.parameters.values() if p.name != 'self')

    def get_params(self, deep=True):
        out = {}
        for key in self._get_param_names():
            for attr in (key, '_' + key):
                if hasattr(self, attr):
                    out[key] = getattr(self, attr)
                    break
        return out

    def set_params(self, **params):
        valid = self._get_param_names()
        for key, value in params.items():
            if key not in valid:
                raise ValueError('Invalid parameter %s for estimator %s. Check the list of available '
                                 'parameters with `estimator.get_params().keys()`.'
                                 % (key, self.__class__.__name__))
            if key in ('n_clusters', 'gpu_id', 'max_iter'):
                setattr(self, '_' + key, value)
            else:
                setattr(self, key, value)
        return self

    # -- properties of the reference (kmeans.py:566-588) --------------------
    @property
    def n_clusters(self):
        return self._n_clusters

    @n_clusters.setter
    def n_clusters(self, value):
        if value <= 0:
            raise ValueError("Number of clusters must be positive.")
        self._n_clusters = value

    @property
    def gpu_id(self):
        return self._gpu_id

    @gpu_id.setter
    def gpu_id(self, value):
        if value < 0:
            raise ValueError("GPU ID must be non-negative.")
        self._gpu_id = value

    @property
    def max_iter(self):
        return self._max_iter

    @max_iter.setter
    def max_iter(self, value):
        if value <= 0:
            raise ValueError("Number of maximum iterations must be non-negative.")
        self._max_iter = value

    # -- the GPU path ---------------------------------------------------------
    def _load_lib(self):
        """The native module, or None when the caller asked for zero GPUs
        (kmeans.py:539-541).  A missing library or GPU raises."""
        if self._n_gpus_requested == 0:
            return None
        from ..libs import lib_kmeans
        return lib_kmeans.get()

    def _toc(self, data, convert=True):
        if convert and data.dtype != np.float64 and data.dtype != np.float32:
            self._print_verbose(1, "Detected numeric data format which is not supported. "
                                   "Casting to np.float32.")
            data = np.asarray(data, dtype=np.float32)
        if data.dtype == np.float64:
            self.double_precision = 1
        elif data.dtype == np.float32:
            self.double_precision = 0
        return np.ascontiguousarray(data).reshape(-1)

    def _print_verbose(self, level, msg):
        if self.verbose > level:
            print(msg)
            sys.stdout.flush()

    def fit(self, X, y=None, sample_weight=None):
        """Fit on the GPU.  float32 / float64 input goes through the reference's entry points
        (``make_ptr_*_kmeans``); other numeric dtypes and weighted fits - which the reference converts on
        the host or sends to scikit-learn (kmeans.py:508-521, 800-804) - go through the resident engine,
        which converts on the device and carries the weights."""
        X_np = _get_data(X)
        _check_data_content(self.do_checks, "X", X_np)
        if sample_weight is not None or X_np.dtype not in (np.float32, np.float64):
            self._fit_resident(X_np, sample_weight)
        else:
            self._fit(X_np)
        self._did_sklearn_fit = 0
        return self

    def _fit_resident(self, data, sample_weight):
        from .. import engine
        self._load_lib()
        dtype = np.float64 if data.dtype == np.float64 else np.float32
        self.double_precision = int(dtype == np.float64)
        rows, cols = data.shape
        k = min(self._n_clusters, rows)
        ndev = max(1, min(device_count(self.n_gpus)[0], rows))
        total = device_count(-1)[1]
        devices = [(self._gpu_id + i) % total for i in range(ndev)]
        given = isinstance(self.init, np.ndarray) or (not isinstance(self.init, str) and hasattr(self.init, '__array__'))
        if given:
            init = np.ascontiguousarray(np.asarray(self.init), dtype=dtype)
            if init.shape != (self._n_clusters, cols):
                raise ValueError("init has shape %s, expected %s" % (init.shape, (self._n_clusters, cols)))
        h = engine.ResidentKMeans(dtype=dtype, devices=devices)
        try:
            h.upload(data)
            if sample_weight is not None:
                w = np.asarray(sample_weight, dtype=dtype).reshape(-1)
                if w.shape[0] != rows:
                    raise ValueError("sample_weight has %d entries for %d rows" % (w.shape[0], rows))
                h.set_sample_weight(w)
            runs = 1 if given else max(1, int(self.n_init or 1))
            best = None
            for r in range(runs):
                start = init if given else h.init_centroids(
                    k, seed=self.random_state + r, method="k-means||" if self.init == "k-means++" else "random")
                h.fit(start, self._max_iter, threshold=self.tol,
                      flags=engine.FIT_CHECK_EVERY_ITER if self.tol > 0 else 0)
                st = h.stats()
                inertia = h.inertia()
                if best is None or inertia < best[0]:
                    n_iter = st["n_iter_converged"] if st["n_iter_converged"] > 0 else st["iterations"]
                    best = (inertia, n_iter, h.centroids(), h.all_labels())
        finally:
            h.close()
        self.inertia_, self.n_iter_ = best[0], best[1]
        self.cluster_centers_, self.labels_ = best[2], best[3]
        return self.cluster_centers_, self.labels_

    def _fit(self, data):
        lib = self._load_lib()
        c_data = self._toc(data)
        dtype = np.float64 if self.double_precision else np.float32
        rows, cols = data.shape
        k = min(self._n_clusters, rows)
        if isinstance(self.init, np.ndarray) or (not isinstance(self.init, str) and hasattr(self.init, '__array__')):
            init = np.ascontiguousarray(np.asarray(self.init), dtype=dtype)
            if init.shape != (self._n_clusters, cols):
                raise ValueError("init has shape %s, expected %s" % (init.shape, (self._n_clusters, cols)))
            c_init = 2
            centroids = init.reshape(-1)
        else:
            c_init = 1 if self.init == "k-means++" else 0
            centroids = np.empty([], dtype=dtype)
        fn = lib.make_ptr_double_kmeans if self.double_precision else lib.make_ptr_float_kmeans
        # n_init runs from different seeds (one when the start is given), lowest inertia wins
        runs = 1 if c_init == 2 else max(1, int(self.n_init or 1))
        best = None
        for r in range(runs):
            pred_centers = np.zeros(cols * k, dtype=dtype)
            pred_labels = np.zeros(rows, dtype=np.int32)
            fn(0, self.verbose, self.random_state + r, self._gpu_id, self.n_gpus, rows, cols, self._n_clusters,
               self._max_iter, c_init, self.tol, c_data, centroids, pred_centers, pred_labels)
            n_iter, inertia = lib.last_fit_info()
            if best is None or inertia < best[0]:
                best = (inertia, n_iter, pred_centers, pred_labels)
        self.inertia_, self.n_iter_ = best[0], best[1]
        self.cluster_centers_ = np.reshape(best[2], (k, cols))
        self.labels_ = np.reshape(best[3], rows)
        return self.cluster_centers_, self.labels_

    def _validate_centroids(self, X):
        assert self.cluster_centers_ is not None, "Centroids are None. Run fit() first."
        rows = np.shape(X)[0]
        cols = np.shape(X)[1]
        centroids_dim = np.shape(self.cluster_centers_)[1]
        assert cols == centroids_dim, \
            "The dimension of X [%d] and centroids [%d] is not equal." % (cols, centroids_dim)
        return cols, rows

    def _resident_apply(self, X_np, what):
        """predict / transform for input that is not float32 / float64: the matrix goes down in its own
        dtype (converted on the device) through a resident handle."""
        from .. import engine
        self._load_lib()
        dtype = np.float64 if self.double_precision else np.float32
        rows = X_np.shape[0]
        ndev = max(1, min(device_count(self.n_gpus)[0], rows))
        total = device_count(-1)[1]
        h = engine.ResidentKMeans(dtype=dtype, devices=[(self._gpu_id + i) % total for i in range(ndev)])
        try:
            h.upload(X_np)
            h.set_centroids(np.ascontiguousarray(self.cluster_centers_, dtype=dtype))
            if what == "predict":
                h.assign()
                return h.all_labels()
            return np.concatenate([h.transform(i) for i in range(ndev)], axis=0)
        finally:
            h.close()

    def predict(self, X):
        lib = self._load_lib()
        X_np = _get_data(X)
        cols, rows = self._validate_centroids(X_np)
        _check_data_content(self.do_checks, "X", X_np)
        if X_np.dtype not in (np.float32, np.float64):
            return self._resident_apply(X_np, "predict")
        c_X = self._toc(X_np)
        dtype = np.float64 if self.double_precision else np.float32
        centers = np.ascontiguousarray(self.cluster_centers_, dtype=dtype).reshape(-1)
        c_res = np.zeros(rows, np.int32)
        fn = lib.make_ptr_double_kmeans if self.double_precision else lib.make_ptr_float_kmeans
        fn(1, self.verbose, self.random_state, self._gpu_id, self.n_gpus, rows, cols,
           self.cluster_centers_.shape[0], self._max_iter, 0, self.tol, c_X, centers,
           np.empty([], dtype), c_res)
        return c_res

    def transform(self, X, y=None):
        """Squared distances to every centre, shape (n_samples, k) — the GPU
        reference's convention (kmeans.py:389-422; sklearn's transform returns
        the square roots)."""
        lib = self._load_lib()
        X_np = _get_data(X)
        cols, rows = self._validate_centroids(X_np)
        if X_np.dtype not in (np.float32, np.float64):
            return self._resident_apply(X_np, "transform")
        c_X = self._toc(X_np)
        dtype = np.float64 if self.double_precision else np.float32
        k = self.cluster_centers_.shape[0]
        centers = np.ascontiguousarray(self.cluster_centers_, dtype=dtype).reshape(-1)
        c_res = np.zeros(rows * k, dtype)
        fn = lib.kmeans_transform_double if self.double_precision else lib.kmeans_transform_float
        fn(self.verbose, self._gpu_id, self.n_gpus, rows, cols, k, c_X, centers, c_res)
        return np.reshape(c_res, (rows, k), order='F')

    def fit_transform(self, X, y=None, sample_weight=None):
        return self.fit(X, y, sample_weight).transform(X)

    def score(self, X, y=None, sample_weight=None):
        """Opposite of the k-means objective on X (sklearn's convention): minus the (weighted) sum of
        squared distances of the rows to their nearest centre, computed on the GPU."""
        from .. import engine
        self._load_lib()
        X_np = _get_data(X)
        self._validate_centroids(X_np)
        dtype = np.float64 if self.double_precision else np.float32
        h = engine.ResidentKMeans(dtype=dtype, devices=(self._gpu_id,))
        try:
            h.upload(X_np)
            if sample_weight is not None:
                h.set_sample_weight(sample_weight)
            h.set_centroids(np.ascontiguousarray(self.cluster_centers_, dtype=dtype))
            h.assign()
            return -h.inertia()
        finally:
            h.close()

    def fit_predict(self, X, y=None, sample_weight=None):
        return self.fit(X, y, sample_weight).labels_

    # -- CPU re-seeding helpers of the reference (kmeans.py:321-343, 376-387, 424-436)
    def sklearn_fit(self, X, y=None):
        assert self.cluster_centers_ is not None, "Centroids are None. Run fit() first."
        if self._did_sklearn_fit == 0:
            X_np = _get_data(X)
            _check_data_content(self.do_checks, "X", X_np)
            self._did_sklearn_fit = 1
            import sklearn.cluster as sk_cluster
            self.sklearn_model = sk_cluster.KMeans(self.cluster_centers_.shape[0], max_iter=1,
                                                   init=self.cluster_centers_, n_init=1)
            self.sklearn_model.fit(X_np)
            self.sklearn_model.cluster_centers_ = self.cluster_centers_

    def sklearn_predict(self, X, y=None):
        _check_data_content(self.do_checks, "X", np.asarray(X))
        self.sklearn_fit(X)
        return self.sklearn_model.predict(X)

    def sklearn_transform(self, X, y=None):
        _check_data_content(self.do_checks, "X", np.asarray(X))
        self.sklearn_fit(X)
        return self.sklearn_model.transform(X)


class KMeans(object):
    """Backend selector with the reference's rules (kmeans.py:685-773):
    ``backend`` in 'auto' | 'sklearn' | 'h2o4gpu', overridden by the environment
    variable ``H2O4GPU_BACKEND``; ``n_gpus=0`` selects scikit-learn."""

    def __init__(self, n_clusters=8, init='k-means++', n_init=1, max_iter=300, tol=1e-4,
                 precompute_distances='auto', verbose=0, random_state=None, copy_x=True, n_jobs=1,
                 algorithm='auto', gpu_id=0, n_gpus=-1, do_checks=1, backend='auto'):
        os_val = os.environ.get('H2O4GPU_BACKEND')
        if os_val is not None:
            backend = os_val
        assert backend in ['auto', 'sklearn', 'h2o4gpu'], \
            "Invalid backend '%s': must be 'auto', 'sklearn' or 'h2o4gpu'" % backend
        self.backend = backend
        self.do_sklearn = (backend == 'sklearn') or (n_gpus == 0)
        if self.do_sklearn:
            from sklearn.cluster import KMeans as KMeansSklearn
            alg = 'lloyd' if algorithm in ('auto', 'full') else algorithm
            self.model_sklearn = KMeansSklearn(n_clusters=n_clusters, init=init, n_init=n_init,
                                               max_iter=max_iter, tol=tol, verbose=verbose,
                                               random_state=random_state, copy_x=copy_x, algorithm=alg)
            self.model_h2o4gpu = None
            self.model = self.model_sklearn
        else:
            self.model_h2o4gpu = KMeansH2O(n_clusters=n_clusters, init=init, n_init=n_init, max_iter=max_iter,
                                           tol=tol, precompute_distances=precompute_distances, verbose=verbose,
                                           random_state=random_state, copy_x=copy_x, n_jobs=n_jobs,
                                           algorithm=algorithm, gpu_id=gpu_id, n_gpus=n_gpus,
                                           do_checks=do_checks)
            self.model_h2o4gpu._load_lib()  # raises when the library or a GPU is missing
            self.model_sklearn = None
            self.model = self.model_h2o4gpu
        if verbose:
            print("Using %s backend" % ("sklearn" if self.do_sklearn else "h2o4gpu"))

    def fit(self, X, y=None, sample_weight=None):
        res = self.model.fit(X, y, sample_weight)
        self.set_attributes()
        return res

    def fit_predict(self, X, y=None, sample_weight=None):
        res = self.model.fit_predict(X, y, sample_weight)
        self.set_attributes()
        return res

    def fit_transform(self, X, y=None, sample_weight=None):
        res = self.model.fit_transform(X, y, sample_weight)
        self.set_attributes()
        return res

    def get_params(self, deep=True):
        return self.model.get_params(deep)

    def set_params(self, **params):
        return self.model.set_params(**params)

    def predict(self, X, sample_weight=None):
        res = self.model.predict(X)
        self.set_attributes()
        return res

    def transform(self, X):
        res = self.model.transform(X)
        self.set_attributes()
        return res

    def score(self, X, y=None, sample_weight=None):
        return self.model.score(X, y, sample_weight)

    def set_attributes(self):
        for name in ('cluster_centers_', 'labels_', 'inertia_', 'n_iter_'):
            setattr(self, name, getattr(self.model, name, None))
