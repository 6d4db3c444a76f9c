"""Handle-based access to the engine for data resident on the device(s).

Thin Python over the ``kmeans_create`` / ``kmeans_attach_device`` /
``kmeans_fit_resident`` family of include/h2o4gpu_kmeans.h.  Device memory may
come from anywhere (a torch tensor's ``data_ptr()``, cuda-python, ...): only raw
pointers cross the boundary.
"""
import ctypes

import numpy as np

from .libs import lib_kmeans as _lk


class ResidentKMeans(object):
    """One engine handle.

    devices: local CUDA device ids driven by this process.
    rank0 / world_size: position of the first local device among all ranks when
    several processes cooperate (one per GPU); ``nccl_id`` is then the 128-byte
    id from :func:`nccl_unique_id`, identical on every rank.
    """

    def __init__(self, dtype=np.float32, devices=(0,), rank0=0, world_size=None, nccl_id=None):
        self._lib = _lk.cdll()
        self.dtype = np.dtype(dtype)
        if self.dtype not in (np.dtype(np.float32), np.dtype(np.float64)):
            raise ValueError("dtype must be float32 or float64")
        devices = list(devices)
        world_size = len(devices) if world_size is None else world_size
        arr = (ctypes.c_int * len(devices))(*devices)
        h = ctypes.c_void_p()
        idbuf = None
        if nccl_id is not None:
            idbuf = ctypes.create_string_buffer(bytes(nccl_id), 128)
        _lk.check(self._lib.kmeans_create(ctypes.byref(h), 1 if self.dtype == np.float64 else 0, len(devices), arr,
                                          rank0, world_size, idbuf))
        self._h = h
        self.n_local = len(devices)
        self.k = None
        self.cols = None
        self._rows = [0] * len(devices)

    @staticmethod
    def nccl_unique_id():
        buf = ctypes.create_string_buffer(128)
        _lk.check(_lk.cdll().kmeans_nccl_unique_id(buf))
        return buf.raw

    def close(self):
        if getattr(self, "_h", None):
            self._lib.kmeans_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def attach_device(self, local, ptr, rows, cols, n_total=None):
        """Borrow a row-major rows x cols shard at device address ``ptr``."""
        _lk.check(self._lib.kmeans_attach_device(self._h, local, ctypes.c_void_p(ptr), rows, cols,
                                                 rows if n_total is None else n_total))
        self._rows[local] = rows
        self.cols = cols

    def upload(self, X, order=None):
        """Copy a host matrix to the device(s).  Any dtype of ``DTYPE_CODES`` goes down as it is and is
        converted to the handle's dtype on the device; ``order`` 'r' / 'c' forces a layout, None keeps the
        array's own when it is C- or Fortran-contiguous."""
        X = np.asarray(X)
        if X.ndim != 2:
            raise ValueError("X must be two-dimensional")
        if X.dtype == np.bool_:
            X = X.view(np.uint8)
        if X.dtype not in DTYPE_CODES:   # also: non-native byte order
            X = X.astype(self.dtype)
        if order is None:
            order = 'c' if (X.flags.f_contiguous and not X.flags.c_contiguous) else 'r'
        X = np.ascontiguousarray(X) if order == 'r' else np.asfortranarray(X)
        rows, cols = X.shape
        _lk.check(self._lib.kmeans_upload_host_typed(self._h, X.ctypes.data_as(ctypes.c_void_p),
                                                     DTYPE_CODES[X.dtype], rows, cols, order.encode()))
        per, extra = divmod(rows, self.n_local)   # the library's balanced contiguous split
        self._rows = [per + (1 if i < extra else 0) for i in range(self.n_local)]
        self.cols = cols

    def set_sample_weight(self, w):
        """Per-row weights (all local rows, shard after shard) for the next fits and ``inertia()``; None
        restores unit weights."""
        if w is None:
            _lk.check(self._lib.kmeans_set_sample_weight(self._h, None, 0))
            return
        w = np.ascontiguousarray(w, dtype=self.dtype).reshape(-1)
        _lk.check(self._lib.kmeans_set_sample_weight(self._h, w.ctypes.data_as(ctypes.c_void_p), w.shape[0]))

    def fit(self, init, max_iter, threshold=0.0, flags=0):
        init = np.ascontiguousarray(init, dtype=self.dtype)
        self.k = init.shape[0]
        _lk.check(self._lib.kmeans_fit_resident(self._h, self.k, max_iter, float(threshold),
                                                init.ctypes.data_as(ctypes.c_void_p), flags))
        return self

    def init_centroids(self, k, seed=0, method="k-means||", return_rows=False):
        """Initial centroids from the attached data, on the device: "k-means||" (k-means|| rounds, then
        weighted k-means++ over the candidates) or "random" (first k rows of a seeded shuffle)."""
        m = {"random": 0, "k-means||": 1, "k-means++": 1}[method]
        out = np.empty((int(k), self.cols), dtype=self.dtype)
        rows = np.empty(int(k), dtype=np.int64)
        _lk.check(self._lib.kmeans_init_resident(self._h, int(k), int(seed), m, out.ctypes.data_as(ctypes.c_void_p),
                                                 rows.ctypes.data_as(ctypes.c_void_p)))
        return (out, rows) if return_rows else out

    def set_centroids(self, C):
        C = np.ascontiguousarray(C, dtype=self.dtype)
        self.k = C.shape[0]
        _lk.check(self._lib.kmeans_set_centroids(self._h, self.k, C.ctypes.data_as(ctypes.c_void_p)))

    def assign(self):
        _lk.check(self._lib.kmeans_assign_resident(self._h))

    def centroids(self):
        out = np.empty((self.k, self.cols), dtype=self.dtype)
        _lk.check(self._lib.kmeans_get_centroids(self._h, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def labels(self, local=0):
        out = np.empty(self._rows[local], dtype=np.int32)
        _lk.check(self._lib.kmeans_get_labels(self._h, local, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def all_labels(self):
        return np.concatenate([self.labels(i) for i in range(self.n_local)])

    def labels_device_ptr(self, local=0):
        p = ctypes.c_void_p()
        _lk.check(self._lib.kmeans_labels_device(self._h, local, ctypes.byref(p)))
        return p.value

    def transform(self, local=0):
        """Squared distances of one shard, (rows, k), Fortran-ordered."""
        rows = self._rows[local]
        out = np.empty(rows * self.k, dtype=self.dtype)
        _lk.check(self._lib.kmeans_transform_resident(self._h, local, out.ctypes.data_as(ctypes.c_void_p), rows))
        return out.reshape((rows, self.k), order='F')

    def stats(self):
        st = _lk.Stats()
        _lk.check(self._lib.kmeans_get_stats(self._h, ctypes.byref(st)))
        return st.as_dict()

    def inertia(self):
        v = ctypes.c_double()
        _lk.check(self._lib.kmeans_inertia(self._h, ctypes.byref(v)))
        return v.value


DTYPE_CODES = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.float16): 2, np.dtype(np.int8): 3,
               np.dtype(np.uint8): 4, np.dtype(np.int16): 5, np.dtype(np.uint16): 6, np.dtype(np.int32): 7,
               np.dtype(np.uint32): 8, np.dtype(np.int64): 9, np.dtype(np.uint64): 10}

FIT_NO_FINAL_ASSIGN = 1
FIT_FORCE_SIMT = 2
FIT_FORCE_SPLIT = 4
FIT_CHECK_EVERY_ITER = 8
FIT_FULL_SUMS = 16
FIT_PRESPLIT = 32


def centroid_sums(X, labels, k, gpu_id=0):
    """Un-normalised per-cluster sums (float64, k x d) and counts (int64) of a labelled matrix."""
    lib = _lk.cdll()
    X = np.ascontiguousarray(X)
    if X.dtype not in (np.float32, np.float64):
        X = X.astype(np.float32)
    labels = np.ascontiguousarray(labels, dtype=np.int32)
    rows, cols = X.shape
    sums = np.empty((k, cols), np.float64)
    counts = np.empty(k, np.int64)
    fn = lib.kmeans_centroid_sums_f64 if X.dtype == np.float64 else lib.kmeans_centroid_sums_f32
    _lk.check(fn(gpu_id, X.ctypes.data_as(ctypes.c_void_p), labels.ctypes.data_as(ctypes.c_void_p), rows, cols, k,
                 sums.ctypes.data_as(ctypes.c_void_p), counts.ctypes.data_as(ctypes.c_void_p)))
    return sums, counts


def synth_device(ptr, rows, cols, dtype=np.float32, row0=0, kind=0, centers=None, weights=None, sigma=1.0, seed=0,
                 gpu_id=0):
    """Fill device memory at ``ptr`` with one of the benchmark distributions."""
    lib = _lk.cdll()
    dtype = np.dtype(dtype)
    c = None if centers is None else np.ascontiguousarray(centers, dtype=dtype)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=dtype)
    fn = lib.kmeans_synth_f64 if dtype == np.float64 else lib.kmeans_synth_f32
    _lk.check(fn(gpu_id, ctypes.c_void_p(ptr), rows, cols, row0, kind,
                 None if c is None else c.ctypes.data_as(ctypes.c_void_p), 0 if c is None else c.shape[0],
                 None if w is None else w.ctypes.data_as(ctypes.c_void_p), float(sigma), seed))
