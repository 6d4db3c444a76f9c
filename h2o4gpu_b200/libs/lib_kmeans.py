"""ctypes binding of libh2o4gpu_kmeans.so.

Takes the place of the SWIG module the reference loads through
``GPUlib().get()`` (src/interface_py/h2o4gpu/libs/lib_utils.py:34-55,
src/swig/solver/kmeans.i:1-13): the object returned by :func:`get` exposes
``make_ptr_float_kmeans``, ``make_ptr_double_kmeans``, ``kmeans_transform_float``
and ``kmeans_transform_double`` taking numpy arrays the way the SWIG typemaps
do (inputs as contiguous arrays, outputs written into the arrays passed in).

There is no CPU implementation behind this module: if the shared library is
missing or no CUDA device is visible, loading raises.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("H2O4GPU_KM_LIB") or os.path.join(os.path.dirname(_HERE), "lib", "libh2o4gpu_kmeans.so")

_c = ctypes
_sz = _c.c_size_t
_vp = _c.c_void_p


class KMeansLibError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("libh2o4gpu_kmeans: error %d: %s" % (code, msg))
        self.code = code


class Stats(ctypes.Structure):
    _fields_ = [("iterations", _c.c_int), ("n_iter_converged", _c.c_int), ("relocations", _c.c_int),
                ("path", _c.c_int), ("gpu_launches", _c.c_int), ("incremental_iterations", _c.c_int),
                ("last_shift_sq", _c.c_double), ("inertia", _c.c_double),
                ("seconds_upload", _c.c_double), ("seconds_fit", _c.c_double),
                ("ms_assign", _c.c_float), ("ms_update", _c.c_float), ("ms_loop", _c.c_float),
                ("ms_final_assign", _c.c_float), ("refined_rows", _c.c_longlong),
                ("ms_transform", _c.c_float), ("allreduce_path", _c.c_int)]

    def as_dict(self):
        out = {n: getattr(self, n) for n, _ in self._fields_ if not n.startswith("reserved")}
        out["allreduce_path_name"] = {0: "none (one rank)", 1: "one-shot push over peer memory",
                                      2: "ncclAllReduce(int64)"}.get(self.allreduce_path)
        return out


# name -> (restype, argtypes); every symbol include/h2o4gpu_kmeans.h declares extern "C"
SIGNATURES = {
    "kmeans_last_error": (_c.c_char_p, []),
    "kmeans_trim_memory": (_c.c_int, []),
    "kmeans_set_wait_limits": (_c.c_int, [_c.c_double, _c.c_double]),
    "kmeans_selftest_wait_timeout": (_c.c_int, [_c.c_int, _c.c_int, _c.POINTER(_c.c_int)]),
    "kmeans_last_fit_info": (_c.c_int, [_c.POINTER(_c.c_int), _c.POINTER(_c.c_double)]),
    "kmeans_fit_f32": (_c.c_int, [_c.c_int] * 4 + [_sz, _sz, _c.c_int, _c.c_int, _c.c_int, _c.c_float, _vp, _vp, _vp, _vp]),
    "kmeans_fit_f64": (_c.c_int, [_c.c_int] * 4 + [_sz, _sz, _c.c_int, _c.c_int, _c.c_int, _c.c_double, _vp, _vp, _vp, _vp]),
    "kmeans_predict_f32": (_c.c_int, [_c.c_int] * 3 + [_sz, _sz, _c.c_int, _vp, _vp, _vp]),
    "kmeans_predict_f64": (_c.c_int, [_c.c_int] * 3 + [_sz, _sz, _c.c_int, _vp, _vp, _vp]),
    "kmeans_transform_f32": (_c.c_int, [_c.c_int] * 3 + [_sz, _sz, _c.c_int, _vp, _vp, _vp]),
    "kmeans_transform_f64": (_c.c_int, [_c.c_int] * 3 + [_sz, _sz, _c.c_int, _vp, _vp, _vp]),
    "kmeans_free": (None, [_vp]),
    "kmeans_device_count": (_c.c_int, []),
    "kmeans_create": (_c.c_int, [_c.POINTER(_vp), _c.c_int, _c.c_int, _c.POINTER(_c.c_int), _c.c_int, _c.c_int, _vp]),
    "kmeans_destroy": (_c.c_int, [_vp]),
    "kmeans_nccl_unique_id": (_c.c_int, [_vp]),
    "kmeans_attach_device": (_c.c_int, [_vp, _c.c_int, _vp, _sz, _sz, _sz]),
    "kmeans_upload_host": (_c.c_int, [_vp, _vp, _sz, _sz, _c.c_char]),
    "kmeans_set_sample_weight": (_c.c_int, [_vp, _vp, _sz]),
    "kmeans_upload_host_typed": (_c.c_int, [_vp, _vp, _c.c_int, _sz, _sz, _c.c_char]),
    "kmeans_fit_resident": (_c.c_int, [_vp, _c.c_int, _c.c_int, _c.c_double, _vp, _c.c_int]),
    "kmeans_assign_resident": (_c.c_int, [_vp]),
    "kmeans_set_centroids": (_c.c_int, [_vp, _c.c_int, _vp]),
    "kmeans_init_resident": (_c.c_int, [_vp, _c.c_int, _c.c_int, _c.c_int, _vp, _vp]),
    "kmeans_get_centroids": (_c.c_int, [_vp, _vp]),
    "kmeans_get_labels": (_c.c_int, [_vp, _c.c_int, _vp]),
    "kmeans_labels_device": (_c.c_int, [_vp, _c.c_int, _c.POINTER(_vp)]),
    "kmeans_transform_resident": (_c.c_int, [_vp, _c.c_int, _vp, _sz]),
    "kmeans_get_stats": (_c.c_int, [_vp, _c.POINTER(Stats)]),
    "kmeans_inertia": (_c.c_int, [_vp, _c.POINTER(_c.c_double)]),
    "kmeans_centroid_sums_f32": (_c.c_int, [_c.c_int, _vp, _vp, _sz, _sz, _c.c_int, _vp, _vp]),
    "kmeans_centroid_sums_f64": (_c.c_int, [_c.c_int, _vp, _vp, _sz, _sz, _c.c_int, _vp, _vp]),
    "kmeans_centroid_sums_noalloc_f32": (_c.c_int, [_vp, _vp, _sz, _sz, _c.c_int, _vp, _vp, _vp]),
    "kmeans_synth_f32": (_c.c_int, [_c.c_int, _vp, _sz, _sz, _sz, _c.c_int, _vp, _c.c_int, _vp, _c.c_float, _c.c_uint64]),
    "kmeans_synth_f64": (_c.c_int, [_c.c_int, _vp, _sz, _sz, _sz, _c.c_int, _vp, _c.c_int, _vp, _c.c_double, _c.c_uint64]),
}

_cdll = None


def cdll():
    """The raw ctypes library with argtypes set.  Raises if it is not built."""
    global _cdll
    if _cdll is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: build it with `python -m h2o4gpu_b200.build`; "
                              "this package has no CPU implementation" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _cdll = lib
    return _cdll


def check(rc):
    if rc != 0:
        msg = cdll().kmeans_last_error()
        raise KMeansLibError(rc, msg.decode() if msg else "")
    return rc


def _ptr(a):
    return a.ctypes.data_as(_vp)


def _in(a, dtype):
    a = np.ascontiguousarray(a, dtype=dtype)
    return a


class _Module:
    """The callables the reference's Python wrapper uses on its SWIG module."""

    def __init__(self):
        self._lib = cdll()
        if self._lib.kmeans_device_count() < 1:
            raise RuntimeError("no CUDA device visible; this library has no CPU implementation")

    def _fit_predict(self, suffix, dtype, dopredict, verbose, seed, gpu_id, n_gpu, rows, cols, k, max_iter,
                     init_from_data, threshold, srcdata, centroids, pred_centroids, pred_labels):
        X = _in(srcdata, dtype)
        C = _in(centroids, dtype) if np.size(centroids) >= k * cols else None
        if dopredict == 0:
            assert pred_centroids.dtype == dtype and pred_centroids.flags.c_contiguous
            assert pred_labels.dtype == np.int32 and pred_labels.flags.c_contiguous
            pc = _vp(pred_centroids.ctypes.data)
            pl = _vp(pred_labels.ctypes.data)
            fn = getattr(self._lib, "kmeans_fit_" + suffix)
            return check(fn(verbose, seed, gpu_id, n_gpu, rows, cols, k, max_iter, init_from_data, threshold,
                            _ptr(X), _ptr(C) if C is not None else None, ctypes.byref(pc), ctypes.byref(pl)))
        assert pred_labels.dtype == np.int32 and pred_labels.flags.c_contiguous
        pl = _vp(pred_labels.ctypes.data)
        fn = getattr(self._lib, "kmeans_predict_" + suffix)
        return check(fn(verbose, gpu_id, n_gpu, rows, cols, k, _ptr(X), _ptr(C) if C is not None else None,
                        ctypes.byref(pl)))

    def last_fit_info(self):
        """(iterations, inertia) of this thread's last fit through make_ptr_*_kmeans."""
        it = _c.c_int(0)
        inertia = _c.c_double(-1.0)
        check(self._lib.kmeans_last_fit_info(ctypes.byref(it), ctypes.byref(inertia)))
        return it.value, inertia.value

    def make_ptr_float_kmeans(self, *a):
        return self._fit_predict("f32", np.float32, *a)

    def make_ptr_double_kmeans(self, *a):
        return self._fit_predict("f64", np.float64, *a)

    def _transform(self, suffix, dtype, verbose, gpu_id, n_gpu, rows, cols, k, srcdata, centroids, preds):
        X = _in(srcdata, dtype)
        C = _in(centroids, dtype)
        assert preds.dtype == dtype and preds.flags.c_contiguous and preds.size >= rows * k
        pp = _vp(preds.ctypes.data)
        fn = getattr(self._lib, "kmeans_transform_" + suffix)
        return check(fn(verbose, gpu_id, n_gpu, rows, cols, k, _ptr(X), _ptr(C), ctypes.byref(pp)))

    def kmeans_transform_float(self, *a):
        return self._transform("f32", np.float32, *a)

    def kmeans_transform_double(self, *a):
        return self._transform("f64", np.float64, *a)

    def device_count(self):
        return self._lib.kmeans_device_count()


_module = None


def get():
    """Returns the module object, or raises when the library or a GPU is missing."""
    global _module
    if _module is None:
        _module = _Module()
    return _module
