"""Parity of the CUDA path with the CPU oracle, through the C ABI.

Tolerances (stated by the task for this path): final centroids within 1e-4
relative for float32 and 1e-10 for float64; labels identical except rows whose
two nearest-centre squared distances differ by less than 1e-5 relative, which
are counted.  "Relative" for a centroid table is max|diff| / max|reference|.
"""
import ctypes

import numpy as np
import pytest

from conftest import GOLDEN_CASES, load_golden
from oracle import cref, lloyd

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4
F64_TOL = 1e-10
GAP_REL = 1e-5


def rel_err(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-300))


def check_labels(X, C, got, want, allow_frac=0.0):
    """Mismatches must all be near ties (gap < 1e-5 relative); returns their count."""
    bad = np.flatnonzero(got != want)
    if bad.size == 0:
        return 0
    tie = lloyd.near_tie_mask(X[bad], C, rel=GAP_REL)
    hard = int((~tie).sum())
    assert hard <= allow_frac * X.shape[0], "%d label mismatches outside the near-tie band" % hard
    return int(bad.size)


@pytest.fixture(scope="module")
def eng(built_lib):
    import h2o4gpu_b200.engine as e
    return e


def check_step(X, C_prev, got_C, got_labels, want_C, want_labels, want_moved, relocations, tol=F32_TOL):
    """Labels and centroids of one GPU step against the oracle's step from the same centres.

    Labels may differ only inside the near-tie band.  The centroids are always checked: when the
    labels agree, against the oracle's; when near-tie rows differ, against the oracle's M-step
    (sums, empty-cluster rule, averaging) recomputed from the GPU's labels.  Returns the number
    of near-tie label differences."""
    bad = check_labels(X, C_prev, got_labels, want_labels)
    if bad:
        k = C_prev.shape[0]
        sums, counts = lloyd.sums_counts(X, got_labels, k)
        want_moved = lloyd.relocate_empty(X, got_labels, C_prev, sums, counts, order="descending")
        want_C = lloyd.average(sums, counts)
    assert rel_err(got_C, want_C) < tol
    assert relocations == len(want_moved)
    return bad


def one_step(eng, X, C, flags=0, dtype=None):
    """One Lloyd iteration on the GPU from centres C: (C_new, labels of the E-step)."""
    dtype = X.dtype if dtype is None else dtype
    h = eng.ResidentKMeans(dtype=dtype)
    h.upload(X)
    h.fit(C, 1, flags=flags | eng.FIT_NO_FINAL_ASSIGN)
    out = h.centroids(), h.labels(), h.stats()
    h.close()
    return out


# ---- golden fixtures (scikit-learn = the reference's CPU path) --------------------
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fit_f64(eng, name):
    g = load_golden(name)
    X = g["X"].astype(np.float64)
    init = g["init"].astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float64)
    h.upload(X)
    h.fit(init, int(g["T"]))
    C, lab = h.centroids(), h.labels()
    ref = g["centers_f64"]
    if name.startswith("empty"):
        perm = lloyd.match_centers(ref, C)   # relocated cluster ids may be permuted
        assert rel_err(C[perm], ref) < F64_TOL
        inv = np.empty_like(perm)
        inv[perm] = np.arange(perm.size)
        assert np.array_equal(inv[lab], g["labels_f64"])
        assert h.stats()["relocations"] == 2
    else:
        assert rel_err(C, ref) < F64_TOL
        assert np.array_equal(lab, g["labels_f64"])
    assert abs(h.inertia() / float(g["inertia_f64"]) - 1) < 1e-9
    h.close()


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_fit_f32(eng, name):
    g = load_golden(name)
    X, init = g["X"], g["init"]
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    h.fit(init, int(g["T"]))
    C, lab = h.centroids(), h.labels()
    ref = g["centers_f32"].astype(np.float64)
    want = g["labels_f32"]
    if name.startswith("empty"):
        perm = lloyd.match_centers(ref, C)
        C = C[perm]
        inv = np.empty_like(perm)
        inv[perm] = np.arange(perm.size)
        lab = inv[lab]
    assert rel_err(C, ref) < F32_TOL
    check_labels(X, ref, lab, want)
    h.close()


# ---- reference entry points with host pointers -------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_abi_fit_predict_transform(built_lib, dtype):
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.get()
    g = load_golden("blobs_n2000_d32_k8")
    tag = "f32" if dtype == np.float32 else "f64"
    X = g["X"].astype(dtype)
    init = g["init"].astype(dtype)
    rows, cols = X.shape
    k = init.shape[0]
    centers = np.zeros(k * cols, dtype)
    labels = np.zeros(rows, np.int32)
    fn = lib.make_ptr_float_kmeans if dtype == np.float32 else lib.make_ptr_double_kmeans
    fn(0, 0, 0, 0, 1, rows, cols, k, int(g["T"]), 2, 0.0, X.reshape(-1), init.reshape(-1), centers, labels)
    C = centers.reshape(k, cols)
    ref = g["centers_" + tag].astype(np.float64)
    assert rel_err(C, ref) < (F32_TOL if dtype == np.float32 else F64_TOL)
    check_labels(X, ref, labels, g["labels_" + tag])
    # predict with the oracle's centres
    pl = np.zeros(rows, np.int32)
    fn(1, 0, 0, 0, 1, rows, cols, k, 0, 0, 0.0, X.reshape(-1), g["centers_" + tag].astype(dtype).reshape(-1),
       np.empty([], dtype), pl)
    check_labels(X, ref, pl, g["predict_" + tag])
    # transform: squared, column-major over the whole matrix
    tr = np.zeros(rows * k, dtype)
    tf = lib.kmeans_transform_float if dtype == np.float32 else lib.kmeans_transform_double
    tf(0, 0, 1, rows, cols, k, X.reshape(-1), g["centers_" + tag].astype(dtype).reshape(-1), tr)
    D = tr.reshape((rows, k), order="F")
    want = g["transform_" + tag].astype(np.float64) ** 2
    tol = 1e-4 if dtype == np.float32 else 1e-10
    floor = np.finfo(dtype).eps * ((X[:64].astype(np.float64) ** 2).sum(1)[:, None] + (ref ** 2).sum(1)[None, :])
    assert (np.abs(D[:64] - want) <= tol * want + 8 * floor).all()
    colmajor = lloyd.transform_sq_colmajor(X, ref)
    assert np.abs(tr - colmajor).max() <= tol * colmajor.max()


def test_abi_library_allocates_when_output_null(built_lib):
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.cdll()
    g = load_golden("blobs_n600_d5_k4")
    X, init = g["X"], g["init"]
    pc, pl = ctypes.c_void_p(), ctypes.c_void_p()
    rc = lib.kmeans_fit_f32(0, 0, 0, 1, X.shape[0], X.shape[1], 4, 10, 2, 0.0, X.ctypes.data_as(ctypes.c_void_p),
                            init.ctypes.data_as(ctypes.c_void_p), ctypes.byref(pc), ctypes.byref(pl))
    assert rc == 0 and pc.value and pl.value
    C = np.ctypeslib.as_array(ctypes.cast(pc, ctypes.POINTER(ctypes.c_float)), (4, 5)).copy()
    assert rel_err(C, g["centers_f32"].astype(np.float64)) < F32_TOL
    lib.kmeans_free(pc)
    lib.kmeans_free(pl)


def test_abi_errors(built_lib):
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.cdll()
    X = np.zeros((4, 2), np.float32)
    pc, pl = ctypes.c_void_p(), ctypes.c_void_p()
    rc = lib.kmeans_fit_f32(0, 0, 0, 1, 4, 2, 0, 5, 0, 0.0, X.ctypes.data_as(ctypes.c_void_p), None,
                            ctypes.byref(pc), ctypes.byref(pl))
    assert rc == -1 and b"bad argument" in lib.kmeans_last_error()
    rc = lib.kmeans_fit_f32(0, 0, 0, 1, 4, 2, 2, 5, 2, 0.0, X.ctypes.data_as(ctypes.c_void_p), None,
                            ctypes.byref(pc), ctypes.byref(pl))
    assert rc == -1
    X[1, 1] = np.nan
    rc = lib.kmeans_fit_f32(0, 0, 0, 1, 4, 2, 2, 5, 0, 0.0, X.ctypes.data_as(ctypes.c_void_p), None,
                            ctypes.byref(pc), ctypes.byref(pl))
    assert rc == -6 and b"NaN" in lib.kmeans_last_error()


# ---- the reference's kernel tests, re-expressed -------------------------------------
def test_ref_calculate_centroids_gpu(eng):
    # tests/cpp/gpu/kmeans/test_kmeans_centroids.cu:7-78
    X = np.array([[0, 0], [0, 1], [1, 1], [1, 0]], np.float32)
    sums, counts = eng.centroid_sums(X, np.array([0, 0, 1, 1], np.int32), 2)
    assert np.array_equal(sums, [[0, 1], [2, 1]]) and np.array_equal(counts, [2, 2])


def test_ref_two_shards_add_up_gpu(eng):
    # test_kmeans_centroids.cu:82-251
    Xa = np.array([[4, 2], [1, 0], [4, 0]], np.float32)
    Xb = np.array([[4, 4], [1, 4], [1, 2]], np.float32)
    la, lb = np.array([0, 0, 0], np.int32), np.array([0, 1, 1], np.int32)
    sa, ca = eng.centroid_sums(Xa, la, 2)
    sb, cb = eng.centroid_sums(Xb, lb, 2)
    s, c = eng.centroid_sums(np.vstack([Xa, Xb]), np.r_[la, lb], 2)
    assert np.array_equal(sa + sb, s) and np.array_equal(ca + cb, c)
    assert np.array_equal(s, [[13, 6], [2, 6]])


def test_ref_counts_per_centroid_gpu(eng):
    # tests/cpp/gpu/kmeans/test_kmeans_h2o4gpu.cu:67-174
    X = np.array([[0, 0], [2, 2], [2, 3], [3, 2]], np.float32)
    h = eng.ResidentKMeans()
    h.upload(X)
    h.set_centroids(np.array([[0, 0], [2, 2]], np.float32))
    h.assign()
    assert np.bincount(h.labels(), minlength=2).tolist() == [1, 3]
    P = np.array([[1, 2], [1, 4], [1, 0], [4, 2], [4, 4], [4, 0]], np.float32)
    h.upload(P)
    h.set_centroids(P)
    h.assign()
    assert h.labels().tolist() == [0, 1, 2, 3, 4, 5]
    h.close()


def test_ref_copy_data_orders_gpu(eng):
    # test_kmeans_h2o4gpu.cu:9-65: row- and column-major sources give the same shard
    X = np.arange(9, dtype=np.float32).reshape(3, 3)
    C = np.array([[0, 1, 2], [6, 7, 8]], np.float32)
    for order in ("r", "c"):
        h = eng.ResidentKMeans()
        h.upload(X, order=order)
        h.set_centroids(C)
        h.assign()
        D = h.transform()
        assert np.allclose(D, lloyd.transform_sq_exact(X, C))
        assert h.labels().tolist() == [0, 0, 1]     # row 1 is equidistant: first minimum wins
        h.close()


def test_ref_scaling_and_empty_rule_gpu(eng):
    # test_kmeans_centroids.cu:308-346 (sums/counts) through one full step; and the CPU
    # path's empty rule instead of revert_zeroed_centroids (:253-306)
    X = np.array([[1, 2], [0, 0], [0, 0], [0, 0], [1, 2], [2, 2]], np.float32)
    C0 = np.array([[0.1, 0.1], [1.5, 2.0], [50, 50]], np.float32)
    C, lab, st = one_step(eng, X, C0)
    Cn, labn, _, moved = lloyd.step(X, C0.astype(np.float64), order="descending")
    assert np.array_equal(lab, labn) and st["relocations"] == len(moved) == 1
    assert rel_err(C, Cn) < 1e-6


# ---- teacher-forced parity on the benchmark distributions ---------------------------
CASES = [
    ("c1", dict(n=20000), 6),
    ("c2", dict(n=30000), 5),
    ("c3", dict(n=20000), 3),
    ("c4", dict(n=4000), 4),
    ("c5", dict(n=9000), 2),
]


@pytest.mark.parametrize("cfg,kw,steps", CASES)
def test_teacher_forced_f32(eng, cfg, kw, steps):
    from h2o4gpu_b200 import synth
    X, init, _ = synth.CONFIGS[cfg](**kw)
    C = init.astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    ties = 0
    for _ in range(steps):
        C32 = C.astype(np.float32)
        Cn, labn, _, moved = lloyd.step(X, C32.astype(np.float64), order="descending")
        h.fit(C32, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        got, lab = h.centroids(), h.labels()
        ties += check_step(X, C32.astype(np.float64), got, lab, Cn, labn, moved, h.stats()["relocations"])
        C = Cn
    h.close()
    print("near-tie label differences over the run:", ties)


@pytest.mark.parametrize("cfg,kw,steps", [("c2", dict(n=20000), 8), ("c5", dict(n=6000, k=512), 3),
                                          ("c4", dict(n=3000), 6)])
def test_end_to_end_f64(eng, cfg, kw, steps):
    from h2o4gpu_b200 import synth
    X, init, _ = synth.CONFIGS[cfg](dtype=np.float64, **kw)
    r = lloyd.fit(X, init, steps, dtype=np.float64, center=False, order="descending", stop_on_repeat=False)
    h = eng.ResidentKMeans(dtype=np.float64)
    h.upload(X)
    h.fit(init, steps)
    assert rel_err(h.centroids(), r["centers"]) < F64_TOL
    assert np.array_equal(h.labels(), r["labels"])
    h.close()


def test_fused_and_split_paths_agree_bitwise(eng):
    from h2o4gpu_b200 import synth
    X, init, _ = synth.c1(n=30000)
    a = one_step(eng, X, init)
    b = one_step(eng, X, init, flags=eng.FIT_FORCE_SPLIT)
    assert a[2]["path"] == 1 and b[2]["path"] == 2
    if np.array_equal(a[1], b[1]):
        assert np.array_equal(a[0], b[0])          # integer sums: same labels -> same bits
    else:
        check_labels(X, init.astype(np.float64), a[1], b[1])


def test_deterministic_across_runs(eng):
    from h2o4gpu_b200 import synth
    X, init, _ = synth.c2(n=40000)
    outs = []
    for _ in range(2):
        h = eng.ResidentKMeans()
        h.upload(X)
        h.fit(init, 6)
        outs.append((h.centroids(), h.labels()))
        h.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("dtype,cfg,kw,iters", [(np.float32, "c2", dict(n=60000), 12),
                                                (np.float64, "c2", dict(n=30000), 10),
                                                (np.float32, "c3", dict(n=30000, k=300), 8),
                                                (np.float32, "c5", dict(n=8000, k=512), 6),
                                                # wide rows: a moved row is spread over several warps;
                                                # overlapping blobs keep 0.03-10 % of the labels moving
                                                (np.float32, "wide", dict(n=20011, d=784, k=10, scale=0.15), 10),
                                                (np.float32, "wide", dict(n=3001, d=1000, k=12, scale=0.12), 10)])
def test_incremental_sums_equal_full_recompute_bitwise(eng, dtype, cfg, kw, iters):
    """The M-step that moves only the rows whose label changed gives the same integers as a
    full pass: centroids and labels of every iteration count agree bit for bit."""
    from h2o4gpu_b200 import synth
    if cfg == "wide":
        rng = np.random.default_rng(5)
        centers = kw["scale"] * rng.standard_normal((kw["k"], kw["d"]))
        X = (centers[rng.integers(0, kw["k"], kw["n"])] + rng.standard_normal((kw["n"], kw["d"]))).astype(np.float32)
        init = X[:kw["k"]].copy()
    else:
        X, init, _ = getattr(synth, cfg)(**kw)
    X = X.astype(dtype)
    init = init.astype(dtype)
    outs = []
    for flags in (0, eng.FIT_FULL_SUMS):
        h = eng.ResidentKMeans(dtype=dtype)
        h.upload(X)
        h.fit(init, iters, flags=flags)
        outs.append((h.centroids(), h.labels(), h.stats()))
        h.close()
    assert outs[0][2]["incremental_iterations"] > 0 and outs[1][2]["incremental_iterations"] == 0
    assert outs[0][2]["relocations"] == outs[1][2]["relocations"]
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][1], outs[1][1])


# ---- edge cases ------------------------------------------------------------------------
@pytest.mark.parametrize("n,d,k", [(1, 1, 1), (3, 2, 2), (5, 3, 5), (129, 7, 3), (257, 33, 17), (1000, 130, 20),
                                   (300, 4, 16), (300, 4, 18), (2049, 64, 100), (700, 1030, 6),
                                   # few centroids, wide rows: the chunked tensor-core kernel (d % 4 == 0, d >= 128)
                                   (1000, 132, 5), (257, 784, 16), (3000, 2048, 3), (129, 128, 1), (40000, 200, 10)])
def test_ragged_shapes(eng, n, d, k):
    rng = np.random.default_rng(n * 1000 + d * 10 + k)
    X = rng.standard_normal((n, d)).astype(np.float32) * 3
    init = X[rng.choice(n, k, replace=False)].copy()
    Cn, labn, _, moved = lloyd.step(X, init.astype(np.float64), order="descending")
    C, lab, st = one_step(eng, X, init)
    check_step(X, init.astype(np.float64), C, lab, Cn, labn, moved, st["relocations"])


def test_k_larger_than_rows_is_clamped(built_lib):
    from h2o4gpu_b200 import KMeansH2O
    X = np.array([[0., 0.], [1., 1.], [5., 5.]], np.float32)
    m = KMeansH2O(n_clusters=5, init="random", max_iter=3, random_state=1, n_gpus=1).fit(X)
    assert m.cluster_centers_.shape == (3, 2)      # src/gpu/kmeans/kmeans_h2o4gpu.cu:629-635
    assert sorted(m.labels_.tolist()) == [0, 1, 2]


def test_duplicate_points_more_clusters_than_distinct(eng):
    X = np.repeat(np.array([[1., 2.], [3., 4.]], np.float32), 10, axis=0)
    init = np.array([[1, 2], [3, 4], [9, 9]], np.float32)
    C, lab, st = one_step(eng, X, init)
    Cn, labn, _, moved = lloyd.step(X, init.astype(np.float64), order="descending")
    assert np.array_equal(lab, labn) and st["relocations"] == len(moved) == 0   # max distance is 0: nothing moves
    assert rel_err(C, Cn) < 1e-6                   # the empty cluster copies the largest one


def test_tolerance_stops_early(eng):
    g = load_golden("blobs_n2000_d32_k8")
    h = eng.ResidentKMeans()
    h.upload(g["X"])
    h.fit(g["init"], 50, threshold=1e-3)
    st = h.stats()
    assert 0 < st["iterations"] < 50 and st["last_shift_sq"] < 1e-3
    h.fit(g["init"], 50, flags=eng.FIT_CHECK_EVERY_ITER)
    assert h.stats()["iterations"] == int(g["n_iter_f32"])     # stops when labels repeat, like the CPU path
    h.close()


# ---- estimator -------------------------------------------------------------------------
def test_estimator_matches_cpu_backend(built_lib):
    import h2o4gpu_b200
    g = load_golden("blobs_n2000_d32_k8")
    X, init = g["X"], g["init"]
    gpu = h2o4gpu_b200.KMeans(n_clusters=8, init=init, max_iter=int(g["T"]), tol=0.0, n_gpus=1).fit(X)
    cpu = h2o4gpu_b200.KMeans(n_clusters=8, init=init, max_iter=int(g["T"]), tol=0.0, n_gpus=0).fit(X)
    assert rel_err(gpu.cluster_centers_, cpu.cluster_centers_.astype(np.float64)) < F32_TOL
    check_labels(X, cpu.cluster_centers_.astype(np.float64), gpu.labels_, cpu.labels_)
    assert np.array_equal(gpu.predict(X), gpu.labels_)
    D = gpu.transform(X)
    assert D.shape == (2000, 8)
    assert np.allclose(np.sqrt(D), cpu.transform(X), rtol=1e-3, atol=1e-2)
    # README.md:115-133 shapes (R tests: src/interface_r/tests/testthat/test_model.R:5-22)
    Xs = np.array([[1., 1.], [1., 4.], [1., 0.]])
    m = h2o4gpu_b200.KMeans(n_clusters=2, random_state=1234).fit(Xs)
    assert m.cluster_centers_.shape == (2, 2) and m.predict(Xs).shape == (3,) and m.transform(Xs).shape == (3, 2)


def test_estimator_sklearn_surface(built_lib):
    """inertia_, n_iter_, score and n_init of the GPU estimator against scikit-learn on the same start."""
    import h2o4gpu_b200
    g = load_golden("blobs_n2000_d32_k8")
    X, init = g["X"], g["init"]
    gpu = h2o4gpu_b200.KMeans(n_clusters=8, init=init, max_iter=50, tol=0.0, n_gpus=1).fit(X)
    cpu = h2o4gpu_b200.KMeans(n_clusters=8, init=init, max_iter=50, tol=0.0, n_gpus=0).fit(X)
    assert abs(gpu.inertia_ - cpu.inertia_) <= 1e-4 * cpu.inertia_
    assert gpu.n_iter_ == cpu.n_iter_
    assert abs(gpu.score(X) + gpu.inertia_) <= 1e-6 * gpu.inertia_
    assert abs(gpu.score(X[:500]) - cpu.score(X[:500])) <= 1e-4 * abs(cpu.score(X[:500]))
    # default start (k-means|| on the device), three runs: the best of them is kept
    one = h2o4gpu_b200.KMeans(n_clusters=8, n_init=1, max_iter=20, tol=0.0, random_state=5, n_gpus=1).fit(X)
    three = h2o4gpu_b200.KMeans(n_clusters=8, n_init=3, max_iter=20, tol=0.0, random_state=5, n_gpus=1).fit(X)
    assert three.inertia_ <= one.inertia_ * (1 + 1e-12)
    assert three.cluster_centers_.shape == (8, 32) and np.isfinite(three.cluster_centers_).all()


def test_staged_upload_of_a_pageable_matrix(eng):
    """A pageable matrix above 64 MB goes down through the pinned staging pool (worker threads,
    4 MB pieces): every row must land where it belongs."""
    from h2o4gpu_b200 import synth
    from oracle import lloyd
    X, init, _ = synth.c2(n=300001)            # 76.8 MB, not a multiple of the piece size
    h = eng.ResidentKMeans()
    h.upload(X)
    h.fit(init, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
    lab = h.labels()
    h.set_centroids(np.zeros((1, X.shape[1]), np.float32))
    h.assign()
    total = h.inertia()
    h.close()
    want = lloyd.assign(X, init.astype(np.float64))
    check_labels(X, init.astype(np.float64), lab, want)
    assert abs(total - (X.astype(np.float64) ** 2).sum()) <= 1e-12 * total


def test_bitmap_fed_incremental_sums_in_a_child_process(built_lib):
    """The optional variant that feeds the incremental M-step from the E-step's moved-rows bit map
    (environment switch, read once per process) gives the same bits as the full pass."""
    import os
    import subprocess
    import sys
    code = (
        "import numpy as np\n"
        "from h2o4gpu_b200 import engine, synth\n"
        "X, init, _ = synth.c2(n=60000)\n"
        "outs = []\n"
        "for flags in (0, engine.FIT_FULL_SUMS):\n"
        "    h = engine.ResidentKMeans(); h.upload(X); h.fit(init, 12, flags=flags)\n"
        "    outs.append((h.centroids(), h.labels(), h.stats()['incremental_iterations'])); h.close()\n"
        "assert outs[0][2] > 0 and outs[1][2] == 0\n"
        "assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])\n"
        "print('bitmap ok')\n")
    env = dict(os.environ, H2O4GPU_KM_DELTA_BITMAP="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "bitmap ok" in r.stdout, r.stdout + r.stderr


def test_memory_pool_trim_and_reuse(eng, built_lib):
    """Buffers come from a per-device pool that keeps freed memory; trimming it leaves the library usable."""
    from h2o4gpu_b200 import synth
    from h2o4gpu_b200.libs import lib_kmeans
    X, init, _ = synth.c2(n=40000)
    outs = []
    for rep in range(3):
        h = eng.ResidentKMeans()
        h.upload(X)
        h.fit(init, 4)
        outs.append((h.centroids(), h.labels()))
        h.close()
        if rep == 1:
            assert lib_kmeans.cdll().kmeans_trim_memory() == 0
    assert all(np.array_equal(outs[0][0], o[0]) and np.array_equal(outs[0][1], o[1]) for o in outs[1:])


# ---- several GPUs in one process ------------------------------------------------------
def test_multi_gpu_equals_single_gpu(eng):
    from h2o4gpu_b200.libs import lib_kmeans
    ndev = lib_kmeans.cdll().kmeans_device_count()
    if ndev < 2:
        pytest.skip("one GPU visible")
    from h2o4gpu_b200 import synth
    X, init, _ = synth.c2(n=50001)
    h1 = eng.ResidentKMeans()
    h1.upload(X)
    h1.fit(init, 5)
    h2 = eng.ResidentKMeans(devices=list(range(min(ndev, 4))))
    h2.upload(X)
    h2.fit(init, 5)
    assert h1.stats()["relocations"] == h2.stats()["relocations"] > 0
    assert np.array_equal(h1.centroids(), h2.centroids())      # integer sums: bit-identical
    assert np.array_equal(h1.labels(), h2.all_labels())
    h1.close()
    h2.close()


@pytest.mark.parametrize("n,d,k", [(30001, 128, 300), (20001, 784, 10), (15001, 300, 40), (20001, 50, 100)])
def test_multi_gpu_other_tensor_core_kernels_equal_single_gpu(eng, n, d, k):
    """The streamed-table, wide-row and streaming kernels and the padded copy of unaligned rows, several
    devices driven by one process against one device: centroids and labels bit-identical."""
    from h2o4gpu_b200.libs import lib_kmeans
    ndev = lib_kmeans.cdll().kmeans_device_count()
    if ndev < 2:
        pytest.skip("one GPU visible")
    rng = np.random.default_rng(n + d + k)
    centers = rng.uniform(-4, 4, (max(k // 3, 5), d))
    X = (centers[rng.integers(0, centers.shape[0], n)] + rng.standard_normal((n, d))).astype(np.float32)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    h1 = eng.ResidentKMeans()
    h1.upload(X)
    h1.fit(init, 4)
    h2 = eng.ResidentKMeans(devices=list(range(min(ndev, 4))))
    h2.upload(X)
    h2.fit(init, 4)
    assert h1.stats()["path"] == 3 and h2.stats()["path"] == 3
    assert h1.stats()["relocations"] == h2.stats()["relocations"]
    assert np.array_equal(h1.centroids(), h2.centroids())      # integer sums: bit-identical
    assert np.array_equal(h1.labels(), h2.all_labels())
    h1.close()
    h2.close()


@pytest.mark.parametrize("n", [2, 5, 9, 41])
def test_multi_gpu_ragged_row_counts(eng, n):
    """Row counts that a ceil split would leave a device without (9 rows on 8 devices, 5 on 4): the balanced
    split gives every device at least one row and the result equals the single-GPU one."""
    from h2o4gpu_b200.libs import lib_kmeans
    ndev = lib_kmeans.cdll().kmeans_device_count()
    if ndev < 2:
        pytest.skip("one GPU visible")
    rng = np.random.default_rng(n)
    X = rng.standard_normal((n, 3)).astype(np.float32)
    init = X[:2].copy()
    h1 = eng.ResidentKMeans()
    h1.upload(X)
    h1.fit(init, 3)
    g = min(ndev, n, 8)
    h2 = eng.ResidentKMeans(devices=list(range(g)))
    h2.upload(X)
    assert sum(h2._rows) == n and min(h2._rows) >= 1
    h2.fit(init, 3)
    assert np.array_equal(h1.centroids(), h2.centroids())
    assert np.array_equal(h1.labels(), h2.all_labels())
    h1.close()
    h2.close()


# ---- ingest of other element types: converted on the device ------------------------
_TYPED = [np.float16, np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64, np.bool_,
          np.float64, np.float32]


def _typed_matrix(rng, dt, rows, cols):
    dt = np.dtype(dt)
    if dt == np.bool_:
        return rng.integers(0, 2, (rows, cols)).astype(np.bool_)
    if dt.kind == 'f':
        return (rng.standard_normal((rows, cols)) * 8).astype(dt)
    info = np.iinfo(dt)
    # wide integers carry more bits than the float mantissa: conversion must round like astype
    lo, hi = max(info.min, -(1 << 40)), min(info.max, 1 << 40)
    return rng.integers(lo, hi, (rows, cols), dtype=np.int64 if dt.kind == 'i' else np.uint64).astype(dt)


@pytest.mark.parametrize("handle_dtype", [np.float32, np.float64])
@pytest.mark.parametrize("order", ["r", "c"])
def test_typed_upload_matches_astype(eng, handle_dtype, order):
    """kmeans_upload_host_typed gives the shard that a host-side astype + native upload gives, bit for bit
    (seen through the transform of every row, which reads every element)."""
    rng = np.random.default_rng(5)
    rows, cols, k = 1003, 19, 5
    for dt in _TYPED:
        X = _typed_matrix(rng, dt, rows, cols)
        Xn = X.astype(handle_dtype)
        scale = max(float(np.abs(Xn).max()), 1.0)
        C = (rng.standard_normal((k, cols)) * scale).astype(handle_dtype)
        outs = []
        for src in (X if order == "r" else np.asfortranarray(X), Xn):
            h = eng.ResidentKMeans(dtype=handle_dtype)
            h.upload(src, order=order)
            h.set_centroids(C)
            h.assign()
            outs.append((h.transform().copy(), h.labels().copy()))
            h.close()
        assert np.array_equal(outs[0][0], outs[1][0]), np.dtype(dt).name
        assert np.array_equal(outs[0][1], outs[1][1]), np.dtype(dt).name


def test_typed_upload_staged_u8_fit(eng):
    """An 8-bit matrix large enough for the pinned staging pool: a fit on it equals, bit for bit, the fit on
    its float32 copy (image-like data, a quarter of the bytes on the bus)."""
    rng = np.random.default_rng(9)
    rows, cols, k = 600_000, 128, 10
    X = (rng.integers(1, 256, (rows, cols)) * (rng.random((rows, cols)) < 0.2)).astype(np.uint8)
    init = X[:k].astype(np.float32)
    res = []
    for src in (X, X.astype(np.float32)):
        h = eng.ResidentKMeans()
        h.upload(src)
        h.fit(init, 5)
        res.append((h.centroids(), h.labels()))
        h.close()
    assert np.array_equal(res[0][0], res[1][0])
    assert np.array_equal(res[0][1], res[1][1])


# ---- sample weights ------------------------------------------------------------------
def _weighted_case(rng, n, d, k, dtype):
    centers = rng.uniform(-8, 8, (k, d))
    noise = rng.standard_normal((n, d))
    X = (centers[rng.integers(0, k, n)] + noise).astype(dtype)
    w = rng.gamma(2.0, 1.5, n).astype(dtype)
    # some rows of weight zero, taken among those nearest to their centre: a row of weight zero that is
    # relocated into an empty cluster leaves it empty, and scikit-learn then copies un-averaged sums of
    # centred data into it, which no other implementation can be compared with
    w[np.argsort((noise ** 2).sum(1))[:max(1, n // 60)]] = 0
    init = X[rng.choice(n, k, replace=False)].copy()
    return X, w, init


@pytest.mark.parametrize("dtype,n,d,k", [(np.float64, 3000, 6, 7), (np.float32, 20000, 64, 100),
                                         (np.float32, 4000, 33, 5), (np.float32, 30000, 256, 300)])
def test_weighted_fit_matches_oracle(eng, dtype, n, d, k):
    """fit with sample weights against the restatement (itself pinned to scikit-learn's
    fit(X, sample_weight=w)): teacher-forced steps, then a whole fit, inertia included.  Weights enter
    the counts as 30-bit fixed-point numbers, so the float64 bound here is 1e-8, not 1e-10."""
    rng = np.random.default_rng(33)
    X, w, init = _weighted_case(rng, n, d, k, dtype)
    tol = F32_TOL if dtype == np.float32 else 1e-8
    T = 6
    ref = lloyd.fit(X, init, T, dtype=np.float64, sample_weight=w, keep_trajectory=True, stop_on_repeat=False,
                    order="descending")
    h = eng.ResidentKMeans(dtype=dtype)
    h.upload(X)
    h.set_sample_weight(w)
    C = init.astype(np.float64)
    for Cn, labels, _ in ref["trajectory"]:
        h.fit(C.astype(dtype), 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        check_labels(X, C, h.labels(), labels)
        assert rel_err(h.centroids(), Cn) < tol
        C = Cn
    h.fit(init, T)
    assert rel_err(h.centroids(), ref["centers"]) < tol
    check_labels(X, ref["centers"], h.labels(), ref["labels"])
    want = lloyd.inertia(X, ref["centers"], ref["labels"], sample_weight=w)
    assert abs(h.inertia() / want - 1) < (1e-4 if dtype == np.float32 else 1e-8)
    # incremental weighted sums (rows that moved leave and join with w * x) against a full weighted
    # pass in every iteration: the same integers
    h.fit(init, 12)
    inc = (h.centroids(), h.labels(), h.stats()["incremental_iterations"])
    h.fit(init, 12, flags=eng.FIT_FULL_SUMS)
    assert np.array_equal(inc[0], h.centroids()) and np.array_equal(inc[1], h.labels())
    assert inc[2] > 0 and h.stats()["incremental_iterations"] == 0
    # unit weights again: the plain fit, bit for bit
    h.set_sample_weight(None)
    h.fit(init, T)
    plain = h.centroids()
    h.set_sample_weight(np.ones(n, dtype))
    h.fit(init, T)
    assert np.array_equal(h.centroids(), plain)
    h.close()


def test_weighted_fit_equals_repeated_rows(eng):
    """Integer weights mean repeated rows: the weighted fit of X equals the plain fit of X with row i
    written w_i times (same partition, hence the same centres up to the fixed-point quantum)."""
    rng = np.random.default_rng(34)
    n, d, k = 5000, 32, 20
    X, _, init = _weighted_case(rng, n, d, k, np.float32)
    w = rng.integers(0, 4, n)
    h = eng.ResidentKMeans()
    h.upload(X)
    h.set_sample_weight(w)
    h.fit(init, 8)
    Cw, lw = h.centroids(), h.labels()
    h.close()
    rep = np.repeat(np.arange(n), w)
    h = eng.ResidentKMeans()
    h.upload(X[rep])
    h.fit(init, 8)
    Cr, lr = h.centroids(), h.labels()
    h.close()
    assert rel_err(Cw, Cr.astype(np.float64)) < 1e-6
    assert np.array_equal(lw[rep], lr)


def test_weighted_relocation_and_errors(eng):
    """An empty cluster in a weighted fit takes the farthest row with that row's weight; bad weights are
    refused."""
    rng = np.random.default_rng(35)
    X, w, init = _weighted_case(rng, 3000, 6, 7, np.float64)
    init[3] = 1e3
    ref = lloyd.fit(X, init, 10, dtype=np.float64, sample_weight=w, order="descending")
    h = eng.ResidentKMeans(dtype=np.float64)
    h.upload(X)
    h.set_sample_weight(w)
    h.fit(init, 10)
    assert h.stats()["relocations"] >= 1
    assert rel_err(h.centroids(), ref["centers"]) < 1e-8
    assert np.array_equal(h.labels(), ref["labels"])
    from h2o4gpu_b200.libs import lib_kmeans
    for bad in (np.full(3000, -1.0), np.zeros(3000), np.r_[np.ones(2999), np.nan], np.ones(17)):
        with pytest.raises(lib_kmeans.KMeansLibError):
            h.set_sample_weight(bad)
    h.close()


def test_estimator_weights_and_other_dtypes(built_lib):
    """fit(X, sample_weight=w) and 8-bit input stay on the GPU backend and agree with scikit-learn (the
    reference's CPU backend) on the same start."""
    import h2o4gpu_b200
    rng = np.random.default_rng(41)
    X, w, init = _weighted_case(rng, 4000, 16, 6, np.float32)
    gpu = h2o4gpu_b200.KMeans(n_clusters=6, init=init, max_iter=15, tol=0.0, n_gpus=1)
    gpu.fit(X, sample_weight=w)
    cpu = h2o4gpu_b200.KMeans(n_clusters=6, init=init, max_iter=15, tol=0.0, n_gpus=0)
    cpu.fit(X, sample_weight=w)
    assert rel_err(gpu.cluster_centers_, cpu.cluster_centers_.astype(np.float64)) < F32_TOL
    check_labels(X, cpu.cluster_centers_.astype(np.float64), gpu.labels_, cpu.labels_)
    assert abs(gpu.inertia_ - cpu.inertia_) <= 1e-4 * cpu.inertia_
    assert abs(gpu.score(X, sample_weight=w) - cpu.score(X, sample_weight=w)) <= 1e-4 * cpu.inertia_
    assert np.array_equal(gpu.fit_predict(X, sample_weight=w), gpu.labels_)
    # 8-bit pixels: converted on the device, same result as their float32 copy
    P = rng.integers(0, 256, (3000, 24)).astype(np.uint8)
    pinit = P[:5].astype(np.float32)
    a = h2o4gpu_b200.KMeans(n_clusters=5, init=pinit, max_iter=10, tol=0.0, n_gpus=1).fit(P)
    b = h2o4gpu_b200.KMeans(n_clusters=5, init=pinit, max_iter=10, tol=0.0, n_gpus=1).fit(P.astype(np.float32))
    assert a.cluster_centers_.dtype == np.float32
    assert np.array_equal(a.cluster_centers_, b.cluster_centers_)
    assert np.array_equal(a.labels_, b.labels_)
    assert abs(a.inertia_ - b.inertia_) <= 1e-9 * b.inertia_
    assert np.array_equal(a.predict(P), b.predict(P.astype(np.float32)))
    assert np.array_equal(a.transform(P), b.transform(P.astype(np.float32)))
    assert abs(a.score(P) - b.score(P.astype(np.float32))) <= 1e-9 * abs(b.inertia_)


def test_multi_gpu_weighted_and_typed_equal_single_gpu(eng):
    """Weighted fit with an empty cluster, and an 8-bit upload, sharded over several GPUs of one process:
    integer sums make the result identical, bit for bit, to the one-GPU run."""
    from h2o4gpu_b200.libs import lib_kmeans
    ndev = lib_kmeans.cdll().kmeans_device_count()
    if ndev < 2:
        pytest.skip("one GPU visible")
    rng = np.random.default_rng(51)
    X, w, init = _weighted_case(rng, 40001, 32, 24, np.float32)
    init[5] = 1e3                                            # empty in the first M-step: relocation
    P = rng.integers(0, 256, (30001, 48)).astype(np.uint8)
    res = []
    for devs in ([0], list(range(min(ndev, 4)))):
        h = eng.ResidentKMeans(devices=devs)
        h.upload(X)
        h.set_sample_weight(w)
        h.fit(init, 6)
        out = [h.centroids(), h.all_labels(), h.stats()["relocations"], h.inertia()]
        h.upload(P)
        h.fit(P[:7].astype(np.float32), 4)
        out += [h.centroids(), h.all_labels()]
        h.close()
        res.append(out)
    assert res[0][2] == res[1][2] >= 1
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])
    assert abs(res[0][3] - res[1][3]) <= 1e-9 * res[0][3]
    assert np.array_equal(res[0][4], res[1][4]) and np.array_equal(res[0][5], res[1][5])


# ---- one process per GPU (the layout of the bench under torchrun) ---------------------------
_RANK_CODE = r'''
import os, sys, time
import numpy as np
import torch
from h2o4gpu_b200 import engine, synth
rank, world, tmp = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
idf = os.path.join(tmp, "nccl_id")
if rank == 0:
    nid = engine.ResidentKMeans.nccl_unique_id()
    with open(idf + ".part", "wb") as f:
        f.write(nid)
    os.replace(idf + ".part", idf)
else:
    t0 = time.time()
    while not os.path.exists(idf):
        if time.time() - t0 > 120:
            sys.exit("no NCCL id from rank 0")
        time.sleep(0.05)
    nid = open(idf, "rb").read()
X, init, _ = synth.c2(n=50001)
w = np.random.default_rng(3).gamma(2.0, 1.5, X.shape[0]).astype(np.float32)
per = -(-X.shape[0] // world)
lo, hi = rank * per, min(X.shape[0], (rank + 1) * per)
dev = torch.device("cuda", rank)
Xd = torch.from_numpy(X[lo:hi]).to(dev)
h = engine.ResidentKMeans(devices=[rank], rank0=rank, world_size=world, nccl_id=nid)
h.attach_device(0, Xd.data_ptr(), hi - lo, X.shape[1], n_total=X.shape[0])
out = {}
h.fit(init, 5)
out["C"], out["lab"], out["reloc"] = h.centroids(), h.labels(), h.stats()["relocations"]
out["inertia"] = h.inertia()
h.set_sample_weight(w[lo:hi])
h.fit(init, 5)
out["Cw"], out["labw"], out["inertia_w"] = h.centroids(), h.labels(), h.inertia()
h.close()
np.savez(os.path.join(tmp, "rank%d.npz" % rank), **out)
print("rank ok")
'''


@pytest.mark.parametrize("push", ["1", "0"])
def test_one_process_per_gpu_equals_single_gpu(eng, tmp_path, push):
    """Two processes, one GPU each, exchanging the centroid sums by the push all-reduce over peer memory
    (push = 1) or by NCCL (push = 0): the same bits as one GPU, with an empty cluster repaired across ranks,
    without and with sample weights."""
    import os
    import subprocess
    import sys
    from h2o4gpu_b200.libs import lib_kmeans
    if lib_kmeans.cdll().kmeans_device_count() < 2:
        pytest.skip("one GPU visible")
    from h2o4gpu_b200 import synth
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, H2O4GPU_KM_PUSH_ALLREDUCE=push, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", _RANK_CODE, str(r), "2", str(tmp_path)], cwd=root, env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    assert all(p.returncode == 0 for p in procs) and all("rank ok" in o for o in outs), "\n".join(outs)
    X, init, _ = synth.c2(n=50001)
    w = np.random.default_rng(3).gamma(2.0, 1.5, X.shape[0]).astype(np.float32)
    h = eng.ResidentKMeans()
    h.upload(X)
    h.fit(init, 5)
    C, lab, reloc, inertia = h.centroids(), h.labels(), h.stats()["relocations"], h.inertia()
    h.set_sample_weight(w)
    h.fit(init, 5)
    Cw, labw, inertia_w = h.centroids(), h.labels(), h.inertia()
    h.close()
    r = [np.load(tmp_path / ("rank%d.npz" % i)) for i in range(2)]
    assert reloc > 0
    for i in range(2):
        assert int(r[i]["reloc"]) == reloc
        assert np.array_equal(r[i]["C"], C) and np.array_equal(r[i]["Cw"], Cw)
        assert abs(float(r[i]["inertia"]) - inertia) <= 1e-9 * inertia
        assert abs(float(r[i]["inertia_w"]) - inertia_w) <= 1e-9 * inertia_w
    assert np.array_equal(np.concatenate([r[0]["lab"], r[1]["lab"]]), lab)
    assert np.array_equal(np.concatenate([r[0]["labw"], r[1]["labw"]]), labw)


# ---- float64 E-step on the matrix unit -----------------------------------------------------
_DMMA_SHAPES = [(30011, 50, 777), (5003, 6, 40), (20000, 256, 300), (777, 34, 33)]
_DMMA_CODE = r'''
import sys
import numpy as np
from h2o4gpu_b200 import engine
shapes = %r
out = {}
for i, (n, d, k) in enumerate(shapes):
    rng = np.random.default_rng(100 + i)
    centers = rng.uniform(-6, 6, (k, d))
    X = centers[rng.integers(0, k, n)] + rng.standard_normal((n, d))
    init = X[rng.choice(n, k, replace=False)].copy()
    h = engine.ResidentKMeans(dtype=np.float64)
    h.upload(X)
    h.fit(init, 3)
    out["C%%d" %% i], out["lab%%d" %% i] = h.centroids(), h.labels()
    h.close()
np.savez(sys.argv[1], **out)
print("simt ok")
'''


def test_f64_matrix_unit_kernel_matches_simt_kernel_and_oracle(eng, tmp_path):
    """The float64 E-step on the double-precision matrix unit (default for k > 32) against the register-tiled
    kernel (environment switch, child process) - same labels and centroids, ragged n, d and k - and its
    labels against the numpy E-step from the same centres."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = str(tmp_path / "simt.npz")
    r = subprocess.run([sys.executable, "-c", _DMMA_CODE % (_DMMA_SHAPES,), path], cwd=root,
                       env=dict(os.environ, H2O4GPU_KM_DMMA="0"), capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "simt ok" in r.stdout, r.stdout + r.stderr
    simt = np.load(path)
    for i, (n, d, k) in enumerate(_DMMA_SHAPES):
        rng = np.random.default_rng(100 + i)
        centers = rng.uniform(-6, 6, (k, d))
        X = centers[rng.integers(0, k, n)] + rng.standard_normal((n, d))
        init = X[rng.choice(n, k, replace=False)].copy()
        h = eng.ResidentKMeans(dtype=np.float64)
        h.upload(X)
        h.fit(init, 3)
        C, lab = h.centroids(), h.labels()
        h.set_centroids(init)
        h.assign()
        lab0 = h.labels()
        h.close()
        assert np.array_equal(lab, simt["lab%d" % i]), (n, d, k)
        assert rel_err(C, simt["C%d" % i]) < 1e-13
        check_labels(X, init, lab0, lloyd.assign(X, init))


def test_presplit_tensor_core_kernel_matches_converting_kernel(eng, tmp_path):
    """d = 64, 16 iterations or more: the E-step that reads rows split once into fp16 halves against the kernel that
    converts every tile (environment switch, child process): the same labels and centroids, bit for bit;
    and new data at the same address and shape on one handle is not mistaken for the old."""
    import os
    import subprocess
    import sys
    code = (
        "import sys, numpy as np\n"
        "from h2o4gpu_b200 import engine, synth\n"
        "X, init, _ = synth.c2(n=300001)\n"
        "h = engine.ResidentKMeans(); h.upload(X); h.fit(init, 16)\n"
        "np.savez(sys.argv[1], C=h.centroids(), lab=h.labels()); h.close(); print('conv ok')\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = str(tmp_path / "conv.npz")
    r = subprocess.run([sys.executable, "-c", code, path], cwd=root, env=dict(os.environ, H2O4GPU_KM_TC_PRESPLIT="0"),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "conv ok" in r.stdout, r.stdout + r.stderr
    conv = np.load(path)
    from h2o4gpu_b200 import synth
    X, init, _ = synth.c2(n=300001)
    h = eng.ResidentKMeans()
    h.upload(X)
    h.fit(init, 16)
    assert h.stats()["path"] == 3
    assert np.array_equal(h.centroids(), conv["C"]) and np.array_equal(h.labels(), conv["lab"])
    # a short fit takes the converting kernel unless told otherwise: both give the same bits
    outs = []
    for flags in (0, eng.FIT_PRESPLIT):
        h2 = eng.ResidentKMeans()
        h2.upload(X)
        h2.fit(init, 2, flags=flags)
        outs.append((h2.centroids(), h2.labels()))
        h2.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    # other rows, same shape, same handle (the pool hands back the same address)
    X2 = np.ascontiguousarray(X[::-1])
    h.upload(X2)
    h.fit(init, 16)
    C2, lab2 = h.centroids(), h.labels()
    h.close()
    h = eng.ResidentKMeans()
    h.upload(X2)
    h.fit(init, 16)
    assert np.array_equal(C2, h.centroids()) and np.array_equal(lab2, h.labels())
    h.close()


# ---- the tensor-core kernels at sizes that wrap their rings many times -------------------
@pytest.mark.parametrize("cfg,kw,steps", [("c2", dict(n=1_200_000), 3), ("c3", dict(n=300_000), 2)])
def test_teacher_forced_large_f32(eng, cfg, kw, steps):
    """1.2e6 rows of the C2 shape are 9,375 row tiles on 148 persistent CTAs (63 tiles per CTA: the
    five-stage ring, the two issuers' hand-over and the three accumulators all wrap a dozen times);
    3e5 rows of the C3 shape walk the streamed centroid table 2,344 times."""
    from h2o4gpu_b200 import synth
    X, init, _ = synth.CONFIGS[cfg](**kw)
    C = init.astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    ties = 0
    for _ in range(steps):
        C32 = C.astype(np.float32)
        Cn, labn, _, moved = lloyd.step(X, C32.astype(np.float64), order="descending")
        h.fit(C32, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        st = h.stats()
        assert st["path"] == 3
        ties += check_step(X, C32.astype(np.float64), h.centroids(), h.labels(), Cn, labn, moved, st["relocations"])
        C = Cn
    h.close()
    print("near-tie label differences over the run:", ties)


@pytest.mark.parametrize("cfg,kw", [("c2", dict(n=2_000_000)), ("c3", dict(n=200_000)), ("c5", dict(n=30_000))])
def test_tensor_core_labels_equal_float64_engine(eng, cfg, kw):
    """The float32 tensor-core E-step re-evaluates its ambiguous rows in double, so its labels are the
    float64 argmin on the float32 data: compared here with the float64 engine on X.astype(float64)."""
    from h2o4gpu_b200 import synth
    X, init, _ = synth.CONFIGS[cfg](**kw)
    C32, lab32, st32 = one_step(eng, X, init)
    assert st32["path"] == 3
    C64, lab64, _ = one_step(eng, X.astype(np.float64), init.astype(np.float64))
    bad = np.flatnonzero(lab32 != lab64)
    print("rows re-evaluated: %d, labels that differ from the float64 engine: %d" % (st32["refined_rows"], bad.size))
    assert bad.size <= 2
    if bad.size:
        assert lloyd.near_tie_mask(X[bad], init.astype(np.float64), rel=1e-12).all()
    else:
        assert rel_err(C32, C64.astype(np.float64)) < 1e-6


# ---- data spanning many orders of magnitude ----------------------------------------------
@pytest.mark.parametrize("case", ["outlier_1e4", "outlier_1e6", "outlier_1e8", "column_1e6"])
def test_wide_dynamic_range_f32(eng, case):
    """The tensor-core kernel scales X by one power of two taken from max|x| before it splits the values into
    fp16 halves, so an element far above the rest pushes the low halves of ordinary elements below fp16's
    normal range.  The ambiguity threshold carries an absolute term for that; labels must stay the float64
    argmin outside the 1e-5 band.  Centroids: 1e-4 of the largest reference coordinate (the exact integer
    sums resolve max|x| * 2^-30, not each centroid's own magnitude)."""
    from h2o4gpu_b200 import synth
    X, init, _ = synth.c2(n=30000)
    X = X.copy()
    if case.startswith("outlier"):
        X[5, 7] = float(case.split("_")[1]) * 10.0
    else:
        X[:, 3] *= 1e6
        init = X[np.sort(np.random.default_rng(3).choice(30000, 100, replace=False))].copy()
    C = init.astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    refined = 0
    for _ in range(3):
        C32 = C.astype(np.float32)
        Cn, labn, _, moved = lloyd.step(X, C32.astype(np.float64), order="descending")
        h.fit(C32, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        st = h.stats()
        assert st["path"] == 3
        refined += st["refined_rows"]
        check_step(X, C32.astype(np.float64), h.centroids(), h.labels(), Cn, labn, moved, st["relocations"])
        C = Cn
    h.close()
    print("%s: %d rows re-evaluated in double over 3 steps" % (case, refined))


# ---- the reference header's own (C++-linkage) names, called ------------------------------
def test_cxx_linkage_entry_points_are_callable(built_lib):
    """src/include/solver/kmeans.h:56-76 declares the four functions without extern "C"; code compiled
    against that header binds the mangled names.  Look them up with nm and call them."""
    import re
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", built_lib], capture_output=True, text=True).stdout
    sym = {}
    for n in ("make_ptr_float_kmeans", "make_ptr_double_kmeans", "kmeans_transform_float", "kmeans_transform_double"):
        sym[n] = re.search(r" T (_Z\d+%s\w*)" % n, out).group(1)
    lib = ctypes.CDLL(built_lib)
    g = load_golden("blobs_n600_d5_k4")
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    for dtype, tag, cfloat in ((np.float32, "float", ctypes.c_float), (np.float64, "double", ctypes.c_double)):
        X = g["X"].astype(dtype)
        init = g["init"].astype(dtype)
        rows, cols = X.shape
        k = init.shape[0]
        fit = getattr(lib, sym["make_ptr_%s_kmeans" % tag])
        fit.restype = ci
        fit.argtypes = [ci] * 5 + [sz, sz, ci, ci, ci, cfloat, vp, vp, vp, vp]
        centers = np.zeros((k, cols), dtype)
        labels = np.zeros(rows, np.int32)
        pc, pl = vp(centers.ctypes.data), vp(labels.ctypes.data)
        rc = fit(0, 0, 0, 0, 1, rows, cols, k, int(g["T"]), 2, 0.0, X.ctypes.data_as(vp), init.ctypes.data_as(vp),
                 ctypes.byref(pc), ctypes.byref(pl))
        assert rc == 0
        f = "f32" if dtype == np.float32 else "f64"
        ref = g["centers_" + f].astype(np.float64)
        assert rel_err(centers, ref) < (F32_TOL if dtype == np.float32 else F64_TOL)
        check_labels(X, ref, labels, g["labels_" + f])
        # dopredict = 1 through the same symbol
        pred = np.zeros(rows, np.int32)
        pl = vp(pred.ctypes.data)
        rc = fit(1, 0, 0, 0, 1, rows, cols, k, 0, 0, 0.0, X.ctypes.data_as(vp), centers.ctypes.data_as(vp),
                 ctypes.byref(pc), ctypes.byref(pl))
        assert rc == 0
        check_labels(X, centers.astype(np.float64), pred, lloyd.assign(X, centers.astype(np.float64)))
        tr = getattr(lib, sym["kmeans_transform_%s" % tag])
        tr.restype = ci
        tr.argtypes = [ci] * 3 + [sz, sz, ci, vp, vp, vp]
        D = np.zeros(rows * k, dtype)
        pp = vp(D.ctypes.data)
        rc = tr(0, 0, 1, rows, cols, k, X.ctypes.data_as(vp), centers.ctypes.data_as(vp), ctypes.byref(pp))
        assert rc == 0
        want = lloyd.transform_sq_colmajor(X, centers)
        assert np.abs(D - want).max() <= (1e-4 if dtype == np.float32 else 1e-10) * want.max()


# ---- failure detection: a bounded device-side wait that runs out ------------------------
def test_bounded_waits_give_up_and_leave_the_device_usable(eng, built_lib):
    """Nothing faults: a kernel waits for a flag that nothing raises, the wait's limit (set to about 10 ms)
    runs out, the kernel records its code and ends, the call returns KM_ETIMEOUT, and the handle made
    before still fits afterwards with the same result."""
    import time
    from h2o4gpu_b200 import synth
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.cdll()
    X, init, _ = synth.c2(n=20000)
    h = eng.ResidentKMeans()
    h.upload(X)
    h.fit(init, 3)
    before = h.centroids()
    assert lib.kmeans_set_wait_limits(10.0, 10.0) == 0
    try:
        for which, code in ((0, 11), (1, 9)):
            got = ctypes.c_int(0)
            t0 = time.perf_counter()
            rc = lib.kmeans_selftest_wait_timeout(0, which, ctypes.byref(got))
            dt = time.perf_counter() - t0
            assert rc == -7 and got.value == code, (rc, got.value)      # KM_ETIMEOUT, the wait's code
            assert b"gave up" in lib.kmeans_last_error()
            assert dt < 1.5, dt                                          # the short limit was honoured
    finally:
        assert lib.kmeans_set_wait_limits(0.0, 0.0) == 0                 # defaults back
    h.fit(init, 3)
    assert np.array_equal(h.centroids(), before)
    h.close()


# ---- few centroids, wide rows: tensor-core kernel against the FMA kernel, and its transform ---------
def test_wide_rows_tensor_core_kernel_matches_simt_kernel_and_transform(eng, tmp_path):
    from h2o4gpu_b200 import synth
    X, init, _ = synth.c4(n=50000)
    C0 = init.astype(np.float64)
    a = one_step(eng, X, init)
    b = one_step(eng, X, init, flags=eng.FIT_FORCE_SIMT)
    assert a[2]["path"] == 3 and b[2]["path"] == 2
    bad = check_labels(X, C0, a[1], b[1])
    if bad == 0:
        assert np.array_equal(a[0], b[0])          # integer sums: same labels -> same bits
    # transform on the fitted centroids: one block, and row batches that are not the whole shard
    import os
    import subprocess
    import sys
    h = eng.ResidentKMeans()
    h.upload(X)
    h.fit(init, 3)
    C = h.centroids()
    D = h.transform()
    h.close()
    want = lloyd.transform_sq_exact(X, C.astype(np.float64))
    floor = np.finfo(np.float32).eps * ((X.astype(np.float64) ** 2).sum(1)[:, None] + (C.astype(np.float64) ** 2).sum(1)[None, :])
    assert (np.abs(D - want) <= 1e-4 * want + 8 * floor).all()
    code = ("import sys, numpy as np; sys.path.insert(0, %r); import h2o4gpu_b200.engine as e; "
            "X = np.load(%r); C = np.load(%r); h = e.ResidentKMeans(); h.upload(X); h.set_centroids(C); "
            "np.save(%r, h.transform())")
    np.save(tmp_path / "X.npy", X)
    np.save(tmp_path / "C.npy", C)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, H2O4GPU_KM_TRANSFORM_BATCH_ROWS="12800")
    subprocess.run([sys.executable, "-c", code % (root, str(tmp_path / "X.npy"), str(tmp_path / "C.npy"),
                                                  str(tmp_path / "D.npy"))], check=True, env=env)
    assert np.array_equal(np.load(tmp_path / "D.npy"), D)          # batching changes no value


# ---- row widths between the compiled variants of the tensor-core kernels --------------------
@pytest.mark.parametrize("n,d,k", [(20000, 48, 100), (30000, 100, 17), (20000, 100, 300), (9000, 200, 1000),
                                   (5000, 36, 129), (7000, 252, 6144)])
def test_any_row_width_reaches_the_tensor_cores(eng, n, d, k):
    """16-byte aligned rows of up to 256 columns take the tcgen05 kernel compiled for the next of 32 / 64 /
    128 / 256 columns (the copy engine zero-fills the missing columns); results as for any other shape."""
    rng = np.random.default_rng(n + d + k)
    centers = rng.uniform(-8, 8, (max(k // 3, 5), d))
    X = (centers[rng.integers(0, centers.shape[0], n)] + rng.standard_normal((n, d))).astype(np.float32)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    C = init.astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    for _ in range(2):
        C32 = C.astype(np.float32)
        Cn, labn, _, moved = lloyd.step(X, C32.astype(np.float64), order="descending")
        h.fit(C32, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        st = h.stats()
        assert st["path"] == 3
        check_step(X, C32.astype(np.float64), h.centroids(), h.labels(), Cn, labn, moved, st["relocations"])
        C = Cn
    h.close()


# ---- rows wider than 256 columns with many centroids: both operands streamed ---------------
@pytest.mark.parametrize("n,d,k", [(20000, 784, 100), (9001, 300, 40), (6000, 1000, 300), (5000, 512, 600),
                                   (3000, 260, 17)])
def test_wide_rows_many_centroids_reach_the_tensor_cores(eng, n, d, k):
    """16-byte aligned rows of more than 256 columns with more than 16 centroids take the tcgen05 kernel
    that streams both operands in chunks of 64 columns (one pass per 128 or 256 centroids); results as for
    any other shape, checked against the float64 oracle step by step, and labels against the FMA kernel."""
    rng = np.random.default_rng(n + d + k)
    centers = rng.uniform(-4, 4, (max(k // 3, 5), d))
    X = (centers[rng.integers(0, centers.shape[0], n)] + rng.standard_normal((n, d))).astype(np.float32)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    C = init.astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    for _ in range(2):
        C32 = C.astype(np.float32)
        Cn, labn, _, moved = lloyd.step(X, C32.astype(np.float64), order="descending")
        h.fit(C32, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        st = h.stats()
        assert st["path"] == 3
        check_step(X, C32.astype(np.float64), h.centroids(), h.labels(), Cn, labn, moved, st["relocations"])
        C = Cn
    h.close()
    a = one_step(eng, X, init)
    b = one_step(eng, X, init, flags=eng.FIT_FORCE_SIMT)
    assert a[2]["path"] == 3 and b[2]["path"] == 2
    if check_labels(X, init.astype(np.float64), a[1], b[1]) == 0:
        assert np.array_equal(a[0], b[0])          # integer sums: same labels -> same bits


@pytest.mark.parametrize("n,d,k", [(30000, 64, 100), (20000, 128, 300), (4000, 256, 1000), (12000, 784, 100),
                                   (5000, 48, 33), (3333, 1000, 300)])
def test_transform_on_the_tensor_cores_matches_exact_distances(eng, tmp_path, n, d, k):
    """transform (n x k squared distances) of every float32 shape with more than 16 centroids and 16-byte
    aligned rows of 32 columns or more runs on the streaming tcgen05 kernel with its store epilogue:
    values against exact float64 distances, and unchanged by row batching."""
    import os
    import subprocess
    import sys
    rng = np.random.default_rng(n + d + k)
    centers = rng.uniform(-4, 4, (max(k // 3, 5), d))
    X = (centers[rng.integers(0, centers.shape[0], n)] + rng.standard_normal((n, d))).astype(np.float32)
    C = X[np.sort(rng.choice(n, k, replace=False))].copy()
    h = eng.ResidentKMeans()
    h.upload(X)
    h.set_centroids(C)
    D = h.transform()
    assert h.stats()["path"] == 3
    h.close()
    want = lloyd.transform_sq_exact(X, C.astype(np.float64))
    floor = np.finfo(np.float32).eps * ((X.astype(np.float64) ** 2).sum(1)[:, None] + (C.astype(np.float64) ** 2).sum(1)[None, :])
    assert D.shape == want.shape
    # the centroids are rows of X, so some distances are exactly zero: there only the cancellation floor
    # counts - the error bound of a score is 2^-19 (0.8 + d / 200) (|x|^2 + |c|^2), i.e. 16 float32
    # epsilons of that sum times the row-width factor (the ambiguity threshold of the labelling kernels),
    # plus the float32 rounding of |x|^2, |c|^2 and their sum
    bound = 16 * (0.8 + d / 200.0) + 16
    assert (np.abs(D - want) <= 1e-4 * want + bound * floor).all()
    code = ("import sys, numpy as np; sys.path.insert(0, %r); import h2o4gpu_b200.engine as e; "
            "X = np.load(%r); C = np.load(%r); h = e.ResidentKMeans(); h.upload(X); h.set_centroids(C); "
            "np.save(%r, h.transform())")
    np.save(tmp_path / "X.npy", X)
    np.save(tmp_path / "C.npy", C)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, H2O4GPU_KM_TRANSFORM_BATCH_ROWS="1280")
    subprocess.run([sys.executable, "-c", code % (root, str(tmp_path / "X.npy"), str(tmp_path / "C.npy"),
                                                  str(tmp_path / "D.npy"))], check=True, env=env)
    assert np.array_equal(np.load(tmp_path / "D.npy"), D)          # batching changes no value


# ---- data far from the origin: the tensor core's accumulation error grows with the row width -----
@pytest.mark.parametrize("d,k", [(64, 100), (256, 300), (784, 10), (784, 100), (2048, 40)])
@pytest.mark.parametrize("offset", [6.0, 25.0])
def test_offset_data_labels_equal_float64_argmin(eng, d, k, offset):
    """All coordinates near a common offset make |x.c| = |x||c|, the worst case for the fp32 accumulation of
    the tensor-core products (a one-sided error per K = 16 slice, so it grows with d); the ambiguity
    threshold scales with the row width and hands the doubtful rows to the exact pass.  With the flat
    threshold rows of 2048 columns were mislabelled (gaps up to 3e-4 relative).  Labels must equal the
    float64 argmin except inside the 1e-5 near-tie band."""
    n = 20000
    rng = np.random.default_rng(d + k)
    X = (offset + rng.standard_normal((n, d))).astype(np.float32)
    C = np.stack([X[rng.choice(n, 50, replace=False)].mean(0) for _ in range(k)]).astype(np.float32)
    h = eng.ResidentKMeans()
    h.upload(X)
    h.fit(C, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
    lab = h.labels()
    st = h.stats()
    h.close()
    assert st["path"] == 3
    want = lloyd.assign(X, C.astype(np.float64), dtype=np.float64)
    check_labels(X, C.astype(np.float64), lab, want)


# ---- rows that are not a multiple of 16 bytes: tensor cores through a zero-padded copy --------------
@pytest.mark.parametrize("n,d,k", [(20000, 50, 100), (9000, 101, 300), (5000, 785, 40), (8000, 786, 12),
                                   (6000, 30, 64), (4001, 255, 17)])
def test_unaligned_row_widths_reach_the_tensor_cores(eng, n, d, k):
    """d % 4 != 0: TMA cannot address the rows, so the tensor-core kernels read a copy of the shard padded
    with zero columns to the next multiple of four (built once per matrix); sums, exact pass and everything
    else keep the rows as they are.  Results as for any other shape; labels against the FMA kernel too."""
    rng = np.random.default_rng(n + d + k)
    centers = rng.uniform(-4, 4, (max(k // 3, 5), d))
    X = (centers[rng.integers(0, centers.shape[0], n)] + rng.standard_normal((n, d))).astype(np.float32)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    C = init.astype(np.float64)
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    for _ in range(2):
        C32 = C.astype(np.float32)
        Cn, labn, _, moved = lloyd.step(X, C32.astype(np.float64), order="descending")
        h.fit(C32, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
        st = h.stats()
        assert st["path"] == 3
        check_step(X, C32.astype(np.float64), h.centroids(), h.labels(), Cn, labn, moved, st["relocations"])
        C = Cn
    # several iterations through the incremental sums as well, then predict and transform on the result
    h.fit(init, 6)
    Cfit = h.centroids()
    lab_fit = h.labels()
    h.assign()
    assert np.array_equal(h.labels(), lab_fit)
    D = h.transform()
    h.close()
    want = lloyd.transform_sq_exact(X, Cfit.astype(np.float64))
    floor = np.finfo(np.float32).eps * ((X.astype(np.float64) ** 2).sum(1)[:, None] + (Cfit.astype(np.float64) ** 2).sum(1)[None, :])
    assert (np.abs(D - want) <= 1e-4 * want + (16 * (0.8 + d / 200.0) + 16) * floor).all()
    a = one_step(eng, X, init)
    b = one_step(eng, X, init, flags=eng.FIT_FORCE_SIMT)
    assert a[2]["path"] == 3 and b[2]["path"] == 2
    if check_labels(X, init.astype(np.float64), a[1], b[1]) == 0:
        assert np.array_equal(a[0], b[0])          # integer sums: same labels -> same bits


# ---- seeded random shapes across all distance kernels ------------------------------------------
def _fuzz_shapes():
    rng = np.random.default_rng(20261126)
    shapes = []
    for _ in range(28):
        d = int(rng.choice([rng.integers(2, 40), rng.integers(40, 300), rng.integers(300, 1300)]))
        k = int(rng.choice([rng.integers(2, 17), rng.integers(17, 130), rng.integers(130, 700)]))
        n = int(rng.integers(max(k, 130), 6000))
        shapes.append((n, d, k))
    # edge sizes: fewer rows than one tile, one row more than a tile, k = n
    shapes += [(k0, d0, k0) for k0, d0 in ((37, 64), (129, 300), (200, 785))] + [(129, 128, 40), (257, 784, 10)]
    return shapes


@pytest.mark.parametrize("n,d,k", _fuzz_shapes())
def test_random_shapes_one_step_matches_oracle(eng, n, d, k):
    """Whatever kernel a shape selects (fused small-k, FMA tiles, one of the four tensor-core kernels, the padded
    copy for unaligned rows), one Lloyd step equals the float64 oracle's: labels outside the near-tie band,
    centroids to 1e-4, relocations counted alike; predict on the result reproduces the labels."""
    rng = np.random.default_rng(n * 7 + d * 3 + k)
    centers = rng.uniform(-5, 5, (max(k // 2, 3), d))
    X = (centers[rng.integers(0, centers.shape[0], n)] + rng.standard_normal((n, d))).astype(np.float32)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    h = eng.ResidentKMeans(dtype=np.float32)
    h.upload(X)
    Cn, labn, _, moved = lloyd.step(X, init.astype(np.float64), order="descending")
    h.fit(init, 1, flags=eng.FIT_NO_FINAL_ASSIGN)
    st = h.stats()
    check_step(X, init.astype(np.float64), h.centroids(), h.labels(), Cn, labn, moved, st["relocations"])
    # labels of the new centroids: fit's closing E-step against predict
    h.fit(init, 2)
    lab2 = h.labels()
    h.assign()
    assert np.array_equal(h.labels(), lab2)
    h.close()
