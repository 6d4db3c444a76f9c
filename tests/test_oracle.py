"""The CPU oracle against its pins: scikit-learn fixtures (the reference's CPU
path) and the literal arrays of the reference's kernel tests."""
import numpy as np
import pytest

from conftest import GOLDEN_CASES, load_golden
from oracle import cref, lloyd


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_restatement_matches_sklearn_fp64(name):
    g = load_golden(name)
    X, init, T = g["X"], g["init"], int(g["T"])
    r = lloyd.fit(X, init, T, dtype=np.float64)
    ref = g["centers_f64"]
    rel = np.abs(r["centers"] - ref).max() / np.abs(ref).max()
    assert rel < 1e-12
    assert np.array_equal(r["labels"], g["labels_f64"])
    assert r["n_iter"] == int(g["n_iter_f64"])
    assert abs(lloyd.inertia(X, r["centers"], r["labels"]) / float(g["inertia_f64"]) - 1) < 1e-10


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_restatement_fp32_close_to_sklearn_fp32(name):
    # float32 runs differ by rounding order only; these cases are well separated
    g = load_golden(name)
    X, init, T = g["X"], g["init"], int(g["T"])
    r = lloyd.fit(X, init, T, dtype=np.float32)
    ref = g["centers_f32"]
    assert np.abs(r["centers"] - ref).max() / np.abs(ref).max() < 1e-4
    assert (r["labels"] != g["labels_f32"]).mean() < 1e-3


def test_predict_transform_conventions():
    g = load_golden("blobs_n600_d5_k4")
    X, C = g["X"].astype(np.float64), g["centers_f64"]
    assert np.array_equal(lloyd.assign(X, C), g["predict_f64"])
    sq = lloyd.transform_sq_colmajor(X[:64], C).reshape((64, C.shape[0]), order="F")
    assert np.allclose(np.sqrt(sq), g["transform_f64"], rtol=1e-9, atol=1e-9)
    assert np.allclose(sq, lloyd.transform_sq_exact(X[:64], C), rtol=1e-9, atol=1e-9)


def test_empty_cluster_rule_is_exercised():
    g = load_golden("empty_n500_d3_k6")
    r = lloyd.fit(g["X"], g["init"], int(g["T"]), dtype=np.float64, keep_trajectory=True)
    moved = [m for _, _, m in r["trajectory"] if m]
    assert moved and len(moved[0]) == 2          # both far centres are empty in step 1
    # the engine's deterministic order gives the same set of centres
    r2 = lloyd.fit(g["X"], g["init"], int(g["T"]), dtype=np.float64, order="descending")
    perm = lloyd.match_centers(r["centers"], r2["centers"])
    assert np.abs(r["centers"] - r2["centers"][perm]).max() < 1e-9


def test_c_restatement_matches_numpy():
    g = load_golden("empty_n500_d3_k6")
    X = g["X"]
    C = g["init"].astype(np.float64)
    for _ in range(4):
        Cn, lab, cnt, moved = cref.step(X, C)
        Cp, labp, cntp, movedp = lloyd.step(X, C, order="descending")
        assert np.array_equal(lab, labp)
        assert np.array_equal(cnt, cntp)
        assert moved == len(movedp)
        assert np.abs(Cn - Cp).max() < 1e-12
        C = Cn
    lab, best = cref.assign(X, C)
    assert np.array_equal(lab, lloyd.assign(X, C))
    t = cref.transform(X[:50], C)
    assert np.allclose(t, lloyd.transform_sq_colmajor(X[:50], C), rtol=1e-12, atol=1e-12)


# ---- literal arrays of the reference's kernel tests -------------------------------
def test_ref_calculate_centroids():
    # tests/cpp/gpu/kmeans/test_kmeans_centroids.cu:7-78: n=4, d=2, k=2, un-normalised sums
    X = np.array([[0, 0], [0, 1], [1, 1], [1, 0]], np.float32)
    labels = np.array([0, 0, 1, 1], np.int32)
    sums, counts = lloyd.sums_counts(X, labels, 2)
    assert np.array_equal(sums, [[0, 1], [2, 1]])
    assert np.array_equal(counts, [2, 2])


def test_ref_two_shards_add_up():
    # test_kmeans_centroids.cu:82-251: sums over two halves == sums over all rows
    Xa = np.array([[4, 2], [1, 0], [4, 0]], np.float32)
    la = np.array([0, 0, 0], np.int32)
    Xb = np.array([[4, 4], [1, 4], [1, 2]], np.float32)
    lb = np.array([0, 1, 1], np.int32)
    sa, ca = lloyd.sums_counts(Xa, la, 2)
    sb, cb = lloyd.sums_counts(Xb, lb, 2)
    s, c = lloyd.sums_counts(np.vstack([Xa, Xb]), np.r_[la, lb], 2)
    assert np.array_equal(sa + sb, s) and np.array_equal(ca + cb, c)
    assert np.array_equal(s, [[13, 6], [2, 6]])


def test_ref_centroid_scaling():
    # test_kmeans_centroids.cu:308-346: sums [[1,2],[3,4]] / counts [4,2]
    C = lloyd.average(np.array([[1., 2.], [3., 4.]]), np.array([4, 2]))
    assert np.array_equal(C, [[0.25, 0.5], [1.5, 2.0]])


def test_ref_counts_per_centroid():
    # tests/cpp/gpu/kmeans/test_kmeans_h2o4gpu.cu:67-112 and :114-174
    X = np.array([[0, 0], [2, 2], [2, 3], [3, 2]], np.float32)
    C = np.array([[0, 0], [2, 2]], np.float32)
    assert np.array_equal(np.bincount(lloyd.assign(X, C), minlength=2), [1, 3])
    P = np.array([[1, 2], [1, 4], [1, 0], [4, 2], [4, 4], [4, 0]], np.float32)
    assert np.array_equal(np.bincount(lloyd.assign(P, P), minlength=6), [1] * 6)


def test_ref_readme_example():
    # README.md:115-133: X=[[1,1],[1,4],[1,0]], k=2 -> centres {[1, 0.5], [1, 4]}; the
    # README prints [[1,1],[1,4]] for the default max_iter of its time; a converged
    # Lloyd run gives the two means below from any init that separates row 1.
    X = np.array([[1., 1.], [1., 4.], [1., 0.]])
    r = lloyd.fit(X, X[[0, 1]], 10)
    assert np.allclose(sorted(map(tuple, r["centers"])), [(1.0, 0.5), (1.0, 4.0)])
    assert r["labels"].tolist() == [0, 1, 0]


@pytest.mark.parametrize("empty", [False, True])
def test_weighted_restatement_matches_sklearn(empty):
    """fit(X, sample_weight=w): the restatement against scikit-learn itself (installed on every box this
    suite runs on), float64, with and without an empty cluster to relocate."""
    from oracle import sklearn_oracle
    rng = np.random.default_rng(21)
    n, d, k, T = 3000, 6, 7, 12
    centers = rng.uniform(-8, 8, (k, d))
    X = centers[rng.integers(0, k, n)] + rng.standard_normal((n, d))
    w = rng.gamma(2.0, 1.5, n)
    w[rng.integers(0, n, 50)] = 0.0
    init = X[rng.choice(n, k, replace=False)].copy()
    if empty:
        init[3] = 1e3      # no row is nearest to it: relocation in the first M-step
    ref = sklearn_oracle.fit(X, init, T, sample_weight=w)
    r = lloyd.fit(X, init, T, dtype=np.float64, sample_weight=w)
    assert np.abs(r["centers"] - ref["centers"]).max() / np.abs(ref["centers"]).max() < 1e-12
    assert np.array_equal(r["labels"], ref["labels"])
    assert r["n_iter"] == ref["n_iter"]
    assert abs(lloyd.inertia(X, r["centers"], r["labels"], sample_weight=w) / ref["inertia"] - 1) < 1e-10
