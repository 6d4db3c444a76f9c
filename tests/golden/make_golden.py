"""Generates tests/golden/*.npz: inputs and outputs of scikit-learn's Lloyd solver,
the library the reference's CPU k-means path (h2o4gpu.KMeans(n_gpus=0)) runs.

Run from the repository root:  python tests/golden/make_golden.py
(--tensor-core-cases writes only the two fixtures shaped for the tensor-core kernels).
Recorded with the scikit-learn / numpy versions stored in each file.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
from oracle import sklearn_oracle as sk  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def blobs(rng, n, d, k, spread=6.0, sigma=1.0):
    centers = rng.uniform(-spread, spread, (k, d))
    comp = rng.integers(0, k, n)
    return (centers[comp] + sigma * rng.standard_normal((n, d))).astype(np.float32)


def record(name, X, init, T):
    import sklearn
    out = {"X": X, "init": init, "T": np.int64(T),
           "sklearn_version": sklearn.__version__, "numpy_version": np.__version__}
    for tag, dt in (("f32", np.float32), ("f64", np.float64)):
        Xd, Id = X.astype(dt), init.astype(dt)
        r = sk.fit(Xd, Id, T)
        out["centers_" + tag] = r["centers"]
        out["labels_" + tag] = r["labels"]
        out["n_iter_" + tag] = np.int64(r["n_iter"])
        out["inertia_" + tag] = np.float64(r["inertia"])
        out["predict_" + tag] = sk.predict(Xd, r["centers"])
        out["transform_" + tag] = sk.transform(Xd[:64], r["centers"])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, X.shape, init.shape, "n_iter", out["n_iter_f32"], out["n_iter_f64"])


def tensor_core_cases():
    """Shapes that the tcgen05 kernels serve: d = 64, k = 100 (centroid table resident in shared memory)
    and d = 128, k = 300 (table streamed).  Values lie on a grid of 1/32 so that the files compress;
    T is large enough for scikit-learn to converge in float32 and float64 alike."""
    rng = np.random.default_rng(20250311)
    for name, n, d, k, spread, T in (("blobs_n3000_d64_k100", 3000, 64, 100, 10.0, 30),
                                     ("blobs_n3600_d128_k300", 3600, 128, 300, 12.0, 30)):
        X = np.round(blobs(rng, n, d, k, spread=spread) * 32.0) / 32.0
        X = X.astype(np.float32)
        record(name, X, X[np.sort(rng.choice(n, k, replace=False))].copy(), T)


def main():
    if "--tensor-core-cases" in sys.argv:
        tensor_core_cases()
        return
    rng = np.random.default_rng(20240607)
    X = blobs(rng, 600, 5, 4)
    record("blobs_n600_d5_k4", X, X[:4].copy(), 10)
    X = blobs(rng, 2000, 32, 8, spread=10.0)
    record("blobs_n2000_d32_k8", X, X[:8].copy(), 20)
    # two initial centres far from all data: both end up empty and are relocated
    X = blobs(rng, 500, 3, 4)
    init = np.vstack([X[:4], [[100, 100, 100]], [[-90, 80, -70]]]).astype(np.float32)
    record("empty_n500_d3_k6", X, init, 8)
    # odd sizes: d not a multiple of 4, k = 17 (> the fused-kernel bound)
    X = blobs(rng, 1500, 7, 17, spread=8.0)
    record("blobs_n1500_d7_k17", X, X[rng.choice(1500, 17, replace=False)].copy(), 12)
    tensor_core_cases()


if __name__ == "__main__":
    main()
