"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (host-sized; the device-side generator for inputs too
large for host memory lives in csrc/synth.cuh and draws from the same
distributions with a counter-based generator).

Each ``cN(n=..., seed=...)`` returns ``(X, init, T)``: the data (row-major,
float32 unless ``dtype`` says otherwise), the explicit k x d initial centroids
and the configured number of Lloyd iterations.
"""
import numpy as np


def _mixture(rng, n, centers, sigma, weights=None, dtype=np.float32, chunk=1 << 20):
    k, d = centers.shape
    if weights is None:
        comp = rng.integers(0, k, n)
    else:
        comp = rng.choice(k, n, p=weights)
    X = np.empty((n, d), dtype=dtype)
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        X[s:e] = (centers[comp[s:e]] + sigma * rng.standard_normal((e - s, d))).astype(dtype)
    return X


def c1(n=100_000, seed=0, dtype=np.float32):
    """8 isotropic Gaussians (sigma 1), centres U(-10,10)^32, k=8, init = first 8 rows, T=20."""
    rng = np.random.default_rng(seed)
    centers = rng.uniform(-10, 10, (8, 32))
    X = _mixture(rng, n, centers, 1.0, dtype=dtype)
    return X, X[:8].copy(), 20


def c2(n=10_000_000, seed=0, dtype=np.float32):
    """100-component mixture, Dirichlet(1) weights, d=64, k=100, init = 100 seeded rows, T=50."""
    rng = np.random.default_rng(seed)
    centers = rng.uniform(-10, 10, (100, 64))
    w = rng.dirichlet(np.ones(100))
    X = _mixture(rng, n, centers, 1.0, weights=w, dtype=dtype)
    init = X[np.sort(rng.choice(n, 100, replace=False))].copy()
    return X, init, 50


def c3(n=500_000, seed=0, dtype=np.float32, k=1000, d=128):
    """1000 equal-weight components (sigma 2), centres U(-20,20)^128, k=1000, T=30."""
    rng = np.random.default_rng(seed)
    centers = rng.uniform(-20, 20, (k, d))
    X = _mixture(rng, n, centers, 2.0, dtype=dtype)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    return X, init, 30


def c4(n=200_000, seed=0, dtype=np.float32, d=784, k=10):
    """Image-like: 0 w.p. 0.8 else an integer in [1,255]; k=10, init = first 10 rows, T=100."""
    rng = np.random.default_rng(seed)
    X = np.empty((n, d), dtype=dtype)
    chunk = 1 << 16
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        v = rng.integers(1, 256, (e - s, d))
        z = rng.random((e - s, d)) < 0.8
        v[z] = 0
        X[s:e] = v
    return X, X[:k].copy(), 100


def c5(n=100_000, seed=0, dtype=np.float32, k=4096, d=256):
    """Standard normal plus a 4096-component offset (centres N(0,4I)); k=4096, T=10."""
    rng = np.random.default_rng(seed)
    centers = 2.0 * rng.standard_normal((k, d))
    X = _mixture(rng, n, centers, 1.0, dtype=dtype)
    init = X[np.sort(rng.choice(n, k, replace=False))].copy()
    return X, init, 10


CONFIGS = {"c1": c1, "c2": c2, "c3": c3, "c4": c4, "c5": c5}
