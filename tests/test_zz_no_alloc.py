"""The allocation-free centroid-sum entry point against the ordinary one.

Collected last on purpose (file name): if it fails, a run that stops at the first
failure has already been through every other test.

Who needs it: callers that may not allocate device memory at the point of the call,
for instance a serving loop whose memory is fixed after start-up, or a host where the
synchronisation hidden in cudaMalloc/cudaFree would stall other streams.  The test
drives it with device pointers only (inputs and
outputs are torch tensors made beforehand) and checks two consecutive calls, since
the static scratch array keeps the previous call's numbers until it is cleared.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ordinary(X, labels, k):
    from h2o4gpu_b200 import engine
    return engine.centroid_sums(X, labels, k)


def _no_alloc(lib, X, labels, k, check_driver_free=False):
    import torch
    dev = torch.device("cuda", 0)
    dX = torch.from_numpy(X).to(dev)
    dL = torch.from_numpy(labels).to(dev)
    dS = torch.full((k, X.shape[1]), float("nan"), dtype=torch.float64, device=dev)
    dC = torch.full((k,), -7, dtype=torch.int64, device=dev)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]      # the driver's view: sees any allocation, not only torch's
    rc = lib.kmeans_centroid_sums_noalloc_f32(ctypes.c_void_p(dX.data_ptr()), ctypes.c_void_p(dL.data_ptr()),
                                              X.shape[0], X.shape[1], k, ctypes.c_void_p(dS.data_ptr()),
                                              ctypes.c_void_p(dC.data_ptr()), None)
    assert rc == 0, lib.kmeans_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    if check_driver_free:
        assert torch.cuda.mem_get_info()[0] == free_before
    return dS.cpu().numpy(), dC.cpu().numpy()


def test_no_alloc_matches_ordinary_entry_point_twice(built_lib):
    import torch
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.cdll()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(11)
    # two different problems back to back: the second must not see the first one's sums
    cases = [(40_000, 64, 100), (9_001, 7, 5)]
    for n, d, k in cases:
        X = (rng.standard_normal((n, d)) * 5 + 3).astype(np.float32)
        labels = rng.integers(0, k, n).astype(np.int32)
        s_ref, c_ref = _ordinary(X, labels, k)
        s, c = _no_alloc(lib, X, labels, k)
        assert np.array_equal(c, c_ref)
        # both paths add the same fixed-point pieces: equal up to the final conversion
        assert np.abs(s - s_ref).max() <= 1e-9 * max(np.abs(s_ref).max(), 1.0)
        exact = np.zeros((k, d))
        np.add.at(exact, labels, X.astype(np.float64))
        assert np.abs(s - exact).max() <= 1e-4 * np.abs(exact).max()      # the suite's float32 tolerance
    # the same call again on the first problem gives the same bits
    n, d, k = cases[0]
    X = (np.random.default_rng(5).standard_normal((n, d)) * 2).astype(np.float32)
    labels = np.random.default_rng(6).integers(0, k, n).astype(np.int32)
    a = _no_alloc(lib, X, labels, k)
    b = _no_alloc(lib, X, labels, k, check_driver_free=True)   # a warm call leaves the device's free memory as it was
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_no_alloc_rejects_sizes_beyond_the_scratch(built_lib):
    from h2o4gpu_b200.libs import lib_kmeans
    lib = lib_kmeans.cdll()
    one = ctypes.c_void_p(256)   # never dereferenced: the size check comes first
    rc = lib.kmeans_centroid_sums_noalloc_f32(one, one, 10, 1000, 100, one, one, None)
    assert rc == -1 and b"exceeds the static scratch" in lib.kmeans_last_error()
