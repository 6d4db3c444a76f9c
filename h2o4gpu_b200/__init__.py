"""B200-native k-means engine behind the k-means interface of h2o4gpu.

``KMeans`` / ``KMeansH2O`` mirror the reference's estimators
(src/interface_py/h2o4gpu/solvers/kmeans.py); ``ResidentKMeans`` drives the
engine on data that already lives on the GPU(s).  The compute path is
``libh2o4gpu_kmeans.so`` (CUDA, sm_100a); there is no CPU implementation.
"""
from .solvers.kmeans import KMeans, KMeansH2O  # noqa: F401
from .engine import ResidentKMeans  # noqa: F401

__all__ = ["KMeans", "KMeansH2O", "ResidentKMeans"]
