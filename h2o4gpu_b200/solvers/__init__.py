from .kmeans import KMeans, KMeansH2O  # noqa: F401
