"""flashlib_b200 -- the fused squared-L2 distance + top-k hot path of flashlib, rebuilt for
NVIDIA B200 (sm_100a) behind a C ABI.

The public names are the ones flashlib exports for this path
(``flashlib/__init__.py:41-138``): ``flash_knn``, ``flash_kmeans``, ``flash_ivf_flat*``, the
sklearn-style classes ``KMeans`` / ``NearestNeighbors`` / ``IVFFlat`` and the lower-level
entry points whose names callers of the reference import directly.  Attributes are resolved
lazily so that importing the package never needs a GPU.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_LAZY = {
    "flash_knn": "knn", "flash_knn_dispatch": "knn", "flash_knn_triton": "knn",
    "triton_knn_gather_sqdist": "knn", "row_sqnorm": "knn", "topk_merge": "knn", "DbPlane": "knn", "check_pending": "knn",
    "kmeans_largeN": "kmeans_large", "kmeans_largeN_assign": "kmeans_large",
    "flash_kmeans": "kmeans", "batch_kmeans_Euclid": "kmeans", "euclid_assign_triton": "kmeans",
    "triton_lloyd_centroid_step_euclid": "kmeans", "triton_centroid_finalize": "kmeans",
    "triton_centroid_update_euclid": "kmeans", "triton_centroid_update_sorted_euclid": "kmeans",
    "flash_ivf_flat": "ivf_flat", "flash_ivf_flat_build": "ivf_flat", "flash_ivf_flat_search": "ivf_flat",
    "IvfFlatIndex": "ivf_flat",
    "KMeans": "applications", "FlashKMeans": "applications", "NearestNeighbors": "applications",
    "IVFFlat": "applications",
    "sharded_knn": "sharded", "sharded_kmeans": "sharded",
}


def __getattr__(name: str):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'flashlib_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(f".{mod}", __name__), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
