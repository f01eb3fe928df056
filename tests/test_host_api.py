"""Host-side behaviour of the Python mirror that needs no GPU: argument validation and
error types follow the reference's."""
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200 import synthetic


def test_lazy_names_resolve():
    for name in ("flash_knn", "flash_kmeans", "flash_ivf_flat_build", "flash_ivf_flat_search",
                 "KMeans", "NearestNeighbors", "IVFFlat", "euclid_assign_triton",
                 "triton_knn_gather_sqdist", "IvfFlatIndex"):
        assert getattr(fl, name) is not None
    with pytest.raises(AttributeError):
        fl.not_a_name


def test_knn_rejects_unknown_backend_and_cpu():
    x = torch.zeros(4, 8)
    with pytest.raises(ValueError):
        fl.flash_knn(x, x, 1, backend="cuda")      # knn/impl.py:52-57
    with pytest.raises(RuntimeError):
        fl.flash_knn(x, x, 1)                       # no CPU fallback in this library


def test_kmeans_metric_errors():
    x = torch.zeros(8, 4)
    with pytest.raises(NotImplementedError):
        fl.flash_kmeans(x, 2, metric="cosine")
    with pytest.raises(ValueError):
        fl.flash_kmeans(x, 2, metric="manhattan")
    with pytest.raises(RuntimeError):
        fl.flash_kmeans(x, 2)


def test_app_classes_unfitted():
    with pytest.raises(RuntimeError):
        fl.NearestNeighbors().kneighbors(torch.zeros(2, 2))
    with pytest.raises(RuntimeError):
        fl.IVFFlat().kneighbors(torch.zeros(2, 2))
    with pytest.raises(ValueError):
        fl.NearestNeighbors().fit(torch.zeros(2, 2))   # CPU tensor
    with pytest.raises(ValueError):
        fl.IVFFlat().fit(torch.zeros(2, 2, 2))


def test_synthetic_is_seeded():
    a, qa = synthetic.mixture(100, 8, 4, seed=5, nq=10, clamp=True)
    b, qb = synthetic.mixture(100, 8, 4, seed=5, nq=10, clamp=True)
    assert torch.equal(a, b) and torch.equal(qa, qb) and a.min() >= 0
