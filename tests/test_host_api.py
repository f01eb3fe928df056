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


def test_cache_entries_die_with_their_tensor():
    """Operand-plane caches are keyed by address, shape and version; an entry must go when the
    tensor that owns the memory is freed, because a new tensor can be given the same key."""
    import gc
    import torch
    from flashlib_b200.knn import _evict_when_freed, _plane_key
    cache = {}
    base = torch.zeros(8, 4)
    view = base[2:6]
    cache[_plane_key(view)] = "plane of a view"
    _evict_when_freed(cache, _plane_key(view), view)
    key = _plane_key(view)
    del view
    gc.collect()
    assert key in cache            # the owner of the memory is still alive
    del base
    gc.collect()
    assert key not in cache


def test_large_kmeans_block_partition():
    """Blocks of the host-resident sample set are dealt to the ranks contiguously, the first
    ranks taking the remainder (flashlib/primitives/kmeans/large.py:74-78)."""
    from flashlib_b200.kmeans_large import block_range
    assert [block_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [block_range(2, 4, r) for r in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    assert block_range(7, 1, 0) == (0, 7)
