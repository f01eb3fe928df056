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


def test_kmeans_class_routes_large_host_data_to_the_streaming_path(monkeypatch):
    """CPU-resident data with more rows than chunk_size_data_cpu goes to kmeans_largeN /
    kmeans_largeN_assign with that block size (flashlib/applications/kmeans.py:139-156, 229-240),
    not to one whole-tensor copy."""
    import torch
    import flashlib_b200.kmeans_large as large
    from flashlib_b200.applications import KMeans
    calls = {}

    def fake_fit(x, k, **kw):
        calls["fit"] = (tuple(x.shape), k, kw["BLOCK_N"], kw["max_iters"])
        return torch.zeros(x.shape[0], dtype=torch.int32), torch.zeros(k, x.shape[1])

    def fake_assign(x, c, **kw):
        calls["assign"] = (tuple(x.shape), tuple(c.shape), kw["BLOCK_N"])
        return torch.zeros(x.shape[0], dtype=torch.int32)

    monkeypatch.setattr(large, "kmeans_largeN", fake_fit)
    monkeypatch.setattr(large, "kmeans_largeN_assign", fake_assign)
    km = KMeans(d=4, k=3, niter=2, chunk_size_data_cpu=100, device="cpu")
    x = torch.randn(250, 4)
    assert km.fit_predict(x).shape == (250,)
    assert calls["fit"] == ((250, 4), 3, 100, 2)
    assert km.predict(x).shape == (250,)
    assert calls["assign"] == ((250, 4), (3, 4), 100)


def test_ivf_index_save_and_load_round_trip(tmp_path):
    """Index persistence (torch.save of the reference's IvfFlatIndex fields): every field comes
    back, caches are left to be rebuilt, a foreign file is refused."""
    import torch
    from flashlib_b200.ivf_flat import IvfFlatIndex, load_ivf_flat_index
    g = torch.Generator().manual_seed(0)
    idx = IvfFlatIndex(centroids=torch.randn(3, 16, generator=g), data=torch.randn(10, 16, generator=g),
                       ids=torch.randperm(10, generator=g), list_offsets=torch.tensor([0, 4, 4, 10]), metric="l2",
                       D=12, Dp=16, nlist=3, nprobe=2, max_list_len=torch.tensor([6], dtype=torch.int32))
    path = tmp_path / "index.pt"
    idx.save(path)
    back = load_ivf_flat_index(path)
    for f in ("centroids", "data", "ids", "list_offsets"):
        assert torch.equal(getattr(back, f), getattr(idx, f))
    assert (back.metric, back.D, back.Dp, back.nlist, back.nprobe, back.max_list_len) == ("l2", 12, 16, 3, 2, 6)
    assert back._tc_plane is None and back._hnorm is None
    assert isinstance(IvfFlatIndex.load(path), IvfFlatIndex)
    other = tmp_path / "other.pt"
    torch.save({"format": "something else"}, other)
    import pytest
    with pytest.raises(ValueError):
        load_ivf_flat_index(other)


def test_tol_to_storage_dtype_follows_the_reference_rule():
    """Pairs recorded from the reference's ``storage_dtype_for`` (flashlib/linalg/gemm/__init__.py:163-207):
    fp16 from its declared residual 4e-4 upwards (it out-ranks bf16 by listed throughput wherever both
    qualify), nothing below (tf32 alone qualifies from 3e-4 and names no storage dtype)."""
    import torch
    from flashlib_b200.knn import storage_dtype_for
    recorded = [(None, None), (0, None), (-1, None), (1e-8, None), (1e-6, None), (2e-4, None), (3e-4, None), (3.5e-4, None),
                (4e-4, torch.float16), (1e-3, torch.float16), (3e-3, torch.float16), (1e-2, torch.float16), (1.0, torch.float16)]
    for tol, want in recorded:
        assert storage_dtype_for(tol) is want, (tol, want)
