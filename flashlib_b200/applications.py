"""sklearn-style wrappers with the reference's class names and constructor arguments.

``KMeans`` follows ``flashlib/applications/kmeans.py:30-286``, ``NearestNeighbors``
``flashlib/applications/knn.py:13-58`` and ``IVFFlat`` ``flashlib/applications/ivf_flat.py:25-105``.
They hold fitted state and call the functional API; there is no PyTorch or CPU fallback, so
arguments that select one in the reference (``use_triton=False``, ``backend="torch"``) raise.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ivf_flat import flash_ivf_flat_build, flash_ivf_flat_search
from .kmeans import batch_kmeans_Euclid, euclid_assign_triton
from .knn import DbPlane, flash_knn_dispatch


class KMeans:
    """Batched Lloyd k-means.  Constructor arguments as in the reference (``d``, ``k``,
    ``niter=25``, ``tol=1e-8``, ``seed=0``, ...); the chunking knobs of the reference's
    PyTorch fallback are accepted and unused."""

    def __init__(self, d: int, k: int, niter: int = 25, tol: float = 1e-8, use_triton: bool = True,
                 seed: int = 0, chunk_size_data: int = 32768, chunk_size_centroids: int = 1024,
                 chunk_size_data_cpu: int = 1048576, verbose: bool = False,
                 dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None):
        if not use_triton:
            raise NotImplementedError("flashlib_b200 has no PyTorch fallback (use_triton=False)")
        self.d = int(d)
        self.k = int(k)
        self.niter = int(niter)
        self.tol = float(tol)
        self.use_triton = True
        self.seed = int(seed)
        self.chunk_size_data = int(chunk_size_data)
        self.chunk_size_centroids = int(chunk_size_centroids)
        self.chunk_size_data_cpu = int(chunk_size_data_cpu)
        self.verbose = bool(verbose)
        self.dtype = dtype
        self.device = torch.device("cuda:0") if device is None else torch.device(device)
        self.centroids_b = None
        self.cluster_ids_b = None
        self._batch_size = None

    def _as_batch(self, data: torch.Tensor):
        if data.ndim == 2:
            return None, data.unsqueeze(0)
        if data.ndim == 3:
            return data.shape[0], data
        raise ValueError("data must be of shape (n_samples, n_features) or "
                         "(batch_size, n_samples, n_features)")

    def train(self, data: torch.Tensor):
        """Fit on ``data``; seeds torch's generators first, like the reference
        (``applications/kmeans.py:136-137``), so the ``randint`` initialisation matches."""
        B, x_b = self._as_batch(data)
        torch.manual_seed(self.seed)
        torch.cuda.manual_seed_all(self.seed)
        if data.device.type == "cpu" and x_b.shape[1] > self.chunk_size_data_cpu:
            # host-resident data too large to copy in one piece: streamed in blocks, as the reference
            # does (applications/kmeans.py:139-156)
            if B is not None:
                raise AssertionError("Batched data with large N on CPU is not supported yet.")
            from .kmeans_large import kmeans_largeN
            ids, cents = kmeans_largeN(x_b[0], self.k, max_iters=self.niter, tol=self.tol, verbose=self.verbose,
                                       dtype=self.dtype, BLOCK_N=self.chunk_size_data_cpu, device=self.device)
            self.centroids_b = cents.unsqueeze(0)
            self.cluster_ids_b = ids.unsqueeze(0)
            self._batch_size = B
            return
        x_b = x_b.to(device=self.device, dtype=self.dtype or x_b.dtype)
        ids, cents, _ = batch_kmeans_Euclid(x_b, self.k, max_iters=self.niter, tol=self.tol,
                                            init_centroids=None, verbose=self.verbose)
        self.centroids_b = cents
        self.cluster_ids_b = ids
        self._batch_size = B

    def fit(self, data: torch.Tensor):
        self.train(data)
        return self

    def predict(self, data: torch.Tensor) -> torch.Tensor:
        if self.centroids_b is None:
            raise RuntimeError("Model not trained. Call train() or fit() first.")
        B, x_b = self._as_batch(data)
        if B != self._batch_size:
            raise ValueError(f"Model was trained with batch size B={self._batch_size}, "
                             f"but predict received B={B}. Provide matching batch size.")
        if data.device.type == "cpu" and x_b.shape[1] > self.chunk_size_data_cpu:
            if B is not None:
                raise AssertionError("Batched data with large N on CPU is not supported yet.")
            from .kmeans_large import kmeans_largeN_assign
            return kmeans_largeN_assign(x_b[0], self.centroids_b[0], BLOCK_N=self.chunk_size_data_cpu,
                                        device=self.device)
        x_b = x_b.to(device=self.device, dtype=self.dtype or x_b.dtype)
        labels = euclid_assign_triton(x_b, self.centroids_b.to(x_b.dtype))
        return labels.squeeze(0) if B is None else labels

    def fit_predict(self, data: torch.Tensor) -> torch.Tensor:
        self.train(data)
        return self.cluster_ids_b.squeeze(0) if self._batch_size is None else self.cluster_ids_b


FlashKMeans = KMeans


class NearestNeighbors:
    """Exact nearest-neighbour search over a fitted database (squared L2)."""

    def __init__(self, n_neighbors: int = 5, *, backend: Optional[str] = None):
        self.n_neighbors = int(n_neighbors)
        self.backend = backend
        self._X = None

    def fit(self, X: torch.Tensor) -> "NearestNeighbors":
        if not X.is_cuda or X.ndim != 2:
            raise ValueError("NearestNeighbors requires a 2D CUDA tensor")
        self._X = X
        return self

    def kneighbors(self, Q: Optional[torch.Tensor] = None, n_neighbors: Optional[int] = None,
                   return_distance: bool = True, *, backend: Optional[str] = None):
        if self._X is None:
            raise RuntimeError("NearestNeighbors not fitted; call fit() first.")
        k = n_neighbors if n_neighbors is not None else self.n_neighbors
        if Q is None:
            Q = self._X
        res = flash_knn_dispatch(Q.unsqueeze(0), self._X.unsqueeze(0), k, backend=backend or self.backend,
                                 return_distances=return_distance)
        if return_distance:
            return res[0].squeeze(0), res[1].squeeze(0)
        return res.squeeze(0)


class IVFFlat:
    """Approximate nearest neighbours via an inverted-file index (``nlist`` lists, ``nprobe``
    probed per query)."""

    def __init__(self, nlist: int = 1024, *, nprobe: int = 8, n_neighbors: int = 5, metric: str = "l2",
                 niter: int = 20, train_size: Optional[int] = None, seed: int = 0,
                 backend: Optional[str] = None):
        self.nlist = int(nlist)
        self.nprobe = int(nprobe)
        self.n_neighbors = int(n_neighbors)
        self.metric = metric
        self.niter = int(niter)
        self.train_size = train_size
        self.seed = int(seed)
        self.backend = backend
        self.index_ = None

    def fit(self, X: torch.Tensor) -> "IVFFlat":
        if X.ndim != 2:
            raise ValueError("IVFFlat requires a 2D (M, D) tensor")
        self.index_ = flash_ivf_flat_build(X, self.nlist, metric=self.metric, nprobe=self.nprobe,
                                           niter=self.niter, train_size=self.train_size, seed=self.seed,
                                           backend=self.backend)
        return self

    def kneighbors(self, Q: torch.Tensor, n_neighbors: Optional[int] = None, return_distance: bool = True,
                   *, nprobe: Optional[int] = None, variant: str = "auto"):
        if self.index_ is None:
            raise RuntimeError("IVFFlat not fitted; call fit() first.")
        k = n_neighbors if n_neighbors is not None else self.n_neighbors
        vals, ids = flash_ivf_flat_search(self.index_, Q, k, nprobe=nprobe or self.nprobe,
                                          backend=self.backend, variant=variant)
        if return_distance:
            return vals, ids
        return ids

    def fit_kneighbors(self, X, Q, n_neighbors=None, **kw):
        return self.fit(X).kneighbors(Q, n_neighbors=n_neighbors, **kw)


__all__ = ["KMeans", "FlashKMeans", "NearestNeighbors", "IVFFlat", "DbPlane"]
