"""CPU restatement (numpy, fp32) of the reference algorithms on the hot path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``flashlib_b200/`` imports this module; it is
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py`` as the checker / timed baseline, never as the product.

The reference (FlashML-org/flashlib) implements these paths in Python on top of torch
CPU operators; every function below cites the file:line it restates.  The arithmetic that
the reference delegates to torch (``bmm``, ``topk``, ``argmin``, ``index_add_``, ``cdist``;
torch 2.11 in this build's environment) is restated with the numpy equivalents in fp32.
Summation order inside a matrix product is not specified by either library, so distances
agree to fp32 round-off, not bit for bit; index sets agree except between candidates whose
distances differ by round-off.

Parity pin: ``tests/golden/*.npz`` were produced by running the reference itself
(``tests/golden/make_golden.py``), and ``tests/test_oracle_golden.py`` checks every function
here against them.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32


def _topk_smallest(dist: np.ndarray, k: int):
    """k smallest entries per row, ascending, ties by lower index (``torch.topk(largest=False,
    sorted=True)`` leaves the tie order unspecified)."""
    n, m = dist.shape
    if k < m:
        part = np.argpartition(dist, k - 1, axis=1)[:, :k]
    else:
        part = np.broadcast_to(np.arange(m), (n, m)).copy()
    pv = np.take_along_axis(dist, part, axis=1)
    order = np.lexsort((part, pv), axis=1)
    idx = np.take_along_axis(part, order, axis=1)
    return np.take_along_axis(dist, idx, axis=1), idx.astype(np.int64)


def knn_naive(x: np.ndarray, c: np.ndarray, k: int):
    """``knn_torch_naive`` -- flashlib/primitives/knn/torch_fallback.py:6-30.

    ``x`` (N, D), ``c`` (M, D): ``dist = x_sq + c_sq^T - 2 x c^T`` clamped at 0, then the k
    smallest per row.  Returns ``(vals fp32 (N,k), idxs int64 (N,k))``.
    """
    x = np.asarray(x, dtype=F32)
    c = np.asarray(c, dtype=F32)
    x_sq = (x * x).sum(-1, keepdims=True, dtype=F32)
    c_sq = (c * c).sum(-1, keepdims=True, dtype=F32)
    cross = x @ c.T
    dist = x_sq + c_sq.T - F32(2.0) * cross
    np.maximum(dist, F32(0.0), out=dist)
    return _topk_smallest(dist, k)


def knn_chunked(x: np.ndarray, c: np.ndarray, k: int, chunk_size: int = 1024):
    """``knn_torch_chunked`` -- flashlib/primitives/knn/torch_fallback.py:33-79: the same
    distances per database chunk with a running top-k over ``[kept | chunk]``."""
    x = np.asarray(x, dtype=F32)
    c = np.asarray(c, dtype=F32)
    n = x.shape[0]
    m = c.shape[0]
    x_sq = (x * x).sum(-1, keepdims=True, dtype=F32)
    top_v = np.full((n, k), np.inf, dtype=F32)
    top_i = np.full((n, k), -1, dtype=np.int64)
    for s in range(0, m, chunk_size):
        e = min(s + chunk_size, m)
        cc = c[s:e]
        c_sq = (cc * cc).sum(-1, keepdims=True, dtype=F32)
        dist = x_sq + c_sq.T - F32(2.0) * (x @ cc.T)
        np.maximum(dist, F32(0.0), out=dist)
        comb_v = np.concatenate([top_v, dist], axis=1)
        comb_i = np.concatenate([top_i, np.broadcast_to(np.arange(s, e), (n, e - s))], axis=1)
        # ties by lower database index; the kept part carries global ids, so sort on them
        kk = min(k, comb_v.shape[1])
        part = np.argpartition(comb_v, kk - 1, axis=1)[:, :kk]
        pv = np.take_along_axis(comb_v, part, axis=1)
        pi = np.take_along_axis(comb_i, part, axis=1)
        order = np.lexsort((pi, pv), axis=1)
        top_v = np.take_along_axis(pv, order, axis=1)
        top_i = np.take_along_axis(pi, order, axis=1)
    return top_v, top_i


def exact_sqdist(x: np.ndarray, c: np.ndarray, idx: np.ndarray) -> np.ndarray:
    """``triton_knn_gather_sqdist`` -- flashlib/kernels/distance/triton/knn_gather_l2sq.py:1-12:
    ``out[i,j] = sum_d (x[i,d] - c[idx[i,j],d])^2`` (fp64 accumulation here; it is the yardstick
    for returned distances)."""
    x = np.asarray(x, dtype=np.float64)
    c = np.asarray(c, dtype=np.float64)
    out = np.empty(idx.shape, dtype=np.float64)
    for j in range(idx.shape[1]):
        diff = x - c[idx[:, j]]
        out[:, j] = (diff * diff).sum(-1)
    return out


# ---------------------------------------------------------------------------------------
# k-means
# ---------------------------------------------------------------------------------------
def kmeans_assign(x: np.ndarray, centroids: np.ndarray, chunk_n: int = 32768, chunk_k: int = 1024):
    """``euclid_assign_torch_native_chunked`` -- flashlib/primitives/kmeans/torch_fallback.py:4-51:
    ``argmin_k (||c_k||^2 - 2 <x, c_k>)`` per point, int32 labels."""
    x = np.asarray(x, dtype=F32)
    c = np.asarray(centroids, dtype=F32)
    n = x.shape[0]
    K = c.shape[0]
    c_sq = (c * c).sum(-1, dtype=F32)
    out = np.empty(n, dtype=np.int32)
    for s in range(0, n, chunk_n):
        e = min(s + chunk_n, n)
        d = np.empty((e - s, K), dtype=F32)
        for ks in range(0, K, chunk_k):
            ke = min(ks + chunk_k, K)
            d[:, ks:ke] = c_sq[None, ks:ke] - F32(2.0) * (x[s:e] @ c[ks:ke].T)
        out[s:e] = d.argmin(-1)
    return out


def kmeans_score_gap(x: np.ndarray, centroids: np.ndarray, labels: np.ndarray):
    """For each point: (true squared distance to centroid ``labels[i]``, smallest true squared
    distance to any centroid) in fp64 -- used to accept label differences inside a tie band."""
    x = np.asarray(x, dtype=np.float64)
    c = np.asarray(centroids, dtype=np.float64)
    d = (x * x).sum(-1, keepdims=True) + (c * c).sum(-1)[None, :] - 2.0 * (x @ c.T)
    return d[np.arange(x.shape[0]), labels], d.min(-1)


def kmeans_update(x: np.ndarray, labels: np.ndarray, old_centroids: np.ndarray):
    """``_centroid_update_torch_native`` -- flashlib/primitives/kmeans/torch_fallback.py:71-107:
    fp32 sums and counts per cluster; an empty cluster keeps its old centroid."""
    x = np.asarray(x, dtype=F32)
    old = np.asarray(old_centroids, dtype=F32)
    K, D = old.shape
    sums = np.zeros((K, D), dtype=F32)
    np.add.at(sums, labels, x)
    cnts = np.bincount(labels, minlength=K).astype(F32)
    empty = cnts == 0
    new = sums / np.maximum(cnts, F32(1.0))[:, None]
    new[empty] = old[empty]
    return new.astype(F32), sums, cnts.astype(np.int64)


def kmeans_iter(x, centroids):
    """``_euclid_iter_torch_naive`` -- flashlib/primitives/kmeans/torch_fallback.py:110-132."""
    labels = kmeans_assign(x, centroids)
    new, _, _ = kmeans_update(x, labels, centroids)
    shift = np.sqrt(((new - centroids) ** 2).sum(-1, dtype=F32)).max()
    return new, shift, labels


def kmeans(x, n_clusters: int, max_iters: int = 100, tol: float = 0.0, init_centroids=None,
           return_history: bool = False):
    """``batch_kmeans_Euclid_torch_native`` (one batch) --
    flashlib/primitives/kmeans/torch_fallback.py:134-172.  Returns ``(labels of the last
    assignment, centroids, iterations)``; as in the reference the centroids returned are the
    ones the last assignment used when the loop breaks on ``shift < tol``, and the updated ones
    otherwise."""
    if init_centroids is None:
        raise ValueError("the oracle needs explicit init_centroids (the reference draws them from torch's RNG)")
    c = np.asarray(init_centroids, dtype=F32).reshape(n_clusters, -1).copy()
    hist = []
    labels = None
    it = 0
    for it in range(max_iters):
        new, shift, labels = kmeans_iter(x, c)
        hist.append((c.copy(), labels.copy(), new.copy()))
        if shift < tol:
            break
        c = new.copy()
    if return_history:
        return labels, c, it + 1, hist
    return labels, c, it + 1


# ---------------------------------------------------------------------------------------
# IVF-Flat
# ---------------------------------------------------------------------------------------
def pad_features(x: np.ndarray, Dp: int) -> np.ndarray:
    """``_pad_features`` -- flashlib/primitives/ivf_flat/torch_fallback.py:22-28."""
    D = x.shape[-1]
    if D >= Dp:
        return x
    return np.concatenate([x, np.zeros((*x.shape[:-1], Dp - D), dtype=x.dtype)], axis=-1)


def cdist_sq(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``torch.cdist(a, b) ** 2`` as the reference calls it
    (ivf_flat/torch_fallback.py:41,85,128): the euclidean distance through the matrix-product
    expansion, clamped at zero, square-rooted and squared again in fp32."""
    a = np.asarray(a, dtype=F32)
    b = np.asarray(b, dtype=F32)
    d2 = (a * a).sum(-1, keepdims=True, dtype=F32) + (b * b).sum(-1, dtype=F32)[None, :] - F32(2.0) * (a @ b.T)
    np.maximum(d2, F32(0.0), out=d2)
    d = np.sqrt(d2)
    return d * d


def ivf_assign_lists(Xp: np.ndarray, centroids: np.ndarray):
    """The CSR layout step of ``ivf_flat_build_torch`` --
    flashlib/primitives/ivf_flat/torch_fallback.py:85-96: nearest centroid per row, counts,
    offsets, stable order."""
    nlist = centroids.shape[0]
    assign = np.empty(Xp.shape[0], dtype=np.int64)
    for s in range(0, Xp.shape[0], 65536):
        assign[s:s + 65536] = cdist_sq(Xp[s:s + 65536], centroids).argmin(1)
    counts = np.bincount(assign, minlength=nlist)
    offsets = np.zeros(nlist + 1, dtype=np.int64)
    offsets[1:] = np.cumsum(counts)
    order = np.argsort(assign, kind="stable")
    return assign, offsets, order


def ivf_search(centroids, data, ids, list_offsets, Q, k: int, nprobe: int, probed=None):
    """``ivf_flat_search_torch`` -- flashlib/primitives/ivf_flat/torch_fallback.py:113-151:
    probe the ``nprobe`` nearest lists (``cdist^2`` top-nprobe), compute ``sum (q - x)^2``
    directly for every row of those lists and keep the k smallest.  Returns
    ``(vals fp32 (nq,k) inf-padded, ids int64 (nq,k) -1-padded, probed (nq,nprobe))``."""
    centroids = np.asarray(centroids, dtype=F32)
    data = np.asarray(data, dtype=F32)
    Dp = data.shape[1]
    Qp = pad_features(np.asarray(Q, dtype=F32), Dp)
    nq = Qp.shape[0]
    nlist = centroids.shape[0]
    nprobe = min(nprobe, nlist)
    if probed is None:
        _, probed = _topk_smallest(cdist_sq(Qp, centroids), nprobe)
    out_v = np.full((nq, k), np.inf, dtype=F32)
    out_i = np.full((nq, k), -1, dtype=np.int64)
    for i in range(nq):
        pos = [np.arange(list_offsets[c], list_offsets[c + 1]) for c in probed[i]
               if list_offsets[c + 1] > list_offsets[c]]
        if not pos:
            continue
        pos = np.concatenate(pos)
        diff = Qp[i][None, :] - data[pos]
        dist = (diff * diff).sum(1, dtype=F32)
        kk = min(k, dist.shape[0])
        v, sel = _topk_smallest(dist[None, :], kk)
        out_v[i, :kk] = v[0]
        out_i[i, :kk] = ids[pos[sel[0]]]
    return out_v, out_i, probed
