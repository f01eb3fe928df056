"""Lloyd k-means behind flashlib's ``flash_kmeans`` / ``batch_kmeans_Euclid`` API.

Mirrors ``flashlib/primitives/kmeans/impl.py:110-189`` and the fused loop of
``flashlib/primitives/kmeans/triton/kmeans.py:61-153`` (ping-pong centroid buffers,
preallocated sums/counts/shift, no host synchronisation while ``tol == 0``).  The
function names of the reference's Triton entry points are kept so callers can switch
imports; all of them run the sm_100a kernels behind the C ABI.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib
from .knn import _as_f32_rows, _defer_status_check, _evict_when_freed, _stream_ptr


_XPLANE_CACHE = {}


def _x_plane(x: torch.Tensor) -> torch.Tensor:
    """bf16 operand plane of the sample rows for the tensor-core assignment, built once per
    data set (keyed like the reference's per-``data_ptr`` norm cache,
    ``flashlib/primitives/knn/triton/_row_norm.py:82-93``)."""
    key = (x.data_ptr(), tuple(x.shape), x.stride(0), x._version, x.device.index)
    hit = _XPLANE_CACHE.get(key)
    if hit is not None:
        return hit
    lib = _lib.load()
    n, d = x.shape
    nbytes = lib.fl_kmeans_xplane_bytes(n, d)
    buf = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    _lib.check(lib.fl_kmeans_prepare_x_f32(x.data_ptr(), n, d, x.stride(0), buf.data_ptr(), nbytes,
                                           _stream_ptr(x.device)))
    if len(_XPLANE_CACHE) >= 2:
        _XPLANE_CACHE.pop(next(iter(_XPLANE_CACHE)))
    _XPLANE_CACHE[key] = buf
    _evict_when_freed(_XPLANE_CACHE, key, x)
    return buf


def _use_tensor_cores(n: int, K: int, d: int, mode: Optional[str]) -> bool:
    if mode in ("exact", "simt"):
        return False
    if d > 256:
        if mode in ("bf16", "tc"):
            raise NotImplementedError("tensor-core assignment supports d <= 256")
        return False
    if mode in ("bf16", "tc"):
        return True
    return n * K >= (1 << 24) and K >= 64


def _assign_2d(x: torch.Tensor, c: torch.Tensor, out: torch.Tensor, mode: Optional[str] = None) -> None:
    lib = _lib.load()
    n, d = x.shape
    K = c.shape[0]
    if mode is None:
        mode = os.environ.get("FLASHLIB_B200_ASSIGN_MODE") or None
    if _use_tensor_cores(n, K, d, mode):
        xplane = _x_plane(x)
        ws_bytes = lib.fl_kmeans_assign_tc_workspace_bytes(n, K, d, 1)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
        status = torch.zeros(_lib.FL_STATUS_WORDS, dtype=torch.int32, device=x.device)
        _lib.check(lib.fl_kmeans_assign_tc_f32(x.data_ptr(), n, x.stride(0), xplane.data_ptr(), c.data_ptr(), K,
                                               c.stride(0), d, out.data_ptr(), ws.data_ptr(), ws_bytes,
                                               status.data_ptr(), _stream_ptr(x.device)))
        # a bounded wait that gave up leaves garbage labels: the status words are looked at by a
        # later call or by check_pending(), without a host round trip per iteration
        _defer_status_check(status)
        return
    ws_bytes = lib.fl_kmeans_assign_workspace_bytes(n, K, d)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    _lib.check(lib.fl_kmeans_assign_f32(x.data_ptr(), n, x.stride(0), c.data_ptr(), K, c.stride(0), d,
                                        out.data_ptr(), ws.data_ptr(), ws_bytes, _stream_ptr(x.device)))


def euclid_assign_triton(x: torch.Tensor, centroids: torch.Tensor, out: Optional[torch.Tensor] = None,
                         c_sq: Optional[torch.Tensor] = None, *, mode: Optional[str] = None,
                         **_ignored) -> torch.Tensor:
    """Nearest-centroid labels ``(B, N) int32`` (lowest index on exact ties).

    Same arguments as ``flashlib/primitives/kmeans/triton/assign.py:1439-1479``; ``c_sq`` and
    the tile-config keywords are accepted and ignored (norms are computed on the device).
    ``mode`` (``"exact"`` | ``"bf16"`` | ``None`` = by size) picks the CUDA-core or the tensor-core kernel;
    both return the same labels.
    """
    assert x.is_cuda and centroids.is_cuda, "All tensors must be on CUDA"
    assert centroids.dtype == x.dtype, "centroids dtype mismatch"
    B, N, D = x.shape
    K = centroids.shape[1]
    assert centroids.shape == (B, K, D), "centroids shape mismatch"
    _lib.require_device()
    if out is None:
        out = torch.empty((B, N), device=x.device, dtype=torch.int32)
    else:
        assert out.shape == (B, N) and out.dtype == torch.int32 and out.is_contiguous()
    if mode is None:
        mode = os.environ.get("FLASHLIB_B200_ASSIGN_MODE") or None
    with torch.cuda.device(x.device):
        if B > 1 and not _use_tensor_cores(N, K, D, mode):
            # many small problems (IVF-PQ's sub-quantisers: a few features, 256 centroids each):
            # one launch with the batch on a grid axis instead of 2 B launches
            lib = _lib.load()
            xb = x.float().contiguous()
            cb = centroids.float().contiguous()
            ws_bytes = lib.fl_kmeans_assign_batch_workspace_bytes(B, N, K, D)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
            _lib.check(lib.fl_kmeans_assign_batch_f32(xb.data_ptr(), B, N, xb.stride(1), xb.stride(0), cb.data_ptr(), K,
                                                      cb.stride(1), cb.stride(0), D, out.data_ptr(), ws.data_ptr(),
                                                      ws_bytes, _stream_ptr(x.device)))
            return out
        for b in range(B):
            _assign_2d(_as_f32_rows(x[b]), _as_f32_rows(centroids[b]), out[b], mode)
    return out


def triton_centroid_update_euclid(x: torch.Tensor, cluster_ids: torch.Tensor, old_centroids: torch.Tensor,
                                  *, centroid_sums: Optional[torch.Tensor] = None,
                                  centroid_cnts: Optional[torch.Tensor] = None, calculate_new: bool = True,
                                  **_ignored):
    """Per-cluster sums ``(B,K,D) fp32`` and counts ``(B,K) int32``; with ``calculate_new`` the
    new centroids (empty clusters keep the old centroid), as
    ``flashlib/primitives/kmeans/triton/update.py:313-384``."""
    lib = _lib.load()
    _lib.require_device()
    B, N, D = x.shape
    K = old_centroids.shape[1]
    if centroid_sums is None:
        centroid_sums = torch.empty((B, K, D), device=x.device, dtype=torch.float32)
    if centroid_cnts is None:
        centroid_cnts = torch.empty((B, K), device=x.device, dtype=torch.int32)
    assert centroid_sums.is_contiguous() and centroid_cnts.is_contiguous()
    with torch.cuda.device(x.device):
        if B > 1:
            xb = x.float().contiguous()
            lab = cluster_ids.to(torch.int32).contiguous()
            _lib.check(lib.fl_kmeans_update_batch_f32(xb.data_ptr(), B, N, xb.stride(1), D, lab.data_ptr(), K,
                                                      centroid_sums.data_ptr(), centroid_cnts.data_ptr(),
                                                      _stream_ptr(x.device)))
        else:
            xb = _as_f32_rows(x[0])
            lab = cluster_ids[0]
            if lab.dtype != torch.int32 or not lab.is_contiguous():
                lab = lab.to(torch.int32).contiguous()
            _lib.check(lib.fl_kmeans_update_f32(xb.data_ptr(), N, xb.stride(0), D, lab.data_ptr(), K,
                                                centroid_sums[0].data_ptr(), centroid_cnts[0].data_ptr(),
                                                _stream_ptr(x.device)))
    if not calculate_new:
        return centroid_sums, centroid_cnts
    new, _ = triton_centroid_finalize(centroid_sums, centroid_cnts, old_centroids)
    return new


triton_centroid_update_sorted_euclid = triton_centroid_update_euclid


def triton_centroid_finalize(sums: torch.Tensor, cnts: torch.Tensor, old_centroids: torch.Tensor, *,
                             out: Optional[torch.Tensor] = None, shift: Optional[torch.Tensor] = None,
                             **_ignored):
    """``new = cnt ? sums / cnt : old`` and ``shift[b,k] = ||new - old||_2``
    (``flashlib/primitives/kmeans/triton/update.py:456-498``)."""
    assert sums.is_cuda and cnts.is_cuda and old_centroids.is_cuda
    B, K, D = sums.shape
    assert cnts.shape == (B, K)
    assert old_centroids.shape == (B, K, D)
    lib = _lib.load()
    _lib.require_device()
    old32 = old_centroids if old_centroids.dtype == torch.float32 else old_centroids.float()
    old32 = old32.contiguous()
    direct = out is not None and out.dtype == torch.float32 and out.is_contiguous()
    new32 = out if direct else torch.empty((B, K, D), device=sums.device, dtype=torch.float32)
    if shift is None:
        shift = torch.empty((B, K), device=sums.device, dtype=torch.float32)
    sums = sums.contiguous()
    cnts = cnts.contiguous()
    assert shift.is_contiguous() and new32.is_contiguous()
    with torch.cuda.device(sums.device):
        # the (B, K, D) arrays are contiguous: the batch is K * B centroids to the kernel
        _lib.check(lib.fl_kmeans_finalize_f32(sums.data_ptr(), cnts.data_ptr(), old32.data_ptr(), new32.data_ptr(),
                                              shift.data_ptr(), K * B, D, _stream_ptr(sums.device)))
    if direct:
        return out, shift
    if out is None:
        return new32.to(old_centroids.dtype), shift
    out.copy_(new32)
    return out, shift


def centroid_update_delta(x: torch.Tensor, cluster_ids: torch.Tensor, prev_ids: torch.Tensor,
                          centroid_sums: torch.Tensor, centroid_cnts: torch.Tensor) -> None:
    """Brings ``centroid_sums (1,K,D)`` / ``centroid_cnts (1,K)`` from the labels in ``prev_ids``
    to those in ``cluster_ids`` by moving only the rows whose label changed, and copies the labels
    into ``prev_ids`` (``fl_kmeans_update_delta_f32``).  ``x`` is ``(1, N, D)`` fp32."""
    lib = _lib.load()
    xb = x[0]
    assert xb.dtype == torch.float32 and xb.stride(1) == 1
    assert cluster_ids.dtype == torch.int32 and prev_ids.dtype == torch.int32
    assert cluster_ids.is_contiguous() and prev_ids.is_contiguous() and centroid_sums.is_contiguous()
    K, D = centroid_sums.shape[1], centroid_sums.shape[2]
    with torch.cuda.device(x.device):
        _lib.check(lib.fl_kmeans_update_delta_f32(xb.data_ptr(), xb.shape[0], xb.stride(0), D, cluster_ids.data_ptr(),
                                                  prev_ids.data_ptr(), K, centroid_sums.data_ptr(),
                                                  centroid_cnts.data_ptr(), _stream_ptr(x.device)))


# Lloyd iterations between two full recomputations of the sums when they are maintained
# incrementally: bounds the rounding drift of adding and taking out rows.
DELTA_REFRESH = 16


def triton_lloyd_centroid_step_euclid(x: torch.Tensor, cluster_ids: torch.Tensor, old_centroids: torch.Tensor,
                                      *, sums_buf: Optional[torch.Tensor] = None,
                                      cnts_buf: Optional[torch.Tensor] = None,
                                      new_buf: Optional[torch.Tensor] = None,
                                      shift_buf: Optional[torch.Tensor] = None,
                                      prev_ids: Optional[torch.Tensor] = None, refresh: bool = True,
                                      want_shift: bool = True, **_ignored):
    """One centroid step: sums/counts, finalize, max shift
    (``flashlib/primitives/kmeans/triton/update.py:501-554``).  Returns
    ``(new_centroids, cluster_ids, max_shift)`` with ``max_shift`` a 0-d device tensor.
    With ``prev_ids`` (B = 1; the labels ``sums_buf`` / ``cnts_buf`` currently stand for) and
    ``refresh=False`` the sums are brought up to date from the changed labels only."""
    if prev_ids is not None and not refresh and x.shape[0] == 1 and x.dtype == torch.float32:
        centroid_update_delta(x, cluster_ids, prev_ids, sums_buf, cnts_buf)
    else:
        sums_buf, cnts_buf = triton_centroid_update_euclid(
            x, cluster_ids, old_centroids, centroid_sums=sums_buf, centroid_cnts=cnts_buf, calculate_new=False)
        if prev_ids is not None:
            prev_ids.copy_(cluster_ids)
    new_centroids, shift_per_k = triton_centroid_finalize(sums_buf, cnts_buf, old_centroids,
                                                          out=new_buf, shift=shift_buf)
    # (a loop that neither tests convergence nor prints the shift spares itself the two reductions)
    max_shift = shift_per_k.amax(dim=-1).amax() if want_shift else None
    return new_centroids, cluster_ids, max_shift


def batch_kmeans_Euclid(x: torch.Tensor, n_clusters: int, max_iters: int = 100, tol: float = 0.0,
                        init_centroids: Optional[torch.Tensor] = None, verbose: bool = False, **_ignored):
    """Batched Lloyd k-means, ``x`` ``(B, N, D)`` on CUDA.

    Returns ``(cluster_ids int32 (B,N) from the last assignment, centroids after the last
    update, iterations run)`` exactly like ``flashlib/primitives/kmeans/triton/kmeans.py:61-153``.
    Without ``init_centroids`` the start is ``torch.randint`` rows drawn on ``x.device`` from the
    global generator, the same call the reference makes (``kmeans.py:92-101``).
    """
    if not x.is_cuda:
        raise RuntimeError("flashlib_b200 k-means needs CUDA tensors (no CPU fallback)")
    B, N, D = x.shape
    K = int(n_clusters)
    if init_centroids is None:
        indices = torch.randint(0, N, (B, K), device=x.device)
        centroids = torch.gather(x, dim=1, index=indices[..., None].expand(-1, -1, D))
    else:
        centroids = init_centroids
    centroids = centroids.reshape(B, K, D)
    x32 = x if x.dtype == torch.float32 else x.float()
    cur = centroids.float().contiguous().clone()
    nxt = torch.empty_like(cur)
    sums_buf = torch.empty((B, K, D), device=x.device, dtype=torch.float32)
    cnts_buf = torch.empty((B, K), device=x.device, dtype=torch.int32)
    shift_buf = torch.empty((B, K), device=x.device, dtype=torch.float32)
    cluster_ids = torch.empty((B, N), device=x.device, dtype=torch.int32)
    # B = 1: the sums are kept from iteration to iteration and only the rows whose label changed are
    # moved between them (after the first iterations under 1 % of the points); every
    # DELTA_REFRESH-th iteration recomputes them from all rows
    incremental = B == 1 and x32.stride(2) == 1 and os.environ.get("FLASHLIB_B200_KMEANS_DELTA", "1") != "0"
    prev_ids = torch.empty((B, N), device=x.device, dtype=torch.int32) if incremental else None
    it = 0
    for it in range(max_iters):
        euclid_assign_triton(x32, cur, out=cluster_ids)
        _, _, max_shift = triton_lloyd_centroid_step_euclid(
            x32, cluster_ids, cur, sums_buf=sums_buf, cnts_buf=cnts_buf, new_buf=nxt, shift_buf=shift_buf,
            prev_ids=prev_ids, refresh=(it % DELTA_REFRESH == 0), want_shift=(tol > 0.0 or verbose))
        if verbose:
            print(f"Iter {it}, center shift: {max_shift.item():.6f}")
        cur, nxt = nxt, cur
        if tol > 0.0 and max_shift < tol:
            break
    return cluster_ids, cur.to(x.dtype), it + 1


def flash_kmeans(x: torch.Tensor, n_clusters: int, *, max_iters: int = 100, tol: float = 0.0,
                 init_centroids=None, verbose: bool = False, metric: str = "euclidean",
                 backend: Optional[str] = None, variant: Optional[str] = None, **kwargs):
    """k-means with flashlib's ``flash_kmeans`` signature (``kmeans/impl.py:110-189``).

    ``x`` is ``(B, N, D)`` or ``(N, D)``; returns ``(cluster_ids int32, centroids, n_iter)``.
    Only the euclidean metric is built; ``backend`` / ``variant`` are accepted and ignored.
    """
    if metric != "euclidean":
        if metric in ("cosine", "dot"):
            raise NotImplementedError(f"flashlib_b200 builds the euclidean metric only (got {metric!r})")
        raise ValueError(f"unknown metric {metric!r}")
    squeeze = x.ndim == 2
    x_b = x.unsqueeze(0) if squeeze else x
    cluster_ids, centroids, n_iter = batch_kmeans_Euclid(
        x_b, n_clusters, max_iters=max_iters, tol=tol, init_centroids=init_centroids, verbose=verbose)
    if squeeze:
        cluster_ids = cluster_ids.squeeze(0)
        centroids = centroids.squeeze(0)
    return cluster_ids, centroids, n_iter
