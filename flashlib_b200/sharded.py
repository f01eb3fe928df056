"""Row-sharded kNN and k-means over the GPUs of one box: one process per GPU,
``torch.distributed`` (NCCL over NVLink) for the exchange step.

The reference has no sharded kNN; its only multi-device code is the single-process k-means
of ``flashlib/primitives/kmeans/large.py:35-280``, which copies per-GPU partial sums to GPU 0
and adds them there.  Here every rank owns a contiguous row range of the database (or of the
sample set), runs the single-GPU kernels on it and exchanges only what the algorithm needs:

* kNN: the ``(nq, k)`` local candidates with global row ids are all-gathered and every rank
  picks the k best of ``world * k`` per query with ``fl_topk_merge_f32``;
* k-means: the per-cluster sums and counts are all-reduced, every rank finalises the same
  centroids (no broadcast), labels stay sharded;
* IVF-Flat: every rank indexes its own rows under the SAME coarse centroids, so a query probes
  the same lists on every rank and the union of the ranks' list members is the unsharded list;
  the per-rank ``(nq, k)`` results (global row ids) are all-gathered and merged like kNN.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(m: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous row range ``[start, end)`` of ``rank``; the first ``m % world`` ranks hold
    one extra row."""
    base, rem = divmod(int(m), int(world))
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def gather_candidates(local_d: torch.Tensor, local_i: torch.Tensor, group=None):
    """All-gathers ``(nq, k)`` candidates from every rank into ``(nq, world * k)`` tensors
    (rank-major along the candidate axis).  Distances (fp32 bits) and row ids (int32) travel in
    one int32 message per rank."""
    world = dist.get_world_size(group)
    nq, k = local_d.shape
    packed = torch.cat([local_d.contiguous().view(torch.int32), local_i.to(torch.int32)], dim=1).contiguous()
    g = torch.empty((world, nq, 2 * k), dtype=torch.int32, device=local_d.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(g, packed, group=group)
    else:
        # list form: the gloo backend has no tensor form
        dist.all_gather(list(g.unbind(0)), packed, group=group)
    g = g.permute(1, 0, 2)
    cand_d = g[:, :, :k].reshape(nq, world * k).view(torch.float32)
    cand_i = g[:, :, k:].reshape(nq, world * k)
    return cand_d, cand_i


def exchange_candidates(local_d: torch.Tensor, local_i: torch.Tensor, group=None):
    """All-to-all form of :func:`gather_candidates`: rank ``r`` receives, from every rank, only the
    candidates of the queries ``shard_bounds(nq, world, r)`` it owns.  Returns ``(cand_d, cand_i)`` of
    shape ``(owned, world * k)``; inbound volume and merge work are ``1/world`` of the all-gather's."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    nq, k = local_d.shape
    packed = torch.cat([local_d.contiguous().view(torch.int32), local_i.to(torch.int32)], dim=1).contiguous()
    counts = [shard_bounds(nq, world, r)[1] - shard_bounds(nq, world, r)[0] for r in range(world)]
    mine = counts[rank]
    g = torch.empty((world * mine, 2 * k), dtype=torch.int32, device=local_d.device)
    dist.all_to_all_single(g, packed, output_split_sizes=[mine] * world, input_split_sizes=counts, group=group)
    g = g.view(world, mine, 2 * k).permute(1, 0, 2)
    cand_d = g[:, :, :k].reshape(mine, world * k).view(torch.float32)
    cand_i = g[:, :, k:].reshape(mine, world * k)
    return cand_d, cand_i


def sharded_knn(q: torch.Tensor, db_shard: torch.Tensor, k: int, *, row_offset: int, group=None,
                mode: Optional[str] = None, plane=None, result: str = "replicated",
                local_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None):
    """Exact kNN of the replicated queries ``q`` against a row-sharded database.

    ``db_shard`` is this rank's rows, ``row_offset`` its first global row id.  A shard with
    fewer than ``k`` rows contributes ``+inf`` / ``-1`` padding.  ``result="replicated"`` returns
    the same ``(dist fp32 (nq,k), idx int32 (nq,k))`` on every rank (all-gather of the candidates,
    every rank merges all queries); ``result="owner"`` returns on rank ``r`` the rows
    ``shard_bounds(nq, world, r)`` of that result only (all-to-all, every rank merges its own
    queries).  ``local_fn`` / ``merge_fn`` replace the device kernels (used by the CPU tests of the
    exchange logic).
    """
    if result not in ("replicated", "owner"):
        raise ValueError(f"result must be 'replicated' or 'owner', got {result!r}")
    if local_fn is None:
        from .knn import _mode_from, knn_f32

        def local_fn(q_, db_, k_, off_):
            d_, i_, _ = knn_f32(q_, db_, k_, mode=_mode_from(mode), row_offset=off_, plane=plane,
                                check_status="deferred")
            return d_, i_
    if merge_fn is None:
        from .knn import topk_merge as merge_fn
    m_local = db_shard.shape[0]
    k_local = min(k, m_local)
    nq = q.shape[0]
    if k_local > 0:
        d_loc, i_loc = local_fn(q, db_shard, k_local, row_offset)
    else:
        d_loc = torch.empty((nq, 0), dtype=torch.float32, device=q.device)
        i_loc = torch.empty((nq, 0), dtype=torch.int32, device=q.device)
    if k_local < k:
        pad_d = torch.full((nq, k - k_local), float("inf"), dtype=torch.float32, device=q.device)
        pad_i = torch.full((nq, k - k_local), -1, dtype=torch.int32, device=q.device)
        d_loc = torch.cat([d_loc, pad_d], 1)
        i_loc = torch.cat([i_loc, pad_i], 1)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return d_loc, i_loc
    if result == "owner":
        cand_d, cand_i = exchange_candidates(d_loc, i_loc, group)
    else:
        cand_d, cand_i = gather_candidates(d_loc, i_loc, group)
    return merge_fn(cand_d, cand_i, k)


def sharded_kmeans(x_shard: torch.Tensor, n_clusters: int, *, max_iters: int = 100, tol: float = 0.0,
                   init_centroids: torch.Tensor, group=None,
                   assign_fn: Optional[Callable] = None, update_fn: Optional[Callable] = None,
                   finalize_fn: Optional[Callable] = None):
    """Lloyd k-means over row-sharded samples.  ``init_centroids`` ``(K, D)`` must be identical
    on every rank.  Per iteration: local assignment, local sums/counts, all-reduce of both,
    identical finalisation on every rank.  Returns ``(labels of this shard int32, centroids,
    iterations)``; the loop and its return convention follow
    ``flashlib/primitives/kmeans/triton/kmeans.py:117-153``."""
    from . import kmeans as km
    if assign_fn is None:
        assign_fn = lambda x, c: km.euclid_assign_triton(x[None], c[None])[0]  # noqa: E731
    if update_fn is None:
        def update_fn(x, lab, c):
            s, n = km.triton_centroid_update_euclid(x[None], lab[None], c[None], calculate_new=False)
            return s[0], n[0]
    if finalize_fn is None:
        def finalize_fn(s, n, c):
            new, shift = km.triton_centroid_finalize(s[None], n[None], c[None])
            return new[0], shift[0]
    K = int(n_clusters)
    cur = init_centroids.reshape(K, -1).float().contiguous().clone()
    multi = dist.is_initialized() and dist.get_world_size(group) > 1
    labels = None
    it = 0
    for it in range(max_iters):
        labels = assign_fn(x_shard, cur)
        sums, cnts = update_fn(x_shard, labels, cur)
        if multi:
            dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
            dist.all_reduce(cnts, op=dist.ReduceOp.SUM, group=group)
        new, shift = finalize_fn(sums, cnts, cur)
        cur = new
        if tol > 0.0 and float(shift.max()) < tol:
            break
    return labels, cur, it + 1


def sharded_ivf_build(x_shard: torch.Tensor, centroids: torch.Tensor, *, row_offset: int, nprobe: int = 8,
                      build_fn: Optional[Callable] = None):
    """This rank's part of a row-sharded IVF-Flat index: its rows assigned to the shared coarse
    ``centroids`` (identical on every rank, e.g. trained on rank 0's sample and broadcast) and
    laid out list-contiguously; ``ids`` are global row ids (``row_offset`` + local row).
    ``build_fn(x_padded, centroids) -> index`` replaces the device path in the CPU tests."""
    if build_fn is None:
        from .ivf_flat import _pad_features, index_from_centroids
        D = x_shard.shape[1]
        Dp = max(int(D), 16)
        xp = _pad_features(x_shard, Dp).contiguous()
        cp = _pad_features(centroids, Dp).contiguous()
        index = index_from_centroids(xp, cp, D=int(D), nprobe=nprobe)
    else:
        index = build_fn(x_shard, centroids)
    index.ids = index.ids + int(row_offset)
    return index


def sharded_ivf_search(index, q: torch.Tensor, k: int, *, nprobe: Optional[int] = None, group=None,
                       search_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None):
    """IVF-Flat search over a row-sharded index (``sharded_ivf_build`` on every rank): the same
    ``(vals fp32, ids int64)`` on every rank as a search of the unsharded index with the same
    centroids.  A rank whose probed lists hold fewer than ``k`` rows contributes ``+inf`` / ``-1``
    padding, which the merge drops."""
    if search_fn is None:
        from .ivf_flat import flash_ivf_flat_search as search_fn
    if merge_fn is None:
        from .knn import topk_merge as merge_fn
    vals, ids = search_fn(index, q, k, nprobe=nprobe)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return vals, ids
    ids32 = ids.to(torch.int32)        # row ids fit 31 bits (the kernels index rows with int32)
    cand_d, cand_i = gather_candidates(vals.float().contiguous(), ids32.contiguous(), group)
    out_d, out_i = merge_fn(cand_d, cand_i, k)
    return out_d, out_i.to(torch.int64)
