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


class DeviceKnnKernels:
    """The device side of :func:`sharded_knn`: every method is one or two C-ABI calls on the
    current stream.  The CPU tests of the exchange logic pass an object with the same methods
    built on the oracle."""

    def tensor_core(self, nq: int, m: int, d: int, k: int, mode) -> bool:
        """True when a shard of ``m`` rows takes the tensor-core path for this call."""
        from . import _lib
        from .knn import _mode_from
        md = _mode_from(mode)
        if md == _lib.FL_KNN_EXACT_SIMT or m < 1:
            return False
        if md == _lib.FL_KNN_AUTO:
            return _lib.load().fl_knn_resolve_mode(nq, m, d, k) == _lib.FL_KNN_BF16_RERANK
        return d <= 256 and k <= 112          # forced: the shapes the tensor-core kernel takes

    def plane_of(self, db: torch.Tensor):
        from .knn import get_plane
        return get_plane(db)

    def max_norm(self, db: torch.Tensor, plane) -> torch.Tensor:
        """Largest row norm of this shard as a 1-element fp32 device tensor."""
        from . import _lib
        off = _lib.load().fl_knn_plane_maxnorm_offset(db.shape[0], db.shape[1])
        return plane.buf[off:off + 4].view(torch.float32).clone()

    def local(self, q, db, k, row_offset, mode, plane):
        from .knn import _mode_from, knn_f32
        d_, i_, info = knn_f32(q, db, k, mode=_mode_from(mode), row_offset=row_offset, plane=plane, check_status=False)
        return d_, i_, info["status"]

    def seed(self, q, db, k, plane):
        from . import _lib
        from .knn import _stream_ptr
        lib = _lib.load()
        nq, d = q.shape
        m = db.shape[0]
        ws_bytes = lib.fl_knn_workspace_bytes(nq, m, d, k, _lib.FL_KNN_BF16_RERANK)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        cls = torch.empty(lib.fl_knn_seed_floats(nq), dtype=torch.float32, device=q.device)
        status = torch.empty(_lib.FL_STATUS_WORDS, dtype=torch.int32, device=q.device)
        _lib.check(lib.fl_knn_seed_f32(q.data_ptr(), nq, q.stride(0), d, k, plane.ptr, m, cls.data_ptr(),
                                       ws.data_ptr(), ws_bytes, status.data_ptr(), _stream_ptr(q.device)))
        return cls, (ws, ws_bytes, status)

    def compress(self, cls: torch.Tensor) -> torch.Tensor:
        """bf16 copy of the class maxima, rounded toward -inf (half the bytes on the wire)."""
        from . import _lib
        from .knn import _stream_ptr
        out = torch.empty(cls.numel(), dtype=torch.bfloat16, device=cls.device)
        _lib.check(_lib.load().fl_f32_to_bf16_down(cls.data_ptr(), out.data_ptr(), cls.numel(), _stream_ptr(cls.device)))
        return out

    def expand(self, comp: torch.Tensor, cls: torch.Tensor) -> torch.Tensor:
        from . import _lib
        from .knn import _stream_ptr
        _lib.check(_lib.load().fl_bf16_to_f32(comp.data_ptr(), cls.data_ptr(), cls.numel(), _stream_ptr(cls.device)))
        return cls

    def seeded(self, q, db, k, row_offset, plane, cls, gmax, ctx):
        from . import _lib
        from .knn import _stream_ptr
        lib = _lib.load()
        ws, ws_bytes, status = ctx
        nq, d = q.shape
        out_d = torch.empty((nq, k), dtype=torch.float32, device=q.device)
        out_i = torch.empty((nq, k), dtype=torch.int32, device=q.device)
        _lib.check(lib.fl_knn_seeded_f32(q.data_ptr(), nq, q.stride(0), db.data_ptr(), db.shape[0], db.stride(0), d, k,
                                         plane.ptr, row_offset, cls.data_ptr(), gmax.data_ptr(), out_d.data_ptr(),
                                         out_i.data_ptr(), ws.data_ptr(), ws_bytes, status.data_ptr(),
                                         _stream_ptr(q.device)))
        return out_d, out_i, status

    def pack(self, d_, i_, status, world: int, owner: bool) -> torch.Tensor:
        from . import _lib
        from .knn import _stream_ptr
        lib = _lib.load()
        nq, k = d_.shape
        out = torch.empty(lib.fl_knn_pack_ints(nq, k, world, int(owner)), dtype=torch.int32, device=d_.device)
        d_, i_ = d_.contiguous(), i_.contiguous()
        _lib.check(lib.fl_knn_pack_f32(d_.data_ptr(), i_.data_ptr(), nq, k, world, int(owner),
                                       status.data_ptr() if status is not None else None, out.data_ptr(),
                                       _stream_ptr(d_.device)))
        return out

    def merge(self, msgs: torch.Tensor, rows: int, k: int, world: int):
        from . import _lib
        from .knn import _stream_ptr
        lib = _lib.load()
        out_d = torch.empty((rows, k), dtype=torch.float32, device=msgs.device)
        out_i = torch.empty((rows, k), dtype=torch.int32, device=msgs.device)
        status = torch.empty(_lib.FL_STATUS_WORDS, dtype=torch.int32, device=msgs.device)
        _lib.check(lib.fl_knn_merge_packed_f32(msgs.data_ptr(), rows, k, world, out_d.data_ptr(), out_i.data_ptr(),
                                               status.data_ptr(), _stream_ptr(msgs.device)))
        return out_d, out_i, status

    def defer(self, status: torch.Tensor) -> None:
        from .knn import _defer_status_check
        _defer_status_check(status)


class ShardedKnnIndex:
    """One rank's shard of a row-sharded database together with the facts that need a collective
    to establish: the smallest shard's row count, whether every shard can take the tensor-core
    path, and the largest row norm over all shards (the scoring error bound of
    ``fl_knn_seeded_f32`` must hold for rows of every shard).

    Constructing it is a COLLECTIVE call: every rank of ``group`` must do so at the same point of
    its program.  It is the ``fit`` step of the sharded search; :func:`sharded_knn` uses it to share
    the threshold seeds between the ranks."""

    def __init__(self, db_shard: torch.Tensor, row_offset: int, *, group=None, plane=None, kernels=None):
        kern = kernels if kernels is not None else DeviceKnnKernels()
        self.db = db_shard
        self.row_offset = int(row_offset)
        self.group = group
        m, d = db_shard.shape
        can_tc = m > 0 and kern.tensor_core(1 << 20, m, d, min(10, m), "bf16")
        self.plane = plane if plane is not None else (kern.plane_of(db_shard) if can_tc else None)
        gmax = kern.max_norm(db_shard, self.plane) if self.plane is not None else torch.zeros(1, device=db_shard.device)
        facts = torch.tensor([m, 1 if self.plane is not None else 0], dtype=torch.int64, device=db_shard.device)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
            dist.all_reduce(facts, op=dist.ReduceOp.MIN, group=group)
        self.global_max_norm = gmax
        self.min_rows, all_tc = (int(v) for v in facts.tolist())
        self.all_tensor_core = bool(all_tc)


def sharded_knn(q: torch.Tensor, db_shard: Optional[torch.Tensor], k: int, *, row_offset: Optional[int] = None,
                group=None, mode: Optional[str] = None, plane=None, result: str = "replicated",
                index: Optional[ShardedKnnIndex] = None, share_seeds: Optional[bool] = None, kernels=None):
    """Exact kNN of the replicated queries ``q`` against a row-sharded database.

    ``db_shard`` is this rank's rows, ``row_offset`` its first global row id (or pass ``index``, a
    :class:`ShardedKnnIndex` built once for the shard).  A shard with fewer than ``k`` rows
    contributes ``+inf`` / ``-1`` padding.  ``result="replicated"`` returns the same
    ``(dist fp32 (nq,k), idx int32 (nq,k))`` on every rank (all-gather of the candidates, every
    rank merges all queries); ``result="owner"`` returns on rank ``r`` the rows
    ``shard_bounds(nq, world, r)`` of that result only (all-to-all, every rank merges its own
    queries).

    With an ``index`` (and ``share_seeds`` not False), k <= 16, at least k rows in every shard and
    the tensor-core path on every rank, the ranks exchange the class maxima of their threshold-
    seeding passes (one all-reduce with MAX, bf16) before they score: every rank then starts from
    thresholds that k + 6 rows of the WHOLE database reach, instead of rows of its own shard, so
    candidate insertion costs what it costs on one GPU, and a rank returns only rows that can
    still be among the database's k nearest.

    The status words of every rank's kernels travel with its candidates; the merged status is
    looked at by a later call or ``flashlib_b200.knn.check_pending()`` on every rank alike, so a
    kernel error on one rank raises everywhere instead of leaving the others in a collective.
    ``kernels`` replaces the device calls (CPU tests of the exchange logic).
    """
    if result not in ("replicated", "owner"):
        raise ValueError(f"result must be 'replicated' or 'owner', got {result!r}")
    kern = kernels if kernels is not None else DeviceKnnKernels()
    if index is not None:
        db_shard, row_offset, group = index.db, index.row_offset, index.group
        plane = index.plane if plane is None else plane
    if db_shard is None or row_offset is None:
        raise ValueError("sharded_knn needs db_shard and row_offset, or an index")
    m_local = db_shard.shape[0]
    nq, d = q.shape
    multi = dist.is_initialized() and dist.get_world_size(group) > 1
    world = dist.get_world_size(group) if multi else 1
    rank = dist.get_rank(group) if multi else 0

    # every rank must take the same branch (the seeded flow has one more collective): the decision
    # uses only facts that are identical everywhere
    seeded = (multi and index is not None and share_seeds is not False and nq > 0 and k <= 16
              and q.dtype == torch.float32 and db_shard.dtype == torch.float32 and d <= 256
              and index.all_tensor_core and index.min_rows >= k
              and (share_seeds is True or kern.tensor_core(nq, index.min_rows, d, k, mode)))
    gmax = index.global_max_norm if index is not None else None

    if seeded:
        cls, ctx = kern.seed(q, db_shard, k, plane)
        comp = kern.compress(cls)
        dist.all_reduce(comp, op=dist.ReduceOp.MAX, group=group)
        cls = kern.expand(comp, cls)
        d_loc, i_loc, status = kern.seeded(q, db_shard, k, row_offset, plane, cls, gmax, ctx)
    else:
        k_local = min(k, m_local)
        status = None
        if k_local > 0 and nq > 0:
            d_loc, i_loc, status = kern.local(q, db_shard, k_local, row_offset, mode, plane)
        else:
            d_loc = torch.empty((nq, 0), dtype=torch.float32, device=q.device)
            i_loc = torch.empty((nq, 0), dtype=torch.int32, device=q.device)
        if k_local < k:
            pad_d = torch.full((nq, k - k_local), float("inf"), dtype=torch.float32, device=q.device)
            pad_i = torch.full((nq, k - k_local), -1, dtype=torch.int32, device=q.device)
            d_loc = torch.cat([d_loc, pad_d], 1)
            i_loc = torch.cat([i_loc, pad_i], 1)
    if not multi:
        if status is not None:
            kern.defer(status)
        return d_loc, i_loc

    owner = result == "owner"
    msg = kern.pack(d_loc, i_loc, status, world, owner)
    words = msg.numel() - nq * 2 * k
    per_status = words // (world if owner else 1)
    if owner:
        counts = [shard_bounds(nq, world, r)[1] - shard_bounds(nq, world, r)[0] for r in range(world)]
        mine = counts[rank]
        recv = torch.empty(world * (mine * 2 * k + per_status), dtype=torch.int32, device=q.device)
        dist.all_to_all_single(recv, msg, output_split_sizes=[mine * 2 * k + per_status] * world,
                               input_split_sizes=[c * 2 * k + per_status for c in counts], group=group)
        rows = mine
    else:
        recv = torch.empty(world * msg.numel(), dtype=torch.int32, device=q.device)
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(recv, msg, group=group)
        else:
            dist.all_gather(list(recv.view(world, -1).unbind(0)), msg, group=group)   # gloo has no tensor form
        rows = nq
    out_d, out_i, merged_status = kern.merge(recv, rows, k, world)
    kern.defer(merged_status)
    return out_d, out_i


def all_reduce_sums_counts(sums: torch.Tensor, cnts: torch.Tensor, group=None) -> None:
    """Sums ``(..., K, D)`` fp32 and counts ``(..., K)`` int32 over the ranks in ONE all-reduce, in
    place.  The counts ride in the same fp32 buffer as two columns, ``cnt // 4096`` and
    ``cnt % 4096``: both stay below 2^24 after the reduction for any int32 count and any world
    size in use (<= 4096 ranks), so the sum of integers is exact."""
    assert sums.is_contiguous() and cnts.is_contiguous(), "all_reduce_sums_counts works in place"
    K, D = sums.shape[-2], sums.shape[-1]
    flat_s = sums.reshape(-1, K, D)
    flat_c = cnts.reshape(-1, K)
    buf = torch.empty((flat_s.shape[0], K, D + 2), dtype=torch.float32, device=sums.device)
    buf[..., :D] = flat_s
    buf[..., D] = torch.div(flat_c, 4096, rounding_mode="floor").to(torch.float32)
    buf[..., D + 1] = (flat_c % 4096).to(torch.float32)
    dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    flat_s.copy_(buf[..., :D])
    flat_c.copy_((buf[..., D].to(torch.int64) * 4096 + buf[..., D + 1].to(torch.int64)).to(cnts.dtype))


def sharded_kmeans(x_shard: torch.Tensor, n_clusters: int, *, max_iters: int = 100, tol: float = 0.0,
                   init_centroids: torch.Tensor, group=None,
                   assign_fn: Optional[Callable] = None, update_fn: Optional[Callable] = None,
                   finalize_fn: Optional[Callable] = None):
    """Lloyd k-means over row-sharded samples.  ``init_centroids`` ``(K, D)`` must be identical
    on every rank.  Per iteration: local assignment, local sums/counts, one all-reduce of both (a fused buffer),
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
            all_reduce_sums_counts(sums, cnts, group)
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
