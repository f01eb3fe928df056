"""Exchange logic of the row-sharded kNN and k-means, run as two gloo ranks on CPU.

The device kernels are replaced by the numpy oracle through the hooks of
``flashlib_b200.sharded`` -- these tests cover the sharding, the collectives, the padding of
short shards and the merge order, not the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashlib_b200 import sharded
from oracle import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_knn(q, db, k, off):
    v, i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    return torch.from_numpy(v), torch.from_numpy((i + off).astype(np.int32))


def _merge(cd, ci, k):
    cd, ci = cd.numpy().copy(), ci.numpy()
    cd[ci < 0] = np.inf
    order = np.lexsort((ci, cd), axis=1)[:, :k]
    return torch.from_numpy(np.take_along_axis(cd, order, 1)), torch.from_numpy(np.take_along_axis(ci, order, 1))


def _knn_worker(rank, world, port, m, k, nq, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)
    db = torch.randn(m, 16, generator=g)
    q = torch.randn(nq, 16, generator=g)
    s, e = sharded.shard_bounds(m, world, rank)
    d, i = sharded.sharded_knn(q, db[s:e], k, row_offset=s, local_fn=_local_knn, merge_fn=_merge)
    ref_v, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    ok = np.array_equal(i.numpy(), ref_i.astype(np.int32)) and np.allclose(d.numpy(), ref_v, rtol=1e-5, atol=1e-5)
    # owner form: every rank holds the rows of its own query slice only (all-to-all exchange)
    qs, qe = sharded.shard_bounds(q.shape[0], world, rank)
    d2, i2 = sharded.sharded_knn(q, db[s:e], k, row_offset=s, result="owner", local_fn=_local_knn, merge_fn=_merge)
    ok = ok and d2.shape == (qe - qs, k) and np.array_equal(i2.numpy(), ref_i[qs:qe].astype(np.int32)) \
        and np.allclose(d2.numpy(), ref_v[qs:qe], rtol=1e-5, atol=1e-5)
    out[rank] = bool(ok)
    dist.destroy_process_group()


# second case: a shard shorter than k; third: fewer queries than ranks (rank 1 owns none)
@pytest.mark.parametrize("m,k,nq", [(1000, 10, 41), (7, 5, 41), (300, 4, 1)])
def test_sharded_knn_two_ranks(m, k, nq):
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_knn_worker, args=(world, _free_port(), m, k, nq, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def _kmeans_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(2001, 8, generator=g)
    init = x[:12].clone()
    s, e = sharded.shard_bounds(x.shape[0], world, rank)

    def assign(xs, c):
        return torch.from_numpy(oracle.kmeans_assign(xs.numpy(), c.numpy()))

    def update(xs, lab, c):
        _, sums, cnts = oracle.kmeans_update(xs.numpy(), lab.numpy().astype(np.int64), c.numpy())
        return torch.from_numpy(sums), torch.from_numpy(cnts.astype(np.int32))

    def finalize(sums, cnts, c):
        cf = cnts.float().clamp_min(1.0)[:, None]
        new = torch.where(cnts[:, None] == 0, c, sums / cf)
        return new, (new - c).norm(dim=-1)

    labels, cents, n_iter = sharded.sharded_kmeans(x[s:e], 12, max_iters=5, init_centroids=init,
                                                   assign_fn=assign, update_fn=update, finalize_fn=finalize)
    ref_l, ref_c, ref_n = oracle.kmeans(x.numpy(), 12, max_iters=5, init_centroids=init.numpy())
    ok = n_iter == ref_n and np.array_equal(labels.numpy(), ref_l[s:e]) and np.allclose(cents.numpy(), ref_c, rtol=1e-4, atol=1e-5)
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_sharded_kmeans_two_ranks():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_kmeans_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_shard_bounds_cover_everything():
    for m in (0, 1, 7, 1000, 1_000_003):
        for world in (1, 2, 3, 8):
            b = [sharded.shard_bounds(m, world, r) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == m
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            assert max(e - s for s, e in b) - min(e - s for s, e in b) <= 1


class _NpIndex:
    """Minimal stand-in for IvfFlatIndex in the CPU test of the sharded IVF exchange."""

    def __init__(self, centroids, data, ids, list_offsets):
        self.centroids, self.data, self.ids, self.list_offsets = centroids, data, ids, list_offsets


def _np_build(x, centroids):
    _, offsets, order = oracle.ivf_assign_lists(x.numpy(), centroids.numpy())
    return _NpIndex(centroids.numpy(), x.numpy()[order], torch.from_numpy(order.astype(np.int64)), offsets)


def _np_search(index, q, k, nprobe=None):
    v, i, _ = oracle.ivf_search(index.centroids, index.data, index.ids.numpy(), index.list_offsets, q.numpy(), k, nprobe)
    return torch.from_numpy(v), torch.from_numpy(i)


def _ivf_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(8)
    x = torch.randn(3000, 16, generator=g)
    q = torch.randn(50, 16, generator=g)
    cents = x[:24].clone()
    s, e = sharded.shard_bounds(x.shape[0], world, rank)
    local = sharded.sharded_ivf_build(x[s:e], cents, row_offset=s, build_fn=_np_build)
    v, i = sharded.sharded_ivf_search(local, q, 7, nprobe=5, search_fn=_np_search, merge_fn=_merge)
    whole = _np_build(x, cents)
    rv, ri = _np_search(whole, q, 7, nprobe=5)
    ok = np.allclose(v.numpy(), rv.numpy(), rtol=1e-5, atol=1e-5) and np.array_equal(np.sort(i.numpy(), 1), np.sort(ri.numpy(), 1))
    out[rank] = bool(ok)
    dist.destroy_process_group()


def test_sharded_ivf_two_ranks():
    """Row-sharded IVF index under shared centroids: same result as the unsharded index."""
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_ivf_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
