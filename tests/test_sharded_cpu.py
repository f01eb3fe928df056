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


STATUS_WORDS = 8
EPS_REL = 0.004          # the scoring error bound of the tensor-core kernels, relative to ||q|| max||x||


class OracleKnnKernels:
    """Stand-in for ``sharded.DeviceKnnKernels`` built on the numpy oracle.

    The seeded flow is modelled at its worst legal behaviour: "tensor-core" scores are the exact
    scores perturbed by up to the error bound, the seeding sample is a quarter of the rows, and a
    shard returns ONLY rows whose perturbed score lies above the certified threshold.  If the
    merged result still equals the oracle's, the margin and the certificate are right.  ``pack`` /
    ``merge`` restate the int32 message format of ``fl_knn_pack_f32`` / ``fl_knn_merge_packed_f32``.
    """

    def __init__(self, fail_rank=None, rank=0):
        self.deferred = []
        self.fail = fail_rank is not None and fail_rank == rank

    def tensor_core(self, nq, m, d, k, mode):
        return mode != "exact" and m >= 1

    def plane_of(self, db):
        return object()

    def max_norm(self, db, plane):
        return db.norm(dim=1).max().reshape(1).float()

    def _status(self):
        st = torch.zeros(STATUS_WORDS, dtype=torch.int32)
        if self.fail:
            st[0], st[1] = -4, (5 << 16) | 3
        return st

    def local(self, q, db, k, off, mode, plane):
        v, i = oracle.knn_naive(q.numpy(), db.numpy(), k)
        return torch.from_numpy(v), torch.from_numpy((i + off).astype(np.int32)), self._status()

    def _scores(self, q, db, gmax):
        """Exact scores perturbed by +-eps (deterministic pattern): what a bf16 scoring pass may return."""
        qn, xn = q.numpy().astype(np.float64), db.numpy().astype(np.float64)
        s = qn @ xn.T - 0.5 * (xn * xn).sum(-1)[None, :]
        eps = EPS_REL * np.sqrt((qn * qn).sum(-1))[:, None] * float(gmax)
        sign = np.where((np.arange(xn.shape[0])[None, :] + np.arange(qn.shape[0])[:, None]) % 2 == 0, 1.0, -1.0)
        return s + 0.999 * eps * sign

    def seed(self, q, db, k, plane):
        gmax = float(db.norm(dim=1).max())           # local norms suffice for local rows
        s = self._scores(q, db, gmax)[:, ::4]
        cls = np.full((q.shape[0], 32), -np.inf, dtype=np.float32)
        for c in range(32):
            part = s[:, c::32]
            if part.shape[1]:
                cls[:, c] = np.floor(part.max(1) * 8) / 8     # rounded down, like the bf16 wire format
        return torch.from_numpy(cls.reshape(-1)), None

    def compress(self, cls):
        return cls.clone()

    def expand(self, comp, cls):
        return comp

    def seeded(self, q, db, k, off, plane, cls, gmax, ctx):
        qn = q.numpy().astype(np.float64)
        g = float(gmax)
        qsq = (qn * qn).sum(-1)
        pick = -np.sort(-cls.numpy().reshape(q.shape[0], 32).astype(np.float64), axis=1)[:, k + 6 - 1]
        cert = pick - 2 * EPS_REL * np.sqrt(qsq) * g - 1e-5 * (qsq + g * g)
        s = self._scores(q, db, g)
        xn = db.numpy().astype(np.float64)
        dist = ((qn[:, None, :] - xn[None, :, :]) ** 2).sum(-1)
        dist[s <= cert[:, None]] = np.inf                    # everything at or below the threshold is dropped
        order = np.argsort(dist, axis=1, kind="stable")[:, :k]
        dv = np.take_along_axis(dist, order, 1)
        iv = np.where(np.isfinite(dv), order + off, -1)
        return torch.from_numpy(dv.astype(np.float32)), torch.from_numpy(iv.astype(np.int32)), self._status()

    def pack(self, d_, i_, status, world, owner):
        nq, k = d_.shape
        st = status if status is not None else torch.zeros(STATUS_WORDS, dtype=torch.int32)
        rows = torch.cat([d_.contiguous().view(torch.int32), i_.to(torch.int32)], 1)
        parts = []
        for r in range(world if owner else 1):
            s, e = sharded.shard_bounds(nq, world, r) if owner else (0, nq)
            parts += [rows[s:e].reshape(-1), st]
        return torch.cat(parts).contiguous()

    def merge(self, msgs, rows, k, world):
        m = msgs.view(world, rows * 2 * k + STATUS_WORDS)
        body = m[:, :rows * 2 * k].reshape(world, rows, 2 * k)
        cd = body[:, :, :k].permute(1, 0, 2).reshape(rows, world * k).contiguous().view(torch.float32).numpy().copy()
        ci = body[:, :, k:].permute(1, 0, 2).reshape(rows, world * k).numpy()
        cd[ci < 0] = np.inf
        order = np.lexsort((ci, cd), axis=1)[:, :k]
        st = torch.zeros(STATUS_WORDS, dtype=torch.int32)
        for r in range(world):
            tail = m[r, rows * 2 * k:]
            if st[0] == 0 and tail[0] != 0:
                st[0], st[1] = tail[0], tail[1]
            st[2] += tail[2]
        ov = np.take_along_axis(cd, order, 1)
        oi = np.where(np.isfinite(ov), np.take_along_axis(ci, order, 1), -1)
        return torch.from_numpy(ov), torch.from_numpy(oi.astype(np.int32)), st

    def defer(self, status):
        self.deferred.append(status.clone())


def _merge(cd, ci, k):
    cd, ci = cd.numpy().copy(), ci.numpy()
    cd[ci < 0] = np.inf
    order = np.lexsort((ci, cd), axis=1)[:, :k]
    return torch.from_numpy(np.take_along_axis(cd, order, 1)), torch.from_numpy(np.take_along_axis(ci, order, 1))


def _knn_worker(rank, world, port, m, k, nq, seeds, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)
    db = torch.randn(m, 16, generator=g)
    if seeds == "skewed":
        # every near neighbour of every query lives on rank 0: the other shard must be allowed to
        # return short lists without hurting the result
        db[m // 2:] += 40.0
    q = torch.randn(nq, 16, generator=g)
    s, e = sharded.shard_bounds(m, world, rank)
    kern = OracleKnnKernels(fail_rank=1 if seeds == "fail" else None, rank=rank)
    index = sharded.ShardedKnnIndex(db[s:e], s, kernels=kern) if seeds else None
    kw = dict(index=index, kernels=kern) if seeds else dict(row_offset=s, kernels=kern)
    d, i = sharded.sharded_knn(q, None if seeds else db[s:e], k, **kw)
    ref_v, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    ok = np.array_equal(i.numpy(), ref_i.astype(np.int32)) and np.allclose(d.numpy(), ref_v, rtol=1e-4, atol=1e-4)
    # owner form: every rank holds the rows of its own query slice only (all-to-all exchange)
    qs, qe = sharded.shard_bounds(q.shape[0], world, rank)
    d2, i2 = sharded.sharded_knn(q, None if seeds else db[s:e], k, result="owner", **kw)
    ok = ok and d2.shape == (qe - qs, k) and np.array_equal(i2.numpy(), ref_i[qs:qe].astype(np.int32)) \
        and np.allclose(d2.numpy(), ref_v[qs:qe], rtol=1e-4, atol=1e-4)
    # the merged status reaches every rank: an error on rank 1 is seen by rank 0 too
    errs = [int(st[0]) for st in kern.deferred]
    ok = ok and len(errs) == 2 and all(e_ == (-4 if seeds == "fail" else 0) for e_ in errs)
    if seeds:
        ok = ok and index.min_rows == min(sharded.shard_bounds(m, world, r)[1] - sharded.shard_bounds(m, world, r)[0]
                                          for r in range(world))
    out[rank] = bool(ok)
    dist.destroy_process_group()


# second case: a shard shorter than k; third: fewer queries than ranks (rank 1 owns none); then the
# shared-seed flow (uniform and skewed shards) and a kernel error on one rank
@pytest.mark.parametrize("m,k,nq,seeds", [(1000, 10, 41, None), (7, 5, 41, None), (300, 4, 1, None),
                                          (2000, 10, 41, "shared"), (2000, 10, 33, "skewed"), (2000, 5, 8, "fail"),
                                          (7, 5, 9, "shared")])
def test_sharded_knn_two_ranks(m, k, nq, seeds):
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_knn_worker, args=(world, _free_port(), m, k, nq, seeds, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def test_pack_format_round_trip():
    """The message format of the exchange, as the oracle kernels restate it: owner and replicated
    forms, uneven query split, padding ids."""
    kern = OracleKnnKernels()
    g = torch.Generator().manual_seed(2)
    nq, k, world = 11, 3, 4
    d_all = [torch.rand(nq, k, generator=g).sort(1).values for _ in range(world)]
    i_all = [torch.randint(0, 1000, (nq, k), generator=g, dtype=torch.int32) for _ in range(world)]
    i_all[2][:, 2] = -1
    cd = torch.cat(d_all, 1)
    ci = torch.cat(i_all, 1)
    want_d, want_i = _merge(cd, ci, k)
    # replicated: every rank's single message, back to back
    msgs = torch.cat([kern.pack(d_all[r], i_all[r], None, world, False) for r in range(world)])
    got_d, got_i, st = kern.merge(msgs, nq, k, world)
    assert torch.equal(got_d, want_d) and torch.equal(got_i, want_i) and int(st[0]) == 0
    # owner: destination r receives block r of every sender
    packed = [kern.pack(d_all[r], i_all[r], None, world, True) for r in range(world)]
    for dest in range(world):
        s, e = sharded.shard_bounds(nq, world, dest)
        sizes = [(sharded.shard_bounds(nq, world, r)[1] - sharded.shard_bounds(nq, world, r)[0]) * 2 * k + STATUS_WORDS
                 for r in range(world)]
        off = sum(sizes[:dest])
        recv = torch.cat([p[off:off + sizes[dest]] for p in packed])
        got_d, got_i, _ = kern.merge(recv, e - s, k, world)
        assert torch.equal(got_d, want_d[s:e]) and torch.equal(got_i, want_i[s:e])


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
    # the fused all-reduce carries integer counts exactly, beyond what one fp32 holds (2^24)
    sums = torch.full((2, 3, 5), float(rank + 1))
    cnts = torch.tensor([[300_000_007, 16_777_217, 0], [5, 4095, 4096]], dtype=torch.int32) + rank * 700_000_001
    sharded.all_reduce_sums_counts(sums, cnts, None)
    want = torch.tensor([[300_000_007, 16_777_217, 0], [5, 4095, 4096]], dtype=torch.int64) * world + 700_000_001 * sum(range(world))
    ok = ok and torch.equal(cnts.to(torch.int64), want) and torch.all(sums == float(sum(range(1, world + 1)))).item()
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
