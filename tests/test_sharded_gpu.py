"""The entry points behind the row-sharded kNN on ONE GPU: the shards of a database are
processed one after the other (seeding pass per shard, element-wise maximum of the class maxima
in place of the all-reduce, seeded scoring per shard, packed messages, merge) and the result is
compared with the oracle on the whole database.  The collectives themselves are covered by the
gloo tests and by the parity check bench.py runs on real ranks."""
import numpy as np
import pytest
import torch

from flashlib_b200 import _lib, sharded, synthetic
from flashlib_b200.knn import DbPlane
from oracle import oracle
from tests import parity
from tests.test_sharded_cpu import OracleKnnKernels

pytestmark = pytest.mark.gpu


def run_shards(X, Q, k, world, owner=False, wire_bf16=True):
    kern = sharded.DeviceKnnKernels()
    bounds = [sharded.shard_bounds(X.shape[0], world, r) for r in range(world)]
    shards = [X[s:e].contiguous() for s, e in bounds]
    planes = [DbPlane(x) for x in shards]
    gmax = torch.stack([kern.max_norm(x, p) for x, p in zip(shards, planes)]).max(0).values.contiguous()
    seeds = [kern.seed(Q, x, k, p) for x, p in zip(shards, planes)]
    cls = torch.stack([c for c, _ in seeds]).max(0).values.contiguous()
    if wire_bf16:
        comp = kern.compress(cls)
        assert torch.all(comp.float() <= cls)                      # rounded down, never up
        cls = kern.expand(comp, torch.empty_like(cls))
    outs = [kern.seeded(Q, x, k, b[0], p, cls, gmax, ctx) for x, p, b, (_, ctx) in zip(shards, planes, bounds, seeds)]
    msgs = [kern.pack(d, i, st, world, owner) for d, i, st in outs]
    return kern, outs, msgs


@pytest.mark.parametrize("skew", [False, True])
def test_seeded_shards_merge_to_the_exact_result(skew):
    # shards of 80,000 rows: large enough for the seeding pass to sample them (>= 256 tiles of 256 rows)
    X, Q = synthetic.mixture(320_000, 128, 256, 7, nq=700, clamp=True)
    if skew:
        # rows ordered by distance to the first query: its neighbours, and those of similar queries,
        # all sit in the first shard
        order = ((X - Q[0]) ** 2).sum(1).argsort()
        X = X[order].contiguous()
    k, world = 10, 4
    Xd, Qd = X.cuda(), Q.cuda()
    kern, outs, msgs = run_shards(Xd, Qd, k, world)
    d, i, st = kern.merge(torch.cat(msgs), Q.shape[0], k, world)
    assert st[_lib.FL_STATUS_ERROR].item() == 0, st.tolist()
    _, ref_i = oracle.knn_chunked(Q.numpy(), X.numpy(), k, chunk_size=8192)
    res = parity.knn_parity(Q.numpy(), X.numpy(), d.cpu().numpy(), i.cpu().numpy(), ref_i)
    assert res["ok"], res
    # shards return short lists where their rows cannot matter, and few queries need the exact pass
    short = sum(int((o[1] < 0).any(dim=1).sum()) for o in outs)
    fallbacks = sum(int(o[2][_lib.FL_STATUS_FALLBACK]) for o in outs)
    if skew:
        # the far shards have nothing above the shared thresholds for most queries
        assert short > 0, "no shard ever returned fewer than k rows: the shared thresholds did not bite"
    assert fallbacks <= world * Q.shape[0] // 20, fallbacks
    assert st[_lib.FL_STATUS_FALLBACK].item() == fallbacks


def test_owner_messages_and_status_fold():
    g = torch.Generator().manual_seed(3)
    X = torch.randn(50_000, 64, generator=g).cuda()
    Q = torch.randn(333, 64, generator=g).cuda()
    k, world = 7, 3
    kern, outs, _ = run_shards(X, Q, k, world)
    cpu = OracleKnnKernels()
    # device pack == the restated format, both forms; a sender's error word survives the merge
    bad = torch.tensor([_lib.FL_ETIMEOUT, 0x50003, 2, 0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")
    for owner in (False, True):
        for r, (d, i, st) in enumerate(outs):
            got = kern.pack(d, i, st, world, owner).cpu()
            want = cpu.pack(d.cpu(), i.cpu(), st.cpu(), world, owner)
            assert torch.equal(got, want)
    packed = [kern.pack(d, i, bad if r == 1 else st, world, True) for r, (d, i, st) in enumerate(outs)]
    full = kern.merge(torch.cat([kern.pack(d, i, st, world, False) for d, i, st in outs]), Q.shape[0], k, world)
    for dest in range(world):
        s, e = sharded.shard_bounds(Q.shape[0], world, dest)
        sizes = [(sharded.shard_bounds(Q.shape[0], world, r)[1] - sharded.shard_bounds(Q.shape[0], world, r)[0]) * 2 * k + 8
                 for r in range(world)]
        off = sum(sizes[:dest])
        recv = torch.cat([p[off:off + sizes[dest]] for p in packed])
        d, i, st = kern.merge(recv, e - s, k, world)
        assert torch.equal(d, full[0][s:e]) and torch.equal(i, full[1][s:e])
        assert st[_lib.FL_STATUS_ERROR].item() == _lib.FL_ETIMEOUT and st[_lib.FL_STATUS_WHERE].item() == 0x50003
    _, ref_i = oracle.knn_naive(Q.cpu().numpy(), X.cpu().numpy(), k)
    res = parity.knn_parity(Q.cpu().numpy(), X.cpu().numpy(), full[0].cpu().numpy(), full[1].cpu().numpy(), ref_i)
    assert res["ok"], res


def test_single_process_index_and_plain_call():
    """Without a process group sharded_knn is the local call; the index is then built without collectives."""
    g = torch.Generator().manual_seed(4)
    X = torch.randn(30_000, 32, generator=g).cuda()
    Q = torch.randn(100, 32, generator=g).cuda()
    index = sharded.ShardedKnnIndex(X, 5)
    assert index.min_rows == 30_000 and index.all_tensor_core
    d, i = sharded.sharded_knn(Q, None, 6, index=index, mode="bf16")
    _, ref_i = oracle.knn_naive(Q.cpu().numpy(), X.cpu().numpy(), 6)
    res = parity.knn_parity(Q.cpu().numpy(), X.cpu().numpy(), d.cpu().numpy(), (i - 5).cpu().numpy(), ref_i)
    assert res["ok"], res


@pytest.mark.parametrize("seed", range(16))
def test_random_seeded_shards(seed):
    """Seeded random sweep of the shared-seed flow on one GPU: shard counts, uneven shard sizes (rows not
    divisible by the shard count), features, k up to 16, data sorted towards one shard or not."""
    r = np.random.RandomState(seed)
    world = int(r.choice([2, 3, 5, 8]))
    m = int(r.choice([world * 300 + 1, 70_001, 200_003]))
    d = int(r.choice([8, 64, 100, 128, 200]))
    k = int(r.choice([1, 5, 10, 16]))
    nq = int(r.choice([1, 129, 700]))
    g = torch.Generator().manual_seed(40 + seed)
    centres = 2 * torch.randn(30, d, generator=g)
    X = centres[torch.randint(0, 30, (m,), generator=g)] + torch.randn(m, d, generator=g)
    Q = centres[torch.randint(0, 30, (nq,), generator=g)] + torch.randn(nq, d, generator=g)
    if r.randint(2):
        X = X[((X - Q[0]) ** 2).sum(1).argsort()].contiguous()
    Xd, Qd = X.cuda(), Q.cuda()
    kern, outs, msgs = run_shards(Xd, Qd, k, world)
    dd, ii, st = kern.merge(torch.cat(msgs), nq, k, world)
    assert st[_lib.FL_STATUS_ERROR].item() == 0, st.tolist()
    qd, xd = Qd.double(), Xd.double()
    d64 = (qd * qd).sum(-1, keepdim=True) + (xd * xd).sum(-1)[None, :] - 2.0 * qd @ xd.T
    ref_i = d64.topk(k, dim=1, largest=False).indices.cpu().numpy()
    res = parity.knn_parity(Q.numpy(), X.numpy(), dd.cpu().numpy(), ii.cpu().numpy(), ref_i)
    assert res["ok"], (seed, world, m, d, k, nq, res)
