"""GPU parity of the kNN path (through the C ABI) against the reference fixtures and the
numpy oracle."""
import os

import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200 import _lib, synthetic
from flashlib_b200.knn import knn_f32
from oracle import oracle
from tests import parity

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")
MODES = ["exact", "auto"]


def dev(a):
    return torch.as_tensor(a).cuda()


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("k", [1, 10, 100])
def test_golden_small(k, mode):
    d = np.load(os.path.join(G, "knn_small.npz"))
    vals, idxs = fl.flash_knn(dev(d["q"]), dev(d["db"]), k, mode=None if mode == "auto" else mode)
    assert vals.dtype == torch.float32 and idxs.dtype == torch.int32
    res = parity.knn_parity(d["q"], d["db"], vals.cpu().numpy(), idxs.cpu().numpy(), d[f"idxs_k{k}"])
    assert res["ok"], res
    assert parity.rel_close(vals.cpu().numpy(), d[f"vals_k{k}"], rel=1e-4, atol=1e-4)


@pytest.mark.parametrize("mode", MODES)
def test_golden_mixture(mode):
    d = np.load(os.path.join(G, "knn_mixture.npz"))
    db, q = d["db"].astype(np.float32), d["q"].astype(np.float32)
    vals, idxs = fl.flash_knn(dev(q), dev(db), int(d["k"]), mode=None if mode == "auto" else mode)
    res = parity.knn_parity(q, db, vals.cpu().numpy(), idxs.cpu().numpy(), d["idxs"])
    assert res["ok"], res


@pytest.mark.parametrize("mode", MODES)
def test_cpu_config_full(mode):
    """The reference's CPU-runnable configuration (20 000 x 64, 1 000 queries, k=10, seed 0)."""
    cfg = synthetic.CONFIGS["knn_cpu_small"]
    db, q = synthetic.randn_knn(cfg["m"], cfg["d"], cfg["nq"], cfg["seed"])
    ref_v, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), cfg["k"])
    vals, idxs = fl.flash_knn(q.cuda(), db.cuda(), cfg["k"], mode=None if mode == "auto" else mode)
    res = parity.knn_parity(q.numpy(), db.numpy(), vals.cpu().numpy(), idxs.cpu().numpy(), ref_i)
    assert res["ok"], res
    d = np.load(os.path.join(G, "knn_cpu_config.npz"))
    res = parity.knn_parity(q.numpy(), db.numpy(), vals.cpu().numpy(), idxs.cpu().numpy(), d["idxs"])
    assert res["ok"], res


SHAPES = [  # nq, m, d, k
    (1, 1, 1, 1), (1, 300, 3, 5), (129, 257, 17, 10), (64, 1000, 200, 32), (33, 4097, 64, 100),
    (7, 600, 128, 512), (500, 50_000, 128, 10), (130, 20_001, 96, 16), (256, 9_000, 256, 10),
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("nq,m,d,k", SHAPES)
def test_shapes_vs_oracle(nq, m, d, k, mode):
    g = torch.Generator().manual_seed(nq * 7919 + m)
    db = torch.randn(m, d, generator=g)
    q = torch.randn(nq, d, generator=g)
    ref_v, ref_i = oracle.knn_naive(q.numpy(), db.numpy(), k)
    vals, idxs = fl.flash_knn(q.cuda(), db.cuda(), k, mode=None if mode == "auto" else mode)
    res = parity.knn_parity(q.numpy(), db.numpy(), vals.cpu().numpy(), idxs.cpu().numpy(), ref_i)
    assert res["ok"], res


def test_strided_rows_batch_and_dtypes():
    g = torch.Generator().manual_seed(3)
    big = torch.randn(2, 700, 80, generator=g).cuda()
    c = big[:, :, :48]                      # rows strided by 80
    x = torch.randn(2, 50, 48, generator=g).cuda()
    vals, idxs = fl.flash_knn(x, c, 6)
    assert vals.shape == (2, 50, 6) and idxs.shape == (2, 50, 6)
    for b in range(2):
        _, ref_i = oracle.knn_naive(x[b].cpu().numpy(), c[b].cpu().numpy(), 6)
        res = parity.knn_parity(x[b].cpu().numpy(), c[b].cpu().numpy(), vals[b].cpu().numpy(),
                                idxs[b].cpu().numpy(), ref_i)
        assert res["ok"], res
    only = fl.flash_knn(x, c, 6, return_distances=False)
    assert torch.equal(only, idxs)
    xb, cb = x[0].bfloat16(), c[0].bfloat16()
    vb, ib = fl.flash_knn(xb, cb, 4)
    _, ref_i = oracle.knn_naive(xb.float().cpu().numpy(), cb.float().cpu().numpy(), 4)
    res = parity.knn_parity(xb.float().cpu().numpy(), cb.float().cpu().numpy(), vb.cpu().numpy(),
                            ib.cpu().numpy(), ref_i)
    assert res["ok"], res
    with pytest.raises(AssertionError):
        fl.flash_knn(x, c, 701)


def test_duplicates_and_self_match():
    g = torch.Generator().manual_seed(5)
    base = torch.randn(300, 32, generator=g)
    db = torch.cat([base, base[:50]]).cuda()       # rows 300..349 duplicate rows 0..49
    nn_ = fl.NearestNeighbors(n_neighbors=3).fit(db)
    dist, idx = nn_.kneighbors()
    assert torch.all(dist[:, 0] == 0)
    assert torch.all(idx[:50, 0] == torch.arange(50, device="cuda"))       # lower row wins the tie
    assert torch.all(idx[:50, 1] == torch.arange(300, 350, device="cuda"))
    assert torch.all(dist[:50, 1] == 0)


def test_gather_and_rownorm():
    g = torch.Generator().manual_seed(6)
    x = torch.randn(1, 40, 70, generator=g).cuda()
    c = torch.randn(1, 90, 70, generator=g).cuda()
    idx = torch.randint(0, 90, (1, 40, 5), generator=g).cuda()
    out = fl.triton_knn_gather_sqdist(x, c, idx)
    ref = ((x[0][:, None, :] - c[0][idx[0]]) ** 2).sum(-1)
    assert torch.allclose(out[0], ref, rtol=1e-5, atol=1e-5)
    out32 = fl.triton_knn_gather_sqdist(x, c, idx.int())
    assert torch.equal(out, out32)
    n = fl.row_sqnorm(c[0])
    assert torch.allclose(n, (c[0] ** 2).sum(-1), rtol=1e-5)


def test_sharded_emulation_and_merge():
    """Row shards with global offsets + fl_topk_merge_f32 reproduce the unsharded result."""
    g = torch.Generator().manual_seed(7)
    db = torch.randn(10_000, 64, generator=g).cuda()
    q = torch.randn(200, 64, generator=g).cuda()
    k = 10
    full_d, full_i, _ = knn_f32(q, db, k)
    parts_d, parts_i = [], []
    bounds = [0, 2500, 5000, 7501, 10_000]
    for s, e in zip(bounds[:-1], bounds[1:]):
        d_, i_, _ = knn_f32(q, db[s:e], k, row_offset=s)
        parts_d.append(d_)
        parts_i.append(i_)
    md, mi = fl.topk_merge(torch.cat(parts_d, 1), torch.cat(parts_i, 1), k)
    assert torch.equal(mi, full_i)
    assert torch.equal(md, full_d)


def test_full_size_properties():
    """1M x 128 clamped mixture, 10 000 queries, k in {10, 100}: oracle parity on a query
    subset plus size-independent properties on all rows."""
    cfg = synthetic.CONFIGS["knn_1m"]
    X, Q = synthetic.mixture(cfg["n"], cfg["d"], cfg["n_comp"], cfg["seed"], nq=cfg["nq"], clamp=True)
    Xd, Qd = X.cuda(), Q.cuda()
    sub = np.arange(0, cfg["nq"], 79)[:128]
    for k in (10, 100):
        vals, idxs = fl.flash_knn(Qd, Xd, k)
        # ascending, unique ids, distances equal to the exact gather
        assert torch.all(vals[:, 1:] >= vals[:, :-1])
        srt = torch.sort(idxs.long(), dim=1).values
        assert torch.all(srt[:, 1:] != srt[:, :-1])
        gathered = fl.triton_knn_gather_sqdist(Qd[None], Xd[None], idxs[None])[0]
        assert torch.allclose(gathered, vals, rtol=1e-5, atol=1e-4)
        ref_v, ref_i = oracle.knn_chunked(Q[sub].numpy(), X.numpy(), k, chunk_size=8192)
        res = parity.knn_parity(Q[sub].numpy(), X.numpy(), vals[sub].cpu().numpy(), idxs[sub].cpu().numpy(), ref_i)
        assert res["ok"], res


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("nq,m,d,k,mode", [(300, 70_000, 128, 10, "bf16"), (64, 5_000, 96, 10, "exact"), (200, 90_000, 64, 32, "bf16"),
                                           (129, 30_001, 100, 5, "bf16"), (33, 2_000, 200, 50, "exact"), (500, 40_000, 128, 10, None)])
def test_sixteen_bit_rows_are_read_as_stored(dtype, nq, m, d, k, mode):
    """bf16 / fp16 inputs: no fp32 copy is made; the result is the exact kNN of the stored values
    (fp64 brute force on them), distances in fp32."""
    g = torch.Generator().manual_seed(nq + m + d)
    db = torch.randn(m, d, generator=g).to(dtype).cuda()
    q = torch.randn(nq, d, generator=g).to(dtype).cuda()
    vals, idxs = fl.flash_knn(q, db, k, mode=mode)
    assert vals.dtype == torch.float32 and idxs.dtype == torch.int32
    qd, dbd = q.double(), db.double()
    d64 = (qd * qd).sum(-1, keepdim=True) + (dbd * dbd).sum(-1)[None, :] - 2.0 * qd @ dbd.T
    ref_i = d64.topk(k, dim=1, largest=False).indices.cpu().numpy()
    res = parity.knn_parity(q.float().cpu().numpy(), db.float().cpu().numpy(), vals.cpu().numpy(), idxs.cpu().numpy(), ref_i)
    assert res["ok"], res
    fl.check_pending()


def test_tol_stores_the_inputs_in_sixteen_bits():
    """``tol`` >= 4e-4 selects fp16 storage (the reference's rule): same result as passing fp16 inputs,
    and the cast database is made once."""
    from flashlib_b200 import knn as knn_mod
    g = torch.Generator().manual_seed(3)
    db = torch.randn(80_000, 128, generator=g).cuda()
    q = torch.randn(400, 128, generator=g).cuda()
    v_tol, i_tol = fl.flash_knn(q, db, 10, tol=1e-3)
    v_16, i_16 = fl.flash_knn(q.half(), db.half(), 10)
    assert torch.equal(i_tol, i_16) and torch.equal(v_tol, v_16)
    n_cached = len(knn_mod._CAST_CACHE)
    fl.flash_knn(q, db, 10, tol=1e-3)
    assert len(knn_mod._CAST_CACHE) == n_cached
    v_32, i_32 = fl.flash_knn(q, db, 10, tol=1e-5)      # too tight for 16-bit storage: fp32 kept
    v_ex, i_ex = fl.flash_knn(q, db, 10)
    assert torch.equal(i_32, i_ex) and torch.equal(v_32, v_ex)
    fl.check_pending()


@pytest.mark.parametrize("B,N,M,d,k", [(16, 200, 300, 2, 5), (16, 257, 1000, 8, 10), (64, 100, 256, 4, 1), (3, 500, 5000, 33, 40)])
def test_batched_small_problems_in_one_call(B, N, M, d, k):
    """B > 1: one launch sequence for the whole batch (problem b on grid axis b), each item equal to
    the oracle on that item alone; strided batches (a slice of a larger tensor) included."""
    g = torch.Generator().manual_seed(B * 1000 + M)
    big_c = torch.randn(B, M + 7, d + 4, generator=g).cuda()
    c = big_c[:, 3:3 + M, :d] if d % 4 == 0 else big_c[:, 3:3 + M, :d].contiguous()
    x = torch.randn(B, N, d, generator=g).cuda()
    lib = _lib.load()
    before = lib.fl_launch_count()
    vals, idxs = fl.flash_knn(x, c, k)
    launches = lib.fl_launch_count() - before
    assert launches <= 4, launches                      # norms, scan, finalisation: not 3 per item
    assert vals.shape == (B, N, k) and idxs.dtype == torch.int32
    for b in range(B):
        _, ref_i = oracle.knn_naive(x[b].cpu().numpy(), c[b].cpu().numpy(), k)
        res = parity.knn_parity(x[b].cpu().numpy(), c[b].cpu().numpy(), vals[b].cpu().numpy(), idxs[b].cpu().numpy(), ref_i)
        assert res["ok"], (b, res)
    only_idx = fl.flash_knn(x, c, k, return_distances=False)
    assert torch.equal(only_idx, idxs)
