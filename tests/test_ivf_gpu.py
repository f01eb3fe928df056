"""GPU parity of the IVF-Flat search against the reference fixture (same index on both
sides, the protocol of the reference's tests/test_primitives_correctness.py:135-164)."""
import os

import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200.ivf_flat import IvfFlatIndex
from oracle import oracle
from tests import parity

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def golden_index():
    d = np.load(os.path.join(G, "ivf_small.npz"))
    idx = IvfFlatIndex(centroids=torch.from_numpy(d["centroids"]).cuda(), data=torch.from_numpy(d["data"]).cuda(),
                       ids=torch.from_numpy(d["ids"]).cuda(), list_offsets=torch.from_numpy(d["list_offsets"]).cuda(),
                       metric="l2", D=d["x"].shape[1], Dp=d["data"].shape[1], nlist=int(d["nlist"]), nprobe=4)
    return d, idx


@pytest.mark.parametrize("k,nprobe", [(10, 4), (5, 32), (10, 1)])
def test_search_matches_reference_on_same_index(k, nprobe):
    d, index = golden_index()
    vals, ids = fl.flash_ivf_flat_search(index, torch.from_numpy(d["q"]).cuda(), k, nprobe=nprobe)
    assert vals.dtype == torch.float32 and ids.dtype == torch.int64
    ref_v, ref_i = d[f"vals_k{k}_p{nprobe}"], d[f"ids_k{k}_p{nprobe}"]
    v, i = vals.cpu().numpy(), ids.cpu().numpy()
    finite = np.isfinite(ref_v)
    assert np.array_equal(np.isfinite(v), finite)
    assert np.all(i[~finite] == -1)
    assert parity.rel_close(v[finite], ref_v[finite], rel=1e-4, atol=1e-4)
    same = np.mean([set(a[f].tolist()) == set(b[f].tolist()) for a, b, f in zip(i, ref_i, finite)])
    assert same >= 0.99, same


def test_exhaustive_probe_equals_brute_force():
    d, index = golden_index()
    q = torch.from_numpy(d["q"]).cuda()
    vals, ids = fl.flash_ivf_flat_search(index, q, 10, nprobe=index.nlist)
    bv, bi = fl.flash_knn(q, torch.from_numpy(d["x"]).cuda(), 10)
    assert torch.allclose(vals, bv, rtol=1e-5, atol=1e-5)
    assert torch.equal(ids, bi.long())


def test_build_and_recall():
    g = torch.Generator().manual_seed(21)
    means = 2 * torch.randn(50, 24, generator=g)
    X = (means[torch.randint(0, 50, (20_000,), generator=g)] + torch.randn(20_000, 24, generator=g)).cuda()
    Q = (means[torch.randint(0, 50, (300,), generator=g)] + torch.randn(300, 24, generator=g)).cuda()
    ivf = fl.IVFFlat(nlist=64, nprobe=8, niter=8, seed=1).fit(X)
    idx = ivf.index_
    assert idx.list_offsets[-1].item() == 20_000 and idx.data.shape == (20_000, 24)
    assert torch.equal(torch.sort(idx.ids).values, torch.arange(20_000, device="cuda"))
    _, bi = fl.flash_knn(Q, X, 10)
    recalls = []
    for nprobe in (1, 8, 64):
        vals, ids = ivf.kneighbors(Q, 10, nprobe=nprobe)
        recalls.append(np.mean([len(set(a.tolist()) & set(b.tolist())) / 10 for a, b in zip(ids.cpu().numpy(), bi.cpu().numpy())]))
    assert recalls[0] <= recalls[1] <= recalls[2] and recalls[2] == 1.0 and recalls[1] > 0.9, recalls
    # same index through the oracle
    ov, oi, _ = oracle.ivf_search(idx.centroids.cpu().numpy(), idx.data.cpu().numpy(), idx.ids.cpu().numpy(),
                                  idx.list_offsets.cpu().numpy(), Q.cpu().numpy(), 10, 8)
    vals, ids = ivf.kneighbors(Q, 10)
    assert parity.rel_close(vals.cpu().numpy(), ov, rel=1e-4, atol=1e-4)
    assert np.mean(np.sort(ids.cpu().numpy(), 1) == np.sort(oi, 1)) >= 0.99


def test_small_dim_padding_and_short_lists():
    g = torch.Generator().manual_seed(22)
    X = torch.randn(200, 5, generator=g).cuda()            # D < 16 is zero padded to 16
    ivf = fl.IVFFlat(nlist=40, nprobe=1, niter=3).fit(X)
    assert ivf.index_.Dp == 16 and ivf.index_.D == 5
    vals, ids = ivf.kneighbors(X[:20], 12)
    assert vals.shape == (20, 12)
    pad = ids < 0
    assert torch.all(torch.isinf(vals[pad])) and torch.all(torch.isfinite(vals[~pad]))
    assert torch.all(ids[:, 0] == torch.arange(20, device="cuda"))
    with pytest.raises(ValueError):
        ivf.kneighbors(X[:2], 201)


@pytest.mark.parametrize("k,nprobe", [(10, 4), (5, 32), (1, 1), (8, 8)])
def test_tensor_core_fine_scan_matches_reference_fixture(k, nprobe):
    """variant="gemm": the fine scan on the tensor-core kernel, against the reference's outputs on
    the same index (and against the CUDA-core variant)."""
    d, index = golden_index()
    q = torch.from_numpy(d["q"]).cuda()
    vals, ids = fl.flash_ivf_flat_search(index, q, k, nprobe=nprobe, variant="gemm")
    ev, ei = fl.flash_ivf_flat_search(index, q, k, nprobe=nprobe, variant="elementwise")
    assert index._tc_plane is not None and index._last_status is not None
    assert index._last_status[0].item() == 0
    torch.testing.assert_close(vals, ev, rtol=1e-5, atol=1e-5)
    assert (ids == ei).float().mean().item() >= 0.999
    key = f"vals_k{k}_p{nprobe}"
    if key in d.files:
        ref_v, ref_i = d[key], d[f"ids_k{k}_p{nprobe}"]
        v, i = vals.cpu().numpy(), ids.cpu().numpy()
        finite = np.isfinite(ref_v)
        assert np.array_equal(np.isfinite(v), finite)
        assert parity.rel_close(v[finite], ref_v[finite], rel=1e-4, atol=1e-4)
        same = np.mean([set(a[f].tolist()) == set(b[f].tolist()) for a, b, f in zip(i, ref_i, finite)])
        assert same >= 0.99, same


@pytest.mark.parametrize("n,dim,nlist,nprobe,nq,k", [(60_000, 64, 128, 8, 700, 10), (30_000, 96, 37, 5, 1500, 16),
                                                   (5_000, 128, 300, 20, 64, 3), (100_000, 128, 256, 16, 4000, 10),
                                                   (40_000, 200, 64, 8, 900, 10), (50_000, 256, 100, 10, 2000, 5)])
def test_tensor_core_fine_scan_equals_cuda_core_scan(n, dim, nlist, nprobe, nq, k):
    """Same index, same probed lists: both fine scans return the same rows and distances.  Shapes
    cover lists shorter than k, empty lists (more lists than a cluster structure fills), query
    tiles with a few pairs and lists probed by more than 128 queries."""
    from flashlib_b200.ivf_flat import ivf_fine_scan
    g = torch.Generator().manual_seed(n + nq)
    means = 2 * torch.randn(40, dim, generator=g)
    X = (means[torch.randint(0, 40, (n,), generator=g)] + torch.randn(n, dim, generator=g)).cuda()
    Q = (means[torch.randint(0, 40, (nq,), generator=g)] + torch.randn(nq, dim, generator=g)).cuda()
    index = fl.flash_ivf_flat_build(X, nlist, nprobe=nprobe, niter=4, seed=3)
    probed = fl.flash_knn(Q, index.centroids, nprobe, return_distances=False, mode="exact")
    ev, ep = ivf_fine_scan(Q, index, probed, k, mode="exact")
    tv, tp = ivf_fine_scan(Q, index, probed, k, mode="bf16")
    st = index._last_status.tolist()
    assert st[0] == 0, st
    assert torch.equal(torch.isfinite(tv), torch.isfinite(ev))
    fin = torch.isfinite(ev)
    torch.testing.assert_close(tv[fin], ev[fin], rtol=1e-5, atol=1e-5)
    assert (tp == ep).float().mean().item() >= 0.9995
    assert st[2] <= nq // 10, st           # few queries need the exact scan


def test_row_sharded_index_merges_to_the_unsharded_result():
    """Two row shards indexed under the same centroids, searched separately and merged with
    fl_topk_merge_f32 (what sharded_ivf_search does per rank) equal the unsharded index."""
    from flashlib_b200 import sharded
    from flashlib_b200.knn import topk_merge
    g = torch.Generator().manual_seed(31)
    means = 2 * torch.randn(30, 48, generator=g)
    X = (means[torch.randint(0, 30, (40_000,), generator=g)] + torch.randn(40_000, 48, generator=g)).cuda()
    Q = (means[torch.randint(0, 30, (500,), generator=g)] + torch.randn(500, 48, generator=g)).cuda()
    whole = fl.flash_ivf_flat_build(X, 64, nprobe=6, niter=4, seed=5)
    wv, wi = fl.flash_ivf_flat_search(whole, Q, 10)
    cents = whole.centroids[:, :48].contiguous()
    parts = []
    for r in range(2):
        s, e = sharded.shard_bounds(X.shape[0], 2, r)
        local = sharded.sharded_ivf_build(X[s:e], cents, row_offset=s, nprobe=6)
        assert int(local.list_offsets[-1].item()) == e - s
        parts.append(sharded.sharded_ivf_search(local, Q, 10))          # world of one: the local result
    cd = torch.cat([p[0] for p in parts], 1)
    ci = torch.cat([p[1] for p in parts], 1).to(torch.int32)
    mv, mi = topk_merge(cd, ci, 10)
    torch.testing.assert_close(mv, wv, rtol=1e-5, atol=1e-5)
    assert (mi.long() == wi).float().mean().item() > 0.999


def test_device_side_build_matches_the_reference_layout():
    """index_from_centroids (histogram + scan + stable partition on the device) against the
    reference-built fixture: same offsets, same row order, same stored rows -- the check of
    tests/test_oracle_golden.py::test_ivf_layout_matches_reference, on the CUDA path."""
    from flashlib_b200.ivf_flat import _pad_features, index_from_centroids
    d, _ = golden_index()
    X = torch.from_numpy(d["x"]).cuda()
    cents = torch.from_numpy(d["centroids"]).cuda()
    Xp = _pad_features(X, d["data"].shape[1]).contiguous()
    idx = index_from_centroids(Xp, cents, D=X.shape[1], nprobe=4)
    assert idx.list_offsets.dtype == torch.int64 and idx.ids.dtype == torch.int64
    assert np.array_equal(idx.list_offsets.cpu().numpy(), d["list_offsets"])
    assert np.array_equal(idx.ids.cpu().numpy(), d["ids"])
    assert np.array_equal(idx.data.cpu().numpy(), d["data"])
    lens = np.diff(d["list_offsets"])
    assert idx.max_list_len == int(lens.max()) and isinstance(idx.max_list_len, int)


@pytest.mark.parametrize("m,dim,nlist", [(1, 16, 1), (33, 16, 7), (5000, 24, 300), (300_000, 32, 1024), (70_000, 128, 5000)])
def test_device_side_build_is_a_stable_partition(m, dim, nlist):
    """Labels straight into fl_ivf_build_csr_f32: the layout must equal numpy's stable argsort by
    label, with empty lists (more lists than labels used) and units that end mid-warp."""
    from flashlib_b200 import _lib
    from flashlib_b200.knn import _stream_ptr
    lib = _lib.load()
    g = torch.Generator().manual_seed(m + nlist)
    x = torch.randn(m, dim, generator=g).cuda()
    used = max(1, nlist - nlist // 3)
    lab = torch.randint(0, used, (m,), generator=g, dtype=torch.int32)
    labd = lab.cuda()
    data = torch.empty_like(x)
    ids = torch.empty(m, dtype=torch.int64, device="cuda")
    offs = torch.empty(nlist + 1, dtype=torch.int64, device="cuda")
    longest = torch.empty(1, dtype=torch.int32, device="cuda")
    ws_bytes = lib.fl_ivf_build_workspace_bytes(m, nlist)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    _lib.check(lib.fl_ivf_build_csr_f32(x.data_ptr(), m, x.stride(0), dim, labd.data_ptr(), nlist, data.data_ptr(),
                                        ids.data_ptr(), offs.data_ptr(), longest.data_ptr(), ws.data_ptr(), ws_bytes,
                                        _stream_ptr(x.device)))
    order = np.argsort(lab.numpy(), kind="stable")
    counts = np.bincount(lab.numpy(), minlength=nlist)
    assert np.array_equal(offs.cpu().numpy(), np.concatenate([[0], np.cumsum(counts)]))
    assert np.array_equal(ids.cpu().numpy(), order)
    assert torch.equal(data.cpu(), x.cpu()[torch.from_numpy(order)])
    assert int(longest.item()) == int(counts.max())
