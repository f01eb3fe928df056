"""GPU parity of the k-means path against the reference fixtures and the numpy oracle."""
import os

import numpy as np
import pytest
import torch

import flashlib_b200 as fl
from flashlib_b200 import synthetic
from oracle import oracle
from tests import parity

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def test_assign_update_golden():
    d = np.load(os.path.join(G, "kmeans_small.npz"))
    x = torch.from_numpy(d["x"]).cuda()
    init = torch.from_numpy(d["init"]).cuda()
    lab = fl.euclid_assign_triton(x[None], init[None])
    assert lab.dtype == torch.int32 and lab.shape == (1, x.shape[0])
    assert parity.label_parity(d["x"], d["init"], lab[0].cpu().numpy(), d["labels0"])["ok"]
    ref_lab = torch.from_numpy(d["labels0"]).cuda()
    new, ids, shift = fl.triton_lloyd_centroid_step_euclid(x[None], ref_lab[None], init[None])
    assert parity.rel_close(new[0].cpu().numpy(), d["new0"], rel=1e-4, atol=1e-5)
    ref_shift = np.sqrt(((d["new0"] - d["init"]) ** 2).sum(-1)).max()
    assert abs(float(shift) - ref_shift) <= 1e-4 * ref_shift


def test_loop_teacher_forced_and_end_to_end():
    d = np.load(os.path.join(G, "kmeans_small.npz"))
    x = torch.from_numpy(d["x"]).cuda()
    hc, hl = d["hist_centroids"], d["hist_labels"]
    for t in range(hl.shape[0]):
        c = torch.from_numpy(hc[t]).cuda()
        lab = fl.euclid_assign_triton(x[None], c[None])
        assert parity.label_parity(d["x"], hc[t], lab[0].cpu().numpy(), hl[t])["ok"]
        new, _, _ = fl.triton_lloyd_centroid_step_euclid(x[None], lab, c[None])
        assert parity.rel_close(new[0].cpu().numpy(), hc[t + 1], rel=1e-4, atol=1e-5)
    ids, cents, n_iter = fl.flash_kmeans(x, int(d["K"]), max_iters=6, init_centroids=torch.from_numpy(d["init"]).cuda())
    assert n_iter == int(d["n_iter"]) and ids.dtype == torch.int32 and ids.shape == (x.shape[0],)
    assert np.mean(ids.cpu().numpy() == d["final_labels"]) > 0.999
    assert parity.rel_close(cents.cpu().numpy(), d["final_centroids"], rel=1e-3, atol=1e-3)


@pytest.mark.parametrize("n,d,K", [(257, 32, 257), (1000, 128, 7), (4096, 768, 64), (5000, 3, 10), (300, 130, 300)])
def test_assign_shapes_vs_oracle(n, d, K):
    g = torch.Generator().manual_seed(n + K)
    x = torch.randn(n, d, generator=g)
    c = torch.randn(K, d, generator=g)
    ref = oracle.kmeans_assign(x.numpy(), c.numpy())
    lab = fl.euclid_assign_triton(x.cuda()[None], c.cuda()[None])[0]
    assert parity.label_parity(x.numpy(), c.numpy(), lab.cpu().numpy(), ref)["ok"]
    new_ref, sums_ref, cnts_ref = oracle.kmeans_update(x.numpy(), ref.astype(np.int64), c.numpy())
    sums, cnts = fl.triton_centroid_update_euclid(x.cuda()[None], torch.from_numpy(ref).cuda()[None],
                                                  c.cuda()[None], calculate_new=False)
    assert np.array_equal(cnts[0].cpu().numpy(), cnts_ref)
    assert parity.rel_close(sums[0].cpu().numpy(), sums_ref, rel=1e-4, atol=1e-4)


def test_empty_cluster_batch_and_tolerance_break():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 400, 8, generator=g).cuda()
    init = x[:, :5].clone()
    init[:, 4] = 1000.0                           # never wins: stays empty, keeps its value
    ids, cents, n_iter = fl.flash_kmeans(x, 5, max_iters=4, init_centroids=init)
    assert ids.shape == (2, 400) and cents.shape == (2, 5, 8) and n_iter == 4
    assert torch.all(cents[:, 4] == 1000.0)
    assert not torch.any(ids == 4)
    ids2, cents2, n2 = fl.flash_kmeans(x, 5, max_iters=100, tol=1e-6, init_centroids=init)
    assert n2 < 100
    km = fl.KMeans(d=8, k=5, niter=3, tol=0.0, seed=0)
    lab = km.fit_predict(x[0])
    assert lab.shape == (400,) and torch.equal(km.predict(x[0]).cpu() >= 0, torch.ones(400, dtype=torch.bool))


def test_full_size_one_iteration():
    """1M x 128 mixture, K = 1024, init = first K rows: one teacher-forced step against the
    oracle plus conservation properties."""
    cfg = synthetic.CONFIGS["kmeans_1m"]
    X, _ = synthetic.mixture(cfg["n"], cfg["d"], cfg["n_comp"], cfg["seed"])
    Xd = X.cuda()
    init = Xd[:cfg["K"]].clone()
    lab = fl.euclid_assign_triton(Xd[None], init[None])[0]
    ref = oracle.kmeans_assign(X.numpy(), X[:cfg["K"]].numpy())
    assert parity.label_parity(X.numpy(), X[:cfg["K"]].numpy(), lab.cpu().numpy(), ref)["ok"]
    sums, cnts = fl.triton_centroid_update_euclid(Xd[None], lab[None], init[None], calculate_new=False)
    assert int(cnts.sum()) == cfg["n"]
    tot = X.double().sum(0)
    assert torch.allclose(sums[0].double().sum(0).cpu(), tot, rtol=1e-5, atol=2.0)  # fp32 sums of 1e6 rows
    new_ref, _, _ = oracle.kmeans_update(X.numpy(), lab.cpu().numpy().astype(np.int64), X[:cfg["K"]].numpy())
    new, _ = fl.triton_centroid_finalize(sums, cnts, init[None])
    assert parity.rel_close(new[0].cpu().numpy(), new_ref, rel=1e-4, atol=1e-5)


@pytest.mark.parametrize("n,d,K", [(300, 32, 40), (5000, 128, 1024), (20_000, 96, 300), (4097, 256, 257), (1000, 16, 3)])
def test_tensor_core_assign_equals_exact_assign(n, d, K):
    g = torch.Generator().manual_seed(n * 3 + K)
    means = 2 * torch.randn(K, d, generator=g)
    x = (means[torch.randint(0, K, (n,), generator=g)] + torch.randn(n, d, generator=g)).cuda()
    c = (means + 0.3 * torch.randn(K, d, generator=g)).cuda()
    ref = oracle.kmeans_assign(x.cpu().numpy(), c.cpu().numpy())
    tc = fl.euclid_assign_triton(x[None], c[None], mode="bf16")[0]
    ex = fl.euclid_assign_triton(x[None], c[None], mode="exact")[0]
    assert parity.label_parity(x.cpu().numpy(), c.cpu().numpy(), tc.cpu().numpy(), ref)["ok"]
    assert parity.label_parity(x.cpu().numpy(), c.cpu().numpy(), tc.cpu().numpy(), ex.cpu().numpy())["ok"]


def test_tensor_core_assign_near_duplicate_centroids():
    """Centroids that nearly coincide cannot be separated by bf16 scores: those points must come
    back through the exact path with the exact winner (lowest index on exact ties)."""
    g = torch.Generator().manual_seed(4)
    base = torch.randn(64, 64, generator=g)
    c = torch.cat([base, base + 1e-3 * torch.randn(64, 64, generator=g), base[:16]]).cuda()   # 144 centroids
    x = (base[torch.randint(0, 64, (3000,), generator=g)] + 0.05 * torch.randn(3000, 64, generator=g)).cuda()
    tc = fl.euclid_assign_triton(x[None], c[None], mode="bf16")[0]
    xd, cd = x.double(), c.double()
    d64 = (xd * xd).sum(-1, keepdim=True) + (cd * cd).sum(-1)[None] - 2 * xd @ cd.T
    best = d64.min(1).values
    got = d64[torch.arange(3000, device="cuda"), tc.long()]
    assert torch.all((got - best).abs() <= 1e-5 * best + 1e-6)
    assert not torch.any(tc >= 128)          # rows 128.. duplicate rows 0..15 exactly: lower index wins


def test_large_n_streaming_matches_resident_kmeans():
    """kmeans_largeN (samples in pinned host memory, streamed in blocks over two streams) follows
    the same Lloyd iterations as flash_kmeans on GPU-resident data.  One iteration is compared
    value for value; over several iterations the fp32 atomics of the centroid sums let a boundary
    point flip between runs (of either path), so the clusterings are compared by their inertia."""
    import flashlib_b200 as fl
    g = torch.Generator().manual_seed(17)
    means = 3 * torch.randn(40, 32, generator=g)
    X = (means[torch.randint(0, 40, (150_000,), generator=g)] + torch.randn(150_000, 32, generator=g))
    init = X[:40].clone()
    Xp, Xd = X.pin_memory(), X.cuda()
    ids_l, cent_l = fl.kmeans_largeN(Xp, 40, max_iters=1, BLOCK_N=40_000, init_centroids=init)
    ids_r, cent_r, _ = fl.flash_kmeans(Xd, 40, max_iters=1, init_centroids=init.cuda())
    assert ids_l.dtype == torch.int32 and not ids_l.is_cuda and ids_l.shape == (150_000,)
    assert torch.equal(ids_l, ids_r.cpu())
    torch.testing.assert_close(cent_l.cpu(), cent_r.cpu(), rtol=1e-4, atol=1e-4)

    def inertia(cent):
        lab = fl.euclid_assign_triton(Xd[None], cent.cuda().float()[None])[0].long()
        return float(((Xd - cent.cuda().float()[lab]) ** 2).sum(1).mean())

    ids_l, cent_l = fl.kmeans_largeN(Xp, 40, max_iters=6, BLOCK_N=40_000, init_centroids=init)
    ids_r, cent_r, _ = fl.flash_kmeans(Xd, 40, max_iters=6, init_centroids=init.cuda())
    assert abs(inertia(cent_l) - inertia(cent_r)) <= 1e-3 * inertia(cent_r)
    assert (ids_l == ids_r.cpu()).float().mean().item() > 0.999
    again = fl.kmeans_largeN_assign(X, cent_l, BLOCK_N=64_000)
    direct = fl.euclid_assign_triton(Xd[None], cent_l.float()[None])[0].cpu()
    assert torch.equal(again, direct)


@pytest.mark.parametrize("B,n,d,K", [(16, 3000, 2, 256), (16, 2500, 8, 256), (5, 777, 3, 17), (3, 4000, 128, 40)])
def test_batched_small_problems_match_the_oracle_per_item(B, n, d, K):
    """Many small problems in one launch (the sub-quantiser regime of the reference's IVF-PQ build,
    ivf_pq/triton/build.py:41-70): assignment, update and finalisation per batch item against the
    oracle, and the batched Lloyd loop end to end."""
    g = torch.Generator().manual_seed(B * 1000 + d)
    x = torch.randn(B, n, d, generator=g)
    c = x[:, :K].clone() + 0.01 * torch.randn(B, K, d, generator=g)
    xd, cd = x.cuda(), c.cuda()
    lab = fl.euclid_assign_triton(xd, cd)
    assert lab.shape == (B, n) and lab.dtype == torch.int32
    sums, cnts = fl.triton_centroid_update_euclid(xd, lab, cd, calculate_new=False)
    new, shift = fl.triton_centroid_finalize(sums, cnts, cd)
    for b in range(B):
        ref = oracle.kmeans_assign(x[b].numpy(), c[b].numpy())
        assert parity.label_parity(x[b].numpy(), c[b].numpy(), lab[b].cpu().numpy(), ref)["ok"], b
        new_ref, sums_ref, cnts_ref = oracle.kmeans_update(x[b].numpy(), lab[b].cpu().numpy().astype(np.int64), c[b].numpy())
        assert np.array_equal(cnts[b].cpu().numpy(), cnts_ref)
        assert parity.rel_close(sums[b].cpu().numpy(), sums_ref, rel=1e-4, atol=1e-4)
        assert parity.rel_close(new[b].cpu().numpy(), new_ref, rel=1e-4, atol=1e-5)
        assert np.allclose(shift[b].cpu().numpy(), np.sqrt(((new_ref - c[b].numpy()) ** 2).sum(-1)), rtol=1e-4, atol=1e-5)
    ids, cents, n_iter = fl.flash_kmeans(xd, K, max_iters=3, init_centroids=cd)
    for b in (0, B - 1):
        rl, rc, _ = oracle.kmeans(x[b].numpy(), K, max_iters=3, init_centroids=c[b].numpy())
        assert (ids[b].cpu().numpy() == rl).mean() > 0.999
        assert parity.rel_close(cents[b].cpu().numpy(), rc, rel=1e-3, atol=1e-4)


@pytest.mark.parametrize("n,d,K", [(200_000, 64, 256), (50_001, 100, 37), (30_000, 7, 16)])
def test_incremental_update_equals_the_full_one(n, d, K):
    """Sums maintained by moving only the rows whose label changed: counts identical, sums equal to
    the full recomputation up to fp32 rounding, labels outside [0, K) ignored, prev brought up to date."""
    from flashlib_b200 import kmeans as km
    g = torch.Generator().manual_seed(n + K)
    x = torch.randn(1, n, d, generator=g).cuda()
    a = torch.randint(0, K, (1, n), generator=g, dtype=torch.int32).cuda()
    b = a.clone()
    pick = torch.randperm(n, generator=g)[: n // 20].cuda()
    b[0, pick] = torch.randint(0, K, (pick.numel(),), generator=g, dtype=torch.int32).cuda()
    b[0, pick[:5]] = -1                                         # a few points drop out altogether
    cents = torch.zeros(1, K, d, device="cuda")
    sums, cnts = km.triton_centroid_update_euclid(x, a, cents, calculate_new=False)
    prev = a.clone()
    km.centroid_update_delta(x, b, prev, sums, cnts)
    want_s, want_c = km.triton_centroid_update_euclid(x, b, cents, calculate_new=False)
    assert torch.equal(cnts, want_c)
    scale = want_s.abs().max().item()
    assert (sums - want_s).abs().max().item() <= 2e-5 * scale
    assert torch.equal(prev[0, pick[5:]], b[0, pick[5:]]) and torch.all(prev[0, pick[:5]] == -1)
    keep = torch.ones(n, dtype=torch.bool, device="cuda")
    keep[pick] = False
    assert torch.equal(prev[0, keep], a[0, keep])


def test_lloyd_loop_with_and_without_incremental_sums(monkeypatch):
    X, _ = synthetic.mixture(120_000, 64, 64, 4)
    Xd = X.cuda()
    init = Xd[:200].clone()
    l1, c1, n1 = fl.flash_kmeans(Xd, 200, max_iters=20, init_centroids=init)
    monkeypatch.setenv("FLASHLIB_B200_KMEANS_DELTA", "0")
    l0, c0, n0 = fl.flash_kmeans(Xd, 200, max_iters=20, init_centroids=init)
    assert n0 == n1 == 20
    # Two runs never agree to the last bit (the sums are fp32 atomics in any order, and a boundary point
    # that changes sides moves its centroids): the yardstick is the objective, as for the oracle.
    def inertia(lab, c):
        return float(((Xd - c[lab.long()]) ** 2).sum())
    i1, i0 = inertia(l1, c1), inertia(l0, c0)
    assert abs(i1 - i0) <= 1e-3 * i0, (i1, i0)
    assert (l0 == l1).float().mean().item() > 0.97
