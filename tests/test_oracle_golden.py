"""Pins the numpy oracle against outputs of the real reference (tests/golden/*.npz)."""
import os

import numpy as np
import pytest

from oracle import oracle
from tests import parity

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(G, name))


@pytest.mark.parametrize("k", [1, 10, 100])
def test_knn_naive_matches_reference(k):
    d = load("knn_small.npz")
    v, i = oracle.knn_naive(d["q"], d["db"], k)
    res = parity.knn_parity(d["q"], d["db"], v, i, d[f"idxs_k{k}"])
    assert res["ok"], res
    assert parity.rel_close(v, d[f"vals_k{k}"], rel=1e-4, atol=1e-4)


@pytest.mark.parametrize("k", [1, 10, 100])
def test_knn_chunked_matches_reference(k):
    d = load("knn_small.npz")
    v, i = oracle.knn_chunked(d["q"], d["db"], k, chunk_size=512)
    res = parity.knn_parity(d["q"], d["db"], v, i, d[f"idxs_chunked_k{k}"])
    assert res["ok"], res
    # the reference's two paths agree with each other as well
    res2 = parity.knn_parity(d["q"], d["db"], d[f"vals_chunked_k{k}"], d[f"idxs_chunked_k{k}"], d[f"idxs_k{k}"])
    assert res2["ok"], res2


def test_knn_mixture_matches_reference():
    d = load("knn_mixture.npz")
    db, q = d["db"].astype(np.float32), d["q"].astype(np.float32)
    v, i = oracle.knn_naive(q, db, int(d["k"]))
    res = parity.knn_parity(q, db, v, i, d["idxs"])
    assert res["ok"], res


def test_knn_cpu_config_matches_reference():
    import hashlib
    import torch  # only for the seeded generator that made the fixture
    from flashlib_b200 import synthetic
    d = load("knn_cpu_config.npz")
    cfg = synthetic.CONFIGS["knn_cpu_small"]
    db, q = synthetic.randn_knn(cfg["m"], cfg["d"], cfg["nq"], cfg["seed"])
    if hashlib.sha1(db.numpy().tobytes()).hexdigest() != str(d["db_sha1"]):
        pytest.skip("torch's CPU generator produced different bits than when the fixture was made")
    v, i = oracle.knn_naive(q.numpy(), db.numpy(), cfg["k"])
    res = parity.knn_parity(q.numpy(), db.numpy(), v, i, d["idxs"])
    assert res["ok"], res
    assert parity.rel_close(v, d["vals"], rel=1e-4, atol=1e-4)


def test_exact_sqdist():
    d = load("knn_small.npz")
    ex = oracle.exact_sqdist(d["q"], d["db"], d["idxs_k10"].astype(np.int64))
    assert parity.rel_close(d["vals_k10"], ex, rel=1e-4, atol=1e-4)


def test_kmeans_assign_update_match_reference():
    d = load("kmeans_small.npz")
    x, init = d["x"], d["init"]
    lab = oracle.kmeans_assign(x, init)
    res = parity.label_parity(x, init, lab, d["labels0"])
    assert res["ok"], res
    new, sums, cnts = oracle.kmeans_update(x, d["labels0"].astype(np.int64), init)
    assert parity.rel_close(new, d["new0"], rel=1e-4, atol=1e-5)


def test_kmeans_loop_matches_reference_per_step():
    d = load("kmeans_small.npz")
    x = d["x"]
    hc, hl = d["hist_centroids"], d["hist_labels"]
    for t in range(hl.shape[0]):  # teacher forcing: start every step from the reference's centroids
        new, _, lab = oracle.kmeans_iter(x, hc[t])
        assert parity.label_parity(x, hc[t], lab, hl[t])["ok"]
        new_ref_labels, _, _ = oracle.kmeans_update(x, hl[t].astype(np.int64), hc[t])
        assert parity.rel_close(new_ref_labels, hc[t + 1], rel=1e-4, atol=1e-5)
    labels, cents, n_iter = oracle.kmeans(x, int(d["K"]), max_iters=6, init_centroids=d["init"])
    assert n_iter == int(d["n_iter"])
    agree = np.mean(labels == d["final_labels"])
    assert agree > 0.999, agree
    assert parity.rel_close(cents, d["final_centroids"], rel=1e-3, atol=1e-3)


def test_kmeans_empty_cluster_keeps_old_centroid():
    x = np.random.default_rng(0).normal(size=(50, 4)).astype(np.float32)
    old = np.vstack([x[:3], np.full((1, 4), 100.0, np.float32)])
    lab = oracle.kmeans_assign(x, old)
    assert 3 not in lab
    new, _, cnts = oracle.kmeans_update(x, lab.astype(np.int64), old)
    assert cnts[3] == 0 and np.array_equal(new[3], old[3])


@pytest.mark.parametrize("k,nprobe", [(10, 4), (5, 32), (10, 1)])
def test_ivf_search_matches_reference(k, nprobe):
    d = load("ivf_small.npz")
    v, ids, _ = oracle.ivf_search(d["centroids"], d["data"], d["ids"], d["list_offsets"], d["q"], k, nprobe)
    ref_v, ref_i = d[f"vals_k{k}_p{nprobe}"], d[f"ids_k{k}_p{nprobe}"]
    finite = np.isfinite(ref_v)
    assert np.array_equal(finite, np.isfinite(v))
    assert np.array_equal(ids[~finite], ref_i[~finite])
    assert parity.rel_close(v[finite], ref_v[finite], rel=1e-4, atol=1e-4)
    same = np.mean([set(a[f].tolist()) == set(b[f].tolist()) for a, b, f in zip(ids, ref_i, finite)])
    assert same >= 0.99, same


def test_ivf_layout_matches_reference():
    d = load("ivf_small.npz")
    Xp = oracle.pad_features(d["x"], d["data"].shape[1])
    assign, offsets, order = oracle.ivf_assign_lists(Xp, d["centroids"])
    assert np.array_equal(offsets, d["list_offsets"])
    assert np.mean(order == d["ids"]) > 0.999


def test_torch_baseline_matches_oracle_and_reference():
    import torch
    from oracle import oracle_torch
    d = load("knn_small.npz")
    v, i = oracle_torch.knn_chunked(torch.from_numpy(d["q"]), torch.from_numpy(d["db"]), 10, chunk_size=512)
    res = parity.knn_parity(d["q"], d["db"], v.numpy(), i.numpy(), d["idxs_chunked_k10"])
    assert res["ok"], res
    _, oi = oracle.knn_naive(d["q"], d["db"], 10)
    assert parity.knn_parity(d["q"], d["db"], v.numpy(), i.numpy(), oi)["ok"]
