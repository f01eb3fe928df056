"""Generates tests/golden/*.npz by running the unmodified reference (FlashML-org/flashlib,
torch CPU path) on small seeded inputs.

Run in a container that has the reference tree:

    PYTHONPATH=<reference root> python tests/golden/make_golden.py

The fixtures hold inputs and the reference's outputs, so the tests that read them never
need the reference itself.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from flashlib_b200 import synthetic  # noqa: E402

import flashlib  # noqa: E402  (the reference)
from flashlib.primitives.knn.torch_fallback import knn_torch_chunked, knn_torch_naive  # noqa: E402
from flashlib.primitives.kmeans.torch_fallback import (  # noqa: E402
    _centroid_update_torch_native, batch_kmeans_Euclid_torch_native, euclid_assign_torch_native_chunked)
from flashlib.primitives.ivf_flat.torch_fallback import ivf_flat_build_torch, ivf_flat_search_torch  # noqa: E402


def sha(t: torch.Tensor) -> str:
    return hashlib.sha1(t.contiguous().numpy().tobytes()).hexdigest()


def main() -> None:
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # --- kNN, small, inputs stored -------------------------------------------------------
    db, q = synthetic.randn_knn(3000, 48, 200, seed=10)
    out = {}
    for k in (1, 10, 100):
        v, i = flashlib.flash_knn(q, db, k)  # routes to knn_torch_naive on CPU
        v2, i2 = knn_torch_chunked(q[None], db[None], k, chunk_size=512)
        out[f"vals_k{k}"] = v.numpy()
        out[f"idxs_k{k}"] = i.numpy().astype(np.int32)
        out[f"vals_chunked_k{k}"] = v2[0].numpy()
        out[f"idxs_chunked_k{k}"] = i2[0].numpy().astype(np.int32)
    np.savez_compressed(os.path.join(HERE, "knn_small.npz"), db=db.numpy(), q=q.numpy(), **out)

    # --- kNN, the CPU configuration (20 000 x 64, 1 000 queries, k=10, seed 0): outputs
    #     plus input checksums (inputs are regenerated from the seed) ------------------------
    cfg = synthetic.CONFIGS["knn_cpu_small"]
    db, q = synthetic.randn_knn(cfg["m"], cfg["d"], cfg["nq"], cfg["seed"])
    v, i = flashlib.flash_knn(q, db, cfg["k"])
    np.savez_compressed(os.path.join(HERE, "knn_cpu_config.npz"), vals=v.numpy(), idxs=i.numpy().astype(np.int32),
                        db_sha1=sha(db), q_sha1=sha(q), k=cfg["k"])

    # --- kNN, clamped mixture (shape of the 1M configuration, scaled down).  Inputs are
    #     rounded to fp16-representable values so the fixture stays small ------------------
    X, Q = synthetic.mixture(4000, 128, 64, seed=12, nq=128, clamp=True)
    Xs, Qs = X.half().float(), Q.half().float()
    v, i = knn_torch_naive(Qs[None], Xs[None], 10)
    np.savez_compressed(os.path.join(HERE, "knn_mixture.npz"), db=Xs.numpy().astype(np.float16),
                        q=Qs.numpy().astype(np.float16), vals=v[0].numpy(),
                        idxs=i[0].numpy().astype(np.int32), k=10)

    # --- k-means: assign / update / full loop with explicit init ---------------------------
    X, _ = synthetic.mixture(6000, 32, 24, seed=11)
    K = 40
    init = X[:K].clone()
    labels0 = euclid_assign_torch_native_chunked(X[None], init[None])
    new0 = _centroid_update_torch_native(X[None], labels0.long(), init[None])
    hist_c = [init.numpy().copy()]
    hist_l = []
    c = init[None].clone()
    for _ in range(6):
        l_it = euclid_assign_torch_native_chunked(X[None], c)
        c = _centroid_update_torch_native(X[None], l_it.long(), c)
        hist_l.append(l_it[0].numpy().copy())
        hist_c.append(c[0].numpy().copy())
    ids, cents, n_iter = flashlib.flash_kmeans(X, K, max_iters=6, init_centroids=init)
    np.savez_compressed(os.path.join(HERE, "kmeans_small.npz"), x=X.numpy(), K=K, init=init.numpy(),
                        labels0=labels0[0].numpy(), new0=new0[0].numpy(),
                        hist_centroids=np.stack(hist_c), hist_labels=np.stack(hist_l),
                        final_labels=ids.numpy(), final_centroids=cents.numpy(), n_iter=n_iter)

    # --- IVF-Flat: reference-built index + reference search --------------------------------
    X, Q = synthetic.mixture(5000, 32, 40, seed=13, nq=150, clamp=True)
    index = ivf_flat_build_torch(X, 32, nprobe=4, niter=5, seed=3)
    out = {}
    for k, nprobe in ((10, 4), (5, 32), (10, 1)):
        v, ids_ = ivf_flat_search_torch(index, Q, k, nprobe=nprobe)
        out[f"vals_k{k}_p{nprobe}"] = v.numpy()
        out[f"ids_k{k}_p{nprobe}"] = ids_.numpy()
    np.savez_compressed(os.path.join(HERE, "ivf_small.npz"), x=X.numpy(), q=Q.numpy(),
                        centroids=index.centroids.numpy(), data=index.data.numpy(), ids=index.ids.numpy(),
                        list_offsets=index.list_offsets.numpy(), nlist=index.nlist, **out)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
