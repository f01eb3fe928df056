"""One rank of the multi-GPU test (launched by tests/test_multi_gpu.py through
``python -m torch.distributed.run``, one process per GPU, NCCL): sharded k-means and sharded kNN
on real ranks, each checked against the single-GPU result of the same library on the whole data
and against the CPU oracle.  Rank 0 prints one JSON line."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import flashlib_b200 as fl                                   # noqa: E402
from flashlib_b200 import sharded, synthetic                 # noqa: E402
from flashlib_b200.knn import check_pending                  # noqa: E402
from oracle import oracle                                    # noqa: E402
from tests import parity                                     # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    report = {}

    # ---- k-means: rows dealt to the ranks, sums and counts all-reduced in one buffer ----------
    X, _ = synthetic.mixture(200_000, 64, 64, 11, clamp=True)
    K, iters = 256, 8
    init = X[torch.randperm(X.shape[0], generator=torch.Generator().manual_seed(2))[:K]].clone()
    s, e = sharded.shard_bounds(X.shape[0], world, rank)
    labels, cents, n_iter = sharded.sharded_kmeans(X[s:e].cuda(), K, max_iters=iters, init_centroids=init.cuda())
    one_l, one_c, one_n = fl.flash_kmeans(X.cuda(), K, max_iters=iters, init_centroids=init.cuda())
    one_l, one_c = one_l.reshape(-1), one_c.reshape(K, -1)
    same = (labels == one_l[s:e]).float().mean().item()
    cdiff = (cents - one_c).abs().max().item() / one_c.abs().max().item()
    ref_l, ref_c, _ = oracle.kmeans(X.numpy(), K, max_iters=iters, init_centroids=init.numpy())
    agree = float((labels.cpu().numpy() == ref_l[s:e]).mean())
    report["kmeans"] = {"label_agreement_with_one_gpu": same, "centroid_rel_diff": cdiff, "label_agreement_with_oracle": agree,
                        "iterations": int(n_iter),
                        # fp32 sums are accumulated in another order on two GPUs than on one: a handful of
                        # boundary points change sides, which moves the centroids of small clusters a little
                        "ok": bool(same > 0.999 and cdiff < 1e-2 and agree > 0.995 and n_iter == one_n)}

    # ---- kNN: row-sharded database, shared threshold seeds, packed exchange --------------------
    Xk, Q = synthetic.mixture(400_000, 128, 256, 7, nq=1000, clamp=True)
    s, e = sharded.shard_bounds(Xk.shape[0], world, rank)
    shard = Xk[s:e].cuda()
    index = sharded.ShardedKnnIndex(shard, s)
    Qd = Q.cuda()
    _, ref_i = oracle.knn_chunked(Q.numpy(), Xk.numpy(), 10, chunk_size=8192)
    for result in ("replicated", "owner"):
        d_, i_ = sharded.sharded_knn(Qd, None, 10, index=index, result=result)
        check_pending()
        qs, qe = (0, Q.shape[0]) if result == "replicated" else sharded.shard_bounds(Q.shape[0], world, rank)
        res = parity.knn_parity(Q[qs:qe].numpy(), Xk.numpy(), d_.cpu().numpy(), i_.cpu().numpy(), ref_i[qs:qe])
        report["knn_" + result] = {"rows": res["rows"], "bad_rows": len(res["bad_rows"]), "ok": bool(res["ok"])}

    ok = torch.tensor([int(all(v["ok"] for v in report.values()))], device="cuda")
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    report["all_ranks_ok"] = bool(ok.item())
    if rank == 0:
        print(json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
